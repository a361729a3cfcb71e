"""Programs exercised by the GPU parity tests, buildable on any device.

Each case returns `(fn, example_inputs, compile_kind, options)`; inputs are
created on `device`.  The same list is walked on a CPU-only machine to
pre-compile every kernel into the in-tree cubin cache (capture only looks at
shapes, strides and dtypes, so the generated source is identical).
"""
from __future__ import annotations

import torch

from trainkernel_b200 import workloads

BF16, F16, F32 = torch.bfloat16, torch.float16, torch.float32


def _rand(shape, dtype, device, seed):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(shape, generator=gen, dtype=torch.float32).to(dtype).to(device)


def gemm_case(m, n, k, a_major, b_major, dtype=BF16, **options):
    """a @ b with either operand K-major or MN-major in memory."""
    def build(device):
        a = _rand((m, k), dtype, device, 1) if a_major == "k" else _rand((k, m), dtype, device, 1).t()
        b = _rand((n, k), dtype, device, 2).t() if b_major == "k" else _rand((k, n), dtype, device, 2)
        return (lambda x, y: x @ y), (a, b), "compile", dict(options)
    return build


def mlp_case(sizes, batch, **options):
    """BF16-compute / FP32-master MLP step of arbitrary layer sizes."""
    def build(device):
        work = workloads.mlp_workload("mlp", sizes, batch, seed=5, device=device, resident=1)
        x, t = work.batches[0]
        return work.fn(), (work.state, x, t), "compile_training", dict(options)
    return build


def workload_case(name, seed=0, **options):
    def build(device):
        work = workloads.build(name, seed=seed, device=device)
        x, t = work.batches[0]
        return work.fn(), (work.state, x, t), "compile_training", dict(options)
    return build


def native_mlp_case(batch, i, h, o, dtype, **options):
    """The reference's irregular 2-layer MLP step in one dtype (reference: tests/test_gpu.py:19-28)."""
    def build(device):
        gen = torch.Generator(device="cpu").manual_seed(17)
        def rand(shape):
            return torch.randn(shape, generator=gen, dtype=dtype).to(device)
        params = (rand((i, h)) / i ** 0.5, rand((h,)), rand((h, o)) / h ** 0.5, rand((o,)))
        x, t = rand((batch, i)), rand((batch, o))
        fn = lambda p, xx, yy: workloads.mlp_native_step(p, xx, yy, 1e-3)  # noqa: E731
        return fn, (params, x, t), "compile_training", dict(options)
    return build


def function_case(fn, shapes, dtype=F32, kind="compile", **options):
    def build(device):
        inputs = tuple(_rand(shape, dtype, device, 10 + i) for i, shape in enumerate(shapes))
        return fn, inputs, kind, dict(options)
    return build


def _onehot_labels_case(device):
    """C3 with integer class labels: the one-hot target is formed inside the step."""
    work = workloads.build("c3", seed=0, device=device)
    features, _ = work.batches[0]
    fn = lambda w, x, labels: workloads.onehot_label_step(w, x, labels, 1e-2)  # noqa: E731
    return fn, (work.state, features, work.labels.to(device)), "compile_training", {}


def _addmm_nan_bias_case(device):
    """beta = 0 must ignore the bias entirely, NaN included (reference: tests/test_gpu.py:79-86)."""
    bias = torch.full((40,), float("nan"), device=device)
    a, b = _rand((24, 56), F32, device, 21), _rand((56, 40), F32, device, 22)
    return (lambda c, x, y: torch.addmm(c, x, y, beta=0, alpha=2.0)), (bias, a, b), "compile", {}


def _linear_module_case(device):
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(11, 17), torch.nn.ReLU(), torch.nn.Linear(17, 5)).to(device)
    params = {k: v.detach() for k, v in model.named_parameters()}
    x, y = _rand((7, 11), F32, device, 3), _rand((7, 5), F32, device, 4)

    def train(p, x, target):
        def loss(q):
            return ((torch.func.functional_call(model, q, (x,)) - target) ** 2).mean()
        grads, value = torch.func.grad_and_value(loss)(p)
        return value, grads, {key: p[key] - 1e-3 * grads[key] for key in p}
    return train, (params, x, y), "compile_training", {}


CASES = {
    # tcgen05 GEMM, every operand-major combination, aligned and ragged sizes
    "gemm_kk_128": gemm_case(128, 128, 128, "k", "k"),
    "gemm_kn_128": gemm_case(128, 128, 128, "k", "mn"),
    "gemm_mk_128": gemm_case(128, 128, 128, "mn", "k"),
    "gemm_mn_128": gemm_case(128, 128, 128, "mn", "mn"),
    "gemm_kn_ragged": gemm_case(200, 136, 72, "k", "mn"),
    "gemm_mk_ragged": gemm_case(200, 136, 72, "mn", "k"),
    "gemm_kn_big": gemm_case(512, 1000, 512, "k", "mn"),
    "gemm_mn_big": gemm_case(1000, 512, 264, "mn", "mn"),
    "gemm_kk_big": gemm_case(384, 640, 1024, "k", "k"),
    "gemm_kn_f16": gemm_case(256, 192, 128, "k", "mn", F16),
    "gemm_kn_wide": gemm_case(2048, 4096, 256, "k", "mn"),
    # two-CTA (cta_group::2) pair tiles, forced on small shapes and chosen automatically on the wide one above
    "gemm2_kk": gemm_case(512, 512, 256, "k", "k", two_cta=True),
    "gemm2_kn": gemm_case(512, 512, 256, "k", "mn", two_cta=True),
    "gemm2_mk": gemm_case(512, 512, 256, "mn", "k", two_cta=True),
    "gemm2_mn": gemm_case(512, 512, 256, "mn", "mn", two_cta=True),
    "gemm2_ragged": gemm_case(300, 520, 200, "k", "mn", two_cta=True),
    "gemm2_ragged_t": gemm_case(520, 264, 1000, "mn", "k", two_cta=True),
    "gemm2_deep": gemm_case(1024, 768, 4096, "k", "mn", two_cta=True),
    # SIMT and GEMV paths
    "gemm_f32": gemm_case(65, 67, 17, "k", "mn", F32),
    "gemm_f32_t": gemm_case(33, 79, 47, "mn", "k", F32),
    "gemm_odd_bf16": gemm_case(17, 65, 33, "k", "mn"),
    "gemv_n": gemm_case(1, 200, 128, "k", "mn"),
    "gemv_k": gemm_case(1, 200, 128, "k", "k"),
    # the five benchmark configurations (C1..C4 here) and the batch-1 pin
    "c1": workload_case("c1"),
    "c2": workload_case("c2"),
    "c1_grid_barrier": workload_case("c1", cluster_barrier=False),
    "c2_grid_barrier": workload_case("c2", cluster_barrier=False),
    "c3_one_cluster": workload_case("c3", cluster_barrier=True),
    "c2_nofuse": workload_case("c2", fuse_epilogues=False, fuse_pointwise=False),
    "c2_notc": workload_case("c2", tensor_cores=False),
    "c3": workload_case("c3"),
    "c3_labels": _onehot_labels_case,
    "c4": workload_case("c4"),
    "gemv": workload_case("gemv"),
    # the reference's irregular MLP shapes in each dtype
    "mlp_f32": native_mlp_case(17, 33, 65, 19, F32),
    "mlp_bf16": native_mlp_case(17, 33, 65, 19, BF16),
    "mlp_f16": native_mlp_case(17, 33, 65, 19, F16),
    "mlp_f32_one_block": native_mlp_case(7, 11, 17, 5, F32, max_blocks=1),
    "linear_module": _linear_module_case,
    "mlp_2cta": mlp_case((512, 1024, 768, 512), 512, two_cta=True),
    "mlp_1cta": mlp_case((512, 1024, 768, 512), 512, two_cta=False),
    "mlp_2cta_background": mlp_case((512, 1024, 768, 512), 512, two_cta=True, background=True),
    # stream warps with real work: the weight casts are not carried, so they run beside the forward GEMMs
    "mlp_2cta_stream_warps": mlp_case((512, 1024, 768, 512), 512, two_cta=True, background=True, carry_shadows=False),
    "mlp_1cta_stream_warps": mlp_case((512, 1024, 768, 512), 512, two_cta=False, background=True, carry_shadows=False),
    # fusion boundaries (reference: tests/test_epilogues_gpu.py, tests/test_side_epilogues.py)
    "observable_product": function_case(lambda a, b: (a @ b, torch.relu(a @ b) + 1.0), [(40, 24), (24, 56)]),
    "transposed_operand_broadcast_chain": function_case(lambda a, b, row, col: torch.relu(a.t() @ b + row) * col, [(24, 40), (24, 56), (56,), (40, 1)]),
    "rounding_boundary_bf16": function_case(lambda a, b, c: (((a @ b).float() * 3.0 + c.float()).to(BF16), (a @ b).float().sum()),
                                            [(136, 72), (72, 200), (136, 200)], BF16),
    "branched_outputs_one_product": function_case(lambda a, b: (torch.relu(a @ b), (a @ b) * 2.0, ((a @ b) + 1.0).t()), [(48, 32), (32, 48)]),
    "huge_reduction": function_case(lambda x: ((x + 0.5).sum(), (x + 0.5).mean(), x.sum(0), x.mean(1)), [(2048, 1031)]),
    "huge_reduction_bf16": function_case(lambda x: ((x.float() + 0.5).sum(), x.sum(0)), [(2048, 1031)], BF16),
    "original_and_update": function_case(lambda x: (x, x + 1.0), [(8192,)], inplace_outputs={1: 0}),
    # general subset
    "addmm_scaled": function_case(lambda c, a, b: torch.relu(torch.addmm(c, a, b, beta=0.5, alpha=-1.5)), [(40,), (24, 56), (56, 40)]),
    "addmm_scaled_bf16": function_case(lambda c, a, b: torch.addmm(c, a, b, beta=2.0, alpha=0.25), [(136, 72), (136, 200), (200, 72)], BF16),
    "addmm_beta0_nan_bias": _addmm_nan_bias_case,
    "add_one_inplace": function_case(lambda x: x + 1, [(1000,)], inplace_outputs={0: 0}),
    "partial_reduce": function_case(lambda x: (x.sum((0, 2)), x.mean(1, keepdim=True), x.t().sum(0) if x.dim() == 2 else x.sum()), [(5, 7, 9)]),
    "big_reduce": function_case(lambda x: (x.sum(), x.mean(0)), [(5003, 3)]),
    "long_reduce": function_case(lambda x: x.sum(), [(32769,)]),
    "views_out": function_case(lambda a, b: (a.t(), a + b, a.unsqueeze(0).expand(2, 4, 3), a.contiguous().view(-1)), [(4, 3), (3,)]),
    "swap_inplace": function_case(lambda a, b: (b * 2.0, a + 1.0), [(64, 3), (64, 3)], inplace_outputs={0: 0, 1: 1}),
    "transposed_update": function_case(lambda a: a.t() + 1.0, [(32, 32)], inplace_outputs={0: 0}),
}


def build(name: str, device):
    return CASES[name](device)
