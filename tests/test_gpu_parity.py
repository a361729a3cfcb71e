"""GPU parity: every registered case, run through the C-ABI shim, against the CPU oracle."""
import pytest
import torch
from torch.utils._pytree import tree_flatten

from tests import cases
from tests.helpers import REL_TOL, assert_outputs_close, assert_step_close, compile_case, oracle_outputs

pytestmark = pytest.mark.gpu

GEMM_CASES = [name for name in cases.CASES if name.startswith(("gemm_", "gemm2_", "gemv_"))]
STEP_CASES = ["c1", "c1_grid_barrier", "c2", "c2_grid_barrier", "c3_one_cluster", "c2_nofuse", "c2_notc", "c3", "c3_labels", "c4", "gemv", "mlp_f32", "mlp_bf16", "mlp_f16",
              "mlp_f32_one_block", "linear_module", "mlp_2cta", "mlp_1cta", "mlp_2cta_background", "mlp_2cta_stream_warps",
              "mlp_1cta_stream_warps"]
GENERAL_CASES = ["partial_reduce", "big_reduce", "long_reduce", "views_out", "addmm_scaled", "addmm_scaled_bf16",
                 "addmm_beta0_nan_bias", "observable_product", "transposed_operand_broadcast_chain", "rounding_boundary_bf16",
                 "branched_outputs_one_product", "huge_reduction", "huge_reduction_bf16", "original_and_update"]


def _compute_dtype(inputs):
    flat, _ = tree_flatten(inputs)
    return torch.float32 if all(t.dtype == torch.float32 for t in flat) else \
        (torch.float16 if any(t.dtype == torch.float16 for t in flat) else torch.bfloat16)


@pytest.mark.parametrize("name", GEMM_CASES)
def test_gemm_paths_match_oracle(name):
    compiled, inputs, cpu_inputs, program = compile_case(name)
    out = compiled(*inputs)
    compiled.runner.status()
    # one rounding of the result: 2^-8 for bf16, 2^-11 for f16, accumulation-order noise for fp32
    tol = {torch.float32: 1e-5, torch.bfloat16: 6e-3, torch.float16: 1e-3}[_compute_dtype(inputs)]
    assert_outputs_close(out, oracle_outputs(program, cpu_inputs), tol, name)


@pytest.mark.parametrize("name", STEP_CASES)
def test_training_step_matches_oracle(name):
    compiled, inputs, cpu_inputs, program = compile_case(name)
    state_leaves, _ = tree_flatten(inputs[0])
    pointers = [t.data_ptr() for t in state_leaves]
    expected = oracle_outputs(program, cpu_inputs)      # computed before the step mutates state
    pristine = tuple(t.clone() for t in tree_flatten(inputs)[0])
    out = compiled(*inputs)
    compiled.runner.status()
    assert_step_close(out, expected, program, pristine, REL_TOL[_compute_dtype(inputs)], name)
    # updated state is written into the caller's state tensors
    updated, _ = tree_flatten(out[2])
    assert [t.data_ptr() for t in updated] == pointers
    n = len(state_leaves)
    for leaf, new in zip(state_leaves, updated):
        assert torch.equal(leaf, new)


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c4"])
def test_training_step_matches_eager_pytorch_on_the_gpu(name):
    """The second yardstick beside the IR oracle: the step function itself, run eagerly by PyTorch on
    the same device and the same seeded inputs (TF32 and reduced-precision reductions off)."""
    from tests import cases
    previous = (torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction, torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction)
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False
    try:
        compiled, inputs, _, _ = compile_case(name)
        fn, eager_inputs, _, _ = cases.build(name, "cuda")
        loss, grads, updated = fn(*eager_inputs)
        expected = [loss, *tree_flatten(grads)[0], *tree_flatten(updated)[0]]
        out = compiled(*inputs)
        compiled.runner.status()
        tol = REL_TOL[_compute_dtype(inputs)]
        if tol < 1e-4:
            tol = 2e-5          # two different FP32 summation orders against each other, not against the exact host sum
        assert_outputs_close(out, expected, tol, f"{name} against eager PyTorch")
    finally:
        (torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction,
         torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction) = previous


@pytest.mark.parametrize("name", GENERAL_CASES)
def test_general_subset_matches_oracle(name):
    compiled, inputs, cpu_inputs, program = compile_case(name)
    expected = oracle_outputs(program, cpu_inputs)
    out = compiled(*inputs)
    compiled.runner.status()
    # FP32 programs: summation-order noise only; 16-bit programs: one rounding of the result
    tol = {torch.float32: 1e-5, torch.bfloat16: 8e-3, torch.float16: 1e-3}[_compute_dtype(inputs)]
    assert_outputs_close(out, expected, tol, name)


def test_direct_commit_add_one_and_graph_replay():
    compiled, inputs, cpu_inputs, _ = compile_case("add_one_inplace")
    x = inputs[0]
    original = x.clone()
    assert compiled.runner.generated.direct_state_commits == 1
    out = compiled(x)
    assert out.data_ptr() == x.data_ptr()
    torch.testing.assert_close(x, original + 1)
    captured = compiled.capture(x)
    torch.testing.assert_close(x, original + 1)          # capture restores state
    for _ in range(4):
        captured.replay()
    torch.cuda.synchronize()
    compiled.runner.status()
    torch.testing.assert_close(x, original + 5)


def test_swap_and_transposed_updates_are_transactional():
    compiled, inputs, _, _ = compile_case("swap_inplace")
    a, b = inputs
    a0, b0 = a.clone(), b.clone()
    assert compiled.runner.generated.staged_state_commits >= 1
    compiled(a, b)
    compiled.runner.status()
    torch.testing.assert_close(a, b0 * 2.0)
    torch.testing.assert_close(b, a0 + 1.0)
    compiled, inputs, _, _ = compile_case("transposed_update")
    (m,) = inputs
    m0 = m.clone()
    assert compiled.runner.generated.direct_state_commits == 0
    compiled(m)
    compiled.runner.status()
    torch.testing.assert_close(m, m0.t() + 1.0)


def test_runtime_rejects_mismatched_inputs_and_aliased_buffers():
    compiled, inputs, _, _ = compile_case("gemm_f32")
    a, b = inputs
    with pytest.raises(ValueError, match="shape, stride"):
        compiled(a[:-1], b)
    buffers = compiled.runner.allocate(a, b)
    aliased = type(buffers)(buffers.outputs, a.reshape(-1)[: buffers.workspace.numel()])
    with pytest.raises(ValueError, match="alias|workspace"):
        compiled.runner.run_into(a, b, buffers=aliased)


def test_barrier_timeout_is_reported_not_hung():
    """A barrier that can never complete must end with an error status, not a stuck device."""
    from trainkernel_b200 import runtime
    compiled, inputs, _, _ = compile_case("c1_grid_barrier")
    runner = compiled.runner
    lib = runtime.library()
    assert runner.module.grid > 1 and runner.generated.barrier == "grid"
    lib.tk_module_set_timeout(runner.module.handle, 20_000_000)               # 20 ms
    lib.tk_module_set_expected_arrivals(runner.module.handle, runner.module.grid + 1)
    state = inputs[0].clone()
    compiled(state, inputs[1], inputs[2])
    with pytest.raises(RuntimeError, match="timed out"):
        runner.status()
    # the context is still usable: reset, restore the defaults, run a correct step
    assert lib.tk_module_reset(runner.module.handle) == 0
    lib.tk_module_set_expected_arrivals(runner.module.handle, 0)
    lib.tk_module_set_timeout(runner.module.handle, 2_000_000_000)
    fresh = inputs[0].clone()
    out = compiled(fresh, inputs[1], inputs[2])
    assert runner.status()[0] == 0
    assert bool(torch.isfinite(out[0]))


@pytest.mark.parametrize("exchange", ["narrow", "float32"])
def test_split_step_without_a_process_group_matches_oracle(exchange):
    """Gradient kernel + update kernel (the data-parallel form, world size 1) equals the one-kernel step."""
    from trainkernel_b200 import dp, workloads
    import trainkernel_b200 as tk
    work = workloads.build("c2", seed=1, device="cuda")
    cpu = workloads.build("c2", seed=1, device="cpu")
    x, t = work.batches[0]
    step = dp.ShardedTrainingStep(work.fn(), (work.state, x, t), exchange=exchange)
    assert step.narrow == (exchange == "narrow")
    program, _ = tk.capture(cpu.fn(), (cpu.state, *cpu.batches[0]))
    expected = oracle_outputs(program, (cpu.state, *cpu.batches[0]))
    pointers = [p.data_ptr() for p in work.state]
    loss, grads, state = step(work.state, x, t)
    step.status()
    assert_outputs_close((loss, grads, state), expected, 2e-2, "split step")
    assert [p.data_ptr() for p in state] == pointers


@pytest.mark.parametrize("stream_warps", [False, True])
def test_fused_exchange_step_with_one_rank_matches_oracle_and_replays(stream_warps):
    """The one-kernel data-parallel form (exchange stages inside the kernel) on a single rank:
    flags, epochs and the pull/reduce/push path all run, with this GPU as its own only peer; with
    stream warps the exchange and the FP32 updates run in warps 6..9 beside the GEMM tiles."""
    from trainkernel_b200 import dp, workloads
    import trainkernel_b200 as tk
    from oracle import interpreter
    work = workloads.build("c2", seed=2, device="cuda")
    cpu = workloads.build("c2", seed=2, device="cpu")
    step = dp.FusedShardedTrainingStep(work.fn(), (work.state, *work.batches[0]), background=stream_warps)
    # 320 threads either way: four stream warps, or without them four more epilogue warps for the tensor-core tiles
    assert step.generated.threads == 320 and ("32-thread slice" in step.generated.source) == stream_warps
    assert ("#define TK_EPI_WARPS 8" in step.generated.source) == (not stream_warps)
    assert step.generated.symmetric_bytes > 4096 and "tk::exchange_mean" in step.generated.source
    program, _ = tk.capture(cpu.fn(), (cpu.state, *cpu.batches[0]))
    ref_state = tuple(cpu.state)
    for i in range(6):                                   # several launches: the epoch advances every time
        loss, grads, state = step(work.state, *work.batches[i % 4])
        expected = interpreter.run(program, (*ref_state, *cpu.batches[i % 4]))
        step.status()
        assert_outputs_close((loss, grads, state), expected, 2e-2, f"fused step {i}")
        ref_state = tuple(e.clone() for e in expected[5:])
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(4):
            step(work.state, *work.batches[i % 4])
    before = [p.clone() for p in work.state]
    graph.replay()
    torch.cuda.synchronize()
    step.status()
    assert any(not torch.equal(a, b) for a, b in zip(before, work.state))
    assert all(bool(torch.isfinite(p).all()) for p in work.state)


def test_label_indexing_is_bit_exact_with_the_dense_one_hot_target():
    """`col == label` evaluated in the GEMM epilogue equals one_hot(labels, C) exactly: loss, gradient and
    updated weights of the label form and of the dense-target form are bit-identical for several steps."""
    dense, dense_inputs, _, _ = compile_case("c3")
    labelled, label_inputs, _, _ = compile_case("c3_labels")
    assert any(op.op == "eq" for op in labelled.program.operations)
    w_dense, w_label = dense_inputs[0], label_inputs[0]
    assert torch.equal(w_dense, w_label)
    for _ in range(5):
        a = dense(w_dense, *dense_inputs[1:])
        b = labelled(w_label, *label_inputs[1:])
        dense.runner.status()
        labelled.runner.status()
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(w_dense, w_label)


def test_captured_program_keeps_its_inputs_alive_and_restores_state():
    """Reference behaviour: tests/test_training_api.py:70-95."""
    import gc
    import weakref
    import trainkernel_b200 as tk
    data = {"x": torch.randn(128, device="cuda")}
    original = data["x"].clone()
    alive = weakref.ref(data["x"])
    compiled = tk.compile(lambda d: d["x"] + 1, (data,), max_blocks=1)
    captured = compiled.capture(data)
    data["x"] = torch.zeros_like(original)
    gc.collect()
    assert alive() is not None
    torch.testing.assert_close(captured.replay(), original + 1)
    # an in-place program: capturing leaves the state as it was, every replay advances it
    x = torch.randn(128, device="cuda")
    before = x.clone()
    stepper = tk.compile(lambda v: v + 1, (x,), inplace_outputs={0: 0}, max_blocks=1)
    graph = stepper.capture(x)
    torch.testing.assert_close(x, before)
    for _ in range(4):
        graph.replay()
    torch.testing.assert_close(x, before + 4)


def test_inplace_targets_must_be_detached_from_autograd():
    """Reference behaviour: tests/test_direct_commits.py:59-63."""
    import trainkernel_b200 as tk
    x = torch.randn(64, device="cuda", requires_grad=True)
    with pytest.raises(ValueError, match="detached|autograd"):
        tk.compile(lambda v: v + 1, (x,), inplace_outputs={0: 0})


def test_aligned_kernels_refuse_unaligned_tensors_and_unaligned_examples_keep_the_fallback():
    """A kernel generated for 16-byte aligned tensors refuses (on the host, before anything is launched) a
    tensor that is not; compiling on such a tensor drops the assumption, and the step still matches the oracle."""
    import trainkernel_b200 as tk
    from oracle import interpreter
    from trainkernel_b200 import workloads
    work = workloads.build("c2", seed=5, device="cuda")
    cpu = workloads.build("c2", seed=5, device="cpu")
    x, target = work.batches[0]
    aligned = tk.compile_training(work.fn(), (work.state, x, target))
    generated = aligned.runner.generated
    assert generated.aligned_inputs and generated.aligned_outputs and "tk::ld_row_full<" in generated.source
    shifted = torch.empty(target.numel() + 2, dtype=target.dtype, device="cuda")[2:].view_as(target)   # 4 bytes off
    shifted.copy_(target)
    assert shifted.data_ptr() % 16 == 4
    before = [p.clone() for p in work.state]
    with pytest.raises(RuntimeError, match="not 16-byte aligned"):
        aligned(work.state, x, shifted)
    torch.cuda.synchronize()
    aligned.runner.status()
    assert all(torch.equal(a, b) for a, b in zip(before, work.state))          # nothing ran
    general = tk.compile_training(work.fn(), (work.state, x, shifted))
    assert not general.runner.generated.aligned_inputs and "_full<" not in general.runner.generated.source
    program, _ = tk.capture(cpu.fn(), (cpu.state, *cpu.batches[0]))
    expected = interpreter.run(program, (*cpu.state, *cpu.batches[0]))
    out = general(work.state, x, shifted)
    general.runner.status()
    assert_outputs_close(out, expected, 2e-2, "step on an unaligned target")
