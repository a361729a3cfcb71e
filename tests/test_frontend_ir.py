"""Front end, IR validation and the transposed-matmul pass (CPU)."""
import json
from pathlib import Path

import pytest
import torch

import trainkernel_b200 as tk
from oracle.interpreter import run
from trainkernel_b200 import workloads
from trainkernel_b200.codegen import generate
from trainkernel_b200.ir import Operation, Program, TensorSpec, row_major, validate
from trainkernel_b200.passes import canonicalize_transposed_mm, split_at_gradients

GOLDEN = Path(__file__).resolve().parent / "golden"


def spec(name, shape, strides=None, buffer=None, offset=0):
    return TensorSpec(name, shape, "float32", strides if strides is not None else row_major(shape), buffer or name, offset)


def program_to_json(program):
    import dataclasses

    def s(x):
        return dataclasses.asdict(x)

    return {
        "inputs": [s(x) for x in program.inputs],
        "operations": [{"name": op.name, "op": op.op,
                        "inputs": [s(x) if dataclasses.is_dataclass(x) else {"scalar": x} for x in op.inputs],
                        "output": s(op.output),
                        "attrs": {k: (list(v) if isinstance(v, tuple) else v) for k, v in op.attrs.items()}}
                       for op in program.operations],
        "outputs": [s(x) for x in program.outputs],
    }


def test_capture_lowers_an_mlp_forward():
    program, _ = tk.capture(lambda x, w, b: torch.relu(x @ w + b).mean(), (torch.randn(4, 3), torch.randn(3, 5), torch.randn(5)))
    assert [i.shape for i in program.inputs] == [(4, 3), (3, 5), (5,)]
    assert {"mm", "relu", "mean"} <= {op.op for op in program.operations}
    assert program.outputs[0].shape == ()


def test_capture_rejections():
    with pytest.raises(TypeError, match="tensors only"):
        tk.capture(lambda x, n: x + n, (torch.ones(2), 1))
    with pytest.raises(ValueError, match="cross-device"):
        tk.capture(lambda x: x.to("meta"), (torch.ones(3),))
    with pytest.raises(ValueError, match="lazy negative"):
        tk.capture(lambda x: x + 1, (torch._neg_view(torch.ones(3)),))
    x = torch.ones(4)
    with pytest.raises(ValueError, match="mutation"):
        tk.capture(lambda x: x.add_(2), (x,))
    torch.testing.assert_close(x, torch.ones(4))
    with pytest.raises(ValueError, match="unsupported ATen op aten.sin"):
        tk.capture(torch.sin, (torch.ones(3),))
    for dtype in (torch.int32, torch.int64, torch.float64):
        with pytest.raises(ValueError, match="unsupported dtype"):
            tk.capture(lambda x: x + 1, (torch.ones(3, dtype=dtype),))


@pytest.mark.parametrize("case,workload,seed", [("c1_seed0", "c1", 0), ("c2_seed0", "c2", 0), ("c3_seed0", "c3", 0),
                                                ("c4_seed0", "c4", 0), ("gemv_seed0", "gemv", 0)])
def test_captured_program_equals_the_reference_capture(case, workload, seed):
    """The IR this front end produces is field-for-field what the reference's `capture` produced."""
    stored = json.loads((GOLDEN / "programs.json").read_text())[case]
    work = workloads.build(workload, seed=seed)
    program, _ = tk.capture(work.fn(), (work.state, *work.batches[0]))
    assert json.loads(json.dumps(program_to_json(program))) == stored


def test_validation_bounds_views_and_ssa_order():
    x = spec("x", (2, 3))
    with pytest.raises(ValueError, match="allocation"):
        generate(Program((x,), (), (spec("bad", (2, 3), (300, 1), "x"),)))
    future, out = spec("future", (2, 3)), spec("out", (2, 3))
    with pytest.raises(ValueError, match="future|undefined"):
        generate(Program((x,), (Operation("bad", "add", (x, future), out),), (out,)))
    with pytest.raises(ValueError, match="new roots"):
        generate(Program((x,), (Operation("bad", "add", (x, 1), x),), (x,)))
    a, b = spec("a", (2, 3)), spec("b", (3, 4))
    with pytest.raises(ValueError, match="matrix output shape"):
        generate(Program((a, b), (Operation("bad", "mm", (a, b), spec("out", (2, 2))),), (spec("out", (2, 2)),)))
    b = spec("b", (2, 2))
    with pytest.raises(ValueError, match="broadcast"):
        generate(Program((a, b), (Operation("bad", "add", (a, b), spec("out", (2, 3))),), (spec("out", (2, 3)),)))


@pytest.mark.parametrize("observed", [False, True])
def test_transpose_rewrite_preserves_results(observed):
    a, b = torch.randn(3, 5), torch.randn(5, 7)

    def fn(a, b):
        x = a @ b
        return (x, x.t() + 1) if observed else x.t() + 1

    program, _ = tk.capture(fn, (a, b))
    rewritten = canonicalize_transposed_mm(program)
    validate(rewritten)
    torch.testing.assert_close(run(rewritten, (a, b)), run(program, (a, b)))
    assert (rewritten == program) == observed
    assert canonicalize_transposed_mm(rewritten) == rewritten


def test_dependent_transposed_matmuls_rewrite_together():
    a, b, c = torch.randn(3, 5), torch.randn(5, 7), torch.randn(3, 4)
    program, _ = tk.capture(lambda a, b, c: ((a @ b).t() @ c).t() + 1, (a, b, c))
    rewritten = canonicalize_transposed_mm(program)
    validate(rewritten)
    torch.testing.assert_close(run(rewritten, (a, b, c)), run(program, (a, b, c)))
    assert canonicalize_transposed_mm(rewritten) == rewritten


def test_split_at_gradients_reassembles_the_step():
    work = workloads.build("c2")
    x, t = work.batches[0]
    program, _ = tk.capture(work.fn(), (work.state, x, t))
    first, second = split_at_gradients(program, 4)
    validate(first)
    validate(second)
    whole = run(program, (*work.state, x, t))
    part = run(first, (*work.state, x, t))
    updated = run(second, (*work.state, *part[1:]))
    for a, b in zip((*part, *updated), whole):
        assert torch.equal(a, b)
    assert {op.op for op in second.operations} == {"mul", "sub"}


def test_training_api_uses_the_runtime_seam(monkeypatch):
    parameter, inputs = torch.randn(3, 2), torch.randn(4, 3)

    class FakeRunner:
        source = "// generated CUDA"

        def __call__(self, parameter, inputs):
            return (inputs @ parameter).mean(), torch.ones_like(parameter), parameter - 1e-3

    monkeypatch.setattr("trainkernel_b200.runtime.compile_program", lambda *a, **k: FakeRunner())

    def step(parameter, inputs):
        return (inputs @ parameter).mean(), torch.ones_like(parameter), parameter - 1e-3

    compiled = tk.compile_training(step, (parameter, inputs))
    assert isinstance(compiled, tk.CompiledTrainingStep)
    assert compiled.source == "// generated CUDA"
    loss, grad, new = compiled(parameter, inputs)
    assert loss.shape == () and grad.shape == parameter.shape and new.shape == parameter.shape


def test_training_api_rejects_wrong_structures():
    p, x = torch.randn(3, 2), torch.randn(4, 3)
    with pytest.raises(ValueError, match="return loss, gradients"):
        tk.compile_training(lambda p, x: x @ p, (p, x))
    with pytest.raises(ValueError, match="pytree"):
        tk.compile_training(lambda p, x: ((x @ p).mean(), (p,), p), (p, x))
    with pytest.raises(ValueError, match="scalar loss"):
        tk.compile_training(lambda p, x: (x @ p, p, p + 1), (p, x))
    with pytest.raises(ValueError, match="gradient.*shapes"):
        tk.compile_training(lambda p, x: ((x @ p).mean(), p.sum(), p + 1), (p, x))
    with pytest.raises(ValueError, match="derives its own"):
        tk.compile_training(lambda p, x: ((x @ p).mean(), p, p + 1), (p, x), inplace_outputs={})


def test_compile_without_gpu_fails_loudly():
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError, match="CUDA sm_100a GPU required"):
        tk.compile(lambda x: x + 1, (torch.ones(4),))


def test_integer_labels_flow_only_through_one_hot():
    work = workloads.build("c3")
    features, dense = work.batches[0]
    fn = lambda w, x, labels: workloads.onehot_label_step(w, x, labels, 1e-2)  # noqa: E731
    program, _ = tk.capture(fn, (work.state, features, work.labels))
    assert program.inputs[2].dtype == "int64"
    assert {"arange", "eq"} <= {op.op for op in program.operations}
    got = run(program, (work.state, features, work.labels))
    want = run(tk.capture(work.fn(), (work.state, features, dense))[0], (work.state, features, dense))
    for a, b in zip(got, want):
        assert torch.equal(a, b)                       # label form == dense one-hot form, bit for bit
    g = generate(program, inplace_outputs={2: 0})
    assert g.tensor_core_operations == 2 and "==" in g.source
    with pytest.raises(ValueError, match="unsupported dtype"):
        tk.capture(lambda x: x + 1, (torch.ones(3, dtype=torch.int64),))
