"""Pin the CPU oracle (`oracle/interpreter.py`) against fixtures made by the unmodified reference."""
from pathlib import Path

import numpy as np
import pytest
import torch

import trainkernel_b200 as tk
from oracle.interpreter import run
from trainkernel_b200 import workloads

GOLDEN = Path(__file__).resolve().parent / "golden"
SAMPLE = 2048

# (fixture, workload, seed, steps checked here, relative tolerance).  The fixtures were produced by the
# same torch CPU kernels, so differences come only from a different host CPU's vector width.
CASES = [("c1_seed0", "c1", 0, 100, 2e-6), ("c2_seed0", "c2", 0, 100, 2e-3), ("c2_seed1", "c2", 1, 100, 2e-3),
         ("c2_seed2", "c2", 2, 100, 2e-3), ("c3_seed0", "c3", 0, 20, 2e-3), ("c3_seed1", "c3", 1, 5, 2e-3),
         ("c3_seed2", "c3", 2, 5, 2e-3), ("c4_seed0", "c4", 0, 100, 2e-3), ("gemv_seed0", "gemv", 0, 100, 2e-3)]


def _leaves(state):
    return tuple(state) if isinstance(state, (tuple, list)) else (state,)


def _sample(t):
    flat = t.detach().float().reshape(-1)
    stride = max(1, flat.numel() // SAMPLE)
    return flat[::stride][:SAMPLE].numpy()


@pytest.mark.parametrize("fixture,name,seed,steps,tol", CASES)
def test_oracle_reproduces_reference_trajectory(fixture, name, seed, steps, tol):
    golden = np.load(GOLDEN / f"{fixture}.npz")
    work = workloads.build(name, seed=seed)
    x0, t0 = work.batches[0]
    checks = np.stack([[float(v.double().sum()), float(v.double().abs().sum())] for v in (*_leaves(work.state), x0, t0)])
    np.testing.assert_allclose(checks, golden["input_checksum"], rtol=1e-9, atol=1e-9)   # generator did not drift
    program, _ = tk.capture(work.fn(), (work.state, x0, t0))
    state = _leaves(work.state)
    n = len(state)
    total = len(golden["losses"])
    out = None
    for step in range(steps):
        x, t = work.batches[step % len(work.batches)]
        out = run(program, (*state, x, t))
        want = float(golden["losses"][step])
        assert abs(float(out[0]) - want) <= tol * abs(want), f"loss at step {step}"
        state = tuple(o.clone() for o in out[1 + n:])
    if steps == total:
        for i in range(n):
            for kind, tensor in (("grad", out[1 + i]), ("state", state[i])):
                want = golden[f"{kind}{i}_sample"]
                err = float(np.max(np.abs(_sample(tensor) - want))) / max(float(np.max(np.abs(want))), 1e-30)
                assert err <= tol, f"{kind}{i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
def test_oracle_reproduces_reference_on_irregular_mlp(dtype):
    golden = np.load(GOLDEN / f"mlp_7_11_17_5_{dtype}.npz")
    torch_dtype = getattr(torch, dtype)
    params = tuple(torch.from_numpy(golden[f"param{i}"]).to(torch_dtype) for i in range(4))
    x, target = torch.from_numpy(golden["x"]).to(torch_dtype), torch.from_numpy(golden["target"]).to(torch_dtype)
    fn = lambda p, xx, yy: workloads.mlp_native_step(p, xx, yy, 1e-3)  # noqa: E731
    program, _ = tk.capture(fn, (params, x, target))
    assert sum(op.op == "mm" for op in program.operations) == 5
    assert any(op.op == "threshold_backward" for op in program.operations)
    assert len(program.outputs) == 9
    tol = {"float32": 2e-6, "bfloat16": 1e-2, "float16": 2e-3}[dtype]
    state = params
    for step in range(3):
        out = run(program, (*state, x, target))
        eager = fn(state, x, target)
        for j, o in enumerate(out):
            want = golden[f"step{step}_out{j}"]
            err = float(np.max(np.abs(o.float().numpy() - want))) / max(float(np.max(np.abs(want))), 1e-30)
            assert err <= tol, f"step {step} output {j}: {err}"
        # interpreter == eager on the same inputs (the reference's own check)
        for got, want in zip(out, (eager[0], *eager[1], *eager[2])):
            torch.testing.assert_close(got, want, rtol=4e-2 if dtype != "float32" else 2e-4, atol=4e-3 if dtype != "float32" else 2e-5)
        state = tuple(out[-4:])


@pytest.mark.parametrize("dims", [(0,), (1,), (-1,), (0, 2), ()])
@pytest.mark.parametrize("keepdim", [False, True])
def test_oracle_partial_reductions(dims, keepdim):
    x = torch.randn(2, 3, 4)
    fn = lambda x: (x.sum(dims, keepdim=keepdim), x.mean(dims, keepdim=keepdim))  # noqa: E731
    program, _ = tk.capture(fn, (x,))
    for got, want in zip(run(program, (x,)), fn(x)):
        torch.testing.assert_close(got, want)


def test_oracle_views_broadcast_alpha_and_cast():
    x, y = torch.randn(3, 4).t(), torch.randn(3)
    fn = lambda a, b: (a.t(), a + b, a.unsqueeze(0).expand(2, 4, 3), a.contiguous().view(-1))  # noqa: E731
    program, _ = tk.capture(fn, (x, y))
    for got, want in zip(run(program, (x, y)), fn(x, y)):
        torch.testing.assert_close(got, want)
    p = (torch.randn(3, 4), torch.randn(3, 4))
    fn2 = lambda p: (torch.add(p[0], p[1], alpha=0.25).to(torch.bfloat16), p[0].sum())  # noqa: E731
    program, _ = tk.capture(fn2, (p,))
    for got, want in zip(run(program, p), fn2(p)):
        torch.testing.assert_close(got, want)
