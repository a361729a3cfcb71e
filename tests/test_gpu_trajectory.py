"""100-step trajectories and 20-step CUDA-graph replays of the benchmark configurations C1..C4.

Every step's loss, the last step's gradients and the final state are compared
with the fixtures that the unmodified reference produced
(`tests/golden/make_golden.py`), within 1e-5 relative for the FP32 step and
2e-2 relative for BF16-compute / FP32-master steps.
"""
from pathlib import Path

import numpy as np
import pytest
import torch
from torch.utils._pytree import tree_flatten

import trainkernel_b200 as tk
from oracle import interpreter
from trainkernel_b200 import workloads
from tests.helpers import REL_TOL, rel_error

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
SAMPLE = 2048

TRAJECTORIES = [("c1", 0, 100), ("c2", 0, 100), ("c2", 1, 100), ("c2", 2, 100), ("c3", 0, 100), ("c3", 1, 100),
                ("c3", 2, 100), ("c4", 0, 4), ("gemv", 0, 100)]


def _sample(t: torch.Tensor) -> np.ndarray:
    flat = t.detach().float().reshape(-1)
    stride = max(1, flat.numel() // SAMPLE)
    return flat[::stride][:SAMPLE].cpu().numpy()


def _leaves(state):
    return tuple(state) if isinstance(state, (tuple, list)) else (state,)


@pytest.mark.parametrize("name,seed,steps", TRAJECTORIES)
def test_trajectory_matches_reference_fixture(name, seed, steps):
    golden = np.load(GOLDEN / f"{name}_seed{seed}.npz")
    work = workloads.build(name, seed=seed, device="cuda")
    tol = REL_TOL[work.compute_dtype]
    x0, t0 = work.batches[0]
    compiled = tk.compile_training(work.fn(), (work.state, x0, t0))
    state = work.state
    losses, out = [], None
    for step in range(steps):
        x, t = work.batches[step % len(work.batches)]
        out = compiled(state, x, t)
        losses.append(out[0].clone())
    compiled.runner.status()
    losses = torch.stack(losses).float().cpu().numpy()
    expected = golden["losses"]
    assert np.all(np.isfinite(losses))
    assert float(np.max(np.abs(losses - expected) / np.maximum(np.abs(expected), 1e-30))) <= tol
    grads, final = _leaves(out[1]), _leaves(out[2])
    for i, (g, s) in enumerate(zip(grads, final)):
        for kind, tensor in (("grad", g), ("state", s)):
            want = golden[f"{kind}{i}_sample"]
            got = _sample(tensor)
            err = float(np.max(np.abs(got - want))) / max(float(np.max(np.abs(want))), 1e-30)
            assert err <= tol, f"{name} seed {seed}: {kind}{i} relative error {err:.3e}"
            total, absolute = golden[f"{kind}{i}_checksum"]
            assert abs(float(tensor.double().abs().sum()) - absolute) <= max(tol * absolute, 1e-6), f"{kind}{i} |sum|"


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "gemv"])
def test_twenty_step_graph_replay_matches_oracle(name):
    work = workloads.build(name, seed=0, device="cuda")
    cpu = workloads.build(name, seed=0, device="cpu")
    tol = REL_TOL[work.compute_dtype]
    x0, t0 = work.batches[0]
    compiled = tk.compile_training(work.fn(), (work.state, x0, t0))
    state = work.state
    initial = [p.clone() for p in _leaves(state)]
    for i in range(3):                                   # warm-up outside the graph
        compiled(state, *work.batches[i % len(work.batches)])
    torch.cuda.synchronize()
    for p, saved in zip(_leaves(state), initial):
        p.copy_(saved)
    losses = []
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(20):
            out = compiled(state, *work.batches[i % len(work.batches)])
            losses.append(out[0])
    for p, saved in zip(_leaves(state), initial):
        p.copy_(saved)
    graph.replay()
    torch.cuda.synchronize()
    compiled.runner.status()
    # oracle: the same 20 steps through the CPU interpreter
    program, _ = tk.capture(cpu.fn(), (cpu.state, *cpu.batches[0]))
    ref_state = _leaves(cpu.state)
    n = len(ref_state)
    for i in range(20):
        expected = interpreter.run(program, (*ref_state, *cpu.batches[i % len(cpu.batches)]))
        assert rel_error(losses[i], expected[0]) <= tol, f"{name}: replayed loss {i}"
        ref_state = tuple(e.clone() for e in expected[1 + n:])
    for i, (got, want) in enumerate(zip(_leaves(state), ref_state)):
        assert rel_error(got, want) <= tol, f"{name}: state leaf {i} after replay"
    # a second replay continues from the updated state
    before = [p.clone() for p in _leaves(state)]
    graph.replay()
    torch.cuda.synchronize()
    assert any(not torch.equal(a, b) for a, b in zip(before, _leaves(state)))
