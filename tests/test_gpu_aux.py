"""GPU tests of what surrounds the step kernel: the examples, the stage profiler and its barrier
stall figures, guard bands around everything a kernel writes, and waits that give up and report."""
import re
import subprocess
import sys
from pathlib import Path

import pytest
import torch
from torch.utils._pytree import tree_flatten

import trainkernel_b200 as tk
from tests import cases
from tests.helpers import REL_TOL, assert_outputs_close, oracle_outputs
from trainkernel_b200 import codegen, profile, runtime, workloads
from trainkernel_b200.passes import insert_gradient_exchange

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


# ---------------------------------------------------------------------------------------------
# examples (reference: examples/online_training.py:24-49, examples/train.py)
# ---------------------------------------------------------------------------------------------
def _run_example(name: str) -> str:
    done = subprocess.run([sys.executable, str(ROOT / "examples" / name)], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-2000:]
    return done.stdout


def test_online_training_example_tracks_eager_pytorch():
    text = _run_example("online_training.py")
    match = re.search(r"captured loss ([0-9.eE+-]+)\s+eager loss ([0-9.eE+-]+)\s+max \|parameter difference\| ([0-9.eE+-]+)", text)
    assert match, text
    captured, eager, worst = (float(g) for g in match.groups())
    assert abs(captured - eager) <= 2e-2 * abs(eager)
    assert worst < 1e-3               # 100 steps at lr 1e-3 on parameters of magnitude 0.1


def test_module_training_example_reduces_its_loss():
    text = _run_example("train_module.py")
    losses = [float(v) for v in re.findall(r"loss ([0-9.]+)", text)]
    assert len(losses) >= 4 and losses[-1] < losses[0]


# ---------------------------------------------------------------------------------------------
# stage profiler (reference: scripts/profile_stages.py)
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["c2", "c3"])
def test_stage_profile_is_consistent_with_event_timing(name):
    work = workloads.build(name, device="cuda")
    inputs = (work.state, *work.batches[0])
    records = profile.stage_profile(work.fn(), inputs, repeats=5)
    assert [r["stage"] for r in records] == list(range(len(records)))
    assert all(r["min_us"] >= 0 and r["median_us"] >= r["min_us"] and r["units"] for r in records)
    # one more stamped launch under CUDA events: stamps are monotonic and fit inside the event interval
    compiled = tk.compile_training(work.fn(), inputs, stage_stamps=True)
    for _ in range(3):
        compiled(*inputs)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    begin.record()
    compiled(*inputs)
    end.record()
    end.synchronize()
    stamps = compiled.runner.stage_stamps()
    assert len(stamps) == compiled.runner.generated.stages + 1
    assert all(b >= a for a, b in zip(stamps[:-1], stamps[1:]))
    assert (stamps[-1] - stamps[0]) / 1e6 <= begin.elapsed_time(end) + 0.005      # ms; the timer ticks in ~1 us steps
    stalls = compiled.runner.barrier_stalls()
    if compiled.runner.generated.barrier == "grid":
        assert len(stalls) == compiled.runner.generated.grid_barriers
        for record, profiled in zip(stalls, records):
            # block 0 cannot be released before the last block arrived, nor before it arrived itself
            assert record["release"] >= 0 and record["block0_wait"] >= 0
            assert record["block0_wait"] == record["skew"] + record["release"]
            assert "barrier_wait_us" in profiled and profiled["barrier_release_us"] < 100.0
    else:
        assert stalls == []           # one-cluster kernels synchronise in hardware: nothing to stamp
    # prologue, stages and tail add up to the launch as the device saw it, inside the event interval
    span = compiled.runner.launch_span()
    assert span["prologue"] >= 0 and span["tail"] >= 0 and span["stages"] == stamps[-1] - stamps[0]
    assert span["total"] == span["prologue"] + span["stages"] + span["tail"]
    assert span["total"] / 1e6 <= begin.elapsed_time(end) + 0.005


# ---------------------------------------------------------------------------------------------
# guard bands: nothing outside the declared outputs and workspace may be written
# ---------------------------------------------------------------------------------------------
MARGIN = 4096
POISON = 0xA5


def _guarded(shape, dtype, device):
    """A contiguous tensor of `shape` in the middle of a poisoned byte buffer; returns (tensor, buffer)."""
    count = 1
    for extent in shape:
        count *= extent
    nbytes = count * torch.empty((), dtype=dtype).element_size()
    padded = -(-nbytes // 256) * 256
    raw = torch.full((padded + 2 * MARGIN,), POISON, dtype=torch.uint8, device=device)
    view = raw[MARGIN:MARGIN + nbytes].view(dtype).view(shape)
    return view, raw, nbytes


def _margins_intact(raw, nbytes) -> bool:
    return bool((raw[:MARGIN] == POISON).all()) and bool((raw[MARGIN + nbytes:] == POISON).all())


@pytest.mark.parametrize("name", ["gemm_kn_ragged", "gemm2_ragged_t", "mlp_bf16", "c3", "gemm_odd_bf16", "big_reduce"])
def test_kernels_stay_inside_their_outputs_and_workspace(name):
    fn, inputs, kind, options = cases.build(name, "cuda")
    _, cpu_inputs, _, _ = cases.build(name, "cpu")
    compiled = getattr(tk, kind)(fn, inputs, **options)
    runner = compiled.runner
    flat, _ = tree_flatten(inputs)
    expected = oracle_outputs(compiled.program, cpu_inputs)
    guards = []
    # in-place targets are inputs: move them into guarded storage too
    flat = list(flat)
    for target in set(runner.inplace_outputs.values()):
        view, raw, nbytes = _guarded(tuple(flat[target].shape), flat[target].dtype, flat[target].device)
        view.copy_(flat[target])
        flat[target] = view
        guards.append((f"state input {target}", raw, nbytes))
    outputs = []
    for slot, spec in enumerate(runner.program.outputs):
        if slot in runner.inplace_outputs:
            outputs.append(flat[runner.inplace_outputs[slot]])
            continue
        view, raw, nbytes = _guarded(spec.shape, getattr(torch, spec.dtype), runner.device)
        outputs.append(view)
        guards.append((f"output {slot}", raw, nbytes))
    workspace, raw, nbytes = _guarded((runner.generated.workspace_elements,), torch.float32, runner.device)
    guards.append(("workspace", raw, nbytes))
    got = runner.run_into(*flat, buffers=runtime.ExecutionBuffers(tuple(outputs), workspace))
    torch.cuda.synchronize()
    runner.status()
    for label, raw, nbytes in guards:
        assert _margins_intact(raw, nbytes), f"{name}: bytes next to {label} were overwritten"
    dtypes = {t.dtype for t in flat}
    tol = 1e-5 if dtypes == {torch.float32} else 2e-2
    assert_outputs_close(got, expected, tol, name)


# ---------------------------------------------------------------------------------------------
# a wait for a peer that never signals gives up, reports, and leaves the context usable
# ---------------------------------------------------------------------------------------------
def test_peer_flag_wait_gives_up_and_reports():
    """A two-rank step kernel is launched on ONE GPU with a second local buffer standing in for the
    peer; nobody ever raises that peer's flags.  The kernel must come back after its (20 ms) limit with
    the peer-flag error code, further launches must be refused until the module is reset, and after
    the reset the context must still run a correct step."""
    device = torch.device("cuda", 0)
    shard = workloads.mlp_workload("shard", (128, 256, 128), 16, seed=0, device=device, rows=slice(0, 8))
    x, t = shard.batches[0]
    program, _ = tk.capture(shard.fn(), (shard.state, x, t))
    n = len(shard.state)
    inplace = {1 + n + i: i for i in range(n)}
    generated = codegen.generate(insert_gradient_exchange(program, n), inplace_outputs=inplace, world=2)
    assert generated.world == 2 and "tk::dp_wait" in generated.source
    words = generated.symmetric_bytes // 4
    mine = torch.zeros(words, dtype=torch.int32, device=device)
    silent = torch.zeros(words, dtype=torch.int32, device=device)      # the peer that never runs
    silent[1] = 1
    torch.cuda.synchronize()
    module = runtime._Module(generated, runtime.build_cubin(generated.source), device)
    checker = runtime.CompiledProgram(program, generated, module, device, inplace)
    lib = runtime.library()
    lib.tk_module_set_timeout(module.handle, 20_000_000)
    state = tuple(p.clone() for p in shard.state)
    outputs = (torch.zeros((), device=device), *[torch.empty_like(p) for p in state], *state)
    workspace = torch.empty(generated.workspace_elements, dtype=torch.float32, device=device)
    extra = [mine, mine, silent]
    stream = torch.cuda.current_stream(device).cuda_stream
    module.launch(checker.launch_inputs((*state, x, t, *extra)), outputs, workspace, stream)
    with pytest.raises(RuntimeError, match=r"timed out \(code 6,"):
        checker.status()
    with pytest.raises(RuntimeError, match="tk_module_reset"):
        module.launch(checker.launch_inputs((*state, x, t, *extra)), outputs, workspace, stream)
    assert lib.tk_module_reset(module.handle) == 0
    # the context is intact: an ordinary step of the same shapes matches the oracle
    work = workloads.build("c2", device="cuda")
    cpu = workloads.build("c2", device="cpu")
    step = tk.compile_training(work.fn(), (work.state, *work.batches[0]))
    out = step(work.state, *work.batches[0])
    step.runner.status()
    expected = oracle_outputs(step.program, (cpu.state, *cpu.batches[0]))
    assert_outputs_close(out, expected, REL_TOL[torch.bfloat16], "step after the timed-out launch")


# ---------------------------------------------------------------------------------------------
# BF16 weight copies carried from one launch to the next
# ---------------------------------------------------------------------------------------------
def _oracle_step(program, state, batch):
    from oracle import interpreter
    n = len(state)
    out = interpreter.run(program, (*state, *batch))
    return out, tuple(e.clone() for e in out[1 + n:])


@pytest.mark.parametrize("form", ["pingpong", "reorder"])
def test_carried_weight_copies_follow_every_edit_of_the_state(form):
    """The step kernel keeps the BF16 copies of its master weights between launches and skips re-casting them
    when the state tensors are untouched.  Every way of touching them must still give the oracle's result:
    an in-place PyTorch operation (seen through the version counter), a write PyTorch cannot see followed by
    `invalidate_carried()`, and a CUDA-graph replay that starts from restored state."""
    tol = REL_TOL[torch.bfloat16]
    work = workloads.build("c4", device="cuda")
    cpu_program, _ = tk.capture(work.fn(), (work.state, *work.batches[0]))
    compiled = tk.compile_training(work.fn(), (work.state, *work.batches[0]), stage_stamps=True, carry_shadows=form)
    runner = compiled.runner
    copies = 2 if form == "pingpong" else 1
    assert runner.generated.carry_bytes == copies * 2 * work.weight_elements and runner.carried is not None
    state = work.state
    reference = tuple(p.clone() for p in state)
    first_stage = []

    def step_and_check(label, batch):
        nonlocal reference
        expected, reference = _oracle_step(cpu_program, reference, batch)
        out = compiled(state, *batch)
        runner.status()
        stamps = runner.stage_stamps()
        first_stage.append(stamps[1] - stamps[0])
        for index, (got, want) in enumerate(zip([out[0], *out[1], *out[2]], expected)):
            err = float((got.float() - want.float()).abs().max()) / max(float(want.float().abs().max()), 1e-30)
            assert err <= tol, f"{label}: output {index} is {err:.3e} from the oracle"

    step_and_check("first launch (casts)", work.batches[0])
    step_and_check("second launch (carried)", work.batches[1])
    step_and_check("third launch (carried)", work.batches[2])
    assert min(first_stage[1:]) < 0.6 * first_stage[0], f"the casting stage was not skipped: {first_stage}"
    # an in-place edit PyTorch can see
    with torch.no_grad():
        state[0].mul_(0.5)
        state[2].add_(0.01)
    reference = tuple(p.clone() for p in state)
    step_and_check("after an in-place edit", work.batches[3])
    # a write the version counters do not see, declared by the caller
    state[4].data.mul_(2.0)
    runner.invalidate_carried()
    reference = tuple(p.clone() for p in state)
    step_and_check("after invalidate_carried", work.batches[0])
    # graph replays start from whatever state they find
    saved = [p.clone() for p in state]
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(3):
            compiled(state, *work.batches[i])
    results = []
    for scale in (1.0, 0.25):
        for p, s in zip(state, saved):
            p.copy_(s * scale)
        reference = tuple(p.clone() for p in state)
        graph.replay()
        torch.cuda.synchronize()
        runner.status()
        for i in range(3):
            _, reference = _oracle_step(cpu_program, reference, work.batches[i])
        for index, (got, want) in enumerate(zip(state, reference)):
            err = float((got - want).abs().max()) / max(float(want.abs().max()), 1e-30)
            assert err <= tol, f"replay from state x {scale}: parameter {index} is {err:.3e} from the oracle"


# ---------------------------------------------------------------------------------------------
# programmatic dependent launch: a step may start while its predecessor is still finishing
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["c1", "c2", "c3"])
def test_early_launch_gives_bit_identical_steps(name):
    """With `tk_module_set_early_launch` a kernel is allowed to start its prologue before the previous
    kernel on the stream has finished; it waits for it inside the kernel before touching memory.  Twenty
    back-to-back steps (eager and as a CUDA graph) must leave exactly the state an ordinary launch leaves."""
    def leaves(state):
        return tuple(state) if isinstance(state, (tuple, list)) else (state,)

    finals = {}
    for early in (False, True):
        work = workloads.build(name, device="cuda")
        compiled = tk.compile_training(work.fn(), (work.state, *work.batches[0]))
        assert runtime.library().tk_module_set_early_launch(compiled.runner.module.handle, int(early)) == 0
        initial = [p.clone() for p in leaves(work.state)]
        for i in range(20):
            compiled(work.state, *work.batches[i % len(work.batches)])
        torch.cuda.synchronize()
        compiled.runner.status()
        eager_final = [p.clone() for p in leaves(work.state)]
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(20):
                compiled(work.state, *work.batches[i % len(work.batches)])
        for p, saved in zip(leaves(work.state), initial):
            p.copy_(saved)
        graph.replay()
        torch.cuda.synchronize()
        compiled.runner.status()
        for a, b in zip(leaves(work.state), eager_final):
            assert torch.equal(a, b), f"{name}: graph replay differs from the eager loop (early={early})"
        finals[early] = eager_final
    for a, b in zip(finals[False], finals[True]):
        assert torch.equal(a, b), f"{name}: early launch changed the result"
