"""Captured-training-step benchmark on B200.

    python bench.py --gpus N --steps K --warmup W            # this back end
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU path on the host cores

A step is one forward + loss + backward + FP32-master SGD pass of the medium MLP
(4 layers 4096-8192-8192-8192-4096, global batch 8192, BF16 compute) over one
resident synthetic batch.  At N = 1 the whole step is ONE generated sm_100a
kernel replayed from a CUDA graph.  At N > 1 the batch is split evenly over the
ranks (strong scaling); each rank still replays ONE kernel per step, which averages
the BF16 gradients with its peers over NVLink peer memory between the backward
GEMMs and the updates (--dp nccl selects the baseline: gradient kernel -> NCCL
all-reduce -> update kernel).  Exactly K steps are timed with CUDA
events between barrier + synchronize pairs and the maximum over ranks is
reported.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

MEDIUM_SIZES = (4096, 8192, 8192, 8192, 4096)
MEDIUM_BATCH = 8192
TRAFFIC_FILE = ROOT / "profiles" / "dram_traffic.json"


def measured_traffic(generated) -> float | None:
    """DRAM bytes per launch of exactly this kernel (ncu dram__bytes_read.sum + dram__bytes_write.sum of a
    one-pass capture), looked up by the hash of the generated source and device headers; None when the
    kernel has changed since the capture was taken."""
    from trainkernel_b200 import runtime
    try:
        table = json.loads(TRAFFIC_FILE.read_text())
    except (OSError, ValueError):
        return None
    entry = table.get(runtime.cubin_path(generated.source).stem)
    return float(entry["bytes"]) if entry else None


def _peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": data["hbm_gbs"], "tflops": data["bf16_tflops_sustained"], "tflops_burst": data["bf16_tflops"],
                "source": "measured (MEASURED_PEAKS.json, sustained bf16 figure)"}
    return {"hbm_gbs": 6650.0, "tflops": 1400.0, "tflops_burst": 1590.0, "source": "fallback"}


def _medium_program(batch: int):
    """Capture the medium MLP step on meta tensors (shapes only)."""
    import trainkernel_b200 as tk
    from trainkernel_b200 import workloads
    state = []
    for fan_in, fan_out in zip(MEDIUM_SIZES[:-1], MEDIUM_SIZES[1:]):
        state += [torch.empty(fan_in, fan_out, device="meta"), torch.empty(fan_out, device="meta")]
    x = torch.empty(batch, MEDIUM_SIZES[0], dtype=torch.bfloat16, device="meta")
    t = torch.empty(batch, MEDIUM_SIZES[-1], dtype=torch.bfloat16, device="meta")
    program, _ = tk.capture(lambda s, xx, tt: workloads.mlp_master_step(s, xx, tt, 1e-3), (tuple(state), x, t))
    return program


def kernel_sources() -> dict[str, str]:
    """Generated sources of every kernel this benchmark launches (for ahead-of-time compilation)."""
    from trainkernel_b200 import codegen
    from trainkernel_b200.passes import split_at_gradients
    count = 2 * (len(MEDIUM_SIZES) - 1)
    sources = {"medium_n1": codegen.generate(_medium_program(MEDIUM_BATCH),
                                             inplace_outputs={1 + count + i: i for i in range(count)}).source}
    for world in (2, 4, 8):
        gradient, update = split_at_gradients(_medium_program(MEDIUM_BATCH // world), count, narrow_exchange=True)
        sources[f"medium_grad_n{world}"] = codegen.generate(gradient).source
        if world == 2:
            sources["medium_update"] = codegen.generate(update, inplace_outputs={count + i: i for i in range(count)}).source
        from trainkernel_b200.passes import insert_gradient_exchange
        fused = insert_gradient_exchange(_medium_program(MEDIUM_BATCH // world), count)
        for multicast in (False, True):
            name = f"medium_fused_n{world}" + ("_multicast" if multicast else "")
            sources[name] = codegen.generate(fused, inplace_outputs={1 + count + i: i for i in range(count)}, world=world,
                                             multicast=multicast, background=multicast or world >= 4).source
    return sources


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.lines: list[str] = []
        self.process = None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                             "--format=csv,noheader,nounits", "-lms", "20"],
                                            stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _pump(self):
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def wait_first(self, seconds: float = 3.0) -> None:
        """Block until nvidia-smi has produced its first line (it takes a few hundred ms to start)."""
        deadline = time.monotonic() + seconds
        while self.process is not None and not self.lines and time.monotonic() < deadline:
            time.sleep(0.01)

    def mark(self) -> None:
        """Forget the samples taken so far: what follows is the region under load."""
        del self.lines[:]

    def count(self) -> int:
        return len(self.lines)

    def __exit__(self, *exc):
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.process.kill()

    def summary(self) -> dict:
        clocks, maxima, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                clocks.append(float(parts[0]))
                maxima.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[4:8]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(clocks), "sm_max_mhz": max(maxima), "reasons": sorted(reasons), "samples": len(clocks)}


def _leaves(state):
    return tuple(state) if isinstance(state, (tuple, list)) else (state,)


WORKLOAD_TEXT = "{name} medium MLP {sizes}, global batch {batch}, BF16 compute / FP32 master, SGD lr 1e-3"


def _workload_text(name: str) -> str:
    return WORKLOAD_TEXT.format(name=name, sizes="-".join(map(str, MEDIUM_SIZES)), batch=MEDIUM_BATCH)


def _time_cpu(call, limit: int, budget_s: float) -> list[float]:
    """Wall-clock seconds of up to `limit` calls, stopping once `budget_s` has been spent (at least one)."""
    samples, spent = [], 0.0
    while len(samples) < limit and (not samples or spent + samples[-1] <= budget_s):
        begin = time.perf_counter()
        call()
        samples.append(time.perf_counter() - begin)
        spent += samples[-1]
    return samples


def cpu_baseline(steps: int = 3, budget_s: float = 25.0) -> dict:
    """Time FULL medium-MLP steps of the reference's CPU path on the host cores.

    Two forms, both on CPU tensors with every host thread: the IR-interpreter oracle (a port of the
    reference's reference.py) and eager PyTorch running the step function itself.  Up to `steps`
    whole steps each (one at least, more while they fit in `budget_s`), after a warm-up on 256 rows
    that spins the thread pool up; the median is reported.
    """
    import trainkernel_b200 as tk
    from oracle import interpreter
    from trainkernel_b200 import workloads
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    work = workloads.mlp_workload("cpu", MEDIUM_SIZES, MEDIUM_BATCH, seed=0, device="cpu", resident=1)
    x, t = work.batches[0]
    fn = work.fn()
    small, _ = tk.capture(fn, (work.state, x[:256], t[:256]))
    interpreter.run(small, (*work.state, x[:256].contiguous(), t[:256].contiguous()))
    program, _ = tk.capture(fn, (work.state, x, t))
    oracle_s = _time_cpu(lambda: interpreter.run(program, (*work.state, x, t)), steps, budget_s)
    eager_s = _time_cpu(lambda: fn(work.state, x, t), steps, budget_s)
    per_step = statistics.median(oracle_s)
    return {"value": 1.0 / per_step, "unit": "steps/s", "cores": threads, "kind": "port",
            "sample": f"{len(oracle_s)} full step(s) of the IR-interpreter oracle on CPU tensors (all {MEDIUM_BATCH} rows, full-size weights), "
                      f"median {per_step:.2f} s per step; eager PyTorch on the same tensors: {len(eager_s)} step(s), median {statistics.median(eager_s):.2f} s",
            "steps_timed": len(oracle_s), "seconds_per_step": per_step,
            "eager": {"value": 1.0 / statistics.median(eager_s), "unit": "steps/s", "steps_timed": len(eager_s)}}


def run_reference(args) -> None:
    """The reference arm: whole steps of the reference's CPU path, timed on the host cores by rank 0."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base = cpu_baseline(max(1, min(args.steps, 3)))
    timed = base["steps_timed"]
    line = {
        "impl": "reference", "metric": "captured_step_throughput", "value": base["value"], "unit": "steps/s",
        "n_gpus": args.gpus, "steps": timed, "warmup": 1, "ms_per_step": 1e3 / base["value"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": _config(args.workload, args.gpus, MEDIUM_BATCH // max(1, args.gpus), 4),
        "execution": {"how": "IR-interpreter oracle on CPU tensors, all host threads, rank 0 only", "graph_steps": 0},
        "requested": {"steps": args.steps, "warmup": args.warmup,
                      "note": "a CPU step takes seconds: at most 3 whole steps are timed after a 256-row warm-up"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def _config(workload: str, world: int, rows_per_rank: int, resident: int) -> dict:
    """The `config` object: what the workload IS, built the same way by both arms so that the two lines carry
    equal objects; how an arm executes it (parallelism, graph length) goes under `execution`."""
    config = {"workload": _workload_text(workload), "global_batch": MEDIUM_BATCH, "rows_per_rank": rows_per_rank,
              "resident_batches": resident,
              "l2": "inputs larger than L2 (FP32 weights %d MB, %d MB per batch)" % (
                  sum(a * b for a, b in zip(MEDIUM_SIZES[:-1], MEDIUM_SIZES[1:])) * 4 // 2**20,
                  rows_per_rank * (MEDIUM_SIZES[0] + MEDIUM_SIZES[-1]) * 2 // 2**20)}
    return config


def small_cpu_baseline(work_name: str) -> dict:
    """Median seconds per step of the oracle and of eager PyTorch on CPU tensors for a small configuration
    (100 steps; 10 for the small MLP), state carried from step to step as in training."""
    import trainkernel_b200 as tk
    from oracle import interpreter
    from trainkernel_b200 import workloads
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    steps = 10 if work_name == "c4" else 100
    result = {"cores": threads, "steps_timed": steps}
    for kind in ("oracle", "eager"):
        work = workloads.build(work_name, device="cpu")
        fn = work.fn()
        program, _ = tk.capture(fn, (work.state, *work.batches[0]))
        state = work.state
        samples = []
        for i in range(steps + 2):
            x, t = work.batches[i % len(work.batches)]
            begin = time.perf_counter()
            if kind == "oracle":
                out = interpreter.run(program, (*_leaves(state), x, t))
                count = len(_leaves(state))
                new = out[1 + count:]
                state = tuple(new) if isinstance(state, (tuple, list)) else new[0]
            else:
                state = fn(state, x, t)[2]
            if i >= 2:
                samples.append(time.perf_counter() - begin)
        result[f"{kind}_us_per_step"] = round(statistics.median(samples) * 1e6, 1)
    return result


def _percentiles(samples: list[float]) -> dict:
    ordered = sorted(samples)
    pick = lambda q: ordered[min(len(ordered) - 1, int(round(q * (len(ordered) - 1))))]  # noqa: E731
    return {"p10": round(pick(0.1), 2), "p50": round(statistics.median(ordered), 2), "p90": round(pick(0.9), 2),
            "min": round(ordered[0], 2), "max": round(ordered[-1], 2), "replays": len(ordered)}


def small_config_latencies(cpu: bool) -> dict:
    """Graph-replay latency (us per step; 30 timed replays of a 20-step graph after 10 warm-up replays) of
    the small configurations, with the CPU path's time per step beside it when `cpu` is set."""
    import trainkernel_b200 as tk
    from trainkernel_b200 import workloads
    result = {}
    for name in ("c1", "c2", "c3", "c4"):
        work = workloads.build(name, device="cuda")
        x0, t0 = work.batches[0]
        compiled = tk.compile_training(work.fn(), (work.state, x0, t0))
        for i in range(3):
            compiled(work.state, *work.batches[i % len(work.batches)])
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(20):
                compiled(work.state, *work.batches[i % len(work.batches)])
        for _ in range(10):
            graph.replay()
        torch.cuda.synchronize()
        samples = []
        for _ in range(30):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            b.synchronize()
            samples.append(a.elapsed_time(b) * 1e3 / 20)
        compiled.runner.status()
        spread = _percentiles(samples)
        p50 = spread["p50"]
        bound_us = max(work.flops_per_step() / (_peaks()["tflops"] * 1e12), work.bytes_per_step() / (_peaks()["hbm_gbs"] * 1e9)) * 1e6
        result[work.name] = {"latency_us_p50": p50, "latency_us": spread, "steps_per_s": round(1e6 / p50, 1),
                             "grid_barriers": compiled.runner.generated.grid_barriers,
                             "barrier": compiled.runner.generated.barrier, "blocks": compiled.runner.module.grid,
                             "roofline_us": round(bound_us, 3), "roofline_frac": round(bound_us / p50, 4)}
        if cpu:
            result[work.name]["cpu_baseline"] = small_cpu_baseline(name)
        del graph, compiled
    return result


def parity_check(step, state, initial, graph, losses, last_out, steps: int, world: int, rank: int, device, resident: int) -> dict:
    """Replay the timed graph once more from the saved initial state and compare every replayed loss, the
    last step's gradients and the final parameters with the IR-interpreter oracle evaluated on CUDA
    tensors over the FULL batch (outside any timed region).  The oracle here is the checker only."""
    import torch.distributed as dist
    import trainkernel_b200 as tk
    from oracle import interpreter
    from trainkernel_b200 import workloads
    for leaf, saved in zip(_leaves(state), initial):
        leaf.copy_(saved)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    graph.replay()
    torch.cuda.synchronize()
    full = workloads.mlp_workload("oracle", MEDIUM_SIZES, MEDIUM_BATCH, seed=0, device=device, resident=resident)
    reference = tuple(p.clone() for p in initial)
    program, _ = tk.capture(full.fn(), (reference, *full.batches[0]))
    count = len(reference)

    def rel(a, b):
        return float((a.float() - b.float()).abs().max()) / max(float(b.float().abs().max()), 1e-30)

    worst, where, expected = 0.0, "", None
    for i in range(steps):
        expected = interpreter.run(program, (*reference, *full.batches[i % len(full.batches)]))
        err = rel(losses[i], expected[0])
        if err > worst:
            worst, where = err, f"loss of step {i}"
        reference = tuple(e.clone() for e in expected[1 + count:])
    gradient_outliers = []
    for i, (got, want) in enumerate(zip(_leaves(last_out[1]), expected[1:1 + count])):
        err = rel(got, want)
        if err > 2e-2:
            # After many steps the two runs' parameters differ by rounding, so a pre-ReLU value next to zero can get
            # the other mask, which moves one column of a weight gradient by one of its 1/batch terms.  Such a
            # tensor must still agree in the L2 norm and in all but one element in a thousand.
            l2 = float((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-30))
            beyond = float(((got.float() - want.float()).abs() > 2e-2 * want.float().abs().max()).float().mean())
            gradient_outliers.append({"gradient": i, "max": err, "l2": l2, "fraction_beyond": beyond})
            if l2 <= 2e-2 and beyond <= 1e-3:
                continue
        if err > worst:
            worst, where = err, f"gradient {i} of the last step"
    for i, (got, want) in enumerate(zip(_leaves(state), reference)):
        err = rel(got, want)
        if err > worst:
            worst, where = err, f"parameter {i} after {steps} steps"
    if world > 1:
        collected = torch.tensor([worst], device=device)
        dist.all_reduce(collected, op=dist.ReduceOp.MAX)
        worst = float(collected)
    return {"oracle": "IR interpreter on CUDA tensors, full batch, from the same initial state", "steps": steps,
            "compared": f"{steps} losses, {count} gradients of the last step, {count} parameters",
            "worst_rel_error": worst, "worst_at": where, "tolerance": 2e-2, "gradient_outliers": gradient_outliers,
            "passed": bool(worst <= 2e-2)}


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-small-configs", action="store_true")
    parser.add_argument("--no-e2e", action="store_true")
    parser.add_argument("--no-parity", action="store_true", help="skip the oracle check of the replayed steps (for profiler runs)")
    parser.add_argument("--latency-replays", type=int, default=30, help="timed graph replays for the latency distribution (after 10 warm-ups)")
    parser.add_argument("--workload", default="c5", choices=["c5", "c5_half"],
                        help="c5_half (2048-4096-4096-4096-2048, batch 4096) is the small case used for ncu captures")
    parser.add_argument("--eager", action="store_true", help="launch the timed steps directly instead of replaying a CUDA graph")
    parser.add_argument("--single-cta", action="store_true",
                        help="generate the kernel with cta_group::1 128x256 tiles instead of two-CTA pair tiles "
                             "(the variant ncu can profile: ncu fails to launch the clustered cooperative kernel)")
    parser.add_argument("--dp", default="fused", choices=["fused", "nccl"],
                        help="N > 1: gradient exchange inside the step kernel over NVLink peer memory (fused), or "
                             "gradient kernel -> NCCL all-reduce -> update kernel (nccl, the measured baseline)")
    parser.add_argument("--no-cooperative", action="store_true",
                        help="N = 1: launch the step kernel without the cooperative-launch attribute (its grid already "
                             "fits the idle device and its waits are bounded); for hardware profilers that cannot "
                             "replay cooperative cluster launches")
    parser.add_argument("--no-stream-warps", action="store_true",
                        help="N > 1, fused: generate the step kernel without the four stream warps per block that run the "
                             "gradient exchange and the FP32 updates beside the GEMM tiles (for A/B measurements)")
    parser.add_argument("--stream-warps", action="store_true", help="N > 1, fused: stream warps even below the rank count they default from (A/B measurements)")
    parser.add_argument("--multicast", action="store_true", help="N > 1, fused: require the NVSwitch multicast form even below the rank count it defaults from")
    parser.add_argument("--exchange-chunks", type=int, default=None, help="N > 1, fused: owned chunks per exchange work item, 8 or 16 (A/B measurements)")
    parser.add_argument("--stream-everything", action="store_true",
                        help="N > 1, fused: give every pointwise stream to the stream warps, whether the stage's GEMMs cover it or not (A/B measurements)")
    parser.add_argument("--stream-piece", type=int, default=None, help="N > 1, fused: slices per background piece (A/B measurements)")
    parser.add_argument("--no-multicast", action="store_true",
                        help="N > 1, fused: never exchange through the NVSwitch multicast mapping (multimem); "
                             "contributions are then scattered to their owners with plain peer stores")
    args = parser.parse_args()
    global MEDIUM_SIZES, MEDIUM_BATCH
    if args.workload == "c5_half":
        MEDIUM_SIZES, MEDIUM_BATCH = (2048, 4096, 4096, 4096, 2048), 4096
    if args.impl == "reference":
        run_reference(args)
        return

    import torch.distributed as dist
    import trainkernel_b200 as tk
    from trainkernel_b200 import dp, runtime, workloads

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    torch.backends.cuda.matmul.allow_tf32 = False
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    steps, warmup = args.steps, max(3, args.warmup)

    rows = dp.shard_rows(MEDIUM_BATCH, rank, world)
    work = workloads.mlp_workload("c5_medium_mlp" if args.workload == "c5" else "c5_half_mlp", MEDIUM_SIZES, MEDIUM_BATCH,
                                  seed=0, device=device, rows=rows)
    state = work.state
    x0, t0 = work.batches[0]
    if world == 1:
        step = tk.compile_training(work.fn(), (state, x0, t0), **({"two_cta": False} if args.single_cta else {}))
        kernels_per_step = 1
        status = step.runner.status
        generated = step.runner.generated
        if args.no_cooperative:
            runtime.library().tk_module_set_cooperative(step.runner.module.handle, 0)
            # should the blocks not all be resident after all, give up on a barrier after 0.2 s instead of 2 s
            runtime.library().tk_module_set_timeout(step.runner.module.handle, 200_000_000)
    elif args.dp == "fused":
        step = dp.FusedShardedTrainingStep(work.fn(), (state, x0, t0), multicast=False if args.no_multicast else (True if args.multicast else None),
                                           **({"background": False} if args.no_stream_warps else ({"background": True} if args.stream_warps else {})),
                                           **({"stream_piece": args.stream_piece} if args.stream_piece else {}),
                                           **({"stream_everything": True} if args.stream_everything else {}),
                                           **({"exchange_chunks": args.exchange_chunks} if args.exchange_chunks else {}))
        kernels_per_step = step.kernels_per_step
        status = step.status
        generated = step.generated
    else:
        step = dp.ShardedTrainingStep(work.fn(), (state, x0, t0))
        kernels_per_step = step.kernels_per_step
        status = step.status
        generated = step.gradient.generated

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(warmup):
        step(state, *work.batches[i % len(work.batches)])
        if i == 0 and world > 1 and args.dp == "fused" and step.multicast:
            # The multicast form depends on the fabric accepting multimem accesses from inside this kernel.
            # Its waits are bounded, so a refusal shows up as an error status, not a hang: if ANY rank
            # reports one after the first step, every rank rebuilds the step in the peer-store form.
            torch.cuda.synchronize()
            failed = torch.zeros(1, dtype=torch.int32, device=device)
            try:
                status()
            except RuntimeError as error:
                print(f"[bench] rank {rank}: multicast exchange failed on its first step ({error}); using peer stores", file=sys.stderr)
                failed += 1
            dist.all_reduce(failed, op=dist.ReduceOp.MAX)
            if int(failed.item()):
                step.close()                 # unmap the peer-mapped buffer on every rank before a new one is made
                del step
                barrier()
                work = workloads.mlp_workload(work.name, MEDIUM_SIZES, MEDIUM_BATCH, seed=0, device=device, rows=rows)
                state = work.state
                step = dp.FusedShardedTrainingStep(work.fn(), (state, *work.batches[0]), multicast=False, **({"background": False} if args.no_stream_warps else {}))
                status, generated = step.status, step.generated
                step(state, *work.batches[0])
    barrier()
    initial = None if args.no_parity else [p.clone() for p in _leaves(state)]
    losses = []
    last_out = [None]
    if args.eager:
        class _Eager:
            def replay(self):
                losses.clear()
                for i in range(steps):
                    last_out[0] = step(state, *work.batches[i % len(work.batches)])
                    losses.append(last_out[0][0].clone())
        graph = _Eager()
    else:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(steps):
                out = step(state, *work.batches[i % len(work.batches)])
                losses.append(out[0].clone() if world > 1 else out[0])   # sharded steps reuse one loss buffer
                last_out[0] = out
    graph.replay()                       # one untimed replay: graph upload, allocator settled
    barrier()
    launches_before = runtime.library().tk_launch_count()
    with ClockSampler(local) as sampler:
        sampler.wait_first()
        graph.replay()                   # back under load before the samples that count
        barrier()
        sampler.mark()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        begin.record()
        graph.replay()
        end.record()
        barrier()
        elapsed_ms = begin.elapsed_time(end)
        # further replays only for the latency distribution: 10 warm-ups, then `--latency-replays` timed ones
        samples = [elapsed_ms / steps * 1e3]
        settle = 10 if args.latency_replays > 1 else 0       # --latency-replays 1: profiler runs, as few launches as possible
        for i in range(settle + max(0, args.latency_replays - 1)):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            a.record()
            graph.replay()
            b.record()
            barrier()
            if i >= settle:
                samples.append(a.elapsed_time(b) / steps * 1e3)
    status()
    clocks = sampler.summary()
    if world > 1:
        worst = torch.tensor([elapsed_ms], device=device)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        elapsed_ms = float(worst)
        sample_tensor = torch.tensor(samples, device=device)
        dist.all_reduce(sample_tensor, op=dist.ReduceOp.MAX)
        samples = [float(v) for v in sample_tensor]
    assert bool(torch.isfinite(losses[-1])), "loss diverged"

    # per-rank gradient-kernel duration for the roofline (CUDA events on the launching stream)
    kernel_ms = elapsed_ms / steps
    if world > 1 and args.dp == "nccl":
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        flat = tuple(_leaves(state)) + work.batches[0]
        stream = torch.cuda.current_stream().cuda_stream
        torch.cuda.synchronize()
        a.record()
        for _ in range(5):
            step.gradient.module.launch(step.gradient.launch_inputs(flat), (step.loss, *step.views), step.gradient_workspace, stream)
        b.record()
        b.synchronize()
        kernel_ms = a.elapsed_time(b) / 5
    peaks = _peaks()
    local_flops = 4 * work.batch * work.weight_elements + 2 * work.batch * (work.weight_elements - MEDIUM_SIZES[0] * MEDIUM_SIZES[1])
    achieved = local_flops / (kernel_ms * 1e-3) / 1e12
    roofline = {"bound": "tensor", "achieved": round(achieved, 1), "peak": peaks["tflops"], "unit": "TFLOP/s",
                "frac": round(achieved / peaks["tflops"], 4), "traffic": measured_traffic(generated) if world == 1 else None,
                "peak_source": peaks["source"], "kernel_ms": round(kernel_ms, 4),
                "algorithmic_flops_per_launch": local_flops, "frac_of_burst_peak": round(achieved / peaks["tflops_burst"], 4)}

    # end to end: host batches in pinned memory, copied in every step; the loss is read back every step
    e2e = None
    if not args.no_e2e:
        e2e = measure_e2e(step, state, work, steps, world, device)

    parity = None
    if not args.no_parity:
        parity = parity_check(step, state, initial, graph, losses, last_out[0], steps, world, rank, device, len(work.batches))
        if not parity["passed"]:
            print(f"[bench] PARITY FAILED: {parity}", file=sys.stderr)
    final_loss = float(losses[-1])

    parallelism = (f"dp{world} (batch-sharded, BF16 gradient mean exchanged inside the step kernel over NVLink, "
                   + ("multimem.ld_reduce / multimem.st through the NVSwitch multicast mapping)" if getattr(step, "multicast", False)
                      else "peer stores into the owners' staging areas)")
                   if world > 1 and args.dp == "fused" else
                   f"dp{world} (batch-sharded, NCCL all-reduce of the BF16 gradients between two kernels)" if world > 1
                   else "single GPU, one kernel per step")
    line = {
        "metric": "captured_step_throughput", "value": steps / (elapsed_ms * 1e-3), "unit": "steps/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": elapsed_ms / steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": _config(args.workload, world, work.batch, len(work.batches)),
        "execution": {"parallelism": parallelism, "graph_steps": 0 if args.eager else steps},
        "latency_us": _percentiles(samples),
        "clocks": clocks, "roofline": roofline, "e2e": e2e,
        "gpu_launches": steps * kernels_per_step,
        "kernel": {"stages": generated.stages, "grid_barriers": generated.grid_barriers, "grid": generated.grid,
                   "tensor_core_units": generated.tensor_core_operations, "workspace_bytes": generated.workspace_bytes},
        "parity_checked": bool(parity and parity["passed"]), "parity": parity,
        "final_loss": final_loss,
        "shim_launches_recorded": int(runtime.library().tk_launch_count() - launches_before),
    }
    if world > 1:
        # Leave in order: the graphs first (they pin the communicator's kernels), then the step (which
        # unmaps the peer-mapped buffer and its multicast binding), and only then the process group, so
        # that no rank's memory goes away while a peer still has it mapped.
        del graph, out, last_out, losses
        if hasattr(step, "close"):
            step.close()
        del step
        import gc
        gc.collect()
        barrier()
        guard = threading.Timer(60.0, lambda: os._exit(0))     # a teardown that blocks must not hold the box
        guard.daemon = True
        guard.start()
        if rank == 0:
            print(json.dumps(line), flush=True)
        dist.destroy_process_group()
        guard.cancel()
        return
    if not args.no_small_configs:
        line["other_configs"] = small_config_latencies(cpu=not args.no_cpu_baseline)
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line), flush=True)


def measure_e2e(step, state, work, steps: int, world: int, device) -> dict:
    """Steps/s through the public call with host-resident batches.

    Every step copies its batch (x, target) from pinned host memory on a copy stream into one of
    two device buffer pairs while the previous step computes, runs the step, and copies the loss
    back to the host.
    """
    import torch.distributed as dist
    host = [(x.cpu().pin_memory(), t.cpu().pin_memory()) for x, t in work.batches]
    buffers = [(torch.empty_like(work.batches[0][0]), torch.empty_like(work.batches[0][1])) for _ in range(2)]
    copy_stream = torch.cuda.Stream(device)
    main = torch.cuda.current_stream(device)
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]
    loss_host = torch.zeros(steps, dtype=torch.float32).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host[0])

    def prefetch(i: int) -> None:
        slot = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])
            buffers[slot][0].copy_(host[i % len(host)][0], non_blocking=True)
            buffers[slot][1].copy_(host[i % len(host)][1], non_blocking=True)
            ready[slot].record(copy_stream)

    def run(count: int, record: bool) -> float:
        for slot in range(2):
            consumed[slot].record(main)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(main)
        prefetch(0)
        for i in range(count):
            if i + 1 < count:
                prefetch(i + 1)
            slot = i % 2
            main.wait_event(ready[slot])
            out = step(state, buffers[slot][0], buffers[slot][1])
            consumed[slot].record(main)
            if record:
                loss_host[i].copy_(out[0], non_blocking=True)
        end.record(main)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        return begin.elapsed_time(end)

    run(2, False)
    elapsed = run(steps, True)
    if world > 1:
        worst = torch.tensor([elapsed], device=device)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        elapsed = float(worst)
    assert bool(torch.isfinite(loss_host).all())
    return {"value": steps / (elapsed * 1e-3), "unit": "steps/s", "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": 4 * world,
            "ms_per_step": elapsed / steps, "path": "compiled step called with device buffers refilled from pinned host memory every step"}


if __name__ == "__main__":
    main()
