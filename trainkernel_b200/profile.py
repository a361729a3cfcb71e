"""Per-stage timing of a compiled step from stamps written inside the kernel.

The reference measures stages by string-patching `%globaltimer` reads into the
generated source after every grid barrier (reference: scripts/profile_stages.py:36-54).
Here the generator emits those stamps itself when asked (`stage_stamps=True`)
and the runtime shim reads them back, so profiling is an option of `compile`,
not a source rewrite.
"""
from __future__ import annotations

from typing import Any, Callable, Sequence

import torch

from .frontend import compile, compile_training


def stage_profile(fn: Callable[..., Any], example_inputs: Sequence[Any], *, training: bool = True,
                  repeats: int = 10, **options: Any) -> list[dict]:
    """Compile `fn` with stage stamps, run it `repeats` times, and return one record per stage.

    Each record holds the stage index, the fastest and median duration in microseconds (a stage's
    time includes the grid barrier that ends it, as seen by block 0), the units scheduled in it and,
    for every stage that ends in a grid barrier, the barrier's stall times (medians, microseconds):
    `barrier_wait_us` block 0's arrival to its release, `barrier_skew_us` block 0's arrival to the
    last block's arrival, `barrier_release_us` last arrival to release (the cost of the barrier itself).
    State tensors in `example_inputs` are updated by the runs when `training` is true.
    """
    builder = compile_training if training else compile
    compiled = builder(fn, example_inputs, stage_stamps=True, **options)
    runner = compiled.runner
    for _ in range(3):
        compiled(*example_inputs)
    torch.cuda.synchronize(runner.device)
    samples: list[list[float]] = []
    stalls: list[list[dict]] = []
    for _ in range(repeats):
        compiled(*example_inputs)
        stamps = runner.stage_stamps()
        samples.append([(b - a) / 1e3 for a, b in zip(stamps[:-1], stamps[1:])])
        stalls.append(runner.barrier_stalls())
    records = []
    for stage in range(runner.generated.stages):
        column = sorted(sample[stage] for sample in samples)
        units = [f"{name}:{kind}{'/' + path if path else ''}" for s, kind, name, path, _ in runner.generated.units if s == stage]
        record = {"stage": stage, "min_us": column[0], "median_us": column[len(column) // 2], "units": units}
        if stalls and stage < len(stalls[0]):
            for key, label in (("block0_wait", "barrier_wait_us"), ("skew", "barrier_skew_us"), ("release", "barrier_release_us")):
                values = sorted(run[stage][key] / 1e3 for run in stalls)
                record[label] = values[len(values) // 2]
        records.append(record)
    return records


def sharded_stage_profile(sizes, batch: int, *, repeats: int = 5, seed: int = 0, **options: Any) -> list[dict] | None:
    """Per-stage times of the batch-sharded one-kernel step, over ALL ranks (run under torchrun, NCCL group up).

    Every rank runs the step with stage stamps and gathers, per stage of its fastest launch: the stage's
    duration, the time block 0 then spent waiting for its peers' flags (`peer_wait`), and the grid
    barrier's skew and release times.  Rank 0 returns one record per stage with the maximum and minimum
    over ranks (a stage is as slow as its slowest rank; the spread is rank skew), the other ranks None.
    """
    import torch.distributed as dist

    from . import dp, workloads
    rank, world = dist.get_rank(), dist.get_world_size()
    device = torch.device("cuda", torch.cuda.current_device())
    work = workloads.mlp_workload("sharded", tuple(sizes), batch, seed=seed, device=device, rows=dp.shard_rows(batch, rank, world))
    step = dp.FusedShardedTrainingStep(work.fn(), (work.state, *work.batches[0]), stage_stamps=True, **options)
    checker = step._checker
    stages = step.generated.stages
    best = None
    for i in range(3 + repeats):
        step(work.state, *work.batches[i % len(work.batches)])
        stamps = checker.stage_stamps()
        stalls = checker.barrier_stalls()
        total = stamps[-1] - stamps[0]
        if i >= 3 and (best is None or total < best[0]):
            best = (total, [b - a for a, b in zip(stamps[:-1], stamps[1:])], stalls)
    step.status()
    total, durations, stalls = best
    row = torch.zeros(stages, 4, dtype=torch.float64, device=device)
    for s in range(stages):
        row[s, 0] = durations[s]
        if s < len(stalls):
            row[s, 1], row[s, 2] = stalls[s]["skew"], stalls[s]["release"]
        if s > 0 and s - 1 < len(stalls):
            row[s, 3] = stalls[s - 1]["peer_wait"]
    gathered = [torch.zeros_like(row) for _ in range(world)]
    dist.all_gather(gathered, row)
    units = step.generated.units
    multicast = step.multicast
    step.close()
    dist.barrier()
    if rank != 0:
        return None
    table = torch.stack(gathered)                     # [rank, stage, figure]
    records = []
    for s in range(stages):
        records.append({"stage": s, "max_us": float(table[:, s, 0].max()) / 1e3, "min_us": float(table[:, s, 0].min()) / 1e3,
                        "peer_wait_max_us": float(table[:, s, 3].max()) / 1e3, "barrier_skew_max_us": float(table[:, s, 1].max()) / 1e3,
                        "barrier_release_max_us": float(table[:, s, 2].max()) / 1e3,
                        "units": [f"{name}:{kind}{'/' + path if path else ''}x{items}" for st, kind, name, path, items in units if st == s]})
    records.append({"world": world, "multicast": multicast, "sum_max_us": sum(r["max_us"] for r in records)})
    return records


def launch_span_profile(fn: Callable[..., Any], example_inputs: Sequence[Any], batches: Sequence[Any], *, graph_steps: int = 20,
                        replays: int = 10, **options: Any) -> dict:
    """Where a captured step spends its time OUTSIDE the stages: a stamped kernel in a `graph_steps`-step CUDA
    graph, replayed `replays` times under CUDA events.  Microseconds, medians: `period` per step of the replay,
    `prologue` / `stages` / `tail` / `total` of the graph's last launch (`CompiledProgram.launch_span`), and
    `gap_between_launches` = period - total, what the launch itself costs between two dependent kernels."""
    import statistics
    state = example_inputs[0]
    compiled = compile_training(fn, example_inputs, stage_stamps=True, **options)
    for i in range(3):
        compiled(state, *batches[i % len(batches)])
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(graph_steps):
            compiled(state, *batches[i % len(batches)])
    graph.replay()
    torch.cuda.synchronize()
    periods, spans = [], []
    for _ in range(replays):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        graph.replay()
        end.record()
        end.synchronize()
        periods.append(begin.elapsed_time(end) * 1e3 / graph_steps)
        spans.append(compiled.runner.launch_span())
    compiled.runner.status()
    record = {key: statistics.median(span[key] for span in spans) / 1e3 for key in spans[0]}
    record["period"] = statistics.median(periods)
    record["gap_between_launches"] = record["period"] - record["total"]
    return {key: round(value, 2) for key, value in record.items()}


def main(argv=None) -> int:
    """`python -m trainkernel_b200.profile c4` prints the stage table of a named workload as JSON lines;
    `--span` prints what a captured step costs outside its stages instead.

    `--plain` compiles without stamps and only launches the step `--repeats` times: the command to
    put under a hardware profiler.
    """
    import argparse
    import json

    from . import workloads

    parser = argparse.ArgumentParser(description=main.__doc__)
    parser.add_argument("workload", choices=workloads.CONFIG_NAMES)
    parser.add_argument("--sharded", action="store_true",
                        help="c5 only, under torchrun: the batch-sharded one-kernel step, per-stage maximum over ranks")
    parser.add_argument("--no-stream-warps", action="store_true")
    parser.add_argument("--no-multicast", action="store_true")
    parser.add_argument("--repeats", type=int, default=10)
    parser.add_argument("--plain", action="store_true")
    parser.add_argument("--span", action="store_true",
                        help="prologue, stages, tail and launch gap of the step inside a 20-step CUDA graph")
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--trace-stage", type=int, default=None,
                        help="also time the roles of the first single-CTA tensor-core tile of this stage")
    args = parser.parse_args(argv)
    if args.sharded:
        import os

        import torch.distributed as dist
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        sizes, batch = ((4096, 8192, 8192, 8192, 4096), 8192) if args.workload == "c5" else ((1024, 2048, 2048, 1024), 512)
        options = {"background": not args.no_stream_warps}
        if args.no_multicast:
            options["multicast"] = False
        try:
            records = sharded_stage_profile(sizes, batch, repeats=args.repeats, **options)
        except BaseException as error:          # a rank that dies must not leave its peers waiting in a collective
            import os
            import sys
            print(f"[profile] rank {dist.get_rank()} failed: {error!r}", file=sys.stderr, flush=True)
            os._exit(1)
        for record in records or []:
            print(json.dumps(record), flush=True)
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
        return 0
    work = workloads.build(args.workload, device=args.device)
    inputs = (work.state, *work.batches[0])
    if args.span:
        print(json.dumps({"workload": work.name, "us": launch_span_profile(work.fn(), inputs, work.batches, replays=args.repeats)}))
        return 0
    if args.plain:
        compiled = compile_training(work.fn(), inputs)
        for _ in range(args.repeats):
            compiled(*inputs)
        torch.cuda.synchronize()
        compiled.runner.status()
        print(json.dumps({"workload": work.name, "launches": args.repeats, "stages": compiled.runner.generated.stages}))
        return 0
    if args.trace_stage is not None:
        compiled = compile_training(work.fn(), inputs, stage_stamps=True, trace_stage=args.trace_stage)
        best = None
        for _ in range(3 + args.repeats):
            compiled(*inputs)
            stamps = compiled.runner.stage_stamps()
            start = stamps[args.trace_stage]
            points = [(value - start) / 1e3 for value in compiled.runner.role_trace()] + [(stamps[args.trace_stage + 1] - start) / 1e3]
            if best is None or points[-1] < best[-1]:
                best = points
        names = ("producer_starts", "last_tma_issued", "first_operands_landed", "last_mma_committed",
                 "accumulator_complete", "epilogue_done", "stage_ends")
        print(json.dumps({"workload": work.name, "stage": args.trace_stage, "us_after_stage_start": dict(zip(names, best))}))
        return 0
    records = stage_profile(work.fn(), inputs, repeats=args.repeats)
    for record in records:
        print(json.dumps(record))
    print(json.dumps({"workload": work.name, "stages": len(records), "sum_min_us": sum(r["min_us"] for r in records)}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
