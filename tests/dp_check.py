"""Multi-GPU check of the sharded training step, run as one process per GPU under torchrun.

Every rank compiles the full-batch step (the single-GPU kernel, as the yardstick) and the
batch-sharded step in each exchange form the box supports, runs a few steps of each from the same
state, and compares loss, gradients and updated state:

    sharded form  vs  full batch        within the 16-bit-compute bound (2e-2 relative)
    form          vs  form              near-equal (the forms differ only in FP32 summation order)
    rank          vs  rank              bit-identical replicas (checksums gathered over the group)

Rank 0 prints one JSON line; every rank exits non-zero on a failed comparison.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import trainkernel_b200 as tk  # noqa: E402
from trainkernel_b200 import dp, workloads  # noqa: E402

SIZES = {"c2": ((128, 256, 128), 16), "c4": ((1024, 2048, 2048, 1024), 512), "wide": ((512, 1024, 768, 512), 1024)}


def rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))


def run_steps(step, state, batches, steps):
    out = None
    for i in range(steps):
        out = step(state, *batches[i % len(batches)])
    torch.cuda.synchronize()
    loss, grads, _ = out
    return loss.clone(), [g.clone() for g in grads], [p.clone() for p in state]


def kernel_sources() -> dict[str, str]:
    """Generated sources of every kernel this check launches at 2 and 4 ranks (for ahead-of-time compilation)."""
    from trainkernel_b200 import codegen
    from trainkernel_b200.passes import insert_gradient_exchange
    sources = {}
    for name, (sizes, batch) in SIZES.items():
        count = 2 * (len(sizes) - 1)
        inplace = {1 + count + i: i for i in range(count)}
        full = workloads.mlp_workload("full", sizes, batch, seed=3, resident=1)
        program, _ = tk.capture(full.fn(), (full.state, *full.batches[0]))
        sources[f"{name}_full"] = codegen.generate(program, inplace_outputs=inplace).source
        for world in (2, 4):
            shard = workloads.mlp_workload("shard", sizes, batch, seed=3, resident=1, rows=dp.shard_rows(batch, 0, world))
            program, _ = tk.capture(shard.fn(), (shard.state, *shard.batches[0]))
            for multicast in (False, True):
                sources[f"{name}_w{world}_{multicast}"] = codegen.generate(insert_gradient_exchange(program, count), inplace_outputs=inplace,
                                                                          world=world, multicast=multicast).source
    return sources


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--workload", default="c4", choices=sorted(SIZES))
    parser.add_argument("--steps", type=int, default=3)
    args = parser.parse_args()
    world, rank, local = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    sizes, batch = SIZES[args.workload]
    full = workloads.mlp_workload("full", sizes, batch, seed=3, device=device, resident=2)
    shard = workloads.mlp_workload("shard", sizes, batch, seed=3, device=device, resident=2, rows=dp.shard_rows(batch, rank, world))
    failures: list[str] = []
    report: dict = {"workload": args.workload, "world": world, "steps": args.steps}

    state = tuple(p.clone() for p in full.state)
    yardstick = run_steps(tk.compile_training(full.fn(), (state, *full.batches[0])), state, full.batches, args.steps)

    results = {}
    for name, multicast in (("scatter", False), ("multicast", True)):
        state = tuple(p.clone() for p in shard.state)
        try:
            step = dp.FusedShardedTrainingStep(shard.fn(), (state, *shard.batches[0]), multicast=multicast)
        except RuntimeError as error:                          # raised on every rank alike
            if "no multicast mapping" not in str(error):
                raise
            continue                                           # no multicast mapping on this box: one form only
        results[name] = run_steps(step, state, shard.batches, args.steps)
        step.status()
        loss, grads, params = results[name]
        worst = max([rel(loss, yardstick[0])] + [rel(a, b) for a, b in zip(grads, yardstick[1])] + [rel(a, b) for a, b in zip(params, yardstick[2])])
        report[f"{name}_vs_full_batch"] = worst
        if not worst <= 2e-2:
            failures.append(f"{name}: {worst:.3e} from the full-batch step")
        # replicas: a float64 checksum and an exact bit pattern sum of all state must agree on every rank
        bits = torch.stack([p.view(torch.int32).to(torch.int64).sum() for p in params] + [g.view(torch.int32).to(torch.int64).sum() for g in grads])
        gathered = [torch.empty_like(bits) for _ in range(world)]
        dist.all_gather(gathered, bits)
        identical = all(torch.equal(g, gathered[0]) for g in gathered)
        report[f"{name}_replicas_identical"] = identical
        if not identical:
            failures.append(f"{name}: replicas differ")
    if len(results) == 2:
        a, b = results["scatter"], results["multicast"]
        gap = max([rel(a[0], b[0])] + [rel(x, y) for x, y in zip(a[1], b[1])] + [rel(x, y) for x, y in zip(a[2], b[2])])
        report["multicast_vs_scatter"] = gap
        if not gap <= 1e-2:                                    # one BF16 ulp of the largest element at most
            failures.append(f"multicast and scatter forms differ by {gap:.3e}")
    report["forms"] = sorted(results)
    report["failures"] = failures
    if rank == 0:
        print(json.dumps(report), flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(1 if failures else 0)     # graphs and symmetric buffers outlive an orderly teardown of the group


if __name__ == "__main__":
    main()
