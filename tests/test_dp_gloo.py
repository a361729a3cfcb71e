"""Batch-sharded data parallelism on two CPU ranks (gloo): split program + gradient average == full batch."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import trainkernel_b200 as tk
from oracle import interpreter
from trainkernel_b200 import workloads
from trainkernel_b200.dp import shard_rows
from trainkernel_b200.passes import split_at_gradients

SIZES, BATCH, WORLD = (32, 64, 32), 16, 2
NARROW = True      # exchange the BF16 values the FP32 gradients are widened from


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, port: int, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        work = workloads.mlp_workload("shard", SIZES, BATCH, seed=3, rows=shard_rows(BATCH, rank, WORLD))
        n = len(work.state)
        x, t = work.batches[0]
        program, _ = tk.capture(work.fn(), (work.state, x, t))
        gradient_half, update_half = split_at_gradients(program, n, narrow_exchange=NARROW)
        state = work.state
        for step in range(3):
            x, t = work.batches[step % len(work.batches)]
            outputs = [o.clone() for o in interpreter.run(gradient_half, (*state, x, t))]
            for i, tensor in enumerate(outputs):        # loss and gradients: average over ranks
                wide = tensor.float()                   # gloo has no BF16 average; round back afterwards
                dist.all_reduce(wide, op=dist.ReduceOp.SUM)
                outputs[i] = (wide / WORLD).to(tensor.dtype)
            updated = interpreter.run(update_half, (*state, *outputs[1:]))
            state = tuple(o.clone() for o in updated[-n:])
        gathered = [None] * WORLD
        dist.all_gather_object(gathered, [p.numpy().copy() for p in state])
        if rank == 0:
            results.put((float(outputs[0]), gathered))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_step_matches_full_batch_oracle():
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(rank, port, results)) for rank in range(WORLD)]
    for p in procs:
        p.start()
    loss, gathered = results.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # replicas are bit-identical
    for a, b in zip(gathered[0], gathered[1]):
        assert (a == b).all()
    # and match the single-process full-batch oracle within the BF16-compute bound
    work = workloads.mlp_workload("full", SIZES, BATCH, seed=3)
    n = len(work.state)
    program, _ = tk.capture(work.fn(), (work.state, *work.batches[0]))
    state = work.state
    for step in range(3):
        out = interpreter.run(program, (*state, *work.batches[step % len(work.batches)]))
        state = tuple(o.clone() for o in out[1 + n:])
    assert abs(loss - float(out[0])) <= 2e-2 * abs(float(out[0]))
    for got, want in zip(gathered[0], state):
        err = float((torch.from_numpy(got) - want).abs().max()) / max(float(want.abs().max()), 1e-30)
        assert err <= 2e-2


def test_shard_rows_partitions_the_batch():
    covered = []
    for rank in range(4):
        rows = shard_rows(8192, rank, 4)
        covered += list(range(rows.start, rows.stop))
    assert covered == list(range(8192))
    with pytest.raises(ValueError, match="divide evenly"):
        shard_rows(10, 0, 4)


def _exchange_rank(rank: int, port: int, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        from trainkernel_b200.passes import insert_gradient_exchange
        work = workloads.mlp_workload("shard", SIZES, BATCH, seed=3, rows=shard_rows(BATCH, rank, WORLD))
        n = len(work.state)
        program, _ = tk.capture(work.fn(), (work.state, *work.batches[0]))
        exchanged = insert_gradient_exchange(program, n)       # one program, allreduce ops inside
        state = work.state
        for step in range(3):
            out = interpreter.run(exchanged, (*state, *work.batches[step % len(work.batches)]))
            state = tuple(o.clone() for o in out[1 + n:])
        gathered = [None] * WORLD
        dist.all_gather_object(gathered, [p.numpy().copy() for p in state])
        if rank == 0:
            results.put((float(out[0]), gathered))
    finally:
        dist.destroy_process_group()


def test_program_with_allreduce_ops_matches_full_batch_oracle():
    """`insert_gradient_exchange` + the oracle's allreduce (gloo) == the single-process full-batch step."""
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_exchange_rank, args=(rank, port, results)) for rank in range(WORLD)]
    for p in procs:
        p.start()
    loss, gathered = results.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for a, b in zip(gathered[0], gathered[1]):
        assert (a == b).all()
    work = workloads.mlp_workload("full", SIZES, BATCH, seed=3)
    n = len(work.state)
    program, _ = tk.capture(work.fn(), (work.state, *work.batches[0]))
    state = work.state
    for step in range(3):
        out = interpreter.run(program, (*state, *work.batches[step % len(work.batches)]))
        state = tuple(o.clone() for o in out[1 + n:])
    assert abs(loss - float(out[0])) <= 2e-2 * abs(float(out[0]))
    for got, want in zip(gathered[0], state):
        err = float((torch.from_numpy(got) - want).abs().max()) / max(float(want.abs().max()), 1e-30)
        assert err <= 2e-2
