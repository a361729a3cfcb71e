"""Failure detection for the sharded step, made and observed on the host (two gloo ranks on CPU).

The failure is a rank that raises before its gradient exchange (and says so), or one that just stops
taking part.  Its peer must learn of it through `dp.PeerHealth` BEFORE it would launch the next step
kernel, within the configured limit, and neither process may hang.  Nothing here needs a GPU.
"""
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from trainkernel_b200.dp import PeerFailure, PeerHealth

WORLD = 2
FAIL_AT = 3


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, port: int, mode: str, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    store = dist.distributed_c10d._get_default_store()
    health = PeerHealth(store, rank, WORLD, timeout_s=1.0)
    value = torch.ones(4)
    steps_done, outcome = 0, "finished"
    begin = time.monotonic()
    try:
        for step in range(6):
            try:
                if rank == 1 and step == FAIL_AT:
                    if mode == "raises":
                        raise ValueError("input pipeline broke")
                    break                                     # "silent": the rank just stops stepping
                health.arrive(step)
                health.wait_for_peers(step)                   # what the sharded step does before each launch
                dist.all_reduce(value)                        # stands in for the in-kernel gradient exchange
                steps_done += 1
            except ValueError as error:
                health.report_failure(str(error))
                outcome = "raised"
                break
    except PeerFailure as failure:
        outcome = f"peer {failure.rank}: {failure.reason}"
    results.put((rank, steps_done, outcome, time.monotonic() - begin))
    # leave without a collective: the peer may already be gone
    time.sleep(0.2 if rank == 0 else 1.5)
    os._exit(0)


@pytest.mark.parametrize("mode", ["raises", "silent"])
def test_peer_learns_of_a_failed_rank_on_the_host_before_its_next_launch(mode):
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(rank, port, mode, results)) for rank in range(WORLD)]
    for p in procs:
        p.start()
    got = dict()
    for _ in range(WORLD):
        rank, steps, outcome, seconds = results.get(timeout=120)
        got[rank] = (steps, outcome, seconds)
    for p in procs:
        p.join(timeout=30)
        assert not p.is_alive()
    # both ranks completed exactly the steps before the failure; rank 0 did not start step FAIL_AT's exchange
    assert got[0][0] == FAIL_AT and got[1][0] == FAIL_AT
    if mode == "raises":
        assert got[1][1] == "raised"
        assert got[0][1] == "peer 1: input pipeline broke"
    else:
        assert got[0][1].startswith("peer 1: no sign of life")
    assert got[0][2] < 30.0          # bounded: the limit is 1 s per wait


def test_peer_health_needs_every_rank_at_the_step():
    """Single-process check of the bookkeeping against a plain in-memory store."""
    store = dist.HashStore()
    a, b = PeerHealth(store, 0, 2, timeout_s=0.05), PeerHealth(store, 1, 2, timeout_s=0.05)
    a.arrive(0)
    with pytest.raises(PeerFailure, match="no sign of life"):
        a.wait_for_peers(0)
    b.arrive(0)
    a.wait_for_peers(0)
    b.wait_for_peers(0)
    a.arrive(1)
    with pytest.raises(PeerFailure):
        a.wait_for_peers(1)          # rank 1 is still at step 0
    b.report_failure("out of memory")
    with pytest.raises(PeerFailure, match="rank 1 failed: out of memory"):
        a.wait_for_peers(1)
    assert b.failed_peer() is None   # a rank does not report itself
