"""Batch-sharded step on two or more GPUs of one box (skipped where the box has a single GPU).

`dp_check.py` does the work, one process per GPU: every sharded form against the oracle on the full
batch, forms against each other, replicas bit-identical.  The medium MLP (the benchmarked
configuration) is among the workloads.
"""
import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

CHECK = Path(__file__).with_name("dp_check.py")


def _gpus() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as probe:
        probe.bind(("127.0.0.1", 0))
        return probe.getsockname()[1]


@pytest.mark.gpu
@pytest.mark.parametrize("workload", ["c2", "wide", "c4", "c5"])
def test_sharded_step_forms_agree_with_the_oracle_on_the_full_batch(workload):
    count = _gpus()
    if count < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if count < 4 else (4 if count < 8 else 8)
    if workload != "c5":
        world = min(world, 4)
    env = dict(os.environ, NCCL_DEBUG="WARN")
    done = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(CHECK), "--workload", workload],
                          capture_output=True, text=True, timeout=900, env=env)
    lines = [line for line in done.stdout.splitlines() if line.startswith("{")]
    assert done.returncode == 0 and lines, done.stdout[-2000:] + done.stderr[-2000:]
    report = json.loads(lines[-1])
    assert report["failures"] == [] and report["forms"]
    print(json.dumps(report))
