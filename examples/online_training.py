"""Online training with a captured step: 100 graph replays compared with eager PyTorch.

The B200 counterpart of the reference's example of the same name
(reference: examples/online_training.py:24-49): a two-layer BF16-compute /
FP32-master MLP is compiled once, captured into a CUDA graph, replayed, and the
resulting parameters are compared with an eager loop over the same batches.
"""
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import trainkernel_b200 as trainkernel  # noqa: E402
from trainkernel_b200 import workloads  # noqa: E402


def main() -> None:
    if not torch.cuda.is_available():
        raise SystemExit("online_training.py needs a B200 (sm_100) GPU")
    work = workloads.build("c2", seed=0, device="cuda")
    x, target = work.batches[0]
    step = work.fn()
    eager_state = tuple(p.clone() for p in work.state)

    compiled = trainkernel.compile_training(step, (work.state, x, target))
    captured = compiled.capture(work.state, x, target)
    for _ in range(100):
        loss, _, _ = captured.replay()
    torch.cuda.synchronize()

    for _ in range(100):
        eager_loss, _, eager_state = step(eager_state, x, target)
    worst = max(float((a - b).abs().max()) for a, b in zip(work.state, eager_state))
    print(f"captured loss {float(loss):.6f}  eager loss {float(eager_loss):.6f}  max |parameter difference| {worst:.3e}")
    print("kernel:", compiled.runner.generated.stages, "stages,", compiled.runner.generated.grid_barriers, "grid barriers,",
          compiled.runner.resource_usage())


if __name__ == "__main__":
    main()
