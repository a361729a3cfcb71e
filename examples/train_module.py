"""Train an `nn.Module` through `torch.func.functional_call` with one compiled kernel per step.

Counterpart of the reference's `examples/train.py`: parameters stay a plain dict of FP32 tensors
that the compiled step updates in place; the module itself is only used as a pure function.
"""
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import trainkernel_b200 as trainkernel  # noqa: E402


def main() -> None:
    if not torch.cuda.is_available():
        raise SystemExit("train_module.py needs a B200 (sm_100) GPU")
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.ReLU(), torch.nn.Linear(128, 16)).cuda()
    params = {name: p.detach().clone() for name, p in model.named_parameters()}
    x, target = torch.randn(32, 64, device="cuda"), torch.randn(32, 16, device="cuda")

    def step(p, x, target):
        def loss_fn(q):
            return ((torch.func.functional_call(model, q, (x,)) - target) ** 2).mean()
        grads, loss = torch.func.grad_and_value(loss_fn)(p)
        return loss, grads, {name: p[name] - 1e-2 * grads[name] for name in p}

    compiled = trainkernel.compile_training(step, (params, x, target))
    for i in range(200):
        loss, _, params = compiled(params, x, target)
        if i % 50 == 0:
            print(f"step {i:3d}  loss {float(loss):.5f}")
    print(f"final loss {float(loss):.5f}")


if __name__ == "__main__":
    main()
