"""Seeded synthetic workloads: step functions and input generators.

The step functions follow the reference's functional pattern — differentiate
inside the function and return `(loss, grads, updated)` (reference:
benchmarks/train_loop.py:35-45, examples/online_training.py:15-21, README.md:79-86).
All tensors come from a CPU `torch.Generator` and are moved to the target
device afterwards, so CPU and GPU runs see bit-identical inputs (reference:
benchmarks/train_loop.py:53-55).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable

import torch


def least_squares_step(w, x, target, lr: float = 1e-3):
    """Single FP32 layer: loss = mean((relu(x @ w) - target)^2), SGD on w."""
    def loss_fn(weight):
        return ((torch.relu(x @ weight) - target) ** 2).mean()
    grad, loss = torch.func.grad_and_value(loss_fn)(w)
    return loss, grad, w - lr * grad


def mlp_master_step(params, x, target, lr: float = 1e-3):
    """L-layer MLP, FP32 master weights, BF16 compute, FP32 loss and SGD.

    `params` is `(W1, b1, ..., WL, bL)` with `W_l` shaped `[in_l, out_l]`;
    ReLU sits between layers, not after the last one.
    """
    layers = len(params) // 2

    def loss_fn(p):
        q = tuple(v.to(torch.bfloat16) for v in p)
        h = x
        for layer in range(layers):
            h = h @ q[2 * layer] + q[2 * layer + 1]
            if layer + 1 < layers:
                h = torch.relu(h)
        return ((h.float() - target.float()) ** 2).mean()

    grads, loss = torch.func.grad_and_value(loss_fn)(params)
    return loss, grads, tuple(p - lr * g for p, g in zip(params, grads))


def mlp_native_step(params, x, target, lr: float = 1e-3):
    """L-layer MLP computed entirely in the dtype of its parameters."""
    layers = len(params) // 2

    def loss_fn(p):
        h = x
        for layer in range(layers):
            h = h @ p[2 * layer] + p[2 * layer + 1]
            if layer + 1 < layers:
                h = torch.relu(h)
        return ((h - target) ** 2).mean()

    grads, loss = torch.func.grad_and_value(loss_fn)(params)
    return loss, grads, tuple(p - lr * g for p, g in zip(params, grads))


def onehot_head_step(w, features, onehot, lr: float = 1e-2):
    """Bias-free classification head trained with MSE against a dense one-hot target."""
    def loss_fn(weight):
        logits = features @ weight.to(torch.bfloat16)
        return ((logits.float() - onehot.float()) ** 2).mean()
    grad, loss = torch.func.grad_and_value(loss_fn)(w)
    return loss, grad, w - lr * grad


def one_hot(labels, classes: int):
    """`torch.nn.functional.one_hot` spelled as the comparison it decomposes to.

    Inside `torch.func.grad` the library function validates the label range with
    data-dependent checks that fake-tensor tracing cannot evaluate; this form traces to
    `unsqueeze`, `arange` and `eq`, and gives the same result for labels in `[0, classes)`.
    """
    return labels.unsqueeze(-1) == torch.arange(classes, device=labels.device)


def onehot_label_step(w, features, labels, lr: float = 1e-2):
    """The same head with integer class labels; the one-hot target is formed inside the step."""
    def loss_fn(weight):
        logits = features @ weight.to(torch.bfloat16)
        onehot = one_hot(labels, weight.shape[1]).to(torch.bfloat16)
        return ((logits.float() - onehot.float()) ** 2).mean()
    grad, loss = torch.func.grad_and_value(loss_fn)(w)
    return loss, grad, w - lr * grad


@dataclass
class Workload:
    """One named configuration: a step function, its state and its resident batches."""

    name: str
    step: Callable
    state: object                      # tensor or tuple of tensors (FP32 masters)
    batches: list                      # list of (x, target) pairs
    lr: float
    compute_dtype: torch.dtype
    layer_sizes: tuple[int, ...]       # (in_1, out_1 = in_2, ..., out_L)
    batch: int
    has_bias: bool

    def fn(self):
        lr, step = self.lr, self.step
        return lambda state, x, target: step(state, x, target, lr)

    @property
    def weight_elements(self) -> int:
        return sum(a * b for a, b in zip(self.layer_sizes[:-1], self.layer_sizes[1:]))

    @property
    def parameter_elements(self) -> int:
        bias = sum(self.layer_sizes[1:]) if self.has_bias else 0
        return self.weight_elements + bias

    def flops_per_step(self) -> int:
        """Forward + dW for every layer, dX for every layer but the first."""
        p = self.weight_elements
        first = self.layer_sizes[0] * self.layer_sizes[1]
        return 4 * self.batch * p + 2 * self.batch * (p - first)

    def bytes_per_step(self) -> int:
        """Masters read once, FP32 grads and updated state written once, batch read once, loss."""
        element = 4 if self.compute_dtype == torch.float32 else 2
        io = element * self.batch * (self.layer_sizes[0] + self.layer_sizes[-1])
        return 12 * self.parameter_elements + io + 4


def _kaiming_uniform(gen: torch.Generator, fan_in: int, fan_out: int) -> torch.Tensor:
    # nn.Linear's default (kaiming_uniform_ with a=sqrt(5)) is U(-1/sqrt(fan_in), 1/sqrt(fan_in)).
    bound = 1.0 / math.sqrt(fan_in)
    return (torch.rand((fan_in, fan_out), generator=gen, dtype=torch.float32) * 2.0 - 1.0) * bound


def mlp_workload(name: str, sizes: tuple[int, ...], batch: int, *, seed: int = 0, resident: int = 4,
                 lr: float = 1e-3, device: str | torch.device = "cpu", rows: slice | None = None) -> Workload:
    """BF16-compute MLP with Kaiming-uniform weights, zero biases, N(0,1) data.

    `rows` keeps only a slice of every batch (a rank's shard of the global
    batch); weights do not depend on it.
    """
    gen = torch.Generator(device="cpu").manual_seed(seed)
    state = []
    for fan_in, fan_out in zip(sizes[:-1], sizes[1:]):
        state.append(_kaiming_uniform(gen, fan_in, fan_out))
        state.append(torch.zeros(fan_out, dtype=torch.float32))
    batches = []
    for _ in range(resident):
        x = torch.randn((batch, sizes[0]), generator=gen, dtype=torch.float32).to(torch.bfloat16)
        t = torch.randn((batch, sizes[-1]), generator=gen, dtype=torch.float32).to(torch.bfloat16)
        if rows is not None:
            x, t = x[rows].contiguous(), t[rows].contiguous()
        batches.append((x.to(device), t.to(device)))
    local_batch = batches[0][0].shape[0]
    return Workload(name, mlp_master_step, tuple(p.to(device) for p in state), batches, lr,
                    torch.bfloat16, tuple(sizes), local_batch, True)


def least_squares_workload(*, seed: int = 0, device: str | torch.device = "cpu") -> Workload:
    """README least-squares step, FP32: w[256,128]~N(0,1/256), x[64,256], target[64,128]~N(0,1)."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    w = torch.randn((256, 128), generator=gen) / 16.0
    x = torch.randn((64, 256), generator=gen)
    t = torch.randn((64, 128), generator=gen)
    return Workload("c1_least_squares_fp32", least_squares_step, w.to(device), [(x.to(device), t.to(device))],
                    1e-3, torch.float32, (256, 128), 64, False)


def onehot_head_workload(*, seed: int = 0, device: str | torch.device = "cpu",
                         batch: int = 256, features: int = 512, classes: int = 1000) -> Workload:
    """One-hot MSE head: features~N(0,1) bf16, labels uniform in [0,classes), W~N(0,1/features)."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    w = torch.randn((features, classes), generator=gen) / math.sqrt(features)
    f = torch.randn((batch, features), generator=gen).to(torch.bfloat16)
    labels = torch.randint(0, classes, (batch,), generator=gen)
    onehot = torch.nn.functional.one_hot(labels, classes).to(torch.bfloat16)
    work = Workload("c3_onehot_head", onehot_head_step, w.to(device), [(f.to(device), onehot.to(device))],
                    1e-2, torch.bfloat16, (features, classes), batch, False)
    work.labels = labels
    return work


CONFIG_NAMES = ("c1", "c2", "c3", "c4", "c5", "gemv")


def build(name: str, *, seed: int = 0, device: str | torch.device = "cpu", rows: slice | None = None) -> Workload:
    """The benchmark configurations C1..C5 by short name, plus the batch-1 GEMV pin."""
    if name == "c1":
        return least_squares_workload(seed=seed, device=device)
    if name == "c2":
        return mlp_workload("c2_tiny_mlp", (128, 256, 128), 16, seed=seed, device=device)
    if name == "c3":
        return onehot_head_workload(seed=seed, device=device)
    if name == "c4":
        return mlp_workload("c4_small_mlp", (1024, 2048, 2048, 1024), 512, seed=seed, device=device)
    if name == "c5":
        return mlp_workload("c5_medium_mlp", (4096, 8192, 8192, 8192, 4096), 8192, seed=seed, device=device, rows=rows)
    if name == "gemv":
        return mlp_workload("gemv_online_mlp", (128, 128, 16), 1, seed=seed, device=device)
    raise ValueError(f"unknown workload {name}")
