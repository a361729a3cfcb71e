"""CPU/PyTorch interpreter of the training-step IR (test infrastructure).

A restatement of the reference's validation interpreter
(reference: trainkernel/reference.py:9-53): operations run in program order
with eager torch ops on whatever device the inputs live on; operands are
strided windows into their root buffers (:14-16); every result is converted
to its declared IR dtype and made dense row-major (:52), which is the rounding
contract the device kernels must reproduce; program outputs are windows into
the final environment (:53).

Pinned against the reference itself: `tests/golden/make_golden.py` ran the
reference's own `capture` + `reference.run` in the build container and stored
its results; `tests/test_oracle_golden.py` compares this interpreter with
those files.
"""
from __future__ import annotations

from collections.abc import Sequence

import torch

from trainkernel_b200.ir import Operation, Program, TensorSpec


def _window(env: dict[str, torch.Tensor], spec: TensorSpec) -> torch.Tensor:
    root = env[spec.buffer]
    return torch.as_strided(root, spec.shape, spec.strides, root.storage_offset() + spec.offset)


def _reduce(op: Operation, args: list) -> torch.Tensor:
    method = getattr(args[0], op.op)
    return method(dim=op.attrs["dims"], keepdim=op.attrs["keepdim"], dtype=getattr(torch, op.output.dtype))


_EAGER = {
    "mm": lambda op, a: a[0] @ a[1],
    "addmm": lambda op, a: torch.addmm(a[0], a[1], a[2], alpha=op.attrs.get("alpha", 1), beta=op.attrs.get("beta", 1)),
    "add": lambda op, a: torch.add(a[0], a[1], alpha=op.attrs.get("alpha", 1)),
    "sub": lambda op, a: torch.sub(a[0], a[1], alpha=op.attrs.get("alpha", 1)),
    "mul": lambda op, a: a[0] * a[1],
    "div": lambda op, a: a[0] / a[1],
    "neg": lambda op, a: -a[0],
    "relu": lambda op, a: torch.relu(a[0]),
    "pow": lambda op, a: a[0] ** a[1],
    "sum": _reduce,
    "mean": _reduce,
    "threshold_backward": lambda op, a: torch.where(a[1] <= op.attrs["threshold"], 0, a[0]),
    "cast": lambda op, a: a[0].to(dtype=getattr(torch, op.output.dtype)),
}


def _allreduce_mean(op: Operation, args: list) -> torch.Tensor:
    """Mean over the ranks of the default process group (identity without one), in FP32, then rounded.

    Not a reference operation: the reference has no distributed code.  It is the semantics of the
    `allreduce` op that `passes.insert_gradient_exchange` adds for batch-sharded steps.
    """
    import torch.distributed as dist
    value = args[0].float().clone()
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(value, op=dist.ReduceOp.SUM)
        value /= dist.get_world_size()
    return value


_EAGER["allreduce"] = _allreduce_mean
# index helpers behind `one_hot(labels, C)` written inside a step (not in the reference's operator set)
_EAGER["eq"] = lambda op, a: torch.eq(a[0], a[1])
_EAGER["arange"] = lambda op, a: torch.arange(op.attrs["end"])


def run(program: Program, inputs: Sequence[torch.Tensor]) -> tuple[torch.Tensor, ...]:
    """Evaluate `program` on `inputs`; returns one tensor per program output."""
    if len(inputs) != len(program.inputs):
        raise ValueError("oracle: incorrect input count")
    env = {spec.buffer: tensor for spec, tensor in zip(program.inputs, inputs)}
    device = inputs[0].device
    for op in program.operations:
        out_dtype = getattr(torch, op.output.dtype)
        if op.op == "full":
            value = torch.full(op.output.shape, op.attrs["value"], dtype=out_dtype, device=device)
        elif op.op == "arange":
            value = torch.arange(op.attrs["end"], dtype=out_dtype, device=device)
        elif op.op in _EAGER:
            operands = [_window(env, x) if isinstance(x, TensorSpec) else x for x in op.inputs]
            value = _EAGER[op.op](op, operands)
        else:
            raise ValueError(f"oracle: unsupported operation {op.op}")
        env[op.output.buffer] = value.to(dtype=out_dtype).contiguous()
    return tuple(_window(env, spec) for spec in program.outputs)
