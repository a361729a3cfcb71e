"""Static single-assignment tensor IR consumed by the sm_100a generator.

Field-compatible with the reference IR (reference: trainkernel/ir.py:5-26) so a
program captured by either front end can be handed to either back end.  A
`TensorSpec` is a strided window into a named root buffer; an `Operation`
always defines a brand-new contiguous root; a `Program` is inputs, an ordered
operation list, and output windows.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from math import prod

Scalar = int | float


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: tuple[int, ...]
    dtype: str
    strides: tuple[int, ...]
    buffer: str
    offset: int = 0


@dataclass(frozen=True)
class Operation:
    name: str
    op: str
    inputs: tuple["TensorSpec | int | float", ...]
    output: TensorSpec
    attrs: dict[str, object] = field(default_factory=dict)


@dataclass(frozen=True)
class Program:
    inputs: tuple[TensorSpec, ...]
    operations: tuple[Operation, ...]
    outputs: tuple[TensorSpec, ...]


def row_major(shape: tuple[int, ...]) -> tuple[int, ...]:
    """Strides of a dense row-major tensor of `shape`."""
    out, running = [], 1
    for extent in reversed(shape):
        out.append(running)
        running *= extent
    return tuple(reversed(out))


def span(spec: TensorSpec) -> int:
    """One past the largest element index the window can touch (0 if empty)."""
    if prod(spec.shape) == 0:
        return 0
    return spec.offset + 1 + sum((n - 1) * s for n, s in zip(spec.shape, spec.strides))


def _nonneg_int(value: object) -> bool:
    return type(value) is int and value >= 0


def _check_metadata(spec: TensorSpec) -> None:
    well_formed = (
        len(spec.shape) == len(spec.strides)
        and all(_nonneg_int(n) for n in spec.shape)
        and all(_nonneg_int(s) for s in spec.strides)
        and _nonneg_int(spec.offset)
    )
    if not well_formed:
        raise ValueError("trainkernel: invalid tensor shape, stride, or offset")


def validate(program: Program) -> None:
    """Reject programs whose memory accesses could leave their allocations.

    Same rules and messages as the reference validator
    (reference: trainkernel/ir.py:29-63): inputs and operation results are
    distinct roots at offset zero, operands refer only to roots defined
    earlier, a window keeps its root's dtype and stays inside its extent.
    """
    extent_of: dict[str, int] = {}
    dtype_of: dict[str, str] = {}

    def define(spec: TensorSpec, extent: int, message: str) -> None:
        _check_metadata(spec)
        if spec.buffer in extent_of or spec.offset != 0:
            raise ValueError(message)
        extent_of[spec.buffer] = extent
        dtype_of[spec.buffer] = spec.dtype

    def check_window(spec: TensorSpec) -> None:
        _check_metadata(spec)
        if spec.buffer not in extent_of:
            raise ValueError(f"trainkernel: undefined or future buffer {spec.buffer}")
        if dtype_of[spec.buffer] != spec.dtype:
            raise ValueError("trainkernel: views must preserve the root dtype")
        if span(spec) > extent_of[spec.buffer]:
            raise ValueError("trainkernel: tensor view exceeds its root allocation")

    for spec in program.inputs:
        _check_metadata(spec)
        define(spec, span(spec), "trainkernel: input roots must be distinct and have zero offset")
    for operation in program.operations:
        for operand in operation.inputs:
            if isinstance(operand, TensorSpec):
                check_window(operand)
        define(operation.output, prod(operation.output.shape),
               "trainkernel: operation outputs must define new roots at offset zero")
    for spec in program.outputs:
        check_window(spec)
