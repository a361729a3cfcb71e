"""IR-to-IR rewrites that keep every program output bit-for-bit meaningful.

`canonicalize_transposed_mm` mirrors the reference pass of the same name
(reference: trainkernel/passes.py:7-66).  `split_at_gradients` is new: it cuts
a training program at its gradient outputs so that a cross-rank gradient
reduction can run between the two halves (the reference has no distributed
code, reference: README.md:128).
"""
from __future__ import annotations

from dataclasses import replace

from .ir import Operation, Program, TensorSpec, row_major


def _uses_of(program: Program, buffer: str) -> list[TensorSpec]:
    found = [value for op in program.operations for value in op.inputs
             if isinstance(value, TensorSpec) and value.buffer == buffer]
    found += [value for value in program.outputs if value.buffer == buffer]
    return found


def canonicalize_transposed_mm(program: Program) -> Program:
    """Produce `(A @ B).T` directly as `B.T @ A.T` when nobody sees `A @ B`.

    Backward graphs of `nn.Linear`-style layers return weight gradients as the
    transpose of a matmul.  If every reader (operations and program outputs)
    looks at the product only through that transposed window, the product is
    computed in the transposed orientation instead, so it lands in its final
    layout.  Chains of such products are flipped from the consumer end first so
    that neighbouring flips do not cancel.  The pass is idempotent.
    """
    flippable: dict[str, tuple[int, int]] = {}
    for op in program.operations:
        if op.op != "mm" or len(op.output.shape) != 2:
            continue
        lhs, rhs = op.inputs[0], op.inputs[1]
        if not (isinstance(lhs, TensorSpec) and isinstance(rhs, TensorSpec)):
            continue
        if len(lhs.shape) != 2 or len(rhs.shape) != 2:
            continue
        rows, cols = op.output.shape
        if min(rows, cols) <= 1 or lhs.shape != (rows, rhs.shape[0]) or rhs.shape[1] != cols:
            continue
        readers = _uses_of(program, op.output.buffer)
        if readers and all(r.shape == (cols, rows) and r.strides == (1, cols) and r.offset == 0 for r in readers):
            flippable[op.output.buffer] = (rows, cols)
    if not flippable:
        return program

    chosen: dict[str, tuple[int, int]] = {}
    for op in reversed(program.operations):
        name = op.output.buffer
        if name not in flippable:
            continue
        feeds_chosen = any(
            user.output.buffer in chosen
            for user in program.operations
            for value in user.inputs
            if isinstance(value, TensorSpec) and value.buffer == name
        )
        if not feeds_chosen:
            chosen[name] = flippable[name]

    def relayout(value):
        if not isinstance(value, TensorSpec) or value.buffer not in chosen:
            return value
        rows, cols = chosen[value.buffer]
        if value.offset == 0 and value.shape == (cols, rows) and value.strides == (1, cols):
            return replace(value, strides=(rows, 1))
        if value.offset == 0 and value.shape == (rows, cols) and value.strides == (cols, 1):
            # The operand swap of another flipped product looks at this value untransposed.
            return replace(value, strides=(1, rows))
        raise ValueError("trainkernel: unexpected view in transposed GEMM rewrite")

    def transposed(value: TensorSpec) -> TensorSpec:
        return replace(value, shape=value.shape[::-1], strides=value.strides[::-1])

    rewritten: list[Operation] = []
    for op in program.operations:
        if op.output.buffer in chosen:
            rows, cols = chosen[op.output.buffer]
            lhs, rhs = op.inputs[0], op.inputs[1]
            swapped = (relayout(transposed(rhs)), relayout(transposed(lhs)))
            rewritten.append(replace(op, inputs=swapped, output=replace(op.output, shape=(cols, rows), strides=(rows, 1))))
        else:
            rewritten.append(replace(op, inputs=tuple(relayout(value) for value in op.inputs)))
    return Program(program.inputs, tuple(rewritten), tuple(relayout(value) for value in program.outputs))


def split_at_gradients(program: Program, state_count: int, *, narrow_exchange: bool = False) -> tuple[Program, Program]:
    """Cut a training program into a gradient half and an update half.

    With `narrow_exchange=True` a gradient that is merely the FP32 widening of a 16-bit value
    (the usual BF16-compute / FP32-master step) is cut one operation earlier, at the 16-bit
    value: the gradient half then returns `(loss, narrow grads...)`, and the update half takes
    `(state..., narrow grads...)` and returns `(grads..., updated...)`.  Half as many bytes cross
    the cut, which is what a cross-rank exchange pays for.

    `program` follows the `compile_training` contract: inputs start with
    `state_count` state leaves and outputs are `(loss, grads..., updated...)`.
    The first half computes `(loss, grads...)` from the original inputs.  The
    second half takes `(state..., grads...)` as inputs and computes
    `(updated...)`; it contains exactly the operations that depend on a gradient
    output.  A program whose update reads any other intermediate of the first
    half cannot be cut this way and is rejected.
    """
    n = state_count
    if len(program.outputs) != 1 + 2 * n:
        raise ValueError("trainkernel: split requires (loss, gradients, updated state) outputs")
    grad_specs = program.outputs[1:1 + n]
    update_specs = program.outputs[1 + n:]
    input_buffers = {spec.buffer for spec in program.inputs}
    if narrow_exchange:
        return _split_narrow(program, n)
    for spec in grad_specs:
        if spec.buffer in input_buffers or spec.offset or spec.strides != row_major(spec.shape):
            raise ValueError("trainkernel: gradients must be computed dense values to be exchanged")
    grad_buffers = [spec.buffer for spec in grad_specs]
    if len(set(grad_buffers)) != n:
        raise ValueError("trainkernel: gradient outputs must be distinct values")

    dependent: set[str] = set(grad_buffers)
    later: list[Operation] = []
    for op in program.operations:
        if op.output.buffer in dependent:
            continue
        if any(isinstance(value, TensorSpec) and value.buffer in dependent for value in op.inputs):
            dependent.add(op.output.buffer)
            later.append(op)
    later_outputs = {op.output.buffer for op in later}
    # The gradient half keeps every operation the loss and gradients need.
    needed: set[str] = {spec.buffer for spec in program.outputs[:1 + n]}
    first: list[Operation] = []
    for op in reversed(program.operations):
        if op.output.buffer in needed and op.output.buffer not in later_outputs:
            first.append(op)
            needed.update(value.buffer for value in op.inputs if isinstance(value, TensorSpec))
    first.reverse()
    first_outputs = {op.output.buffer for op in first}

    state_inputs = program.inputs[:n]
    grad_inputs = tuple(TensorSpec(spec.buffer, spec.shape, spec.dtype, row_major(spec.shape), spec.buffer) for spec in grad_specs)
    allowed = {spec.buffer for spec in state_inputs} | set(grad_buffers) | later_outputs
    for op in later:
        for value in op.inputs:
            if isinstance(value, TensorSpec) and value.buffer not in allowed:
                raise ValueError(f"trainkernel: update half reads {value.buffer}, which is not state or a gradient")
    for spec in update_specs:
        if spec.buffer not in allowed:
            raise ValueError("trainkernel: updated state must derive from state and gradients only")
    for spec in program.outputs[:1 + n]:
        if spec.buffer not in first_outputs and spec.buffer not in input_buffers:
            raise ValueError("trainkernel: loss or gradient depends on the update half")
    gradient_half = Program(program.inputs, tuple(first), program.outputs[:1 + n])
    update_half = Program(tuple(state_inputs) + grad_inputs, tuple(later), tuple(update_specs))
    return gradient_half, update_half


def _split_narrow(program: Program, n: int) -> tuple[Program, Program]:
    """`split_at_gradients` with the cut moved below the widening cast of each gradient."""
    producer = {op.output.buffer: op for op in program.operations}
    input_buffers = {spec.buffer for spec in program.inputs}
    cuts: list[TensorSpec] = []
    for spec in program.outputs[1:1 + n]:
        op = producer.get(spec.buffer)
        source = op.inputs[0] if op is not None and op.op == "cast" and op.inputs else None
        narrow = (isinstance(source, TensorSpec) and source.buffer in producer and source.dtype in ("bfloat16", "float16")
                  and spec.dtype == "float32" and spec.offset == 0 and spec.strides == row_major(spec.shape))
        if not narrow:
            raise ValueError("trainkernel: narrow exchange needs gradients that are FP32 casts of 16-bit values")
        cuts.append(producer[source.buffer].output)
    cut_buffers = [spec.buffer for spec in cuts]
    if len(set(cut_buffers)) != n:
        raise ValueError("trainkernel: gradient outputs must be distinct values")
    dependent: set[str] = set(cut_buffers)
    later: list[Operation] = []
    for op in program.operations:
        if op.output.buffer in dependent:
            continue
        if any(isinstance(value, TensorSpec) and value.buffer in dependent for value in op.inputs):
            dependent.add(op.output.buffer)
            later.append(op)
    later_outputs = {op.output.buffer for op in later}
    needed: set[str] = {program.outputs[0].buffer, *cut_buffers}
    first: list[Operation] = []
    for op in reversed(program.operations):
        if op.output.buffer in needed and op.output.buffer not in later_outputs:
            first.append(op)
            needed.update(value.buffer for value in op.inputs if isinstance(value, TensorSpec))
    first.reverse()
    if needed & later_outputs:
        raise ValueError("trainkernel: loss or gradient depends on the update half")
    state_inputs = program.inputs[:n]
    allowed = {spec.buffer for spec in state_inputs} | set(cut_buffers) | later_outputs
    for op in later:
        for value in op.inputs:
            if isinstance(value, TensorSpec) and value.buffer not in allowed:
                raise ValueError(f"trainkernel: update half reads {value.buffer}, which is not state or a gradient")
    for spec in program.outputs[1:]:
        if spec.buffer not in later_outputs:
            raise ValueError("trainkernel: gradients and updated state must derive from state and exchanged gradients only")
    gradient_half = Program(program.inputs, tuple(first), (program.outputs[0], *cuts))
    update_half = Program(tuple(state_inputs) + tuple(cuts), tuple(later), tuple(program.outputs[1:]))
    return gradient_half, update_half


def insert_gradient_exchange(program: Program, state_count: int) -> Program:
    """Rewrite a training program so that its loss and gradients are averaged across ranks in place.

    After the value each gradient is derived from (the 16-bit value under the FP32 widening cast
    when there is one, else the gradient itself) an `allreduce` operation is inserted, and every
    later reader is pointed at its result.  `allreduce` means "element-wise mean over all ranks of
    the job, rounded to the value's dtype"; with one rank it is the identity.  The rewritten
    program still follows the `(loss, grads..., updated...)` contract, so it compiles to ONE kernel
    whose exchange stages sit between the backward GEMMs and the updates that consume them.
    """
    n = state_count
    if len(program.outputs) != 1 + 2 * n:
        raise ValueError("trainkernel: exchange requires (loss, gradients, updated state) outputs")
    producer = {op.output.buffer: op for op in program.operations}
    cuts: list[str] = []
    for spec in program.outputs[:1 + n]:
        op = producer.get(spec.buffer)
        if op is None:
            raise ValueError("trainkernel: loss and gradients must be computed values to be exchanged")
        source = op.inputs[0] if op.op == "cast" and op.inputs else None
        if (isinstance(source, TensorSpec) and source.buffer in producer and source.dtype in ("bfloat16", "float16")
                and spec.dtype == "float32"):
            cuts.append(source.buffer)
        else:
            cuts.append(spec.buffer)
    if len(set(cuts)) != len(cuts):
        raise ValueError("trainkernel: loss and gradient values must be distinct")
    renamed = {buffer: buffer + "_avg" for buffer in cuts}

    def redirect(value):
        if isinstance(value, TensorSpec) and value.buffer in renamed:
            return replace(value, buffer=renamed[value.buffer])
        return value

    operations: list[Operation] = []
    for op in program.operations:
        operations.append(replace(op, inputs=tuple(redirect(v) for v in op.inputs)))
        if op.output.buffer in renamed:
            name = renamed[op.output.buffer]
            result = TensorSpec(name, op.output.shape, op.output.dtype, row_major(op.output.shape), name)
            operations.append(Operation(name, "allreduce", (op.output,), result, {}))
    return Program(program.inputs, tuple(operations), tuple(redirect(v) for v in program.outputs))
