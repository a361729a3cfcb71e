"""FX capture of pure tensor functions and the user-facing compiled objects.

The public contract is the reference's (reference: trainkernel/frontend.py):
`capture` (:140) traces with fake tensors and lowers ATen nodes to the IR,
`compile` (:265) and `compile_training` (:284) hand the program to
`runtime.compile_program`, `CompiledFunction.capture` (:69) wraps one call in
a state-preserving CUDA graph and `CapturedProgram.replay` (:34) replays it.
Node names become buffer names, views fold into strides, and every computed
value is a new dense row-major root, so programs are interchangeable with the
reference's.
"""
from __future__ import annotations

from collections.abc import Callable, Sequence
from dataclasses import dataclass
from typing import Any, Generic, TypeVar

import torch
from torch.utils._pytree import TreeSpec, tree_flatten, tree_unflatten

from .ir import Operation, Program, TensorSpec, row_major

R = TypeVar("R")

DTYPE_NAMES = {torch.float32: "float32", torch.float16: "float16", torch.bfloat16: "bfloat16"}
# Integer class labels are accepted as inputs so that `one_hot(labels, C)` can be written inside the step
# (the reference only takes a dense one-hot target built outside, reference: trainkernel/frontend.py:150-151
# and benchmarks/train_loop.py:66-68).  Index dtypes may only flow through arange / eq / casts.
INDEX_DTYPE_NAMES = {torch.int64: "int64", torch.int32: "int32", torch.bool: "bool"}
_INDEX_OPS = ("arange", "eq", "cast")

_PERMUTING = ("aten.t.default", "aten.transpose.int", "aten.permute.default")
_IDENTITY_VIEWS = ("aten.alias.default", "aten.detach.default")
_RESHAPING = ("aten.view.default", "aten._unsafe_view.default", "aten.reshape.default",
              "aten.squeeze.default", "aten.squeeze.dim", "aten.unsqueeze.default")
VIEW_TARGETS = frozenset(_PERMUTING + _IDENTITY_VIEWS + _RESHAPING + ("aten.expand.default",))


# ---------------------------------------------------------------------------
# compiled objects
# ---------------------------------------------------------------------------

@dataclass
class CapturedProgram:
    """A CUDA graph bound to fixed argument buffers; outputs are reused per replay."""

    graph: Any
    inputs: tuple[Any, ...]
    outputs: Any
    input_tensors: tuple[torch.Tensor, ...]

    def replay(self) -> Any:
        self.graph.replay()
        return self.outputs


class CompiledFunction(Generic[R]):
    """One shape/stride/dtype specialisation of a static PyTorch function."""

    def __init__(self, program: Program, runner: Any, input_spec: TreeSpec, output_spec: TreeSpec) -> None:
        self.program = program
        self.runner = runner
        self.input_spec = input_spec
        self.output_spec = output_spec

    @property
    def source(self) -> str:
        """The generated CUDA translation unit."""
        return self.runner.source

    def _flatten_inputs(self, args: tuple[Any, ...]) -> tuple[torch.Tensor, ...]:
        leaves, spec = tree_flatten(args)
        if spec != self.input_spec:
            raise ValueError("trainkernel: runtime input pytree differs from the compiled signature")
        return tuple(leaves)

    def __call__(self, *args: Any) -> R:
        leaves = self._flatten_inputs(args)
        return tree_unflatten(list(self.runner(*leaves)), self.output_spec)

    def capture(self, *args: Any, warmup: int = 3) -> CapturedProgram:
        """Record one call as a replayable CUDA graph without disturbing state.

        In-place targets are snapshotted, the step is warmed up `warmup` times,
        the snapshot is restored, the call is recorded, and the snapshot is
        restored again, so the first `replay()` starts from the caller's state.
        """
        if type(warmup) is not int or warmup < 1:
            raise ValueError("trainkernel: graph warmup must be positive")
        leaves = self._flatten_inputs(args)
        self.runner._validate_inputs(leaves)
        device = self.runner.device
        targets = sorted(set(self.runner.inplace_outputs.values()))

        def restore(snapshot: dict[int, torch.Tensor]) -> None:
            for index, saved in snapshot.items():
                leaves[index].copy_(saved)

        with torch.cuda.device(device):
            snapshot = {index: leaves[index].clone() for index in targets}
            try:
                for _ in range(warmup):
                    self(*args)
                torch.cuda.synchronize(device)
            finally:
                restore(snapshot)
            torch.cuda.synchronize(device)
            graph = torch.cuda.CUDAGraph()
            try:
                with torch.cuda.graph(graph):
                    outputs = self(*args)
            finally:
                restore(snapshot)
                torch.cuda.synchronize(device)
        # The flat leaves are retained so buffers outlive edits of the caller's containers.
        return CapturedProgram(graph, args, outputs, leaves)


class CompiledTrainingStep(CompiledFunction[R]):
    """A compiled `(state, *data) -> (loss, gradients, updated_state)` step."""


# ---------------------------------------------------------------------------
# ATen -> IR lowering
# ---------------------------------------------------------------------------

def _node_signature(node: torch.fx.Node) -> tuple[tuple[int, ...], str]:
    fake = node.meta.get("val")
    if not isinstance(fake, torch.Tensor):
        raise ValueError(f"trainkernel: missing tensor metadata for {node.name}")
    if fake.dtype not in DTYPE_NAMES and fake.dtype not in INDEX_DTYPE_NAMES:
        raise ValueError(f"trainkernel: unsupported dtype {fake.dtype} at {node.name}")
    if not all(isinstance(extent, int) for extent in fake.shape):
        raise ValueError("trainkernel: dynamic shapes are unsupported")
    return tuple(fake.shape), DTYPE_NAMES.get(fake.dtype) or INDEX_DTYPE_NAMES[fake.dtype]


def _fold_view(node: torch.fx.Node, base: TensorSpec, shape: tuple[int, ...], dtype: str) -> TensorSpec:
    """Express a view node as new strides over the same root (no data movement)."""
    target = str(node.target)
    if target in _IDENTITY_VIEWS:
        strides = base.strides
    elif target in _PERMUTING:
        rank = len(base.shape)
        if target == "aten.t.default":
            order = list(reversed(range(rank)))
        elif target == "aten.transpose.int":
            order = list(range(rank))
            i, j = int(node.args[1]), int(node.args[2])
            order[i], order[j] = order[j], order[i]
        else:
            order = [int(axis) for axis in node.args[1]]
        strides = tuple(base.strides[axis] for axis in order)
    elif target == "aten.expand.default":
        lead = len(shape) - len(base.shape)
        old_shape = (1,) * lead + base.shape
        old_strides = (0,) * lead + base.strides
        strides = tuple(0 if (was == 1 and now != 1) else stride
                        for was, now, stride in zip(old_shape, shape, old_strides))
    else:
        # Reshape-like views are resolved against the physical layout chosen
        # here, which may differ from the layout FX recorded for the value.
        try:
            strides = tuple(torch.empty_strided(base.shape, base.strides, device="meta").view(shape).stride())
        except RuntimeError as error:
            raise ValueError(f"trainkernel: {target} requires a contiguous copy; use .contiguous() before reshaping") from error
    return TensorSpec(node.name, shape, dtype, strides, base.buffer, base.offset)


def _operand(arg: Any, specs: dict[torch.fx.Node, TensorSpec], target: str) -> TensorSpec | int | float:
    if isinstance(arg, torch.fx.Node):
        return specs[arg]
    if isinstance(arg, (int, float)):
        return arg
    raise ValueError(f"trainkernel: unsupported argument in {target}: {type(arg).__name__}")


def _lower_call(node: torch.fx.Node, specs: dict[torch.fx.Node, TensorSpec]) -> tuple[str, tuple, dict[str, object]]:
    """Map one ATen call to `(ir_op, operands, attrs)`."""
    target = str(node.target)
    kind = target.split(".")[1] if target.startswith("aten.") else target
    tensors = tuple(specs[arg] for arg in node.args if isinstance(arg, torch.fx.Node))
    if kind in ("add", "sub", "mul", "div", "pow"):
        if kind == "div" and (len(node.args) > 2 or node.kwargs.get("rounding_mode") is not None):
            raise ValueError("trainkernel: rounded division is unsupported")
        pair = tuple(_operand(arg, specs, target) for arg in node.args[:2])
        if kind == "pow" and not isinstance(pair[1], (int, float)):
            raise ValueError("trainkernel: pow supports a scalar exponent only")
        attrs: dict[str, object] = {}
        if kind in ("add", "sub"):
            attrs["alpha"] = node.kwargs.get("alpha", node.args[2] if len(node.args) > 2 else 1)
        return kind, pair, attrs
    if kind == "addmm":
        return kind, tensors, {"alpha": node.kwargs.get("alpha", 1), "beta": node.kwargs.get("beta", 1)}
    if kind in ("mm", "relu", "neg"):
        return kind, tensors, {}
    if kind in ("sum", "mean"):
        source = tensors[0]
        axes = node.args[1] if len(node.args) > 1 else node.kwargs.get("dim")
        rank = len(source.shape)
        if axes is None or (isinstance(axes, (list, tuple)) and len(axes) == 0):
            axes = tuple(range(rank))
        elif isinstance(axes, int):
            axes = (axes,)
        axes = tuple(sorted({int(axis) % rank for axis in axes})) if rank else ()
        keep = node.args[2] if len(node.args) > 2 else node.kwargs.get("keepdim", False)
        return kind, (source,), {"dims": axes, "keepdim": bool(keep)}
    if kind == "threshold_backward":
        return kind, tensors[:2], {"threshold": node.args[2]}
    if kind in ("ones_like", "zeros_like", "full_like"):
        fill = {"ones_like": 1, "zeros_like": 0}.get(kind, node.args[1] if kind == "full_like" else 0)
        return "full", (_operand(fill, specs, target),), {"value": fill}
    if kind in ("_to_copy", "clone"):
        return "cast", (tensors[0],), {}
    if kind == "arange":
        # only the `arange(end)` that one_hot produces: 0, 1, ..., end - 1
        if len(node.args) != 1 or not isinstance(node.args[0], int) or node.kwargs.get("dtype") not in (None, torch.int64):
            raise ValueError("trainkernel: only arange(end) with integer end is supported")
        return "arange", (), {"end": int(node.args[0])}
    if kind == "eq":
        return "eq", tuple(_operand(arg, specs, target) for arg in node.args[:2]), {}
    raise ValueError(f"trainkernel: unsupported ATen op {target} at {node.name}")


def capture(fn: Callable[..., Any], example_inputs: Sequence[Any]) -> tuple[Program, TreeSpec]:
    """Trace a pure function of tensor pytrees into a `Program`.

    Python scalars are baked in as constants.  Tensor constants, input mutation,
    data-dependent control flow and ATen operators outside the supported subset
    are rejected.  Tracing uses fake tensors, so the caller's tensors are never
    read or written.
    """
    leaves, input_tree = tree_flatten(tuple(example_inputs))
    if not leaves or not all(isinstance(leaf, torch.Tensor) for leaf in leaves):
        raise TypeError("trainkernel: example_inputs must contain tensors only and cannot be empty")
    if not all(leaf.dtype in DTYPE_NAMES or leaf.dtype in (torch.int64, torch.int32) for leaf in leaves):
        raise ValueError("trainkernel: unsupported dtype; expected float32, float16, or bfloat16 (int32/int64 for class labels)")
    if not all(leaf.layout == torch.strided for leaf in leaves):
        raise ValueError("trainkernel: only strided tensors are supported")
    if not all(leaf.device == leaves[0].device for leaf in leaves):
        raise ValueError("trainkernel: inputs must use one device")
    if any(leaf.is_neg() or leaf.is_conj() for leaf in leaves):
        raise ValueError("trainkernel: resolve lazy negative or conjugate input views before capture")

    from torch.func import functionalize
    from torch.fx.experimental.proxy_tensor import make_fx

    result_tree: list[TreeSpec] = []

    def on_leaves(*flat: torch.Tensor) -> tuple:
        # FX would freeze dict/list results into its own container types, so only
        # leaves are traced and the user's container spec is kept on the side.
        out_leaves, tree = tree_flatten(fn(*tree_unflatten(list(flat), input_tree)))
        result_tree[:] = [tree]
        return tuple(out_leaves)

    try:
        traced = make_fx(functionalize(on_leaves), tracing_mode="fake", _allow_non_fake_inputs=True)(*leaves)
    except Exception as error:
        raise RuntimeError(f"trainkernel: FX capture failed: {error}") from error

    device = leaves[0].device
    specs: dict[torch.fx.Node, TensorSpec] = {}
    program_inputs: list[TensorSpec] = []
    operations: list[Operation] = []
    returned: list[Any] = []
    for node in traced.graph.nodes:
        if node.op == "output":
            returned, _ = tree_flatten(node.args[0])
        elif node.op == "placeholder":
            shape, dtype = _node_signature(node)
            strides = tuple(leaves[len(program_inputs)].stride())
            specs[node] = TensorSpec(node.name, shape, dtype, strides, node.name)
            program_inputs.append(specs[node])
        elif node.op == "call_function":
            target = str(node.target)
            if target.startswith("aten.copy_"):
                raise ValueError("trainkernel: input mutation is unsupported; return updated tensors instead")
            shape, dtype = _node_signature(node)
            if node.meta["val"].device != device:
                raise ValueError("trainkernel: cross-device operations are unsupported")
            if target in VIEW_TARGETS:
                base = next(specs[arg] for arg in node.args if isinstance(arg, torch.fx.Node))
                specs[node] = _fold_view(node, base, shape, dtype)
                continue
            kind, operands, attrs = _lower_call(node, specs)
            if dtype in INDEX_DTYPE_NAMES.values() and kind not in _INDEX_OPS:
                raise ValueError(f"trainkernel: unsupported dtype {node.meta['val'].dtype} at {node.name}; "
                                 "integer tensors may only feed arange / eq / casts (one-hot labels)")
            result = TensorSpec(node.name, shape, dtype, row_major(shape), node.name)
            specs[node] = result
            operations.append(Operation(node.name, kind, operands, result, attrs))
        else:
            raise ValueError(f"trainkernel: unsupported FX node {node.op} ({node.target}); pass tensor constants as explicit inputs")
    if not result_tree:
        raise RuntimeError("trainkernel: capture did not produce an output structure")
    if not all(isinstance(item, torch.fx.Node) and item in specs for item in returned):
        raise ValueError("trainkernel: outputs must contain tensors only")
    program = Program(tuple(program_inputs), tuple(operations), tuple(specs[item] for item in returned))
    return program, result_tree[0]


# ---------------------------------------------------------------------------
# compile entry points
# ---------------------------------------------------------------------------

def _finish(program: Program, output_tree: TreeSpec, example_inputs: Sequence[Any], options: dict[str, Any],
            cls: type[CompiledFunction[Any]]) -> CompiledFunction[Any]:
    _, input_tree = tree_flatten(tuple(example_inputs))
    # Imported at call time so tests can substitute `runtime.compile_program`.
    from . import runtime
    runner = runtime.compile_program(program, example_inputs, **options)
    return cls(program, runner, input_tree, output_tree)


def compile(fn: Callable[..., Any], example_inputs: Sequence[Any], **options: Any) -> CompiledFunction[Any]:
    """Compile a static pure function of tensors into one sm_100a kernel."""
    program, output_tree = capture(fn, example_inputs)
    return _finish(program, output_tree, example_inputs, options, CompiledFunction)


def _subtrees(tree: TreeSpec) -> Sequence[TreeSpec]:
    # torch 2.11 exposes `children()`, earlier releases `children_specs`.
    accessor = getattr(tree, "children", None)
    return accessor() if callable(accessor) else tree.children_specs


def compile_training(fn: Callable[..., Any], example_inputs: Sequence[Any], **options: Any) -> CompiledTrainingStep[Any]:
    """Compile `(state, *data) -> (scalar_loss, gradients, updated_state)`.

    The gradient and updated-state pytrees must mirror the state pytree.  Each
    updated leaf is written into the storage of the state leaf it replaces:
    directly by the producing stage when the planner proves the old value has
    had its last read, otherwise through a staged copy after a final barrier.
    State tensors must not require grad; differentiation is inside `fn`.
    """
    if "inplace_outputs" in options:
        raise ValueError("trainkernel: compile_training derives its own state mapping")
    program, output_tree = capture(fn, example_inputs)
    _, input_tree = tree_flatten(tuple(example_inputs))
    state_tree = _subtrees(input_tree)[0]
    parts = _subtrees(output_tree)
    if output_tree.type not in (tuple, list) or len(parts) != 3:
        raise ValueError("trainkernel: training function must return loss, gradients, updated state")
    loss_tree, gradient_tree, update_tree = parts
    if not loss_tree.is_leaf() or gradient_tree != state_tree or update_tree != state_tree:
        raise ValueError("trainkernel: gradients and updated state must match the state pytree")
    count = state_tree.num_leaves
    if count == 0 or program.outputs[0].shape != ():
        raise ValueError("trainkernel: training requires nonempty state and a scalar loss")
    for gradient, parameter in zip(program.outputs[1:1 + count], program.inputs[:count]):
        if (gradient.shape, gradient.dtype) != (parameter.shape, parameter.dtype):
            raise ValueError("trainkernel: gradients must match parameter shapes and dtypes")
    options["inplace_outputs"] = {1 + count + leaf: leaf for leaf in range(count)}
    return _finish(program, output_tree, example_inputs, options, CompiledTrainingStep)
