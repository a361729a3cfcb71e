"""Stage planner for the sm_100a training-step kernel.

Turns a validated `Program` into an ordered list of *units* grouped into
*stages* separated by grid barriers.  It makes the same kinds of decisions as
the scheduler half of the reference generator (reference:
trainkernel/codegen.py:84-333, 656-727) — epilogue fusion, pointwise inlining,
direct versus staged state commits, output binding, workspace reuse, barrier
placement — but with a different execution model:

* a unit is a root (GEMM, reduction or nothing) plus an *element DAG* of
  pointwise operations evaluated on the root's elements while they are still
  in registers; any value needed elsewhere is stored in its own dtype;
* units are placed in the earliest stage their data dependencies allow, so
  independent units (dW and dX of a layer, bias-gradient sums, the loss
  reduction) share a stage and a barrier;
* workspace is a byte arena; a region is reused only by a unit in a later
  stage than the previous owner's last reader.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from math import prod

from .ir import Operation, Program, TensorSpec, row_major

POINTWISE = frozenset({"add", "sub", "mul", "div", "neg", "relu", "pow", "threshold_backward", "full", "cast", "eq", "arange"})
REDUCE = frozenset({"sum", "mean"})
GEMM = frozenset({"mm", "addmm"})
EXCHANGE = frozenset({"allreduce"})
SYM_HEADER = 4096                      # flag words at the start of the symmetric buffer
ELEMENT_BYTES = {"float32": 4, "float16": 2, "bfloat16": 2, "int64": 8, "int32": 4, "bool": 1}
SM_COUNT = 148
MAX_CLUSTER = 8                         # portable thread-block cluster size
CLUSTER_WORK_LIMIT = 30_000_000         # flops-equivalents below which a program runs as one cluster (measured crossover: 9 MF wins, 75 MF loses)
THREADS = 192
ALIGN = 256
# tk::kExchangeChunksPerItem: owned chunks one exchange work item covers = 16-byte loads every thread keeps in
# flight through the switch.  16 was tried (`exchange_chunks=16`): the item then needs more registers than a
# called function gets without saving its caller's, and the step was no faster (4 ranks, p50 of 30 replays:
# 2.81 ms against 2.75 ms with 8).
TENSOR_CORE_MIN_FLOPS = 600_000   # 2*M*N*K of the largest product below which a program stays off the tensor path (MLP 32-64-16, batch 16: 17.9 -> 12.0 us per step; the tiny MLP of the benchmark, 1.05 MFLOP per product, is the same either way)
EXCHANGE_CHUNKS_PER_ITEM = 8


# ---------------------------------------------------------------------------
# expressions over a unit's element index space
# ---------------------------------------------------------------------------

@dataclass(frozen=True)
class Access:
    """Affine address of a stored value: offset + sum(coord[d] * strides[d]) elements."""
    buffer: str
    dtype: str
    offset: int
    strides: tuple[int, ...]


@dataclass(frozen=True)
class Load:
    access: Access


@dataclass(frozen=True)
class Const:
    value: float


@dataclass(frozen=True)
class Iota:
    """The element's own coordinate along unit dim `dim` (what `arange` evaluates to when inlined)."""
    dim: int | None


@dataclass(frozen=True)
class Ref:
    """Value of this unit's root or of one of its members at the same element."""
    buffer: str


@dataclass(frozen=True)
class Apply:
    """A pointwise IR operation applied to sub-expressions; the result is rounded to op.output.dtype."""
    op: Operation
    args: tuple


@dataclass
class Store:
    buffer: str
    dtype: str


@dataclass
class FusedReduce:
    """A reduction whose partial sums are formed in a tensor-core GEMM's epilogue, from accumulator registers.

    `mode` "cols": per 32-row chunk and column, the sum over the chunk's rows of member `buffer`, stored at
    scratch[(row / 32), column].  `mode` "all": per 32 x 32 chunk the sum of all its elements, stored at
    scratch[(row / 32) * ceil(N / 32) + column / 32].  The reduce unit that owned the reduction keeps only
    its fixed-order finish over the partials.
    """
    mode: str
    buffer: str
    scratch: str
    parts: int


@dataclass
class GemmOperand:
    buffer: str            # stored buffer the operand is read from
    dtype: str             # storage dtype
    round_to: str          # dtype the value is rounded to before use (a folded cast), else == dtype
    offset: int
    strides: tuple[int, int]


@dataclass
class Unit:
    kind: str                              # "gemm" | "reduce" | "point" | "exchange"
    name: str
    index: int                             # program position of the root / seed (ordering key)
    dims: tuple[int, ...]                  # element index space of the DAG
    root: Operation | None = None
    members: list[Operation] = field(default_factory=list)
    pmaps: dict[str, tuple] = field(default_factory=dict)     # buffer -> per-dim unit dim (or None)
    exprs: dict[str, object] = field(default_factory=dict)    # member buffer -> Apply
    stores: list[Store] = field(default_factory=list)
    reads: set[str] = field(default_factory=set)              # stored buffers read
    stage: int = 0
    # gemm
    path: str = ""                         # "tc" | "simt" | "gemv"
    a: GemmOperand | None = None
    b: GemmOperand | None = None
    mnk: tuple[int, int, int] = (0, 0, 0)
    block_n: int = 0
    bias: object = None                    # addmm bias expression
    # reduce
    kept: tuple[int, ...] = ()             # extents of kept dims (== dims for the finish DAG)
    reduced: tuple[int, ...] = ()
    source: object = None                  # expression over kept + reduced coordinates
    strategy: str = ""                     # "thread" | "block"
    parts: int = 1
    phase: str = ""                        # "" | "partial" | "finish"
    scratch: str = ""                      # partial-sum buffer name
    vector: bool = False                   # thread strategy: 8 adjacent outputs per thread
    wait_barrier: int | None = None        # peers must have passed this grid barrier before the unit starts
    items: int = 1
    fused: list = field(default_factory=list)   # gemm: FusedReduce entries evaluated in the epilogue
    carried: bool = False                  # point: a cast of in-place state whose result the updating unit re-creates for the next launch
    mean_count: int = 0                    # reduce over partials: the element count a mean divides by
    no_split: bool = False                 # reduce over partials: one pass, never split again

    @property
    def writes(self) -> set[str]:
        return {s.buffer for s in self.stores}


def point_unroll(total: int, streams: int = 2) -> int:
    """Independent 8-element chunks each thread of a flat pointwise unit keeps in flight per iteration.

    Large streams need ~50 KiB of LOADS in flight per SM to cover HBM latency at full bandwidth: 8 chunks x
    192 threads x 32 B for a one-input stream; 6 chunks for units with more tensors per element (an FP32
    update reads a master and a mean, 48 B per chunk: 6 x 192 x 48 B = 54 KiB; with 4 chunks it measured
    4.9 of 6.5 TB/s).  Small streams keep more blocks busy with less unrolling.
    """
    if total >= SM_COUNT * THREADS * 8 * 8:
        return 8 if streams <= 2 else 6
    if total >= SM_COUNT * THREADS * 8 * 2:
        return 2
    return 1


class _Materialize(Exception):
    def __init__(self, buffer: str):
        super().__init__(buffer)
        self.buffer = buffer


def _dense(spec: TensorSpec) -> bool:
    return spec.offset == 0 and all(n == 1 or s == r for n, s, r in zip(spec.shape, spec.strides, row_major(spec.shape)))


def _squeeze(shape: tuple[int, ...]) -> tuple[int, ...]:
    return tuple(n for n in shape if n != 1)


@dataclass
class Plan:
    program: Program
    units: list[Unit]
    stages: int
    storage: dict[str, tuple]              # buffer -> ("in", i) | ("out", slot) | ("ws", byte offset)
    dtypes: dict[str, str]
    shapes: dict[str, tuple[int, ...]]
    workspace_bytes: int
    inlined: set[str]
    direct_commits: dict[int, int]
    staged_commits: dict[int, int]
    native_outputs: dict[int, str]
    grid: int
    tensor_core_units: int
    uses_tc: bool
    two_cta: bool = False
    world: int = 1
    symmetric_bytes: int = 0
    signal_barriers: tuple = ()            # grid barriers after which this rank raises its flag at every peer
    background: bool = False               # run memory-bound units inside the epilogue warps of tensor-core stages
    multicast: bool = False                # exchange through the NVSwitch multicast mapping (multimem) instead of scattering
    cluster_blocks: int = 0                # > 0: the whole grid is ONE thread-block cluster of this many blocks, stages end in the hardware cluster barrier
    carry_bytes: int = 0                   # size of the buffer that keeps derived values (BF16 weight copies) from one launch to the next
    carry_pingpong: bool = False           # carried values have two copies; a launch reads one and writes the other
    exchange_chunks: int = 8               # owned chunks per exchange work item (TK_EXCHANGE_CHUNKS of the kernel)


class Planner:
    def __init__(self, program: Program, *, inplace_outputs: dict[int, int] | None = None,
                 fuse_pointwise: bool = True, fuse_epilogues: bool = True, max_blocks: int | None = None,
                 tensor_cores: bool = True, block_n: int | None = None, two_cta: bool | None = None, world: int = 1, background: bool = False,
                 multicast: bool = False, cluster_barrier: bool | None = None, carry: bool | str | None = None,
                 wave_aware_tiles: bool = False, exchange_chunks: int = EXCHANGE_CHUNKS_PER_ITEM, late_casts: bool = False):
        self.program = program
        self.late_casts = bool(late_casts)
        if exchange_chunks not in (8, 16):
            raise ValueError("trainkernel: exchange_chunks must be 8 or 16")
        self.exchange_chunks = exchange_chunks
        self.wave_aware_tiles = wave_aware_tiles
        if carry not in (None, True, False, "pingpong", "reorder"):
            raise ValueError("trainkernel: carry_shadows must be None, True, False, 'pingpong' or 'reorder'")
        self.carry = "pingpong" if carry is True else carry
        self.cluster_barrier = cluster_barrier
        self.inplace = dict(inplace_outputs or {})
        self.fuse_pointwise = fuse_pointwise
        self.fuse_epilogues = fuse_epilogues
        self.max_blocks = max_blocks
        self.tensor_cores = tensor_cores
        self.forced_block_n = block_n
        self.two_cta = two_cta
        self.world = world
        self.background = background
        self.multicast = bool(multicast) and world > 1
        self.ops = list(program.operations)
        # A program whose largest product is below TENSOR_CORE_MIN_FLOPS runs all of them on the SIMT path: the
        # tensor path's fixed costs (tensor-memory allocation, tensor maps, the latency of a TMA round trip and
        # of an accumulator hand-over per tile) are then larger than the products themselves.
        def product_flops(op: Operation) -> int:
            left = op.inputs[-2]                     # mm(a, b) and addmm(bias, a, b): the left operand is second to last
            if not isinstance(left, TensorSpec) or len(left.shape) != 2:
                return TENSOR_CORE_MIN_FLOPS         # malformed; _make_gemm reports it
            return 2 * prod(op.output.shape) * left.shape[1]

        products = [op for op in self.ops if op.op in ("mm", "addmm")]
        self.tiny_products = bool(products) and all(product_flops(op) < TENSOR_CORE_MIN_FLOPS for op in products)
        self.index = {op.output.buffer: i for i, op in enumerate(self.ops)}
        self.producer = {op.output.buffer: op for op in self.ops}
        self.input_index = {spec.buffer: i for i, spec in enumerate(program.inputs)}
        self.output_buffers = {spec.buffer for spec in program.outputs}
        self.use_count: dict[str, int] = {}
        for op in self.ops:
            for value in op.inputs:
                if isinstance(value, TensorSpec):
                    self.use_count[value.buffer] = self.use_count.get(value.buffer, 0) + 1
        self.forced: set[str] = set()

    # -- public --------------------------------------------------------------
    def plan(self) -> Plan:
        for _ in range(len(self.ops) + 2):
            try:
                return self._plan_once()
            except _Materialize as request:
                if request.buffer in self.forced:
                    raise ValueError(f"trainkernel: cannot schedule {request.buffer}") from None
                self.forced.add(request.buffer)
        raise ValueError("trainkernel: planner did not converge")

    # -- inlining policy -------------------------------------------------------
    def _const_only(self, op: Operation) -> bool:
        return all((not isinstance(v, TensorSpec)) or
                   (v.buffer in self.producer and self.producer[v.buffer].op in POINTWISE and self._const_only(self.producer[v.buffer]))
                   for v in op.inputs)

    def _inlinable(self, buffer: str) -> bool:
        op = self.producer.get(buffer)
        if op is None or op.op not in POINTWISE or not self.fuse_pointwise:
            return False
        if buffer in self.output_buffers or buffer in self.forced or buffer in self.claimed:
            return False
        if self.use_count.get(buffer, 0) <= 1:
            return True
        source = op.inputs[0] if op.inputs else None
        if op.op == "cast" and isinstance(source, TensorSpec) and source.buffer in self.input_index:
            return True
        return self._const_only(op)

    def _leaves_before(self, spec: TensorSpec, limit: int) -> bool:
        """True when every stored value `spec` depends on exists before program position `limit`."""
        if spec.buffer in self.input_index:
            return True
        if self._inlinable(spec.buffer):
            return all(self._leaves_before(v, limit) for v in self.producer[spec.buffer].inputs if isinstance(v, TensorSpec))
        return self.index[spec.buffer] < limit

    # -- views in unit coordinates ------------------------------------------------
    @staticmethod
    def _operand_view(op_shape: tuple[int, ...], pmap: tuple, operand: TensorSpec, rank: int) -> Access:
        """Window `operand` of an op whose output elements sit at `pmap` in the unit, as unit strides."""
        lead = len(op_shape) - len(operand.shape)
        if lead < 0:
            raise ValueError("trainkernel: invalid broadcast rank")
        strides = [0] * rank
        for k, extent in enumerate(op_shape):
            j = k - lead
            if j < 0 or operand.shape[j] == 1:
                continue
            if operand.shape[j] != extent:
                raise ValueError("trainkernel: incompatible broadcast dimensions")
            if pmap[k] is not None:
                strides[pmap[k]] += operand.strides[j]
        return Access(operand.buffer, operand.dtype, operand.offset, tuple(strides))

    @staticmethod
    def _compose(access: Access, dims: tuple[int, ...], shape: tuple[int, ...]):
        """Map a dense value of `shape`, seen through `access`, onto unit dims; None if not dimension-wise."""
        if access.offset != 0:
            return None
        dense = row_major(shape)
        pmap: list = [None] * len(shape)
        for d, (extent, stride) in enumerate(zip(dims, access.strides)):
            if extent == 1 or stride == 0:
                continue
            match = [k for k in range(len(shape)) if shape[k] > 1 and dense[k] == stride and pmap[k] is None and extent <= shape[k]]
            if not match:
                return None
            pmap[match[0]] = d
        return tuple(pmap)

    @staticmethod
    def _covers(pmap, dims: tuple[int, ...], shape: tuple[int, ...]) -> bool:
        used = [p for p in pmap if p is not None]
        return (all(p is not None and dims[p] == n for p, n in zip(pmap, shape) if n > 1)
                and sorted(used) == [d for d, n in enumerate(dims) if n > 1])

    def _expr(self, unit: Unit, access: Access, limit: int):
        """Expression for the value seen through `access` (unit coordinates)."""
        buffer = access.buffer
        if buffer in unit.pmaps:
            shape = self.shape_of(buffer)
            pmap = self._compose(access, unit.dims, shape)
            if pmap is None or pmap != unit.pmaps[buffer] or not self._covers(pmap, unit.dims, shape):
                raise _Materialize(buffer)   # never reached for admitted members; defensive
            return Ref(buffer)
        if buffer not in self.input_index and self._inlinable(buffer):
            op = self.producer[buffer]
            pmap = self._compose(access, unit.dims, op.output.shape)
            if pmap is None:
                raise _Materialize(buffer)
            return self._apply(unit, op, pmap, limit)
        unit.reads.add(buffer)
        return Load(access)

    def _apply(self, unit: Unit, op: Operation, pmap: tuple, limit: int) -> Apply:
        if op.op == "arange":
            return Apply(op, (Iota(pmap[0] if pmap else None),))
        args = []
        for value in op.inputs:
            if isinstance(value, TensorSpec):
                args.append(self._expr(unit, self._operand_view(op.output.shape, pmap, value, len(unit.dims)), limit))
            else:
                args.append(Const(float(value)))
        return Apply(op, tuple(args))

    def shape_of(self, buffer: str) -> tuple[int, ...]:
        if buffer in self.input_index:
            return self.program.inputs[self.input_index[buffer]].shape
        return self.producer[buffer].output.shape

    # -- DAG growth ---------------------------------------------------------------
    def _member_pmap(self, unit: Unit, shape: tuple[int, ...]):
        """pmap of a value whose shape matches the unit's index space up to size-1 dims."""
        if _squeeze(shape) != _squeeze(unit.dims):
            return None
        live = [d for d, n in enumerate(unit.dims) if n > 1]
        pmap, cursor = [], 0
        for n in shape:
            if n > 1:
                pmap.append(live[cursor])
                cursor += 1
            else:
                pmap.append(None)
        return tuple(pmap)

    def _grow(self, unit: Unit, start: int) -> None:
        """Absorb later pointwise operations that act element-for-element on unit values."""
        for op in self.ops[start + 1:]:
            buffer = op.output.buffer
            if op.op not in POINTWISE or buffer in self.claimed or not _dense(op.output):
                continue
            tensors = [v for v in op.inputs if isinstance(v, TensorSpec)]
            inside = [v for v in tensors if v.buffer in unit.pmaps]
            if not inside:
                continue
            pmap = self._member_pmap(unit, op.output.shape)
            if pmap is None:
                continue
            rank = len(unit.dims)
            ok = True
            for v in tensors:
                try:
                    access = self._operand_view(op.output.shape, pmap, v, rank)
                except ValueError:
                    ok = False
                    break
                if v.buffer in unit.pmaps:
                    seen = self._compose(access, unit.dims, self.shape_of(v.buffer))
                    if seen is None or seen != unit.pmaps[v.buffer] or not self._covers(seen, unit.dims, self.shape_of(v.buffer)):
                        ok = False
                        break
                elif not self._leaves_before(v, unit.index):
                    ok = False
                    break
            if not ok:
                continue
            self.claimed[buffer] = unit
            unit.members.append(op)
            unit.pmaps[buffer] = pmap

    # -- unit construction ----------------------------------------------------------
    def _gemm_operand(self, spec: TensorSpec, want_tc: bool) -> GemmOperand:
        buffer = spec.buffer
        if buffer not in self.input_index and self._inlinable(buffer):
            op = self.producer[buffer]
            source = op.inputs[0] if op.inputs else None
            if want_tc or op.op != "cast" or not isinstance(source, TensorSpec) or self._inlinable(source.buffer):
                raise _Materialize(buffer)
            # cast folded into the operand load: address the cast's source through this view
            access = Access(buffer, spec.dtype, spec.offset, spec.strides)
            pmap = self._compose(access, spec.shape, op.output.shape)
            if pmap is None:
                raise _Materialize(buffer)
            inner = self._operand_view(op.output.shape, pmap, source, 2)
            return GemmOperand(inner.buffer, inner.dtype, spec.dtype, inner.offset, (inner.strides[0], inner.strides[1]))
        return GemmOperand(buffer, spec.dtype, spec.dtype, spec.offset, (spec.strides[0], spec.strides[1]))

    @staticmethod
    def _tma_major(rows: int, depth: int, strides: tuple[int, int], offset: int):
        """'k' / 'mn' when a [rows, depth] 16-bit operand can be fetched by a 128B-swizzled TMA box."""
        s_row, s_k = strides
        if offset % 8:
            return None
        if (s_k == 1 or depth == 1) and s_row % 8 == 0 and (s_row >= depth or rows == 1):
            return "k"
        if (s_row == 1 or rows == 1) and s_k % 8 == 0 and (s_k >= rows or depth == 1):
            return "mn"
        return None

    def _make_gemm(self, position: int, op: Operation) -> Unit:
        a_spec, b_spec = (op.inputs[1], op.inputs[2]) if op.op == "addmm" else (op.inputs[0], op.inputs[1])
        if not (isinstance(a_spec, TensorSpec) and isinstance(b_spec, TensorSpec)) or len(a_spec.shape) != 2 \
                or len(b_spec.shape) != 2 or a_spec.shape[1] != b_spec.shape[0]:
            raise ValueError("trainkernel: mm requires compatible rank-two tensors")
        m, k = a_spec.shape
        n = b_spec.shape[1]
        if op.output.shape != (m, n):
            raise ValueError("trainkernel: matrix output shape does not match its inputs")
        unit = Unit("gemm", op.name, position, (m, n), root=op, mnk=(m, n, k))
        unit.pmaps[op.output.buffer] = self._member_pmap(unit, (m, n))
        return unit

    def _finish_gemm(self, unit: Unit) -> None:
        op, position = unit.root, unit.index
        a_spec, b_spec = (op.inputs[1], op.inputs[2]) if op.op == "addmm" else (op.inputs[0], op.inputs[1])
        m, n, k = unit.mnk
        sixteen = a_spec.dtype == b_spec.dtype and a_spec.dtype in ("bfloat16", "float16")
        a_major = self._tma_major(m, k, a_spec.strides, a_spec.offset)
        b_major = self._tma_major(n, k, (b_spec.strides[1], b_spec.strides[0]), b_spec.offset)
        want_tc = bool(self.tensor_cores and not self.tiny_products and sixteen and m > 4 and k > 8 and n >= 8 and a_major and b_major)
        unit.a = self._gemm_operand(a_spec, want_tc)
        unit.b = self._gemm_operand(b_spec, want_tc)
        if want_tc:
            unit.path = "tc"
        elif sixteen and m == 1 and k >= 64 and (unit.b.strides[0] == 1 or unit.b.strides[1] == 1):
            unit.path = "gemv"
        else:
            unit.path = "simt"
        unit.reads.update((unit.a.buffer, unit.b.buffer))
        if op.op == "addmm":
            alpha, beta = op.attrs.get("alpha", 1), op.attrs.get("beta", 1)
            if beta != 0:
                unit.bias = self._expr(unit, self._operand_view((m, n), unit.pmaps[op.output.buffer], op.inputs[0], 2), position)

    def _make_reduce(self, position: int, op: Operation) -> Unit:
        source = op.inputs[0]
        if not isinstance(source, TensorSpec):
            raise ValueError("trainkernel: reduction requires a tensor")
        rank = len(source.shape)
        axes = tuple(sorted({int(d) % rank for d in op.attrs.get("dims", tuple(range(rank)))})) if rank else ()
        kept_axes = [d for d in range(rank) if d not in axes]
        kept = tuple(source.shape[d] for d in kept_axes)
        reduced = tuple(source.shape[d] for d in axes)
        if prod(op.output.shape) != prod(kept):
            raise ValueError("trainkernel: reduction output shape does not match its axes")
        unit = Unit("reduce", op.name, position, kept or (1,), root=op, kept=kept or (1,), reduced=reduced or (1,))
        pm = self._member_pmap(unit, op.output.shape)
        unit.pmaps[op.output.buffer] = pm if pm is not None else tuple([None] * len(op.output.shape))
        return unit

    def _finish_reduce(self, unit: Unit) -> None:
        op = unit.root
        source = op.inputs[0]
        rank = len(source.shape)
        axes = tuple(sorted({int(d) % rank for d in op.attrs.get("dims", tuple(range(rank)))})) if rank else ()
        kept_axes = [d for d in range(rank) if d not in axes]
        # The source is evaluated on a (kept..., reduced...) index space.
        space = Unit("reduce", op.name, unit.index, unit.kept + unit.reduced)
        strides = tuple(source.strides[d] for d in kept_axes) if kept_axes else (0,)
        strides += tuple(source.strides[d] for d in axes) if axes else (0,)
        unit.source = self._expr(space, Access(source.buffer, source.dtype, source.offset, strides), unit.index)

    def _wants_pair_tiles(self, units: list[Unit]) -> bool:
        """Two-CTA (256 x 256) pair tiles: when every tensor-core GEMM is large enough to keep the clusters busy."""
        tc = [u for u in units if u.kind == "gemm" and u.path in ("tc", "tc2")]
        eligible = bool(tc) and all(u.mnk[0] >= 256 and u.mnk[1] >= 256 for u in tc)
        if self.two_cta is not None:
            return bool(self.two_cta and eligible)
        return eligible and min(-(-u.mnk[0] // 256) * -(-u.mnk[1] // 256) for u in tc) >= 64

    def _fuse_reduction(self, unit: Unit, dtypes: dict, shapes: dict, absorbed: dict) -> None:
        """Move the summation of `unit` into the epilogue of the tensor-core GEMM that produces its operand."""
        source = unit.source
        if not isinstance(source, Load) or unit.root.op not in ("sum", "mean"):
            return
        access = source.access
        host = self.claimed.get(access.buffer)
        if host is None or host.kind != "gemm" or host.path != "tc" or access.offset != 0:
            return
        if host.pmaps.get(access.buffer) != (0, 1) or shapes[access.buffer] != host.dims:
            return
        m, n = host.dims
        if m < 2 or n < 2:
            return
        if unit.kept == (n,) and unit.reduced == (m,) and access.strides == (1, n):
            mode, parts, outputs = "cols", -(-m // 32), n
        elif prod(unit.kept) == 1 and unit.reduced == (m, n) and access.strides[-2:] == (n, 1) and not any(access.strides[:-2]):
            mode, parts, outputs = "all", -(-m // 32) * -(-n // 32), 1
        else:
            return
        scratch = f"{unit.name}__partials"
        dtypes[scratch], shapes[scratch] = "float32", (parts, outputs)
        host.fused.append(FusedReduce(mode, access.buffer, scratch, parts))
        absorbed.setdefault(access.buffer, set()).add(id(unit.root))
        if mode == "cols":
            unit.phase, unit.scratch, unit.parts = "finish", scratch, parts
        else:
            # the finish is itself a (small) reduction: one block sums the chunk partials in a fixed order
            unit.mean_count = m * n
            unit.no_split = True
            unit.reduced = (parts,)
            unit.source = Load(Access(scratch, "float32", 0, (0, 1)))

    # -- main pass -------------------------------------------------------------------
    def _plan_once(self) -> Plan:
        self.claimed: dict[str, Unit] = {}
        program = self.program
        units: list[Unit] = []
        for position, op in enumerate(self.ops):
            if op.op in GEMM:
                unit = self._make_gemm(position, op)
            elif op.op in REDUCE:
                unit = self._make_reduce(position, op)
            elif op.op in EXCHANGE:
                unit = Unit("exchange", op.name, position, (max(1, prod(op.output.shape)),), root=op)
                unit.pmaps[op.output.buffer] = self._member_pmap(unit, op.output.shape) or tuple([None] * len(op.output.shape))
            elif op.op in POINTWISE:
                continue
            else:
                raise ValueError(f"trainkernel: unsupported CUDA operation {op.op}")
            self.claimed[op.output.buffer] = unit
            units.append(unit)
        if self.fuse_epilogues:
            for unit in units:
                if unit.kind != "exchange":
                    self._grow(unit, unit.index)
        # remaining pointwise operations: inline or seed pointwise units
        for position, op in enumerate(self.ops):
            buffer = op.output.buffer
            if op.op not in POINTWISE or buffer in self.claimed or self._inlinable(buffer):
                continue
            if not _dense(op.output):
                raise ValueError(f"trainkernel: materialized output must be contiguous: {op.name}")
            dims = op.output.shape or (1,)
            unit = Unit("point", op.name, position, dims)
            unit.pmaps[buffer] = tuple(range(len(op.output.shape)))
            unit.members.append(op)
            self.claimed[buffer] = unit
            if self.fuse_pointwise:
                self._grow(unit, position)
            units.append(unit)
        units.sort(key=lambda u: u.index)
        inlined = {op.output.buffer for op in self.ops if op.output.buffer not in self.claimed}

        # operands, sources and member expressions (claims are final from here on)
        for unit in units:
            if unit.kind == "gemm":
                self._finish_gemm(unit)
            elif unit.kind == "reduce":
                self._finish_reduce(unit)
            elif unit.kind == "exchange":
                source = unit.root.inputs[0]
                if not isinstance(source, TensorSpec) or not _dense(source) or source.shape != unit.root.output.shape \
                        or source.buffer in self.input_index or self._inlinable(source.buffer):
                    raise ValueError("trainkernel: allreduce needs a dense computed value")
                unit.source = Load(Access(source.buffer, source.dtype, 0, (1,)))
            for member in unit.members:
                unit.exprs[member.output.buffer] = self._apply(unit, member, unit.pmaps[member.output.buffer], unit.index)

        # which values must be stored: used outside their unit, or returned
        users: dict[str, list[Operation]] = {}
        for op in self.ops:
            for value in op.inputs:
                if isinstance(value, TensorSpec):
                    users.setdefault(value.buffer, []).append(op)
        dtypes = {spec.buffer: spec.dtype for spec in program.inputs}
        dtypes.update({op.output.buffer: op.output.dtype for op in self.ops})
        shapes = {spec.buffer: spec.shape for spec in program.inputs}
        shapes.update({op.output.buffer: op.output.shape for op in self.ops})
        # Reductions over a value that a tensor-core GEMM's epilogue holds in registers (the loss terms, dY for
        # the bias gradients) are summed there, chunk by chunk, instead of re-reading the value from memory.
        absorbed: dict[str, set[int]] = {}
        if self.fuse_epilogues:
            for unit in units:
                if unit.kind == "reduce":
                    self._fuse_reduction(unit, dtypes, shapes, absorbed)
        for unit in units:
            own = {m.output.buffer for m in unit.members}
            if unit.root is not None:
                own.add(unit.root.output.buffer)
            ordered = ([unit.root.output.buffer] if unit.root is not None else []) + [m.output.buffer for m in unit.members]
            for buffer in ordered:
                outside = any(user.output.buffer not in own and id(user) not in absorbed.get(buffer, ())
                              for user in users.get(buffer, []))
                if outside or buffer in self.output_buffers:
                    unit.stores.append(Store(buffer, dtypes[buffer]))
            # drop members that feed no store
            needed = {s.buffer for s in unit.stores} | {f.buffer for f in unit.fused}
            unit.stores += [Store(f.scratch, "float32") for f in unit.fused]
            for member in reversed(unit.members):
                if member.output.buffer in needed:
                    needed |= self._refs(unit.exprs[member.output.buffer])
            unit.members = [m for m in unit.members if m.output.buffer in needed]
            for buffer in list(unit.exprs):
                if buffer not in needed:
                    del unit.exprs[buffer]
            unit.reads = set()
            self._collect_reads(unit)

        # split large reductions into partial + finish
        units = self._split_reductions(units, dtypes, shapes)

        writer = {}
        for unit in units:
            for buffer in unit.writes:
                writer[buffer] = unit

        # output binding
        storage: dict[str, tuple] = {spec.buffer: ("in", i) for i, spec in enumerate(program.inputs)}
        # values that cross ranks live in the symmetric buffer: this rank's contribution and the reduced result
        symmetric = SYM_HEADER
        for unit in units:
            if unit.kind != "exchange":
                continue
            source = unit.root.inputs[0].buffer
            result = unit.root.output.buffer
            element = ELEMENT_BYTES[dtypes[source]]
            chunk = THREADS * 16                                   # bytes per exchange chunk
            chunks = -(-max(1, prod(shapes[source])) * element // chunk)
            owned = -(-chunks // self.world) * chunk               # bytes one rank receives from one source rank
            for buffer in (source, result):
                if buffer in storage:
                    raise ValueError("trainkernel: an exchanged value cannot also be an input or an exchange result")
            if self.multicast:
                # every rank keeps its contribution in its own buffer, laid out like the value; the owner of a
                # chunk fetches the sum over ranks through the multicast mapping
                storage[source] = ("sym", symmetric)
                symmetric += -(-max(1, prod(shapes[source])) * element // ALIGN) * ALIGN
            else:
                # contributions are scattered by their producers straight into the owning rank's staging area,
                # laid out [source rank][owned chunk]; the mean is laid out like the value itself
                storage[source] = ("scatter", symmetric, owned)
                symmetric += -(-self.world * owned // ALIGN) * ALIGN
            storage[result] = ("sym", symmetric)
            symmetric += -(-max(1, prod(shapes[source])) * element // ALIGN) * ALIGN
        native: dict[int, str] = {}
        copies: list[tuple[int, TensorSpec]] = []
        direct_candidates: dict[int, int] = {}
        output_slots: dict[str, list[int]] = {}
        for slot, spec in enumerate(program.outputs):
            output_slots.setdefault(spec.buffer, []).append(slot)
        for slot, spec in enumerate(program.outputs):
            full = spec.buffer in writer and _dense(spec) and _squeeze(spec.shape) == _squeeze(shapes[spec.buffer]) \
                and spec.dtype == dtypes[spec.buffer]
            if slot in self.inplace:
                target = self.inplace[slot]
                if full and spec.buffer not in storage and len(output_slots[spec.buffer]) == 1:
                    direct_candidates[slot] = target
                else:
                    copies.append((slot, spec))
            elif full and spec.buffer not in storage:
                storage[spec.buffer] = ("out", slot)
                native[slot] = spec.buffer
            else:
                copies.append((slot, spec))

        # data dependencies -> earliest stages
        ordering: list[tuple[Unit, Unit]] = []          # (before, after) pairs beyond read-after-write
        self._assign_stages(units, writer, ordering)

        # Direct versus staged commit of in-place state.  A direct commit lets the producing unit
        # overwrite the input; it is legal when the unit touches that input only element-for-element
        # and every other reader of the input can be ordered strictly before it.
        direct: dict[int, int] = {}
        staged: dict[int, int] = {}
        for slot, target in direct_candidates.items():
            spec = program.outputs[slot]
            target_buffer = program.inputs[target].buffer
            owner = writer[spec.buffer]
            readers = [u for u in units if u is not owner and target_buffer in u.reads]
            identity = self._identity_reads(owner, target_buffer, spec.buffer) and \
                not any(view.buffer == target_buffer for _, view in copies)
            trial = ordering + [(reader, owner) for reader in readers]
            if identity and owner.phase != "partial" and self._assign_stages(units, writer, trial):
                ordering = trial
                direct[slot] = target
            else:
                self._assign_stages(units, writer, ordering)
                staged[slot] = target
                copies.append((slot, spec))
        for slot, target in direct.items():
            storage[program.outputs[slot].buffer] = ("out", slot)
        for slot, spec in copies:
            if slot in self.inplace and slot not in staged:
                staged[slot] = self.inplace[slot]

        # Values derived from in-place state by a bare cast (the BF16 copies of FP32 master weights that the
        # tensor-core GEMMs read) are carried from one launch to the next: the unit that commits the updated
        # state also stores its cast, so the next launch can skip the casting unit when it is told that nobody
        # touched the state in between.  Two forms.  "pingpong": every carried value has two copies; a launch
        # reads copy r (a device-side word that flips every launch) and writes copy 1 - r, so the schedule does
        # not change.  "reorder": one copy, rewritten in place, legal when every reader of the copy can be
        # ordered strictly before the rewriting unit (the same constraint-graph test as a direct commit),
        # which moves dW of a layer one stage behind dX of the layer below.
        carry_bytes = 0
        # Left to itself (None) the planner carries only in kernels of large GEMMs (the ones that get two-CTA pair
        # tiles): there the casting stage is a quarter of a millisecond of HBM traffic and the extra BF16 store
        # hides behind a long main loop.  Measured on B200, the small MLP (batch 512) LOSES 5 to 11 us per step
        # with carrying, because its dW stages are bound by their epilogue stores.
        if self.carry is None:
            self.carry = "pingpong" if self._wants_pair_tiles(units) else False
        if self.carry and direct:
            slot_of_target = {target: slot for slot, target in direct.items()}
            for unit in list(units):
                if unit.kind != "point" or len(unit.members) != 1 or unit.members[0].op != "cast" or len(unit.stores) != 1:
                    continue
                cast = unit.members[0]
                source = cast.inputs[0]
                copy = cast.output.buffer
                if not isinstance(source, TensorSpec) or source.buffer not in self.input_index or copy in storage:
                    continue
                target = self.input_index[source.buffer]
                slot = slot_of_target.get(target)
                if slot is None or not _dense(source) or source.shape != program.inputs[target].shape or cast.output.shape != source.shape:
                    continue
                updated = program.outputs[slot].buffer
                owner = writer[updated]
                if owner.phase == "partial" or updated not in owner.pmaps or _squeeze(shapes[updated]) != _squeeze(cast.output.shape):
                    continue
                readers = [u for u in units if u is not unit and copy in u.reads]
                if self.carry == "reorder":
                    if owner in readers:
                        continue
                    trial = ordering + [(reader, owner) for reader in readers]
                    if not self._assign_stages(units, writer, trial):
                        self._assign_stages(units, writer, ordering)
                        continue
                    ordering = trial
                name = copy + "__next"
                value = TensorSpec(updated, shapes[updated], dtypes[updated], row_major(shapes[updated]), updated)
                again = Operation(name, "cast", (value,), TensorSpec(name, shapes[updated], cast.output.dtype, row_major(shapes[updated]), name))
                owner.members.append(again)
                owner.pmaps[name] = owner.pmaps[updated]
                owner.exprs[name] = Apply(again, (Ref(updated),))
                owner.stores.append(Store(name, cast.output.dtype))
                dtypes[name], shapes[name] = cast.output.dtype, shapes[updated]
                size = -(-max(1, prod(cast.output.shape)) * ELEMENT_BYTES[cast.output.dtype] // ALIGN) * ALIGN
                if self.carry == "pingpong":
                    # ("carry", offset when the phase word is 0, offset when it is 1)
                    storage[copy], storage[name] = ("carry", carry_bytes, carry_bytes + size), ("carry", carry_bytes + size, carry_bytes)
                    carry_bytes += 2 * size
                else:
                    storage[copy] = storage[name] = ("carry", carry_bytes, carry_bytes)
                    carry_bytes += size
                unit.carried = True

        # copy units for outputs that are views, duplicates, or staged commits
        position = len(self.ops)
        for slot, spec in copies:
            name = f"out{slot}_copy"
            result = TensorSpec(name, spec.shape, spec.dtype, row_major(spec.shape), name)
            op = Operation(name, "cast", (spec,), result)
            unit = Unit("point", name, position, spec.shape or (1,))
            position += 1
            unit.pmaps[name] = tuple(range(len(spec.shape)))
            unit.members.append(op)
            self.producer[name] = op
            saved = self.claimed
            self.claimed = dict(saved)
            self.claimed[name] = unit
            unit.exprs[name] = self._apply(unit, op, unit.pmaps[name], position)
            self.claimed = saved
            del self.producer[name]
            unit.stores.append(Store(name, spec.dtype))
            unit.reads = set()
            self._collect_reads(unit)
            storage[name] = ("out", slot)
            dtypes[name], shapes[name] = spec.dtype, spec.shape
            if slot in self.inplace:
                # a staged commit overwrites an input: it follows every other reader of that input
                target_buffer = program.inputs[self.inplace[slot]].buffer
                ordering += [(reader, unit) for reader in units if target_buffer in reader.reads]
            units.append(unit)
            writer[name] = unit
        if not self._assign_stages(units, writer, ordering):
            raise ValueError("trainkernel: cyclic stage constraints")

        # Streams that depend on nothing but program inputs (the BF16 weight shadows) run as late as
        # their first consumer allows, in a stage that has tensor-core GEMMs, where the epilogue warps
        # execute them in the background instead of in a stage of their own.
        tensor_stages = {u.stage for u in units if u.kind == "gemm" and u.path == "tc"} if self.background or self.late_casts else set()
        for unit in units:
            if unit.kind != "point" or any(buffer in writer for buffer in unit.reads):
                continue
            consumers = [u.stage for u in units if u is not unit and unit.writes & u.reads]
            if not consumers:
                continue
            target = min(consumers) - 1
            while target > unit.stage and target not in tensor_stages:
                target -= 1
            limit = min((after.stage for before, after in ordering if before is unit), default=target + 1)
            if unit.stage < target < limit:
                unit.stage = target
        occupied = sorted({u.stage for u in units})
        renumber = {old: new for new, old in enumerate(occupied)}
        for unit in units:
            unit.stage = renumber[unit.stage]

        # cross-rank ordering: pulls and reads of pushed results wait for the peers' previous barrier
        remote = {u.root.output.buffer for u in units if u.kind == "exchange"}
        signal: set[int] = set()
        for unit in units:
            if unit.kind == "exchange" or unit.reads & remote:
                if unit.stage == 0:
                    raise ValueError("trainkernel: an exchange cannot be scheduled in the first stage")
                unit.wait_barrier = unit.stage - 1
                signal.add(unit.stage - 1)

        # workspace arena
        stage_count = max((u.stage for u in units), default=0) + 1
        last_read: dict[str, int] = {}
        for unit in units:
            for buffer in unit.reads:
                last_read[buffer] = max(last_read.get(buffer, -1), unit.stage)
        arena: list[tuple[int, int, int]] = []      # (offset, size, free_after_stage)
        total = 0
        for unit in sorted(units, key=lambda u: (u.stage, u.index)):
            for store in unit.stores:
                if store.buffer in storage:
                    continue
                size = -(-max(1, prod(shapes[store.buffer])) * ELEMENT_BYTES[store.dtype] // ALIGN) * ALIGN
                free_after = max(last_read.get(store.buffer, unit.stage), unit.stage)
                best = None
                for i, (offset, room, until) in enumerate(arena):
                    if until < unit.stage and room >= size and (best is None or room < arena[best][1]):
                        best = i
                if best is None:
                    storage[store.buffer] = ("ws", total)
                    arena.append((total, size, free_after))
                    total += size
                else:
                    offset, room, _ = arena[best]
                    storage[store.buffer] = ("ws", offset)
                    arena[best] = (offset, size, free_after)
                    if room > size:
                        arena.append((offset + size, room - size, -1))

        # work items and grid
        tc_units = 0
        for unit in units:
            self._size_unit(unit)
            if unit.kind == "gemm" and unit.path in ("tc", "tc2"):
                tc_units += 1
        # Two-CTA pair tiles (256 x 256) when every tensor-core GEMM is large enough to keep the
        # clusters busy; a kernel uses one cta_group for all of its tcgen05 instructions.
        tc = [u for u in units if u.kind == "gemm" and u.path == "tc"]
        pair_tiles = [-(-u.mnk[0] // 256) * -(-u.mnk[1] // 256) for u in tc]
        two_cta = self._wants_pair_tiles(units)
        if two_cta:
            for unit, tiles in zip(tc, pair_tiles):
                unit.path, unit.block_n, unit.items = "tc2", 256, 2 * tiles
        per_stage = [0] * stage_count
        for unit in units:
            per_stage[unit.stage] += unit.items
        grid = max(1, min(SM_COUNT, max(per_stage)))
        if self.max_blocks is not None:
            grid = max(1, min(grid, self.max_blocks))
        if two_cta:
            grid = max(2, grid - grid % 2)
        # Small programs are bound by the latency of their stage boundaries, not by throughput: run them as
        # ONE cluster of at most 8 blocks, whose hardware barrier costs a fraction of a barrier through global
        # memory, instead of spreading a few microseconds of work over the whole GPU.
        work = 0
        for unit in units:
            if unit.kind == "gemm":
                work += 2 * prod(unit.mnk) * (1 if unit.path in ("tc", "tc2") else 16)      # CUDA-core products want more SMs
            else:
                work += 16 * max(1, prod(unit.dims)) * (max(1, prod(unit.reduced)) if unit.kind == "reduce" else 1)
        small = self.world == 1 and not two_cta and work <= CLUSTER_WORK_LIMIT
        cluster_blocks = 0
        if small if self.cluster_barrier is None else (self.cluster_barrier and self.world == 1 and not two_cta):
            cluster_blocks = 1
            while cluster_blocks * 2 <= min(MAX_CLUSTER, grid):
                cluster_blocks *= 2
            grid = cluster_blocks
        return Plan(program, sorted(units, key=lambda u: (u.stage, u.index)), stage_count, storage, dtypes, shapes,
                    max(total, ALIGN), inlined, direct, staged, native, grid, tc_units, tc_units > 0, two_cta,
                    self.world, symmetric if symmetric > SYM_HEADER else 0, tuple(sorted(signal)), self.background, self.multicast, cluster_blocks,
                    carry_bytes, bool(carry_bytes) and self.carry == "pingpong", self.exchange_chunks)

    # -- helpers ---------------------------------------------------------------------
    def _refs(self, expr) -> set[str]:
        if isinstance(expr, Ref):
            return {expr.buffer}
        if isinstance(expr, Apply):
            out: set[str] = set()
            for arg in expr.args:
                out |= self._refs(arg)
            return out
        return set()

    def _loads(self, expr, out: list) -> None:
        if isinstance(expr, Load):
            out.append(expr.access)
        elif isinstance(expr, Apply):
            for arg in expr.args:
                self._loads(arg, out)

    def _collect_reads(self, unit: Unit) -> None:
        found: list[Access] = []
        for expr in unit.exprs.values():
            self._loads(expr, found)
        if unit.bias is not None:
            self._loads(unit.bias, found)
        if unit.source is not None and unit.phase != "finish":
            self._loads(unit.source, found)
        unit.reads |= {a.buffer for a in found}
        if unit.kind == "gemm":
            unit.reads |= {unit.a.buffer, unit.b.buffer}
        if unit.phase == "finish":
            unit.reads.add(unit.scratch)

    def _identity_reads(self, unit: Unit, target: str, stored: str) -> bool:
        """Every read of `target` inside `unit` touches exactly the element being written."""
        if unit.kind == "gemm" and target in (unit.a.buffer, unit.b.buffer):
            return False
        if unit.kind == "reduce" and unit.source is not None:
            probe: list[Access] = []
            self._loads(unit.source, probe)
            if any(a.buffer == target for a in probe):
                return False
        dense = row_major(unit.dims)
        live = [d for d, n in enumerate(unit.dims) if n > 1]
        found: list[Access] = []
        for expr in unit.exprs.values():
            self._loads(expr, found)
        if unit.bias is not None:
            self._loads(unit.bias, found)
        for access in found:
            if access.buffer == target and (access.offset != 0 or any(access.strides[d] != dense[d] for d in live)):
                return False
        return True

    def _assign_stages(self, units: list[Unit], writer: dict[str, Unit], ordering: list[tuple[Unit, Unit]]) -> bool:
        """Earliest stage per unit (longest path); False, leaving stages untouched, when constraints are cyclic."""
        after: dict[int, list[Unit]] = {id(u): [] for u in units}
        pending: dict[int, int] = {id(u): 0 for u in units}
        edges = list(ordering)
        for unit in units:
            for buffer in unit.reads:
                source = writer.get(buffer)
                if source is not None and source is not unit:
                    edges.append((source, unit))
        for before, later in edges:
            after[id(before)].append(later)
            pending[id(later)] += 1
        stage = {id(u): 0 for u in units}
        ready = [u for u in sorted(units, key=lambda u: u.index) if pending[id(u)] == 0]
        done = 0
        while ready:
            unit = ready.pop()
            done += 1
            for later in after[id(unit)]:
                stage[id(later)] = max(stage[id(later)], stage[id(unit)] + 1)
                pending[id(later)] -= 1
                if pending[id(later)] == 0:
                    ready.append(later)
        if done != len(units):
            return False
        for unit in units:
            unit.stage = stage[id(unit)]
        return True

    def _split_reductions(self, units: list[Unit], dtypes: dict, shapes: dict) -> list[Unit]:
        result: list[Unit] = []
        for unit in units:
            if unit.kind != "reduce" or unit.phase == "finish":
                result.append(unit)
                continue
            outputs, size = prod(unit.kept), prod(unit.reduced)
            if unit.no_split:
                unit.strategy, unit.parts = ("thread" if size <= 32 else "block"), 1
                result.append(unit)
                continue
            loads: list[Access] = []
            self._loads(unit.source, loads)
            wide = [a for a in loads if any(a.strides)]
            kept_rank = len(unit.kept)
            inner_kept = False
            if wide:
                unit_strides = [d for d, s in enumerate(wide[0].strides) if s == 1]
                inner_kept = bool(unit_strides) and unit_strides[-1] < kept_rank
            if (outputs >= 32 and (inner_kept or size <= 128)) or size <= 32:      # a few terms per output: one thread each
                unit.strategy = "thread"
                unit.vector = bool(unit.kept[-1] % 8 == 0 and outputs >= 8 * THREADS and loads
                                   and all(a.strides[kept_rank - 1] in (0, 1) for a in loads))
                blocks = -(-outputs // (THREADS * 8 if unit.vector else THREADS))
                parts = min(max(1, SM_COUNT // blocks), max(1, size // 64), 64)
            else:
                unit.strategy = "block"
                parts = min(max(1, SM_COUNT // max(1, outputs)), max(1, size // (THREADS * 64)), 256)
            unit.parts = parts
            if parts == 1:
                result.append(unit)
                continue
            scratch = f"{unit.name}__partials"
            dtypes[scratch], shapes[scratch] = "float32", (parts, outputs)
            partial = Unit("reduce", unit.name + "_partial", unit.index, unit.dims, root=unit.root, kept=unit.kept,
                           reduced=unit.reduced, source=unit.source, strategy=unit.strategy, parts=parts, phase="partial",
                           scratch=scratch, vector=unit.vector)
            partial.stores.append(Store(scratch, "float32"))
            self._collect_reads(partial)
            unit.phase, unit.scratch = "finish", scratch
            unit.reads = set()
            self._collect_reads(unit)
            result.extend((partial, unit))
        return result

    def _size_unit(self, unit: Unit) -> None:
        if unit.kind == "gemm":
            m, n, k = unit.mnk
            if unit.path == "tc":
                tiles_m = -(-m // 128)
                choice = self.forced_block_n
                if choice is None and self.wave_aware_tiles:
                    # A mid-size GEMM's main loop is bound by what an SM pulls from L2 per K block, (128 + BN) rows of
                    # 128 bytes, and its tiles run in waves of one per SM: take the width with the least waves x bytes.
                    # (An experiment, off by default: on the small MLP it gives the dW GEMMs one 128 x 128 or 128 x 256
                    # tile per block instead of two or four narrow ones, and the step got SLOWER, 144 against 134 us,
                    # because a block with a single tile cannot overlap its epilogue with a next main loop.)
                    choice = min((64, 128, 256), key=lambda bn: (-(-(tiles_m * -(-n // bn)) // SM_COUNT) * (128 + bn), bn))
                    choice = min(choice, max(64, -(-n // 64) * 64))
                elif choice is None:
                    choice = 64
                    for bn in (256, 128):
                        if tiles_m * -(-n // bn) >= SM_COUNT:
                            choice = bn
                            break
                    choice = min(choice, max(64, -(-n // 64) * 64))
                unit.block_n = choice
                unit.items = tiles_m * -(-n // choice)
            elif unit.path == "gemv":
                warps = THREADS // 32
                if unit.b.strides[0] == 1 and unit.b.strides[1] != 1:
                    per = warps                              # K-major weight: one warp per output column
                else:
                    # columns per warp: 64, or 8 when that is what it takes to occupy a handful of blocks
                    unit.block_n = 64 if -(-n // (64 * warps)) >= MAX_CLUSTER else 8
                    per = unit.block_n * warps
                unit.items = -(-n // per)
            else:
                unit.items = -(-m // 32) * -(-n // 32)
        elif unit.kind == "exchange":
            # one item = EXCHANGE_CHUNKS_PER_ITEM owned chunks of THREADS x 16 bytes; chunk c belongs to rank c % world
            nbytes = prod(unit.dims) * ELEMENT_BYTES[unit.root.output.dtype]
            chunks = -(-nbytes // (THREADS * 16))
            unit.items = max(1, -(-(-(-chunks // self.world)) // self.exchange_chunks))
        elif unit.kind == "reduce":
            outputs = prod(unit.kept)
            if unit.phase == "finish":
                unit.items = -(-outputs // THREADS)
            elif unit.strategy == "thread":
                unit.items = -(-outputs // (THREADS * 8 if unit.vector else THREADS)) * unit.parts
            else:
                unit.items = outputs * unit.parts
        else:
            total = prod(unit.dims)
            unit.items = max(1, -(-total // (THREADS * 8 * point_unroll(total, len(unit.reads) + len(unit.stores)))))
