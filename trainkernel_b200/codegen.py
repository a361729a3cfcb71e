"""CUDA emission for the sm_100a training-step kernel.

`generate(program, **options)` validates the program, plans it (`plan.py`) and
emits ONE cooperative persistent kernel `tk_step`: stages separated by the
hand-written grid barrier, dense contractions as `tk::gemm_tc` (tcgen05 + TMEM +
TMA), `tk::gemm_simt` (exact FP32) or `tk::gemv16` calls with a generated
epilogue functor, and generated pointwise / reduction loops.  It needs neither
a GPU nor the CUDA toolkit.  The entry point and the `GeneratedKernel` counters
keep the reference's names (reference: trainkernel/codegen.py:44-55, 771-815);
the emitters themselves (reference: codegen.py:339-646, wmma.py, sm90.py,
gemv.py) are replaced by the sm_100a device library in `csrc/tk_device.cuh`.
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass, field
from math import prod

from .ir import Operation, Program, TensorSpec, row_major, validate
from .plan import (ELEMENT_BYTES, SYM_HEADER, THREADS, Access, Apply, Const, Iota, Load, Plan, Planner, Ref, Unit, point_unroll)

TENSOR_RATE = 1.4e15             # flop/s the planner assumes for tensor-core GEMM tiles when it balances a stage
STREAM_RATE = 5.0e12             # bytes/s it assumes for a pointwise stream run by the worker warps
STREAM_WARPS = 4                 # tk::kStreamWarps: extra warps of a kernel generated with background=True
MAX_STAMPED_STAGES = 55          # stamp area: 64 words per table, the peer-wait table shares its block with the role trace
FLAG_WORDS_PER_RANK = 64         # cross-rank "passed barrier k" words per rank in the symmetric header

CTYPE = {"float32": "float", "float16": "__half", "bfloat16": "__nv_bfloat16", "int64": "long long", "int32": "int", "bool": "bool"}
ROUND = {"float32": "tk::F32", "float16": "tk::F16", "bfloat16": "tk::BF16", "int64": "tk::I64", "int32": "tk::I32", "bool": "tk::B8"}


def contiguous_strides(shape: tuple[int, ...]) -> tuple[int, ...]:
    return row_major(shape)


def numel(shape: tuple[int, ...]) -> int:
    return prod(shape)


def _literal(value: int | float) -> str:
    value = float(value)
    if not math.isfinite(value):
        raise ValueError("trainkernel: non-finite scalar constants are unsupported")
    return f"{value:.17e}f"


@dataclass(frozen=True)
class TensorMapSpec:
    """Recipe for one CUtensorMap, encoded by the runtime shim at launch time."""
    base: tuple            # ("in", i) | ("out", slot) | ("ws", byte offset)
    byte_offset: int       # extra offset from the base pointer
    inner: int             # extent of the unit-stride dimension (elements)
    outer: int
    outer_stride_bytes: int
    box_inner: int
    box_outer: int


@dataclass(frozen=True)
class GeneratedKernel:
    source: str
    workspace_elements: int               # FP32 elements, as the reference counts workspace
    materialized_operations: int
    inlined_operations: int
    tensor_core_operations: int
    blocks_per_sm: int
    max_work_blocks: int
    grid_barriers: int
    direct_outputs: int
    direct_state_commits: int = 0
    # sm_100a additions
    entry: str = "tk_step"
    threads: int = THREADS
    dynamic_smem: int = 0
    grid: int = 1
    tensor_maps: tuple = ()
    input_count: int = 0
    output_count: int = 0
    stages: int = 1
    units: tuple = ()                     # (stage, kind, name, path, items) per unit, for inspection
    staged_state_commits: int = 0
    param_bytes: int = 0
    workspace_bytes: int = 0
    cluster: int = 1                      # thread-block cluster size the kernel must be launched with
    barrier: str = "grid"                 # "grid": barrier through global memory; "cluster": the grid is one cluster, hardware barrier
    world: int = 1                        # ranks the kernel exchanges with (1: no exchange stages)
    multicast: bool = False               # exchanges through the multicast mapping (one more extra input)
    symmetric_bytes: int = 0              # size of the peer-mapped buffer the kernel expects after the program inputs
    carry_bytes: int = 0                  # size of the carry buffer the kernel expects as its LAST input (0: none)
    aligned_inputs: tuple = ()            # kernel inputs whose base pointer must be 16-byte aligned (the launch refuses others)
    aligned_outputs: tuple = ()           # likewise for kernel outputs
    aligned_workspace: bool = False       # likewise for the workspace


class _Body:
    """Line buffer with indentation and unique temporary names."""

    def __init__(self) -> None:
        self.lines: list[str] = []
        self.depth = 0
        self.counter = 0

    def emit(self, text: str) -> None:
        self.lines.append("    " * self.depth + text)

    def temp(self, stem: str) -> str:
        self.counter += 1
        return f"{stem}{self.counter}"

    def text(self) -> str:
        return "\n".join(self.lines)


class _Emitter:
    def __init__(self, plan: Plan):
        self.plan = plan
        read_anywhere = set()
        for unit in plan.units:
            read_anywhere |= unit.reads
        # buffers nobody reads back inside the kernel: written (or, for in-place state, read) exactly once late in the step
        self.write_once = {b for b, where in plan.storage.items() if where[0] == "out" and b not in read_anywhere}
        self.state_inputs = {plan.program.inputs[i].buffer for i in set(plan.direct_commits.values()) | set(plan.staged_commits.values())}
        self.maps: list[TensorMapSpec] = []
        self.functors: list[str] = []
        self.needs_simt = False
        self.raster_group = 8
        self.trace_stage = None
        self.epilogue_lookahead = True
        self.stream_everything = False   # A/B switch: every flat pointwise stream goes to the stream warps, covered or not
        self.stream_piece = 3            # 32-thread slices of a work item that one background piece covers (1, 2, 3 or 6)
        self.rows = False
        self.background = plan.background
        self.wide_epilogue = False       # eight epilogue warps per cta_group::1 GEMM tile instead of four
        self.simt_depth = None           # K depth a SIMT GEMM stages per step; None: 32, 64 or 128 by the product's K
        self.assume_aligned = True       # tensor-core epilogues may lean on 16-byte aligned base pointers (checked at launch)
        self._full_rows = False          # set while the functor of such an epilogue is written
        self.aligned_inputs: set[int] = set()
        self.aligned_outputs: set[int] = set()
        self.aligned_workspace = False
        self.threads = THREADS + (32 * STREAM_WARPS if plan.background else 0)
        exchanging = plan.symmetric_bytes > 0
        # kernel inputs beyond the program's own: [symmetric buffer, every rank's mapping of it, (multicast mapping)], [carry buffer]
        self.exchange_inputs = 1 + plan.world + int(plan.multicast) if exchanging else 0
        self.carry_input = len(plan.program.inputs) + self.exchange_inputs
        self.extra_inputs = self.exchange_inputs + (1 if plan.carry_bytes else 0)

    # -- addressing ------------------------------------------------------------------
    def pointer(self, buffer: str, dtype: str, const: bool) -> str:
        where = self.plan.storage[buffer]
        ctype = CTYPE[dtype]
        if where[0] == "in":
            raw = f"P.in[{where[1]}]"
            return f"reinterpret_cast<const {ctype}*>({raw})" if const else f"reinterpret_cast<{ctype}*>(const_cast<void*>({raw}))"
        if where[0] == "out":
            return f"reinterpret_cast<{'const ' if const else ''}{ctype}*>(P.out[{where[1]}])"
        if where[0] == "scatter":
            raise ValueError(f"trainkernel: {buffer} is staged for a cross-rank exchange and cannot be read in place")
        if where[0] == "carry":
            local = f"reinterpret_cast<uint8_t*>(const_cast<void*>(P.in[{self.carry_input}]))"
            offset = f"{where[1]}ULL" if where[1] == where[2] else f"(tk_carry_phase ? {where[2]}ULL : {where[1]}ULL)"
            return f"reinterpret_cast<{'const ' if const else ''}{ctype}*>({local} + {offset})"
        if where[0] == "sym":
            local = f"reinterpret_cast<uint8_t*>(const_cast<void*>(P.in[{len(self.plan.program.inputs)}]))"
            return f"reinterpret_cast<{'const ' if const else ''}{ctype}*>({local} + {where[1]}ULL)"
        return f"reinterpret_cast<{'const ' if const else ''}{ctype}*>(P.ws + {where[1]}ULL)"

    @staticmethod
    def _affine(offset: int, strides: tuple[int, ...], coords: list[str], skip_last: bool) -> str:
        terms = [f"{offset}LL"] if offset else []
        last = len(strides) - 1
        for d, (stride, coord) in enumerate(zip(strides, coords)):
            if stride == 0 or (skip_last and d == last and False):
                continue
            terms.append(f"(int64_t)({coord}) * {stride}LL")
        return " + ".join(terms) if terms else "0LL"

    # -- expressions -----------------------------------------------------------------
    # Values are emitted either as `float v[W]` (one run of W consecutive elements) or, inside GEMM
    # epilogue functors, as `float v[R][W]` (R such runs in different rows, all loads issued before
    # any store).  `self.rows` selects the second form; coordinates may then mention the row index `r`.
    def _decl(self, name: str, width: str) -> str:
        return f"float {name}[R][{width}];" if self.rows else f"float {name}[{width}];"

    def _loop(self, width: str) -> str:
        inner = f"_Pragma(\"unroll\") for (int j = 0; j < {width}; ++j)"
        return f"_Pragma(\"unroll\") for (int r = 0; r < R; ++r) {inner}" if self.rows else inner

    def _row_loop(self) -> str:
        return "_Pragma(\"unroll\") for (int r = 0; r < R; ++r) " if self.rows else ""

    @property
    def _at(self) -> str:
        return "[r][j]" if self.rows else "[j]"

    @property
    def _row(self) -> str:
        return "[r]" if self.rows else ""

    def value(self, expr, body: _Body, env: dict, width: str, coords: list[str], nvalid: str, vdim: int = -1) -> str:
        """Emit code computing `expr` for `width` consecutive elements along dim `vdim` (default: last); returns the array name."""
        key = id(expr)
        if key in env:
            return env[key]
        if isinstance(expr, Ref):
            return env["ref:" + expr.buffer]
        if isinstance(expr, Const):
            name = body.temp("k")
            body.emit(self._decl(name, width))
            body.emit(f"{self._loop(width)} {name}{self._at} = {_literal(expr.value)};")
            env[key] = name
            return name
        if isinstance(expr, Iota):
            name = body.temp("i")
            rank = len(coords)
            along = expr.dim is not None and (expr.dim == vdim or expr.dim == vdim + rank)
            start = coords[expr.dim] if expr.dim is not None else "0"
            body.emit(self._decl(name, width))
            body.emit(f"{self._loop(width)} {name}{self._at} = (float)(({start}) + {'j' if along else '0'});")
            env[key] = name
            return name
        if isinstance(expr, Load):
            access = expr.access
            cache_key = ("load", access)
            if cache_key in env:
                return env[cache_key]
            name = body.temp("l")
            body.emit(self._decl(name, width))
            self._emit_load(access, body, name, width, coords, nvalid, vdim)
            env[cache_key] = name
            env[key] = name
            return name
        assert isinstance(expr, Apply)
        op = expr.op
        args = []
        for arg in expr.args:
            if isinstance(arg, Const):
                args.append(_literal(arg.value))
            else:
                args.append(self.value(arg, body, env, width, coords, nvalid, vdim) + self._at)
        formula = self.formula(op, args)
        name = body.temp("v")
        body.emit(self._decl(name, width))
        body.emit(f"{self._loop(width)} {name}{self._at} = {ROUND[op.output.dtype]}::rnd({formula});")
        env[key] = name
        return name

    def _aligned_base(self, buffer: str) -> bool:
        """True when `buffer` starts on a 16-byte boundary, given base pointers that do; records which base
        pointers the proof leans on (the host checks those at every launch)."""
        where = self.plan.storage[buffer]
        if where[0] == "in":
            self.aligned_inputs.add(where[1])
        elif where[0] == "out":
            self.aligned_outputs.add(where[1])
        elif where[0] == "carry":
            if where[1] % 16 or where[2] % 16:
                return False
            self.aligned_inputs.add(self.carry_input)
        elif where[0] == "sym":
            if where[1] % 16:
                return False
            self.aligned_inputs.add(len(self.plan.program.inputs))
        elif where[0] == "scatter":
            return False
        else:
            if where[1] % 16:
                return False
            self.aligned_workspace = True
        return True

    def _full_run(self, buffer: str, dtype: str, offset: int, strides: tuple[int, ...], vdim: int = -1) -> bool:
        """Inside a tensor-core epilogue whose N is a multiple of 8: can a run of 4 or 8 elements of this access
        only be wholly valid or wholly invalid, and 16-byte aligned when valid?"""
        if not self._full_rows or dtype not in ("float32", "bfloat16", "float16") or not strides:
            return False
        unit = 16 // ELEMENT_BYTES[dtype]
        axis = vdim % len(strides)
        if strides[axis] != 1 or offset % unit or any(stride % unit for d, stride in enumerate(strides) if d != axis):
            return False
        return self._aligned_base(buffer)

    def _emit_load(self, access: Access, body: _Body, name: str, width: str, coords: list[str], nvalid: str, vdim: int = -1) -> None:
        """`width` consecutive elements (along dim `vdim`) of a stored value at `coords`, into array `name`."""
        address = self._affine(access.offset, access.strides, coords, False)
        step = access.strides[vdim] if access.strides else 0
        if self._full_run(access.buffer, access.dtype, access.offset, access.strides, vdim):
            stream = "true" if access.buffer in self.state_inputs and access.dtype == "float32" else "false"
            body.emit(f"{self._row_loop()}tk::ld_row_full<{width}, {stream}>({self.pointer(access.buffer, access.dtype, True)} + ({address}), {nvalid}, {name}{self._row});")
            return
        loader = "ld_row_stream" if access.buffer in self.state_inputs and access.dtype == "float32" else "ld_row_strided"
        body.emit(f"{self._row_loop()}tk::{loader}<{width}>({self.pointer(access.buffer, access.dtype, True)} + ({address}), {step}LL, {nvalid}, {name}{self._row});")

    @staticmethod
    def formula(op: Operation, a: list[str]) -> str:
        kind = op.op
        if kind in ("add", "sub"):
            sign = "+" if kind == "add" else "-"
            return f"({a[0]} {sign} ({_literal(op.attrs.get('alpha', 1))} * {a[1]}))"
        if kind == "mul":
            return f"({a[0]} * {a[1]})"
        if kind == "div":
            return f"({a[0]} / {a[1]})"
        if kind == "neg":
            return f"(-({a[0]}))"
        if kind == "relu":
            return f"tk::relu({a[0]})"
        if kind == "pow":
            exponent = op.inputs[1] if len(op.inputs) > 1 else op.attrs.get("exponent", 2)
            if not isinstance(exponent, (int, float)):
                raise ValueError("trainkernel: pow exponent must be a scalar")
            if exponent == 2:
                return f"({a[0]} * {a[0]})"
            if exponent == 1:
                return f"({a[0]})"
            return f"powf({a[0]}, {_literal(exponent)})"
        if kind == "threshold_backward":
            return f"(({a[1]} <= {_literal(op.attrs.get('threshold', 0))}) ? 0.0f : {a[0]})"
        if kind == "full":
            return _literal(op.attrs.get("value", op.inputs[0] if op.inputs else 0))
        if kind == "cast":
            return a[0]
        if kind == "eq":
            return f"(({a[0]} == {a[1]}) ? 1.0f : 0.0f)"
        if kind == "arange":
            return a[0]
        raise ValueError(f"trainkernel: unsupported pointwise operation {kind}")

    def _preload(self, expr, body: _Body, env: dict, width: str, coords: list[str], nvalid: str) -> None:
        """Emit only the loads of `expr` (cached in `env`), so they can all be in flight before any store."""
        if isinstance(expr, Load):
            self.value(expr, body, env, width, coords, nvalid)
        elif isinstance(expr, Apply):
            for arg in expr.args:
                self._preload(arg, body, env, width, coords, nvalid)

    def dag(self, unit: Unit, body: _Body, env: dict, width: str, coords: list[str], nvalid: str) -> None:
        """Members in order, then the unit's stores, for `width` elements at `coords`."""
        for member in unit.members:
            buffer = member.output.buffer
            env["ref:" + buffer] = self.value(unit.exprs[buffer], body, env, width, coords, nvalid)
        dense = row_major(unit.dims)
        partials = {f.scratch for f in unit.fused}
        for store in unit.stores:
            if unit.phase == "partial" or store.buffer in partials:
                continue
            address = self._affine(0, dense, coords, False)
            where = self.plan.storage[store.buffer]
            if where[0] == "scatter":
                n_inputs = len(self.plan.program.inputs)
                body.emit(f"{self._row_loop()}tk::st_row_scatter<{width}, {self.plan.world}, {CTYPE[store.dtype]}>(&P.in[{n_inputs + 1}], {where[1]}ULL, {where[2]}ULL, "
                          f"reinterpret_cast<const uint32_t*>(P.in[{n_inputs}])[1], {address}, {nvalid}, {env['ref:' + store.buffer]}{self._row});")
                continue
            if self._full_run(store.buffer, store.dtype, 0, dense):
                stream = "true" if store.buffer in self.write_once else "false"
                body.emit(f"{self._row_loop()}tk::st_row_full<{width}, {stream}>({self.pointer(store.buffer, store.dtype, False)} + ({address}), {nvalid}, {env['ref:' + store.buffer]}{self._row});")
                continue
            storer = "st_row_stream" if store.buffer in self.write_once else "st_row"
            body.emit(f"{self._row_loop()}tk::{storer}<{width}>({self.pointer(store.buffer, store.dtype, False)} + ({address}), {nvalid}, {env['ref:' + store.buffer]}{self._row});")

    # -- units -------------------------------------------------------------------------
    def functor(self, unit: Unit) -> str:
        """Epilogue functor of a GEMM unit: rounds the accumulator, runs the DAG, stores.

        `run_rows<R, W>` handles R runs of W consecutive columns, run r in row `x0 + r * rs`;
        rows at or beyond M get a zero element count, which turns their loads and stores off.
        `run<W>` is the single-run form.
        """
        op = unit.root
        name = f"Epi_{unit.name}"
        # every stored value the epilogue reads, in a fixed order: fetched by `load_rows`, consumed by `run_rows`
        operands: list[Access] = []

        def gather(expr) -> None:
            if isinstance(expr, Load):
                if expr.access not in operands:
                    operands.append(expr.access)
            elif isinstance(expr, Apply):
                for arg in expr.args:
                    gather(arg)

        if unit.bias is not None:
            gather(unit.bias)
        for expr in unit.exprs.values():
            gather(expr)
        self.rows = True
        # N a multiple of 8: every run of 4 or 8 columns a lane handles is wholly inside the tile or wholly outside it
        self._full_rows = self.assume_aligned and unit.path in ("tc", "tc2") and unit.mnk[1] % 8 == 0
        coords = ["(x0 + r * rs)", "x1"]
        mask = f"_Pragma(\"unroll\") for (int r = 0; r < R; ++r) nv[r] = (x0 + r * rs < {unit.mnk[0]}) ? nvalid : 0;"
        fetch = _Body()
        fetch.depth = 2
        fetch.emit("int nv[R];")
        fetch.emit(mask)
        env: dict = {}
        for i, access in enumerate(operands):
            self._emit_load(access, fetch, f"L.l{i}", "W", coords, "nv[r]")
            env[("load", access)] = f"L.l{i}"
        body = _Body()
        body.depth = 2
        body.emit("int nv[R];")
        body.emit(mask)
        root = body.temp("v")
        rounding = ROUND[op.output.dtype]
        if op.op == "addmm":
            alpha, beta = op.attrs.get("alpha", 1), op.attrs.get("beta", 1)
            if unit.bias is not None:
                bias = self.value(unit.bias, body, env, "W", coords, "nv[r]")
            if alpha == 0 and beta == 0:
                combine = "0.0f"
            elif beta == 0:
                combine = f"({_literal(alpha)} * (acc[r][j]))"
            elif alpha == 0:
                combine = f"({_literal(beta)} * ({bias}[r][j]))"
            else:
                combine = f"({_literal(alpha)} * (acc[r][j]) + {_literal(beta)} * ({bias}[r][j]))"
        else:
            combine = "acc[r][j]"
        body.emit(f"float {root}[R][W];")
        body.emit(f"{self._loop('W')} {root}[r][j] = {rounding}::rnd({combine});")
        env["ref:" + op.output.buffer] = root
        self.dag(unit, body, env, "W", coords, "nv[r]")
        for fused in unit.fused:
            self._fused_reduce(unit, fused, body, env)
        self.rows = False
        self._full_rows = False
        partials = {f.scratch for f in unit.fused}
        wide = any(ELEMENT_BYTES[s.dtype] == 4 for s in unit.stores if s.buffer not in partials)
        # tile-shaped operands (same row/column as the accumulator): worth prefetching into L2 a tile ahead
        fetched = [a for a in operands if a.strides[0] != 0 and a.strides[1] == 1]
        prefetch = "".join(
            f"        tk::prefetch_l2({self.pointer(a.buffer, a.dtype, True)} + ({a.offset}LL + (int64_t)row * {a.strides[0]}LL + col0), ncols * {ELEMENT_BYTES[a.dtype]});\n"
            for a in fetched)
        # The tensor-core epilogue keeps the operands of the NEXT 32-column chunk in flight while it works on the
        # current one; each operand costs 32 registers per chunk, so only epilogues with few operands do it.
        pipelined = self.epilogue_lookahead is True and 0 < len(operands) <= (1 if self.threads > THREADS else 2)
        fetch_first = self.epilogue_lookahead == "first" and 0 < len(operands) <= 2
        fields = " ".join(f"float l{i}[R][W];" for i in range(len(operands)))
        self.functors.append(
            f"struct {name} {{\n"
            f"    static constexpr bool kWide = {'true' if wide else 'false'};   // stores FP32 tiles: prefer 4-column runs\n"
            f"    static constexpr bool kPipelined = {'true' if pipelined else 'false'};   // fetch a chunk's operands one chunk ahead\n"
            f"    static constexpr bool kFetchFirst = {'true' if fetch_first else 'false'};   // fetch the first chunk's operands before waiting for the accumulator\n"
            f"    template <int R, int W> struct Ops {{ {fields} }};   // what the epilogue reads for R runs of W columns\n"
            f"    template <int R, int W> static __device__ __forceinline__ void load_rows(const Params& P, int x0, int rs, int x1, int nvalid, Ops<R, W>& L) {{\n"
            f"{fetch.text()}\n"
            f"    }}\n"
            f"    template <int R, int W> static __device__ __forceinline__ void run_rows(const Params& P, int x0, int rs, int x1, int nvalid, const float (*acc)[W], const Ops<R, W>& L) {{\n"
            f"{body.text()}\n"
            f"    }}\n"
            f"    template <int W> static __device__ __forceinline__ void run(const Params& P, int x0, int x1, int nvalid, const float* acc) {{\n"
            f"        Ops<1, W> L;\n"
            f"        load_rows<1, W>(P, x0, 0, x1, nvalid, L);\n"
            f"        run_rows<1, W>(P, x0, 0, x1, nvalid, reinterpret_cast<const float (*)[W]>(acc), L);\n"
            f"    }}\n"
            f"    static __device__ __forceinline__ void prefetch(const Params& P, int row, int col0, int ncols) {{\n"
            f"{prefetch}"
            f"    }}\n}};\n")
        return name

    def _fused_reduce(self, unit: Unit, fused, body: _Body, env: dict) -> None:
        """Partial sums of a member value over the 32 x 32 accumulator chunk a warp's epilogue call covers.

        Inside `run_rows<R, W>` the 32 lanes of the warp hold the chunk as R runs of W columns each: lanes that
        differ only above bit log2(32 / W) hold the same columns of different rows.  Rows at or beyond M and
        columns at or beyond the run's valid count are left out.  The butterfly adds in a fixed order, so the
        partials, and the finish over them, are deterministic.
        """
        m, n = unit.dims
        value = env["ref:" + fused.buffer]
        scratch = self.pointer(fused.scratch, "float32", False)
        body.emit(f"// partial sums of {fused.buffer} for {fused.scratch} ({fused.mode})")
        if fused.mode == "cols":
            name = body.temp("cs")
            body.emit(f"float {name}[W];")
            body.emit(f"_Pragma(\"unroll\") for (int j = 0; j < W; ++j) {{ {name}[j] = 0.0f; _Pragma(\"unroll\") for (int r = 0; r < R; ++r) {name}[j] += (j < nv[r]) ? {value}[r][j] : 0.0f; }}")
            body.emit(f"_Pragma(\"unroll\") for (int o = 32 / W; o < 32; o <<= 1) {{ _Pragma(\"unroll\") for (int j = 0; j < W; ++j) {name}[j] += __shfl_xor_sync(0xffffffffu, {name}[j], o); }}")
            body.emit(f"if ((threadIdx.x & 31) < 32 / W && x0 < {m}) tk::st_row<W>({scratch} + ((int64_t)(x0 >> 5) * {n}LL + x1), nvalid, {name});")
        else:
            name = body.temp("ts")
            chunks_n = -(-n // 32)
            body.emit(f"float {name} = 0.0f;")
            body.emit(f"_Pragma(\"unroll\") for (int r = 0; r < R; ++r) {{ _Pragma(\"unroll\") for (int j = 0; j < W; ++j) {name} += (j < nv[r]) ? {value}[r][j] : 0.0f; }}")
            body.emit(f"_Pragma(\"unroll\") for (int o = 16; o; o >>= 1) {name} += __shfl_xor_sync(0xffffffffu, {name}, o);")
            body.emit(f"if ((threadIdx.x & 31) == 0 && x0 < {m}) {scratch}[(int64_t)(x0 >> 5) * {chunks_n}LL + (x1 >> 5)] = {name};")

    def _tensor_map(self, operand, rows: int, depth: int, box_rows: int) -> tuple[str, bool]:
        """Register the tensor map(s) for a [rows, depth] operand; returns (index expression, is_mn_major).

        An operand in the carry buffer with two copies gets one map per copy, and the index expression
        picks the copy this launch reads.
        """
        s_row, s_k = operand.strides
        k_major = (s_k == 1 or depth == 1) and s_row % 8 == 0 and (s_row >= depth or rows == 1)
        base = self.plan.storage[operand.buffer]
        extras = [0]
        if base[0] == "carry":                      # lives in the carry buffer, which the kernel receives as one more input
            extras = [base[1]] if base[1] == base[2] else [base[1], base[2]]
            base = ("in", self.carry_input)
        indices = []
        for extra in extras:
            if k_major:
                spec = TensorMapSpec(base, extra + operand.offset * 2, depth, rows, max(s_row, 8) * 2, 64, box_rows)
            else:
                spec = TensorMapSpec(base, extra + operand.offset * 2, rows, depth, max(s_k, 8) * 2, 64, 64)
            self.maps.append(spec)
            indices.append(len(self.maps) - 1)
        index = str(indices[0]) if len(indices) == 1 else f"(tk_carry_phase ? {indices[1]} : {indices[0]})"
        return index, not k_major

    def gemm(self, unit: Unit, body: _Body, base: int, bg: str = "tk::NoBg") -> None:
        epi = self.functor(unit)
        m, n, k = unit.mnk
        a, b = unit.a, unit.b
        if unit.path == "tc2":
            ia, a_mn = self._tensor_map(a, m, k, 128)
            flipped = type(b)(b.buffer, b.dtype, b.round_to, b.offset, (b.strides[1], b.strides[0]))
            ib, b_mn = self._tensor_map(flipped, n, k, 128)
            fmt = 1 if a.dtype == "bfloat16" else 0
            body.emit(f"tk::gemm_tc2<{str(a_mn).lower()}, {str(b_mn).lower()}, {fmt}, {self.raster_group}, {epi}, {bg}>"
                      f"(c, P, &P.maps[{ia}], &P.maps[{ib}], {m}, {n}, {k}, {base}LL);")
        elif unit.path == "tc":
            ia, a_mn = self._tensor_map(a, m, k, 128)
            # B is [K, N]: its "rows" are N and strides are (stride along N, stride along K)
            flipped = type(b)(b.buffer, b.dtype, b.round_to, b.offset, (b.strides[1], b.strides[0]))
            ib, b_mn = self._tensor_map(flipped, n, k, unit.block_n)
            fmt = 1 if a.dtype == "bfloat16" else 0
            body.emit(f"tk::gemm_tc<{unit.block_n}, {str(a_mn).lower()}, {str(b_mn).lower()}, {fmt}, {epi}, {bg}>"
                      f"(c, P, &P.maps[{ia}], &P.maps[{ib}], {m}, {n}, {k}, {base}LL);")
        elif unit.path == "gemv":
            k_major = b.strides[0] == 1 and b.strides[1] != 1
            ld = b.strides[1] if k_major else b.strides[0]
            body.emit(f"tk::gemv<{CTYPE[a.dtype]}, {ROUND[a.round_to]}, {CTYPE[b.dtype]}, {ROUND[b.round_to]}, {str(k_major).lower()}, {unit.block_n or 64}, {epi}>(c, P, "
                      f"{self.pointer(a.buffer, a.dtype, True)} + {a.offset}LL, {a.strides[1]}LL, "
                      f"{self.pointer(b.buffer, b.dtype, True)} + {b.offset}LL, {ld}LL, {n}, {k}, {base}LL);")
        else:
            self.needs_simt = True
            depth = self.simt_depth or (32 if k <= 32 else 64 if k <= 64 else 128)
            body.emit(f"tk::gemm_simt<{depth}, {CTYPE[a.dtype]}, {ROUND[a.round_to]}, {CTYPE[b.dtype]}, {ROUND[b.round_to]}, {epi}>(c, P, reinterpret_cast<tk::SimtSmem*>(c.slots), "
                      f"{self.pointer(a.buffer, a.dtype, True)} + {a.offset}LL, {a.strides[0]}LL, {a.strides[1]}LL, "
                      f"{self.pointer(b.buffer, b.dtype, True)} + {b.offset}LL, {b.strides[0]}LL, {b.strides[1]}LL, {m}, {n}, {k}, {base}LL);")

    @staticmethod
    def _unravel(flat: str, dims: tuple[int, ...], prefix: str, body: _Body) -> list[str]:
        names = []
        dense = row_major(dims)
        for d, (extent, stride) in enumerate(zip(dims, dense)):
            name = f"{prefix}{d}"
            if extent == 1:
                body.emit(f"const int64_t {name} = 0;")
            elif d == 0:
                body.emit(f"const int64_t {name} = ({flat}) / {stride}LL;")
            else:
                body.emit(f"const int64_t {name} = (({flat}) / {stride}LL) % {extent}LL;")
            names.append(name)
        return names

    def _flat_ok(self, unit: Unit) -> bool:
        dense = row_major(unit.dims)
        live = [d for d, n in enumerate(unit.dims) if n > 1]
        found: list[Access] = []

        def walk(expr) -> None:
            if isinstance(expr, Load):
                found.append(expr.access)
            elif isinstance(expr, Apply):
                for arg in expr.args:
                    walk(arg)

        for expr in unit.exprs.values():
            walk(expr)
        return all(all(a.strides[d] == dense[d] for d in live) or not any(a.strides[d] for d in live) for a in found)

    def point_item(self, unit: Unit, body: _Body, tid: str) -> None:
        """Body of one item `it` of a flat pointwise unit for the thread slot `tid` (0..THREADS-1)."""
        total = prod(unit.dims)
        # collapse to one dimension, 8 consecutive elements per thread
        flat = Unit(unit.kind, unit.name, unit.index, (total,))
        flat.members, flat.stores = unit.members, unit.stores
        dense = row_major(unit.dims)
        live = [d for d, n in enumerate(unit.dims) if n > 1]

        def rebase(expr):
            if isinstance(expr, Load):
                a = expr.access
                unit_stride = 1 if live and all(a.strides[d] == dense[d] for d in live) else 0
                if not live:
                    unit_stride = 0
                return Load(Access(a.buffer, a.dtype, a.offset, (unit_stride,)))
            if isinstance(expr, Apply):
                return Apply(expr.op, tuple(rebase(arg) for arg in expr.args))
            return expr

        flat.exprs = {k: rebase(v) for k, v in unit.exprs.items()}
        unroll = point_unroll(total, len(unit.reads) + len(unit.stores))
        # Each thread owns `unroll` chunks of 8 consecutive elements, THREADS * 8 elements apart, so every
        # 128-bit access of a warp is contiguous; all loads are issued before the first store.
        envs = []
        for u in range(unroll):
            body.emit(f"const int64_t i{u} = (it * {unroll}LL + {u}LL) * {THREADS * 8}LL + ({tid}) * 8;")
            body.emit(f"const int n{u} = (int)tk::imin(8, tk::imax(0, {total}LL - i{u}));")
            env: dict = {}
            for expr in flat.exprs.values():
                self._preload(expr, body, env, "8", [f"i{u}"], f"n{u}")
            envs.append(env)
        for u in range(unroll):
            body.emit(f"if (n{u} > 0) {{")
            body.depth += 1
            self.dag(flat, body, envs[u], "8", [f"i{u}"], f"n{u}")
            body.depth -= 1
            body.emit("}")

    def point(self, unit: Unit, body: _Body, base: int) -> None:
        total = prod(unit.dims)
        if total == 0:
            return
        body.emit(f"// {unit.name}: pointwise over {list(unit.dims)}")
        if self._flat_ok(unit):
            body.emit(f"for (int64_t it = tk::first_item({base}LL); it < {unit.items}LL; it += gridDim.x) {{")
            body.depth += 1
            self.point_item(unit, body, "threadIdx.x")
            body.depth -= 1
            body.emit("}")
            return
        body.emit(f"for (int64_t it = tk::first_item({base}LL); it < {unit.items}LL; it += gridDim.x) {{")
        body.depth += 1
        body.emit(f"for (int64_t i = it * {THREADS * 8}LL + threadIdx.x; i < tk::imin((it + 1) * {THREADS * 8}LL, {total}LL); i += {THREADS}) {{")
        body.depth += 1
        coords = self._unravel("i", unit.dims, "x", body)
        self.dag(unit, body, {}, "1", coords, "1")
        body.depth -= 1
        body.emit("}")
        body.depth -= 1
        body.emit("}")

    def _finish_value(self, unit: Unit, body: _Body, acc: str, env: dict) -> None:
        op = unit.root
        size = unit.mean_count or prod(unit.reduced)
        value = acc if op.op == "sum" else (f"({acc} / {size}.0f)" if size else "NAN")
        root = body.temp("v")
        body.emit(f"float {root}[1] = {{{ROUND[op.output.dtype]}::rnd({value})}};")
        env["ref:" + op.output.buffer] = root

    def reduce(self, unit: Unit, body: _Body, base: int) -> None:
        outputs, size, parts = prod(unit.kept), prod(unit.reduced), unit.parts
        chunk = -(-(-(-size // parts)) // 4) * 4       # whole runs of 4 per part
        kept_rank = len(unit.kept)
        body.emit(f"// {unit.name}: {unit.root.op} {list(unit.kept)} <- {list(unit.reduced)} ({unit.strategy or 'finish'}, parts={parts})")
        scratch = None
        if unit.scratch:
            scratch = self.pointer(unit.scratch, "float32", unit.phase == "finish")
        if unit.phase == "finish":
            body.emit(f"for (int64_t it = tk::first_item({base}LL); it < {unit.items}LL; it += gridDim.x) {{")
            body.depth += 1
            body.emit(f"const int64_t o = it * {THREADS}LL + threadIdx.x;")
            body.emit(f"if (o < {outputs}LL) {{")
            body.depth += 1
            body.emit("float acc = 0.0f;")
            body.emit(f"_Pragma(\"unroll 8\") for (int p = 0; p < {parts}; ++p) acc += {scratch}[(int64_t)p * {outputs}LL + o];")
            env: dict = {}
            self._finish_value(unit, body, "acc", env)
            coords = self._unravel("o", unit.kept, "x", body)
            self.dag(unit, body, env, "1", coords, "1")
            body.depth -= 1
            body.emit("}")
            body.depth -= 1
            body.emit("}")
            return

        loads: list[Access] = []

        def gather(expr) -> None:
            if isinstance(expr, Load):
                loads.append(expr.access)
            elif isinstance(expr, Apply):
                for arg in expr.args:
                    gather(arg)

        gather(unit.source)
        last_kept = kept_rank - 1

        def accumulate(r_expr: str) -> None:
            names = self._unravel(r_expr, unit.reduced, "r", body)
            env2: dict = {}
            value = self.value(unit.source, body, env2, "1", kcoords + names, "1")
            body.emit(f"acc += {value}[0];")

        if unit.strategy == "thread":
            # Each thread owns 8 adjacent outputs when they are adjacent in memory (column sums of a
            # row-major matrix): one 128-bit load per row, several rows in flight.
            if unit.vector:
                groups = outputs // 8
                body.emit(f"for (int64_t it = tk::first_item({base}LL); it < {unit.items}LL; it += gridDim.x) {{")
                body.depth += 1
                body.emit(f"const int64_t o = ((it / {parts}) * {THREADS}LL + threadIdx.x) * 8;")
                body.emit(f"const int part = (int)(it % {parts});")
                body.emit(f"if (o < {outputs}LL) {{")
                body.depth += 1
                kcoords = self._unravel("o", unit.kept, "x", body)
                body.emit("float acc[8] = {};")
                body.emit(f"const int64_t r_end = tk::imin((int64_t)(part + 1) * {chunk}LL, {size}LL);")
                body.emit(f"_Pragma(\"unroll 8\") for (int64_t r = (int64_t)part * {chunk}LL; r < r_end; ++r) {{")
                body.depth += 1
                names = self._unravel("r", unit.reduced, "r", body)
                value = self.value(unit.source, body, {}, "8", kcoords + names, "8", vdim=last_kept)
                body.emit(f"_Pragma(\"unroll\") for (int j = 0; j < 8; ++j) acc[j] += {value}[j];")
                body.depth -= 1
                body.emit("}")
                if unit.phase == "partial":
                    body.emit(f"tk::st_row<8>({scratch} + ((int64_t)part * {outputs}LL + o), 8, acc);")
                else:
                    op, rsize = unit.root, unit.mean_count or prod(unit.reduced)
                    scale = "acc[j]" if op.op == "sum" else f"(acc[j] / {rsize}.0f)"
                    body.emit("float fin[8];")
                    body.emit(f"_Pragma(\"unroll\") for (int j = 0; j < 8; ++j) fin[j] = {ROUND[op.output.dtype]}::rnd({scale});")
                    env = {"ref:" + op.output.buffer: "fin"}
                    self.dag(unit, body, env, "8", kcoords, "8")
                body.depth -= 1
                body.emit("}")
                body.depth -= 1
                body.emit("}")
                return
            body.emit(f"for (int64_t it = tk::first_item({base}LL); it < {unit.items}LL; it += gridDim.x) {{")
            body.depth += 1
            body.emit(f"const int64_t o = (it / {parts}) * {THREADS}LL + threadIdx.x;")
            body.emit(f"const int part = (int)(it % {parts});")
            body.emit(f"if (o < {outputs}LL) {{")
            body.depth += 1
            kcoords = self._unravel("o", unit.kept, "x", body)
            body.emit("float acc = 0.0f;")
            body.emit(f"const int64_t r_end = tk::imin((int64_t)(part + 1) * {chunk}LL, {size}LL);")
            body.emit(f"_Pragma(\"unroll 8\") for (int64_t r = (int64_t)part * {chunk}LL; r < r_end; ++r) {{")
            body.depth += 1
            accumulate("r")
            body.depth -= 1
            body.emit("}")
            if unit.phase == "partial":
                body.emit(f"{scratch}[(int64_t)part * {outputs}LL + o] = acc;")
            else:
                env = {}
                self._finish_value(unit, body, "acc", env)
                self.dag(unit, body, env, "1", kcoords, "1")
            body.depth -= 1
            body.emit("}")
            body.depth -= 1
            body.emit("}")
            return
        # block strategy: one (output, part) per block iteration, all threads stride the reduced range;
        # runs of 4 consecutive reduced elements per thread when they are adjacent in memory
        vector = unit.reduced[-1] % 4 == 0 and chunk % 4 == 0 and loads and all(a.strides[-1] in (0, 1) for a in loads)
        body.emit(f"for (int64_t it = tk::first_item({base}LL); it < {unit.items}LL; it += gridDim.x) {{")
        body.depth += 1
        body.emit(f"const int64_t o = it / {parts};")
        body.emit(f"const int part = (int)(it % {parts});")
        kcoords = self._unravel("o", unit.kept, "x", body)
        body.emit("float acc = 0.0f;")
        body.emit(f"const int64_t r_end = tk::imin((int64_t)(part + 1) * {chunk}LL, {size}LL);")
        if vector:
            body.emit(f"_Pragma(\"unroll 8\") for (int64_t r = (int64_t)part * {chunk}LL + threadIdx.x * 4; r < r_end; r += {THREADS * 4}) {{")
            body.depth += 1
            names = self._unravel("r", unit.reduced, "r", body)
            value = self.value(unit.source, body, {}, "4", kcoords + names, "4")
            body.emit(f"acc += ({value}[0] + {value}[1]) + ({value}[2] + {value}[3]);")
            body.depth -= 1
            body.emit("}")
        else:
            body.emit(f"_Pragma(\"unroll 4\") for (int64_t r = (int64_t)part * {chunk}LL + threadIdx.x; r < r_end; r += {THREADS}) {{")
            body.depth += 1
            accumulate("r")
            body.depth -= 1
            body.emit("}")
        body.emit("acc = tk::block_sum(c, acc);")
        body.emit("if (threadIdx.x == 0) {")
        body.depth += 1
        if unit.phase == "partial":
            body.emit(f"{scratch}[(int64_t)part * {outputs}LL + o] = acc;")
        else:
            env = {}
            self._finish_value(unit, body, "acc", env)
            self.dag(unit, body, env, "1", kcoords, "1")
        body.depth -= 1
        body.emit("}")
        body.depth -= 1
        body.emit("}")

    # -- whole kernel ------------------------------------------------------------------
    def _exchange_call(self, unit: Unit, peers: str, suffix: str, context: str, tail: str) -> str:
        """The device call of an exchange unit: scatter-staged, or through the multicast mapping."""
        plan, op = self.plan, unit.root
        source, result = plan.storage[op.inputs[0].buffer], plan.storage[op.output.buffer]
        head = f"<{ROUND[op.output.dtype]}, {plan.world}>({context}, {peers}, "
        if plan.multicast:
            mc = f"P.in[{len(plan.program.inputs) + 1 + plan.world}]"
            return f"tk::exchange_mean_mc{suffix}{head}{mc}, {source[1]}ULL, {result[1]}ULL, {prod(unit.dims)}LL, {tail});"
        return f"tk::exchange_mean{suffix}{head}{source[1]}ULL, {source[2]}ULL, {result[1]}ULL, {prod(unit.dims)}LL, {tail});"

    def kernel(self, stage_stamps: bool) -> str:
        plan = self.plan
        body = _Body()
        body.depth = 1
        for stage in range(plan.stages):
            if stage:
                body.emit("tk::cluster_barrier(c);" if plan.cluster_blocks else "tk::grid_barrier(c);")
                if stage - 1 in plan.signal_barriers:
                    body.emit(f"if (blockIdx.x == 0 && threadIdx.x < {plan.world}) tk::dp_signal(c.dp, &P.in[{len(plan.program.inputs) + 1}], threadIdx.x, {stage - 1});")
                if stage_stamps:
                    body.emit(f"if (blockIdx.x == 0 && threadIdx.x == 0) P.stamps[{stage}] = tk::global_timer_ns();")
            if stage == 1 and plan.carry_pingpong:
                body.emit("if (blockIdx.x == 0 && threadIdx.x == 0) P.status[tk::kCarryPhaseWord] = tk_carry_phase ^ 1u;   // every block has read the word by now")
            body.emit(f"// ---- stage {stage} ----")
            base = 0
            members = [u for u in plan.units if u.stage == stage]
            ordered = sorted(members, key=lambda u: (u.kind != "gemm", u.path not in ("tc", "tc2"), u.kind == "exchange", u.index))
            bases = {}
            for unit in ordered:
                bases[id(unit)] = base
                base += unit.items
            peers = f"&P.in[{len(plan.program.inputs) + 1}]"
            # cross-rank ordering first: background work may start as soon as the stage does
            for barrier in sorted({u.wait_barrier for u in members if u.wait_barrier is not None}):
                body.emit(f"tk::dp_wait(c, c.dp, {plan.world}, {barrier});   // every rank has passed grid barrier {barrier}")
            # Memory-bound units (gradient exchange, flat pointwise streams such as the FP32 updates) of a kernel
            # with stream warps: warps 6..9 of every block work through them while warps 0..5 run the stage's
            # other units (the GEMM tiles above all); whoever finishes first helps with what is left.
            # Exchanges always go to the stream warps.  A pointwise stream goes there only while the stage's GEMM
            # tiles last long enough to cover it: pieces handed out 32 threads at a time move fewer bytes per second
            # than the plain 192-thread loop (measured 3.3 against 4.9 TB/s for an FP32 update), so a stream that
            # the tensor work cannot hide is run by the worker warps, after their tiles, while the stream warps
            # carry the stage's exchange.
            background = []
            if self.background:
                tensor_seconds = sum(2.0 * prod(u.mnk) for u in ordered if u.kind == "gemm" and u.path in ("tc", "tc2")) / TENSOR_RATE
                for unit in ordered:
                    if unit.carried:
                        continue
                    if unit.kind == "exchange":
                        background.append(unit)
                    elif unit.kind == "point" and prod(unit.dims) and self._flat_ok(unit):
                        seconds = sum(prod(plan.shapes[b]) * ELEMENT_BYTES[plan.dtypes[b]] for b in unit.reads | unit.writes) / STREAM_RATE
                        if seconds <= tensor_seconds or self.stream_everything:
                            tensor_seconds -= seconds
                            background.append(unit)
            bg = "tk::NoBg"
            if background:
                bg = f"Bg_{stage}"
                if len(background) > 8:
                    raise ValueError("trainkernel: more than 8 background units in one stage")
                runs, setup = [], []
                for k, unit in enumerate(background):
                    fn = _Body()
                    fn.depth = 1
                    if unit.kind == "exchange":
                        fn.emit(self._exchange_call(unit, peers, "_item", "c.dp", "it, tid"))
                    else:
                        self.point_item(unit, fn, "tid")
                    self.functors.append(f"// {unit.name} ({unit.kind}) of stage {stage}, one 32-thread slice of item `it`\n"
                                         f"static __device__ __noinline__ void bg_{stage}_{k}(const Params& P, tk::Ctx& c, int64_t it, int tid) {{\n{fn.text()}\n}}\n")
                    b0, n = bases[id(unit)], unit.items
                    slices = THREADS // 32                      # 32-thread slices of one item
                    per_item = slices // self.stream_piece      # pieces an item is cut into
                    setup.append(f"if (threadIdx.x == {k}) {{ shared_state.bg_count[{k}] = (int)tk::owned_items({b0}LL, {n}LL) * {per_item}; "
                                 f"shared_state.bg_first[{k}] = (int)tk::first_item({b0}LL); }}")
                    runs.append(f"        {{ const int n = c.sh->bg_count[{k}]; if (o < n) {{ const int64_t it = (int64_t)c.sh->bg_first[{k}] + (int64_t)(o / {per_item}) * gridDim.x; "
                                f"_Pragma(\"unroll 1\") for (int s = 0; s < {self.stream_piece}; ++s) bg_{stage}_{k}(P, c, it, ((o % {per_item}) * {self.stream_piece} + s) * 32 + lane); "
                                f"return; }} o -= n; }}")
                # a piece is one 32-thread slice of one of this block's items; the per-unit counts are worked out once per
                # stage, so that handing out a piece costs a shared-memory atomic and a few 32-bit operations
                self.functors.append(
                    f"struct Bg_{stage} {{\n    static constexpr bool kActive = true;\n"
                    f"    static __device__ __forceinline__ void run(const Params& P, tk::Ctx& c, int ordinal, int lane) {{\n        int o = ordinal;\n"
                    + "\n".join(runs) + "\n    }\n};\n")
                for line in setup:
                    body.emit(line)
                body.emit("__syncthreads();")
                total = " + ".join(f"shared_state.bg_count[{k}]" for k in range(len(background)))
                body.emit(f"if (threadIdx.x == 0) {{ shared_state.bg_next = shared_state.bg_back = shared_state.bg_taken = 0; shared_state.bg_total = {total}; }}")
                body.emit("__syncthreads();")
            foreground = [u for u in ordered if u not in background]
            if self.background and foreground:
                body.emit("if (c.warp < tk::kWorkerWarps) {   // stream warps go straight to the background pieces")
                body.depth += 1
            for unit in foreground:
                if unit.carried:
                    guard = "!carried && c.warp < tk::kWorkerWarps" if self.wide_epilogue else "!carried"
                    body.emit(f"if ({guard}) {{   // {unit.name}: skipped when the previous launch left this value behind")
                    body.depth += 1
                    self.point(unit, body, bases[id(unit)])
                    body.depth -= 1
                    body.emit("}")
                    continue
                workers_only = self.wide_epilogue and not (unit.kind == "gemm" and unit.path in ("tc", "tc2"))
                body.emit("if (c.warp < tk::kWorkerWarps) {   // the four extra epilogue warps have no part in this unit" if workers_only else "{")
                body.depth += 1
                if unit.kind == "exchange":
                    op = unit.root
                    source = op.inputs[0].buffer
                    body.emit(f"// {unit.name}: mean of {source} over {plan.world} rank(s)")
                    body.emit(self._exchange_call(unit, peers, "", "c", f"{bases[id(unit)]}LL, {unit.items}LL"))
                elif unit.kind == "gemm":
                    body.emit(f"// {unit.name}: {unit.root.op} {unit.mnk} via {unit.path}")
                    self.gemm(unit, body, bases[id(unit)])
                elif unit.kind == "reduce":
                    self.reduce(unit, body, bases[id(unit)])
                else:
                    self.point(unit, body, bases[id(unit)])
                body.depth -= 1
                body.emit("}")
            if self.background and foreground:
                body.depth -= 1
                body.emit("}")
            if background:
                body.emit(f"tk::bg_drain<{bg}>(c, P);   // the stream warps' whole stage; the other warps help once their units are done")
        exchanging = plan.symmetric_bytes > 0
        n_in = max(1, len(plan.program.inputs) + self.extra_inputs)
        n_out = max(1, len(plan.program.outputs))
        n_maps = max(1, len(self.maps))
        n_maps_used = len(self.maps)
        use_tc = "true" if plan.uses_tc else "false"
        widest = max((u.block_n for u in plan.units if u.kind == "gemm" and u.path == "tc"), default=256)
        ring = ([] if plan.two_cta else [f"#define TK_RING_BN {64 if widest <= 64 else 128 if widest <= 128 else 256}"])
        self.ring_bn = 64 if widest <= 64 else 128 if widest <= 128 else 256
        if self.wide_epilogue:
            ring = ring + ["#define TK_EPI_WARPS 8"]
            self.ring_bn = 128 if plan.two_cta else self.ring_bn   # a pair tile's slot holds 128 of the 256 B columns
        if plan.symmetric_bytes:
            ring = ring + [f"#define TK_EXCHANGE_CHUNKS {plan.exchange_chunks}"]
        header = ring + ([f"#define TK_TRACE_STAGE {int(self.trace_stage)}"] if self.trace_stage is not None else []) + [
            '#include "tk_gemm_2cta.cuh"' if plan.two_cta else '#include "tk_device.cuh"',
            "struct Params {",
            f"    CUtensorMap maps[{n_maps}];",
            f"    const void* in[{n_in}];",
            f"    void* out[{n_out}];",
            "    uint8_t* ws;",
            "    uint32_t* sync;",
            "    uint32_t* status;",
            "    uint64_t* stamps;",
            "    uint64_t timeout_ns;",
            "    uint32_t arrivals;",
            "    uint32_t flags;",
            "};",
            "",
        ] + (["__shared__ uint32_t tk_carry_phase;   // copy of the carried values this launch reads (the other one is written)", ""]
             if plan.carry_pingpong else [])
        entry = [
            f"extern \"C\" __global__ void __launch_bounds__({self.threads}, 1) tk_step(const __grid_constant__ Params P) {{",
            "    extern __shared__ uint8_t dyn_smem[];",
            "    __shared__ tk::SharedState shared_state;",
        ]
        if plan.uses_tc:
            entry.append("    __shared__ tk::EpiStage epi_stage;")
        if stage_stamps:
            entry.append("    const uint64_t tk_entered = tk::global_timer_ns();   // before the prologue (barrier set-up, tensor memory, map prefetch)")
        entry += [
            "    tk::Ctx c;",
            "    tk::ctx_init2(c, P.sync, P.status, P.timeout_ns, P.arrivals, &shared_state, dyn_smem);" if plan.two_cta else
            f"    tk::ctx_init(c, P.sync, P.status, P.timeout_ns, P.arrivals, &shared_state, dyn_smem, {use_tc});",
        ]
        entry.append("    c.flags = P.flags;")
        if stage_stamps:
            entry.append("    c.stamps = P.stamps;")
        if plan.uses_tc:
            entry.append("    c.epi = &epi_stage.t[0][0][0];")
        if n_maps_used:
            entry.append(f"    if (threadIdx.x < {n_maps_used}) tk::tma_prefetch_desc(&P.maps[threadIdx.x]);")
        # Everything above touched only shared memory, tensor memory and the parameter block.  From here on the
        # kernel reads what earlier work on the stream wrote: wait for it (a no-op unless launched early).
        entry.append("    tk::launch_dependents();")
        entry.append("    tk::dependency_wait();")
        if exchanging:
            entry.append(f"    tk::dp_init(c.dp, const_cast<void*>(P.in[{len(plan.program.inputs)}]));")
        if plan.carry_bytes:
            # read before the first stage boundary: the word is rewritten by whichever block finishes this launch first
            entry.append("    const bool carried = (P.flags & tk::kTrustCarried) != 0u && P.status[tk::kCarriedWord] == 1u && P.status[0] == 0u;")
        if plan.carry_pingpong:
            # which copy of the carried values this launch READS; block 0 flips the word after the first stage boundary
            entry.append("    if (threadIdx.x == 0) tk_carry_phase = P.status[tk::kCarryPhaseWord] & 1u;")
            entry.append("    __syncthreads();")
        if stage_stamps:
            entry.append("    if (blockIdx.x == 0 && threadIdx.x == 0) { P.stamps[0] = tk::global_timer_ns(); P.stamps[tk::kStampTrace + 6] = tk_entered; }")
        tail = []
        if plan.carry_bytes:
            tail.append("    if (blockIdx.x == 0 && threadIdx.x == 0) P.status[tk::kCarriedWord] = (c.aborted() || c.grid_aborted()) ? 0u : 1u;")
        if stage_stamps:
            tail.append(f"    __syncthreads();\n    if (blockIdx.x == 0 && threadIdx.x == 0) P.stamps[{plan.stages}] = tk::global_timer_ns();")
        if exchanging:
            tail.append("    if (blockIdx.x == 0 && threadIdx.x == 0) tk::dp_finish(c.dp);")
        tail += ["    tk::ctx_finish2(c);" if plan.two_cta else f"    tk::ctx_finish(c, {use_tc});"]
        if stage_stamps:
            # when the last block is done with its epilogue (tensor memory released): the end of the launch as the device sees it
            tail.append("    if (threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned long long*>(P.stamps + tk::kStampTrace + 7), static_cast<unsigned long long>(tk::global_timer_ns()));")
        tail += ["}", ""]
        return "\n".join(header + self.functors + entry + [body.text()] + tail)


def _check_names(program: Program) -> None:
    for spec in (*program.inputs, *(op.output for op in program.operations), *program.outputs):
        if spec.dtype not in CTYPE:
            raise ValueError(f"trainkernel: unsupported CUDA dtype {spec.dtype}")
        if not re.fullmatch(r"[A-Za-z_][A-Za-z_0-9]*", spec.buffer):
            raise ValueError("trainkernel: invalid buffer identifier")


def _check_broadcasts(program: Program) -> None:
    for op in program.operations:
        if op.op in ("mm", "addmm", "sum", "mean"):
            continue
        for value in op.inputs:
            if not isinstance(value, TensorSpec):
                continue
            if len(value.shape) > len(op.output.shape):
                raise ValueError("trainkernel: invalid broadcast rank")
            tail = op.output.shape[len(op.output.shape) - len(value.shape):] if value.shape else ()
            if any(a != 1 and a != b for a, b in zip(value.shape, tail)):
                raise ValueError("trainkernel: incompatible broadcast dimensions")


def plan_program(program: Program, *, inplace_outputs: dict[int, int] | None = None, fuse_pointwise: bool = True,
                 fuse_epilogues: bool = True, max_blocks: int | None = None, tensor_cores: bool = True,
                 block_n: int | None = None, two_cta: bool | None = None, world: int = 1,
                 background: bool = False, multicast: bool = False, cluster_barrier: bool | None = None,
                 carry_shadows: bool | str | None = None, wave_aware_tiles: bool = False,
                 exchange_chunks: int = 8, late_casts: bool = False) -> Plan:
    """Validate, canonicalise and plan `program` (no code is emitted)."""
    validate(program)
    from .passes import canonicalize_transposed_mm
    program = canonicalize_transposed_mm(program)
    validate(program)
    _check_names(program)
    _check_broadcasts(program)
    if max_blocks is not None and (type(max_blocks) is not int or max_blocks < 1):
        raise ValueError("trainkernel: max_blocks must be positive when provided")
    if block_n is not None and block_n not in (64, 128, 256):
        raise ValueError("trainkernel: block_n must be 64, 128 or 256")
    if type(world) is not int or not 1 <= world <= 8:
        raise ValueError("trainkernel: world must be between 1 and 8")
    mapping = dict(inplace_outputs or {})
    if any(type(i) is not int or type(j) is not int or not 0 <= i < len(program.outputs) or not 0 <= j < len(program.inputs)
           for i, j in mapping.items()):
        raise ValueError("trainkernel: invalid inplace output/input index")
    if len(set(mapping.values())) != len(mapping):
        raise ValueError("trainkernel: inplace outputs must target distinct inputs")
    produced = {op.output.buffer for op in program.operations}
    for slot, target in mapping.items():
        output, source = program.outputs[slot], program.inputs[target]
        if output.shape != source.shape or output.dtype != source.dtype or source.strides != row_major(source.shape):
            raise ValueError("trainkernel: inplace output must match a contiguous input shape and dtype")
        if output.buffer not in produced:
            raise ValueError("trainkernel: inplace outputs must be computed values, not input views")
    return Planner(program, inplace_outputs=mapping, fuse_pointwise=fuse_pointwise, fuse_epilogues=fuse_epilogues,
                   max_blocks=max_blocks, tensor_cores=tensor_cores, block_n=block_n, two_cta=two_cta, world=world,
                   background=background, multicast=multicast, cluster_barrier=cluster_barrier, carry=carry_shadows,
                   wave_aware_tiles=wave_aware_tiles, exchange_chunks=exchange_chunks, late_casts=late_casts).plan()


_IGNORED_REFERENCE_KNOBS = ("blocks_per_sm", "gemm_k_tile", "gemm_tile_n", "shared_skew", "split_k_gemv",
                            "threads_per_block", "inline_input_casts")


def generate(program: Program, *, fuse_pointwise: bool = True, fuse_epilogues: bool = True,
             max_blocks: int | None = None, inplace_outputs: dict[int, int] | None = None,
             tensor_cores: bool = True, block_n: int | None = None, stage_stamps: bool = False,
             two_cta: bool | None = None, raster_group: int | None = None, world: int = 1, background: bool = False,
             multicast: bool = False, cluster_barrier: bool | None = None, trace_stage: int | None = None,
             carry_shadows: bool | str | None = None, epilogue_lookahead: bool | None = None, stream_piece: int = 3,
             stream_everything: bool = False, wave_aware_tiles: bool = False, exchange_chunks: int = 8,
             wide_epilogue: bool | None = None, late_casts: bool = False, assume_aligned: bool = True,
             simt_depth: int | None = None, **reference_knobs) -> GeneratedKernel:
    """Generate the sm_100a kernel source and launch metadata for `program`.

    The reference's SM80/SM90 geometry knobs (`blocks_per_sm`, `gemm_k_tile`,
    `gemm_tile_n`, `shared_skew`, `split_k_gemv`, `threads_per_block`,
    `inline_input_casts`) have no meaning on this back end; they are accepted so
    existing call sites keep working, and ignored.  `hopper_wgmma=True` is rejected.

    `background=True` gives every block four more warps (320 threads instead of 192), the stream
    warps, which execute the flat pointwise and exchange units of each stage while the other six
    warps run the stage's GEMM tiles (and places weight-shadow casts next to the GEMM before their
    first use).  It is what lets a batch-sharded step overlap its gradient exchange and its
    HBM-bound FP32 updates with the backward GEMMs; single-GPU steps have nothing to overlap and
    leave it off.

    `cluster_barrier` (default: decided from the amount of work) runs the whole kernel as ONE
    thread-block cluster of at most 8 blocks whose stages end in the hardware cluster barrier instead
    of the barrier through global memory; `GeneratedKernel.barrier` says which one a kernel uses.

    `stage_stamps=True` makes block 0 record the global timer at every stage boundary and makes every
    grid barrier record when block 0 and when the last block arrived (`CompiledProgram.stage_stamps`,
    `CompiledProgram.barrier_stalls`); the stamp area has room for 55 stages.  `trace_stage=s` (with
    `stage_stamps=True`) also records six role-level timestamps of the first single-CTA tensor-core
    tile of stage `s` (`CompiledProgram.role_trace`).

    `carry_shadows` (default: decided by the planner, on for kernels of large GEMMs, where the casting
    stage costs a quarter of a millisecond of HBM traffic, off for small ones, whose weight-gradient
    stages are bound by their epilogue stores and lose more to the extra store than the skipped stage
    saves): a value that is a bare cast of in-place state and feeds tensor-core
    GEMMs (the BF16 copy of an FP32 master weight) is kept in a carry buffer between launches; the unit
    that commits the updated state also stores its cast there, and the casting unit of the next launch
    is skipped when the launch carries `TK_LAUNCH_TRUST_CARRIED` (`GeneratedKernel.carry_bytes` > 0
    means the kernel takes that buffer as its last input).  `True` / `"pingpong"` keeps two copies of
    every carried value (a launch reads one and writes the other; the schedule is unchanged),
    `"reorder"` keeps one and orders its rewrite behind its last reader, `False` casts in every
    launch.  A module with carried values must not be launched on two streams at once.

    `stream_piece`: how many 32-thread slices of a work item one background piece covers (a piece is what a
    stream warp takes from the stage's list at a time; larger pieces cost fewer shared-memory atomics).

    `wide_epilogue` (default: on for single-CTA tensor-core kernels, off for pair-tile kernels; never with
    stream warps): 320 threads per block, eight epilogue warps per accumulator tile instead of four (two per
    TMEM lane quarter, alternate 32-column chunks), one ring slot less.  Doubles the loads and stores a block
    keeps in flight while it drains an accumulator, which is what bounds the short-K GEMMs of small programs
    (8-14 % per step on the small configurations); the K loops of pair-tile kernels hide their epilogues already.

    `assume_aligned` (default on): the epilogue of a tensor-core GEMM whose N is a multiple of 8 reads and
    writes rows with 16-byte vector accesses only, without the element-wise fallback for ragged or unaligned
    runs, wherever extents, strides and offsets prove that a run is whole and aligned given 16-byte aligned
    base pointers; `GeneratedKernel.aligned_inputs` / `aligned_outputs` / `aligned_workspace` name the
    pointers the proof leans on, and `tk_module_launch` refuses a launch that passes one of them unaligned
    (compile with `assume_aligned=False` for tensors at odd offsets).  The fallback is a third of an
    epilogue's instructions; small programs, which fetch every stage's code cold in every launch, run
    2-11 % faster without it.

    `simt_depth`: K depth a SIMT GEMM stages in shared memory per step (default: 32, 64 or 128 by the
    product's K; the loads of a step are unrolled per staged position, so a shallow product should not carry
    the code of a deep one).

    `late_casts`: place a cast of a program input (a BF16 weight copy) in the stage before its first reader
    instead of the first stage when that stage has tensor-core GEMMs (no measurable difference; off).

    `epilogue_lookahead`: `True` (default with four epilogue warps): tensor-core epilogues that read at most two
    stored operands request the operands of the next 32-column chunk before they read the current chunk out of
    TMEM.  `"first"` (default with eight, where the 168-register ceiling of a 320-thread block makes the full form
    spill): only the first chunk's operands are requested early, before the warp waits for the accumulator.
    `False`: every chunk loads its operands when it starts.

    With `world > 1` the kernel takes `1 + world` extra inputs after the program's own: this rank's
    symmetric buffer, then every rank's mapping of it in rank order.  `multicast=True` adds one more,
    this rank's pointer to the NVSwitch multicast mapping of the buffer, and exchanges through
    `multimem.ld_reduce` / `multimem.st` instead of scattering contributions to their owners.
    """
    if reference_knobs.pop("hopper_wgmma", False):
        raise ValueError("trainkernel: hopper_wgmma is an SM90a option; this back end targets sm_100a")
    unknown = set(reference_knobs) - set(_IGNORED_REFERENCE_KNOBS)
    if unknown:
        raise TypeError(f"trainkernel: unknown option(s) {sorted(unknown)}")
    blocks_per_sm = reference_knobs.get("blocks_per_sm", 1)
    if type(blocks_per_sm) is not int or not 1 <= blocks_per_sm <= 8:
        raise ValueError("trainkernel: blocks_per_sm must be between 1 and 8")
    plan = plan_program(program, inplace_outputs=inplace_outputs, fuse_pointwise=fuse_pointwise,
                        fuse_epilogues=fuse_epilogues, max_blocks=max_blocks, tensor_cores=tensor_cores, block_n=block_n,
                        two_cta=two_cta, world=world, background=background, multicast=multicast,
                        cluster_barrier=cluster_barrier, carry_shadows=carry_shadows, wave_aware_tiles=wave_aware_tiles,
                        exchange_chunks=exchange_chunks, late_casts=late_casts)
    # Fixed-size tables the kernel indexes by stage or barrier number: the stamp area, and (with peers) the
    # 64 flag words per rank in the symmetric buffer's header, laid out from word 16.
    if stage_stamps and plan.stages > MAX_STAMPED_STAGES:
        raise ValueError(f"trainkernel: stage stamps cover at most {MAX_STAMPED_STAGES} stages; this program has {plan.stages}")
    if trace_stage is not None and (not stage_stamps or not 0 <= trace_stage < plan.stages):
        raise ValueError("trainkernel: trace_stage needs stage_stamps=True and a stage of this program")
    if plan.world > 1 or plan.symmetric_bytes:
        if plan.stages - 1 > FLAG_WORDS_PER_RANK:
            raise ValueError(f"trainkernel: a kernel that exchanges with peers can have at most {FLAG_WORDS_PER_RANK} grid barriers; this program has {plan.stages - 1}")
        if 4 * (16 + FLAG_WORDS_PER_RANK * plan.world) > SYM_HEADER:
            raise ValueError("trainkernel: the symmetric buffer's header has no room for this many ranks")
    emitter = _Emitter(plan)
    emitter.trace_stage = trace_stage
    emitter.assume_aligned = bool(assume_aligned)
    if simt_depth not in (None, 32, 64, 128):
        raise ValueError("trainkernel: simt_depth must be 32, 64 or 128")
    emitter.simt_depth = simt_depth
    if wide_epilogue is None:
        wide_epilogue = not plan.two_cta
    if wide_epilogue and plan.uses_tc and not plan.background:
        emitter.wide_epilogue = True
        emitter.threads = THREADS + 32 * 4
    if epilogue_lookahead not in (None, True, False, "first"):
        raise ValueError('trainkernel: epilogue_lookahead must be True, False or "first"')
    emitter.epilogue_lookahead = ("first" if emitter.wide_epilogue else True) if epilogue_lookahead is None else epilogue_lookahead
    if stream_piece not in (1, 2, 3, 6):
        raise ValueError("trainkernel: stream_piece must be 1, 2, 3 or 6")
    emitter.stream_piece = stream_piece
    emitter.stream_everything = bool(stream_everything)
    if raster_group is not None:
        if type(raster_group) is not int or not 1 <= raster_group <= 64:
            raise ValueError("trainkernel: raster_group must be between 1 and 64")
        emitter.raster_group = raster_group
    source = emitter.kernel(stage_stamps)
    extra_inputs = emitter.extra_inputs
    n_in, n_out = max(1, len(plan.program.inputs) + extra_inputs), max(1, len(plan.program.outputs))
    n_maps = max(1, len(emitter.maps))
    param_bytes = 128 * n_maps + 8 * (n_in + n_out) + 8 * 6
    per_stage: dict[int, int] = {}
    for unit in plan.units:
        per_stage[unit.stage] = per_stage.get(unit.stage, 0) + unit.items
    # IR operations that run as (part of) a unit; the re-created casts of carried values are not program operations
    materialized = sum((1 if u.root is not None and u.phase != "partial" else 0)
                       + sum(1 for member in u.members if not member.name.endswith("__next")) for u in plan.units)
    from .plan import SM_COUNT  # noqa: F401
    dyn = 0
    if emitter.needs_simt:
        dyn = 4 * (32 * 129 + 4 + 128 * 36) + 1024          # tk::SimtSmem + alignment slack
    if plan.uses_tc:
        dyn = 4 * (128 * 64 * 2 + 256 * 64 * 2) + 1024
        if emitter.wide_epilogue:                            # one ring slot less: the room goes to four more transposition buffers
            stages = (6 if plan.two_cta else {256: 4, 128: 6, 64: 8}[emitter.ring_bn]) - 1
            dyn = max(stages * (128 * 64 * 2 + emitter.ring_bn * 64 * 2) + 1024,
                      4 * (32 * 129 + 4 + 128 * 36) + 1024 if emitter.needs_simt else 0)
    return GeneratedKernel(
        source=source,
        workspace_elements=-(-plan.workspace_bytes // 4),
        materialized_operations=materialized,
        inlined_operations=len(plan.inlined),
        tensor_core_operations=plan.tensor_core_units,
        blocks_per_sm=1,
        max_work_blocks=max(per_stage.values(), default=1),
        grid_barriers=plan.stages - 1,
        direct_outputs=len(plan.native_outputs) + len(plan.direct_commits),
        direct_state_commits=len(plan.direct_commits),
        threads=emitter.threads,
        dynamic_smem=dyn,
        aligned_inputs=tuple(sorted(emitter.aligned_inputs)),
        aligned_outputs=tuple(sorted(emitter.aligned_outputs)),
        aligned_workspace=emitter.aligned_workspace,
        grid=plan.grid,
        tensor_maps=tuple(emitter.maps),
        input_count=len(plan.program.inputs) + extra_inputs,
        output_count=len(plan.program.outputs),
        stages=plan.stages,
        units=tuple((u.stage, u.kind + (":" + u.phase if u.phase else ""), u.name, u.path, u.items) for u in plan.units),
        staged_state_commits=len(plan.staged_commits),
        param_bytes=param_bytes,
        workspace_bytes=plan.workspace_bytes,
        cluster=2 if plan.two_cta else max(1, plan.cluster_blocks),
        barrier="cluster" if plan.cluster_blocks else "grid",
        world=plan.world,
        multicast=plan.multicast,
        symmetric_bytes=plan.symmetric_bytes,
        carry_bytes=plan.carry_bytes,
    )
