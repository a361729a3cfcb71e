"""Build, load and launch generated kernels through the C-ABI runtime shim.

Keeps the reference's Python surface — `compile_program`, `CompiledProgram`
(`__call__`, `allocate`, `run_into`, `resource_usage`, `_validate_inputs`) and
`ExecutionBuffers` (reference: trainkernel/runtime.py:16-161) — with a
different mechanism underneath: the generated source is compiled by `nvcc`
straight to an sm_100a cubin (no PyTorch or pybind11 headers), cached on disk by
content hash, and loaded and launched by `libtrainkernel_rt.so` (CUDA driver
API, `include/trainkernel_rt.h`) on PyTorch's current stream.  PyTorch is used
for tensors and streams only.  There is no CPU or eager fallback: without the
shim, nvcc or an sm_100 device this module raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import tempfile
import threading
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch
from torch.utils._pytree import tree_flatten

from .codegen import GeneratedKernel, generate
from .ir import Program

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC_DIR = PACKAGE_DIR / "csrc"
INCLUDE_DIR = PACKAGE_DIR.parent / "include"
LIBRARY_PATH = PACKAGE_DIR / "libtrainkernel_rt.so"
CACHE_DIR = Path(os.environ.get("TRAINKERNEL_CACHE", PACKAGE_DIR / "_cache"))
NVCC_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "--fmad=false", "-lineinfo")

_BASE_KIND = {"in": 0, "out": 1, "ws": 2}
_lock = threading.Lock()
_library: ctypes.CDLL | None = None


class TensorMapDesc(ctypes.Structure):
    _fields_ = [
        ("base_kind", ctypes.c_int32), ("base_index", ctypes.c_int32), ("byte_offset", ctypes.c_uint64),
        ("inner", ctypes.c_uint64), ("outer", ctypes.c_uint64), ("outer_stride_bytes", ctypes.c_uint64),
        ("box_inner", ctypes.c_uint32), ("box_outer", ctypes.c_uint32), ("element_bytes", ctypes.c_uint32),
        ("reserved", ctypes.c_uint32),
    ]


def _cuda_home() -> str | None:
    for candidate in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if candidate and (Path(candidate) / "bin" / "nvcc").exists():
            return candidate
    found = shutil.which("nvcc")
    return str(Path(found).resolve().parents[1]) if found else None


def build_library(force: bool = False) -> Path:
    """Compile `csrc/tk_runtime.cpp` into `libtrainkernel_rt.so` next to this file."""
    source = CSRC_DIR / "tk_runtime.cpp"
    header = INCLUDE_DIR / "trainkernel_rt.h"
    fresh = LIBRARY_PATH.exists() and LIBRARY_PATH.stat().st_mtime >= max(source.stat().st_mtime, header.stat().st_mtime)
    if fresh and not force:
        return LIBRARY_PATH
    cuda = _cuda_home()
    if cuda is None:
        raise RuntimeError("trainkernel: CUDA toolkit headers are required to build the runtime shim")
    command = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-I", str(INCLUDE_DIR), "-I", str(Path(cuda) / "include"),
               "-o", str(LIBRARY_PATH), str(source), "-ldl", "-lpthread"]
    done = subprocess.run(command, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"trainkernel: building the runtime shim failed:\n{done.stderr}")
    return LIBRARY_PATH


def library() -> ctypes.CDLL:
    """The loaded shim with argument types declared; built on first use if missing."""
    global _library
    with _lock:
        if _library is not None:
            return _library
        path = build_library()
        lib = ctypes.CDLL(str(path))
        p, u64, u32, i32 = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int
        lib.tk_last_error.restype = ctypes.c_char_p
        lib.tk_launch_count.restype = u64
        lib.tk_module_load.argtypes = [p, ctypes.c_size_t, ctypes.c_char_p, i32, i32, ctypes.c_size_t, i32, i32,
                                       ctypes.POINTER(TensorMapDesc), i32, ctypes.POINTER(p)]
        lib.tk_module_launch.argtypes = [p, ctypes.POINTER(p), ctypes.POINTER(p), p, i32, p]
        lib.tk_module_launch_flags.argtypes = [p, ctypes.POINTER(p), ctypes.POINTER(p), p, i32, p, u32]
        lib.tk_module_invalidate_carried.argtypes = [p, p]
        lib.tk_module_device.argtypes = [p, ctypes.POINTER(i32)]
        lib.tk_module_launches.argtypes = [p, ctypes.POINTER(u64)]
        lib.tk_module_set_workspace_bytes.argtypes = [p, ctypes.c_size_t]
        lib.tk_module_require_alignment.argtypes = [p, ctypes.c_char_p, i32, ctypes.c_char_p, i32, i32]
        lib.tk_module_workspace_bytes.argtypes = [p, ctypes.POINTER(ctypes.c_size_t)]
        lib.tk_module_resource_usage.argtypes = [p, ctypes.POINTER(ctypes.c_int64)]
        lib.tk_module_max_coresident_blocks.argtypes = [p, ctypes.POINTER(i32)]
        lib.tk_module_status.argtypes = [p, p, ctypes.POINTER(u32)]
        lib.tk_module_reset.argtypes = [p]
        lib.tk_module_set_timeout.argtypes = [p, u64]
        lib.tk_module_set_expected_arrivals.argtypes = [p, u32]
        lib.tk_module_stage_stamps.argtypes = [p, p, ctypes.POINTER(u64), i32]
        lib.tk_module_set_cluster.argtypes = [p, i32]
        lib.tk_module_set_cooperative.argtypes = [p, i32]
        lib.tk_module_set_early_launch.argtypes = [p, i32]
        lib.tk_module_unload.argtypes = [p]
        lib.tk_module_unload.restype = None
        _library = lib
        return lib


def _raise(code: int) -> None:
    message = library().tk_last_error().decode() or f"trainkernel: runtime shim error {code}"
    raise RuntimeError(message)


def cubin_path(source: str) -> Path:
    """Where the cubin of `source` lives in the cache: keyed by the source, both device headers and the flags."""
    header = (CSRC_DIR / "tk_device.cuh").read_bytes() + (CSRC_DIR / "tk_gemm_2cta.cuh").read_bytes()
    digest = hashlib.sha256(source.encode() + b"\0" + header + b"\0" + " ".join(NVCC_FLAGS).encode()).hexdigest()[:32]
    return CACHE_DIR / f"{digest}.cubin"


def build_cubin(source: str, *, verbose: bool = False) -> bytes:
    """nvcc-compile generated source to an sm_100a cubin; cached by content hash."""
    cached = cubin_path(source)
    if cached.exists():
        return cached.read_bytes()
    cuda = _cuda_home()
    if cuda is None:
        raise RuntimeError("trainkernel: CUDA toolkit with nvcc is required to compile generated kernels")
    CACHE_DIR.mkdir(parents=True, exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="trainkernel_") as work:
        unit = Path(work) / "kernel.cu"
        unit.write_text(source)
        target = Path(work) / "kernel.cubin"
        command = [str(Path(cuda) / "bin" / "nvcc"), *NVCC_FLAGS, "-I", str(CSRC_DIR), "-cubin", "-o", str(target), str(unit)]
        if verbose:
            command.insert(1, "-Xptxas=-v")
        done = subprocess.run(command, capture_output=True, text=True)
        if verbose:
            print(done.stderr)
        if done.returncode != 0:
            raise RuntimeError(f"trainkernel: nvcc failed on the generated kernel:\n{done.stderr[-4000:]}")
        data = target.read_bytes()
    scratch = cached.with_suffix(f".tmp{os.getpid()}")
    scratch.write_bytes(data)
    os.replace(scratch, cached)
    return data


@dataclass
class ExecutionBuffers:
    """Caller-owned output and workspace storage for one launch.

    Reusing the same buffers for a second launch is only valid when the caller
    orders it after the first on the stream.
    """

    outputs: tuple[torch.Tensor, ...]
    workspace: torch.Tensor


class _Module:
    """Owner of one `tk_module*`."""

    def __init__(self, generated: GeneratedKernel, cubin: bytes, device: torch.device):
        lib = library()
        maps = (TensorMapDesc * max(1, len(generated.tensor_maps)))()
        for i, spec in enumerate(generated.tensor_maps):
            kind, where = spec.base
            maps[i] = TensorMapDesc(_BASE_KIND[kind], 0 if kind == "ws" else where,
                                    spec.byte_offset + (where if kind == "ws" else 0), spec.inner, spec.outer,
                                    spec.outer_stride_bytes, spec.box_inner, spec.box_outer, 2, 0)
        handle = ctypes.c_void_p()
        self._cubin = ctypes.create_string_buffer(cubin, len(cubin))
        index = device.index if device.index is not None else torch.cuda.current_device()
        code = lib.tk_module_load(self._cubin, len(cubin), generated.entry.encode(), index, generated.threads,
                                  generated.dynamic_smem, generated.input_count, generated.output_count,
                                  maps, len(generated.tensor_maps), ctypes.byref(handle))
        if code:
            _raise(code)
        self.handle = handle
        self.lib = lib
        lib.tk_module_set_workspace_bytes(handle, generated.workspace_bytes)
        if generated.aligned_inputs or generated.aligned_outputs or generated.aligned_workspace:
            wanted_in = bytes(int(i in generated.aligned_inputs) for i in range(generated.input_count))
            wanted_out = bytes(int(i in generated.aligned_outputs) for i in range(generated.output_count))
            code = lib.tk_module_require_alignment(handle, wanted_in, len(wanted_in), wanted_out, len(wanted_out), int(generated.aligned_workspace))
            if code:
                _raise(code)
        if generated.cluster > 1:
            code = lib.tk_module_set_cluster(handle, generated.cluster)
            if code:
                _raise(code)
        if generated.barrier == "cluster":
            lib.tk_module_set_cooperative(handle, 0)       # one cluster: co-scheduled by construction
        limit = ctypes.c_int()
        if lib.tk_module_max_coresident_blocks(handle, ctypes.byref(limit)):
            _raise(1)
        self.grid = max(1, min(generated.grid, limit.value))
        if generated.cluster > 1:
            self.grid -= self.grid % generated.cluster
        if generated.barrier == "cluster" and self.grid != generated.cluster:
            raise RuntimeError(f"trainkernel: a kernel synchronised by the cluster barrier must run as one cluster of "
                               f"{generated.cluster} blocks; the device admits {limit.value}")
        self.n_in = max(1, generated.input_count)
        self.n_out = max(1, generated.output_count)

    def launch(self, inputs, outputs, workspace: torch.Tensor, stream: int, flags: int = 0) -> None:
        ins = (ctypes.c_void_p * self.n_in)(*[t.data_ptr() for t in inputs])
        outs = (ctypes.c_void_p * self.n_out)(*[t.data_ptr() for t in outputs])
        code = self.lib.tk_module_launch_flags(self.handle, ins, outs, workspace.data_ptr(), self.grid, stream, flags)
        if code:
            _raise(code)

    def launches(self) -> int:
        count = ctypes.c_uint64()
        self.lib.tk_module_launches(self.handle, ctypes.byref(count))
        return int(count.value)

    def __del__(self):
        handle, self.handle = getattr(self, "handle", None), None
        if handle:
            try:
                self.lib.tk_module_unload(handle)
            except Exception:
                pass


TRUST_CARRIED = 1          # TK_LAUNCH_TRUST_CARRIED


class CarriedState:
    """Host-side bookkeeping for values a kernel carries from one launch to the next.

    A kernel with `GeneratedKernel.carry_bytes > 0` keeps the BF16 copies of its FP32 master weights
    in a buffer owned by this object and re-creates them while it commits the updated masters, so
    the next launch may skip casting them again — but only if nobody changed the state tensors in
    between.  PyTorch counts in-place modifications per tensor (`Tensor._version`): a launch is
    told to trust the carried values exactly when it gets the same state tensors (same addresses)
    whose version counters still have the values this object recorded after the previous launch.
    A write the counters cannot see (a raw pointer handed to another library) needs `invalidate()`.
    Under stream capture the runtime shim additionally ignores the flag for the first launch of
    every capture, so a replayed graph always starts from the state it finds.
    """

    def __init__(self, nbytes: int, device: torch.device, module: Any = None) -> None:
        self.buffer = torch.empty(max(1, nbytes), dtype=torch.uint8, device=device)
        self.module = module
        self.seen: tuple | None = None

    def _snapshot(self, targets) -> tuple:
        # the module's own launch count is part of it: a launch issued by anyone else rewrote the buffer
        count = self.module.launches() if self.module is not None and hasattr(self.module, "launches") else 0
        return (count, *((t.data_ptr(), t._version) for t in targets))

    def flags(self, targets) -> int:
        return TRUST_CARRIED if self.seen is not None and self.seen == self._snapshot(targets) else 0

    def launched(self, targets) -> None:
        """Call after the launch has bumped the targets' version counters."""
        self.seen = self._snapshot(targets)

    def invalidate(self) -> None:
        self.seen = None


class CompiledProgram:
    """One specialised kernel plus the argument checks that guard its launch.

    Every call allocates fresh outputs and workspace unless the caller passes
    its own `ExecutionBuffers`.  Results carry no autograd history; gradients
    come from differentiation inside the compiled function.
    """

    def __init__(self, program: Program, generated: GeneratedKernel, module: Any, device: torch.device,
                 inplace_outputs: dict[int, int] | None = None):
        self.program = program
        self.generated = generated
        self.source = generated.source
        self.module = module
        self.device = device
        self.inplace_outputs = dict(inplace_outputs or {})
        # what every call compares its arguments with, looked up once
        self._input_meta = [(spec.shape, spec.strides, getattr(torch, spec.dtype)) for spec in program.inputs]
        self._output_meta = [(spec.shape, getattr(torch, spec.dtype)) for spec in program.outputs]
        self._targets = sorted(set(self.inplace_outputs.values()))
        self.carried = CarriedState(generated.carry_bytes, device, module) if getattr(generated, "carry_bytes", 0) else None

    def invalidate_carried(self) -> None:
        """Make the next launch recompute what the previous one left behind (the BF16 weight copies): for
        callers that overwrite the state through something PyTorch's version counters do not see."""
        if self.carried is not None:
            self.carried.invalidate()

    def _launch(self, inputs: tuple[torch.Tensor, ...], outputs, workspace: torch.Tensor) -> None:
        stream = torch.cuda.current_stream(self.device).cuda_stream
        targets = [inputs[i] for i in self._targets]
        if self.carried is not None:
            self.module.launch((*inputs, self.carried.buffer), outputs, workspace, stream, self.carried.flags(targets))
        else:
            self.module.launch(inputs, outputs, workspace, stream)
        if targets:
            torch.autograd.graph.increment_version(targets)
        if self.carried is not None:
            self.carried.launched(targets)

    def launch_inputs(self, inputs: tuple[torch.Tensor, ...]) -> tuple:
        """The kernel's full input list for `inputs`: the program's inputs plus the buffers this object owns."""
        return (*inputs, self.carried.buffer) if self.carried is not None else tuple(inputs)

    # -- introspection -------------------------------------------------------------
    def resource_usage(self) -> dict[str, int]:
        """Compiler-reported resources of the kernel (no hardware counters involved)."""
        values = (ctypes.c_int64 * 4)()
        code = self.module.lib.tk_module_resource_usage(self.module.handle, values)
        if code:
            _raise(code)
        names = ("registers_per_thread", "local_bytes_per_thread", "shared_bytes_per_block", "resident_blocks_per_sm")
        return dict(zip(names, (int(v) for v in values)))

    def status(self) -> tuple[int, int, int, int]:
        """Synchronise the current stream and return the kernel's status words; raises on a timed-out wait."""
        words = (ctypes.c_uint32 * 4)()
        stream = torch.cuda.current_stream(self.device).cuda_stream
        code = self.module.lib.tk_module_status(self.module.handle, stream, words)
        if code:
            _raise(code)
        return tuple(int(w) for w in words)

    def _stamps(self, count: int) -> list[int]:
        stamps = (ctypes.c_uint64 * count)()
        stream = torch.cuda.current_stream(self.device).cuda_stream
        code = self.module.lib.tk_module_stage_stamps(self.module.handle, stream, stamps, count)
        if code:
            _raise(code)
        return [int(s) for s in stamps]

    def stage_stamps(self, count: int | None = None) -> list[int]:
        """Per-stage %globaltimer values of the last launch (kernel generated with `stage_stamps=True`)."""
        return self._stamps(self.generated.stages + 1 if count is None else count)

    def barrier_stalls(self) -> list[dict]:
        """Per grid barrier of the last launch (kernel generated with `stage_stamps=True`), nanoseconds:
        `block0_wait` from block 0's arrival to its release, `skew` from block 0's arrival to the last
        block's arrival (negative when block 0 was last), `release` from the last arrival to the release,
        and `peer_wait`, what block 0 then spent waiting for other ranks' flags before the next stage."""
        words = self._stamps(256)
        records = []
        for barrier in range(self.generated.grid_barriers if self.generated.barrier == "grid" else 0):
            arrive, last, release = words[64 + barrier], words[128 + barrier], words[barrier + 1]
            records.append({"barrier": barrier, "block0_wait": release - arrive, "skew": last - arrive,
                            "release": release - last, "peer_wait": words[192 + barrier + 1] if self.generated.world > 1 else 0})
        return records

    def launch_span(self) -> dict:
        """Where the last launch spent its time outside the stages (kernel generated with `stage_stamps=True`),
        nanoseconds: `prologue` from block 0's first instruction to the start of stage 0 (barrier set-up, tensor
        memory allocation, tensor-map prefetch), `stages` from there to block 0's end of the last stage, `tail`
        from there until the last block has released its tensor memory, `total` first instruction to that point."""
        words = self._stamps(256)
        entered, first, last, left = words[254], words[0], words[self.generated.stages], words[255]
        return {"prologue": first - entered, "stages": last - first, "tail": left - last, "total": left - entered}

    def role_trace(self) -> list[int]:
        """The six role-level %globaltimer values of the traced tile (kernel generated with `trace_stage=`)."""
        return self._stamps(256)[248:254]

    # -- argument checks -------------------------------------------------------------
    def _validate_inputs(self, inputs: tuple[torch.Tensor, ...]) -> None:
        expected = self._input_meta
        if len(inputs) != len(expected):
            raise ValueError(f"trainkernel: expected {len(expected)} inputs, got {len(inputs)}")
        for position, (tensor, (shape, strides, dtype)) in enumerate(zip(inputs, expected)):
            if not isinstance(tensor, torch.Tensor):
                raise TypeError(f"trainkernel: input {position} must be a tensor")
            if tensor.is_neg() or tensor.is_conj():
                raise ValueError("trainkernel: resolve lazy negative or conjugate input views before execution")
            same = (tensor.dtype == dtype and tensor.shape == shape and tensor.stride() == strides
                    and tensor.device == self.device)
            if not same:
                raise ValueError(f"trainkernel: input {position} does not match compiled device, shape, stride, or dtype")
        for target in self.inplace_outputs.values():
            if inputs[target].requires_grad:
                raise ValueError("trainkernel: inplace targets must be detached from autograd")

    def allocate(self, *inputs: torch.Tensor) -> ExecutionBuffers:
        if self.inplace_outputs:
            self._validate_inputs(inputs)
        return self._fresh_buffers(inputs)

    def _fresh_buffers(self, inputs: tuple[torch.Tensor, ...]) -> ExecutionBuffers:
        outputs = []
        for slot, (shape, dtype) in enumerate(self._output_meta):
            if slot in self.inplace_outputs:
                outputs.append(inputs[self.inplace_outputs[slot]])
            else:
                outputs.append(torch.empty(shape, dtype=dtype, device=self.device))
        workspace = torch.empty(self.generated.workspace_elements, dtype=torch.float32, device=self.device)
        return ExecutionBuffers(tuple(outputs), workspace)

    def _check_buffers(self, inputs: tuple[torch.Tensor, ...], buffers: ExecutionBuffers) -> None:
        outputs, workspace = buffers.outputs, buffers.workspace
        if (workspace.device != self.device or workspace.dtype != torch.float32 or not workspace.is_contiguous()
                or workspace.numel() < self.generated.workspace_elements):
            raise ValueError("trainkernel: workspace does not match compiled requirements")
        self._check_outputs(inputs, outputs, workspace)

    def _check_outputs(self, inputs: tuple[torch.Tensor, ...], outputs: tuple[torch.Tensor, ...],
                       workspace: torch.Tensor | None = None) -> None:
        """Output count, shape, dtype and layout; in-place slots bound to their inputs; nothing written
        shares storage with anything else that is read or written.  Allocates nothing."""
        if len(outputs) != len(self.program.outputs):
            raise ValueError("trainkernel: incorrect output buffer count")
        # Storage-level disjointness: conservative, but a write can then never clobber something still to be read.
        written: list[int] = []
        shared_with_inputs: set[int] = set()
        for slot, (tensor, spec) in enumerate(zip(outputs, self.program.outputs)):
            fits = (tensor.device == self.device and tensor.dtype == getattr(torch, spec.dtype)
                    and tuple(tensor.shape) == spec.shape and tensor.is_contiguous())
            if not fits:
                raise ValueError("trainkernel: output buffer does not match compiled requirements")
            if tensor.numel():
                written.append(tensor.untyped_storage().data_ptr())
            if slot not in self.inplace_outputs:
                continue
            index = self.inplace_outputs[slot]
            target = inputs[index]
            if tensor.data_ptr() != target.data_ptr() or tuple(tensor.stride()) != tuple(target.stride()):
                raise ValueError("trainkernel: inplace output must bind its declared input")
            if target.numel():
                storage = target.untyped_storage().data_ptr()
                for other, value in enumerate(inputs):
                    if other != index and value.numel() and value.untyped_storage().data_ptr() == storage:
                        raise ValueError("trainkernel: inplace target must not alias another input")
                shared_with_inputs.add(storage)
        if workspace is not None and workspace.numel():
            written.append(workspace.untyped_storage().data_ptr())
        read = {tensor.untyped_storage().data_ptr() for tensor in inputs if tensor.numel()}
        if len(set(written)) != len(written) or (read & set(written)) - shared_with_inputs:
            raise ValueError("trainkernel: execution buffers must not alias inputs or each other")

    # -- execution -------------------------------------------------------------------
    def run_into(self, *inputs: torch.Tensor, buffers: ExecutionBuffers) -> tuple[torch.Tensor, ...]:
        self._validate_inputs(inputs)
        self._check_buffers(inputs, buffers)
        self._launch(inputs, buffers.outputs, buffers.workspace)
        return buffers.outputs

    def __call__(self, *inputs: torch.Tensor) -> tuple[torch.Tensor, ...]:
        # Buffers made here are new allocations (or the in-place targets themselves), so of the buffer checks
        # only one can fail: an in-place target that shares storage with another input.
        self._validate_inputs(inputs)
        for index in self.inplace_outputs.values():
            target = inputs[index]
            if target.numel():
                storage = target.untyped_storage().data_ptr()
                for other, value in enumerate(inputs):
                    if other != index and value.numel() and value.untyped_storage().data_ptr() == storage:
                        raise ValueError("trainkernel: inplace target must not alias another input")
        buffers = self._fresh_buffers(inputs)
        self._launch(inputs, buffers.outputs, buffers.workspace)
        return buffers.outputs


def compile_program(program: Program, example_inputs: tuple[Any, ...] | list[Any], *,
                    inplace_outputs: dict[int, int] | None = None, verbose: bool = False,
                    **options: Any) -> CompiledProgram:
    """Generate, build and load the kernel for `program` on the inputs' device (sm_100 required)."""
    flat, _ = tree_flatten(example_inputs)
    if not flat or any(not isinstance(x, torch.Tensor) for x in flat):
        raise TypeError("trainkernel: nonempty tensor inputs required")
    if len(flat) != len(program.inputs):
        raise ValueError("trainkernel: input count differs from the program signature")
    if not torch.cuda.is_available() or any(x.device.type != "cuda" for x in flat):
        raise RuntimeError("trainkernel: CUDA sm_100a GPU required; CPU IR inspection is available through capture()")
    device = flat[0].device
    if any(x.device != device for x in flat):
        raise ValueError("trainkernel: all inputs must use the same CUDA device")
    capability = torch.cuda.get_device_capability(device)
    if capability[0] != 10:
        raise RuntimeError(f"trainkernel: an sm_100 (B200-class) GPU is required, found compute capability {capability[0]}.{capability[1]}")
    if "assume_aligned" not in options and any(x.data_ptr() % 16 for x in flat):
        options["assume_aligned"] = False     # example tensors at odd offsets: keep the element-wise fallbacks
    generated = generate(program, inplace_outputs=inplace_outputs, **options)
    if any(flat[i].requires_grad for i in (inplace_outputs or {}).values()):
        raise ValueError("trainkernel: inplace targets must be detached from autograd")
    cubin = build_cubin(generated.source, verbose=verbose)
    with torch.cuda.device(device):
        torch.cuda.current_stream(device)     # make sure the primary context exists before the shim retains it
        try:
            module = _Module(generated, cubin, device)
        except RuntimeError:
            # A device partition too small to hold the kernel's one cluster: the same program with the
            # barrier through global memory runs anywhere.  An explicit request for the cluster form stands.
            if generated.barrier != "cluster" or generated.cluster == 1 or options.get("cluster_barrier"):
                raise
            generated = generate(program, inplace_outputs=inplace_outputs, **{**options, "cluster_barrier": False})
            module = _Module(generated, build_cubin(generated.source, verbose=verbose), device)
    runner = CompiledProgram(program, generated, module, device, inplace_outputs)
    runner._validate_inputs(tuple(flat))
    return runner
