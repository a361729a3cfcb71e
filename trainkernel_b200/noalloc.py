"""Python binding of `tk_module_launch_static_workspace` (libtrainkernel_noalloc.so).

For callers that cannot allocate device memory when they launch a step: the
kernel's workspace is a fixed 4 MiB array inside the library's device image
instead of a tensor the caller (or PyTorch) allocates.  See
`csrc/tk_noalloc.cu` for the contract: one shared array per device, overlapping
launches race, larger kernels are rejected, and the first call on a device does
a one-time address lookup that should precede any stream capture.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import torch

from . import runtime

LIBRARY_PATH = runtime.PACKAGE_DIR / "libtrainkernel_noalloc.so"
STATIC_WORKSPACE_BYTES = 4 << 20
_library: ctypes.CDLL | None = None


def build_library(force: bool = False) -> Path:
    """nvcc-compile `csrc/tk_noalloc.cu` for sm_100a into a shared library next to the runtime shim."""
    source = runtime.CSRC_DIR / "tk_noalloc.cu"
    runtime.build_library()
    if LIBRARY_PATH.exists() and LIBRARY_PATH.stat().st_mtime >= source.stat().st_mtime and not force:
        return LIBRARY_PATH
    cuda = runtime._cuda_home()
    if cuda is None:
        raise RuntimeError("trainkernel: CUDA toolkit with nvcc is required to build libtrainkernel_noalloc.so")
    command = [str(Path(cuda) / "bin" / "nvcc"), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O2", "-std=c++17",
               "-shared", "-Xcompiler", "-fPIC", "-I", str(runtime.INCLUDE_DIR), "-o", str(LIBRARY_PATH), str(source),
               "-L", str(runtime.PACKAGE_DIR), "-ltrainkernel_rt", "-Xlinker", "-rpath=$ORIGIN"]
    done = subprocess.run(command, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"trainkernel: building libtrainkernel_noalloc.so failed:\n{done.stderr}")
    return LIBRARY_PATH


def library() -> ctypes.CDLL:
    global _library
    if _library is None:
        runtime.library()                       # the shim must be resident first (same process-wide copy)
        lib = ctypes.CDLL(str(build_library()))
        p = ctypes.c_void_p
        lib.tk_module_launch_static_workspace.argtypes = [p, ctypes.c_int, ctypes.POINTER(p), ctypes.POINTER(p), ctypes.c_size_t,
                                                          ctypes.c_int, p, ctypes.c_char_p, ctypes.c_size_t]
        _library = lib
    return _library


def launch_static_workspace(runner: runtime.CompiledProgram, inputs, outputs) -> None:
    """Launch `runner`'s kernel on the current stream with the library's built-in workspace.

    `outputs` are caller-owned tensors (for in-place slots, the state tensors themselves).
    Raises when the kernel needs more than `STATIC_WORKSPACE_BYTES` of workspace.
    """
    module = runner.module
    inputs, outputs = tuple(inputs), tuple(outputs)
    # the same argument checks as every other launch path; none of them allocates
    runner._validate_inputs(inputs)
    runner._check_outputs(inputs, outputs)
    # buffers the compiled program owns (made when it was compiled, not now) complete the kernel's input list;
    # this entry point passes no launch flags, so values carried over from an earlier launch are recomputed
    ins = (ctypes.c_void_p * module.n_in)(*[t.data_ptr() for t in runner.launch_inputs(inputs)])
    outs = (ctypes.c_void_p * module.n_out)(*[t.data_ptr() for t in outputs])
    message = ctypes.create_string_buffer(512)
    stream = torch.cuda.current_stream(runner.device).cuda_stream
    index = runner.device.index if runner.device.index is not None else torch.cuda.current_device()
    code = library().tk_module_launch_static_workspace(module.handle, index, ins, outs, runner.generated.workspace_bytes,
                                                       module.grid, stream, message, len(message))
    if code:
        raise RuntimeError(message.value.decode() or f"trainkernel: static-workspace launch failed with code {code}")
    if runner.inplace_outputs:
        torch.autograd.graph.increment_version([inputs[i] for i in set(runner.inplace_outputs.values())])
