"""The C-ABI shim loads without a GPU and exports everything its header declares."""
import ctypes
import re
from pathlib import Path

import torch

from trainkernel_b200 import runtime

HEADER = Path(__file__).resolve().parents[1] / "include" / "trainkernel_rt.h"


def test_library_exports_every_declared_symbol():
    declared = set(re.findall(r"\b(tk_[a-z_]+)\s*\(", HEADER.read_text()))
    assert {"tk_module_load", "tk_module_launch", "tk_module_resource_usage", "tk_module_unload", "tk_last_error"} <= declared
    from trainkernel_b200 import noalloc
    shim = ctypes.CDLL(str(runtime.build_library()))
    extra = ctypes.CDLL(str(noalloc.build_library()))      # the allocation-free launch lives in its own library
    for name in sorted(declared):
        assert hasattr(shim, name) or hasattr(extra, name), name


def test_argument_errors_do_not_need_a_device():
    lib = runtime.library()
    handle = ctypes.c_void_p()
    code = lib.tk_module_load(None, 0, b"tk_step", 0, 192, 0, 1, 1, None, 0, ctypes.byref(handle))
    assert code == 100001 and b"invalid argument" in lib.tk_last_error()
    assert lib.tk_module_launch(None, None, None, None, 1, None) == 100001
    assert lib.tk_launch_count() >= 0


def test_missing_driver_is_reported_not_crashed():
    if torch.cuda.is_available():
        return
    lib = runtime.library()
    handle = ctypes.c_void_p()
    blob = ctypes.create_string_buffer(b"\x7fELF" + b"\0" * 60)
    code = lib.tk_module_load(blob, 64, b"tk_step", 0, 192, 0, 1, 1, None, 0, ctypes.byref(handle))
    assert code == 100002 and b"libcuda" in lib.tk_last_error()


def test_tensor_map_descriptor_layout_matches_the_header():
    assert ctypes.sizeof(runtime.TensorMapDesc) == 56
