"""The allocation-free launch entry point gives the same results as the regular one.

`tk_module_launch_static_workspace` is for callers that are not allowed to allocate device
memory when they launch a step; it runs the same kernel with the library's built-in 4 MiB
workspace.  Here the tiny-MLP step is run twice in a row through that entry point (over the
C ABI, via ctypes) and twice through the regular entry point from the same starting state; every
loss, gradient and updated parameter of both calls must be bit-identical: it is the same kernel
on the same inputs, and the kernel is deterministic.  The file name keeps this test last in collection order.
"""
import ctypes

import pytest
import torch

import trainkernel_b200 as tk
from trainkernel_b200 import noalloc, workloads
from tests.helpers import rel_error

pytestmark = pytest.mark.gpu


def _fresh(runner, state):
    """Output tensors for one launch: state tensors for in-place slots, new tensors otherwise."""
    outputs = []
    for slot, spec in enumerate(runner.program.outputs):
        if slot in runner.inplace_outputs:
            outputs.append(state[runner.inplace_outputs[slot]])
        else:
            outputs.append(torch.empty(spec.shape, dtype=getattr(torch, spec.dtype), device=runner.device))
    return outputs


def test_static_workspace_launch_matches_regular_launch_twice():
    work = workloads.build("c2", seed=0, device="cuda")
    x0, t0 = work.batches[0]
    compiled = tk.compile_training(work.fn(), (work.state, x0, t0))
    runner = compiled.runner
    assert runner.generated.workspace_bytes <= noalloc.STATIC_WORKSPACE_BYTES
    regular_state = tuple(p.clone() for p in work.state)
    static_state = tuple(p.clone() for p in work.state)
    for call in range(2):
        x, t = work.batches[call % len(work.batches)]
        expected = runner(*regular_state, x, t)                      # regular entry point, torch-allocated workspace
        outputs = _fresh(runner, static_state)
        noalloc.launch_static_workspace(runner, (*static_state, x, t), outputs)
        torch.cuda.synchronize()
        runner.status()
        assert len(outputs) == len(expected)
        for index, (got, want) in enumerate(zip(outputs, expected)):
            assert bool(torch.isfinite(got.float()).all())
            assert torch.equal(got, want), f"call {call}, output {index}: relative error {rel_error(got, want):.3e}"
    for got, want in zip(static_state, regular_state):
        assert torch.equal(got, want)


def test_static_workspace_rejects_kernels_that_need_more():
    work = workloads.build("c2", seed=0, device="cuda")
    compiled = tk.compile_training(work.fn(), (work.state, *work.batches[0]))
    module = compiled.runner.module
    message = ctypes.create_string_buffer(512)
    ins = (ctypes.c_void_p * module.n_in)()
    outs = (ctypes.c_void_p * module.n_out)()
    code = noalloc.library().tk_module_launch_static_workspace(module.handle, 0, ins, outs, noalloc.STATIC_WORKSPACE_BYTES + 1,
                                                               module.grid, None, message, len(message))
    assert code == 100003
    assert b"built-in workspace holds" in message.value


def test_static_workspace_rejects_a_device_the_module_was_not_loaded_on_and_mismatched_tensors():
    work = workloads.build("c2", seed=0, device="cuda")
    compiled = tk.compile_training(work.fn(), (work.state, *work.batches[0]))
    runner = compiled.runner
    module = runner.module
    message = ctypes.create_string_buffer(512)
    ins = (ctypes.c_void_p * module.n_in)()
    outs = (ctypes.c_void_p * module.n_out)()
    wrong = (runner.device.index or 0) + 1
    code = noalloc.library().tk_module_launch_static_workspace(module.handle, wrong, ins, outs, runner.generated.workspace_bytes,
                                                               module.grid, None, message, len(message))
    assert code == 100001 and b"was loaded on device" in message.value
    # an understated workspace size is raised to what the module's plan needs, so it cannot slip past the limit
    x, t = work.batches[0]
    outputs = _fresh(runner, work.state)
    with pytest.raises(ValueError, match="shape, stride"):
        noalloc.launch_static_workspace(runner, (*work.state, x[:-1], t), outputs)
    with pytest.raises(ValueError, match="output buffer"):
        noalloc.launch_static_workspace(runner, (*work.state, x, t), [o.double() for o in outputs])
