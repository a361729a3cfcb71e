"""Comparison helpers shared by the parity tests."""
from __future__ import annotations

import torch
from torch.utils._pytree import tree_flatten

import trainkernel_b200 as tk
from oracle import interpreter
from tests import cases

# Relative error bound per compute dtype: FP32 steps 1e-5, 16-bit-compute steps 2e-2.
REL_TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-2}


def rel_error(actual: torch.Tensor, expected: torch.Tensor) -> float:
    """max|a - b| / max(max|b|, tiny), the definition every parity bound in this suite uses."""
    a, b = actual.detach().float().cpu(), expected.detach().float().cpu()
    if b.numel() == 0:
        return 0.0
    return float((a - b).abs().max()) / max(float(b.abs().max()), 1e-30)


def compile_case(name: str, device: str = "cuda"):
    """Compile a registered case on `device`; returns (compiled, device inputs, cpu inputs, program)."""
    fn, inputs, kind, options = cases.build(name, device)
    _, cpu_inputs, _, _ = cases.build(name, "cpu")
    compiled = getattr(tk, kind)(fn, inputs, **options)
    return compiled, inputs, cpu_inputs, compiled.program


def oracle_outputs(program, cpu_inputs):
    flat, _ = tree_flatten(cpu_inputs)
    return interpreter.run(program, flat)


def assert_outputs_close(actual, expected, tol: float, label: str = "") -> float:
    got, _ = tree_flatten(actual)
    assert len(got) == len(expected), f"{label}: output count {len(got)} != {len(expected)}"
    worst = 0.0
    for index, (a, b) in enumerate(zip(got, expected)):
        assert tuple(a.shape) == tuple(b.shape), f"{label}: output {index} shape {tuple(a.shape)} != {tuple(b.shape)}"
        assert a.dtype == b.dtype, f"{label}: output {index} dtype {a.dtype} != {b.dtype}"
        assert bool(torch.isfinite(a.float()).all()), f"{label}: output {index} is not finite"
        err = rel_error(a, b)
        worst = max(worst, err)
        assert err <= tol, f"{label}: output {index} relative error {err:.3e} exceeds {tol:.1e}"
    return worst


def l2_error(actual: torch.Tensor, expected: torch.Tensor) -> float:
    a, b = actual.detach().float().cpu(), expected.detach().float().cpu()
    return float((a - b).norm()) / max(float(b.norm()), 1e-30)


def assert_step_close(actual, expected_cpu, program, device_inputs, tol: float, label: str = "", max_fallbacks: int = 2) -> list[dict]:
    """Parity of one training step against the IR oracle.

    The bound is `tol` on max|a-b|/max|b| against the oracle evaluated on the host.  One
    effect can break that bound without any arithmetic being wrong: an activation whose
    pre-ReLU value is within an ulp of zero gets a different ReLU mask on the host than on
    the GPU (different FP32 summation order inside the matmul), which moves a whole column
    of the next weight gradient by one of its 1/batch terms.  When the host comparison
    fails for a 16-bit-compute step, the same oracle is therefore also evaluated on the
    device (same IR, same rounding points, cuBLAS summation order); the output passes if it
    is within `tol` of that evaluation and within `tol` of the host oracle in the L2 norm.

    Every output that needed this second comparison is printed and returned (index, host error,
    device-oracle error, L2 error, fraction of elements beyond the bound); at most
    `max_fallbacks` outputs of a step may need it, and in each of them the elements beyond
    the bound must be a small minority (a few flipped columns, not a wrong tensor).
    """
    got, _ = tree_flatten(actual)
    assert len(got) == len(expected_cpu), f"{label}: output count"
    on_device = None
    fallbacks: list[dict] = []
    for index, (a, b) in enumerate(zip(got, expected_cpu)):
        assert tuple(a.shape) == tuple(b.shape) and a.dtype == b.dtype, f"{label}: output {index} signature"
        assert bool(torch.isfinite(a.float()).all()), f"{label}: output {index} is not finite"
        err = rel_error(a, b)
        if err <= tol:
            continue
        assert tol > 1e-4, f"{label}: output {index} relative error {err:.3e} exceeds {tol:.1e}"
        if on_device is None:
            flat, _ = tree_flatten(device_inputs)
            on_device = interpreter.run(program, flat)
        l2 = l2_error(a, b)
        assert l2 <= tol, f"{label}: output {index} L2 relative error {l2:.3e}"
        err_device = rel_error(a, on_device[index])
        assert err_device <= tol, f"{label}: output {index} relative error {err:.3e} (host) / {err_device:.3e} (device oracle)"
        host = b.detach().float()
        beyond = float(((a.detach().float().cpu() - host).abs() > tol * float(host.abs().max())).float().mean())
        assert beyond <= 0.02, f"{label}: output {index}: {beyond:.2%} of the elements are beyond the bound, not a few flipped ReLU masks"
        record = {"output": index, "host_oracle": err, "device_oracle": err_device, "l2": l2, "fraction_beyond_bound": beyond}
        print(f"[parity] {label}: output {index} passed through the device-oracle comparison: {record}")
        fallbacks.append(record)
    assert len(fallbacks) <= max_fallbacks, f"{label}: {len(fallbacks)} outputs needed the device-oracle comparison: {fallbacks}"
    return fallbacks
