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
