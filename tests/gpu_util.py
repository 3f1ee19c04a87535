"""Helpers for the GPU parity tests: move numpy data through the backend's transfer entries and
compare with a stated tolerance."""
from __future__ import annotations

import numpy as np
import torch

from conftest import graft

pkg = graft.load_package()
abi, runtime = pkg.abi, pkg.runtime
F16, BF16, F32, I32, U8 = abi.F16, abi.BF16, abi.F32, abi.I32, abi.U8

# Tolerances used across the GPU tests: one rounding of the storage dtype plus FP32
# reassociation noise. Integer, mask and copy work is compared bit-exact.
TOL = {F16: dict(atol=2e-3, rtol=4e-3), BF16: dict(atol=1.6e-2, rtol=1.6e-2), F32: dict(atol=2e-5, rtol=2e-5)}


def dev(ctx, a, dtype, arena=None):
    """Upload a numpy/torch array as a tensor of `dtype` (values are rounded to the storage grid)."""
    if isinstance(a, torch.Tensor):
        a = a.numpy()
    a = np.asarray(a)
    return ctx.from_numpy(arena or ctx.scratch, dtype, a)


def host(t) -> np.ndarray:
    return t.read_f32() if t.dtype in (F16, BF16, F32) else t.read()


def storage_name(dtype) -> str:
    return {F16: "f16", BF16: "bf16", F32: "f32"}[dtype]


def rnd_np(a: np.ndarray, dtype) -> np.ndarray:
    if dtype == F16:
        return a.astype(np.float16).astype(np.float32)
    if dtype == BF16:
        return runtime.f32_from_bf16_bits(runtime.bf16_bits_from_f32(a)).reshape(a.shape)
    return a.astype(np.float32)


def close(got, want, dtype, scale: float = 1.0, what: str = ""):
    tol = TOL[dtype]
    if isinstance(want, torch.Tensor):
        want = want.numpy()
    np.testing.assert_allclose(np.asarray(got, dtype=np.float32).reshape(np.shape(want)), want,
                               atol=tol["atol"] * scale, rtol=tol["rtol"], err_msg=what)
