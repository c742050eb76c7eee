"""Shared helpers for the GPU parity tests (torch is used for device memory only)."""
import numpy as np

import oracle
from oracle import BF16, F32

RTOL = {F32: 1e-4, BF16: 2e-2}


def torch_mod():
    import torch
    return torch


def to_dev(a: np.ndarray, dtype: int):
    """numpy (float32 / uint16 bf16 bits / int32) → cuda tensor of the matching torch dtype."""
    torch = torch_mod()
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
    return torch.from_numpy(a).cuda()


def to_host(t) -> np.ndarray:
    torch = torch_mod()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def empty_dev(shape, dtype: int):
    torch = torch_mod()
    td = {F32: torch.float32, BF16: torch.bfloat16, oracle.I32: torch.int32}[dtype]
    return torch.empty(shape, dtype=td, device="cuda")


def rnd(rng, shape, dtype, scale=1.0):
    a = (rng.standard_normal(shape) * scale).astype(np.float32)
    return a if dtype == F32 else oracle.to_bf16(a)


def close(got: np.ndarray, want: np.ndarray, dtype: int, rtol=None):
    """|a-b| <= rtol*|b| + rtol*rms(b) elementwise; returns (ok, worst ratio, inf-norm rel err)."""
    g = oracle.as_float(got, dtype).astype(np.float64)
    w = oracle.as_float(want, dtype).astype(np.float64)
    rtol = RTOL[dtype] if rtol is None else rtol
    rms = float(np.sqrt(np.mean(w * w))) if w.size else 0.0
    bound = rtol * np.abs(w) + rtol * rms
    err = np.abs(g - w)
    worst = float((err / np.maximum(bound, 1e-30)).max()) if w.size else 0.0
    rel_inf = float(err.max() / max(np.abs(w).max(), 1e-30)) if w.size else 0.0
    return bool(np.all(err <= bound)) and bool(np.isfinite(g).all()), worst, rel_inf


def assert_close(got, want, dtype, rtol=None, what="", worst_cap=1.0):
    """``worst_cap`` > 1 relaxes the elementwise bound by that factor while still holding the
    norm-wise error ``max|a-b| / max|b|`` to the tolerance (used where outputs are averages over
    hundreds of terms, much smaller than the tensor's RMS, and one bf16 rounding of a term shows)."""
    ok, worst, rel_inf = close(got, want, dtype, rtol)
    tol = RTOL[dtype] if rtol is None else rtol
    ok = ok or (worst_cap > 1.0 and worst <= worst_cap and rel_inf <= tol and np.isfinite(
        oracle.as_float(got, dtype)).all())
    assert ok, f"{what}: worst err/bound {worst:.3g}, rel-inf {rel_inf:.3g}"
