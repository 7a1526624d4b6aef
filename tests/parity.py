"""Comparison rules used by the parity tests, taken from the reference's own tests."""
import numpy as np

import h3_oracle as o


def assert_bf16_ulp(got, want, name="", ulps=1):
    """Elementwise / row ops: at most one BF16 ulp (tests/test_cuda_dit.c:57-71)."""
    g, w = o.from_bf16(got).astype(np.float64), o.from_bf16(want).astype(np.float64)
    err = np.abs(g - w)
    ulp = np.maximum(np.abs(g), np.abs(w)) * 2.0 ** -8 * ulps
    bad = (got != want) & ~(err <= ulp + 1e-30)
    assert not bad.any(), f"{name}: {int(bad.sum())} of {bad.size} beyond {ulps} ulp, max err {err.max():.3g}"


def assert_gemm_close(got, want, name=""):
    """GEMM-routed ops and flash attention: 1e-3 + 1e-2*|ref|
    (tests/test_cuda_dit.c:73-91, tests/test_cuda_attention.c:112-114)."""
    g, w = o.from_bf16(got).astype(np.float64), o.from_bf16(want).astype(np.float64)
    err = np.abs(g - w)
    bad = ~(err <= 1e-3 + 1e-2 * np.abs(w))
    assert not bad.any(), f"{name}: {int(bad.sum())} of {bad.size} out of tolerance, max err {err.max():.3g}"


def block_metrics(got, want):
    g, w = o.from_bf16(got).astype(np.float64), o.from_bf16(want).astype(np.float64)
    return float(np.linalg.norm(g - w) / np.linalg.norm(w)), float(np.abs(g - w).max())


def assert_block_close(got, want, name="", rel_l2=1e-2, max_abs=5e-2):
    """Per-block bar: rel-L2 <= 1e-2 and max-abs <= 5e-2."""
    r, m = block_metrics(got, want)
    assert r <= rel_l2 and m <= max_abs, f"{name}: rel_l2={r:.3e} max_abs={m:.3e}"
    return r, m
