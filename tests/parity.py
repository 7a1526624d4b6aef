"""Comparison rules used by the parity tests, taken from the reference's own tests."""
import numpy as np

import h3_oracle as o


def _ordered(bits):
    """BF16 bit patterns mapped to integers that are monotone in the value."""
    b = np.asarray(bits, np.uint16).astype(np.int32)
    return np.where(b & 0x8000, -(b & 0x7FFF), b)


def assert_bf16_ulp(got, want, name="", ulps=1, atol=2e-4):
    """Elementwise / row ops: the two BF16 results are equal or adjacent representable
    values. The reference's own check (tests/test_cuda_dit.c:57-71) allows |diff| <=
    max(|a|,|b|) * 2^-8, i.e. between half a BF16 spacing and one; it holds there because
    its 8-wide rows reduce in the same order on CPU and GPU. At the model's row width the
    sum of squares is reduced in a different order (the reference's GPU kernels use a
    256-thread tree as well), so results may land on the neighbouring BF16 value.
    Where `a*b + c` nearly cancels, the last F32 bits of O(1..100) operands (and nvcc's
    fused multiply-add against the CPU's separate rounding) are many ulps of the tiny
    result, hence the small absolute floor."""
    diff = np.abs(_ordered(got) - _ordered(want))
    close = np.abs(o.from_bf16(got).astype(np.float64) - o.from_bf16(want).astype(np.float64)) <= atol
    bad = (diff > ulps) & ~close
    assert not bad.any(), (f"{name}: {int(bad.sum())} of {bad.size} differ by more than {ulps} "
                           f"BF16 ulp (max {int(diff.max())})")


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


def assert_aggregate_close(got, want, name="", rel_l2=5e-3, max_abs=5e-2):
    """Composite ops (several BF16-rounded stages) and attention on peaked score
    distributions: single roundings of intermediates legitimately move isolated outputs by
    an ulp or two, so the elementwise GEMM tolerance does not apply; bound the aggregate
    error instead, well inside the per-block bar (rel-L2 1e-2, max-abs 5e-2)."""
    r, m = block_metrics(got, want)
    assert r <= rel_l2 and m <= max_abs, f"{name}: rel_l2={r:.3e} max_abs={m:.3e}"
    return r, m
