"""Parity at the benchmark's full sizes, where the CPU oracle cannot recompute everything:

  * one block at S = 6,400 and the model's full width against the CPU oracle (about a minute of
    host time);
  * attention at S = 50,476: sampled query rows against the oracle's exact rows (the first rows,
    tile boundaries, the ragged last tile), and the size-independent property that constant
    values come back unchanged (softmax rows sum to one);
  * the fused QKV projection (GEMM + head norm + RoPE) at M = 50,476 rows: sampled rows against
    the oracle's projection and RoPE of exactly those rows."""
import numpy as np
import pytest

import h3_oracle as o
from block_case import make_block_case, run_block_on_gpu
from parity import assert_aggregate_close, assert_block_close

pytestmark = pytest.mark.gpu
S4 = 50476            # 50,220 video + 256 text rows
SCALE = 1.0 / np.sqrt(128.0)


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as entry
    return entry.load_package()


def fast_bf16(n, seed, std=1.0):
    rng = np.random.default_rng(seed)
    out = np.empty(n, np.uint16)
    for i in range(0, n, 1 << 24):
        m = min(1 << 24, n - i)
        out[i:i + m] = o.to_bf16(rng.standard_normal(m, dtype=np.float32) * np.float32(std))
    return out


def test_block_at_s6400_full_width_matches_oracle(pkg):
    case = make_block_case(rows=6400, text_rows=256, heads=56, hidden=5376, ffn=14336, seed=2, fast=True)
    gpu = pkg.Gpu(0)
    try:
        got = run_block_on_gpu(pkg, gpu, case)
    finally:
        gpu.close()
    want = o.dit_block(case.hidden, case.weights, case.row_map, case.rope_cos, case.rope_sin,
                       rows=case.rows, width=5376, heads=56, head_dim=128, ffn=14336, rope_half=48,
                       round_p=1)
    r, m = assert_block_close(got, want, "block S=6400 full width")
    print(f"S=6400 full-width block vs CPU oracle: rel_l2={r:.3e} max_abs={m:.3e}")


def test_attention_at_s50476_sampled_rows_and_constant_values(pkg):
    heads = 4
    n = S4 * heads * 128
    q, k, v = (fast_bf16(n, s) for s in (10, 11, 12))
    rows = [0, 1, 127, 128, 255, 256, 25000, 25087, S4 - 129, S4 - 45, S4 - 44, S4 - 1]
    gpu = pkg.Gpu(0)
    try:
        tq, tk, tv = gpu.bf16(q), gpu.bf16(k), gpu.bf16(v)
        out = gpu.new(n, pkg.BF16)
        gpu.begin()
        gpu.op("sdpa_bf16", out, tq, tk, tv, S4, heads, 128, SCALE)
        gpu.submit()
        got = out.read().reshape(S4, heads * 128)
        ones = gpu.bf16(np.full(n, 0x3f80, np.uint16))
        gpu.begin()
        gpu.op("sdpa_bf16", out, tq, tk, ones, S4, heads, 128, SCALE)
        gpu.submit()
        const = o.from_bf16(out.read())
    finally:
        gpu.close()
    for r in rows:
        want = o.sdpa_bf16(q, k, v, S4, heads, 128, SCALE, round_p=1, rows=(r, r + 1))
        want = want.reshape(S4, heads * 128)[r]
        assert_aggregate_close(got[r], want, f"attention S={S4} row {r}")
    # P is rounded to BF16 for the numerator only: values within a few 2^-9 of one
    assert np.all(np.abs(const - 1.0) <= 2.0 ** -7), float(np.abs(const - 1.0).max())


def test_fused_qkv_projection_at_50476_rows_sampled(pkg):
    heads, hidden = 56, 5376
    inner = heads * 128
    x = fast_bf16(S4 * hidden, 20)
    w = fast_bf16(3 * inner * hidden, 21, 0.02)
    one = np.full(128, 0x3f80, np.uint16)
    rng = np.random.default_rng(22)
    cos = o.to_bf16(np.cos(rng.uniform(0, 6.28, S4 * 48)).astype(np.float32))
    sin = o.to_bf16(np.sin(rng.uniform(0, 6.28, S4 * 48)).astype(np.float32))
    rows = np.array([0, 127, 128, 4095, 4096, 30001, S4 - 129, S4 - 2, S4 - 1])
    gpu = pkg.Gpu(0)
    try:
        tx, tw, tn = gpu.bf16(x), gpu.bf16(w), gpu.bf16(one)
        tc, ts = gpu.bf16(cos), gpu.bf16(sin)
        tq, tk, tv = (gpu.new(S4 * inner, pkg.BF16) for _ in range(3))
        scratch = gpu.new(S4 * 3 * inner, pkg.BF16)
        gpu.begin()
        gpu.op("grouped_qkv_linear_rope_bf16", tq, tk, tv, scratch, tx, tw, tn, tn, tc, ts, S4, hidden,
               heads, 128, 48, 1e-5)
        gpu.submit()
        got = [t.read().reshape(S4, inner)[rows] for t in (tq, tk, tv)]
    finally:
        gpu.close()
    xs = np.ascontiguousarray(x.reshape(S4, hidden)[rows]).reshape(-1)
    qkv = o.linear_bf16(xs, w, None, len(rows), hidden, 3 * inner)
    cs = np.ascontiguousarray(cos.reshape(S4, 48)[rows]).reshape(-1)
    sn = np.ascontiguousarray(sin.reshape(S4, 48)[rows]).reshape(-1)
    want = o.qkv_rope_bf16(qkv, one, one, cs, sn, len(rows), heads, 128, 48, grouped=1)
    for name, g, wv in zip("qkv", got, want):
        assert_aggregate_close(g.reshape(-1), wv, f"fused QKV projection M={S4}: {name}")
