"""Parity of every hot-path op of libh3b200.so against the CPU oracle, through the C ABI.

Shapes cross every tile boundary of the kernels (rows/keys not multiples of 64/128, one
short tile, odd widths that force the scalar paths) and include the model's real widths.
"""
import numpy as np
import pytest

import h3_oracle as o
from parity import assert_aggregate_close, assert_bf16_ulp, assert_gemm_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as entry
    return entry.load_package()


@pytest.fixture(scope="module")
def gpu(pkg):
    g = pkg.Gpu(0)
    yield g
    g.close()


def run(gpu, fn):
    gpu.begin()
    fn()
    gpu.submit()


def bf(n, seed, std=1.0):
    return o.normal_bf16(n, seed, 0.0, std)


def uniform_bf(n, seed, span=1.0):
    """Uniform in [-span, span] rounded to BF16: the input style of the reference's tests."""
    rng = np.random.default_rng(seed)
    return o.to_bf16(rng.uniform(-span, span, n).astype(np.float32))


# ------------------------------------------------------------------ row ops
@pytest.mark.parametrize("rows,width", [(4, 8), (7, 5376), (33, 130), (5, 2048), (3, 4096), (2, 5)])
def test_adaln_gate_and_fused(gpu, pkg, rows, width):
    slots, mod_rows = 6, 5
    x, br = bf(rows * width, 1, 3.0), bf(rows * width, 4, 3.0)
    w, mod = bf(width, 2, 2.0), bf(mod_rows * slots * width, 3)
    row_map = ((np.arange(rows, dtype=np.uint32) * 3 + 1) % mod_rows).astype(np.uint32)
    tx, tb, tw, tm, tr = gpu.bf16(x), gpu.bf16(br), gpu.bf16(w), gpu.bf16(mod), gpu.u32(row_map)
    out, gated = gpu.new(rows * width, pkg.BF16), gpu.new(rows * width, pkg.BF16)
    run(gpu, lambda: gpu.op("adaln_bf16", out, tx, tw, tm, tr, rows, width, slots, 0, 1, 1e-5))
    assert_bf16_ulp(out.read(), o.adaln_bf16(x, w, mod, row_map, rows, width, slots, 0, 1), "adaln")
    run(gpu, lambda: gpu.op("gate_bf16", out, tx, tb, tm, tr, rows, width, slots, 2))
    assert_bf16_ulp(out.read(), o.gate_bf16(x, br, mod, row_map, rows, width, slots, 2), "gate")
    run(gpu, lambda: gpu.op("rms_norm_bf16", out, tx, tw, rows, width, 1e-5))
    assert_bf16_ulp(out.read(), o.rms_norm_bf16(x, w, rows, width), "rms_norm")
    run(gpu, lambda: gpu.op("gate_adaln_bf16", gated, out, tx, tb, tw, tm, tm, tr, rows, width,
                            slots, 2, 3, 4, 1e-5))
    want_gated, want_out = o.gate_adaln_bf16(x, br, w, mod, mod, row_map, rows, width, slots, 2, 3, 4)
    assert_bf16_ulp(gated.read(), want_gated, "gate_adaln.gated")
    assert_bf16_ulp(out.read(), want_out, "gate_adaln.out")
    # in place, as run_block calls it (gated_residual aliases residual)
    run(gpu, lambda: gpu.op("gate_adaln_bf16", tx, out, tx, tb, tw, tm, tm, tr, rows, width, slots,
                            2, 3, 4, 1e-5))
    assert_bf16_ulp(tx.read(), want_gated, "gate_adaln.inplace")
    assert_bf16_ulp(out.read(), want_out, "gate_adaln.inplace.out")


def test_adaln_offset_and_errors(gpu, pkg):
    rows, width, slots = 3, 64, 3
    x = bf((rows + 2) * width, 5)
    w, mod = bf(width, 6), bf(4 * slots * width, 7)
    row_map = np.array([2, 0, 3], np.uint32)
    tx, tw, tm, tr = gpu.bf16(x), gpu.bf16(w), gpu.bf16(mod), gpu.u32(row_map)
    out = gpu.new(rows * width, pkg.BF16)
    run(gpu, lambda: gpu.op("adaln_bf16_offset", out, tx, 2 * width, tw, tm, tr, rows, width,
                            slots, 0, 1, 1e-5))
    assert_bf16_ulp(out.read(), o.adaln_bf16(x[2 * width:], w, mod, row_map, rows, width, slots, 0, 1))
    # outside begin..submit every op fails (h3_cuda_internal.h:163-167)
    assert not gpu.try_op("adaln_bf16", out, tx, tw, tm, tr, rows, width, slots, 0, 1, 1e-5)
    assert "no active command" in gpu.error()
    gpu.begin()
    assert not gpu.try_op("adaln_bf16", out, tx, tw, tm, tr, rows, width, slots, 3, 1, 1e-5)
    big = gpu.new(2 * 5384, pkg.BF16)
    assert not gpu.try_op("gate_adaln_bf16", big, big, big, big, tw, tm, tm, tr, 2, 5384, slots,
                          0, 1, 2, 1e-5)                       # width > 5376 is rejected
    f32 = gpu.new(rows * width, pkg.F32)
    assert not gpu.try_op("adaln_bf16", f32, tx, tw, tm, tr, rows, width, slots, 0, 1, 1e-5)
    gpu.submit()


def test_f32_adaln_and_gate(gpu, pkg):
    rows, width, slots = 4, 8, 3
    x, br = o.normal_f32(rows * width, 1, 0, 3), o.normal_f32(rows * width, 2, 0, 3)
    w, mod = o.normal_f32(width, 3, 0, 2), o.normal_f32(4 * slots * width, 4)
    row_map = np.array([2, 0, 3, 1], np.uint32)
    tx, tb, tw, tm, tr = gpu.f32(x), gpu.f32(br), gpu.f32(w), gpu.f32(mod), gpu.u32(row_map)
    out = gpu.new(rows * width, pkg.F32)
    run(gpu, lambda: gpu.op("adaln_f32", out, tx, tw, tm, tr, rows, width, slots, 0, 1, 1e-5))
    np.testing.assert_allclose(out.read(), o.adaln_f32(x, w, mod, row_map, rows, width, slots, 0, 1),
                               rtol=1e-5, atol=1e-5)
    run(gpu, lambda: gpu.op("gate_f32", out, tx, tb, tm, tr, rows, width, slots, 2))
    np.testing.assert_allclose(out.read(), o.gate_f32(x, br, mod, row_map, rows, width, slots, 2),
                               rtol=1e-6, atol=1e-6)


def test_elementwise(gpu, pkg):
    n = 1003
    a, b = bf(n, 1, 4.0), bf(n, 2, 4.0)
    ta, tb = gpu.bf16(a), gpu.bf16(b)
    out = gpu.new(n, pkg.BF16)
    run(gpu, lambda: gpu.op("add_bf16", out, ta, tb, n))
    assert np.array_equal(out.read(), o.add_bf16(a, b))
    run(gpu, lambda: gpu.op("sub_bf16", out, ta, tb, n))
    assert np.array_equal(out.read(), o.sub_bf16(a, b))
    run(gpu, lambda: gpu.op("silu_bf16", out, ta, n))
    assert_bf16_ulp(out.read(), o.silu_bf16(a), "silu")
    rows, width = 7, 72
    fused = bf(rows * width * 2, 3, 4.0)
    tf, to = gpu.bf16(fused), gpu.new(rows * width, pkg.BF16)
    run(gpu, lambda: gpu.op("swiglu_bf16", to, tf, rows, width))
    assert_bf16_ulp(to.read(), o.swiglu_bf16(fused, rows, width), "swiglu")
    x = o.normal_f32(n, 5, 0, 3)
    tx, t16, t32 = gpu.f32(x), gpu.new(n, pkg.BF16), gpu.new(n, pkg.F32)
    run(gpu, lambda: (gpu.op("cast_f32_to_bf16", t16, tx, n), gpu.op("cast_bf16_to_f32", t32, t16, n)))
    assert np.array_equal(t16.read(), o.to_bf16(x))
    assert np.array_equal(t32.read(), o.from_bf16(o.to_bf16(x)))
    run(gpu, lambda: gpu.op("silu_f32", t32, tx, n))
    np.testing.assert_allclose(t32.read(), o.silu_f32(x), rtol=1e-5, atol=1e-6)
    dst = gpu.bf16(np.zeros(64, np.uint16))
    run(gpu, lambda: gpu.op("copy_bf16", dst, 8, ta, 3, 40))
    want = np.zeros(64, np.uint16)
    want[8:48] = a[3:43]
    assert np.array_equal(dst.read(), want)


def test_euler(gpu, pkg):
    n = 777
    sample = o.normal_f32(n + 5, 1)
    last, prev = bf(n, 2), bf(n, 3)
    ts, tl, tp = gpu.f32(sample), gpu.bf16(last), gpu.bf16(prev)
    run(gpu, lambda: gpu.op("euler_bf16", ts, 5, tl, tp, n, -0.05, 0.25))
    want = sample.copy()
    want[5:] = o.euler_bf16(sample[5:], last, prev, -0.05, 0.25)
    np.testing.assert_allclose(ts.read(), want, rtol=1e-6, atol=1e-7)


def test_token_pool_and_expand(gpu, pkg):
    width, input_rows = 64, 10
    pairs = np.array([[0, 0], [1, 1], [2, 3], [4, 5], [6, 7], [8, 9]], np.uint32).reshape(-1)
    rows = 6
    baseline_idx = np.array([0xFFFFFFFF, 0xFFFFFFFF, 0, 1, 2, 3], np.uint32)
    x = bf(input_rows * width, 1)
    base0 = np.zeros(4 * width, np.uint16)
    want_out, want_orig, want_base = o.token_pool_bf16(x, base0, baseline_idx, pairs, input_rows, rows, width)
    tx, tp, tb = gpu.bf16(x), gpu.u32(pairs), gpu.u32(baseline_idx)
    out, orig, base = gpu.new(rows * width, pkg.BF16), gpu.bf16(np.zeros(input_rows * width, np.uint16)), gpu.bf16(base0)
    run(gpu, lambda: gpu.op("token_pool_bf16", out, tx, 0, orig, 0, base, 0, tb, tp, input_rows, rows, 4, width))
    assert np.array_equal(out.read(), want_out)
    assert np.array_equal(orig.read(), want_orig)
    assert np.array_equal(base.read(), want_base)
    # fused pool + adaLN == pool then adaLN of the pooled rows
    slots = 3
    w, mod = bf(width, 2, 2.0), bf(4 * slots * width, 3)
    row_map = np.array([0, 1, 2, 3, 0, 1], np.uint32)
    tw, tm, tr = gpu.bf16(w), gpu.bf16(mod), gpu.u32(row_map)
    res, out2 = gpu.new(rows * width, pkg.BF16), gpu.new(rows * width, pkg.BF16)
    run(gpu, lambda: gpu.op("token_pool_adaln_bf16", res, out2, tx, 0, orig, 0, base, 0, tb, tp, tw, tm,
                            tr, input_rows, rows, 4, width, slots, 0, 1, 1e-5))
    assert np.array_equal(res.read(), want_out)
    assert_bf16_ulp(out2.read(), o.adaln_bf16(want_out, w, mod, row_map, rows, width, slots, 0, 1))
    # expand
    parents = np.array([0, 1, 2, 2, 3, 3, 4, 4, 5, 5], np.uint32)
    reduced = bf(rows * width, 4)
    want = o.token_expand_delta_bf16(want_orig, reduced, want_base, baseline_idx, parents,
                                     input_rows, width, 2, 0.75)
    tred, tpar, full = gpu.bf16(reduced), gpu.u32(parents), gpu.new(input_rows * width, pkg.BF16)
    run(gpu, lambda: gpu.op("token_expand_delta_bf16", full, orig, 0, tred, base, 0, tb, tpar,
                            input_rows, rows, 4, width, 2, 0.75))
    assert_bf16_ulp(full.read(), want, "token_expand")
    row_map10 = (np.arange(10, dtype=np.uint32) % 4).astype(np.uint32)
    tr10 = gpu.u32(row_map10)
    res10, out10 = gpu.new(input_rows * width, pkg.BF16), gpu.new(input_rows * width, pkg.BF16)
    run(gpu, lambda: gpu.op("token_expand_adaln_bf16", res10, out10, orig, 0, tred, base, 0, tb, tpar,
                            tw, tm, tr10, input_rows, rows, 4, width, 2, 0.75, slots, 0, 1, 1e-5))
    assert_bf16_ulp(res10.read(), want, "token_expand_adaln.residual")
    assert_bf16_ulp(out10.read(), o.adaln_bf16(res10.read(), w, mod, row_map10, input_rows, width, slots, 0, 1))


# ---------------------------------------------------------------- projections
@pytest.mark.parametrize("rows,k,n,bias", [
    (5, 7, 9, True),            # scalar kernel, odd everything (reference's small case)
    (64, 2048, 256, True),      # tensor cores, one tile
    (130, 512, 1000, True),     # ragged rows and columns
    (257, 5376, 768, False),    # model K, three row tiles with a 1-row tail
    (128, 200, 264, False),     # K tail inside a 64-element slab
    (300, 7168, 5376, False),   # attention out-projection shape
    (42, 2688, 96768, True),    # adaLN modulation projection at its largest row count
                                # (h3_dit_schedule.c:264-301: rows = time rows <= 42)
    (2, 2688, 96768, True),     # ... and at the two time rows of a single-step run
])
def test_linear_bf16(gpu, pkg, rows, k, n, bias):
    x, w = bf(rows * k, 1), bf(n * k, 2, 0.05)
    b = bf(n, 3) if bias else None
    tx, tw, tb = gpu.bf16(x), gpu.bf16(w), (gpu.bf16(b) if bias else None)
    out = gpu.new(rows * n, pkg.BF16)
    before = gpu.stats()
    run(gpu, lambda: gpu.op("linear_bf16", out, tx, tw, tb, rows, k, n))
    after = gpu.stats()
    assert_gemm_close(out.read(), o.linear_bf16(x, w, b, rows, k, n), f"linear {rows}x{k}x{n}")
    routed = rows >= 32 and k >= 256 and n >= 256      # reference's counter rule
    assert after.mps_linear_dispatches - before.mps_linear_dispatches == (1 if routed else 0)
    assert after.direct_dispatches - before.direct_dispatches == (0 if routed else 1)


def test_linear_bf16_exact_route(gpu, pkg, monkeypatch):
    """The SIMT route keeps one sequential fmaf chain per output: bit-identical to the oracle."""
    monkeypatch.setenv("H3B_NO_TENSOR_CORES", "1")
    rows, k, n = 70, 256, 130
    x, w, b = bf(rows * k, 1), bf(n * k, 2, 0.5), bf(n, 3)
    out = gpu.new(rows * n, pkg.BF16)
    tx, tw, tb = gpu.bf16(x), gpu.bf16(w), gpu.bf16(b)
    run(gpu, lambda: gpu.op("linear_bf16", out, tx, tw, tb, rows, k, n))
    assert np.array_equal(out.read(), o.linear_bf16(x, w, b, rows, k, n))


def test_linear_f32(gpu, pkg):
    rows, k, n = 9, 256, 70
    x, w, b = o.normal_f32(rows * k, 1), o.normal_f32(n * k, 2, 0, 0.1), o.normal_f32(n, 3)
    out = gpu.new(rows * n, pkg.F32)
    tx, tw, tb = gpu.f32(x), gpu.f32(w), gpu.f32(b)
    run(gpu, lambda: gpu.op("linear_f32", out, tx, tw, tb, rows, k, n))
    assert np.array_equal(out.read().view(np.uint32), o.linear_f32(x, w, b, rows, k, n).view(np.uint32))


@pytest.mark.parametrize("rows,k,hidden,n", [(4, 8, 6, 5), (200, 512, 1024, 512), (130, 5376, 256, 5376)])
@pytest.mark.parametrize("unfused", [False, True])
def test_mlp_bf16(gpu, pkg, monkeypatch, rows, k, hidden, n, unfused):
    if unfused:
        monkeypatch.setenv("H3B_UNFUSED_MLP", "1")
    w1 = 1.0 / np.sqrt(k)          # keeps every stage O(1), as N(0, 0.02) does at the model width
    w2 = 1.0 / np.sqrt(hidden)
    x, fc1, fc2 = bf(rows * k, 1), bf(2 * hidden * k, 2, w1), bf(n * hidden, 3, w2)
    out = gpu.new(rows * n, pkg.BF16)
    tx, t1, t2 = gpu.bf16(x), gpu.bf16(fc1), gpu.bf16(fc2)
    before = gpu.stats()
    run(gpu, lambda: gpu.op("mlp_bf16", out, tx, t1, t2, rows, k, hidden, n))
    assert gpu.stats().mps_linear_dispatches - before.mps_linear_dispatches == 2
    want = o.mlp_bf16(x, fc1, fc2, rows, k, hidden, n)
    if rows * k * hidden <= 1024:
        assert_gemm_close(out.read(), want, "mlp")        # the reference's own tiny case
    else:
        assert_aggregate_close(out.read(), want, "mlp")


def test_patch_linear(gpu, pkg):
    rows, k, n = 37, 96, 5376
    x, w, b = o.normal_f32(rows * k, 1), o.normal_f32(n * k, 2, 0, 0.05), o.normal_f32(n, 3, 0, 0.1)
    tx, tw, tb = gpu.f32(x), gpu.f32(w), gpu.f32(b)
    hidden = gpu.bf16(np.zeros((rows + 3) * n, np.uint16))
    run(gpu, lambda: gpu.op("patch_linear_bf16_offset", hidden, 3 * n, tx, 0, tw, tb, rows, k, n))
    want = np.zeros((rows + 3) * n, np.uint16)
    o.patch_linear_bf16(want, x, w, b, None, 3, rows, k, n)
    assert np.array_equal(hidden.read(), want)
    perm = np.random.default_rng(0).permutation(rows + 3)[:rows].astype(np.uint32)
    scat = gpu.bf16(np.zeros((rows + 3) * n, np.uint16))
    tp = gpu.u32(perm)
    run(gpu, lambda: gpu.op("patch_linear_bf16_map", scat, tx, tw, tb, tp, rows + 3, rows, k, n))
    want = np.zeros((rows + 3) * n, np.uint16)
    o.patch_linear_bf16(want, x, w, b, perm, 0, rows, k, n)
    assert np.array_equal(scat.read(), want)
    gpu.begin()
    assert not gpu.try_op("patch_linear_bf16", hidden, tx, tw, tb, rows, 64, n)   # shape rule
    gpu.submit()


@pytest.mark.parametrize("out_dim,bias", [(96, True), (32, False), (9, True)])
def test_adaln_linear_final_head(gpu, pkg, out_dim, bias):
    rows, width, slots, off = 70, 5376, 2, 5376
    x = bf(rows * width + off, 1, 3.0)
    nw, mod = bf(width, 2, 2.0), bf(3 * slots * width, 3)
    w, b = bf(out_dim * width, 4, 0.02), (bf(out_dim, 5) if bias else None)
    row_map = (np.arange(rows, dtype=np.uint32) % 3).astype(np.uint32)
    out, inv = gpu.new(rows * out_dim, pkg.BF16), gpu.new(rows, pkg.F32)
    tx, tn, tm, tr, tw = gpu.bf16(x), gpu.bf16(nw), gpu.bf16(mod), gpu.u32(row_map), gpu.bf16(w)
    tb = gpu.bf16(b) if bias else None
    run(gpu, lambda: gpu.op("adaln_linear_bf16", out, inv, tx, off, tn, tm, tr, tw, tb, rows, width,
                            out_dim, slots, 0, 1, 1e-5))
    want, want_inv = o.adaln_linear_bf16(x[off:], nw, mod, row_map, w, b, rows, width, out_dim, slots, 0, 1)
    assert_gemm_close(out.read(), want, "final head")
    np.testing.assert_allclose(inv.read(), want_inv, rtol=1e-5)


# ----------------------------------------------------------------- attention
@pytest.mark.parametrize("grouped", [0, 1])
@pytest.mark.parametrize("seq,heads,hd,half", [(5, 3, 16, 6), (9, 2, 128, 48), (3, 4, 8, 0), (70, 56, 128, 48)])
def test_qkv_rope(gpu, pkg, seq, heads, hd, half, grouped):
    qkv = bf(seq * heads * hd * 3, 10, 2.0)
    qw, kw = bf(hd, 11), bf(hd, 12)
    cos, sin = bf(max(seq * half, 1), 13), bf(max(seq * half, 1), 14)
    n = seq * heads * hd
    tq, tk, tv = (gpu.new(n, pkg.BF16) for _ in range(3))
    t = [gpu.bf16(a) for a in (qkv, qw, kw, cos, sin)]
    name = "grouped_qkv_rope_bf16" if grouped else "qkv_rope_bf16"
    run(gpu, lambda: gpu.op(name, tq, tk, tv, *t, seq, heads, hd, half, 1e-5))
    q, k, v = o.qkv_rope_bf16(qkv, qw, kw, cos, sin, seq, heads, hd, half, grouped)
    assert_bf16_ulp(tq.read(), q, "q")
    assert_bf16_ulp(tk.read(), k, "k")
    assert np.array_equal(tv.read(), v)


@pytest.mark.parametrize("seq,heads,hd", [
    (5, 2, 8), (100, 3, 64), (130, 2, 128),      # the reference's own test shapes
    (64, 1, 128), (65, 2, 128), (128, 1, 128), (129, 3, 128), (1000, 4, 128), (1, 1, 128),
    (1000, 3, 64), (129, 2, 64),                 # head_dim 64 on the one-tile tensor-core kernel
    (1000, 20, 128), (520, 64, 128), (1100, 40, 64),   # more (query block, head) tiles than SMs
])
@pytest.mark.parametrize("head_major", [0, 1])
@pytest.mark.parametrize("two_tiles", [False, True])
def test_sdpa(gpu, pkg, monkeypatch, seq, heads, hd, head_major, two_tiles):
    """Dense attention on both tensor-core kernels: the default (one query tile per CTA, softmax
    groups alternating over key steps) and the one with two query tiles in ping-pong, which
    H3B_SDPA_TWO_TILES=1 selects."""
    if two_tiles:
        if hd != 128:
            pytest.skip("head_dim != 128 takes the SIMT kernel either way")
        monkeypatch.setenv("H3B_SDPA_TWO_TILES", "1")
    n = seq * heads * hd
    scale = 1.0 / np.sqrt(hd)
    name = "sdpa_bf16_head_major_output" if head_major else "sdpa_bf16"
    # (a) inputs uniform in [-1, 1] as in the reference's tests: its elementwise tolerance
    q, k, v = uniform_bf(n, 15), uniform_bf(n, 16), uniform_bf(n, 17)
    tq, tk, tv, to = gpu.bf16(q), gpu.bf16(k), gpu.bf16(v), gpu.new(n, pkg.BF16)
    before = gpu.stats()
    run(gpu, lambda: gpu.op(name, to, tq, tk, tv, seq, heads, hd, scale))
    assert gpu.stats().mps_sdpa_dispatches - before.mps_sdpa_dispatches == 1
    want = o.sdpa_bf16(q, k, v, seq, heads, hd, scale, head_major, round_p=0)
    assert_gemm_close(to.read(), want, f"sdpa {seq}x{heads}x{hd}")
    # (b) N(0,1) inputs (peaked softmax): P is rounded to BF16 before P.V, as on the
    # reference's tensor-core path, so near-cancelling outputs move by a few 1e-3
    q, k, v = bf(n, 15), bf(n, 16), bf(n, 17)
    tq, tk, tv = gpu.bf16(q), gpu.bf16(k), gpu.bf16(v)
    run(gpu, lambda: gpu.op(name, to, tq, tk, tv, seq, heads, hd, scale))
    want = o.sdpa_bf16(q, k, v, seq, heads, hd, scale, head_major, round_p=0)
    assert_aggregate_close(to.read(), want, f"sdpa normal {seq}x{heads}x{hd}", rel_l2=4e-3, max_abs=2e-2)


@pytest.mark.parametrize("two_tiles", [False, True])
def test_sdpa_sharp_scores_rescale(gpu, pkg, monkeypatch, two_tiles):
    """Scores whose running maximum keeps growing by more than the lazy-rescale threshold:
    keys are scaled up along the sequence so every tile raises the maximum."""
    if two_tiles:
        monkeypatch.setenv("H3B_SDPA_TWO_TILES", "1")
    seq, heads, hd = 700, 2, 128
    n = seq * heads * hd
    q = o.from_bf16(bf(n, 1)).reshape(seq, heads, hd)
    k = o.from_bf16(bf(n, 2)).reshape(seq, heads, hd).copy()
    k *= np.linspace(0.2, 6.0, seq, dtype=np.float32)[:, None, None]
    q8, k8, v8 = o.to_bf16(q.reshape(-1)), o.to_bf16(k.reshape(-1)), bf(n, 3)
    scale = 1.0 / np.sqrt(hd)
    to = gpu.new(n, pkg.BF16)
    tq, tk, tv = gpu.bf16(q8), gpu.bf16(k8), gpu.bf16(v8)
    run(gpu, lambda: gpu.op("sdpa_bf16", to, tq, tk, tv, seq, heads, hd, scale))
    assert_aggregate_close(to.read(), o.sdpa_bf16(q8, k8, v8, seq, heads, hd, scale, 0, round_p=0),
                           "sharp sdpa", rel_l2=4e-3, max_abs=2e-2)


def test_sdpa_simt_matches_tensor_core(gpu, pkg, monkeypatch):
    seq, heads, hd = 333, 2, 128
    n = seq * heads * hd
    q, k, v = bf(n, 21), bf(n, 22), bf(n, 23)
    tq, tk, tv = gpu.bf16(q), gpu.bf16(k), gpu.bf16(v)
    a, b = gpu.new(n, pkg.BF16), gpu.new(n, pkg.BF16)
    run(gpu, lambda: gpu.op("sdpa_bf16", a, tq, tk, tv, seq, heads, hd, 0.0884))
    monkeypatch.setenv("H3B_SDPA_SIMT", "1")
    run(gpu, lambda: gpu.op("sdpa_bf16", b, tq, tk, tv, seq, heads, hd, 0.0884))
    assert_aggregate_close(a.read(), b.read(), "tc vs simt", rel_l2=4e-3, max_abs=2e-2)


@pytest.mark.parametrize("unfused", [False, True])
@pytest.mark.parametrize("rows,k,heads", [(150, 512, 4), (300, 5376, 7), (129, 1024, 56)])
def test_grouped_qkv_linear_rope(gpu, pkg, monkeypatch, rows, k, heads, unfused):
    """Projection + head norm + RoPE: fused into the GEMM epilogue (default) and as the
    reference's two calls; heads=7 leaves an odd number of 128-column units (half-empty tile)."""
    if unfused:
        monkeypatch.setenv("H3B_UNFUSED_QKV_ROPE", "1")
    hd, half = 128, 48
    x, w = bf(rows * k, 1), bf(3 * heads * hd * k, 2, 1.0 / np.sqrt(k))
    qw, kw = bf(hd, 3, 0.5), bf(hd, 4, 0.5)
    cos, sin = bf(rows * half, 5), bf(rows * half, 6)
    n = rows * heads * hd
    tq, tk, tv = (gpu.new(n, pkg.BF16) for _ in range(3))
    tqkv = gpu.new(3 * n, pkg.BF16)
    t = [gpu.bf16(a) for a in (x, w, qw, kw, cos, sin)]
    before = gpu.stats()
    run(gpu, lambda: gpu.op("grouped_qkv_linear_rope_bf16", tq, tk, tv, tqkv, *t, rows, k, heads, hd, half, 1e-5))
    after = gpu.stats()
    assert after.mps_linear_dispatches - before.mps_linear_dispatches == 1
    assert after.direct_dispatches - before.direct_dispatches == 1
    qkv = o.linear_bf16(x, w, None, rows, k, 3 * heads * hd)
    q, kk, v = o.qkv_rope_bf16(qkv, qw, kw, cos, sin, rows, heads, hd, half, 1)
    assert_aggregate_close(tq.read(), q, "q", rel_l2=3e-3, max_abs=5e-2)
    assert_aggregate_close(tk.read(), kk, "k", rel_l2=3e-3, max_abs=5e-2)
    assert_gemm_close(tv.read(), v, "v")


def test_qkv_push_form_with_one_rank_equals_the_local_form(gpu, pkg):
    """h3x_grouped_qkv_linear_rope_push with a one-rank peer table stores every head's q/k/v row
    into this GPU's own gathered buffers, [row][head][128] like the local outputs: the GEMM's
    sequence-parallel epilogue on a single GPU, bit for bit what the local call gives."""
    rows, k, heads, hd, half = 300, 5376, 7, 128, 48
    x, w = bf(rows * k, 1), bf(3 * heads * hd * k, 2, 1.0 / np.sqrt(k))
    qw, kw = bf(hd, 3, 0.5), bf(hd, 4, 0.5)
    cos, sin = bf(rows * half, 5), bf(rows * half, 6)
    n = rows * heads * hd
    local = [gpu.new(n, pkg.BF16) for _ in range(3)]
    pushed = [gpu.new(n, pkg.BF16) for _ in range(3)]
    scratch = gpu.new(3 * n, pkg.BF16)
    t = [gpu.bf16(a) for a in (x, w, qw, kw, cos, sin)]
    run(gpu, lambda: gpu.op("grouped_qkv_linear_rope_bf16", *local, scratch, *t, rows, k, heads, hd, half, 1e-5))
    peers = pkg.UlyssesPeers()
    peers.world, peers.rank, peers.rows_local = 1, 0, rows
    peers.q[0], peers.k[0], peers.v[0] = (tensor.pointer for tensor in pushed)
    run(gpu, lambda: gpu.op("h3x_grouped_qkv_linear_rope_push", peers, *t, rows, k, heads, hd, half, 1e-5))
    for name, a, b in zip("qkv", pushed, local):
        assert np.array_equal(a.read(), b.read()), name


@pytest.mark.parametrize("kernel", ["pairs", "lone"])
def test_split_tail_round_of_the_tensor_core_gemm(gpu, pkg, monkeypatch, kernel):
    """Tile counts that leave a partly filled last round: the leftover tiles are split along K
    over all CTAs (F32 partial tiles, fixed-order merge, then the usual epilogue). Covered for
    the plain, SwiGLU and QKV epilogues on CTA pairs (256 x 256 tiles, 74 pairs) and on lone
    CTAs (128 x 256 tiles, 148 CTAs), against the oracle and against the same launch with the
    split switched off."""
    if kernel == "lone":
        monkeypatch.setenv("H3B_NO_CTA_PAIRS", "1")
    rows = 512 if kernel == "pairs" else 384          # 2 pair row tiles / 3 lone row tiles
    col_tiles = 38 if kernel == "pairs" else 50       # 76 pair tiles on 74 pairs / 150 tiles on 148 CTAs
    k = 1024                                          # 16 K blocks: slices of 4
    results = {}
    for split in ("1", "0"):
        monkeypatch.setenv("H3B_NO_SPLIT_K", "0" if split == "1" else "1")
        # plain projection + bias
        n = col_tiles * 256 - 40                      # ragged last column tile
        x, w, b = bf(rows * k, 1), bf(n * k, 2, 1.0 / np.sqrt(k)), bf(n, 3)
        tx, tw, tb, out = gpu.bf16(x), gpu.bf16(w), gpu.bf16(b), gpu.new(rows * n, pkg.BF16)
        run(gpu, lambda: gpu.op("linear_bf16", out, tx, tw, tb, rows, k, n))
        results["linear", split] = out.read()
        if split == "1":
            assert_gemm_close(results["linear", split], o.linear_bf16(x, w, b, rows, k, n), "split linear")
        # fc1 + SwiGLU (a column tile = 128 gate + 128 up columns)
        hidden = col_tiles * 128
        fc1 = bf(2 * hidden * k, 4, 1.0 / np.sqrt(k))
        t1, act = gpu.bf16(fc1), gpu.new(rows * hidden, pkg.BF16)
        run(gpu, lambda: gpu.op("h3x_linear_swiglu_bf16", act, tx, t1, rows, k, hidden))
        results["swiglu", split] = act.read()
        if split == "1":
            fused = o.linear_bf16(x, fc1, None, rows, k, 2 * hidden)
            assert_aggregate_close(results["swiglu", split], o.swiglu_bf16(fused, rows, hidden), "split swiglu")
        # QKV + head norm + RoPE (a column tile = two 128-column units)
        heads = (col_tiles * 2 - 1) // 3              # 25 / 33 heads: 75 / 99 units, last tile half empty
        wq = bf(3 * heads * 128 * k, 5, 1.0 / np.sqrt(k))
        qw, kw, cos, sin = bf(128, 6, 0.5), bf(128, 7, 0.5), bf(rows * 48, 8), bf(rows * 48, 9)
        cnt = rows * heads * 128
        tq, tk, tv = (gpu.new(cnt, pkg.BF16) for _ in range(3))
        scratch = gpu.new(3 * cnt, pkg.BF16)
        t = [gpu.bf16(a) for a in (wq, qw, kw, cos, sin)]
        run(gpu, lambda: gpu.op("grouped_qkv_linear_rope_bf16", tq, tk, tv, scratch, tx, *t, rows, k, heads,
                                128, 48, 1e-5))
        results["qkv", split] = np.concatenate([tq.read(), tk.read(), tv.read()])
        if split == "1":
            qkv = o.linear_bf16(x, wq, None, rows, k, 3 * heads * 128)
            q, kk, v = o.qkv_rope_bf16(qkv, qw, kw, cos, sin, rows, heads, 128, 48, 1)
            assert_aggregate_close(tq.read(), q, "split q", rel_l2=3e-3, max_abs=5e-2)
            assert_aggregate_close(tk.read(), kk, "split k", rel_l2=3e-3, max_abs=5e-2)
            assert_gemm_close(tv.read(), v, "split v")
    assert lib_status(gpu) == 0
    for name in ("linear", "swiglu", "qkv"):
        # the split changes the order of the F32 sum for the split tiles only: isolated last-bit moves
        a, b_ = results[name, "1"], results[name, "0"]
        assert_aggregate_close(a, b_, f"{name}: split vs whole", rel_l2=2e-3, max_abs=5e-2)
        assert np.mean(a != b_) < 0.05


def lib_status(gpu):
    return gpu.lib.h3x_kernel_status(gpu.handle)


def test_ulysses_pack_unpack_roundtrip(gpu, pkg):
    rows, heads, hd, world = 37, 8, 128, 4
    x = bf(rows * heads * hd, 1)
    tx, tp, tu = gpu.bf16(x), gpu.new(x.size, pkg.BF16), gpu.new(x.size, pkg.BF16)
    run(gpu, lambda: gpu.op("h3x_ulysses_pack_heads", tp, tx, rows, heads, hd, world))
    want = x.reshape(rows, world, heads // world, hd).transpose(1, 0, 2, 3).reshape(-1)
    assert np.array_equal(tp.read(), want)
    run(gpu, lambda: gpu.op("h3x_ulysses_unpack_heads", tu, tp, rows, heads, hd, world))
    assert np.array_equal(tu.read(), x)
