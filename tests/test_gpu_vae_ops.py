"""Parity of the video-VAE decoder's F32 operations (h3_video_vae.c:425-461: 36 transformer
blocks of hidden 2048, 32 heads x 64, FFN 8192) through the C ABI.

Checkers: the CPU oracle (pinned bit for bit to the reference's own CPU test references,
tests/test_oracle_pin.py) with the tolerances of the reference's tests, and, for the decoder's
shapes, the reference's own CUDA backend (oracle/_ref/libh3ref.so) on the same inputs.
Tolerances (reference): row ops 1e-5 (tests/test_cuda_core.c:305,371,442); QKV split 1e-5
(tests/test_cuda_attention.c:483-485); F32 attention 1e-4 on the exact route, 1e-2 at head_dim
64 / 128 where the reference itself rounds q, k, v to BF16 (:112,514,676); projections 1e-3
relative exact and 1e-2 relative + 1e-3 from a reduction of 1,024 on, where the reference
uses TF32 (tests/test_cuda_core.c:646-649)."""
from pathlib import Path

import numpy as np
import pytest

import h3_oracle as o

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
REF_CUDA = ROOT / "oracle" / "_ref" / "libh3ref.so"
HIDDEN, HEADS, HEAD_DIM, FFN, ROPE_HALF = 2048, 32, 64, 8192, 24


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


def nf(n, seed, std=1.0):
    return np.random.default_rng(seed).standard_normal(n, dtype=np.float32) * np.float32(std)


def close(got, want, rel, absolute=0.0, what=""):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert np.all(np.isfinite(got)), what
    worst = np.max(np.abs(got - want) - rel * np.maximum(np.abs(want), 1.0))
    assert worst <= absolute, f"{what}: exceeds {rel} relative + {absolute} by {worst:.3e}"


@pytest.mark.parametrize("rows,width", [(3, 8), (3, 5), (1801, HIDDEN), (7, 130), (5, 4100)])
def test_norms_scale_add(gpu, pkg, rows, width):
    n = rows * width
    x, br = nf(n, 1, 3.0), nf(n, 2, 2.0)
    w, b, s = nf(width, 3, 2.0), nf(width, 4), nf(width, 5, 2.0)
    tx, tbr, tw, tb, ts = gpu.f32(x), gpu.f32(br), gpu.f32(w), gpu.f32(b), gpu.f32(s)
    out = gpu.new(n, pkg.F32)
    run(gpu, lambda: gpu.op("rms_norm_f32", out, tx, tw, rows, width, 1e-5))
    close(out.read(), o.rms_norm_f32(x, w, rows, width), 1e-5, what="rms_norm_f32")
    run(gpu, lambda: gpu.op("layer_norm_f32", out, tx, tw, tb, rows, width, 1e-5))
    close(out.read(), o.layer_norm_f32(x, w, b, rows, width), 1e-5, 1e-5, what="layer_norm_f32")
    run(gpu, lambda: gpu.op("scale_add_f32", out, tx, tbr, ts, rows, width))
    close(out.read(), o.scale_add_f32(x, br, s, rows, width), 1e-6, what="scale_add_f32")
    # in place, as the decoder calls it (output aliases the residual)
    run(gpu, lambda: gpu.op("scale_add_f32", tx, tx, tbr, ts, rows, width))
    close(tx.read(), o.scale_add_f32(x, br, s, rows, width), 1e-6, what="scale_add_f32 in place")


@pytest.mark.parametrize("rows,width", [(3, 4), (5, 7), (1801, FFN)])
def test_swiglu_f32(gpu, pkg, rows, width):
    fused = nf(rows * width * 2, 6, 4.0)
    out = gpu.new(rows * width, pkg.F32)
    tf = gpu.f32(fused)
    run(gpu, lambda: gpu.op("swiglu_f32", out, tf, rows, width))
    close(out.read(), o.swiglu_f32(fused, rows, width), 1e-5, what="swiglu_f32")


@pytest.mark.parametrize("seq,heads,hd,half", [(5, 3, 16, 6), (9, 2, 128, 48), (3, 4, 8, 0), (1801, HEADS, HEAD_DIM, ROPE_HALF),
                                               (4, 2, 40, 20)])
def test_video_qkv_rope_f32(gpu, pkg, seq, heads, hd, half):
    n = seq * heads * hd
    qkv, cos, sin = nf(n * 3, 7, 2.0), nf(max(seq * half, 1), 8), nf(max(seq * half, 1), 9)
    t = [gpu.f32(a) for a in (qkv, cos, sin)]
    q, k, v = (gpu.new(n, pkg.F32) for _ in range(3))
    run(gpu, lambda: gpu.op("video_qkv_rope_f32", q, k, v, *t, seq, heads, hd, half, 1e-5))
    wq, wk, wv = o.video_qkv_rope_f32(qkv, cos, sin, seq, heads, hd, half)
    close(q.read(), wq, 1e-5, what="q")
    close(k.read(), wk, 1e-5, what="k")
    assert np.array_equal(v.read().view(np.uint32), wv.view(np.uint32))


def test_video_qkv_rope_rejects_bad_arguments(gpu, pkg):
    n = 4 * 2 * 8
    f = gpu.new(n * 3, pkg.F32)
    h = gpu.new(n * 3, pkg.BF16)
    q, k, v, c, s = (gpu.new(n, pkg.F32) for _ in range(5))
    gpu.begin()
    with pytest.raises(pkg.H3Error):       # BF16 input must fail (tests/test_cuda_attention.c:469-471)
        gpu.op("video_qkv_rope_f32", q, k, v, h, c, s, 4, 2, 8, 2, 1e-5)
    with pytest.raises(pkg.H3Error):       # RoPE wider than the head
        gpu.op("video_qkv_rope_f32", q, k, v, f, c, s, 4, 2, 8, 5, 1e-5)
    gpu.submit()


@pytest.mark.parametrize("seq,heads,hd,rel", [
    (33, 2, 16, 1e-4), (5, 2, 8, 1e-4),                 # exact F32 route (the reference's own shapes)
    (100, 3, 64, 1e-2), (130, 2, 128, 1e-2), (1801, 4, 64, 1e-2),   # BF16 tensor-core route
])
def test_sdpa_f32(gpu, pkg, seq, heads, hd, rel):
    n = seq * heads * hd
    q, k, v = nf(n, 10), nf(n, 11), nf(n, 12)
    t = [gpu.f32(a) for a in (q, k, v)]
    out = gpu.new(n, pkg.F32)
    scale = 1.0 / np.sqrt(hd)
    before = gpu.stats()
    run(gpu, lambda: gpu.op("sdpa_f32", out, *t, seq, heads, hd, scale))
    assert gpu.stats().mps_sdpa_dispatches - before.mps_sdpa_dispatches == 1
    close(out.read(), o.sdpa_f32(q, k, v, seq, heads, hd, scale), rel, what=f"sdpa_f32 {seq}x{heads}x{hd}")


def test_sdpa_f32_exact_switch(gpu, pkg, monkeypatch):
    """H3B_SDPA_F32_EXACT=1 (the reference's H3_CUDA_SDPA_F32_EXACT) keeps head_dim 64 in F32."""
    seq, heads, hd = 200, 2, 64
    n = seq * heads * hd
    q, k, v = nf(n, 13), nf(n, 14), nf(n, 15)
    t = [gpu.f32(a) for a in (q, k, v)]
    out = gpu.new(n, pkg.F32)
    monkeypatch.setenv("H3B_SDPA_F32_EXACT", "1")
    run(gpu, lambda: gpu.op("sdpa_f32", out, *t, seq, heads, hd, 0.125))
    close(out.read(), o.sdpa_f32(q, k, v, seq, heads, hd, 0.125), 1e-4, what="exact sdpa_f32")


@pytest.mark.parametrize("rows,k,n,bias", [
    (5, 7, 9, True), (64, 512, 512, True),                       # exact route (tests/test_cuda_core.c:586-644)
    (64, 2048, 256, True), (300, 2048, 6144, True), (129, 8192, 2048, False), (1801, 2048, 3072, True),
    (40, 1024, 100, True),                                        # 100 columns: the last tile is partial
])
def test_linear_f32(gpu, pkg, rows, k, n, bias):
    x, w = nf(rows * k, 16, 0.5), nf(n * k, 17, 1.0 / np.sqrt(k))
    b = nf(n, 18) if bias else None
    tx, tw = gpu.f32(x), gpu.f32(w)
    tb = gpu.f32(b) if bias else None
    out = gpu.new(rows * n, pkg.F32)
    run(gpu, lambda: gpu.op("linear_f32", out, tx, tw, tb, rows, k, n))
    want = (x.reshape(rows, k).astype(np.float64) @ w.reshape(n, k).astype(np.float64).T
            + (b.astype(np.float64) if bias else 0.0)).reshape(-1)
    if k >= 1024:
        close(out.read(), want, 1e-2, 1e-3, what="linear_f32 (tensor-core route)")
        # FP16 operands rounded to nearest carry 11 significant bits per factor: as a whole the result
        # sits well inside what TF32 (10 bits, truncated) leaves
        assert rel_l2(out.read(), want) < 5e-4
    else:
        close(out.read(), want, 1e-3, what="linear_f32 exact")


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))


def test_linear_f32_rows_of_very_different_magnitude(gpu, pkg):
    """Each row of X and of W is scaled by its own power of two before it is rounded to FP16, so rows
    around 1e-20 and rows around 1e+15 in one call lose nothing (unscaled FP16 spans 6e-8 .. 65,504)."""
    rows, k, n = 96, 1024, 64
    x, w = nf(rows * k, 30).reshape(rows, k), nf(n * k, 31, 1.0 / np.sqrt(k)).reshape(n, k)
    x *= np.float32(10.0) ** np.linspace(-20, 15, rows, dtype=np.float32)[:, None]
    w *= np.float32(10.0) ** np.linspace(-12, 10, n, dtype=np.float32)[:, None]
    tx, tw = gpu.f32(x), gpu.f32(w)
    out = gpu.new(rows * n, pkg.F32)
    run(gpu, lambda: gpu.op("linear_f32", out, tx, tw, None, rows, k, n))
    got = out.read().reshape(rows, n).astype(np.float64)
    want = x.astype(np.float64) @ w.astype(np.float64).T
    assert np.all(np.isfinite(got))
    # against the sum of the products' magnitudes (a dot product itself may cancel to near zero):
    # two factors of 11 significant bits each leave at most 2^-10 of it
    budget = np.abs(x).astype(np.float64) @ np.abs(w).astype(np.float64).T
    assert np.all(np.abs(got - want) <= 2.0 ** -10 * budget), float(np.max(np.abs(got - want) / budget))


def test_linear_f32_forgets_the_weight_rows_when_the_weight_changes(gpu, pkg):
    """A weight tensor created with contents keeps its FP16 rows between calls; writing the tensor
    (host write, device copy, or as an op's output) drops them."""
    rows, k, n = 64, 1024, 128
    x, w1, w2 = nf(rows * k, 32), nf(n * k, 33, 0.03), nf(n * k, 34, 0.03)
    tx, tw, tw2 = gpu.f32(x), gpu.f32(w1), gpu.f32(w2)
    out = gpu.new(rows * n, pkg.F32)

    def product(w):
        return (x.reshape(rows, k).astype(np.float64) @ w.reshape(n, k).astype(np.float64).T).reshape(-1)
    run(gpu, lambda: gpu.op("linear_f32", out, tx, tw, None, rows, k, n))
    assert rel_l2(out.read(), product(w1)) < 5e-4
    run(gpu, lambda: gpu.op("linear_f32", out, tx, tw, None, rows, k, n))          # from the kept rows
    assert rel_l2(out.read(), product(w1)) < 5e-4
    assert gpu.lib.h3_gpu_tensor_write_f32(tw.handle, w2.ctypes.data, w2.size) == 1
    run(gpu, lambda: gpu.op("linear_f32", out, tx, tw, None, rows, k, n))
    assert rel_l2(out.read(), product(w2)) < 5e-4
    run(gpu, lambda: gpu.op("copy_f32", tw, 0, gpu.f32(w1), 0, w1.size))
    run(gpu, lambda: gpu.op("linear_f32", out, tx, tw, None, rows, k, n))
    assert rel_l2(out.read(), product(w1)) < 5e-4
    run(gpu, lambda: gpu.op("scale_add_f32", tw, tw2, tw2, gpu.f32(np.zeros(k, np.float32)), n, k))   # tw = w2
    run(gpu, lambda: gpu.op("linear_f32", out, tx, tw, None, rows, k, n))
    assert rel_l2(out.read(), product(w2)) < 5e-4


@pytest.mark.parametrize("layer", [False, True])
def test_norm_rows_left_for_the_projection_equal_converted_rows(gpu, pkg, layer):
    """A norm leaves its output rows as scaled FP16 beside the F32 result; the projection that
    follows uses them. The same projection on a fresh copy of the F32 result (converted by the
    projection itself) must give the same bits."""
    rows, k, n = 257, 2048, 384
    x, w, b = nf(rows * k, 40, 3.0), nf(k, 41, 0.1) + 1.0, nf(k, 42)
    weight, bias = nf(n * k, 43, 1.0 / np.sqrt(k)), nf(n, 44)
    tx, tw, tb, tweight, tbias = gpu.f32(x), gpu.f32(w), gpu.f32(b), gpu.f32(weight), gpu.f32(bias)
    normed, out_a, out_b = gpu.new(rows * k, pkg.F32), gpu.new(rows * n, pkg.F32), gpu.new(rows * n, pkg.F32)

    def norm():
        if layer:
            gpu.op("layer_norm_f32", normed, tx, tw, tb, rows, k, 1e-5)
        else:
            gpu.op("rms_norm_f32", normed, tx, tw, rows, k, 1e-5)
    run(gpu, lambda: (norm(), gpu.op("linear_f32", out_a, normed, tweight, tbias, rows, k, n)))
    copy = gpu.f32(normed.read())
    run(gpu, lambda: gpu.op("linear_f32", out_b, copy, tweight, tbias, rows, k, n))
    assert np.array_equal(out_a.read().view(np.uint32), out_b.read().view(np.uint32))
    want = o.layer_norm_f32(x, w, b, rows, k) if layer else o.rms_norm_f32(x, w, rows, k)
    close(normed.read(), want, 1e-5, 1e-5, what="norm")
    # writing the normed tensor again drops the rows: the next projection sees the new contents
    run(gpu, lambda: gpu.op("scale_add_f32", normed, normed, normed, gpu.f32(np.ones(k, np.float32)), rows, k))
    run(gpu, lambda: gpu.op("linear_f32", out_a, normed, tweight, tbias, rows, k, n))
    doubled = (2.0 * want.reshape(rows, k).astype(np.float64)) @ weight.reshape(n, k).astype(np.float64).T + bias
    assert rel_l2(out_a.read(), doubled.reshape(-1)) < 5e-4


def decoder_block_weights(seed):
    rng = np.random.default_rng(seed)

    def mat(n, k):
        return (rng.standard_normal(n * k, dtype=np.float32) / np.float32(np.sqrt(k)))

    def vec(n, std=0.02, mean=0.0):
        return rng.standard_normal(n, dtype=np.float32) * np.float32(std) + np.float32(mean)
    inner = HEADS * HEAD_DIM
    return dict(norm1=vec(HIDDEN, 0.1, 1.0), qkv_w=mat(inner * 3, HIDDEN), qkv_b=vec(inner * 3),
                out_w=mat(HIDDEN, inner), out_b=vec(HIDDEN), scale1=vec(HIDDEN, 0.1, 0.5),
                norm2=vec(HIDDEN, 0.1, 1.0), w1=mat(FFN * 2, HIDDEN), w1_b=vec(FFN * 2),
                w2=mat(HIDDEN, FFN), w2_b=vec(HIDDEN), scale2=vec(HIDDEN, 0.1, 0.5))


def run_decoder_block(pkg, gpu, w, hidden, cos, sin, rows):
    """The op sequence of the reference's run_block (h3_video_vae.c:425-461)."""
    inner = HEADS * HEAD_DIM
    t = {name: gpu.f32(value) for name, value in w.items()}
    th, tc, ts = gpu.f32(hidden), gpu.f32(cos), gpu.f32(sin)
    norm, qkv = gpu.new(rows * HIDDEN, pkg.F32), gpu.new(rows * inner * 3, pkg.F32)
    q, k, v, heads = (gpu.new(rows * inner, pkg.F32) for _ in range(4))
    branch, ff1, act = gpu.new(rows * HIDDEN, pkg.F32), gpu.new(rows * FFN * 2, pkg.F32), gpu.new(rows * FFN, pkg.F32)
    gpu.begin()
    gpu.op("rms_norm_f32", norm, th, t["norm1"], rows, HIDDEN, 1e-5)
    gpu.op("linear_f32", qkv, norm, t["qkv_w"], t["qkv_b"], rows, HIDDEN, inner * 3)
    gpu.op("video_qkv_rope_f32", q, k, v, qkv, tc, ts, rows, HEADS, HEAD_DIM, ROPE_HALF, 1e-5)
    gpu.op("sdpa_f32", heads, q, k, v, rows, HEADS, HEAD_DIM, 1.0 / np.sqrt(HEAD_DIM))
    gpu.op("linear_f32", branch, heads, t["out_w"], t["out_b"], rows, inner, HIDDEN)
    gpu.op("scale_add_f32", th, th, branch, t["scale1"], rows, HIDDEN)
    gpu.op("rms_norm_f32", norm, th, t["norm2"], rows, HIDDEN, 1e-5)
    gpu.op("linear_f32", ff1, norm, t["w1"], t["w1_b"], rows, HIDDEN, FFN * 2)
    gpu.op("swiglu_f32", act, ff1, rows, FFN)
    gpu.op("linear_f32", branch, act, t["w2"], t["w2_b"], rows, FFN, HIDDEN)
    gpu.op("scale_add_f32", th, th, branch, t["scale2"], rows, HIDDEN)
    gpu.submit()
    return th.read()


def oracle_decoder_block(w, hidden, cos, sin, rows):
    inner = HEADS * HEAD_DIM
    norm = o.rms_norm_f32(hidden, w["norm1"], rows, HIDDEN)
    qkv = o.linear_f32(norm, w["qkv_w"], w["qkv_b"], rows, HIDDEN, inner * 3)
    q, k, v = o.video_qkv_rope_f32(qkv, cos, sin, rows, HEADS, HEAD_DIM, ROPE_HALF)
    heads = o.sdpa_f32(q, k, v, rows, HEADS, HEAD_DIM, 1.0 / np.sqrt(HEAD_DIM))
    branch = o.linear_f32(heads, w["out_w"], w["out_b"], rows, inner, HIDDEN)
    hidden = o.scale_add_f32(hidden, branch, w["scale1"], rows, HIDDEN)
    norm = o.rms_norm_f32(hidden, w["norm2"], rows, HIDDEN)
    ff1 = o.linear_f32(norm, w["w1"], w["w1_b"], rows, HIDDEN, FFN * 2)
    act = o.swiglu_f32(ff1, rows, FFN)
    branch = o.linear_f32(act, w["w2"], w["w2_b"], rows, FFN, HIDDEN)
    return o.scale_add_f32(hidden, branch, w["scale2"], rows, HIDDEN)


def test_decoder_block_matches_oracle(gpu, pkg):
    """One decoder block at the model's widths on 200 rows against the exact-F32 oracle."""
    rows = 200
    w = decoder_block_weights(3)
    hidden = nf(rows * HIDDEN, 20)
    angle = nf(rows * ROPE_HALF, 21, 2.0)
    cos, sin = np.cos(angle), np.sin(angle)
    got = run_decoder_block(pkg, gpu, w, hidden, cos, sin, rows)
    want = oracle_decoder_block(w, hidden, cos, sin, rows)
    err = rel_l2(got, want)
    print(f"decoder block vs oracle: rel_l2 = {err:.3e}")
    assert err < 3e-3                      # the BF16 rounding of q, k, v in attention is what is left


@pytest.mark.skipif(not REF_CUDA.exists(), reason="reference CUDA backend was not built")
def test_decoder_block_matches_reference_cuda_backend(pkg):
    """A tile's sequence (1,801 rows: 7 x 16 x 16 latent patches + registers + suffix) through one
    decoder block on this library and on the reference's CUDA backend (TF32 projections, BF16
    flash attention). The two differ by their own distances from exact F32."""
    rows = 1801
    w = decoder_block_weights(4)
    hidden = nf(rows * HIDDEN, 22)
    angle = nf(rows * ROPE_HALF, 23, 2.0)
    cos, sin = np.cos(angle), np.sin(angle)
    out = {}
    for name, path in (("b200", None), ("reference", REF_CUDA)):
        gpu = pkg.Gpu(0, lib_path=path)
        try:
            out[name] = run_decoder_block(pkg, gpu, w, hidden, cos, sin, rows)
        finally:
            gpu.close()
    err = rel_l2(out["b200"], out["reference"])
    print(f"decoder block, 1801 rows: this library vs reference CUDA backend rel_l2 = {err:.3e}")
    assert err < 5e-3
