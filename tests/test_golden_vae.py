"""Golden vectors of the video-VAE decoder's F32 operations, produced by the reference's own CPU
test references (tests/golden/make_golden_vae.py).

CPU part: the oracle reproduces them bit for bit (the pin that travels to machines without the
reference tree). GPU part: libh3b200.so matches them within the reference's own per-op tolerances
(tests/test_cuda_core.c: 1e-5 for the row ops; tests/test_cuda_attention.c: 1e-5 for the
QKV split, 1e-2 for F32 attention at head_dim 64, which the reference also runs in BF16;
1e-2 relative + 1e-3 for a projection with a reduction >= 1024, the reference's TF32 bar,
tests/test_cuda_core.c:646-649)."""
from pathlib import Path

import numpy as np
import pytest

import h3_oracle as o

G = np.load(Path(__file__).parent / "golden" / "ref_cpu_vectors_vae.npz")
ROWS, WIDTH = 3, 2048


def same_bits(a, b):
    return np.array_equal(np.asarray(a, np.float32).view(np.uint32), np.asarray(b, np.float32).view(np.uint32))


def test_norms_golden():
    assert same_bits(o.rms_norm_f32(G["norm_x"], G["norm_w"], ROWS, WIDTH), G["rms_out"])
    assert same_bits(o.layer_norm_f32(G["norm_x"], G["norm_w"], G["norm_b"], ROWS, WIDTH), G["layer_out"])


def test_scale_add_and_swiglu_golden():
    assert same_bits(o.scale_add_f32(G["norm_x"], G["scale_add_branch"], G["scale_add_scale"], ROWS, WIDTH),
                     G["scale_add_out"])
    assert same_bits(o.swiglu_f32(G["swiglu_in"], ROWS, WIDTH), G["swiglu_out"])


def test_video_qkv_rope_golden():
    q, k, v = o.video_qkv_rope_f32(G["rope_qkv"], G["rope_cos"], G["rope_sin"], 7, 8, 64, 24)
    assert same_bits(q, G["rope_q"]) and same_bits(k, G["rope_k"]) and same_bits(v, G["rope_v"])


def test_sdpa_and_linear_golden():
    seq, heads, hd = (int(x) for x in G["sdpa_shape"])
    assert same_bits(o.sdpa_f32(G["sdpa_q"], G["sdpa_k"], G["sdpa_v"], seq, heads, hd, 0.125), G["sdpa_out"])
    assert same_bits(o.linear_f32(G["linear_x"], G["linear_w"], G["linear_b"], 8, 2048, 24), G["linear_out"])


@pytest.fixture(scope="module")
def gpu():
    import __graft_entry__ as entry
    pkg = entry.load_package()
    g = pkg.Gpu(0)
    yield g, pkg
    g.close()


def close(got, want, rel, absolute=0.0):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert np.all(np.isfinite(got))
    assert np.all(np.abs(got - want) <= absolute + rel * np.maximum(np.abs(want), 1.0)), \
        float(np.max(np.abs(got - want)))


@pytest.mark.gpu
def test_gpu_matches_golden(gpu):
    g, pkg = gpu
    n = ROWS * WIDTH
    x, w, b = g.f32(G["norm_x"]), g.f32(G["norm_w"]), g.f32(G["norm_b"])
    out = g.new(n, pkg.F32)
    g.begin(); g.op("rms_norm_f32", out, x, w, ROWS, WIDTH, 1e-5); g.submit()
    close(out.read(), G["rms_out"], 1e-5)
    g.begin(); g.op("layer_norm_f32", out, x, w, b, ROWS, WIDTH, 1e-5); g.submit()
    close(out.read(), G["layer_out"], 1e-5)
    branch, scale = g.f32(G["scale_add_branch"]), g.f32(G["scale_add_scale"])
    g.begin(); g.op("scale_add_f32", out, x, branch, scale, ROWS, WIDTH); g.submit()
    close(out.read(), G["scale_add_out"], 1e-6)
    fused = g.f32(G["swiglu_in"])
    g.begin(); g.op("swiglu_f32", out, fused, ROWS, WIDTH); g.submit()
    close(out.read(), G["swiglu_out"], 1e-5)
    qkv, cos, sin = g.f32(G["rope_qkv"]), g.f32(G["rope_cos"]), g.f32(G["rope_sin"])
    q, k, v = (g.new(7 * 8 * 64, pkg.F32) for _ in range(3))
    g.begin(); g.op("video_qkv_rope_f32", q, k, v, qkv, cos, sin, 7, 8, 64, 24, 1e-5); g.submit()
    close(q.read(), G["rope_q"], 1e-5); close(k.read(), G["rope_k"], 1e-5)
    assert same_bits(v.read(), G["rope_v"])
    seq, heads, hd = (int(s) for s in G["sdpa_shape"])
    tq, tk, tv = g.f32(G["sdpa_q"]), g.f32(G["sdpa_k"]), g.f32(G["sdpa_v"])
    to = g.new(seq * heads * hd, pkg.F32)
    g.begin(); g.op("sdpa_f32", to, tq, tk, tv, seq, heads, hd, 0.125); g.submit()
    close(to.read(), G["sdpa_out"], 1e-2)
    lx, lw, lb = g.f32(G["linear_x"]), g.f32(G["linear_w"]), g.f32(G["linear_b"])
    lo = g.new(8 * 24, pkg.F32)
    g.begin(); g.op("linear_f32", lo, lx, lw, lb, 8, 2048, 24); g.submit()
    close(lo.read(), G["linear_out"], 1e-2, 1e-3)
