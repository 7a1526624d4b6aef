"""Pins the CPU oracle (oracle/h3_oracle.c) against the reference's own CPU test
references, compiled in place from the reference tree into oracle/_ref/libh3refcpu.so.

The comparison is bit-exact: both sides are compiled with the same flags and follow
the same summation order. Skipped where the reference-derived library was not built
(the committed golden vectors in tests/golden/ then carry the pin)."""
import ctypes as C

import numpy as np
import pytest

import h3_oracle as o

ref = o.ref_cpu()
pytestmark = pytest.mark.skipif(ref is None, reason="oracle/_ref/libh3refcpu.so not built")

u32, f32 = C.c_uint32, C.c_float


def p(a):
    return a.ctypes.data_as(C.c_void_p)


def rnd_bf16(n, seed, std=1.0):
    return o.normal_bf16(n, seed, 0.0, std)


def test_bf16_conversion_matches_reference():
    ref.refcpu_f32_to_bf16.restype = C.c_uint16
    ref.refcpu_f32_to_bf16.argtypes = [f32]
    x = o.normal_f32(4096, 11, 0.0, 3.0)
    x[:8] = [0.0, -0.0, 1.0, 1.00390625, 1.001953125, 3.3895314e38, 1e-40, -2.5]
    ours = o.to_bf16(x)
    theirs = np.array([ref.refcpu_f32_to_bf16(float(v)) for v in x], np.uint16)
    assert np.array_equal(ours, theirs)


def test_rng_matches_reference_host():
    class Rng(C.Structure):
        _fields_ = [("state", C.c_uint64), ("increment", C.c_uint64), ("spare", f32),
                    ("has_spare", C.c_int)]
    for seed in (0, 1, 7, 42, 2**40 + 5):
        r = Rng()
        ref.h3_rng_seed(C.byref(r), C.c_uint64(seed))
        theirs = np.empty(1001, np.float32)
        ref.h3_rng_fill_normal(C.byref(r), p(theirs), C.c_size_t(theirs.size))
        ours = o.normal_f32(theirs.size, seed)
        assert np.array_equal(ours.view(np.uint32), theirs.view(np.uint32))


@pytest.mark.parametrize("rows,width,slots", [(4, 8, 3), (7, 5376, 6), (33, 130, 6)])
def test_adaln_and_gate(rows, width, slots):
    mod_rows = 5
    x = rnd_bf16(rows * width, 1, 3.0)
    w = rnd_bf16(width, 2, 2.0)
    mod = rnd_bf16(mod_rows * slots * width, 3)
    br = rnd_bf16(rows * width, 4, 3.0)
    row_map = (np.arange(rows, dtype=np.uint32) * 3 + 1) % mod_rows
    fx, fw, fmod, fbr = map(o.from_bf16, (x, w, mod, br))
    theirs = np.empty(rows * width, np.float32)
    ref.refcpu_adaln(p(fx), p(fw), p(fmod), p(row_map), p(theirs), u32(rows), u32(width),
                     u32(slots), u32(0), u32(1), f32(1e-5))
    ours = o.adaln_bf16(x, w, mod, row_map, rows, width, slots, 0, 1)
    assert np.array_equal(ours, o.to_bf16(theirs))
    assert np.array_equal(o.adaln_f32(fx, fw, fmod, row_map, rows, width, slots, 0, 1).view(np.uint32),
                          theirs.view(np.uint32))
    ref.refcpu_gate(p(fx), p(fbr), p(fmod), p(row_map), p(theirs), u32(rows), u32(width),
                    u32(slots), u32(2))
    assert np.array_equal(o.gate_bf16(x, br, mod, row_map, rows, width, slots, 2), o.to_bf16(theirs))
    # fused gate + adaLN == gate, round, adaLN of the rounded row (test_cuda_dit.c:395-416)
    gated, out = o.gate_adaln_bf16(x, br, w, mod, mod, row_map, rows, width, slots, 2, 0, 1)
    assert np.array_equal(gated, o.to_bf16(theirs))
    fg = o.from_bf16(gated)
    ref.refcpu_adaln(p(fg), p(fw), p(fmod), p(row_map), p(theirs), u32(rows), u32(width),
                     u32(slots), u32(0), u32(1), f32(1e-5))
    assert np.array_equal(out, o.to_bf16(theirs))


@pytest.mark.parametrize("rows,k,n,bias", [(5, 7, 9, True), (5, 7, 9, False), (70, 256, 130, True)])
def test_linear(rows, k, n, bias):
    x, w = rnd_bf16(rows * k, 5), rnd_bf16(n * k, 6, 0.5)
    b = rnd_bf16(n, 7) if bias else None
    fx, fw = o.from_bf16(x), o.from_bf16(w)
    fb = o.from_bf16(b) if bias else None
    theirs = np.empty(rows * n, np.float32)
    ref.refcpu_linear_f32(p(fx), p(fw), p(fb) if bias else None, p(theirs), u32(rows), u32(k), u32(n))
    assert np.array_equal(o.linear_bf16(x, w, b, rows, k, n), o.to_bf16(theirs))
    assert np.array_equal(o.linear_f32(fx, fw, fb, rows, k, n).view(np.uint32), theirs.view(np.uint32))


def test_swiglu_and_silu():
    rows, width = 6, 50
    fused = rnd_bf16(rows * width * 2, 8, 4.0)
    theirs = np.empty(rows * width, np.float32)
    ref.refcpu_swiglu(p(o.from_bf16(fused)), p(theirs), u32(rows), u32(width))
    assert np.array_equal(o.swiglu_bf16(fused, rows, width), o.to_bf16(theirs))
    ref.refcpu_silu.restype = f32
    ref.refcpu_silu.argtypes = [f32]
    x = o.normal_f32(300, 9, 0.0, 4.0)
    assert np.array_equal(o.silu_f32(x), np.array([ref.refcpu_silu(float(v)) for v in x], np.float32))


@pytest.mark.parametrize("grouped", [0, 1])
@pytest.mark.parametrize("seq,heads,hd,half", [(5, 3, 16, 6), (9, 2, 128, 48), (3, 4, 8, 0)])
def test_qkv_rope(seq, heads, hd, half, grouped):
    qkv = rnd_bf16(seq * heads * hd * 3, 10, 2.0)
    qw, kw = rnd_bf16(hd, 11), rnd_bf16(hd, 12)
    cos, sin = rnd_bf16(max(seq * half, 1), 13), rnd_bf16(max(seq * half, 1), 14)
    n = seq * heads * hd
    tq, tk, tv = (np.empty(n, np.float32) for _ in range(3))
    ref.refcpu_qkv_rope(p(o.from_bf16(qkv)), p(o.from_bf16(qw)), p(o.from_bf16(kw)),
                        p(o.from_bf16(cos)), p(o.from_bf16(sin)), p(tq), p(tk), p(tv), u32(seq),
                        u32(heads), u32(hd), u32(half), C.c_int(grouped), C.c_int(1), f32(1e-5))
    q, k, v = o.qkv_rope_bf16(qkv, qw, kw, cos, sin, seq, heads, hd, half, grouped)
    assert np.array_equal(q, o.to_bf16(tq))
    assert np.array_equal(k, o.to_bf16(tk))
    assert np.array_equal(v, o.to_bf16(tv))


@pytest.mark.parametrize("head_major", [0, 1])
@pytest.mark.parametrize("seq,heads,hd", [(5, 2, 8), (100, 3, 64), (130, 2, 128)])
def test_sdpa(seq, heads, hd, head_major):
    n = seq * heads * hd
    q, k, v = rnd_bf16(n, 15), rnd_bf16(n, 16), rnd_bf16(n, 17)
    theirs = np.empty(n, np.float32)
    scale = 1.0 / np.sqrt(hd)
    ref.refcpu_sdpa(p(o.from_bf16(q)), p(o.from_bf16(k)), p(o.from_bf16(v)), p(theirs), u32(1),
                    u32(seq), u32(heads), u32(hd), f32(scale), C.c_int(0), C.c_int(head_major))
    ours = o.sdpa_bf16(q, k, v, seq, heads, hd, scale, head_major, round_p=0)
    assert np.array_equal(ours, o.to_bf16(theirs))
    # the tensor-core rounding boundary (P rounded to BF16) stays inside the reference's
    # own flash tolerance 1e-3 + 1e-2*|ref| (tests/test_cuda_attention.c:112-114)
    rounded = o.from_bf16(o.sdpa_bf16(q, k, v, seq, heads, hd, scale, head_major, round_p=1))
    assert np.all(np.abs(rounded - theirs) <= 1e-3 + 1e-2 * np.abs(theirs))


# ---- F32 operations of the video-VAE decoder ---------------------------------------------

def bits(a):
    return np.asarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("rows,width", [(3, 8), (5, 2048), (2, 130)])
def test_f32_norms(rows, width):
    x, w, b = o.normal_f32(rows * width, 41, 0.0, 3.0), o.normal_f32(width, 42, 0.0, 2.0), o.normal_f32(width, 43)
    theirs = np.empty(rows * width, np.float32)
    ref.refcpu_rms_norm(p(x), p(w), p(theirs), u32(rows), u32(width), f32(1e-5))
    assert np.array_equal(bits(o.rms_norm_f32(x, w, rows, width)), bits(theirs))
    ref.refcpu_layer_norm(p(x), p(w), p(b), p(theirs), u32(rows), u32(width), f32(1e-5))
    assert np.array_equal(bits(o.layer_norm_f32(x, w, b, rows, width)), bits(theirs))


def test_f32_swiglu():
    rows, width = 4, 96
    fused = o.normal_f32(rows * width * 2, 44, 0.0, 4.0)
    theirs = np.empty(rows * width, np.float32)
    ref.refcpu_swiglu(p(fused), p(theirs), u32(rows), u32(width))
    assert np.array_equal(bits(o.swiglu_f32(fused, rows, width)), bits(theirs))


@pytest.mark.parametrize("seq,heads,hd,half", [(5, 3, 16, 6), (4, 32, 64, 24), (3, 2, 8, 0)])
def test_video_qkv_rope_f32(seq, heads, hd, half):
    qkv = o.normal_f32(seq * heads * hd * 3, 45, 0.0, 2.0)
    cos, sin = o.normal_f32(max(seq * half, 1), 46), o.normal_f32(max(seq * half, 1), 47)
    n = seq * heads * hd
    tq, tk, tv = (np.empty(n, np.float32) for _ in range(3))
    ref.refcpu_qkv_rope(p(qkv), None, None, p(cos), p(sin), p(tq), p(tk), p(tv), u32(seq), u32(heads),
                        u32(hd), u32(half), C.c_int(1), C.c_int(0), f32(1e-5))
    q, k, v = o.video_qkv_rope_f32(qkv, cos, sin, seq, heads, hd, half)
    assert np.array_equal(bits(q), bits(tq)) and np.array_equal(bits(k), bits(tk))
    assert np.array_equal(bits(v), bits(tv))


@pytest.mark.parametrize("seq,heads,hd", [(5, 2, 8), (100, 3, 64)])
def test_sdpa_f32(seq, heads, hd):
    n = seq * heads * hd
    q, k, v = o.normal_f32(n, 48), o.normal_f32(n, 49), o.normal_f32(n, 50)
    theirs = np.empty(n, np.float32)
    ref.refcpu_sdpa(p(q), p(k), p(v), p(theirs), u32(1), u32(seq), u32(heads), u32(hd), f32(0.7), C.c_int(0),
                    C.c_int(0))
    assert np.array_equal(bits(o.sdpa_f32(q, k, v, seq, heads, hd, 0.7)), bits(theirs))
