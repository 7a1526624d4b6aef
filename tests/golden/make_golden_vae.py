#!/usr/bin/env python3
"""Generate tests/golden/ref_cpu_vectors_vae.npz from the reference's OWN CPU code: the F32
operations of the video-VAE decoder's transformer (h3_video_vae.c:425-461).

Run where the reference tree is available, after `python oracle/build_ref.py --no-cuda`:

    python tests/golden/make_golden_vae.py

Every output array is produced by a CPU reference function of the reference's CUDA test programs
(tests/test_cuda_core.c ref_rms_norm / ref_layer_norm / ref_swiglu / ref_linear_f32,
tests/test_cuda_attention.c ref_qkv_rope with weighted = 0 / ref_sdpa) called through
oracle/_ref/libh3refcpu.so; scale-add has no function of its own there and is the test's inline
expression residual + branch * scale (tests/test_cuda_core.c:296-299), evaluated in numpy F32.
Inputs are seeded with the reference's host RNG. Shapes: the decoder's widths (hidden 2048,
32 heads x 64, rope_half 24) on a few rows.
"""
import ctypes as C
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "oracle"))
import h3_oracle as o  # noqa: E402  (only the ctypes handle of the reference-derived library is used)

u32, f32 = C.c_uint32, C.c_float


def p(a):
    return a.ctypes.data_as(C.c_void_p)


class Rng(C.Structure):
    _fields_ = [("state", C.c_uint64), ("increment", C.c_uint64), ("spare", f32), ("has_spare", C.c_int)]


def main():
    ref = o.ref_cpu()
    if ref is None:
        raise SystemExit("oracle/_ref/libh3refcpu.so is missing: run oracle/build_ref.py first")

    def normal(n, seed, std=1.0):
        r = Rng()
        ref.h3_rng_seed(C.byref(r), C.c_uint64(seed))
        out = np.empty(n, np.float32)
        ref.h3_rng_fill_normal(C.byref(r), p(out), C.c_size_t(n))
        return out * np.float32(std)

    g = {}
    rows, width = 3, 2048
    x, w, b = normal(rows * width, 21, 3.0), normal(width, 22, 2.0), normal(width, 23)
    out = np.empty(rows * width, np.float32)
    ref.refcpu_rms_norm(p(x), p(w), p(out), u32(rows), u32(width), f32(1e-5))
    g.update(norm_x=x, norm_w=w, norm_b=b, rms_out=out.copy())
    ref.refcpu_layer_norm(p(x), p(w), p(b), p(out), u32(rows), u32(width), f32(1e-5))
    g["layer_out"] = out.copy()

    branch, scale = normal(rows * width, 24, 2.0), normal(width, 25, 2.0)
    g.update(scale_add_branch=branch, scale_add_scale=scale,
             scale_add_out=(x.reshape(rows, width) + branch.reshape(rows, width) * scale).reshape(-1))

    rows, width = 3, 2048
    fused = normal(rows * width * 2, 26, 4.0)
    out = np.empty(rows * width, np.float32)
    ref.refcpu_swiglu(p(fused), p(out), u32(rows), u32(width))
    g.update(swiglu_in=fused, swiglu_out=out.copy())

    seq, heads, hd, half = 7, 8, 64, 24
    qkv = normal(seq * heads * hd * 3, 27, 2.0)
    cos, sin = normal(seq * half, 28), normal(seq * half, 29)
    q, k, v = (np.empty(seq * heads * hd, np.float32) for _ in range(3))
    ref.refcpu_qkv_rope(p(qkv), None, None, p(cos), p(sin), p(q), p(k), p(v), u32(seq), u32(heads), u32(hd),
                        u32(half), C.c_int(1), C.c_int(0), f32(1e-5))
    g.update(rope_qkv=qkv, rope_cos=cos, rope_sin=sin, rope_q=q.copy(), rope_k=k.copy(), rope_v=v.copy())

    seq, heads, hd = 70, 2, 64
    n = seq * heads * hd
    q, k, v = normal(n, 30), normal(n, 31), normal(n, 32)
    out = np.empty(n, np.float32)
    ref.refcpu_sdpa(p(q), p(k), p(v), p(out), u32(1), u32(seq), u32(heads), u32(hd), f32(0.125), C.c_int(0),
                    C.c_int(0))
    g.update(sdpa_q=q, sdpa_k=k, sdpa_v=v, sdpa_out=out.copy(), sdpa_shape=np.array([seq, heads, hd], np.uint32))

    rows, k_dim, n_dim = 8, 2048, 24
    x, w, b = normal(rows * k_dim, 33, 0.5), normal(n_dim * k_dim, 34, 0.05), normal(n_dim, 35)
    out = np.empty(rows * n_dim, np.float32)
    ref.refcpu_linear_f32(p(x), p(w), p(b), p(out), u32(rows), u32(k_dim), u32(n_dim))
    g.update(linear_x=x, linear_w=w, linear_b=b, linear_out=out.copy())

    path = Path(__file__).with_name("ref_cpu_vectors_vae.npz")
    np.savez_compressed(path, **g)
    print(f"wrote {path} ({path.stat().st_size / 1024:.0f} KiB, {len(g)} arrays)")


if __name__ == "__main__":
    main()
