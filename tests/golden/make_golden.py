#!/usr/bin/env python3
"""Generate tests/golden/ref_cpu_vectors.npz from the reference's OWN CPU code.

Run where the reference tree is available (H3_REFERENCE_DIR, default: a directory named
"reference" beside the repository):

    python oracle/build_ref.py --no-cuda      # compiles the reference's test references in place
    python tests/golden/make_golden.py

Every output array below is produced by a function of the reference itself - the CPU
reference functions of its CUDA test programs (tests/test_cuda_dit.c ref_adaln / ref_gate,
tests/test_cuda_attention.c ref_qkv_rope / ref_sdpa, tests/test_cuda_core.c ref_linear_f32 /
ref_swiglu / ref_silu) and its host RNG (h3_host.c h3_rng_*) - called through
oracle/_ref/libh3refcpu.so. Inputs are seeded with that same RNG. The vectors travel with the
repository so that machines without the reference tree can still pin the oracle and the CUDA
kernels to the reference's arithmetic.
"""
import ctypes as C
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "oracle"))
import h3_oracle as o  # noqa: E402  (only its bf16 helpers and the ctypes handle are used)

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

    def bf(n, seed, std=1.0):      # BF16-representable F32 values, as the reference tests use
        return o.from_bf16(o.to_bf16(normal(n, seed, std)))

    g = {}
    for seed in (0, 7, 42):
        g[f"rng_normal_seed{seed}"] = normal(256, seed)

    # adaLN / gate at the model width
    rows, width, slots, mod_rows = 6, 5376, 6, 4
    x, br = bf(rows * width, 1, 3.0), bf(rows * width, 2, 3.0)
    w, mod = bf(width, 3, 2.0), bf(mod_rows * slots * width, 4)
    row_map = np.array([2, 0, 3, 1, 1, 2], np.uint32)
    out = np.empty(rows * width, np.float32)
    ref.refcpu_adaln(p(x), p(w), p(mod), p(row_map), p(out), u32(rows), u32(width), u32(slots), u32(0),
                     u32(1), f32(1e-5))
    g.update(adaln_x=o.to_bf16(x), adaln_w=o.to_bf16(w), adaln_mod=o.to_bf16(mod), adaln_row_map=row_map,
             adaln_out=out.copy(), adaln_br=o.to_bf16(br))
    ref.refcpu_gate(p(x), p(br), p(mod), p(row_map), p(out), u32(rows), u32(width), u32(slots), u32(2))
    g["gate_out"] = out.copy()

    # linear (sequential fmaf from the bias)
    rows, k, n = 40, 512, 136
    x, w, b = bf(rows * k, 5), bf(n * k, 6, 0.05), bf(n, 7)
    out = np.empty(rows * n, np.float32)
    ref.refcpu_linear_f32(p(x), p(w), p(b), p(out), u32(rows), u32(k), u32(n))
    g.update(linear_x=o.to_bf16(x), linear_w=o.to_bf16(w), linear_b=o.to_bf16(b), linear_out=out.copy())

    # SwiGLU
    rows, width = 5, 96
    fused = bf(rows * width * 2, 8, 4.0)
    out = np.empty(rows * width, np.float32)
    ref.refcpu_swiglu(p(fused), p(out), u32(rows), u32(width))
    g.update(swiglu_in=o.to_bf16(fused), swiglu_out=out.copy())

    # grouped QKV split + RMSNorm + RoPE at head_dim 128 / half 48
    seq, heads, hd, half = 12, 3, 128, 48
    qkv = bf(seq * heads * hd * 3, 9, 2.0)
    qw, kw = bf(hd, 10), bf(hd, 11)
    cos, sin = bf(seq * half, 12), bf(seq * half, 13)
    q, kk, v = (np.empty(seq * heads * hd, np.float32) for _ in range(3))
    ref.refcpu_qkv_rope(p(qkv), p(qw), p(kw), p(cos), p(sin), p(q), p(kk), p(v), u32(seq), u32(heads),
                        u32(hd), u32(half), C.c_int(1), C.c_int(1), f32(1e-5))
    g.update(rope_qkv=o.to_bf16(qkv), rope_qw=o.to_bf16(qw), rope_kw=o.to_bf16(kw), rope_cos=o.to_bf16(cos),
             rope_sin=o.to_bf16(sin), rope_q=q.copy(), rope_k=kk.copy(), rope_v=v.copy())

    # joint attention: the reference's own test shapes S=100 (hd 64) and S=130 (hd 128)
    for tag, (seq, heads, hd) in {"a": (100, 2, 64), "b": (130, 2, 128)}.items():
        n = seq * heads * hd
        q, kk, v = bf(n, 14), bf(n, 15), bf(n, 16)
        out = np.empty(n, np.float32)
        ref.refcpu_sdpa(p(q), p(kk), p(v), p(out), u32(1), u32(seq), u32(heads), u32(hd),
                        f32(1.0 / np.sqrt(hd)), C.c_int(0), C.c_int(0))
        g.update({f"sdpa_{tag}_q": o.to_bf16(q), f"sdpa_{tag}_k": o.to_bf16(kk), f"sdpa_{tag}_v": o.to_bf16(v),
                  f"sdpa_{tag}_out": out.copy(), f"sdpa_{tag}_shape": np.array([seq, heads, hd], np.uint32)})

    path = Path(__file__).with_name("ref_cpu_vectors.npz")
    np.savez_compressed(path, **g)
    print(f"wrote {path} ({path.stat().st_size / 1024:.0f} KiB, {len(g)} arrays)")


if __name__ == "__main__":
    main()
