"""ctypes binding of the CPU oracle (oracle/libh3oracle.so) and, where it was built,
of the reference's own CPU test references (oracle/_ref/libh3refcpu.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the benchmark's
CPU-baseline leg, never by the shipped library or its Python host layer.

All BF16 tensors are numpy uint16 arrays holding raw bits.
"""
from __future__ import annotations

import ctypes as C
import subprocess
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_LIB = None
_REF = None

u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
u32 = C.c_uint32
f32 = C.c_float


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = HERE / "libh3oracle.so"
        if not path.exists():
            subprocess.run([sys.executable, str(HERE / "build_ref.py"), "--no-cuda"], check=True)
        _LIB = C.CDLL(str(path))
        _LIB.h3o_threads.restype = C.c_int
        _LIB.h3o_named_seed.restype = C.c_uint64
        _LIB.h3o_named_seed.argtypes = [C.c_uint64, C.c_char_p]
    return _LIB


def ref_cpu() -> C.CDLL | None:
    """The reference's own CPU references, or None where they were not built."""
    global _REF
    if _REF is None:
        path = HERE / "_ref" / "libh3refcpu.so"
        if not path.exists():
            return None
        _REF = C.CDLL(str(path))
    return _REF


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def threads() -> int:
    return lib().h3o_threads()


def set_threads(count: int) -> None:
    """Use `count` OpenMP threads from now on (torch.distributed.run exports OMP_NUM_THREADS=1)."""
    lib().h3o_set_threads(int(count))


# ----------------------------------------------------------------- bf16
def to_bf16(x: np.ndarray) -> np.ndarray:
    """F32 -> raw BF16 bits, round to nearest even (reference formula)."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    bits = bits + 0x7FFF + ((bits >> 16) & 1)
    return ((bits >> 16) & 0xFFFF).astype(np.uint16)


def from_bf16(x: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(x, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ------------------------------------------------------------------ rng
def named_seed(seed: int, name: str) -> int:
    return int(lib().h3o_named_seed(C.c_uint64(seed), name.encode()))


def normal_f32(count: int, seed: int, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    out = np.empty(count, np.float32)
    lib().h3o_fill_normal_f32(_p(out), C.c_size_t(count), C.c_uint64(seed), f32(mean), f32(std))
    return out


def normal_bf16(count: int, seed: int, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    out = np.empty(count, np.uint16)
    lib().h3o_fill_normal_bf16(_p(out), C.c_size_t(count), C.c_uint64(seed), f32(mean), f32(std))
    return out


# ------------------------------------------------------------------ ops
def linear_bf16(x, w, bias, rows, in_dim, out_dim):
    out = np.empty(rows * out_dim, np.uint16)
    lib().h3o_linear_bf16(_p(out), _p(x), _p(w), _p(bias), u32(rows), u32(in_dim), u32(out_dim))
    return out


def linear_f32(x, w, bias, rows, in_dim, out_dim):
    out = np.empty(rows * out_dim, np.float32)
    lib().h3o_linear_f32(_p(out), _p(x), _p(w), _p(bias), u32(rows), u32(in_dim), u32(out_dim))
    return out


def swiglu_bf16(fused, rows, width):
    out = np.empty(rows * width, np.uint16)
    lib().h3o_swiglu_bf16(_p(out), _p(fused), u32(rows), u32(width))
    return out


def silu_bf16(x):
    out = np.empty_like(x)
    lib().h3o_silu_bf16(_p(out), _p(x), C.c_size_t(x.size))
    return out


def silu_f32(x):
    out = np.empty_like(x)
    lib().h3o_silu_f32(_p(out), _p(x), C.c_size_t(x.size))
    return out


def add_bf16(a, b):
    out = np.empty_like(a)
    lib().h3o_add_bf16(_p(out), _p(a), _p(b), C.c_size_t(a.size))
    return out


def sub_bf16(a, b):
    out = np.empty_like(a)
    lib().h3o_sub_bf16(_p(out), _p(a), _p(b), C.c_size_t(a.size))
    return out


def mlp_bf16(x, fc1, fc2, rows, in_dim, hidden, out_dim):
    out = np.empty(rows * out_dim, np.uint16)
    lib().h3o_mlp_bf16(_p(out), _p(x), _p(fc1), _p(fc2), u32(rows), u32(in_dim), u32(hidden),
                       u32(out_dim))
    return out


def adaln_bf16(x, norm, mod, row_map, rows, width, slots, shift, scale, eps=1e-5):
    out = np.empty(rows * width, np.uint16)
    lib().h3o_adaln_bf16(_p(out), _p(x), _p(norm), _p(mod), _p(row_map), u32(rows), u32(width),
                         u32(slots), u32(shift), u32(scale), f32(eps))
    return out


def adaln_f32(x, norm, mod, row_map, rows, width, slots, shift, scale, eps=1e-5):
    out = np.empty(rows * width, np.float32)
    lib().h3o_adaln_f32(_p(out), _p(x), _p(norm), _p(mod), _p(row_map), u32(rows), u32(width),
                        u32(slots), u32(shift), u32(scale), f32(eps))
    return out


def rms_norm_bf16(x, norm, rows, width, eps=1e-5):
    out = np.empty(rows * width, np.uint16)
    lib().h3o_rms_norm_bf16(_p(out), _p(x), _p(norm), u32(rows), u32(width), f32(eps))
    return out


def gate_bf16(res, branch, mod, row_map, rows, width, slots, gate):
    out = np.empty(rows * width, np.uint16)
    lib().h3o_gate_bf16(_p(out), _p(res), _p(branch), _p(mod), _p(row_map), u32(rows), u32(width),
                        u32(slots), u32(gate))
    return out


def gate_f32(res, branch, mod, row_map, rows, width, slots, gate):
    out = np.empty(rows * width, np.float32)
    lib().h3o_gate_f32(_p(out), _p(res), _p(branch), _p(mod), _p(row_map), u32(rows), u32(width),
                       u32(slots), u32(gate))
    return out


def gate_adaln_bf16(res, branch, norm, gate_mod, norm_mod, row_map, rows, width, slots, gate,
                    shift, scale, eps=1e-5):
    gated = np.empty(rows * width, np.uint16)
    out = np.empty(rows * width, np.uint16)
    lib().h3o_gate_adaln_bf16(_p(gated), _p(out), _p(res), _p(branch), _p(norm), _p(gate_mod),
                              _p(norm_mod), _p(row_map), u32(rows), u32(width), u32(slots),
                              u32(gate), u32(shift), u32(scale), f32(eps))
    return gated, out


def adaln_linear_bf16(x, norm, mod, row_map, weight, bias, rows, width, out_dim, slots, shift,
                      scale, eps=1e-5):
    out = np.empty(rows * out_dim, np.uint16)
    inverse = np.empty(rows, np.float32)
    lib().h3o_adaln_linear_bf16(_p(out), _p(inverse), _p(x), _p(norm), _p(mod), _p(row_map),
                                _p(weight), _p(bias), u32(rows), u32(width), u32(out_dim),
                                u32(slots), u32(shift), u32(scale), f32(eps))
    return out, inverse


def qkv_rope_bf16(qkv, q_norm, k_norm, cos, sin, seq, heads, hd, rope_half, grouped=1, eps=1e-5):
    n = seq * heads * hd
    q, k, v = (np.empty(n, np.uint16) for _ in range(3))
    lib().h3o_qkv_rope_bf16(_p(q), _p(k), _p(v), _p(qkv), _p(q_norm), _p(k_norm), _p(cos), _p(sin),
                            u32(seq), u32(heads), u32(hd), u32(rope_half), C.c_int(grouped),
                            f32(eps))
    return q, k, v


def sdpa_bf16(q, k, v, seq, heads, hd, scale, head_major=0, round_p=0, rows=None):
    out = np.zeros(seq * heads * hd, np.uint16)
    begin, end = (0, seq) if rows is None else rows
    lib().h3o_sdpa_bf16_rows(_p(out), _p(q), _p(k), _p(v), u32(seq), u32(heads), u32(hd),
                             f32(scale), C.c_int(head_major), C.c_int(round_p), u32(begin),
                             u32(end))
    return out


def sdpa_bf16_sparse(q, k, v, seq, heads, hd, scale, sparse_ptr, sparse_idx, head_major=0, round_p=0):
    out = np.empty(seq * heads * hd, np.uint16)
    ptr = np.ascontiguousarray(sparse_ptr, np.uint32)
    idx = np.ascontiguousarray(sparse_idx, np.uint32)
    lib().h3o_sdpa_bf16_sparse(_p(out), _p(q), _p(k), _p(v), u32(seq), u32(heads), u32(hd),
                               f32(scale), C.c_int(head_major), C.c_int(round_p), _p(ptr), _p(idx))
    return out


def rms_norm_f32(x, weight, rows, width, eps=1e-5):
    out = np.empty(rows * width, np.float32)
    lib().h3o_rms_norm_f32(_p(out), _p(x), _p(weight), u32(rows), u32(width), f32(eps))
    return out


def layer_norm_f32(x, weight, bias, rows, width, eps=1e-5):
    out = np.empty(rows * width, np.float32)
    lib().h3o_layer_norm_f32(_p(out), _p(x), _p(weight), _p(bias), u32(rows), u32(width), f32(eps))
    return out


def scale_add_f32(residual, branch, scale, rows, width):
    out = np.empty(rows * width, np.float32)
    lib().h3o_scale_add_f32(_p(out), _p(residual), _p(branch), _p(scale), u32(rows), u32(width))
    return out


def swiglu_f32(fused, rows, width):
    out = np.empty(rows * width, np.float32)
    lib().h3o_swiglu_f32(_p(out), _p(fused), u32(rows), u32(width))
    return out


def video_qkv_rope_f32(qkv, cos, sin, seq, heads, hd, rope_half, eps=1e-5):
    q, k, v = (np.empty(seq * heads * hd, np.float32) for _ in range(3))
    lib().h3o_video_qkv_rope_f32(_p(q), _p(k), _p(v), _p(qkv), _p(cos), _p(sin), u32(seq), u32(heads),
                                 u32(hd), u32(rope_half), f32(eps))
    return q, k, v


def sdpa_f32(q, k, v, seq, heads, hd, scale):
    out = np.empty(seq * heads * hd, np.float32)
    lib().h3o_sdpa_f32(_p(out), _p(q), _p(k), _p(v), u32(seq), u32(heads), u32(hd), f32(scale))
    return out


def patch_linear_bf16(out, x, weight, bias, row_map, offset_rows, rows, in_dim, out_dim):
    lib().h3o_patch_linear_bf16(_p(out), _p(x), _p(weight), _p(bias), _p(row_map),
                                u32(offset_rows), u32(rows), u32(in_dim), u32(out_dim))
    return out


def euler_bf16(sample, last, previous, delta, ratio):
    out = sample.copy()
    lib().h3o_euler_bf16(_p(out), _p(last), _p(previous), C.c_size_t(last.size), f32(delta),
                         f32(ratio))
    return out


def cfg_combine_bf16(cond, uncond, guidance):
    out = np.empty_like(cond)
    lib().h3o_cfg_combine_bf16(_p(out), _p(cond), _p(uncond), C.c_size_t(cond.size), f32(guidance))
    return out


def token_pool_bf16(x, baseline, baseline_indices, pairs, input_rows, rows, width):
    out = np.empty(rows * width, np.uint16)
    original = np.zeros(input_rows * width, np.uint16)
    baseline = baseline.copy()
    lib().h3o_token_pool_bf16(_p(out), _p(x), _p(original), _p(baseline), _p(baseline_indices),
                              _p(pairs), u32(rows), u32(width))
    return out, original, baseline


def token_expand_delta_bf16(original, reduced, baseline, baseline_indices, parents, rows, width,
                            exact_prefix_rows, update_scale):
    out = np.empty(rows * width, np.uint16)
    lib().h3o_token_expand_delta_bf16(_p(out), _p(original), _p(reduced), _p(baseline),
                                      _p(baseline_indices), _p(parents), u32(rows), u32(width),
                                      u32(exact_prefix_rows), f32(update_scale))
    return out


def time_features(times):
    times = np.ascontiguousarray(times, np.float32)
    out = np.empty(times.size * 256, np.float32)
    lib().h3o_time_features(_p(out), _p(times), u32(times.size))
    return out


def rope_tables(positions, inv_freq):
    positions = np.ascontiguousarray(positions, np.float32)
    rows = positions.shape[0]
    cos = np.empty(rows * 48, np.uint16)
    sin = np.empty(rows * 48, np.uint16)
    lib().h3o_rope_tables(_p(cos), _p(sin), _p(positions),
                          _p(np.ascontiguousarray(inv_freq, np.float32)), u32(rows))
    return cos, sin


class BlockWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in
                ("norm1", "norm2", "qkv_weight", "q_norm", "k_norm", "out_weight", "fc1_weight",
                 "fc2_weight", "modulation")]


class BlockShape(C.Structure):
    _fields_ = [("rows", u32), ("width", u32), ("heads", u32), ("head_dim", u32), ("ffn", u32),
                ("rope_half", u32), ("eps", f32), ("scale", f32), ("round_p", C.c_int)]


def dit_block(hidden, weights: dict, row_map, cos, sin, *, rows, width, heads, head_dim, ffn,
              rope_half, eps=1e-5, scale=None, round_p=1, dumps=False):
    """Returns the block output (and the four stage dumps when dumps=True)."""
    hidden = hidden.copy()
    w = BlockWeights(**{k: _p(weights[k]).value for k, _ in BlockWeights._fields_})
    s = BlockShape(rows, width, heads, head_dim, ffn, rope_half, eps,
                   scale if scale is not None else 1.0 / np.sqrt(head_dim), round_p)
    inner = heads * head_dim
    d = [np.empty(rows * width, np.uint16), np.empty(rows * inner, np.uint16),
         np.empty(rows * width, np.uint16), np.empty(rows * width, np.uint16)] if dumps else [None] * 4
    lib().h3o_dit_block(_p(hidden), C.byref(w), _p(row_map), _p(cos), _p(sin), C.byref(s),
                        _p(d[0]), _p(d[1]), _p(d[2]), _p(d[3]))
    if dumps:
        return hidden, dict(mod_attention=d[0], attention=d[1], attention_output=d[2], mod_mlp=d[3])
    return hidden
