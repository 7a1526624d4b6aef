"""Golden vectors produced by the reference's own CPU code (tests/golden/make_golden.py).

CPU part: the oracle must reproduce them bit-for-bit (this is the pin that travels to
machines without the reference tree). GPU part: libh3b200.so must match them within the
reference's own per-op tolerances."""
from pathlib import Path

import numpy as np
import pytest

import h3_oracle as o
from parity import assert_bf16_ulp, assert_gemm_close

G = np.load(Path(__file__).parent / "golden" / "ref_cpu_vectors.npz")


def test_rng_golden():
    for seed in (0, 7, 42):
        want = G[f"rng_normal_seed{seed}"]
        assert np.array_equal(o.normal_f32(want.size, seed).view(np.uint32), want.view(np.uint32))


def test_adaln_gate_golden():
    rows, width, slots = 6, 5376, 6
    got = o.adaln_bf16(G["adaln_x"], G["adaln_w"], G["adaln_mod"], G["adaln_row_map"], rows, width, slots, 0, 1)
    assert np.array_equal(got, o.to_bf16(G["adaln_out"]))
    got = o.gate_bf16(G["adaln_x"], G["adaln_br"], G["adaln_mod"], G["adaln_row_map"], rows, width, slots, 2)
    assert np.array_equal(got, o.to_bf16(G["gate_out"]))


def test_linear_swiglu_golden():
    assert np.array_equal(o.linear_bf16(G["linear_x"], G["linear_w"], G["linear_b"], 40, 512, 136),
                          o.to_bf16(G["linear_out"]))
    assert np.array_equal(o.swiglu_bf16(G["swiglu_in"], 5, 96), o.to_bf16(G["swiglu_out"]))


def test_qkv_rope_golden():
    q, k, v = o.qkv_rope_bf16(G["rope_qkv"], G["rope_qw"], G["rope_kw"], G["rope_cos"], G["rope_sin"],
                              12, 3, 128, 48, 1)
    assert np.array_equal(q, o.to_bf16(G["rope_q"]))
    assert np.array_equal(k, o.to_bf16(G["rope_k"]))
    assert np.array_equal(v, o.to_bf16(G["rope_v"]))


@pytest.mark.parametrize("tag", ["a", "b"])
def test_sdpa_golden(tag):
    seq, heads, hd = (int(x) for x in G[f"sdpa_{tag}_shape"])
    got = o.sdpa_bf16(G[f"sdpa_{tag}_q"], G[f"sdpa_{tag}_k"], G[f"sdpa_{tag}_v"], seq, heads, hd,
                      1.0 / np.sqrt(hd), 0, round_p=0)
    assert np.array_equal(got, o.to_bf16(G[f"sdpa_{tag}_out"]))


# ------------------------------------------------------------------ GPU
@pytest.fixture(scope="module")
def ctx():
    import __graft_entry__ as entry
    pkg = entry.load_package()
    gpu = pkg.Gpu(0)
    yield pkg, gpu
    gpu.close()


@pytest.mark.gpu
def test_cuda_matches_reference_cpu_vectors(ctx):
    pkg, gpu = ctx
    rows, width, slots = 6, 5376, 6
    tx, tb, tw, tm = (gpu.bf16(G[k]) for k in ("adaln_x", "adaln_br", "adaln_w", "adaln_mod"))
    tr = gpu.u32(G["adaln_row_map"])
    out = gpu.new(rows * width, pkg.BF16)
    gpu.begin()
    gpu.op("adaln_bf16", out, tx, tw, tm, tr, rows, width, slots, 0, 1, 1e-5)
    gpu.submit()
    assert_bf16_ulp(out.read(), o.to_bf16(G["adaln_out"]), "adaln vs reference CPU")
    gpu.begin()
    gpu.op("gate_bf16", out, tx, tb, tm, tr, rows, width, slots, 2)
    gpu.submit()
    assert_bf16_ulp(out.read(), o.to_bf16(G["gate_out"]), "gate vs reference CPU")

    lx, lw, lb = (gpu.bf16(G[k]) for k in ("linear_x", "linear_w", "linear_b"))
    lo = gpu.new(40 * 136, pkg.BF16)
    gpu.begin()
    gpu.op("linear_bf16", lo, lx, lw, lb, 40, 512, 136)
    gpu.submit()
    assert_gemm_close(lo.read(), o.to_bf16(G["linear_out"]), "linear vs reference CPU")

    n = 12 * 3 * 128
    tq, tk, tv = (gpu.new(n, pkg.BF16) for _ in range(3))
    t = [gpu.bf16(G[k]) for k in ("rope_qkv", "rope_qw", "rope_kw", "rope_cos", "rope_sin")]
    gpu.begin()
    gpu.op("grouped_qkv_rope_bf16", tq, tk, tv, *t, 12, 3, 128, 48, 1e-5)
    gpu.submit()
    assert_bf16_ulp(tq.read(), o.to_bf16(G["rope_q"]), "rope q vs reference CPU")
    assert_bf16_ulp(tk.read(), o.to_bf16(G["rope_k"]), "rope k vs reference CPU")
    assert np.array_equal(tv.read(), o.to_bf16(G["rope_v"]))

    for tag in ("a", "b"):
        seq, heads, hd = (int(x) for x in G[f"sdpa_{tag}_shape"])
        q, k, v = (gpu.bf16(G[f"sdpa_{tag}_{x}"]) for x in "qkv")
        so = gpu.new(seq * heads * hd, pkg.BF16)
        gpu.begin()
        gpu.op("sdpa_bf16", so, q, k, v, seq, heads, hd, 1.0 / np.sqrt(hd))
        gpu.submit()
        assert_gemm_close(so.read(), o.to_bf16(G[f"sdpa_{tag}_out"]), f"sdpa {tag} vs reference CPU")
