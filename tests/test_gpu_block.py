"""Block-level parity through the host driver (the reference's run_block op sequence):

  * against the CPU oracle composed in run_block order (per-block bar rel-L2 <= 1e-2,
    max-abs <= 5e-2), at a reduced width and at the model's full width;
  * against the reference's own CUDA backend (oracle/_ref/libh3ref.so, built from the
    reference's sources for sm_100), driven through the same C ABI with the same inputs;
  * by running the reference's own op test program (tests/test_cuda_dit.c, compiled in
    place and linked against libh3b200.so) and requiring every check to pass.
"""
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest

import h3_oracle as o
from block_case import make_block_case, run_block_on_gpu
from parity import assert_block_close, block_metrics

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
REF_CUDA = ROOT / "oracle" / "_ref" / "libh3ref.so"
REF_DIT_TESTS = ROOT / "oracle" / "_ref" / "test_cuda_dit_b200"


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as entry
    return entry.load_package()


def oracle_block(case, dumps=False):
    return o.dit_block(case.hidden, case.weights, case.row_map, case.rope_cos, case.rope_sin,
                       rows=case.rows, width=case.hidden_dim, heads=case.heads, head_dim=128,
                       ffn=case.ffn, rope_half=48, round_p=1, dumps=dumps)


@pytest.mark.parametrize("rows,text_rows", [(320, 64), (200, 8), (129, 1)])
def test_block_matches_oracle_reduced_width(pkg, rows, text_rows):
    case = make_block_case(rows=rows, text_rows=text_rows, heads=4, hidden=512, ffn=1024, seed=rows)
    gpu = pkg.Gpu(0)
    try:
        got = run_block_on_gpu(pkg, gpu, case)
    finally:
        gpu.close()
    assert_block_close(got, oracle_block(case), f"block rows={rows}")


def test_block_matches_oracle_full_width(pkg):
    """One block at the model's dims (hidden 5376, 56 heads, FFN 14336), 384 rows."""
    case = make_block_case(rows=384, text_rows=64, heads=56, hidden=5376, ffn=14336, seed=0, fast=True)
    gpu = pkg.Gpu(0)
    try:
        got = run_block_on_gpu(pkg, gpu, case)
    finally:
        gpu.close()
    r, m = assert_block_close(got, oracle_block(case), "full-width block")
    print(f"full-width block vs CPU oracle: rel_l2={r:.3e} max_abs={m:.3e}")


@pytest.mark.skipif(not REF_CUDA.exists(), reason="reference CUDA backend was not built")
def test_block_matches_reference_cuda_backend(pkg):
    """Same inputs through libh3b200.so and through the reference's CUDA backend (cuBLASLt
    GEMMs + its mma.sync flash attention): 'the reference BF16 path' of the parity bar."""
    case = make_block_case(rows=1664, text_rows=128, heads=56, hidden=5376, ffn=14336, seed=0, fast=True)
    outs = {}
    for name, path in (("b200", None), ("reference", REF_CUDA)):
        gpu = pkg.Gpu(0, lib_path=path)
        try:
            outs[name] = run_block_on_gpu(pkg, gpu, case)
        finally:
            gpu.close()
    r, m = assert_block_close(outs["b200"], outs["reference"], "block vs reference CUDA backend")
    print(f"config-1 block (S=1664) vs reference CUDA backend: rel_l2={r:.3e} max_abs={m:.3e}")


@pytest.mark.parametrize("heads", [24, 56])
def test_standalone_attention_config2(pkg, heads):
    """BASELINE config 2: [1, heads, 6400 tokens (6,144 video on a 6x32x32 grid + 256 text), 128],
    N(0,1) seed 3, 3-D RoPE on video rows and 1-D on text rows applied by the QKV op first.
    Checked against the oracle on a sample of query rows (full attention over all keys) and,
    where it was built, against the reference's CUDA backend on every row."""
    seq, hd, text = 6400, 128, 256
    n = seq * heads * hd
    rng = np.random.default_rng(3)
    qkv = o.to_bf16(rng.standard_normal(3 * n, dtype=np.float32))
    pos = np.zeros((seq, 3), np.float32)
    pos[:text, 0] = np.arange(text)
    idx = np.arange(seq - text)
    pos[text:, 0], pos[text:, 1], pos[text:, 2] = idx // 1024, (idx % 1024) // 32, idx % 32
    cos, sin = o.rope_tables(pos, (10000.0 ** (-np.arange(16) / 16.0)).astype(np.float32))
    one = np.full(hd, o.to_bf16(np.ones(1, np.float32))[0], np.uint16)
    scale = 1.0 / np.sqrt(hd)
    outs = {}
    for name, path in (("b200", None), ("reference", REF_CUDA)):
        if path is not None and not path.exists():
            continue
        gpu = pkg.Gpu(0, lib_path=path)
        try:
            tq, tk, tv, to = (gpu.new(n, pkg.BF16) for _ in range(4))
            t = [gpu.bf16(a) for a in (qkv, one, one, cos, sin)]
            gpu.begin()
            gpu.op("grouped_qkv_rope_bf16", tq, tk, tv, *t, seq, heads, hd, 48, 1e-5)
            gpu.op("sdpa_bf16", to, tq, tk, tv, seq, heads, hd, scale)
            gpu.submit()
            outs[name] = (to.read(), tq.read(), tk.read(), tv.read())
        finally:
            gpu.close()
    got, q, k, v = outs["b200"]
    rows = (3000, 3064)
    want = o.sdpa_bf16(q, k, v, seq, heads, hd, scale, 0, round_p=0, rows=rows)
    sl = slice(rows[0] * heads * hd, rows[1] * heads * hd)
    r, m = block_metrics(got[sl], want[sl])
    print(f"config-2 attention heads={heads} vs CPU oracle (64 query rows): rel_l2={r:.3e} max_abs={m:.3e}")
    assert r <= 4e-3 and m <= 2e-2
    if "reference" in outs:
        r, m = block_metrics(got, outs["reference"][0])
        print(f"config-2 attention heads={heads} vs reference CUDA backend: rel_l2={r:.3e} max_abs={m:.3e}")
        assert r <= 4e-3 and m <= 2e-2


@pytest.mark.skipif(not REF_DIT_TESTS.exists(), reason="reference test program was not built")
def test_reference_dit_op_tests_pass_on_this_backend():
    """tests/test_cuda_dit.c of the reference (12 fused DiT ops against its own CPU references,
    error paths, Metal-only stubs), linked against libh3b200.so."""
    env = dict(os.environ)
    res = subprocess.run([str(REF_DIT_TESTS)], capture_output=True, text=True, timeout=300, env=env)
    print(res.stdout[-3000:])
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "FAIL" not in res.stdout
