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


@pytest.mark.skipif(not REF_DIT_TESTS.exists(), reason="reference test program was not built")
def test_reference_dit_op_tests_pass_on_this_backend():
    """tests/test_cuda_dit.c of the reference (12 fused DiT ops against its own CPU references,
    error paths, Metal-only stubs), linked against libh3b200.so."""
    env = dict(os.environ)
    res = subprocess.run([str(REF_DIT_TESTS)], capture_output=True, text=True, timeout=300, env=env)
    print(res.stdout[-3000:])
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "FAIL" not in res.stdout
