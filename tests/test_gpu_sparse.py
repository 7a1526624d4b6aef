"""Block-sparse attention (h3_gpu_sdpa_set_sparse): CSR over 64-key tiles per 128-row query block.

  * registration follows the reference's validation (h3_cuda_attention.cu:1812-1857);
  * a mask that lists every tile gives the dense result bit for bit;
  * random and windowed masks against the CPU oracle's masked attention, including a ragged
    sequence, lists that differ between neighbouring query blocks and single 64-key halves, with
    each of the two tensor-core kernels;
  * the same mask through the reference's own CUDA backend (oracle/_ref/libh3ref.so);
  * calls with another row count stay dense;
  * the sequence-parallel (push) instances of the kernels with a one-rank peer table."""
from pathlib import Path

import numpy as np
import pytest

import h3_oracle as o
from parity import assert_aggregate_close

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
REF_CUDA = ROOT / "oracle" / "_ref" / "libh3ref.so"
SCALE = 1.0 / np.sqrt(128.0)


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as entry
    return entry.load_package()


def set_sparse(gpu, ptr, idx, rows):
    if ptr is None:
        return gpu.lib.h3_gpu_sdpa_set_sparse(gpu.handle, None, 0, None, 0, 0)
    ptr = np.ascontiguousarray(ptr, np.uint32)
    idx = np.ascontiguousarray(idx, np.uint32)
    return gpu.lib.h3_gpu_sdpa_set_sparse(gpu.handle, ptr.ctypes.data, ptr.size, idx.ctypes.data,
                                          idx.size, rows)


def csr(lists):
    ptr = np.concatenate([[0], np.cumsum([len(l) for l in lists])]).astype(np.uint32)
    idx = np.concatenate([np.asarray(l, np.uint32) for l in lists]).astype(np.uint32)
    return ptr, idx


def random_mask(seq, rng, density):
    qb, kt = (seq + 127) // 128, (seq + 63) // 64
    lists = []
    for b in range(qb):
        keep = rng.random(kt) < density
        keep[min(kt - 1, 2 * b)] = True          # the block's own keys
        lists.append(np.nonzero(keep)[0])
    return csr(lists)


def window_mask(seq, radius):
    qb, kt = (seq + 127) // 128, (seq + 63) // 64
    return csr([[k for k in range(kt) if abs(k - 2 * b) <= radius] for b in range(qb)])


def qkv(seq, heads, seed):
    rng = np.random.default_rng(seed)
    return [o.to_bf16(rng.standard_normal(seq * heads * 128, dtype=np.float32)) for _ in range(3)]


def run_sdpa(pkg, gpu, q, k, v, seq, heads):
    tq, tk, tv = gpu.bf16(q), gpu.bf16(k), gpu.bf16(v)
    out = gpu.new(seq * heads * 128, pkg.BF16)
    gpu.begin()
    gpu.op("sdpa_bf16", out, tq, tk, tv, seq, heads, 128, SCALE)
    gpu.submit()
    return out.read()


def test_registration_validation(pkg):
    gpu = pkg.Gpu(0)
    try:
        ptr, idx = window_mask(512, 1)
        assert set_sparse(gpu, ptr, idx, 512) == 1
        assert set_sparse(gpu, None, None, 0) == 1                      # clear
        bad = ptr.copy(); bad[0] = 1
        assert set_sparse(gpu, bad, idx, 512) == 0                       # offsets must start at 0
        bad = ptr.copy(); bad[-1] += 1
        assert set_sparse(gpu, bad, idx, 512) == 0                       # ... and end at the index count
        bad = ptr.copy(); bad[1], bad[2] = bad[2], bad[1] - 1 if bad[1] else 0
        if np.any(np.diff(bad.astype(np.int64)) < 0):
            assert set_sparse(gpu, bad, idx, 512) == 0                   # monotone
        bad = idx.copy(); bad[0] = 8                                     # 512 rows = 8 tiles: 0..7
        assert set_sparse(gpu, ptr, bad, 512) == 0
    finally:
        gpu.close()


@pytest.fixture(params=[False, True], ids=["one_tile", "two_tiles"])
def two_tiles(request, monkeypatch):
    """Both tensor-core kernels walk masks: the default one (one query tile per CTA, one step list
    per query block) and, with H3B_SDPA_TWO_TILES=1, the one with two query tiles per CTA (the
    union of its two blocks' lists)."""
    if request.param:
        monkeypatch.setenv("H3B_SDPA_TWO_TILES", "1")
    return request.param


@pytest.mark.parametrize("seq", [512, 700])
def test_full_mask_is_dense(pkg, seq, two_tiles):
    """A mask that lists every key tile gives bit for bit what the same kernel gives without a
    mask."""
    heads = 2
    q, k, v = qkv(seq, heads, 1)
    qb, kt = (seq + 127) // 128, (seq + 63) // 64
    gpu = pkg.Gpu(0)
    try:
        dense = run_sdpa(pkg, gpu, q, k, v, seq, heads)
        assert set_sparse(gpu, *csr([np.arange(kt)] * qb), seq) == 1
        masked = run_sdpa(pkg, gpu, q, k, v, seq, heads)
    finally:
        gpu.close()
    assert np.array_equal(dense, masked)


@pytest.mark.parametrize("seq,kind", [(512, "random"), (700, "random"), (1100, "window"), (700, "halves")])
def test_masked_attention_matches_oracle(pkg, seq, kind, two_tiles):
    heads = 3
    q, k, v = qkv(seq, heads, seq)
    rng = np.random.default_rng(seq + 5)
    if kind == "random":
        ptr, idx = random_mask(seq, rng, 0.4)
    elif kind == "window":
        ptr, idx = window_mask(seq, 2)
    else:   # every block sees exactly one 64-key half, a different one per block
        qb, kt = (seq + 127) // 128, (seq + 63) // 64
        ptr, idx = csr([[(3 * b + 1) % kt] for b in range(qb)])
    want = o.sdpa_bf16_sparse(q, k, v, seq, heads, 128, SCALE, ptr, idx, round_p=1)
    gpu = pkg.Gpu(0)
    try:
        assert set_sparse(gpu, ptr, idx, seq) == 1
        got = run_sdpa(pkg, gpu, q, k, v, seq, heads)
        other = run_sdpa(pkg, gpu, q[:256 * heads * 128], k[:256 * heads * 128], v[:256 * heads * 128],
                         256, heads)           # another row count: stays dense
    finally:
        gpu.close()
    assert_aggregate_close(got, want, f"sparse {kind} S={seq}")
    dense_small = o.sdpa_bf16(q[:256 * heads * 128], k[:256 * heads * 128], v[:256 * heads * 128],
                              256, heads, 128, SCALE, round_p=1)
    assert_aggregate_close(other, dense_small, "dense call while a mask for other rows is registered")


def test_query_blocks_that_list_nothing_give_zero_rows(pkg, two_tiles):
    """A 128-row query block with an empty list attends nothing: its rows are zeros, not NaN
    (h3_cuda_attention.cu:1790,1800). Covered: an empty block beside a listed one (the same CTA
    in the two-tile kernel), neighbouring blocks that are both empty, and blocks past the end of
    a short ptr array."""
    seq, heads = 900, 2                      # 8 query blocks (the last ragged) = 4 CTAs
    q, k, v = qkv(seq, heads, 9)
    kt = (seq + 63) // 64
    lists = [[0, 3], [], [], [], [1, kt - 1], [2]]       # blocks 6 and 7 are not listed at all
    ptr, idx = csr(lists)
    want = o.sdpa_bf16_sparse(q, k, v, seq, heads, 128, SCALE,
                              *csr(lists + [[], []]), round_p=1)
    gpu = pkg.Gpu(0)
    try:
        assert set_sparse(gpu, ptr, idx, seq) == 1
        got = run_sdpa(pkg, gpu, q, k, v, seq, heads)
    finally:
        gpu.close()
    rows = got.reshape(seq, heads * 128)
    for block in (1, 2, 3, 6, 7):
        assert not rows[block * 128:(block + 1) * 128].any(), f"query block {block} is not zero"
    assert rows[:128].any() and rows[4 * 128:6 * 128].any()
    assert_aggregate_close(got, want, "sparse mask with empty query blocks")


@pytest.mark.skipif(not REF_CUDA.exists(), reason="reference CUDA backend was not built")
def test_masked_attention_matches_reference_cuda_backend(pkg):
    seq, heads = 1664, 8
    q, k, v = qkv(seq, heads, 3)
    ptr, idx = random_mask(seq, np.random.default_rng(11), 0.3)
    out = {}
    for name, path in (("b200", None), ("reference", REF_CUDA)):
        gpu = pkg.Gpu(0, lib_path=path)
        try:
            assert set_sparse(gpu, ptr, idx, seq) == 1
            out[name] = run_sdpa(pkg, gpu, q, k, v, seq, heads)
        finally:
            gpu.close()
    assert_aggregate_close(out["b200"], out["reference"], "sparse vs reference CUDA backend")


@pytest.mark.parametrize("masked", [False, True], ids=["dense", "masked"])
def test_push_form_with_one_rank_equals_the_local_form(pkg, masked, two_tiles):
    """h3x_sdpa_push with a one-rank peer table stores every output row into this GPU's own
    buffer: the kernels' sequence-parallel instances (dense and under a mask) on a single GPU,
    bit for bit what the local call gives."""
    seq, heads = 900, 3
    q, k, v = qkv(seq, heads, 21)
    gpu = pkg.Gpu(0)
    try:
        if masked:
            assert set_sparse(gpu, *random_mask(seq, np.random.default_rng(4), 0.4), seq) == 1
        local = run_sdpa(pkg, gpu, q, k, v, seq, heads)
        tq, tk, tv = gpu.bf16(q), gpu.bf16(k), gpu.bf16(v)
        out = gpu.new(seq * heads * 128, pkg.BF16)
        peers = pkg.UlyssesPeers()
        peers.world, peers.rank, peers.rows_local = 1, 0, seq
        peers.o[0] = out.pointer
        gpu.begin()
        gpu.op("h3x_sdpa_push", peers, tq, tk, tv, seq, heads, 128, SCALE)
        gpu.submit()
        pushed = out.read()
    finally:
        gpu.close()
    assert np.array_equal(pushed, local)
