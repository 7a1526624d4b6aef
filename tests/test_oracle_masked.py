"""CPU checks of the oracle's block-sparse attention on the cases the reference kernel guards:
a query block that lists no key tile writes zero rows (h3_cuda_attention.cu:1790,1800), and a
mask that lists every tile equals dense attention."""
import numpy as np

import h3_oracle as o

SCALE = 1.0 / np.sqrt(128.0)


def qkv(seq, heads, seed):
    rng = np.random.default_rng(seed)
    return [o.to_bf16(rng.standard_normal(seq * heads * 128, dtype=np.float32)) for _ in range(3)]


def test_unlisted_query_blocks_are_zero_and_listed_ones_finite():
    seq, heads = 300, 2                                  # 3 query blocks, 5 key tiles of 64
    q, k, v = qkv(seq, heads, 1)
    ptr = np.array([0, 2, 2, 3], np.uint32)              # block 1 lists nothing
    idx = np.array([0, 4, 2], np.uint32)
    out = o.sdpa_bf16_sparse(q, k, v, seq, heads, 128, SCALE, ptr, idx, round_p=1)
    rows = out.reshape(seq, heads * 128)
    assert not rows[128:256].any()
    values = o.from_bf16(out)
    assert np.isfinite(values).all() and rows[:128].any() and rows[256:].any()


def test_full_mask_equals_dense():
    seq, heads = 200, 1
    q, k, v = qkv(seq, heads, 2)
    ptr = np.array([0, 4, 8], np.uint32)
    idx = np.array([0, 1, 2, 3] * 2, np.uint32)
    masked = o.sdpa_bf16_sparse(q, k, v, seq, heads, 128, SCALE, ptr, idx, round_p=1)
    dense = o.sdpa_bf16(q, k, v, seq, heads, 128, SCALE, round_p=1)
    assert np.array_equal(masked, dense)
