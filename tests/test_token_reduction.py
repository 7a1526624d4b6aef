"""Token reduction (the reference's --token-reduction mode, h3_dit.c:440-505, 1258-1310,
1921-1981, 2316-2345): pooled token maps on the CPU, and on the GPU a block stack whose middle
blocks run on the pooled grid, against the CPU oracle composed the same way."""
import numpy as np
import pytest

import h3_oracle as o
from block_case import ORACLE_TO_DRIVER, _normal_bf16


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as entry
    return entry.load_package()


class MapsOnly:
    """Stand-in context: the maps are plain arrays, no device."""

    def u32(self, values):
        return np.asarray(values, np.uint32)

    def new(self, n, dtype):
        return None


def test_maps_for_an_odd_width(pkg):
    # 2 kept rows, then a 1 x 2 x 5 video grid: 3 pooled columns per row, the last one single
    red = pkg.TokenReduction(MapsOnly(), pkg.DitShape(hidden=64), sequence=12, video_start=2,
                             t=1, h=2, w=5, begin=1, end=3)
    assert red.reduced_sequence == 2 + 6 and red.baseline_rows == 4
    assert red.pairs.tolist() == [[0, 0], [1, 1], [2, 3], [4, 5], [6, 6], [7, 8], [9, 10], [11, 11]]
    assert red.baseline_index_values.tolist() == [0xFFFFFFFF, 0xFFFFFFFF, 0, 1, 0xFFFFFFFF, 2, 3, 0xFFFFFFFF]
    assert red.parents.tolist() == [0, 1, 2, 2, 3, 3, 4, 5, 5, 6, 6, 7]
    pos = np.arange(36, dtype=np.float32).reshape(12, 3)
    assert np.allclose(red.reduced_positions(pos)[2], (pos[2] + pos[3]) / 2)
    assert np.allclose(red.reduced_positions(pos)[4], pos[6])
    assert red.reduced_row_map(np.arange(12, dtype=np.uint32)).tolist() == [0, 1, 2, 4, 6, 7, 9, 11]


def test_layout_must_end_with_the_video(pkg):
    with pytest.raises(ValueError):
        pkg.TokenReduction(MapsOnly(), pkg.DitShape(hidden=64), sequence=13, video_start=2,
                           t=1, h=2, w=5, begin=1, end=3)


@pytest.mark.gpu
@pytest.mark.parametrize("fused", [True, False])  # pool / expand kernels with or without the next adaLN
@pytest.mark.parametrize("end", [3, 4])          # leave before the last block / after the last block
def test_reduced_block_range_matches_oracle(pkg, end, fused):
    hidden, heads, ffn, n_blocks = 512, 4, 1024, 4
    text_rows, t, h, w = 24, 2, 6, 9
    rows = text_rows + t * h * w
    one = o.to_bf16(np.ones(1, np.float32))[0]
    blocks = []
    for b in range(n_blocks):
        wts = {name: _normal_bf16(count, o.named_seed(7, f"b{b}.{name}"), 0.02, False)
               for name, count in (("qkv_weight", 3 * heads * 128 * hidden), ("out_weight", hidden * heads * 128),
                                   ("fc1_weight", 2 * ffn * hidden), ("fc2_weight", hidden * ffn))}
        wts.update(norm1=np.full(hidden, one, np.uint16), norm2=np.full(hidden, one, np.uint16),
                   q_norm=np.full(128, one, np.uint16), k_norm=np.full(128, one, np.uint16),
                   modulation=_normal_bf16(6 * 6 * hidden, o.named_seed(7, f"b{b}.mod"), 0.13, False))
        blocks.append(wts)
    x = _normal_bf16(rows * hidden, 11, 1.0, False)
    pos = np.zeros((rows, 3), np.float32)
    pos[:text_rows, 0] = np.arange(text_rows)
    tt, hh, ww = np.meshgrid(np.arange(t), np.arange(h), np.arange(w), indexing="ij")
    pos[text_rows:, 0], pos[text_rows:, 1], pos[text_rows:, 2] = (a.reshape(-1) for a in (tt, hh, ww))
    inv_freq = (10000.0 ** (-np.arange(16, dtype=np.float64) / 16.0)).astype(np.float32)
    row_map = np.concatenate([np.full(text_rows, 4, np.uint32), np.full(rows - text_rows, 3, np.uint32)])

    gpu = pkg.Gpu(0)
    try:
        shape = pkg.DitShape(hidden=hidden, heads=heads, ffn=ffn, blocks=n_blocks)
        dit = pkg.Dit(gpu, shape, rows)
        red = pkg.TokenReduction(gpu, shape, sequence=rows, video_start=text_rows, t=t, h=h, w=w,
                                 begin=1, end=end, scale=0.75)
        cos, sin = o.rope_tables(pos, inv_freq)
        rcos, rsin = o.rope_tables(red.reduced_positions(pos), inv_freq)
        red.set_rope(gpu.bf16(rcos), gpu.bf16(rsin))
        weights = [pkg.BlockWeights(**{drv: gpu.bf16(wts[orc]) for orc, drv in ORACLE_TO_DRIVER.items()})
                   for wts in blocks]
        dit.hidden.write(x)
        gpu.begin()
        dit.run_blocks(weights, gpu.u32(row_map), gpu.bf16(cos), gpu.bf16(sin), reduction=red,
                       reduced_row_map=gpu.u32(red.reduced_row_map(row_map)), fused_boundaries=fused)
        gpu.submit()
        got = dit.hidden.read()[:rows * hidden]
    finally:
        gpu.close()

    def run(hid, lo, hi, n_rows, rm, c, s):
        for wts in blocks[lo:hi]:
            hid = o.dit_block(hid, wts, rm, c, s, rows=n_rows, width=hidden, heads=heads, head_dim=128,
                              ffn=ffn, rope_half=48, round_p=1)
        return hid
    want = run(x, 0, 1, rows, row_map, cos, sin)
    pooled, original, baseline = o.token_pool_bf16(
        want, np.zeros(red.baseline_rows * hidden, np.uint16), red.baseline_index_values,
        red.pairs.reshape(-1), rows, red.reduced_sequence, hidden)
    pooled = run(pooled, 1, end, red.reduced_sequence, red.reduced_row_map(row_map), rcos, rsin)
    want = o.token_expand_delta_bf16(original, pooled, baseline, red.baseline_index_values, red.parents,
                                     rows, hidden, text_rows, 0.75)
    want = run(want, end, n_blocks, rows, row_map, cos, sin)
    g, wv = o.from_bf16(got).astype(np.float64), o.from_bf16(want).astype(np.float64)
    rel, mx = np.linalg.norm(g - wv) / np.linalg.norm(wv), np.abs(g - wv).max()
    print(f"token reduction blocks [1,{end}) fused={fused}: rel_l2={rel:.3e} max_abs={mx:.3e}")
    assert rel <= 1e-2 and mx <= 1e-1
