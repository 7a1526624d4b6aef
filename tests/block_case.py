"""Seeded synthetic DiT block cases shared by the GPU tests, the smoke check and the bench.

Inputs follow the synthetic-input plan: activations N(0,1), weights N(0,0.02), RMSNorm gains
1.0 (so activations keep O(1) scale), modulation N(0,0.13) (the scale the adaLN projection
yields from N(0,0.02) time-embedder and projection weights: 0.02*sqrt(2688)*|silu| ~ 0.13), text rows at (index,0,0) and video
rows on an integer t x h x w grid, rope.inv_freq[i] = 10000^(-i/16). Small cases draw from
the reference's PCG32 + Box-Muller generator (oracle restatement, pinned to h3_host.c);
full-width cases use numpy's seeded generator because the scalar generator would take
minutes for 385 M weights. The same arrays feed the oracle, libh3b200 and, where present,
the reference's CUDA backend, so the choice of generator does not affect parity.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

import h3_oracle as o


@dataclass
class BlockCase:
    rows: int
    text_rows: int
    heads: int
    hidden_dim: int
    ffn: int
    hidden: np.ndarray
    weights: dict
    row_map: np.ndarray
    rope_cos: np.ndarray
    rope_sin: np.ndarray


def _normal_bf16(n, seed, std, fast):
    if fast:
        rng = np.random.default_rng(seed)
        out = np.empty(n, np.uint16)
        step = 1 << 24
        for i in range(0, n, step):
            m = min(step, n - i)
            out[i:i + m] = o.to_bf16(rng.standard_normal(m, dtype=np.float32) * np.float32(std))
        return out
    return o.normal_bf16(n, seed, 0.0, std)


def video_grid(video_rows: int):
    """t x h x w with h*w = 64 when it divides, else a single row of tokens."""
    if video_rows % 64 == 0:
        return video_rows // 64, 8, 8
    return 1, 1, video_rows


def make_block_case(rows=320, text_rows=64, heads=4, hidden=512, ffn=1024, seed=0, mod_rows=6,
                    fast=False) -> BlockCase:
    inner = heads * 128
    video_rows = rows - text_rows
    names = {
        "qkv_weight": 3 * inner * hidden, "out_weight": hidden * inner,
        "fc1_weight": 2 * ffn * hidden, "fc2_weight": hidden * ffn,
    }
    weights = {}
    for i, (name, count) in enumerate(names.items()):
        weights[name] = _normal_bf16(count, o.named_seed(seed, name), 0.02, fast)
    one = o.to_bf16(np.ones(1, np.float32))[0]
    weights["norm1"] = np.full(hidden, one, np.uint16)
    weights["norm2"] = np.full(hidden, one, np.uint16)
    weights["q_norm"] = np.full(128, one, np.uint16)
    weights["k_norm"] = np.full(128, one, np.uint16)
    weights["modulation"] = _normal_bf16(mod_rows * 6 * hidden, o.named_seed(seed, "modulation"),
                                         0.13, fast)
    x = _normal_bf16(rows * hidden, seed + 1, 1.0, fast)
    t, h, w = video_grid(video_rows)
    pos = np.zeros((rows, 3), np.float32)
    pos[:text_rows, 0] = np.arange(text_rows)
    tt, hh, ww = np.meshgrid(np.arange(t), np.arange(h), np.arange(w), indexing="ij")
    pos[text_rows:, 0], pos[text_rows:, 1], pos[text_rows:, 2] = (a.reshape(-1) for a in (tt, hh, ww))
    inv_freq = (10000.0 ** (-np.arange(16, dtype=np.float64) / 16.0)).astype(np.float32)
    cos, sin = o.rope_tables(pos, inv_freq)
    tags = np.concatenate([np.ones(text_rows, np.uint32), np.zeros(video_rows, np.uint32)])
    row_map = (tags + 3 * 1).astype(np.uint32)     # time row 1 of mod_rows/3
    return BlockCase(rows, text_rows, heads, hidden, ffn, x, weights, row_map, cos, sin)


ORACLE_TO_DRIVER = {"norm1": "norm1", "norm2": "norm2", "qkv_weight": "qkv", "q_norm": "q_norm",
                    "k_norm": "k_norm", "out_weight": "out", "fc1_weight": "fc1",
                    "fc2_weight": "fc2", "modulation": "modulation"}


def upload_block(pkg, gpu, case: BlockCase):
    tensors = {drv: gpu.bf16(case.weights[orc]) for orc, drv in ORACLE_TO_DRIVER.items()}
    return pkg.BlockWeights(**tensors)


def run_block_on_gpu(pkg, gpu, case: BlockCase, return_driver=False):
    """One block through the host driver (the run_block op sequence) on `gpu`."""
    shape = pkg.DitShape(hidden=case.hidden_dim, heads=case.heads, ffn=case.ffn, blocks=1)
    dit = pkg.Dit(gpu, shape, case.rows)
    w = upload_block(pkg, gpu, case)
    row_map, cos, sin = gpu.u32(case.row_map), gpu.bf16(case.rope_cos), gpu.bf16(case.rope_sin)
    dit.hidden.write(case.hidden)
    gpu.begin()
    dit.run_block(w, row_map, cos, sin, False, None)
    gpu.submit()
    out = dit.hidden.read()
    return (out, dit) if return_driver else out
