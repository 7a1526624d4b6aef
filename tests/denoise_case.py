"""Seeded synthetic multi-step denoise cases: a small DiT (a few blocks) with patch projection,
final head, one modulation row per Euler step, and two text embeddings (cond / uncond). The
hidden width stays 5376 even in small cases (few heads, narrow MLP) because the patch
projection accepts only the model's width, as in the reference (h3_cuda_core.cu:929-931).

`oracle_denoise` composes the CPU oracle in the order of the reference's encode_forward
(h3_dit.c:2182-2528: text rows copied in, patch projection of the F32 latent rows, the blocks,
final adaLN + projection) and denoise_euler_gpu (h3_dit.c:2805-2893: Euler update per step);
`gpu_denoise` drives the same case through the library's host driver on any exchange."""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

import h3_oracle as o
from block_case import ORACLE_TO_DRIVER, _normal_bf16, video_grid

PATCH = 96


@dataclass
class DenoiseCase:
    rows: int
    text_rows: int
    heads: int
    hidden_dim: int
    ffn: int
    steps: int
    blocks: list = field(default_factory=list)          # oracle-named weight dicts
    patch_weight: np.ndarray = None                     # F32 [hidden][96]
    patch_bias: np.ndarray = None                       # F32 [hidden]
    final_norm: np.ndarray = None
    final_modulation: np.ndarray = None                 # bf16 [steps][2][hidden]
    final_weight: np.ndarray = None                     # bf16 [96][hidden]
    final_bias: np.ndarray = None
    text: np.ndarray = None                             # bf16 [text_rows][hidden] (cond)
    text_uncond: np.ndarray = None
    latent: np.ndarray = None                           # F32 [video_rows][96]
    rope_cos: np.ndarray = None
    rope_sin: np.ndarray = None
    sigmas: np.ndarray = None

    @property
    def video_rows(self):
        return self.rows - self.text_rows

    def row_map(self, step):
        tags = np.concatenate([np.ones(self.text_rows, np.uint32), np.zeros(self.video_rows, np.uint32)])
        return (tags + 3 * step).astype(np.uint32)

    def final_row_map(self, step):
        return np.full(self.video_rows, step, np.uint32)


def make_denoise_case(rows=200, text_rows=40, heads=4, hidden=5376, ffn=1024, blocks=2, steps=4,
                      seed=0, fast=False, sigmas=None, distinct=None) -> DenoiseCase:
    """distinct: number of different sets of projection weights; block b uses set b % distinct
    (the arrays are shared, and uploaded once), while every block keeps its own modulation
    table. Deep cases (50 blocks) then cost a few GB instead of 38."""
    c = DenoiseCase(rows, text_rows, heads, hidden, ffn, steps)
    inner = heads * 128
    one = o.to_bf16(np.ones(1, np.float32))[0]
    distinct = blocks if distinct is None else min(distinct, blocks)
    for b in range(blocks):
        w = {}
        for name, count in (("qkv_weight", 3 * inner * hidden), ("out_weight", hidden * inner),
                            ("fc1_weight", 2 * ffn * hidden), ("fc2_weight", hidden * ffn)):
            if b >= distinct:
                w[name] = c.blocks[b % distinct][name]
                continue
            w[name] = _normal_bf16(count, o.named_seed(seed, f"blocks.{b}.{name}"), 0.02, fast)
        w["norm1"] = np.full(hidden, one, np.uint16)
        w["norm2"] = np.full(hidden, one, np.uint16)
        w["q_norm"] = np.full(128, one, np.uint16)
        w["k_norm"] = np.full(128, one, np.uint16)
        w["modulation"] = _normal_bf16(steps * 3 * 6 * hidden, o.named_seed(seed, f"blocks.{b}.modulation"),
                                       0.13, fast)
        c.blocks.append(w)
    rng = np.random.default_rng(seed + 77)
    # patch projection N(0, 1/sqrt(96)) so hidden rows start at O(1) like the block tests
    c.patch_weight = (rng.standard_normal(hidden * PATCH, dtype=np.float32) / np.float32(np.sqrt(PATCH)))
    c.patch_bias = rng.standard_normal(hidden, dtype=np.float32) * np.float32(0.02)
    c.final_norm = np.full(hidden, one, np.uint16)
    c.final_modulation = _normal_bf16(steps * 2 * hidden, o.named_seed(seed, "final.modulation"), 0.13, fast)
    c.final_weight = _normal_bf16(PATCH * hidden, o.named_seed(seed, "final.weight"), 0.02, fast)
    c.final_bias = _normal_bf16(PATCH, o.named_seed(seed, "final.bias"), 0.02, fast)
    c.text = _normal_bf16(text_rows * hidden, seed + 2, 1.0, fast)
    c.text_uncond = _normal_bf16(text_rows * hidden, seed + 4, 1.0, fast)
    c.latent = rng.standard_normal(c.video_rows * PATCH, dtype=np.float32)
    t, h, w_ = video_grid(c.video_rows)
    pos = np.zeros((rows, 3), np.float32)
    pos[:text_rows, 0] = np.arange(text_rows)
    tt, hh, ww = np.meshgrid(np.arange(t), np.arange(h), np.arange(w_), indexing="ij")
    pos[text_rows:, 0], pos[text_rows:, 1], pos[text_rows:, 2] = (a.reshape(-1) for a in (tt, hh, ww))
    inv_freq = (10000.0 ** (-np.arange(16, dtype=np.float64) / 16.0)).astype(np.float32)
    c.rope_cos, c.rope_sin = o.rope_tables(pos, inv_freq)
    c.sigmas = sigmas
    return c


# ------------------------------------------------------------------ CPU oracle

def oracle_velocity(c: DenoiseCase, latent, text, step):
    hidden = np.empty(c.rows * c.hidden_dim, np.uint16)
    hidden[:c.text_rows * c.hidden_dim] = text
    o.patch_linear_bf16(hidden, latent, c.patch_weight, c.patch_bias, None, c.text_rows,
                        c.video_rows, PATCH, c.hidden_dim)
    row_map = c.row_map(step)
    for w in c.blocks:
        hidden = o.dit_block(hidden, w, row_map, c.rope_cos, c.rope_sin, rows=c.rows,
                             width=c.hidden_dim, heads=c.heads, head_dim=128, ffn=c.ffn,
                             rope_half=48, round_p=1)
    video = hidden[c.text_rows * c.hidden_dim:]
    velocity, _ = o.adaln_linear_bf16(video, c.final_norm, c.final_modulation, c.final_row_map(step),
                                      c.final_weight, c.final_bias, c.video_rows, c.hidden_dim,
                                      PATCH, 2, 0, 1)
    return velocity


def oracle_denoise(c: DenoiseCase, guidance=None, selected=None, ratio_of=None):
    """selected[i] = 0 skips the model at step i and applies the last velocity extrapolated from
    the last two evaluations with weight ratio_of(current, last, previous, have_previous), as the
    reference's reuse schedule does (h3_dit.c:2805-2863)."""
    latent = c.latent.copy()
    v = prev_v = None
    last = previous = -1
    for i in range(c.steps):
        evaluate = selected is None or selected[i]
        if evaluate:
            if last >= 0 and selected is not None:
                prev_v, previous = v, last
            v = oracle_velocity(c, latent, c.text, i)
            if guidance is not None:
                v = o.cfg_combine_bf16(v, oracle_velocity(c, latent, c.text_uncond, i), guidance)
            last = i
        ratio = 0.0 if evaluate else ratio_of(c.sigmas[i], c.sigmas[last],
                                              c.sigmas[previous] if previous >= 0 else 0.0, previous >= 0)
        latent = o.euler_bf16(latent, v, prev_v if previous >= 0 else v,
                              float(c.sigmas[i] - c.sigmas[i + 1]), ratio)
    return latent


# ------------------------------------------------------------------ library

def gpu_denoise(pkg, gpu, c: DenoiseCase, *, guidance=None, exchange=None, pair=None, text=None,
                alloc=None, reuse_interval=1):
    """Runs the whole loop on `gpu`; with an exchange, on this rank's row slice. Returns the
    F32 latent rows this rank owns (video rows only)."""
    shape = pkg.DitShape(hidden=c.hidden_dim, heads=c.heads, ffn=c.ffn, blocks=len(c.blocks))
    dit = pkg.Dit(gpu, shape, c.rows, exchange=exchange, alloc=alloc)
    r0, rl, valid = dit.row_begin, dit.rows_local, dit.rows_valid
    uploaded = {}

    def upload_once(array):      # blocks of a deep case share their projection weights
        if id(array) not in uploaded:
            uploaded[id(array)] = gpu.bf16(array)
        return uploaded[id(array)]
    blocks = [pkg.BlockWeights(**{drv: upload_once(w[orc]) for orc, drv in ORACLE_TO_DRIVER.items()})
              for w in c.blocks]

    def rows_of(a, width, dtype, lo=r0, n=valid, pad=rl):
        out = np.zeros(max(1, pad) * width, dtype)
        out[:n * width] = a.reshape(-1, width)[lo:lo + n].reshape(-1)
        return out

    local_text = max(0, min(c.text_rows, r0 + valid) - r0)
    local_video = valid - local_text
    video_begin = max(0, r0 - c.text_rows)
    text_src = c.text if text is None else text
    step = pkg.DenoiseStep(
        dit, blocks, video_rows=local_video, text_rows=local_text,
        patch_weight=gpu.f32(c.patch_weight), patch_bias=gpu.f32(c.patch_bias),
        text_hidden=gpu.bf16(rows_of(text_src, c.hidden_dim, np.uint16, r0, local_text, local_text)),
        final_norm=gpu.bf16(c.final_norm), final_modulation=gpu.bf16(c.final_modulation),
        final_weight=gpu.bf16(c.final_weight), final_bias=gpu.bf16(c.final_bias),
        row_map=None, final_row_map=None,
        rope_cos=gpu.bf16(rows_of(c.rope_cos, 48, np.uint16)),
        rope_sin=gpu.bf16(rows_of(c.rope_sin, 48, np.uint16)))
    step.latent.write(rows_of(c.latent, PATCH, np.float32, video_begin, local_video, local_video))
    row_maps = [gpu.u32(rows_of(c.row_map(i), 1, np.uint32)) for i in range(c.steps)]
    final_maps = [gpu.u32(np.full(max(1, local_video), i, np.uint32)) for i in range(c.steps)]
    uncond = None
    if guidance is not None and pair is None:
        uncond = gpu.bf16(rows_of(c.text_uncond, c.hidden_dim, np.uint16, r0, local_text, local_text))
    sampler = pkg.EulerSampler(step, c.sigmas, row_maps, final_maps, guidance=guidance,
                               uncond_text=uncond, pair=pair, reuse_interval=reuse_interval)
    sampler.run()
    return step.latent.read()[:local_video * PATCH], (video_begin, local_video)


def cosine(a, b):
    a, b = a.astype(np.float64), b.astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))
