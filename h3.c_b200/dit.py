"""Host-side driver of the DiT denoiser forward over the C ABI.

Mirrors the reference's model layer for this path: the per-block op sequence of
`run_block` (h3_dit.c:2008-2180) with the cross-block gate+adaLN carry, the activation
aliasing of `allocate_activations` (h3_dit.c:1548-1551: attention_heads = mod_mlp = qkv,
MLP output reuses attention_output), the step structure of `encode_forward`
(h3_dit.c:2182-2528: patch projection, text rows copied in, 50 blocks, final heads) and
the Euler update of `denoise_euler_gpu` (h3_dit.c:2805-2893). Every arithmetic step is a
call into libh3b200.so with the reference's op names and argument meaning.

Sequence parallelism (no counterpart in the reference): each rank owns a contiguous
slice of rows; around attention the Q/K/V slices are regrouped by head and exchanged
all-to-all so that each rank attends over the full sequence for heads/world heads
(Ulysses), then exchanged back. Two forms: (1) the exchange is supplied by the caller (an
object with all_to_all(out, inp)), e.g. torch.distributed over NCCL, and this module issues
the layout kernels and attention; (2) the exchange object is a `PeerExchange` (peer-mapped
buffers): the QKV projection's epilogue and the attention epilogue store straight into the
owning rank's buffers over NVLink, and only two stream barriers per block remain.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

from .binding import BF16, F32, Gpu, Tensor


@dataclass
class DitShape:
    """Model constants (h3_dit.c:16-31, h3_dit_schedule.h:11-15)."""
    hidden: int = 5376
    heads: int = 56
    head_dim: int = 128
    ffn: int = 14336
    blocks: int = 50
    rope_half: int = 48
    slots: int = 6
    final_slots: int = 2
    modalities: int = 3
    time_dim: int = 2688
    video_patch: int = 96
    audio_channels: int = 32
    eps: float = 1e-5

    @property
    def inner(self) -> int:
        return self.heads * self.head_dim

    @property
    def scale(self) -> float:
        return 1.0 / math.sqrt(self.head_dim)

    def gemm_flops_per_row(self) -> int:
        h, i, f = self.hidden, self.inner, self.ffn
        return 2 * (h * 3 * i + i * h + h * 2 * f + f * h)

    def block_flops(self, rows: int) -> int:
        return rows * self.gemm_flops_per_row() + 4 * rows * rows * self.heads * self.head_dim


BLOCK_TENSORS = ("norm1", "norm2", "qkv", "q_norm", "k_norm", "out", "fc1", "fc2", "modulation")


class BlockWeights:
    """The eight checkpoint tensors of a block (h3_dit.c:518-525) + its modulation table."""

    def __init__(self, **tensors: Tensor):
        for name in BLOCK_TENSORS:
            setattr(self, name, tensors[name])


def block_tensor_shapes(s: DitShape, mod_rows: int) -> dict[str, int]:
    return {
        "norm1": s.hidden, "norm2": s.hidden,
        "qkv": 3 * s.inner * s.hidden,
        "q_norm": s.head_dim, "k_norm": s.head_dim,
        "out": s.hidden * s.inner,
        "fc1": 2 * s.ffn * s.hidden,
        "fc2": s.hidden * s.ffn,
        "modulation": mod_rows * s.slots * s.hidden,
    }


def shard_rows(sequence: int, world: int, rank: int) -> tuple[int, int, int]:
    """(rows_local, row_begin, rows_valid): every rank holds rows_local = ceil(S/world) rows;
    the last ranks may hold fewer valid rows, padding sits at the global tail."""
    rows_local = (sequence + world - 1) // world
    begin = min(sequence, rank * rows_local)
    valid = max(0, min(sequence, begin + rows_local) - begin)
    return rows_local, begin, valid


def ulysses_pack_order(rows_local: int, heads: int, world: int) -> np.ndarray:
    """Index map of h3x_ulysses_pack_heads in units of one head vector:
    packed[(p*rows_local + r)*hpr + hl] = src[r*heads + p*hpr + hl]. Host-side layout
    bookkeeping only (tests and buffer sizing); the data movement is the CUDA kernel."""
    hpr = heads // world
    p, r, hl = np.meshgrid(np.arange(world), np.arange(rows_local), np.arange(hpr), indexing="ij")
    return (r * heads + p * hpr + hl).reshape(-1)


class SingleRank:
    """Exchange for world size 1: attention sees the local rows directly."""
    world, rank = 1, 0


class Dit:
    """Activations + op sequence for `rows_local` rows of a (possibly sharded) sequence."""

    def __init__(self, gpu: Gpu, shape: DitShape, sequence: int, exchange=None,
                 alloc=None):
        self.gpu, self.s, self.sequence = gpu, shape, sequence
        self.exchange = exchange or SingleRank()
        world = self.exchange.world
        if shape.heads % world:
            raise ValueError("heads must divide by the number of ranks")
        self.rows_local, self.row_begin, self.rows_valid = shard_rows(sequence, world,
                                                                      self.exchange.rank)
        rows, s = self.rows_local, shape
        # rows the block ops work on: all local rows, or the pooled rows while a token
        # reduction is active (single rank only)
        self.active_rows, self.active_sequence = rows, sequence
        new = alloc or (lambda n: gpu.new(n, BF16))
        self.hidden = new(rows * s.hidden)
        self.mod_attention = new(rows * s.hidden)
        self.push = world > 1 and hasattr(self.exchange, "setup")
        self.qkv = new(rows * max(3 * s.inner, s.hidden))   # also attention_heads and mod_mlp
        self.mod_mlp = self.qkv
        self.attention_output = new(rows * s.hidden)  # also the MLP output
        if self.push:
            # q/k/v land in the owning ranks' gathered buffers, attention output in the owning
            # rank's attention_heads: no local q/k/v, no send/receive staging
            shared = self.exchange.setup(rows, s.heads, s.head_dim)
            self.gathered = [shared["q"], shared["k"], shared["v"]]
            self.attention_heads = shared["o"]
            return
        self.query = new(rows * s.inner)
        self.key = new(rows * s.inner)
        self.value = new(rows * s.inner)
        self.attention_heads = self.qkv
        if world > 1:
            # exchange buffers: [world][rows_local][heads/world][head_dim] x (q, k, v) and o
            n = world * rows * (s.heads // world) * s.head_dim
            self.send = [new(n) for _ in range(3)]
            self.recv = [new(n) for _ in range(3)]
            self.o_gathered = new(n)
            self.o_returned = new(n)

    # ------------------------------------------------------------ attention
    def _attention(self):
        g, s, rows = self.gpu, self.s, self.rows_local
        ex = self.exchange
        if ex.world == 1:
            g.op("sdpa_bf16", self.attention_heads, self.query, self.key, self.value,
                 self.active_sequence, s.heads, s.head_dim, s.scale)
            return
        hpr = s.heads // ex.world
        for src, dst in zip((self.query, self.key, self.value), self.send):
            g.op("h3x_ulysses_pack_heads", dst, src, rows, s.heads, s.head_dim, ex.world)
        for snd, rcv in zip(self.send, self.recv):
            ex.all_to_all(rcv, snd)
        # gathered rows are in global order (rank-major); padding rows, if any, are the tail
        g.op("sdpa_bf16", self.o_gathered, self.recv[0], self.recv[1], self.recv[2],
             self.sequence, hpr, s.head_dim, s.scale)
        ex.all_to_all(self.o_returned, self.o_gathered)
        g.op("h3x_ulysses_unpack_heads", self.attention_heads, self.o_returned, rows, s.heads,
             s.head_dim, ex.world)

    # ---------------------------------------------------------------- block
    def run_block(self, w: BlockWeights, row_map: Tensor, rope_cos: Tensor, rope_sin: Tensor,
                  adaln_ready: bool, next_w: BlockWeights | None) -> bool:
        """One block; returns whether the next block's attention adaLN is already in
        mod_attention (the cross-block fusion of h3_dit.c:2139-2177)."""
        g, s, rows = self.gpu, self.s, self.active_rows
        if not adaln_ready:
            g.op("adaln_bf16", self.mod_attention, self.hidden, w.norm1, w.modulation, row_map,
                 rows, s.hidden, s.slots, 0, 1, s.eps)
        if self.push:
            ex = self.exchange
            g.op("h3x_grouped_qkv_linear_rope_push", ex.peers, self.mod_attention, w.qkv, w.q_norm,
                 w.k_norm, rope_cos, rope_sin, rows, s.hidden, s.heads, s.head_dim, s.rope_half,
                 s.eps)
            ex.barrier()      # every rank's q/k/v rows have arrived
            g.op("h3x_sdpa_push", ex.peers, self.gathered[0], self.gathered[1], self.gathered[2],
                 self.sequence, s.heads, s.head_dim, s.scale)
            ex.barrier()      # every head of this rank's rows has arrived
        else:
            g.op("grouped_qkv_linear_rope_bf16", self.query, self.key, self.value, self.qkv,
                 self.mod_attention, w.qkv, w.q_norm, w.k_norm, rope_cos, rope_sin, rows, s.hidden,
                 s.heads, s.head_dim, s.rope_half, s.eps)
            self._attention()
        g.op("linear_bf16", self.attention_output, self.attention_heads, w.out, None, rows,
             s.inner, s.hidden)
        g.op("gate_adaln_bf16", self.hidden, self.mod_mlp, self.hidden, self.attention_output,
             w.norm2, w.modulation, w.modulation, row_map, rows, s.hidden, s.slots, 2, 3, 4, s.eps)
        g.op("mlp_bf16", self.attention_output, self.mod_mlp, w.fc1, w.fc2, rows, s.hidden, s.ffn,
             s.hidden)
        if next_w is not None:
            g.op("gate_adaln_bf16", self.hidden, self.mod_attention, self.hidden,
                 self.attention_output, next_w.norm1, w.modulation, next_w.modulation, row_map,
                 rows, s.hidden, s.slots, 5, 0, 1, s.eps)
            return True
        g.op("gate_bf16", self.hidden, self.hidden, self.attention_output, w.modulation, row_map,
             rows, s.hidden, s.slots, 5)
        return False

    def run_blocks(self, blocks: list[BlockWeights], row_map: Tensor, rope_cos: Tensor,
                   rope_sin: Tensor, reduction: "TokenReduction | None" = None,
                   reduced_row_map: Tensor | None = None, fused_boundaries: bool = True) -> None:
        """All blocks. With `reduction`, blocks [begin, end) run on the pooled token grid
        (h3_dit.c:2316-2345): pool before block `begin`, expand before block `end` (or after the
        last block); the cross-block adaLN fusion is not carried over either boundary. With
        fused_boundaries (the reference's default) the pool / expand kernel also applies the
        attention adaLN of the block that follows."""
        red = reduction
        if red is not None and self.exchange.world != 1:
            raise ValueError("token reduction is not combined with sequence parallelism")
        ready = False
        for i, w in enumerate(blocks):
            if red is not None and i == red.begin:
                ready = self._enter_reduction(red, w if fused_boundaries else None, reduced_row_map)
            if red is not None and i == red.end:
                ready = self._leave_reduction(red, w if fused_boundaries else None, row_map)
            boundary = red is not None and i + 1 in (red.begin, red.end)
            nxt = blocks[i + 1] if i + 1 < len(blocks) and not boundary else None
            if red is not None and red.active:
                ready = self.run_block(w, reduced_row_map, red.rope_cos, red.rope_sin, ready, nxt)
            else:
                ready = self.run_block(w, row_map, rope_cos, rope_sin, ready, nxt)
            if i == int(len(blocks) * 0.6):
                self.gpu.flush()     # the reference's mid-step command split (h3_dit.c:2403-2406)
        if red is not None and red.active:
            self._leave_reduction(red)

    def _enter_reduction(self, red: "TokenReduction", w: BlockWeights | None = None,
                         reduced_row_map: Tensor | None = None) -> bool:
        """enter_token_reduction / enter_token_reduction_adaln (h3_dit.c:1921-1961): snapshot
        the full rows, pool horizontally adjacent video tokens into attention_output, which
        becomes the hidden state; with the next block's weights also its attention adaLN into
        mod_attention. Returns whether that adaLN is ready."""
        s = self.s
        if w is None:
            self.gpu.op("token_pool_bf16", self.attention_output, self.hidden, 0, red.original, 0,
                        red.baseline, 0, red.baseline_indices, red.pool_pairs, self.sequence,
                        red.reduced_sequence, red.baseline_rows, s.hidden)
        else:
            self.gpu.op("token_pool_adaln_bf16", self.attention_output, self.mod_attention,
                        self.hidden, 0, red.original, 0, red.baseline, 0, red.baseline_indices,
                        red.pool_pairs, w.norm1, w.modulation, reduced_row_map, self.sequence,
                        red.reduced_sequence, red.baseline_rows, s.hidden, s.slots, 0, 1, s.eps)
        self.hidden, self.attention_output = self.attention_output, self.hidden
        self.active_rows = self.active_sequence = red.reduced_sequence
        red.active = True
        return w is not None

    def _leave_reduction(self, red: "TokenReduction", w: BlockWeights | None = None,
                         row_map: Tensor | None = None) -> bool:
        """leave_token_reduction / leave_token_reduction_adaln (h3_dit.c:1963-2006): every full
        row gets its snapshot plus update_scale times what its pooled parent gained. Plain form:
        the result lands in mod_attention, which becomes the hidden state. Fused form: the result
        lands in attention_output (the new hidden state) and the next block's attention adaLN in
        mod_attention."""
        s = self.s
        if w is None:
            self.gpu.op("token_expand_delta_bf16", self.mod_attention, red.original, 0, self.hidden,
                        red.baseline, 0, red.baseline_indices, red.expand_parents, self.sequence,
                        red.reduced_sequence, red.baseline_rows, s.hidden, red.video_start,
                        float(red.scale))
            self.hidden, self.mod_attention = self.mod_attention, self.hidden
        else:
            self.gpu.op("token_expand_adaln_bf16", self.attention_output, self.mod_attention,
                        red.original, 0, self.hidden, red.baseline, 0, red.baseline_indices,
                        red.expand_parents, w.norm1, w.modulation, row_map, self.sequence,
                        red.reduced_sequence, red.baseline_rows, s.hidden, red.video_start,
                        float(red.scale), s.slots, 0, 1, s.eps)
            self.hidden, self.attention_output = self.attention_output, self.hidden
        self.active_rows, self.active_sequence = self.rows_local, self.sequence
        red.active = False
        return w is not None


class TokenReduction:
    """Maps and buffers of the reference's token-reduction mode (h3_dit.c:440-505, 1258-1310):
    between blocks `begin` and `end` every pair of horizontally adjacent video tokens is
    averaged into one (an odd last column stays single); text / conditioning rows before the
    target video are kept. The video must end the row layout.

    video grid: t x h x w tokens (the reference's latent_t x latent_h/2 x latent_w/2)."""

    def __init__(self, gpu: Gpu, shape: DitShape, *, sequence: int, video_start: int, t: int,
                 h: int, w: int, begin: int, end: int, scale: float = 1.0):
        if video_start + t * h * w != sequence or not (0 <= begin < end):
            raise ValueError("the target video must end the row layout and begin < end")
        self.begin, self.end, self.scale, self.video_start = begin, end, scale, video_start
        self.sequence, self.width = sequence, w
        self.reduced_width = (w + 1) // 2
        self.reduced_sequence = video_start + t * h * self.reduced_width
        self.baseline_rows = t * h * w - t * h * self.reduced_width
        self.pairs = np.array([self.pool_sources(r) for r in range(self.reduced_sequence)],
                              np.uint32)
        merged = (np.arange(self.reduced_sequence) >= video_start) & (self.pairs[:, 0] != self.pairs[:, 1])
        indices = np.full(self.reduced_sequence, 0xFFFFFFFF, np.uint32)
        indices[merged] = np.arange(int(merged.sum()), dtype=np.uint32)
        if int(merged.sum()) != self.baseline_rows:
            raise ValueError("token-reduction baseline map is inconsistent")
        self.baseline_index_values = indices
        self.parents = np.array([self.reduced_parent(r) for r in range(sequence)], np.uint32)
        self.pool_pairs = gpu.u32(self.pairs.reshape(-1))
        self.baseline_indices = gpu.u32(indices)
        self.expand_parents = gpu.u32(self.parents)
        self.original = gpu.new(sequence * shape.hidden, BF16)
        self.baseline = gpu.new(max(1, self.baseline_rows) * shape.hidden, BF16)
        self.rope_cos = self.rope_sin = None
        self.active = False

    def pool_sources(self, reduced_row: int) -> tuple[int, int]:
        """token_pool_sources (h3_dit.c:478-494)."""
        if reduced_row < self.video_start:
            return reduced_row, reduced_row
        local = reduced_row - self.video_start
        source = self.video_start + (local // self.reduced_width) * self.width + \
            (local % self.reduced_width) * 2
        second = source + (1 if (source - self.video_start) % self.width + 1 < self.width else 0)
        return source, second

    def reduced_parent(self, full_row: int) -> int:
        """token_reduced_parent (h3_dit.c:496-503)."""
        if full_row < self.video_start:
            return full_row
        local = full_row - self.video_start
        return self.video_start + (local // self.width) * self.reduced_width + (local % self.width) // 2

    def reduced_positions(self, positions: np.ndarray) -> np.ndarray:
        """Positions of the pooled rows: the mean of their two sources (h3_dit.c:930-940)."""
        return ((positions[self.pairs[:, 0]].astype(np.float64) +
                 positions[self.pairs[:, 1]].astype(np.float64)) * 0.5).astype(np.float32)

    def reduced_row_map(self, row_map: np.ndarray) -> np.ndarray:
        """Modulation row of a pooled row = that of its first source (h3_dit.c:1164-1171)."""
        return np.ascontiguousarray(row_map[self.pairs[:, 0]], np.uint32)

    def set_rope(self, rope_cos: Tensor, rope_sin: Tensor) -> None:
        self.rope_cos, self.rope_sin = rope_cos, rope_sin


class DenoiseStep:
    """encode_forward for a video(+text) layout: patch projection into `hidden`, text rows
    copied in, the blocks, the final head, and (optionally) the Euler update."""

    def __init__(self, dit: Dit, blocks: list[BlockWeights], *, video_rows: int, text_rows: int,
                 patch_weight: Tensor, patch_bias: Tensor, text_hidden: Tensor,
                 final_norm: Tensor, final_modulation: Tensor, final_weight: Tensor,
                 final_bias: Tensor, row_map: Tensor, final_row_map: Tensor, rope_cos: Tensor,
                 rope_sin: Tensor):
        self.dit, self.blocks = dit, blocks
        self.video_rows, self.text_rows = video_rows, text_rows
        self.patch_weight, self.patch_bias, self.text_hidden = patch_weight, patch_bias, text_hidden
        self.final_norm, self.final_modulation = final_norm, final_modulation
        self.final_weight, self.final_bias = final_weight, final_bias
        self.row_map, self.final_row_map = row_map, final_row_map
        self.rope_cos, self.rope_sin = rope_cos, rope_sin
        g, s = dit.gpu, dit.s
        self.latent = g.new(max(1, video_rows) * s.video_patch, F32)       # patchified video rows
        self.velocity = g.new(max(1, video_rows) * s.video_patch, BF16)
        self.inverse = g.new(max(1, video_rows), F32)

    def forward(self) -> None:
        """Text rows first, then video rows (layout order of h3_layout_build: text segment
        first, video target last). On a sharded run each rank projects its own video rows."""
        d, g, s = self.dit, self.dit.gpu, self.dit.s
        if self.text_rows:
            g.op("copy_bf16", d.hidden, 0, self.text_hidden, 0, self.text_rows * s.hidden)
        if self.video_rows:
            g.op("patch_linear_bf16_offset", d.hidden, self.text_rows * s.hidden, self.latent, 0,
                 self.patch_weight, self.patch_bias, self.video_rows, s.video_patch, s.hidden)
        d.run_blocks(self.blocks, self.row_map, self.rope_cos, self.rope_sin)
        if self.video_rows:
            g.op("adaln_linear_bf16", self.velocity, self.inverse, d.hidden,
                 self.text_rows * s.hidden, self.final_norm, self.final_modulation,
                 self.final_row_map, self.final_weight, self.final_bias, self.video_rows, s.hidden,
                 s.video_patch, s.final_slots, 0, 1, s.eps)

    def euler(self, delta: float, ratio: float = 0.0, previous: Tensor | None = None) -> None:
        """sample += delta * (last + ratio * (last - previous)) (h3_gpu_euler_bf16)."""
        if self.video_rows:
            self.dit.gpu.op("euler_bf16", self.latent, 0, self.velocity, previous or self.velocity,
                            self.video_rows * self.dit.s.video_patch, delta, ratio)


def serving_sigmas(evaluations: int, shift: float = 12.0) -> np.ndarray:
    """sigma[0..evaluations] of h3_serving_schedule_build (h3_host.c:152-167) for the video
    stream (shift 12, h3_host.h:12), in F32 arithmetic like the reference."""
    f = np.float32
    out = np.zeros(evaluations + 1, np.float32)
    for i in range(evaluations):
        base = f(1.0) - f(i) / f(evaluations)
        out[i] = f(shift) * base / (f(1.0) + (f(shift) - f(1.0)) * base)
    return out


def reuse_schedule(steps: int, reuse_interval: int) -> list[int]:
    """Which steps evaluate the model (h3_dit_reuse_schedule, h3_dit.c:2672-2688): the first,
    the last and every reuse_interval-th; the others reuse an extrapolated velocity."""
    if steps < 1 or not 1 <= reuse_interval <= 32:
        raise ValueError("steps >= 1 and 1 <= reuse_interval <= 32")
    return [int(reuse_interval == 1 or i == 0 or i == steps - 1 or i % reuse_interval == 0)
            for i in range(steps)]


def extrapolation_ratio(current_sigma: float, last_sigma: float, previous_sigma: float,
                        have_previous: bool) -> float:
    """Linear extrapolation weight of the velocity in sigma, clamped to [-2, 2]
    (h3_dit.c:2644-2655), in F32 arithmetic like the reference."""
    if not have_previous:
        return 0.0
    f = np.float32
    denominator = f(last_sigma) - f(previous_sigma)
    ratio = (f(current_sigma) - f(last_sigma)) / denominator if denominator != 0 else f(0.0)
    return float(min(f(2.0), max(f(-2.0), ratio)))


class EulerSampler:
    """The device-resident Euler loop of denoise_euler_gpu (h3_dit.c:2805-2893) with every
    step evaluated: per step the forward with that step's time row, then
    sample += (sigma[i] - sigma[i+1]) * velocity; one submit at the end, flush hints between.

    Classifier-free guidance (no counterpart in the reference) replaces the velocity by
    uncond + guidance * (cond - uncond) before the update, in one of two ways:
      * `uncond_text`: this rank (group) evaluates both branches one after the other;
      * `pair`: this rank evaluates one branch (pair.is_cond says which) and swaps velocities
        with the matching rank of the other group through pair.swap(out, inp)."""

    def __init__(self, step: DenoiseStep, sigmas: np.ndarray, row_maps: list[Tensor],
                 final_row_maps: list[Tensor], *, guidance: float | None = None,
                 uncond_text: Tensor | None = None, pair=None, reuse_interval: int = 1):
        self.step, self.sigmas = step, np.asarray(sigmas, np.float32)
        self.selected = reuse_schedule(len(self.sigmas) - 1, reuse_interval)
        self.reuse_interval = reuse_interval
        self.previous_velocity = None
        if reuse_interval > 1:
            self.previous_velocity = step.dit.gpu.new(
                max(1, step.video_rows) * step.dit.s.video_patch, BF16)
        self.row_maps, self.final_row_maps = row_maps, final_row_maps
        self.guidance, self.uncond_text, self.pair = guidance, uncond_text, pair
        if guidance is not None and (uncond_text is None) == (pair is None):
            raise ValueError("guidance needs exactly one of uncond_text and pair")
        self.other = None
        if guidance is not None:
            self.other = step.dit.gpu.new(max(1, step.video_rows) * step.dit.s.video_patch, BF16)

    def _velocity(self, index: int) -> None:
        st, g = self.step, self.step.dit.gpu
        st.row_map, st.final_row_map = self.row_maps[index], self.final_row_maps[index]
        st.forward()
        if self.guidance is None:
            return
        n = st.video_rows * st.dit.s.video_patch
        if self.pair is not None:
            self.pair.swap(self.other, st.velocity)
            cond, uncond = (st.velocity, self.other) if self.pair.is_cond else (self.other, st.velocity)
        else:
            if n:
                g.op("copy_bf16", self.other, 0, st.velocity, 0, n)
            text, st.text_hidden = st.text_hidden, self.uncond_text
            st.forward()
            st.text_hidden = text
            cond, uncond = self.other, st.velocity
        if n:
            g.op("h3x_cfg_combine_bf16", st.velocity, cond, uncond, n, float(self.guidance))

    def run(self) -> None:
        """With reuse_interval > 1 only the selected steps evaluate the model; the others apply
        the last velocity extrapolated linearly in sigma from the last two evaluations
        (h3_dit.c:2805-2863)."""
        st, g, sig = self.step, self.step.dit.gpu, self.sigmas
        steps = len(sig) - 1
        n = st.video_rows * st.dit.s.video_patch
        last, previous = -1, -1
        g.begin()
        for i in range(steps):
            evaluate = self.selected[i]
            if evaluate:
                if last >= 0 and self.reuse_interval > 1:
                    if n:
                        g.op("copy_bf16", self.previous_velocity, 0, st.velocity, 0, n)
                    previous = last
                self._velocity(i)
                last = i
            ratio = 0.0 if evaluate else extrapolation_ratio(
                sig[i], sig[last], sig[previous] if previous >= 0 else 0.0, previous >= 0)
            st.euler(float(sig[i] - sig[i + 1]), ratio,
                     self.previous_velocity if previous >= 0 else None)
            if evaluate and i + 1 < steps:
                g.flush()
        g.submit()


# ------------------------------------------------------------------ synthetic inputs

def grid_positions(text_rows: int, t: int, h: int, w: int) -> np.ndarray:
    """Positions (t, h, w) per row: text rows (index, 0, 0), then an integer t x h x w video grid."""
    pos = np.zeros((text_rows + t * h * w, 3), np.float32)
    pos[:text_rows, 0] = np.arange(text_rows)
    tt, hh, ww = np.meshgrid(np.arange(t), np.arange(h), np.arange(w), indexing="ij")
    pos[text_rows:, 0] = tt.reshape(-1)
    pos[text_rows:, 1] = hh.reshape(-1)
    pos[text_rows:, 2] = ww.reshape(-1)
    return pos


def default_inv_freq() -> np.ndarray:
    """Stand-in for the checkpoint tensor rope.inv_freq[16] (h3_dit.c:887)."""
    return (10000.0 ** (-np.arange(16, dtype=np.float64) / 16.0)).astype(np.float32)


def row_map_for(text_rows: int, video_rows: int, time_row: int = 0) -> np.ndarray:
    """row_map[row] = time_row * 3 + modality tag (video 0, text 1, audio 2;
    h3_dit_schedule.c:448-482)."""
    tags = np.concatenate([np.full(text_rows, 1, np.uint32), np.zeros(video_rows, np.uint32)])
    return (time_row * 3 + tags).astype(np.uint32)
