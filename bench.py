#!/usr/bin/env python3
"""Benchmark of the H3 DiT denoise step on B200 through libh3b200.so.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3|c4|c1|ref512|ref864]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference        # the CPU arm (oracle port on the host cores)

A step = one full 50-block denoiser forward (patch projection, 50 blocks, final head, Euler
update) on synthetic latents with random-init weights. Default workload: BASELINE config 3,
512x512x22 frames = 6,144 video + 256 text rows (S = 6,400). With N > 1 the sequence is
sharded by rows (Ulysses sequence parallelism: all-to-all over NCCL around attention) and
the same workload is strong-scaled.

Prints ONE JSON line (rank 0): ms per step (max over ranks, CUDA events), the fraction of the
measured BF16 tensor peak, an end-to-end number with host<->device copies inside the timed
region, the live roofline of the dominant kernel, a bounded CPU baseline, and sampled clocks.
PyTorch is used only for device memory, streams/events and torch.distributed.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (text rows, video rows, description)
    "c1": (128, 1536, "one-block config: 1,536 video + 128 text rows"),
    "c3": (256, 6144, "512x512x22f: 6,144 video + 256 text rows (S=6,400), 50 blocks"),
    "c4": (256, 50220, "864x480x121f: 50,220 video + 256 text rows (S=50,476), 50 blocks"),
    "ref512": (256, 1792 + 74, "reference-true 512x512x22f layout: 1,866 video/audio + 256 text rows"),
    "ref864": (256, 14985 + 414, "reference-true 864x480x124f layout: 15,399 video/audio + 256 text rows"),
    "c3_eighth": (256, 544, "an eighth of the 512x512x22f rows (S=800: the per-rank GEMM size of c3 on 8 GPUs), 50 blocks"),
    "c4_quarter": (256, 12363, "a quarter of the 864x480x121f rows (S=12,619: the per-rank GEMM size of c4 on 4 GPUs), 50 blocks"),
    "c5": (256, 50220, "864x480x121f (S=50,476), 20 Euler steps with classifier-free guidance, "
                       "cond/uncond on two GPU groups, 50 blocks"),
    "c5small": (256, 6144, "512x512x22f (S=6,400), 20 Euler steps with classifier-free guidance, "
                           "cond/uncond on two GPU groups, 50 blocks"),
    "vae_tile": (0, 1797, "one tile of the video-VAE decoder (the step after the DiT): metric vae_tile_decode_ms"),
}


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the roofline kernel (fc1 + SwiGLU)
# from an ncu capture of this file with --blocks 1; (workload, ranks) -> bytes. Configurations
# without a capture report "traffic": null. To be re-captured whenever the GEMM tile walk changes.
NCU_DRAM_BYTES_PER_LAUNCH = {("c3", 1): 1148.4e6}
NCU_DRAM_SOURCE = ("one ncu capture of `bench.py --blocks 1` on a B200 (dram read 970.3 MB + write 178.1 MB for "
                   "the fc1 + SwiGLU launch; summary in profiles/h3b_gemm_dram_traffic_c3.md)")


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"],
                "hbm_gbs": d["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0,
            "source": "fallback"}


# ------------------------------------------------------------------ CPU arm

def cpu_sample(shape, sequence, gemm_rows=256, attn_rows=128):
    """Time the oracle port on a bounded sample of one block and extrapolate to a step.

    GEMMs and row ops: `gemm_rows` rows of the block (cost is linear in rows).
    Attention: `attn_rows` query rows against all `sequence` keys, all heads (linear in
    query rows). Returns (ms per step extrapolated, description, threads, seconds spent)."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import h3_oracle as o
    # a launcher may have exported OMP_NUM_THREADS=1 (torch.distributed.run does): the baseline
    # uses every core this process may run on
    o.set_threads(len(os.sched_getaffinity(0)))
    s = shape
    rng = np.random.default_rng(0)

    def rand(n, std):
        out = np.empty(n, np.uint16)
        for i in range(0, n, 1 << 22):
            m = min(1 << 22, n - i)
            out[i:i + m] = o.to_bf16(rng.standard_normal(m, dtype=np.float32) * np.float32(std))
        return out

    gemm_rows = min(gemm_rows, sequence)
    attn_rows = min(attn_rows, sequence)
    x = rand(gemm_rows * s.hidden, 1.0)
    w_qkv, w_out = rand(3 * s.inner * s.hidden, 0.02), rand(s.hidden * s.inner, 0.02)
    w_fc1, w_fc2 = rand(2 * s.ffn * s.hidden, 0.02), rand(s.hidden * s.ffn, 0.02)
    mod = rand(3 * s.slots * s.hidden, 0.3)
    norm = o.to_bf16(np.ones(s.hidden, np.float32))
    hn = o.to_bf16(np.ones(s.head_dim, np.float32))
    row_map = np.zeros(gemm_rows, np.uint32)
    cos, sin = rand(gemm_rows * s.rope_half, 0.7), rand(gemm_rows * s.rope_half, 0.7)
    t0 = time.perf_counter()
    m = o.adaln_bf16(x, norm, mod, row_map, gemm_rows, s.hidden, s.slots, 0, 1)
    qkv = o.linear_bf16(m, w_qkv, None, gemm_rows, s.hidden, 3 * s.inner)
    q, k, v = o.qkv_rope_bf16(qkv, hn, hn, cos, sin, gemm_rows, s.heads, s.head_dim, s.rope_half, 1)
    br = o.linear_bf16(q, w_out, None, gemm_rows, s.inner, s.hidden)
    x2, m2 = o.gate_adaln_bf16(x, br, norm, mod, mod, row_map, gemm_rows, s.hidden, s.slots, 2, 3, 4)
    y = o.mlp_bf16(m2, w_fc1, w_fc2, gemm_rows, s.hidden, s.ffn, s.hidden)
    o.gate_bf16(x2, y, mod, row_map, gemm_rows, s.hidden, s.slots, 5)
    t_rows = time.perf_counter() - t0
    n = sequence * s.inner
    qa, ka, va = rand(n, 1.0), rand(n, 1.0), rand(n, 1.0)
    t0 = time.perf_counter()
    o.sdpa_bf16(qa, ka, va, sequence, s.heads, s.head_dim, s.scale, 0, 1, rows=(0, attn_rows))
    t_attn = time.perf_counter() - t0
    block_s = t_rows * sequence / gemm_rows + t_attn * sequence / attn_rows
    desc = (f"one block: GEMMs+row ops on {gemm_rows} of {sequence} rows, attention for {attn_rows} "
            f"query rows x {sequence} keys x {s.heads} heads; extrapolated linearly to {s.blocks} blocks")
    return block_s * s.blocks * 1e3, desc, o.threads(), t_rows + t_attn


REF_CUDA = ROOT / "oracle" / "_ref" / "libh3ref.so"


def reference_cuda_block(shape, sequence, text_rows, repeats=10):
    """One DiT block at the workload's S through the reference's own CUDA backend (its sources
    compiled as a checker under oracle/_ref: cuBLASLt GEMMs, mma.sync attention, unfused row
    kernels), driven by the same host sequence: the kernel path to beat on the same GPU.
    Returns None when the library or a GPU is absent."""
    try:
        import torch
        if not (REF_CUDA.exists() and torch.cuda.is_available()):
            return None
        import __graft_entry__ as entry
        pkg = entry.load_package()
        gpu = pkg.Gpu(0, lib_path=REF_CUDA)
    except Exception as err:                       # the supplementary figure must not sink the arm
        return {"unavailable": str(err)[:200]}
    try:
        s = shape
        rng = np.random.default_rng(0)

        def normal(n, std):
            out = np.empty(n, np.uint16)
            for i in range(0, n, 1 << 24):
                m = min(1 << 24, n - i)
                f = (rng.standard_normal(m, dtype=np.float32) * np.float32(std)).view(np.uint32)
                out[i:i + m] = ((f + 0x7fff + ((f >> 16) & 1)) >> 16).astype(np.uint16)
            return out
        one = np.uint16(0x3f80)
        t = {}
        for name, count in pkg.block_tensor_shapes(s, 6).items():
            if name in ("norm1", "norm2", "q_norm", "k_norm"):
                t[name] = gpu.bf16(np.full(count, one, np.uint16))
            else:
                t[name] = gpu.bf16(normal(count, 0.13 if name == "modulation" else 0.02))
        w = pkg.BlockWeights(**t)
        dit = pkg.Dit(gpu, s, sequence)
        dit.hidden.write(normal(sequence * s.hidden, 1.0))
        row_map = gpu.u32(np.concatenate([np.full(text_rows, 4, np.uint32),
                                          np.full(sequence - text_rows, 3, np.uint32)]))
        pos = pkg.grid_positions(text_rows, max(1, -(-(sequence - text_rows) // 1024)), 32, 32)[:sequence]
        ang = pos[:, :, None] * pkg.default_inv_freq()[None, None, :]
        tables = []
        for fn in (np.cos, np.sin):
            f = fn(ang).reshape(-1).astype(np.float32).view(np.uint32)
            tables.append(gpu.bf16(((f + 0x7fff + ((f >> 16) & 1)) >> 16).astype(np.uint16)))
        import torch
        for _ in range(2):
            gpu.begin(); dit.run_block(w, row_map, tables[0], tables[1], False, None); gpu.submit()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        gpu.begin()
        a.record()
        for _ in range(repeats):
            dit.run_block(w, row_map, tables[0], tables[1], False, None)
        b.record()
        gpu.submit()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / repeats
        return {"ms_per_block": ms, "ms_per_step_extrapolated": ms * s.blocks,
                "tflops": s.block_flops(sequence) / (ms * 1e-3) / 1e12,
                "what": "one block through oracle/_ref/libh3ref.so (the reference's CUDA backend, sm_100 build), "
                        f"CUDA events, mean of {repeats}; step = block x {s.blocks}"}
    except Exception as err:
        return {"unavailable": str(err)[:200]}
    finally:
        gpu.close()


def run_reference_arm(args, shape, sequence):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    values, spent, desc, threads = [], 0.0, "", 1
    for i in range(args.warmup + args.steps):
        ms, desc, threads, sec = cpu_sample(shape, sequence, gemm_rows=128, attn_rows=64)
        spent += sec
        if i >= args.warmup:
            values.append(ms)
    value = statistics.mean(values)
    line = {
        "impl": "reference", "metric": "dit_denoise_step_ms", "value": value, "unit": "ms/step",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": value,
        "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(args, sequence),
        "cpu_baseline": {"value": value, "unit": "ms/step", "cores": threads, "kind": "port",
                         "sample": desc, "note": "the reference has no CPU implementation of the DiT; "
                         "this is the oracle port of its CPU test references, OpenMP over rows/heads"},
        "e2e": {"value": value, "unit": "ms/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if sequence <= 8192:      # supplementary: the reference's GPU path on this box (value stays the CPU arm)
        line["reference_cuda_backend"] = reference_cuda_block(shape, sequence, WORKLOADS[args.workload][0])
    print(json.dumps(line), flush=True)


def workload_config(args, sequence):
    text, video, desc = WORKLOADS[args.workload]
    return {"workload": f"{args.workload}: {desc}", "rows": sequence, "blocks": args.blocks,
            "parallelism": f"sp{args.gpus}" if args.gpus > 1 else "single",
            "l2": "weights (770 MB per block) and activations exceed the 126 MB L2 between reuses"}


# -------------------------------------------------------------- clock sampling

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.proc, self.path = device, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.device), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in Path(self.path).read_text().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------- GPU arm

class Weights:
    """Random-init weights of the architecture, shared by every workload of a run."""


def build_weights(torch, pkg, gpu, mem, shape, time_rows=2, seed=0):
    """50 blocks (770 MB each), modulation tables computed by the adaLN projection (rows = time
    rows, 2688 -> 3*6*5376: the load-time GEMM of the reference's h3_dit_schedule_precompute,
    h3_dit_schedule.c:264-301), final head and patch projection."""
    s = shape
    w = Weights()
    w.time_rows = time_rows
    gen = torch.Generator(device=mem.device)
    gen.manual_seed(seed)
    w.generator = gen
    w.silu_time = mem.bf16(time_rows * s.time_dim, std=0.125, generator=gen)   # modulation std ~0.13
    mod_cols = s.modalities * s.slots * s.hidden
    w.proj_w = mem.bf16(mod_cols * s.time_dim)
    w.proj_b = mem.bf16(mod_cols)
    w.blocks = []
    for _ in range(s.blocks):
        t = {}
        for name, count in pkg.block_tensor_shapes(s, time_rows * s.modalities).items():
            if name in ("norm1", "norm2", "q_norm", "k_norm"):
                t[name] = mem.bf16(count, fill=1.0)
            elif name == "modulation":
                t[name] = mem.bf16(count)
            else:
                t[name] = mem.bf16(count, std=0.02, generator=gen)
        mem.torch_of(w.proj_w).normal_(0.0, 0.02, generator=gen)
        mem.torch_of(w.proj_b).normal_(0.0, 0.02, generator=gen)
        gpu.begin()
        gpu.op("linear_bf16", t["modulation"], w.silu_time, w.proj_w, w.proj_b, time_rows, s.time_dim, mod_cols)
        gpu.submit()
        w.blocks.append(pkg.BlockWeights(**t))
    w.final_mod = mem.bf16(time_rows * s.final_slots * s.hidden, std=0.3, generator=gen)
    w.final_w = mem.bf16(s.video_patch * s.hidden, std=0.02, generator=gen)
    w.final_b = mem.bf16(s.video_patch, std=0.02, generator=gen)
    w.final_norm = mem.bf16(s.hidden, fill=1.0)
    w.patch_w = mem.f32(s.hidden * s.video_patch, std=0.02, generator=gen)
    w.patch_b = mem.f32(s.hidden, std=0.02, generator=gen)
    return w


def workload_positions(sequence, text_rows, padded_rows):
    """(t, h, w) per global row: text rows (index, 0, 0), then video rows on a t x 32 x 32 grid."""
    video_rows_total = sequence - text_rows
    pos = np.zeros((padded_rows, 3), np.float32)
    pos[:text_rows, 0] = np.arange(text_rows)
    idx = np.arange(video_rows_total)
    pos[text_rows:sequence, 0] = idx // 1024 if video_rows_total >= 1024 else 0
    pos[text_rows:sequence, 1] = (idx % 1024) // 32
    pos[text_rows:sequence, 2] = idx % 32
    return pos


def build_workload(torch, pkg, gpu, mem, shape, w, sequence, text_rows, exchange, text_seed=None):
    """Activations, rope tables, row maps and the denoise step of one workload (this rank's row
    slice: text rows first, then video rows) on the shared weights."""
    s = shape
    dit = pkg.Dit(gpu, s, sequence, exchange=exchange, alloc=lambda n: mem.bf16(n))
    text_gen = w.generator
    if text_seed is not None:
        text_gen = torch.Generator(device=mem.device)
        text_gen.manual_seed(text_seed)
    text_hidden = mem.bf16(max(1, text_rows) * s.hidden, std=1.0, generator=text_gen)
    r0, rows = dit.row_begin, dit.rows_local
    world = dit.exchange.world
    pos = workload_positions(sequence, text_rows, dit.rows_local * world)
    local = pos[r0:r0 + rows]
    ang = local[:, :, None] * pkg.default_inv_freq()[None, None, :]          # [rows, 3 axes, 16 freqs]
    cos = torch.from_numpy(np.cos(ang).reshape(rows, 48).astype(np.float32))
    sin = torch.from_numpy(np.sin(ang).reshape(rows, 48).astype(np.float32))
    rope_cos, rope_sin = mem.bf16(rows * 48), mem.bf16(rows * 48)
    mem.torch_of(rope_cos).copy_(cos.reshape(-1).to(torch.bfloat16))
    mem.torch_of(rope_sin).copy_(sin.reshape(-1).to(torch.bfloat16))
    tags = np.zeros(dit.rows_local * world, np.uint32)
    tags[:text_rows] = 1
    local_text = max(0, min(text_rows, r0 + dit.rows_valid) - r0)
    local_video = dit.rows_valid - local_text
    # one row map per time row (row_map[row] = time_row * 3 + modality tag); a single-step
    # measurement uses time row 1
    row_maps = [gpu.u32(tags[r0:r0 + rows] + 3 * t) for t in range(w.time_rows)]
    final_row_maps = [gpu.u32(np.full(max(1, local_video), t, np.uint32)) for t in range(w.time_rows)]
    step = pkg.DenoiseStep(dit, w.blocks, video_rows=local_video, text_rows=local_text,
                           patch_weight=w.patch_w, patch_bias=w.patch_b, text_hidden=text_hidden,
                           final_norm=w.final_norm, final_modulation=w.final_mod, final_weight=w.final_w,
                           final_bias=w.final_b, row_map=row_maps[min(1, w.time_rows - 1)],
                           final_row_map=final_row_maps[min(1, w.time_rows - 1)],
                           rope_cos=rope_cos, rope_sin=rope_sin)
    step.row_maps, step.final_row_maps = row_maps, final_row_maps
    return dit, step


def time_kernel(torch, gpu, fn, work, repeats=8):
    """Average duration of one launch, CUDA events on the launching (default) stream.
    Returns (ms, work per second / 1e12): TFLOP/s for flops, TB/s for bytes."""
    for _ in range(2):
        gpu.begin(); fn(); gpu.submit()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gpu.begin()
    start.record()
    for _ in range(repeats):
        fn()
    stop.record()
    gpu.submit()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / repeats
    return ms, work / (ms * 1e-3) / 1e12


def kernel_timings(torch, pkg, gpu, shape, dit, step, exchange, sequence, world, repeats=8):
    """The block's hot kernels timed alone on this rank's rows: name -> (ms, TFLOP/s)."""
    s, rows, w = shape, dit.rows_local, step.blocks[0]
    out = {}
    qkv_flops = 2.0 * rows * s.hidden * 3 * s.inner
    if dit.push:
        def qkv_op():
            gpu.op("h3x_grouped_qkv_linear_rope_push", exchange.peers, dit.mod_attention, w.qkv,
                   w.q_norm, w.k_norm, step.rope_cos, step.rope_sin, rows, s.hidden, s.heads,
                   s.head_dim, s.rope_half, s.eps)
    else:
        def qkv_op():
            gpu.op("grouped_qkv_linear_rope_bf16", dit.query, dit.key, dit.value, dit.qkv,
                   dit.mod_attention, w.qkv, w.q_norm, w.k_norm, step.rope_cos, step.rope_sin,
                   rows, s.hidden, s.heads, s.head_dim, s.rope_half, s.eps)
    out["qkv_proj_norm_rope"] = time_kernel(torch, gpu, qkv_op, qkv_flops, repeats)
    # the MLP's two launches; the activation lands in the (idle) qkv buffer
    out["mlp_fc1_swiglu"] = time_kernel(
        torch, gpu, lambda: gpu.op("h3x_linear_swiglu_bf16", dit.qkv, dit.mod_attention, w.fc1, rows,
                                   s.hidden, s.ffn), 2.0 * rows * s.hidden * 2 * s.ffn, repeats)
    out["mlp_fc2"] = time_kernel(
        torch, gpu, lambda: gpu.op("linear_bf16", dit.attention_output, dit.qkv, w.fc2, None, rows,
                                   s.ffn, s.hidden), 2.0 * rows * s.ffn * s.hidden, repeats)
    out["gemm_out_proj"] = time_kernel(
        torch, gpu, lambda: gpu.op("linear_bf16", dit.attention_output, dit.attention_heads, w.out,
                                   None, rows, s.inner, s.hidden), 2.0 * rows * s.inner * s.hidden, repeats)
    if dit.push:
        attn_flops = 4.0 * sequence * sequence * (s.heads // world) * s.head_dim
        out["attention"] = time_kernel(
            torch, gpu, lambda: gpu.op("h3x_sdpa_push", exchange.peers, dit.gathered[0],
                                       dit.gathered[1], dit.gathered[2], sequence, s.heads,
                                       s.head_dim, s.scale), attn_flops, repeats)
    elif world == 1:
        attn_flops = 4.0 * sequence * sequence * s.heads * s.head_dim
        out["attention"] = time_kernel(
            torch, gpu, lambda: gpu.op("sdpa_bf16", dit.attention_heads, dit.query, dit.key,
                                       dit.value, sequence, s.heads, s.head_dim, s.scale),
            attn_flops, repeats)
    return out


def reference_cuda_ops(torch, pkg, gpu, shape, dit, step, sequence, rounds=3, repeats=8):
    """The same projections and attention through the reference's CUDA backend (cuBLASLt GEMMs,
    mma.sync attention; oracle/_ref/libh3ref.so) on the same GPU, timed back to back with this
    library's launch of the same op: per op `rounds` alternations of (ours x repeats, theirs x
    repeats), CUDA events, so both see the same clocks and temperature. Returns
    name -> {"ms": ours, "reference_cuda_ms": theirs}. The reference's linears carry no fused
    epilogue (its norm + RoPE and its SwiGLU are separate kernels, not timed here), so its
    figure is a lower bound of what it spends on the op this library does in one launch."""
    if not REF_CUDA.exists():
        return None
    s, rows, w = shape, dit.rows_local, step.blocks[0]
    ref = pkg.Gpu(gpu.device, lib_path=REF_CUDA)
    try:
        def copy(tensor, elements):
            return ref.bf16(tensor.read(elements))
        x = copy(dit.mod_attention, rows * s.hidden)
        heads_in = copy(dit.query, rows * s.inner)
        wide = ref.new(rows * 2 * s.ffn, pkg.BF16)
        act = copy(dit.qkv, rows * s.ffn)
        narrow = ref.new(rows * s.hidden, pkg.BF16)
        weights = {n: copy(getattr(w, n), c) for n, c in
                   (("qkv", 3 * s.inner * s.hidden), ("out", s.hidden * s.inner),
                    ("fc1", 2 * s.ffn * s.hidden), ("fc2", s.hidden * s.ffn))}
        q, k, v = (copy(t, rows * s.inner) for t in (dit.query, dit.key, dit.value))
        norms = [copy(w.q_norm, s.head_dim), copy(w.k_norm, s.head_dim)]
        ropes = [copy(step.rope_cos, rows * s.rope_half), copy(step.rope_sin, rows * s.rope_half)]
        rq, rk, rv = (ref.new(rows * s.inner, pkg.BF16) for _ in range(3))
        theirs = {
            # like for like: its projection followed by its norm + RoPE kernel, as its host calls it
            "qkv_proj_norm_rope": lambda: ref.op("grouped_qkv_linear_rope_bf16", rq, rk, rv, wide, x,
                                                 weights["qkv"], *norms, *ropes, rows, s.hidden,
                                                 s.heads, s.head_dim, s.rope_half, s.eps),
            "qkv_gemm_only": lambda: ref.op("linear_bf16", wide, x, weights["qkv"], None, rows,
                                            s.hidden, 3 * s.inner),
            # its whole MLP (two cuBLASLt GEMMs + a SwiGLU pass) against this library's two launches
            "mlp_fc1_swiglu_fc2": lambda: ref.op("mlp_bf16", narrow, x, weights["fc1"], weights["fc2"],
                                                 rows, s.hidden, s.ffn, s.hidden),
            "mlp_fc1_swiglu": lambda: ref.op("linear_bf16", wide, x, weights["fc1"], None, rows,
                                             s.hidden, 2 * s.ffn),
            "mlp_fc2": lambda: ref.op("linear_bf16", narrow, act, weights["fc2"], None, rows, s.ffn,
                                      s.hidden),
            "gemm_out_proj": lambda: ref.op("linear_bf16", narrow, heads_in, weights["out"], None,
                                            rows, s.inner, s.hidden),
            "attention": lambda: ref.op("sdpa_bf16", heads_in, q, k, v, sequence, s.heads,
                                        s.head_dim, s.scale),
        }
        ours = {
            "qkv_proj_norm_rope": lambda: gpu.op(
                "grouped_qkv_linear_rope_bf16", dit.query, dit.key, dit.value, dit.qkv, dit.mod_attention,
                w.qkv, w.q_norm, w.k_norm, step.rope_cos, step.rope_sin, rows, s.hidden, s.heads,
                s.head_dim, s.rope_half, s.eps),
            "mlp_fc1_swiglu": lambda: gpu.op("h3x_linear_swiglu_bf16", dit.qkv, dit.mod_attention, w.fc1,
                                             rows, s.hidden, s.ffn),
            "mlp_fc1_swiglu_fc2": lambda: gpu.op("mlp_bf16", dit.attention_output, dit.mod_attention, w.fc1,
                                                 w.fc2, rows, s.hidden, s.ffn, s.hidden),
            "mlp_fc2": lambda: gpu.op("linear_bf16", dit.attention_output, dit.qkv, w.fc2, None, rows,
                                      s.ffn, s.hidden),
            "gemm_out_proj": lambda: gpu.op("linear_bf16", dit.attention_output, dit.attention_heads,
                                            w.out, None, rows, s.inner, s.hidden),
            "attention": lambda: gpu.op("sdpa_bf16", dit.attention_heads, dit.query, dit.key, dit.value,
                                        sequence, s.heads, s.head_dim, s.scale),
        }
        ours["qkv_gemm_only"] = ours["qkv_proj_norm_rope"]     # this library has no unfused form to time
        out = {}
        for name in theirs:
            a, b = [], []
            for _ in range(rounds):
                a.append(time_kernel(torch, gpu, ours[name], 0.0, repeats)[0])
                b.append(time_kernel(torch, ref, theirs[name], 0.0, repeats)[0])
            out[name] = {"ms": statistics.mean(a), "reference_cuda_ms": statistics.mean(b)}
        out["qkv_gemm_only"]["note"] = ("reference: the cuBLASLt projection alone; ms: this library's fused "
                                        "projection + head norm + RoPE launch")
        return out
    except Exception as err:                      # a supplementary figure must not sink the run
        return {"unavailable": str(err)[:200]}
    finally:
        ref.close()


PARITY_ROWS, PARITY_TEXT = 1664, 128


def parity_vs_single(torch, dist, pkg, gpu, mem, shape, weights, make_exchange, world, rank):
    """One full-width block (hidden 5376, 56 heads) at S = 1,664 sharded over the ranks, against
    the same block unsharded on rank 0 (weights are replicated, so rank 0 has everything).
    Returns {"rel_l2", "max_abs", "ok"} on rank 0 (bar: 1e-2 / 5e-2), None elsewhere."""
    s, seq = shape, PARITY_ROWS
    w = weights.blocks[0]
    rng = np.random.default_rng(7)
    f = rng.standard_normal(seq * s.hidden, dtype=np.float32).view(np.uint32)
    hidden = ((f + 0x7fff + ((f >> 16) & 1)) >> 16).astype(np.uint16)

    def run(exchange):
        dit, step = build_workload(torch, pkg, gpu, mem, s, weights, seq, PARITY_TEXT, exchange)
        local = np.zeros(dit.rows_local * s.hidden, np.uint16)
        local[:dit.rows_valid * s.hidden] = hidden[dit.row_begin * s.hidden:
                                                   (dit.row_begin + dit.rows_valid) * s.hidden]
        dit.hidden.write(local)
        gpu.begin()
        dit.run_block(w, step.row_map, step.rope_cos, step.rope_sin, False, None)
        gpu.submit()
        return dit, mem.torch_of(dit.hidden).view(torch.bfloat16)

    exchange = make_exchange()
    dit, mine = run(exchange)
    gathered = torch.empty(world * mine.numel(), dtype=torch.bfloat16, device=mine.device)
    dist.all_gather_into_tensor(gathered, mine.contiguous())
    result = None
    if rank == 0:
        _, single = run(None)
        a = gathered[:seq * s.hidden].float()
        b = single[:seq * s.hidden].float()
        rel = float((a - b).norm() / b.norm())
        worst = float((a - b).abs().max())
        result = {"rel_l2": rel, "max_abs": worst, "ok": bool(rel <= 1e-2 and worst <= 5e-2),
                  "what": f"one full-width block, S={seq}, {s.heads // world} heads and "
                          f"{dit.rows_local} rows per rank, sharded vs unsharded on rank 0",
                  "bar": {"rel_l2": 1e-2, "max_abs": 5e-2}}
    dist.barrier()
    torch.cuda.synchronize()
    if hasattr(exchange, "close"):
        exchange.close()
    return result


def run_gpu_arm(args, shape, sequence, text_rows):
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry

    pkg = entry.load_package()
    from h3c_b200.plumbing import NcclExchange, TorchMemory
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    gpu = pkg.Gpu(local_rank)          # raises if the CUDA library or the device is missing
    mem = TorchMemory(torch, gpu, device)
    peaks = measured_peaks()
    s = shape

    def gather(obj):
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    def make_exchange():
        if world == 1:
            return None
        if args.exchange in ("push", "loopback"):
            return pkg.PeerExchange(gpu, world, rank, gather, loopback=args.exchange == "loopback")
        return NcclExchange(dist, mem, world, rank)

    weights = build_weights(torch, pkg, gpu, mem, shape)
    exchange = make_exchange()
    try:
        dit, step = build_workload(torch, pkg, gpu, mem, shape, weights, sequence, text_rows, exchange)
    except pkg.H3Error as err:
        # peer mappings (CUDA IPC) are refused on this machine: every rank gets the same error
        # and falls back to the NCCL form of the exchange
        if not isinstance(exchange, pkg.PeerExchange):
            raise
        if rank == 0:
            print(f"bench: {err}; using pack + NCCL all-to-all + unpack", file=sys.stderr, flush=True)
        args.exchange = "nccl"
        exchange = make_exchange()
        dit, step = build_workload(torch, pkg, gpu, mem, shape, weights, sequence, text_rows, exchange)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def fill_loopback(d):
        # the slots other ranks would fill must not stay zero: attention's cost and power draw
        # depend on the data (rescale decisions, switching activity)
        if world > 1 and args.exchange == "loopback":
            for t in d.gathered:
                mem.torch_of(t).view(torch.bfloat16).normal_(0.0, 1.0)

    def reduce_max(*values):
        if world == 1:
            return list(values)
        t = torch.tensor(values, device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t]

    parity = None
    if world > 1 and args.exchange != "loopback" and not args.no_parity:
        parity = parity_vs_single(torch, dist, pkg, gpu, mem, shape, weights, make_exchange, world, rank)

    fill_loopback(dit)

    class Latents:
        """Pinned host latents in, device latents, BF16 velocities out, for one workload."""

        def __init__(self, st):
            self.n = max(1, st.video_rows) * s.video_patch
            self.host_latent = torch.randn(self.n, dtype=torch.float32).pin_memory()
            self.host_velocity = torch.empty(self.n, dtype=torch.bfloat16).pin_memory()
            self.latent = torch.empty(self.n, dtype=torch.float32, device=device)
            self.velocity = torch.empty(self.n, dtype=torch.bfloat16, device=device)
            st.latent = gpu.wrap(self.latent.data_ptr(), self.n, pkg.F32)
            st.velocity = gpu.wrap(self.velocity.data_ptr(), self.n, pkg.BF16)
            self.latent.copy_(self.host_latent)

    io = Latents(step)
    n_latent = io.n

    def stepper(st):
        def one_step():
            gpu.begin()
            st.forward()
            st.euler(-0.05)
            gpu.submit()          # one synchronisation per evaluated step, as the reference sampler
        return one_step

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier()
        return a.elapsed_time(b) / steps

    one_step = stepper(step)

    def one_step_e2e():
        io.latent.copy_(io.host_latent, non_blocking=True)       # H2D from pinned memory
        gpu.begin()
        step.forward()
        gpu.submit()
        io.host_velocity.copy_(io.velocity, non_blocking=True)   # D2H of the step's result
        torch.cuda.synchronize()

    # the clock sampler starts before the warm-up steps: its start-up (NVML initialisation in the
    # child process) must not fall into the timed region
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        one_step()
    barrier()
    before = gpu.stats()
    ms_local = timed(one_step, args.steps, 0)
    after = gpu.stats()
    clocks = sampler.stop() if rank == 0 else None
    launches = ((after.direct_dispatches + after.mps_linear_dispatches + after.mps_sdpa_dispatches) -
                (before.direct_dispatches + before.mps_linear_dispatches + before.mps_sdpa_dispatches))

    # end to end: host buffers in, host buffers out, copies inside the timed region
    e2e_local = timed(one_step_e2e, args.steps, 1)
    ms, e2e_ms = reduce_max(ms_local, e2e_local)
    launches_total = launches
    if world > 1:
        count = torch.tensor([launches], device=device, dtype=torch.int64)
        dist.all_reduce(count)
        launches_total = int(count[0])

    kernels = kernel_timings(torch, pkg, gpu, shape, dit, step, exchange, sequence, world)

    # the second configuration the metric is quoted on, on the same weights: 864x480x121f
    c4 = None
    if args.workload == "c3" and not args.no_c4:
        c4_text, c4_video, c4_desc = WORKLOADS["c4"]
        c4_seq = c4_text + c4_video
        ex4 = make_exchange()
        dit4, step4 = build_workload(torch, pkg, gpu, mem, shape, weights, c4_seq, c4_text, ex4)
        fill_loopback(dit4)
        Latents(step4)
        c4_steps, c4_warmup = 3, 1
        (c4_ms,) = reduce_max(timed(stepper(step4), c4_steps, c4_warmup))
        c4_kernels = kernel_timings(torch, pkg, gpu, shape, dit4, step4, ex4, c4_seq, world, repeats=3)
        c4_tf = s.blocks * s.block_flops(c4_seq) / (c4_ms * 1e-3) / 1e12 / world
        c4 = {"workload": f"c4: {c4_desc}", "rows": c4_seq, "rows_per_rank": dit4.rows_local,
              "ms_per_step": c4_ms, "ms_per_block": c4_ms / s.blocks, "steps": c4_steps,
              "warmup": c4_warmup, "tflops_per_gpu": c4_tf,
              "frac_of_burst": c4_tf / peaks["bf16_tflops"],
              "frac_of_sustained": c4_tf / peaks["bf16_tflops_sustained"],
              "kernels": {k: {"ms": v[0], "tflops": v[1], "frac_of_burst_peak": v[1] / peaks["bf16_tflops"]}
                          for k, v in c4_kernels.items()}}
        barrier()
        if hasattr(ex4, "close"):
            ex4.close()

    line = None
    if rank == 0:
        flops_step = s.blocks * s.block_flops(sequence)
        achieved = flops_step / (ms * 1e-3) / 1e12 / world       # per GPU
        rows = dit.rows_local
        pair_kernel = 128 < rows <= 8192
        # the adaLN projection of h3_dit_schedule_precompute at its largest row count: HBM-bound
        a12_rows = 42
        mod_cols = s.modalities * s.slots * s.hidden
        a12_in = mem.bf16(a12_rows * s.time_dim, std=0.125, generator=weights.generator)
        a12_out = mem.bf16(a12_rows * mod_cols)
        a12_bytes = 2.0 * (mod_cols * s.time_dim + mod_cols + a12_rows * (s.time_dim + mod_cols))
        a12_ms, a12_tbs = time_kernel(
            torch, gpu, lambda: gpu.op("linear_bf16", a12_out, a12_in, weights.proj_w, weights.proj_b,
                                       a12_rows, s.time_dim, mod_cols), a12_bytes)
        ref_ops = None
        if world == 1 and not args.no_reference_cuda:
            ref_ops = reference_cuda_ops(torch, pkg, gpu, shape, dit, step, sequence)

        def kernel_entry(name, v):
            e = {"ms": v[0], "tflops": v[1], "frac_of_burst_peak": v[1] / peaks["bf16_tflops"]}
            if ref_ops and name in ref_ops:
                # this library and the reference's CUDA backend timed alternately, same GPU state
                e["paired_with_reference_cuda"] = ref_ops[name]
            return e
        kernel_lines = {k: kernel_entry(k, v) for k, v in kernels.items()}
        if ref_ops and "unavailable" in ref_ops:
            kernel_lines["reference_cuda"] = ref_ops
        elif ref_ops:
            kernel_lines["paired_only"] = {k: v for k, v in ref_ops.items() if k not in kernels}
        kernel_lines["adaln_projection"] = {
            "ms": a12_ms, "gbs": a12_tbs * 1e3, "frac_of_hbm_peak": a12_tbs * 1e3 / peaks["hbm_gbs"],
            "bytes_per_launch": a12_bytes, "shape": f"{a12_rows} x {s.time_dim} -> {mod_cols} (+bias)"}
        fc1_ms, fc1_tf = kernels["mlp_fc1_swiglu"]
        family = "h3b_gemm_pair" if pair_kernel else "h3b_gemm_tc"
        roofline = {"bound": "tensor",
                    "kernel": f"{family}<swiglu> (MLP up projection {s.hidden} -> 2 x {s.ffn} with the "
                              "SwiGLU epilogue: the launch with the largest share of the step)",
                    "achieved": fc1_tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": fc1_tf / peaks["bf16_tflops"], "peak_source": peaks["source"] + " burst",
                    "ms_per_launch": fc1_ms, "flops_per_launch": 2.0 * rows * s.hidden * 2 * s.ffn,
                    "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get((args.workload, world)),
                    "traffic_unit": "bytes per launch (dram read+write, one ncu capture)",
                    "traffic_source": NCU_DRAM_SOURCE if (args.workload, world) in NCU_DRAM_BYTES_PER_LAUNCH
                    else None}
        if "attention" in kernels:
            at_ms, at_tf = kernels["attention"]
            roofline["furthest_from_roof"] = {
                "kernel": "h3b_sdpa_tc2 (joint attention)", "achieved": at_tf,
                "frac": at_tf / peaks["bf16_tflops"], "ms_per_launch": at_ms}
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cpu_ms, desc, threads, _ = cpu_sample(s, sequence)
            cpu = {"value": cpu_ms, "unit": "ms/step", "cores": threads, "kind": "port", "sample": desc}
        line = {
            "metric": "dit_denoise_step_ms", "value": ms, "unit": "ms/step", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "ms_per_block": ms / s.blocks,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(args, sequence),
            "tflops_per_gpu": achieved,
            "frac_of_bf16_peak": {"burst": achieved / peaks["bf16_tflops"],
                                  "sustained": achieved / peaks["bf16_tflops_sustained"],
                                  "datasheet_2250": achieved / 2250.0, "source": peaks["source"]},
            "e2e": {"value": e2e_ms, "unit": "ms/step",
                    "h2d_bytes_per_step": n_latent * 4 * world, "d2h_bytes_per_step": n_latent * 2 * world},
            "gpu_launches": launches_total,
            "roofline": roofline,
            "kernels": kernel_lines,
            "c4": c4,
            "parity_vs_single": parity,
            "cpu_baseline": cpu,
            "clocks": clocks,
        }
        if isinstance(exchange, NcclExchange):
            line["all_to_all_calls_per_step"] = exchange.calls // max(1, (args.warmup + 2 * args.steps + 1))
        if world > 1:
            line["config"]["exchange"] = {
                "push": "peer stores from the QKV and attention epilogues + 2 flag barriers per block",
                "loopback": "MEASUREMENT AID, results invalid: peer stores redirected to local memory, no barriers "
                            "(step time without any exchange cost)",
                "nccl": "pack + NCCL all-to-all + unpack"}[args.exchange]
    if world > 1:
        dist.barrier()
        if dit.push:
            torch.cuda.synchronize()
            exchange.close()
        dist.destroy_process_group()
    gpu.close()
    if line is not None:
        print(json.dumps(line), flush=True)
        if parity is not None and not parity["ok"]:
            raise SystemExit("bench: the sharded block differs from the single-GPU block beyond the parity bar")


def run_cfg_arm(args, shape, sequence, text_rows):
    """20 Euler steps with classifier-free guidance. With N >= 2 ranks the first half evaluates
    the cond branch and the second half the uncond branch (sequence-parallel inside each half),
    matching ranks swap velocities over NCCL after every forward; with one rank both branches
    run one after the other. value = seconds for the whole loop, device-timed, max over ranks."""
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry

    pkg = entry.load_package()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus or (world > 1 and world % 2):
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N (N = 1 or even) for --gpus N")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    gpu = pkg.Gpu(local_rank)
    from h3c_b200.plumbing import NcclPair, TorchMemory
    mem = TorchMemory(torch, gpu, device)
    euler_steps, guidance = args.euler_steps, args.guidance
    exchange, pair, group_id, half = None, None, 0, 1
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        half = world // 2
        group_id, group_rank = rank // half, rank % half
        groups = [dist.new_group(list(range(g * half, (g + 1) * half))) for g in range(2)]
        if half > 1:
            def gather(obj):
                out = [None] * half
                dist.all_gather_object(out, obj, group=groups[group_id])
                return out
            exchange = pkg.PeerExchange(gpu, half, group_rank, gather)
        pair = NcclPair(dist, mem, (rank + half) % world, is_cond=group_id == 0)
    weights = build_weights(torch, pkg, gpu, mem, shape, time_rows=euler_steps)
    dit, step = build_workload(torch, pkg, gpu, mem, shape, weights, sequence, text_rows, exchange,
                               text_seed=2 if group_id == 0 else 4)
    s = shape
    n_latent = max(1, step.video_rows) * s.video_patch
    noise = torch.Generator()
    noise.manual_seed(1)
    host_latent = torch.randn(n_latent, dtype=torch.float32, generator=noise).pin_memory()
    host_final = torch.empty(n_latent, dtype=torch.float32).pin_memory()
    latent_t = torch.empty(n_latent, dtype=torch.float32, device=device)
    step.latent = gpu.wrap(latent_t.data_ptr(), n_latent, pkg.F32)
    uncond = None
    if world == 1:
        g4 = torch.Generator(device=device)
        g4.manual_seed(4)
        uncond = mem.bf16(max(1, text_rows) * s.hidden, std=1.0, generator=g4)
    sigmas = pkg.serving_sigmas(euler_steps)

    def sampler_for(first, count):
        return pkg.EulerSampler(step, sigmas[first:first + count + 1], step.row_maps[first:first + count],
                                step.final_row_maps[first:first + count], guidance=guidance,
                                uncond_text=uncond, pair=pair)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    latent_t.copy_(host_latent)
    sampler_for(0, max(3, args.warmup)).run()               # untimed warm-up steps
    full = sampler_for(0, euler_steps)
    clock = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        clock.start()
    before = gpu.stats()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        latent_t.copy_(host_latent, non_blocking=True)      # seeded N(0,1) noise from pinned memory
        full.run()
        host_final.copy_(latent_t, non_blocking=True)       # final latent back to the host
    t1.record()
    barrier()
    after = gpu.stats()
    clocks = clock.stop() if rank == 0 else None
    seconds = t0.elapsed_time(t1) / 1e3 / args.steps
    launches = ((after.direct_dispatches + after.mps_linear_dispatches + after.mps_sdpa_dispatches) -
                (before.direct_dispatches + before.mps_linear_dispatches + before.mps_sdpa_dispatches))
    if world > 1:
        t = torch.tensor([seconds], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        seconds = float(t[0])
        l = torch.tensor([launches], device=device, dtype=torch.int64)
        dist.all_reduce(l)
        launches = int(l[0])
    if rank == 0:
        peaks = measured_peaks()
        forwards = 2 * euler_steps
        flops = forwards * s.blocks * s.block_flops(sequence)
        per_gpu = flops / seconds / 1e12 / world
        finite = bool(torch.isfinite(host_final).all())
        line = {
            "metric": "cfg_denoise_total_s", "value": seconds, "unit": "s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": seconds * 1e3 / euler_steps,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": dict(workload_config(args, sequence), euler_steps=euler_steps, guidance=guidance,
                           parallelism=(f"2 guidance groups x sp{half}" if world > 1
                                        else "single GPU, cond and uncond in turn"),
                           forwards_per_denoise=forwards),
            "tflops_per_gpu": per_gpu,
            "frac_of_bf16_peak": {"burst": per_gpu / peaks["bf16_tflops"],
                                  "sustained": per_gpu / peaks["bf16_tflops_sustained"],
                                  "source": peaks["source"]},
            "e2e": {"value": seconds, "unit": "s", "h2d_bytes_per_step": n_latent * 4 * world,
                    "d2h_bytes_per_step": n_latent * 4 * world},
            "gpu_launches": launches, "final_latent_finite": finite, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        if exchange is not None:
            exchange.close()
        dist.destroy_process_group()
    gpu.close()


# ------------------------------------------------------------- video-VAE decoder tile

VAE = dict(latent=24, hidden=2048, layers=36, heads=32, head_dim=64, ffn=8192, rope_half=24,
           output_patch=3 * 4 * 16 * 16, registers=4, suffix=5)
VAE_TILE_ROWS = 7 * 16 * 16 + 5     # one 256-pixel tile of seven latent frames (h3_video_vae.c:1013-1019)


def vae_cpu_sample(rows=VAE_TILE_ROWS, gemm_rows=128, attn_rows=256):
    """The oracle port on a bounded sample of one decoder block, extrapolated linearly to a tile
    decode (36 blocks): (ms per tile, description, threads, seconds spent)."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import h3_oracle as o
    o.set_threads(len(os.sched_getaffinity(0)))
    v, rng = VAE, np.random.default_rng(0)
    inner = v["heads"] * v["head_dim"]

    def rand(n, std=1.0):
        return rng.standard_normal(n, dtype=np.float32) * np.float32(std)
    x = rand(gemm_rows * v["hidden"])
    ones, scale = np.ones(v["hidden"], np.float32), np.full(v["hidden"], 0.25, np.float32)
    w_qkv, w_out = rand(3 * inner * v["hidden"], 0.02), rand(v["hidden"] * inner, 0.02)
    w1, w2 = rand(2 * v["ffn"] * v["hidden"], 0.02), rand(v["hidden"] * v["ffn"], 0.02)
    cos, sin = rand(gemm_rows * v["rope_half"]), rand(gemm_rows * v["rope_half"])
    t0 = time.perf_counter()
    n1 = o.rms_norm_f32(x, ones, gemm_rows, v["hidden"])
    qkv = o.linear_f32(n1, w_qkv, None, gemm_rows, v["hidden"], 3 * inner)
    q, _, _ = o.video_qkv_rope_f32(qkv, cos, sin, gemm_rows, v["heads"], v["head_dim"], v["rope_half"])
    br = o.linear_f32(q, w_out, None, gemm_rows, inner, v["hidden"])
    x = o.scale_add_f32(x, br, scale, gemm_rows, v["hidden"])
    n2 = o.rms_norm_f32(x, ones, gemm_rows, v["hidden"])
    act = o.swiglu_f32(o.linear_f32(n2, w1, None, gemm_rows, v["hidden"], 2 * v["ffn"]), gemm_rows, v["ffn"])
    o.scale_add_f32(x, o.linear_f32(act, w2, None, gemm_rows, v["ffn"], v["hidden"]), scale, gemm_rows, v["hidden"])
    t_rows = time.perf_counter() - t0
    # attention is quadratic: all keys, a slice of the query rows, by running the oracle on the first
    # attn_rows rows of a problem whose keys are the full tile (cost is linear in query rows)
    n = rows * inner
    qa, ka, va = rand(n), rand(n), rand(n)
    t0 = time.perf_counter()
    o.sdpa_f32(qa[:attn_rows * inner], ka, va, attn_rows, v["heads"], v["head_dim"], 0.125)
    t_attn = (time.perf_counter() - t0) * rows / attn_rows    # attn_rows x attn_rows -> attn_rows x rows keys
    block_s = t_rows * rows / gemm_rows + t_attn * rows / attn_rows
    desc = (f"one decoder block: projections + row ops on {gemm_rows} of {rows} rows, attention on {attn_rows} x "
            f"{attn_rows} rows scaled to {rows} x {rows}; extrapolated linearly to {v['layers']} blocks")
    return block_s * v["layers"] * 1e3, desc, o.threads(), t_rows + t_attn


def run_vae_reference_arm(args):
    """The CPU arm for the VAE tile: the oracle port on the host cores (rank 0 only)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    values, desc, threads = [], "", 1
    for i in range(args.warmup + args.steps):
        ms, desc, threads, _ = vae_cpu_sample(gemm_rows=64, attn_rows=128)
        if i >= args.warmup:
            values.append(ms)
    value = statistics.mean(values)
    line = {"impl": "reference", "metric": "vae_tile_decode_ms", "value": value, "unit": "ms/tile", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": value, "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "vae_tile: " + WORKLOADS["vae_tile"][2], "rows": VAE_TILE_ROWS, "blocks": VAE["layers"]},
            "cpu_baseline": {"value": value, "unit": "ms/tile", "cores": threads, "kind": "port", "sample": desc},
            "e2e": {"value": value, "unit": "ms/tile", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_vae_arm(args):
    """One tile of the video-VAE decoder (the step after the DiT on the reference's pipeline): the op
    sequence of run_resident_tile / run_block (h3_video_vae.c:425-461, 600-660) on 1,797 rows with
    all 36 blocks' F32 weights resident (9.7 GB), through the C ABI."""
    import torch
    import __graft_entry__ as entry
    pkg = entry.load_package()
    from h3c_b200.plumbing import TorchMemory
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    gpu = pkg.Gpu(local_rank)
    mem, peaks, rows = TorchMemory(torch, gpu, device), measured_peaks(), VAE_TILE_ROWS
    v = dict(VAE, layers=min(args.blocks, VAE["layers"]))       # --blocks 1: a small case for profiler captures
    inner, patches = v["heads"] * v["head_dim"], VAE_TILE_ROWS - v["suffix"]
    generator = torch.Generator(device=device).manual_seed(0)

    def weight(n, std=0.02, fill=None):
        t = mem.f32(n, std=None if fill is not None else std, generator=generator)
        if fill is not None:
            mem.torch_of(t).fill_(fill)
        gpu.lib.h3x_tensor_keep_half_rows(t.handle, 1)
        return t
    blocks = [dict(norm1=weight(v["hidden"], fill=1.0), qkv_w=weight(3 * inner * v["hidden"]), qkv_b=weight(3 * inner),
                   out_w=weight(v["hidden"] * inner), out_b=weight(v["hidden"]), scale1=weight(v["hidden"], fill=0.25),
                   norm2=weight(v["hidden"], fill=1.0), w1=weight(2 * v["ffn"] * v["hidden"]), w1_b=weight(2 * v["ffn"]),
                   w2=weight(v["hidden"] * v["ffn"]), w2_b=weight(v["hidden"]), scale2=weight(v["hidden"], fill=0.25))
              for _ in range(v["layers"])]
    post_w, post_b = weight(v["latent"] ** 2, 0.2), weight(v["latent"])
    embed_w, embed_b = weight(v["hidden"] * v["latent"], 0.2), weight(v["hidden"])
    registers, zero = weight(v["registers"] * v["hidden"], 1.0), weight(v["hidden"], fill=0.0)
    norm_out_w, norm_out_b = weight(v["hidden"], fill=1.0), weight(v["hidden"])
    proj_w, proj_b = weight(v["output_patch"] * v["hidden"]), weight(v["output_patch"])
    # the library's own tensors, as the reference's host allocates them (h3_video_vae.c:399-423)
    act = {name: gpu.new(n, pkg.F32) for name, n in dict(
        latent=patches * v["latent"], post=patches * v["latent"], patch_hidden=patches * v["hidden"],
        hidden=rows * v["hidden"], norm=rows * v["hidden"], qkv=rows * inner * 3, query=rows * inner, key=rows * inner,
        value=rows * inner, heads=rows * inner, branch=rows * v["hidden"], ff1=rows * v["ffn"] * 2,
        activated=rows * v["ffn"], projected=rows * v["output_patch"]).items()}
    angle = torch.randn(rows * v["rope_half"], device=device, generator=generator) * 2.0
    rope_cos, rope_sin = mem.f32(rows * v["rope_half"]), mem.f32(rows * v["rope_half"])
    mem.torch_of(rope_cos).copy_(angle.cos())
    mem.torch_of(rope_sin).copy_(angle.sin())
    host_latent = torch.randn(patches * v["latent"], generator=torch.Generator().manual_seed(1)).pin_memory()
    host_out = torch.empty(rows * v["output_patch"], dtype=torch.float32).pin_memory()

    def block_ops(w):
        h = v["hidden"]
        return [
            ("rms_norm", lambda: gpu.op("rms_norm_f32", act["norm"], act["hidden"], w["norm1"], rows, h, 1e-5), 0.0),
            ("qkv_proj", lambda: gpu.op("linear_f32", act["qkv"], act["norm"], w["qkv_w"], w["qkv_b"], rows, h, inner * 3),
             2.0 * rows * h * inner * 3),
            ("qkv_norm_rope", lambda: gpu.op("video_qkv_rope_f32", act["query"], act["key"], act["value"], act["qkv"],
                                             rope_cos, rope_sin, rows, v["heads"], v["head_dim"], v["rope_half"], 1e-5), 0.0),
            ("attention", lambda: gpu.op("sdpa_f32", act["heads"], act["query"], act["key"], act["value"], rows,
                                         v["heads"], v["head_dim"], 0.125), 4.0 * rows * rows * inner),
            ("out_proj", lambda: gpu.op("linear_f32", act["branch"], act["heads"], w["out_w"], w["out_b"], rows, inner, h),
             2.0 * rows * inner * h),
            ("scale_add", lambda: gpu.op("scale_add_f32", act["hidden"], act["hidden"], act["branch"], w["scale1"], rows, h), 0.0),
            ("rms_norm", lambda: gpu.op("rms_norm_f32", act["norm"], act["hidden"], w["norm2"], rows, h, 1e-5), 0.0),
            ("mlp_w1", lambda: gpu.op("linear_f32", act["ff1"], act["norm"], w["w1"], w["w1_b"], rows, h, v["ffn"] * 2),
             2.0 * rows * h * v["ffn"] * 2),
            ("swiglu", lambda: gpu.op("swiglu_f32", act["activated"], act["ff1"], rows, v["ffn"]), 0.0),
            ("mlp_w2", lambda: gpu.op("linear_f32", act["branch"], act["activated"], w["w2"], w["w2_b"], rows, v["ffn"], h),
             2.0 * rows * v["ffn"] * h),
            ("scale_add", lambda: gpu.op("scale_add_f32", act["hidden"], act["hidden"], act["branch"], w["scale2"], rows, h), 0.0),
        ]
    launches_before = None

    def decode_tile():
        h = v["hidden"]
        gpu.begin()
        gpu.op("linear_f32", act["post"], act["latent"], post_w, post_b, patches, v["latent"], v["latent"])
        gpu.op("linear_f32", act["patch_hidden"], act["post"], embed_w, embed_b, patches, v["latent"], h)
        gpu.op("copy_f32", act["hidden"], 0, act["patch_hidden"], 0, patches * h)
        gpu.op("copy_f32", act["hidden"], patches * h, registers, 0, v["registers"] * h)
        gpu.op("copy_f32", act["hidden"], (patches + v["registers"]) * h, zero, 0, h)
        for w in blocks:
            for _, op, _ in block_ops(w):
                op()
        gpu.op("layer_norm_f32", act["norm"], act["hidden"], norm_out_w, norm_out_b, rows, h, 1e-5)
        gpu.op("linear_f32", act["projected"], act["norm"], proj_w, proj_b, rows, h, v["output_patch"])
        gpu.submit()

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        decode_tile()
    sync()
    stats0 = gpu.stats()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        decode_tile()
    stop.record()
    sync()
    stats1 = gpu.stats()
    ms = start.elapsed_time(stop) / args.steps
    # end to end: host latent rows in, projected pixels out, every step
    latent_view = mem.torch_of(act["latent"]).view(torch.float32)        # byte views of the library's memory
    out_view = mem.torch_of(act["projected"]).view(torch.float32)
    sync()
    start.record()
    for _ in range(args.steps):
        latent_view.copy_(host_latent, non_blocking=True)
        decode_tile()
        host_out.copy_(out_view, non_blocking=True)
    stop.record()
    sync()
    e2e_ms = start.elapsed_time(stop) / args.steps
    clocks = sampler.stop()
    if world > 1:
        both = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(both, op=dist.ReduceOp.MAX)
        ms, e2e_ms = (float(x) for x in both)
    launches = sum(getattr(stats1, f) - getattr(stats0, f) for f in
                   ("direct_dispatches", "mps_linear_dispatches", "mps_sdpa_dispatches")) // args.steps
    kernels = {}
    for name, op, flops in block_ops(blocks[0]):
        if name in kernels:
            continue
        t, tf = time_kernel(torch, gpu, op, flops, 10)
        kernels[name] = {"ms": t}
        if flops:
            kernels[name].update(tflops=tf, frac_of_burst_peak=tf / peaks["bf16_tflops"])
    if rank == 0 and world == 1 and REF_CUDA.exists() and not args.no_reference_cuda:
        for name, t in vae_reference_cuda_ops(pkg, rows).items():
            kernels[name]["reference_cuda_ms"] = t
        kernels["block"] = {"ms": sum(k["ms"] * (2 if n in ("rms_norm", "scale_add") else 1) for n, k in kernels.items()),
                            "reference_cuda_ms": sum(k["reference_cuda_ms"] * (2 if n in ("rms_norm", "scale_add") else 1)
                                                     for n, k in kernels.items())}
    flops = sum(f for _, _, f in block_ops(blocks[0])) * v["layers"] + 2.0 * rows * v["hidden"] * v["output_patch"]
    top = kernels["mlp_w1"]
    line = {
        "metric": "vae_tile_decode_ms", "value": ms, "unit": "ms/tile", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 tensors; projections on the FP16 tensor cores (row-scaled, F32 accumulate), attention in BF16",
        "data": "synthetic",
        "config": {"workload": "vae_tile: one 256-pixel tile of seven latent frames through the video-VAE decoder: "
                               f"1,797 rows, hidden 2048, 32 heads x 64, FFN 8192, {v['layers']} blocks, "
                               f"{v['layers'] * 0.268:.1f} GB of F32 weights resident",
                   "rows": rows, "blocks": v["layers"], "parallelism": "single" if world == 1 else f"{world} replicas",
                   "l2": "a block's weights (268 MB) exceed the 126 MB L2 between reuses"},
        "tflops_per_gpu": flops / (ms * 1e-3) / 1e12,
        "e2e": {"value": e2e_ms, "unit": "ms/tile", "h2d_bytes_per_step": host_latent.numel() * 4,
                "d2h_bytes_per_step": host_out.numel() * 4},
        "gpu_launches": int(launches),
        "roofline": {"bound": "tensor", "kernel": "h3b_gemm_pair<store f32> (MLP input projection 2048 -> 2 x 8192: the "
                     "launch with the largest share of a block)", "achieved": top["tflops"], "peak": peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": top["tflops"] / peaks["bf16_tflops"],
                     "peak_source": f"{peaks['source']} burst (16-bit dense)", "ms_per_launch": top["ms"],
                     "flops_per_launch": 2.0 * rows * v["hidden"] * v["ffn"] * 2, "traffic": None,
                     "note": "ms includes the conversion of the activation rows to FP16 (its own small launch)"},
        "kernels": kernels, "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_ms, desc, threads, _ = vae_cpu_sample()
        line["cpu_baseline"] = {"value": cpu_ms, "unit": "ms/tile", "cores": threads, "kind": "port", "sample": desc}
    if rank == 0:
        print(json.dumps(line), flush=True)
    gpu.close()
    if world > 1:
        dist.destroy_process_group()


def vae_reference_cuda_ops(pkg, rows):
    """The decoder block's ops through the reference's own CUDA backend (TF32 cuBLASLt projections,
    BF16 flash attention, its row kernels) on this GPU: name -> ms."""
    import torch
    v = VAE
    inner, h = v["heads"] * v["head_dim"], v["hidden"]
    gpu = pkg.Gpu(0, lib_path=REF_CUDA)
    rng = np.random.default_rng(0)

    def T(n, std=1.0):
        return gpu.f32(rng.standard_normal(n, dtype=np.float32) * np.float32(std))
    x, norm, qkv = T(rows * h), T(rows * h), T(rows * inner * 3)
    q, k, val, heads = T(rows * inner), T(rows * inner), T(rows * inner), T(rows * inner)
    branch, ff1, act = T(rows * h), T(rows * v["ffn"] * 2), T(rows * v["ffn"])
    cos, sin = T(rows * v["rope_half"]), T(rows * v["rope_half"])
    w = dict(norm=T(h), qkv_w=T(inner * 3 * h, 0.02), qkv_b=T(inner * 3, 0.02), out_w=T(h * inner, 0.02), out_b=T(h, 0.02),
             scale=T(h, 0.1), w1=T(v["ffn"] * 2 * h, 0.02), w1_b=T(v["ffn"] * 2, 0.02), w2=T(h * v["ffn"], 0.01), w2_b=T(h, 0.02))
    ops = {
        "rms_norm": lambda: gpu.op("rms_norm_f32", norm, x, w["norm"], rows, h, 1e-5),
        "qkv_proj": lambda: gpu.op("linear_f32", qkv, norm, w["qkv_w"], w["qkv_b"], rows, h, inner * 3),
        "qkv_norm_rope": lambda: gpu.op("video_qkv_rope_f32", q, k, val, qkv, cos, sin, rows, v["heads"], v["head_dim"],
                                        v["rope_half"], 1e-5),
        "attention": lambda: gpu.op("sdpa_f32", heads, q, k, val, rows, v["heads"], v["head_dim"], 0.125),
        "out_proj": lambda: gpu.op("linear_f32", branch, heads, w["out_w"], w["out_b"], rows, inner, h),
        "scale_add": lambda: gpu.op("scale_add_f32", x, x, branch, w["scale"], rows, h),
        "mlp_w1": lambda: gpu.op("linear_f32", ff1, norm, w["w1"], w["w1_b"], rows, h, v["ffn"] * 2),
        "swiglu": lambda: gpu.op("swiglu_f32", act, ff1, rows, v["ffn"]),
        "mlp_w2": lambda: gpu.op("linear_f32", branch, act, w["w2"], w["w2_b"], rows, v["ffn"], h),
    }
    out = {name: time_kernel(torch, gpu, fn, 0.0, 10)[0] for name, fn in ops.items()}
    gpu.close()
    return out


def run_sdpa_only(pkg, rows, heads, window=0, timed=0):
    """The attention kernel on its own: three launches (a case small enough for a multi-section
    profiler capture: rows x heads x 128 x 3 inputs; 6400,12 holds 118 MB), then `timed` more
    between CUDA events. window > 0 registers a block-sparse mask first: every 128-row query
    block lists the 64-key tiles within `window` tiles of its own first one."""
    import numpy as np
    import torch
    gpu = pkg.Gpu(0)
    count = rows * heads * 128
    generator = torch.Generator(device="cuda").manual_seed(1)
    tensors = [torch.randn(count, device="cuda", dtype=torch.bfloat16, generator=generator) for _ in range(3)]
    tensors.append(torch.empty(count, device="cuda", dtype=torch.bfloat16))
    q, k, v, out = [gpu.wrap(t.data_ptr(), count, pkg.BF16) for t in tensors]
    density = 1.0
    if window > 0:
        blocks, tiles = (rows + 127) // 128, (rows + 63) // 64
        lists = [[t for t in range(tiles) if abs(t - 2 * b) <= window] for b in range(blocks)]
        ptr = np.concatenate([[0], np.cumsum([len(l) for l in lists])]).astype(np.uint32)
        idx = np.concatenate([np.asarray(l, np.uint32) for l in lists]).astype(np.uint32)
        if gpu.lib.h3_gpu_sdpa_set_sparse(gpu.handle, ptr.ctypes.data, ptr.size, idx.ctypes.data, idx.size,
                                          rows) != 1:
            raise RuntimeError("h3_gpu_sdpa_set_sparse refused the window mask")
        density = idx.size / (blocks * tiles)
    scale = 1.0 / math.sqrt(128)
    for _ in range(3):
        gpu.begin()
        gpu.op("sdpa_bf16", out, q, k, v, rows, heads, 128, scale)
        gpu.submit()
    line = f"sdpa {rows} x {heads} x 128, mask density {density:.2f}: mean |out| = {float(tensors[3].float().abs().mean()):.4f}"
    if timed > 0:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        gpu.begin()
        start.record()
        for _ in range(timed):
            gpu.op("sdpa_bf16", out, q, k, v, rows, heads, 128, scale)
        stop.record()
        gpu.submit()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / timed
        line += f"; {ms:.3f} ms per launch ({4.0 * rows * rows * heads * 128 * density / ms / 1e9:.0f} TFLOP/s of listed tiles)"
    print(line)
    gpu.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--blocks", type=int, default=50)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-c4", action="store_true", help="skip the 864x480x121f measurement of the default run")
    ap.add_argument("--no-parity", action="store_true", help="N>1: skip the sharded-vs-single block check")
    ap.add_argument("--no-reference-cuda", action="store_true",
                    help="N=1: skip the per-op timing of the reference's CUDA backend")
    ap.add_argument("--exchange", default="push", choices=["push", "nccl", "loopback"],
                    help="N>1: peer stores fused into the kernels, or pack + NCCL all-to-all + unpack; "
                         "loopback = same kernels with the stores kept local and no barriers, to "
                         "measure the exposed cost of the exchange (results invalid)")
    ap.add_argument("--sdpa-only", metavar="ROWS,HEADS", default=None,
                    help="profiler target: three dense attention launches (head_dim 128, N(0,1) inputs) "
                         "and nothing else; prints no bench line")
    ap.add_argument("--sdpa-window", type=int, default=0, metavar="TILES",
                    help="--sdpa-only under a block-sparse window mask: 64-key tiles kept either side of a "
                         "query block's own (0 = dense)")
    ap.add_argument("--sdpa-time", type=int, default=0, metavar="LAUNCHES",
                    help="--sdpa-only: time this many further launches with CUDA events")
    ap.add_argument("--euler-steps", type=int, default=20, help="c5: Euler steps per denoise")
    ap.add_argument("--guidance", type=float, default=5.0,
                    help="c5: guidance scale (the reference has no guidance pass; harness parameter)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    import __graft_entry__ as entry
    pkg = entry.load_package()
    if args.sdpa_only:
        run_sdpa_only(pkg, *map(int, args.sdpa_only.split(",")), window=args.sdpa_window, timed=args.sdpa_time)
        return
    if args.workload == "vae_tile":
        if args.impl == "reference":
            run_vae_reference_arm(args)
        else:
            run_vae_arm(args)
        return
    text_rows, video_rows, _ = WORKLOADS[args.workload]
    shape = pkg.DitShape(blocks=args.blocks)
    sequence = text_rows + video_rows
    if args.impl == "reference":
        run_reference_arm(args, shape, sequence)
    elif args.workload.startswith("c5"):
        run_cfg_arm(args, shape, sequence, text_rows)
    else:
        run_gpu_arm(args, shape, sequence, text_rows)


if __name__ == "__main__":
    main()
