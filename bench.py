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
}


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the roofline kernel, from the
# ncu capture summarised in profiles/h3b_gemm_tc_dram_traffic_c3.md; (workload, ranks) -> bytes
NCU_DRAM_BYTES_PER_LAUNCH = {("c3", 1): 1050.3e6}


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


def reference_cuda_block(shape, sequence, text_rows, repeats=3):
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

class TorchMemory:
    """Device memory from torch (caching allocator), wrapped into library tensors."""

    def __init__(self, torch, pkg, gpu, device):
        self.torch, self.pkg, self.gpu, self.device = torch, pkg, gpu, device
        self.by_handle = {}

    def bf16(self, elements, fill=None, std=None, generator=None):
        t = self.torch.empty(max(1, elements), dtype=self.torch.bfloat16, device=self.device)
        if std is not None:
            t.normal_(0.0, std, generator=generator)
        elif fill is not None:
            t.fill_(fill)
        else:
            t.zero_()
        wrapped = self.gpu.wrap(t.data_ptr(), elements, self.pkg.BF16)
        self.by_handle[wrapped.handle] = t
        return wrapped

    def f32(self, elements, std=None, generator=None):
        t = self.torch.zeros(max(1, elements), dtype=self.torch.float32, device=self.device)
        if std is not None:
            t.normal_(0.0, std, generator=generator)
        wrapped = self.gpu.wrap(t.data_ptr(), elements, self.pkg.F32)
        self.by_handle[wrapped.handle] = t
        return wrapped

    def torch_of(self, tensor):
        """torch view of a library tensor: the torch allocation it wraps, else a zero-copy byte
        view of the library's own allocation through the CUDA array interface (bytes, because
        the collectives this is used for do not take 16-bit integers)."""
        if tensor.handle not in self.by_handle:
            size = {self.pkg.BF16: 2, self.pkg.F32: 4}[tensor.dtype]

            class _Span:
                __cuda_array_interface__ = {
                    "shape": (tensor.elements * size,), "version": 2, "typestr": "|u1",
                    "data": (tensor.pointer, False)}
            view = self.torch.as_tensor(_Span(), device=self.device)
            self.by_handle[tensor.handle] = view
        return self.by_handle[tensor.handle]


class NcclExchange:
    """all-to-all of equal blocks over NCCL (torch.distributed), on torch's current stream."""

    def __init__(self, dist, memory, world, rank):
        self.dist, self.memory, self.world, self.rank = dist, memory, world, rank
        self.calls = 0

    def all_to_all(self, out, inp):
        self.dist.all_to_all_single(self.memory.torch_of(out), self.memory.torch_of(inp))
        self.calls += 1


class NcclPair:
    """Velocity swap between the two classifier-free-guidance groups: rank i of the cond group
    and rank i of the uncond group exchange their local velocity rows over NCCL."""

    def __init__(self, dist, memory, partner, is_cond):
        self.dist, self.memory, self.partner, self.is_cond = dist, memory, partner, is_cond

    def swap(self, out, inp):
        d = self.dist
        ops = [d.P2POp(d.isend, self.memory.torch_of(inp), self.partner),
               d.P2POp(d.irecv, self.memory.torch_of(out), self.partner)]
        for req in d.batch_isend_irecv(ops):
            req.wait()


def build_model(torch, pkg, gpu, mem, shape, sequence, text_rows, exchange, seed=0, time_rows=2,
                text_seed=None):
    """Random-init weights of the architecture, modulation tables computed by the adaLN
    projection (rows = time rows, 2688 -> 3*6*5376, the load-time GEMM of the reference's
    h3_dit_schedule_precompute), rope tables and row maps for this rank's rows."""
    s = shape
    gen = torch.Generator(device=mem.device)
    gen.manual_seed(seed)
    dit = pkg.Dit(gpu, s, sequence, exchange=exchange, alloc=lambda n: mem.bf16(n))
    silu_time = mem.bf16(time_rows * s.time_dim, std=0.125, generator=gen)   # modulation std ~0.13
    mod_cols = s.modalities * s.slots * s.hidden
    proj_w = mem.bf16(mod_cols * s.time_dim)
    proj_b = mem.bf16(mod_cols)
    blocks = []
    for _ in range(s.blocks):
        t = {}
        for name, count in pkg.block_tensor_shapes(s, time_rows * s.modalities).items():
            if name in ("norm1", "norm2", "q_norm", "k_norm"):
                t[name] = mem.bf16(count, fill=1.0)
            elif name == "modulation":
                t[name] = mem.bf16(count)
            else:
                t[name] = mem.bf16(count, std=0.02, generator=gen)
        mem.torch_of(proj_w).normal_(0.0, 0.02, generator=gen)
        mem.torch_of(proj_b).normal_(0.0, 0.02, generator=gen)
        gpu.begin()
        gpu.op("linear_bf16", t["modulation"], silu_time, proj_w, proj_b, time_rows, s.time_dim, mod_cols)
        gpu.submit()
        blocks.append(pkg.BlockWeights(**t))
    final_mod = mem.bf16(time_rows * s.final_slots * s.hidden, std=0.3, generator=gen)
    final_w = mem.bf16(s.video_patch * s.hidden, std=0.02, generator=gen)
    final_b = mem.bf16(s.video_patch, std=0.02, generator=gen)
    final_norm = mem.bf16(s.hidden, fill=1.0)
    patch_w = mem.f32(s.hidden * s.video_patch, std=0.02, generator=gen)
    patch_b = mem.f32(s.hidden, std=0.02, generator=gen)
    text_gen = gen
    if text_seed is not None:
        text_gen = torch.Generator(device=mem.device)
        text_gen.manual_seed(text_seed)
    text_hidden = mem.bf16(max(1, text_rows) * s.hidden, std=1.0, generator=text_gen)

    # this rank's slice of the global rows: text rows first, then video rows
    r0, rows = dit.row_begin, dit.rows_local
    video_rows_total = sequence - text_rows
    sys.path.insert(0, str(ROOT / "oracle"))
    world = dit.exchange.world
    pos = np.zeros((dit.rows_local * world, 3), np.float32)
    pos[:text_rows, 0] = np.arange(text_rows)
    idx = np.arange(video_rows_total)
    pos[text_rows:sequence, 0] = idx // 1024 if video_rows_total >= 1024 else 0
    pos[text_rows:sequence, 1] = (idx % 1024) // 32
    pos[text_rows:sequence, 2] = idx % 32
    inv_freq = pkg.default_inv_freq()
    local = pos[r0:r0 + rows]
    ang = local[:, :, None] * inv_freq[None, None, :]          # [rows, 3 axes, 16 freqs]
    cos = torch.from_numpy(np.cos(ang).reshape(rows, 48).astype(np.float32))
    sin = torch.from_numpy(np.sin(ang).reshape(rows, 48).astype(np.float32))
    rope_cos, rope_sin = mem.bf16(rows * 48), mem.bf16(rows * 48)
    mem.torch_of(rope_cos).copy_(cos.reshape(-1).to(torch.bfloat16))
    mem.torch_of(rope_sin).copy_(sin.reshape(-1).to(torch.bfloat16))
    tags = np.zeros(dit.rows_local * world, np.uint32)
    tags[:text_rows] = 1
    local_text = max(0, min(text_rows, r0 + dit.rows_valid) - r0)
    local_video = dit.rows_valid - local_text
    # one row map per time row (row_map[row] = time_row * 3 + modality tag); the single-step
    # bench uses time row 1
    row_maps = [gpu.u32(tags[r0:r0 + rows] + 3 * t) for t in range(time_rows)]
    final_row_maps = [gpu.u32(np.full(max(1, local_video), t, np.uint32)) for t in range(time_rows)]
    row_map, final_row_map = row_maps[1], final_row_maps[1]
    step = pkg.DenoiseStep(dit, blocks, video_rows=local_video, text_rows=local_text,
                           patch_weight=patch_w, patch_bias=patch_b, text_hidden=text_hidden,
                           final_norm=final_norm, final_modulation=final_mod, final_weight=final_w,
                           final_bias=final_b, row_map=row_map, final_row_map=final_row_map,
                           rope_cos=rope_cos, rope_sin=rope_sin)
    step.row_maps, step.final_row_maps = row_maps, final_row_maps
    return dit, step


def time_kernel(torch, gpu, fn, flops, repeats=8):
    """Average duration of one launch, CUDA events on the launching (default) stream."""
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
    return ms, flops / (ms * 1e-3) / 1e12


def run_gpu_arm(args, shape, sequence, text_rows):
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry

    pkg = entry.load_package()
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
    mem = TorchMemory(torch, pkg, gpu, device)
    exchange = None
    if world > 1 and args.exchange in ("push", "loopback"):
        def gather(obj):
            out = [None] * world
            dist.all_gather_object(out, obj)
            return out
        exchange = pkg.PeerExchange(gpu, world, rank, gather, loopback=args.exchange == "loopback")
    elif world > 1:
        exchange = NcclExchange(dist, mem, world, rank)
    peaks = measured_peaks()

    try:
        dit, step = build_model(torch, pkg, gpu, mem, shape, sequence, text_rows, exchange)
    except pkg.H3Error as err:
        # peer mappings (CUDA IPC) are refused on this machine: every rank gets the same error
        # and falls back to the NCCL form of the exchange
        if not isinstance(exchange, pkg.PeerExchange):
            raise
        if rank == 0:
            print(f"bench: {err}; using pack + NCCL all-to-all + unpack", file=sys.stderr, flush=True)
        args.exchange = "nccl"
        exchange = NcclExchange(dist, mem, world, rank)
        dit, step = build_model(torch, pkg, gpu, mem, shape, sequence, text_rows, exchange)
    if world > 1 and args.exchange == "loopback":
        # the slots other ranks would fill must not stay zero: attention's cost and power draw
        # depend on the data (rescale decisions, switching activity)
        for t in dit.gathered:
            mem.torch_of(t).view(torch.bfloat16).normal_(0.0, 1.0)
    s = shape
    n_latent = max(1, step.video_rows) * s.video_patch
    host_latent = torch.randn(n_latent, dtype=torch.float32).pin_memory()
    host_velocity = torch.empty(n_latent, dtype=torch.bfloat16).pin_memory()
    latent_t = torch.empty(n_latent, dtype=torch.float32, device=device)
    velocity_t = torch.empty(n_latent, dtype=torch.bfloat16, device=device)
    step.latent = gpu.wrap(latent_t.data_ptr(), n_latent, pkg.F32)
    step.velocity = gpu.wrap(velocity_t.data_ptr(), n_latent, pkg.BF16)
    latent_t.copy_(host_latent)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def one_step():
        gpu.begin()
        step.forward()
        step.euler(-0.05)
        gpu.submit()          # one synchronisation per evaluated step, as the reference sampler

    def one_step_e2e():
        latent_t.copy_(host_latent, non_blocking=True)       # H2D from pinned memory
        gpu.begin()
        step.forward()
        gpu.submit()
        host_velocity.copy_(velocity_t, non_blocking=True)   # D2H of the step's result
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        one_step()
    sampler = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        sampler.start()
    before = gpu.stats()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        one_step()
    stop.record()
    barrier()
    after = gpu.stats()
    clocks = sampler.stop() if rank == 0 else None
    ms_local = start.elapsed_time(stop) / args.steps
    launches = ((after.direct_dispatches + after.mps_linear_dispatches + after.mps_sdpa_dispatches) -
                (before.direct_dispatches + before.mps_linear_dispatches + before.mps_sdpa_dispatches))

    # end to end: host buffers in, host buffers out, copies inside the timed region
    one_step_e2e()
    barrier()
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        one_step_e2e()
    t1.record()
    barrier()
    e2e_local = t0.elapsed_time(t1) / args.steps

    if world > 1:
        t = torch.tensor([ms_local, e2e_local], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
        l = torch.tensor([launches], device=device, dtype=torch.int64)
        dist.all_reduce(l)
        launches_total = int(l[0])
    else:
        ms, e2e_ms, launches_total = ms_local, e2e_local, launches

    line = None
    if rank == 0:
        flops_step = s.blocks * s.block_flops(sequence)
        achieved = flops_step / (ms * 1e-3) / 1e12 / world       # per GPU
        # live roofline of the dominant kernel (the tensor-core GEMM), timed alone -> burst peak
        rows = dit.rows_local
        w = step.blocks[0]
        kernels = {}
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
        kernels["qkv_proj_norm_rope"] = time_kernel(torch, gpu, qkv_op, qkv_flops)
        mlp_flops = 2.0 * rows * s.hidden * 2 * s.ffn + 2.0 * rows * s.ffn * s.hidden
        kernels["mlp_fc1_swiglu_fc2"] = time_kernel(
            torch, gpu, lambda: gpu.op("mlp_bf16", dit.attention_output, dit.mod_mlp, w.fc1, w.fc2,
                                       rows, s.hidden, s.ffn, s.hidden), mlp_flops)
        out_flops = 2.0 * rows * s.inner * s.hidden
        kernels["gemm_out_proj"] = time_kernel(
            torch, gpu, lambda: gpu.op("linear_bf16", dit.attention_output, dit.attention_heads, w.out,
                                       None, rows, s.inner, s.hidden), out_flops)
        if dit.push:
            attn_flops = 4.0 * sequence * sequence * (s.heads // world) * s.head_dim
            kernels["attention"] = time_kernel(
                torch, gpu, lambda: gpu.op("h3x_sdpa_push", exchange.peers, dit.gathered[0],
                                           dit.gathered[1], dit.gathered[2], sequence, s.heads,
                                           s.head_dim, s.scale), attn_flops)
        if world == 1:
            attn_flops = 4.0 * sequence * sequence * s.heads * s.head_dim
            kernels["attention"] = time_kernel(
                torch, gpu, lambda: gpu.op("sdpa_bf16", dit.attention_heads, dit.query, dit.key,
                                           dit.value, sequence, s.heads, s.head_dim, s.scale),
                attn_flops)
        qkv_ms, qkv_tf = kernels["qkv_proj_norm_rope"]
        roofline = {"bound": "tensor",
                    "kernel": ("h3b_gemm_pair<qkv+norm+rope> (QKV projection with fused head norm and RoPE, CTA pairs)"
                               if 128 < rows <= 8192 else
                               "h3b_gemm_tc<qkv+norm+rope> (QKV projection with fused head norm and RoPE)"),
                    "achieved": qkv_tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": qkv_tf / peaks["bf16_tflops"], "peak_source": peaks["source"] + " burst",
                    "ms_per_launch": qkv_ms, "flops_per_launch": qkv_flops,
                    "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get((args.workload, world)),
                    "traffic_unit": "bytes per launch (dram read+write, one ncu capture)"}
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
            "kernels": {k: {"ms": v[0], "tflops": v[1], "frac_of_burst_peak": v[1] / peaks["bf16_tflops"]}
                        for k, v in kernels.items()},
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
    mem = TorchMemory(torch, pkg, gpu, device)
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
    dit, step = build_model(torch, pkg, gpu, mem, shape, sequence, text_rows, exchange,
                            time_rows=euler_steps, text_seed=2 if group_id == 0 else 4)
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--blocks", type=int, default=50)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", default="push", choices=["push", "nccl", "loopback"],
                    help="N>1: peer stores fused into the kernels, or pack + NCCL all-to-all + unpack; "
                         "loopback = same kernels with the stores kept local and no barriers, to "
                         "measure the exposed cost of the exchange (results invalid)")
    ap.add_argument("--euler-steps", type=int, default=20, help="c5: Euler steps per denoise")
    ap.add_argument("--guidance", type=float, default=5.0,
                    help="c5: guidance scale (the reference has no guidance pass; harness parameter)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    import __graft_entry__ as entry
    pkg = entry.load_package()
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
