"""Sequence-parallel (Ulysses) host logic on CPU: two gloo ranks exchange head slices
around attention exactly as the GPU path does (pack order, equal-block all-to-all, tail
padding, unpack) and must reproduce single-rank attention bit-for-bit. Attention itself is
computed by the oracle here; on the GPU it is the tensor-core kernel."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, seq, heads, hd, results):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "oracle"))
    import __graft_entry__ as entry
    import h3_oracle as o
    pkg = entry.load_package()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n = seq * heads * hd
        q, k, v = (o.normal_bf16(n, s) for s in (1, 2, 3))
        rows_local, begin, valid = pkg.shard_rows(seq, world, rank)
        order = pkg.ulysses_pack_order(rows_local, heads, world)
        hpr = heads // world

        def local_rows(a):
            out = np.zeros((rows_local, heads, hd), np.uint16)          # padding rows stay zero
            out[:valid] = a.reshape(seq, heads, hd)[begin:begin + valid]
            return out

        def exchange(a):
            out = torch.empty_like(a)
            dist.all_to_all_single(out, a)
            return out

        gathered = []
        for a in (q, k, v):
            packed = local_rows(a).reshape(rows_local * heads, hd)[order]       # pack kernel
            t = torch.from_numpy(np.ascontiguousarray(packed).view(np.int32))   # gloo lacks 16-bit types
            gathered.append(exchange(t).numpy().view(np.uint16).reshape(-1))    # [world*rows_local][hpr][hd]
        total = world * rows_local
        # attention over the true sequence length: padding rows are the tail and are ignored
        o_g = np.zeros(total * hpr * hd, np.uint16)
        o_g[:seq * hpr * hd] = o.sdpa_bf16(gathered[0][:seq * hpr * hd], gathered[1][:seq * hpr * hd],
                                           gathered[2][:seq * hpr * hd], seq, hpr, hd, 1.0 / np.sqrt(hd))
        back = exchange(torch.from_numpy(o_g.view(np.int32))).numpy().view(np.uint16)
        out = np.empty((rows_local * heads, hd), np.uint16)
        out[order] = back.reshape(-1, hd)                                        # unpack kernel
        want = o.sdpa_bf16(q, k, v, seq, heads, hd, 1.0 / np.sqrt(hd)).reshape(seq, heads, hd)
        ok = np.array_equal(out.reshape(rows_local, heads, hd)[:valid], want[begin:begin + valid])
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("seq", [64, 37])     # 37: ragged, the last rank holds a padding row
def test_two_rank_ulysses_matches_single_rank(seq):
    world, heads, hd = 2, 4, 16
    port = 29500 + (os.getpid() % 2000) + seq
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, port, seq, heads, hd, results), nprocs=world, join=True)
    assert all(results.get(r) for r in range(world)), dict(results)


def test_shard_rows_covers_the_sequence():
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry
    pkg = entry.load_package()
    for seq, world in [(6400, 8), (50476, 8), (37, 2), (5, 8)]:
        spans = [pkg.shard_rows(seq, world, r) for r in range(world)]
        assert sum(v for _, _, v in spans) == seq
        assert all(rl == spans[0][0] for rl, _, _ in spans)
        assert [b for _, b, _ in spans] == sorted(b for _, b, _ in spans)
