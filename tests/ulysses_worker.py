"""Worker for tests/test_gpu_ulysses.py: run under torch.distributed.run with N ranks.

Every rank holds a row slice of one DiT block's input, runs the block through the host
driver with the exchange around attention (argv[2]: nccl = pack + all-to-all + unpack,
push = peer stores from the kernels' epilogues), and rank 0 checks the gathered output
(per-block bar). argv[3] picks the case: "small" (hidden 512, 8 heads) is checked against the
CPU oracle's single-device block; "full" (the model's width: hidden 5376, 56 heads, FFN 14336,
so 28 / 14 / 7 heads per rank at 2 / 4 / 8 ranks) against the same block run unsharded on
rank 0, which the single-GPU tests pin to the oracle and to the reference's CUDA backend."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "oracle", ROOT / "tests"):
    sys.path.insert(0, str(p))

import h3_oracle as o  # noqa: E402
from block_case import make_block_case, run_block_on_gpu, upload_block  # noqa: E402
from parity import block_metrics  # noqa: E402
import __graft_entry__ as entry  # noqa: E402

entry.load_package()
from h3c_b200.plumbing import NcclExchange, TorchMemory  # noqa: E402


def main():
    rows = int(sys.argv[1]) if len(sys.argv) > 1 else 301
    mode = sys.argv[2] if len(sys.argv) > 2 else "nccl"
    full = len(sys.argv) > 3 and sys.argv[3] == "full"
    pkg = entry.load_package()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    gpu = pkg.Gpu(local)
    mem = TorchMemory(torch, gpu, device)
    heads, hidden, ffn = (56, 5376, 14336) if full else (8, 512, 1024)
    case = make_block_case(rows=rows, text_rows=37, heads=heads, hidden=hidden, ffn=ffn, seed=5,
                           fast=full)
    shape = pkg.DitShape(hidden=hidden, heads=heads, ffn=ffn, blocks=1)
    if mode == "push":
        def gather(obj):
            out = [None] * world
            dist.all_gather_object(out, obj)
            return out
        exchange = pkg.PeerExchange(gpu, world, rank, gather)
    else:
        exchange = NcclExchange(dist, mem, world, rank)
    dit = pkg.Dit(gpu, shape, rows, exchange=exchange, alloc=lambda n: mem.bf16(n))
    w = upload_block(pkg, gpu, case)
    r0, rl, valid = dit.row_begin, dit.rows_local, dit.rows_valid

    def local_slice(a, width, dtype):
        out = np.zeros(rl * width, dtype)
        out[:valid * width] = a.reshape(rows, width)[r0:r0 + valid].reshape(-1)
        return out

    row_map = gpu.u32(local_slice(case.row_map, 1, np.uint32))
    cos = gpu.bf16(local_slice(case.rope_cos, 48, np.uint16))
    sin = gpu.bf16(local_slice(case.rope_sin, 48, np.uint16))
    dit.hidden.write(local_slice(case.hidden, hidden, np.uint16))
    dist.barrier()
    gpu.begin()
    dit.run_block(w, row_map, cos, sin, False, None)
    gpu.submit()
    mine = torch.from_numpy(dit.hidden.read().astype(np.int32)).to(device)
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    ok = True
    if rank == 0:
        got = np.concatenate([g.cpu().numpy().astype(np.uint16) for g in gathered])[:rows * hidden]
        if full:
            want = run_block_on_gpu(pkg, gpu, case)
        else:
            want = o.dit_block(case.hidden, case.weights, case.row_map, case.rope_cos, case.rope_sin,
                               rows=rows, width=hidden, heads=heads, head_dim=128, ffn=ffn,
                               rope_half=48, round_p=1)
        r, m = block_metrics(got, want)
        ok = r <= 1e-2 and m <= 5e-2
        print(f"ulysses {mode} world={world} rows={rows} heads={heads}: rel_l2={r:.3e} max_abs={m:.3e} "
              f"{'PASS' if ok else 'FAIL'}", flush=True)
    dist.barrier()
    if mode == "push":
        exchange.close()
    dist.destroy_process_group()
    gpu.close()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
