"""Worker for tests/test_gpu_ulysses.py: classifier-free guidance split over two GPU groups.

Run under torch.distributed.run with an even number of ranks. The first half of the ranks is
the cond group, the second half the uncond group; inside a group the sequence is sharded with
the kernels' own peer stores (groups of one rank run unsharded). After every forward, rank i of
one group swaps its velocity rows with rank i of the other group over NCCL, both combine, both
apply the Euler update. Rank 0 gathers the cond group's latents and checks the final latent
against the CPU oracle's guided loop (cosine >= 0.999)."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "oracle", ROOT / "tests"):
    sys.path.insert(0, str(p))

from denoise_case import PATCH, cosine, gpu_denoise, make_denoise_case, oracle_denoise  # noqa: E402
import __graft_entry__ as entry  # noqa: E402

entry.load_package()
from h3c_b200.plumbing import NcclPair, TorchMemory  # noqa: E402


def main():
    pkg = entry.load_package()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    half = world // 2
    group_id, group_rank = rank // half, rank % half
    groups = [dist.new_group(list(range(g * half, (g + 1) * half))) for g in range(2)]
    gpu = pkg.Gpu(local)
    mem = TorchMemory(torch, gpu, device)
    guidance = 3.0
    case = make_denoise_case(rows=203, text_rows=40, blocks=2, steps=3, seed=9,
                             sigmas=pkg.serving_sigmas(3))
    exchange = None
    if half > 1:
        def gather(obj):
            out = [None] * half
            dist.all_gather_object(out, obj, group=groups[group_id])
            return out
        exchange = pkg.PeerExchange(gpu, half, group_rank, gather)
    pair = NcclPair(dist, mem, (rank + half) % world, is_cond=group_id == 0)
    dist.barrier()
    latent, (begin, count) = gpu_denoise(pkg, gpu, case, guidance=guidance, exchange=exchange,
                                         pair=pair, text=case.text if group_id == 0 else case.text_uncond)
    full = torch.zeros(case.video_rows * PATCH, dtype=torch.float32, device=device)
    if group_id == 0:
        full[begin * PATCH:(begin + count) * PATCH] = torch.from_numpy(latent).to(device)
    dist.all_reduce(full)
    ok = True
    if rank == 0:
        want = oracle_denoise(case, guidance)
        got = full.cpu().numpy()
        cos = cosine(got, want)
        rel = float(np.linalg.norm(got - want) / np.linalg.norm(want))
        ok = cos >= 0.999 and rel <= 3e-2
        print(f"cfg world={world} (2 groups x {half}): cosine={cos:.7f} rel_l2={rel:.3e} "
              f"{'PASS' if ok else 'FAIL'}", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    if exchange is not None:
        exchange.close()
    dist.destroy_process_group()
    gpu.close()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
