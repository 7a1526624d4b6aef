"""Worker for tests/test_gpu_ulysses.py::test_checkpoint_tensor_is_read_once_and_broadcast: N ranks,
rank 0 reads a tensor from a file with the library's loader, NCCL broadcasts it, every rank
checks the bytes it received."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

entry.load_package()
from h3c_b200.plumbing import TorchMemory, load_bf16_once  # noqa: E402


def main():
    path, offset, elements = sys.argv[1], int(sys.argv[2]), int(sys.argv[3])
    pkg = entry.load_package()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    gpu = pkg.Gpu(local)
    mem = TorchMemory(torch, gpu, device)
    tensor = load_bf16_once(dist, mem, gpu, path, offset, elements, rank)
    torch.cuda.synchronize()
    want = np.fromfile(path, np.uint16, count=elements, offset=offset)
    ok = np.array_equal(tensor.read(), want)
    try:
        load_bf16_once(dist, mem, gpu, path + ".missing", 0, 16, rank)
        ok = False
    except RuntimeError:
        pass                                     # every rank gets the source rank's error
    flags = torch.tensor([int(ok)], device=device)
    dist.all_reduce(flags)
    if rank == 0:
        print(f"broadcast load world={world}: {'PASS' if int(flags[0]) == world else 'FAIL'}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    gpu.close()
    sys.exit(0 if int(flags[0]) == world else 1)


if __name__ == "__main__":
    main()
