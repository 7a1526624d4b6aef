"""Sequence-parallel block on real GPUs: N ranks (one process per GPU) must reproduce the
single-device block, with both forms of the exchange around attention: pack + NCCL all-to-all +
unpack, and peer stores from the kernels' epilogues over CUDA IPC mappings. Needs at least two
GPUs; skipped otherwise."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def gpu_count():
    import torch
    return torch.cuda.device_count()


def run_worker(world, *argv):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    port = 29600 + os.getpid() % 300
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                          f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                          "--master-port", str(port), str(ROOT / "tests" / "ulysses_worker.py"),
                          *map(str, argv)],
                         capture_output=True, text=True, timeout=900, env=env)
    print(res.stdout[-2000:])
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert "PASS" in res.stdout


@pytest.mark.parametrize("mode", ["nccl", "push"])
@pytest.mark.parametrize("rows", [300, 301])      # 301: the last rank holds a padding row
def test_sharded_block_matches_oracle(rows, mode):
    if gpu_count() < 2:
        pytest.skip("needs at least two GPUs")
    run_worker(2, rows, mode, "small")


@pytest.mark.parametrize("world", [4, 8])
def test_sharded_block_matches_oracle_on_more_ranks(world):
    """2 heads / 1 head per rank, ragged last shard (301 rows over 4 or 8 ranks)."""
    if gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    run_worker(world, 301, "push", "small")


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("mode", ["push", "nccl"])
def test_full_width_sharded_block_matches_single_gpu(world, mode):
    """The model's width (56 heads: 28 / 14 / 7 per rank; at 8 ranks the 21 q/k/v units of a
    rank leave the last 256-column QKV tile half empty) at S = 1,664 (208 rows per rank at 8)."""
    if gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    run_worker(world, 1664, mode, "full")


@pytest.mark.parametrize("world", [2, 4])
def test_guidance_groups_match_oracle(world):
    """Classifier-free guidance over two groups of world/2 ranks (tests/cfg_worker.py)."""
    if gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    port = 29300 + os.getpid() % 300
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                          f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                          "--master-port", str(port), str(ROOT / "tests" / "cfg_worker.py")],
                         capture_output=True, text=True, timeout=600, env=env)
    print(res.stdout[-2000:])
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert "PASS" in res.stdout


def test_checkpoint_tensor_is_read_once_and_broadcast(tmp_path):
    """One rank reads a checkpoint tensor from disk, NCCL hands it to the others over NVLink
    (h3.c_b200/plumbing.py load_bf16_once): with N ranks the file is read once, not N times."""
    import numpy as np
    n = gpu_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 2
    rng = np.random.default_rng(5)
    elements = (40 << 20) // 2 + 77
    path = tmp_path / "weights.bin"
    with open(path, "wb") as f:
        f.write(b"x" * 100)
        f.write(rng.integers(0, 1 << 16, elements, dtype=np.uint16).tobytes())
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    port = 29200 + os.getpid() % 300
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                          f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", str(port),
                          str(ROOT / "tests" / "broadcast_worker.py"), str(path), "100", str(elements)],
                         capture_output=True, text=True, timeout=600, env=env)
    print(res.stdout[-1500:])
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-3000:]
    assert "PASS" in res.stdout
