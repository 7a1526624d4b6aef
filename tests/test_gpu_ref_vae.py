"""The reference's own, unmodified video-VAE decoder host on both device backends.

oracle/build_ref.py compiles the reference's h3_video_vae.c, h3_weights.c and h3_safetensors.c in
place, together with tests/vae_host_driver.c, and links the result once against libh3b200.so
(vae_host_b200) and once against the reference's CUDA backend (vae_host_ref). Both programs load
the same synthetic checkpoint (tests/vae_host_case.py) through the reference's loader and decode
the same latent: the streamed single-tile path (run_decoder: weights loaded and freed block by
block) and the resident tiled path (decode_chunked: overlapping spatial tiles, temporal chunks
of seven latent frames, blending on the host).

Bar: decoded RGB frames cosine >= 0.999 and rel-L2 <= 2e-2 against the reference's backend, which
computes the same projections in TF32 and the same attention in BF16 (36 blocks deep)."""
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest

from vae_host_case import write_checkpoint

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
HOSTS = {"b200": ROOT / "oracle" / "_ref" / "vae_host_b200", "reference": ROOT / "oracle" / "_ref" / "vae_host_ref"}
needs_hosts = pytest.mark.skipif(not all(p.exists() for p in HOSTS.values()),
                                 reason="the reference-derived host programs were not built (oracle/build_ref.py)")


@pytest.fixture(scope="module")
def checkpoint(tmp_path_factory):
    return write_checkpoint(tmp_path_factory.mktemp("h3_vae_checkpoint"))


def run_host(which, checkpoint, out, latent, seed=1, extra_env=None):
    cmd = [str(HOSTS[which]), str(checkpoint), str(out), *map(str, latent), str(seed)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=1500, env=dict(os.environ, **(extra_env or {})))
    print(which, res.stdout.strip())
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-2500:]
    raw = np.fromfile(out, np.uint8)
    frames, height, width = np.frombuffer(raw[:12], np.int32)
    rgb = np.frombuffer(raw[12:], np.float32)
    assert rgb.size == frames * height * width * 3
    return (int(frames), int(height), int(width)), rgb


def compare(got, want, what):
    assert got[0] == want[0], (got[0], want[0])
    a, b = got[1].astype(np.float64), want[1].astype(np.float64)
    assert np.isfinite(a).all()
    cosine = float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))
    rel = float(np.linalg.norm(a - b) / np.linalg.norm(b))
    print(f"{what}: {got[0][0]} frames of {got[0][2]} x {got[0][1]}: cosine={cosine:.7f} rel_l2={rel:.3e} "
          f"max_abs={float(np.max(np.abs(a - b))):.3e} (values span {b.min():.3f} .. {b.max():.3f})")
    assert cosine >= 0.999 and rel <= 2e-2, what


@needs_hosts
def test_streamed_single_tile_decode(checkpoint, tmp_path):
    """Seven latent frames of 8 x 8 (128 x 128 pixels, 453 rows): one tile, weights streamed per block."""
    out = {w: run_host(w, checkpoint, tmp_path / f"{w}.bin", (7, 8, 8)) for w in HOSTS}
    compare(out["b200"], out["reference"], "single tile")


@needs_hosts
def test_resident_tiled_decode(checkpoint, tmp_path):
    """Twelve latent frames of 24 x 20 (384 x 320 pixels): two temporal chunks, and the reference's tile rule
    (h3_video_vae.c:738-762: the tile size between 256 and 320 pixels with the least total area) splits the
    height into overlapping tiles, all on the resident decoder."""
    out = {w: run_host(w, checkpoint, tmp_path / f"{w}.bin", (12, 24, 20)) for w in HOSTS}
    compare(out["b200"], out["reference"], "tiled")
