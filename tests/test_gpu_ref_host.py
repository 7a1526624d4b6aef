"""The reference's own, unmodified C host on both device backends.

oracle/build_ref.py compiles the reference's h3_dit.c, h3_dit_schedule.c, h3_host.c,
h3_weights.c and h3_safetensors.c in place, together with tests/dit_host_driver.c, and links
the result once against libh3b200.so (dit_host_b200) and once against the reference's CUDA
backend (dit_host_ref). Both programs load the same synthetic checkpoint (tests/dit_host_case.py)
through the reference's loader and run its text refiner, adaLN schedule precompute (the
2688 -> 96768 projection at its real row count), rope and row maps, the audio segment and audio
head, the row-map patch scatter, one forward, and whole samplers.

Bar: final latents cosine >= 0.999 (the denoise bar); the single forward's velocity likewise.
This is the drop-in claim itself: nothing of this repository's Python host layer is involved."""
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest

from dit_host_case import write_checkpoint

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
HOSTS = {"b200": ROOT / "oracle" / "_ref" / "dit_host_b200", "reference": ROOT / "oracle" / "_ref" / "dit_host_ref"}


@pytest.fixture(scope="module")
def checkpoint(tmp_path_factory):
    directory = tmp_path_factory.mktemp("h3_dit_checkpoint")
    write_checkpoint(directory)
    return directory


def run_host(which, checkpoint, out, layout, steps, core_reuse, token_reduction, passes, extra_env=None,
             ssd_streaming=0):
    cmd = [str(HOSTS[which]), str(checkpoint), str(out), *map(str, layout), str(steps), str(core_reuse),
           str(token_reduction), str(ssd_streaming), *passes]
    env = dict(os.environ, **(extra_env or {}))
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=1500, env=env)
    print(which, res.stdout.strip().replace("\n", "\n" + which + " "))
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-2500:]
    raw = np.fromfile(out, np.uint8)
    video, audio, count = np.frombuffer(raw[:12], np.int32)
    values = np.frombuffer(raw[12:], np.float32)
    assert count == len(passes) and values.size == (1 + count) * (video + audio)
    parts = values.reshape(1 + count, video + audio)
    return [(p[:video], p[video:]) for p in parts]


def cosine(a, b):
    a, b = a.astype(np.float64), b.astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


def rel_l2(a, b):
    a, b = a.astype(np.float64), b.astype(np.float64)
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))


def compare(label, got, want, check=True, who="b200 vs reference"):
    for (gv, ga), (wv, wa), what in zip(got, want, label):
        assert np.isfinite(gv).all() and np.isfinite(ga).all()
        cv, ca = cosine(gv, wv), cosine(ga, wa)
        print(f"{who}: {what}: video cosine={cv:.7f} rel_l2={rel_l2(gv, wv):.3e}; "
              f"audio cosine={ca:.7f} rel_l2={rel_l2(ga, wa):.3e}")
        if check:
            assert cv >= 0.999 and ca >= 0.999, what


def check_against_floor(labels, got, own, want):
    compare(labels, own, want, check=False, who="reference (other attention kernel) vs reference")
    compare(labels, got, want, check=False)
    for what, g, o_, w in zip(labels, got, own, want):
        for part, name in ((0, "video"), (1, "audio")):
            allowed = max(1e-3, 2.0 * (1.0 - cosine(o_[part], w[part])))
            assert 1.0 - cosine(g[part], w[part]) <= allowed, f"{what}, {name}"


needs_hosts = pytest.mark.skipif(not all(p.exists() for p in HOSTS.values()),
                                 reason="the reference host programs were not built")


@needs_hosts
def test_reference_host_runs_on_both_backends(checkpoint, tmp_path):
    """Production defaults (50 blocks, no reuse, no token reduction): text 64 rows, latent
    7 x 16 x 16 -> 448 video rows, 2 x 37 audio rows; one forward, the serving Euler sampler
    over 4 steps with every step evaluated and with reuse interval 3, and the RES solver."""
    layout, passes = (64, 7, 16, 16, 37), ["euler:1", "euler:3", "res"]
    out = {w: run_host(w, checkpoint, tmp_path / f"{w}.bin", layout, 4, 1, 0, passes) for w in HOSTS}
    # How much this 50-block model amplifies a change of rounding order by itself: the reference's
    # backend against itself with its other attention kernel (H3_CUDA_SDPA_FA2=0: same math,
    # another summation order; same cuBLASLt GEMMs). Samplers that take few, large steps feed
    # the difference back through the model, so each output is held to the bar of the denoise
    # (cosine >= 0.999) or, where the reference's own two routes are further apart than that,
    # to twice their distance.
    floor = run_host("reference", checkpoint, tmp_path / "floor.bin", layout, 4, 1, 0, passes,
                     extra_env={"H3_CUDA_SDPA_FA2": "0"})
    labels = ["forward velocity"] + [f"final latents, {p}" for p in passes]
    check_against_floor(labels, out["b200"], floor, out["reference"])
    # the serving sampler itself meets the plain bar
    for index in (1, 2):
        assert cosine(out["b200"][index][0], out["reference"][index][0]) >= 0.999
        assert cosine(out["b200"][index][1], out["reference"][index][1]) >= 0.999
    # the samplers moved the latents: the comparison is not vacuous
    assert rel_l2(out["reference"][1][0], out["reference"][2][0]) > 1e-3


@needs_hosts
def test_reference_host_speed_modes_on_both_backends(checkpoint, tmp_path):
    """The reference's speed modes, all host logic of h3_dit.c driving the same ops: token
    reduction (pooled blocks 4..30 with the fused pool/expand + adaLN kernels) and core reuse
    (block skipping with residual replay, interval 2); 6 Euler steps, reuse interval 2."""
    layout, passes = (64, 5, 16, 16, 21), ["euler:2"]
    out = {w: run_host(w, checkpoint, tmp_path / f"{w}.bin", layout, 6, 2, 1, passes) for w in HOSTS}
    floor = run_host("reference", checkpoint, tmp_path / "floor.bin", layout, 6, 2, 1, passes,
                     extra_env={"H3_CUDA_SDPA_FA2": "0"})
    check_against_floor(["forward velocity", "final latents, token reduction + core reuse"], out["b200"], floor,
                        out["reference"])


@needs_hosts
def test_reference_host_weight_streaming_gives_the_resident_result(checkpoint, tmp_path):
    """The reference's SSD-streaming mode (h3_dit.c:2355-2433): block weights are not resident,
    an I/O thread fills one of two slots through h3_gpu_tensor_stream_file_bf16 while the other
    slot's block runs. Same kernels, same weights: on this backend the result must equal the
    resident run bit for bit, which it only does if the streamed bytes are in place before the
    block that uses them starts and are not overwritten while it runs."""
    layout, passes = (32, 3, 16, 16, 11), ["euler:1"]
    resident = run_host("b200", checkpoint, tmp_path / "resident.bin", layout, 2, 1, 0, passes)
    streamed = run_host("b200", checkpoint, tmp_path / "streamed.bin", layout, 2, 1, 0, passes, ssd_streaming=1)
    for (rv, ra), (sv, sa) in zip(resident, streamed):
        assert np.array_equal(rv, sv) and np.array_equal(ra, sa)


@needs_hosts
def test_reference_host_sparse_attention_on_both_backends(checkpoint, tmp_path):
    """H3_SPARSE_ATTN: the reference's host builds the block-sparse mask from the token layout
    (h3_dit.c:1006-1132: video tiles attend video tiles within a window of latent positions, tiles
    with text or audio rows stay global) and registers it with h3_gpu_sdpa_set_sparse; every
    attention of the denoise then runs under it. Radius 0 in time keeps, for a video tile, only
    the tiles that share a frame with it. The mask must have changed the result. Bar: cosine
    >= 0.999 on the video latents; 0.998 on the 74 audio rows, which move most when 50 blocks
    amplify a change of summation order (measured here: video 0.9997-0.9998, audio 0.9992-0.9995;
    the dense test above holds them to twice the distance between the reference's own two
    attention kernels for the same reason)."""
    layout, passes = (64, 7, 16, 16, 37), ["euler:1"]
    window = {"H3_SPARSE_ATTN": "0:8:8"}
    out = {w: run_host(w, checkpoint, tmp_path / f"{w}.bin", layout, 4, 1, 0, passes, extra_env=window)
           for w in HOSTS}
    labels = ["forward velocity", "final latents, windowed attention"]
    compare(labels, out["b200"], out["reference"], check=False)
    for what, (gv, ga), (wv, wa) in zip(labels, out["b200"], out["reference"]):
        assert cosine(gv, wv) >= 0.999 and cosine(ga, wa) >= 0.998, what
    dense = run_host("b200", checkpoint, tmp_path / "dense.bin", layout, 4, 1, 0, passes)
    assert rel_l2(out["b200"][0][0], dense[0][0]) > 1e-3, "the mask left the forward pass unchanged"
