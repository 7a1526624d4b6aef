"""A synthetic MiniMax-H3 DiT checkpoint that the reference's own loader accepts.

The reference host (h3_dit.c load_dit, h3_dit_schedule.c, h3_weights.c) opens a directory of
safetensors shards and asks for tensors by name with exact dtype and shape. The released
checkpoint (65 GB) is not available, so this writes one shard with every name and shape that
loader requests (h3_dit.c:518-525, 811-826, 887, 1426-1443; h3_dit_schedule.c:169-178,
266-269, 303-308). The safetensors parser checks that a tensor's byte range lies inside the
file and matches its shape, not that ranges are disjoint (h3_safetensors.c:323-342), so every
large tensor is a window into one pool of seeded N(0, 0.02) values: a different window per
tensor name, hence different weights per block, in a file of ~0.65 GB.

Values: projection matrices and biases N(0, 0.02) (BF16 pool and F32 pool), the two patch
projections N(0, 0.1) so that latent rows enter the residual stream at O(1) like the refined
text rows, norm gains 1, rope.inv_freq[i] = 10000^(-i/16). The same file feeds every backend under test, so its
contents do not enter parity; they only have to keep activations finite and O(1).
"""
from __future__ import annotations

import json
import struct
import zlib
from pathlib import Path

import numpy as np

HIDDEN, HEADS, HEAD_DIM, FFN, TEXT_DIM = 5376, 56, 128, 14336, 5120
INNER = HEADS * HEAD_DIM
TIME_DIM, TIME_INPUT, TIME_HIDDEN = 2688, 256, 5376
BLOCKS, MODALITIES, SLOTS = 50, 3, 6
VIDEO_PATCH, AUDIO_CHANNELS, ROPE_FREQS = 96, 32, 16


def tensor_list():
    """(name, dtype, shape, kind) for everything the loader asks for; kind: pool | patch | ones |
    inv_freq."""
    out = []

    def block(prefix):
        out.append((prefix + "norm1.weight", "BF16", [HIDDEN], "ones"))
        out.append((prefix + "norm2.weight", "BF16", [HIDDEN], "ones"))
        out.append((prefix + "attn.qkv_proj.weight", "BF16", [INNER * 3, HIDDEN], "pool"))
        out.append((prefix + "attn.q_norm.weight", "BF16", [HEAD_DIM], "ones"))
        out.append((prefix + "attn.k_norm.weight", "BF16", [HEAD_DIM], "ones"))
        out.append((prefix + "attn.out_proj.weight", "BF16", [HIDDEN, INNER], "pool"))
        out.append((prefix + "mlp.fc1.weight", "BF16", [FFN * 2, HIDDEN], "pool"))
        out.append((prefix + "mlp.fc2.weight", "BF16", [HIDDEN, FFN], "pool"))

    for b in range(BLOCKS):
        block(f"blocks.{b}.")
        out.append((f"blocks.{b}.adaln_proj.linear.weight", "BF16",
                    [MODALITIES * SLOTS * HIDDEN, TIME_DIM], "pool"))
        out.append((f"blocks.{b}.adaln_proj.linear.bias", "BF16", [MODALITIES * SLOTS * HIDDEN], "pool"))
    for b in range(2):
        block(f"token_refiner.blocks.{b}.")
    out += [
        ("token_refiner.final_norm.weight", "BF16", [HIDDEN], "ones"),
        ("condition_proj.weight", "BF16", [HIDDEN, TEXT_DIM], "pool"),
        ("condition_proj.bias", "BF16", [HIDDEN], "pool"),
        ("final_layer.norm.weight", "BF16", [HIDDEN], "ones"),
        ("final_layer.adaln_proj.linear.weight", "BF16", [2 * HIDDEN, TIME_DIM], "pool"),
        ("final_layer.adaln_proj.linear.bias", "BF16", [2 * HIDDEN], "pool"),
        ("rope.inv_freq", "F32", [ROPE_FREQS], "inv_freq"),
        ("video_patch_proj.weight", "F32", [HIDDEN, VIDEO_PATCH], "patch"),
        ("video_patch_proj.bias", "F32", [HIDDEN], "pool"),
        ("audio_patch_proj.weight", "F32", [HIDDEN, AUDIO_CHANNELS], "patch"),
        ("audio_patch_proj.bias", "F32", [HIDDEN], "pool"),
        ("final_layer.video_out.weight", "F32", [VIDEO_PATCH, HIDDEN], "pool"),
        ("final_layer.video_out.bias", "F32", [VIDEO_PATCH], "pool"),
        ("final_layer.audio_out.weight", "F32", [AUDIO_CHANNELS, HIDDEN], "pool"),
        ("final_layer.audio_out.bias", "F32", [AUDIO_CHANNELS], "pool"),
        ("time_embedder.proj_in.weight", "F32", [TIME_HIDDEN, TIME_INPUT], "pool"),
        ("time_embedder.proj_in.bias", "F32", [TIME_HIDDEN], "pool"),
        ("time_embedder.proj_out.weight", "F32", [TIME_DIM, TIME_HIDDEN], "pool"),
        ("time_embedder.proj_out.bias", "F32", [TIME_DIM], "pool"),
    ]
    return out


def _to_bf16(x: np.ndarray) -> np.ndarray:
    bits = x.view(np.uint32)
    return ((bits + 0x7fff + ((bits >> 16) & 1)) >> 16).astype(np.uint16)


def write_checkpoint(directory: Path, seed: int = 0, spread_bytes: int = 32 << 20) -> Path:
    """Writes <directory>/model.safetensors and returns its path."""
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    tensors = tensor_list()
    size = {"BF16": 2, "F32": 4}
    largest = {d: max(int(np.prod(shape)) * size[d] for _, dtype, shape, kind in tensors
                      if dtype == d and kind == "pool") for d in ("BF16", "F32")}
    # data section: ones | inv_freq | patch pool | F32 pool | BF16 pool (each 256-byte aligned)
    ones_bytes = HIDDEN * 2
    patch_bytes = HIDDEN * VIDEO_PATCH * 4
    regions, cursor = {}, 0
    for name, nbytes in (("ones", ones_bytes), ("inv_freq", ROPE_FREQS * 4), ("patch", 2 * patch_bytes),
                         ("F32", largest["F32"] + spread_bytes), ("BF16", largest["BF16"] + spread_bytes)):
        regions[name] = (cursor, nbytes)
        cursor = (cursor + nbytes + 255) & ~255
    total = cursor
    header = {}
    for name, dtype, shape, kind in tensors:
        nbytes = int(np.prod(shape)) * size[dtype]
        if kind == "ones":
            begin = regions["ones"][0]
        elif kind == "inv_freq":
            begin = regions["inv_freq"][0]
        else:
            # a window that depends on the name: distinct weights for distinct tensors
            start, span = regions["patch" if kind == "patch" else dtype]
            slack = span - nbytes
            begin = start + (zlib.crc32(name.encode()) % (slack // 256 + 1)) * 256
        header[name] = {"dtype": dtype, "shape": shape, "data_offsets": [begin, begin + nbytes]}
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * ((-(8 + len(text))) % 256)           # data section starts 256-byte aligned
    path = directory / "model.safetensors"
    rng = np.random.default_rng(seed)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        base = f.tell()

        def put(region, payload: bytes):
            f.seek(base + regions[region][0])
            f.write(payload)
        put("ones", np.full(HIDDEN, 0x3f80, np.uint16).tobytes())
        put("inv_freq", (10000.0 ** (-np.arange(ROPE_FREQS, dtype=np.float64) / ROPE_FREQS))
            .astype(np.float32).tobytes())
        for region, item, std, convert in (("patch", 4, 0.1, lambda x: x), ("F32", 4, 0.02, lambda x: x),
                                           ("BF16", 2, 0.02, _to_bf16)):
            start, span = regions[region]
            f.seek(base + start)
            left = span // item
            while left:
                n = min(left, 1 << 24)
                f.write(convert(rng.standard_normal(n, dtype=np.float32) * np.float32(std)).tobytes())
                left -= n
        f.truncate(base + total)
    return path
