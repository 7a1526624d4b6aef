"""A synthetic video-VAE decoder checkpoint that the reference's own loader accepts.

The reference's decoder host (h3_video_vae.c:170-260) opens a directory of safetensors shards,
asks for F32 tensors by name with exact rank and shape, and reads `<dir>/../config.json` for the
latent normalisation. The released checkpoint (9.7 GB) is not available, so this writes one
shard with every name and shape that loader requests. As for the DiT checkpoint of
dit_host_case.py, every large tensor is a window into one pool of seeded values (the parser
checks that a tensor's bytes lie inside the file, not that tensors are disjoint,
h3_safetensors.c:323-342): a different window per name, hence different weights per block, in
a file of ~0.17 GB.

Values: matrices, biases and register tokens N(0, 0.02) (1/sqrt(2048) = 0.022), norm gains 1,
residual scales 0.25, latents_mean 0 and latents_std 1. The same file feeds every backend under
test, so its contents do not enter parity; they only keep activations finite and O(1).
"""
from __future__ import annotations

import json
import struct
import zlib
from pathlib import Path

import numpy as np

LATENT, HIDDEN, LAYERS, HEADS, HEAD_DIM, FFN, REGISTERS = 24, 2048, 36, 32, 64, 8192, 4
INNER = HEADS * HEAD_DIM
OUTPUT_PATCH = 3 * 4 * 16 * 16


def tensor_list():
    """(name, shape, kind) for everything the loader asks for; kind: pool | ones | quarter."""
    out = [("post_quant_conv.weight", [LATENT, LATENT, 1, 1, 1], "pool"), ("post_quant_conv.bias", [LATENT], "pool"),
           ("decoder.x_embedder.weight", [HIDDEN, LATENT], "pool"), ("decoder.x_embedder.bias", [HIDDEN], "pool"),
           ("decoder.register_tokens", [1, REGISTERS, HIDDEN], "pool"),
           ("decoder.norm_out.weight", [HIDDEN], "ones"), ("decoder.norm_out.bias", [HIDDEN], "pool"),
           ("decoder.proj_out.weight", [OUTPUT_PATCH, HIDDEN], "pool"), ("decoder.proj_out.bias", [OUTPUT_PATCH], "pool")]
    for b in range(LAYERS):
        p = f"decoder.transformer_blocks.{b}."
        out += [(p + "norm1.weight", [HIDDEN], "ones"), (p + "attn.to_qkv.weight", [INNER * 3, HIDDEN], "pool"),
                (p + "attn.to_qkv.bias", [INNER * 3], "pool"), (p + "attn.to_out.weight", [HIDDEN, INNER], "pool"),
                (p + "attn.to_out.bias", [HIDDEN], "pool"), (p + "scale1", [HIDDEN], "quarter"),
                (p + "norm2.weight", [HIDDEN], "ones"), (p + "ff.w1.weight", [FFN * 2, HIDDEN], "pool"),
                (p + "ff.w1.bias", [FFN * 2], "pool"), (p + "ff.w2.weight", [HIDDEN, FFN], "pool"),
                (p + "ff.w2.bias", [HIDDEN], "pool"), (p + "scale2", [HIDDEN], "quarter")]
    return out


def write_checkpoint(root: Path, seed: int = 0, spread_bytes: int = 32 << 20) -> Path:
    """Writes <root>/config.json and <root>/vae/model.safetensors; returns the weight directory."""
    root = Path(root)
    directory = root / "vae"
    directory.mkdir(parents=True, exist_ok=True)
    (root / "config.json").write_text(json.dumps({"latents_mean": [0.0] * LATENT, "latents_std": [1.0] * LATENT}))
    tensors = tensor_list()
    largest = max(int(np.prod(shape)) * 4 for _, shape, kind in tensors if kind == "pool")
    regions, cursor = {}, 0
    for name, nbytes in (("ones", HIDDEN * 4), ("quarter", HIDDEN * 4), ("pool", largest + spread_bytes)):
        regions[name] = (cursor, nbytes)
        cursor = (cursor + nbytes + 255) & ~255
    total = cursor
    header = {}
    for name, shape, kind in tensors:
        nbytes = int(np.prod(shape)) * 4
        start, span = regions[kind]
        begin = start if kind != "pool" else start + (zlib.crc32(name.encode()) % ((span - nbytes) // 256 + 1)) * 256
        header[name] = {"dtype": "F32", "shape": shape, "data_offsets": [begin, begin + nbytes]}
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * ((-(8 + len(text))) % 256)           # data section starts 256-byte aligned
    path = directory / "model.safetensors"
    rng = np.random.default_rng(seed)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        base = f.tell()
        f.seek(base + regions["ones"][0])
        f.write(np.ones(HIDDEN, np.float32).tobytes())
        f.seek(base + regions["quarter"][0])
        f.write(np.full(HIDDEN, 0.25, np.float32).tobytes())
        f.seek(base + regions["pool"][0])
        left = regions["pool"][1] // 4
        while left:
            n = min(left, 1 << 24)
            f.write((rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)).tobytes())
            left -= n
        f.truncate(base + total)
    return directory
