#!/usr/bin/env python
"""Packed / raw size of the lossless bf16 codec for KV-like value distributions (CPU only).

The headline benchmark fills the cache with N(0,1) values. Real KV has per-channel scales, a few outlier
channels and heavy tails, which widen the exponent histogram of a tile. This script computes the size the
codec's format gives each tile (sampled histogram, 16 ranked exponents, the shorter of two prefix codes, per-chunk byte
rounding, raw fallback: the rules of ``flexkv_b200/csrc/kernels/kv_compress.h``) with numpy, checks the
first tile of every case against the byte-level reference encoder, and prints one JSON line per case.
"""
import argparse
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flexkv_b200.ops import kv_compress as K  # noqa: E402

TILE = 8192


def tile_bytes(v: np.ndarray) -> int:
    """v: uint16 bit patterns of one tile (TILE values)."""
    n = v.size
    C = n // K.CHUNK_VALS
    e = ((v >> 7) & 0xFF).astype(np.int64)
    ew = e.reshape(K.CHUNK_VALS // 2, C, 2)                  # word w = k*C + t holds values 2w, 2w+1
    hist = np.bincount(ew[::K.SAMPLE_STRIDE].reshape(-1), minlength=256)
    order = sorted((b for b in range(256) if hist[b] > 0), key=lambda b: (-int(hist[b]), b))[:K.RANKS]
    rank = np.full(256, K.RANKS, dtype=np.int64)
    rank[order] = np.arange(len(order))
    lens = {m: np.array([K._code_of(r, 0, m)[1] for r in range(K.RANKS + 1)], dtype=np.int64) for m in (1, 2)}
    cost = {m: int((hist * lens[m][rank]).sum()) for m in (1, 2)}
    length = lens[2 if cost[2] < cost[1] else 1][rank]
    bits = length[ew].sum(axis=(0, 2))                        # per chunk t
    payload = int(((bits + 7) // 8).sum())
    total = (K.HEADER_BYTES + C + n + payload + 15) // 16 * 16
    return min(total, 16 + 2 * n)


def cases(rng: np.random.Generator, tokens: int, heads: int, dim: int):
    shape = (tokens, heads, dim)
    ch = np.exp2(rng.uniform(-3, 3, size=dim)).astype(np.float32)
    out = {"N(0,1) (the benchmark's fill)": rng.standard_normal(shape, dtype=np.float32)}
    out["per-channel scales, log-uniform over 2^-3..2^3"] = rng.standard_normal(shape, dtype=np.float32) * ch
    x = rng.standard_normal(shape, dtype=np.float32)
    x[..., rng.choice(dim, 2, replace=False)] *= 30.0
    out["2 of 128 channels 30x larger (outlier channels)"] = x
    out["Student-t, 3 degrees of freedom (heavy tails)"] = rng.standard_t(3, size=shape).astype(np.float32)
    x = rng.standard_normal(shape, dtype=np.float32) * ch + rng.standard_normal(dim).astype(np.float32) * 2
    out["per-channel scales and per-channel offsets"] = x
    out["N(0,1) x per-token scale, log-normal sigma 1"] = rng.standard_normal(shape, dtype=np.float32) * \
        np.exp(rng.standard_normal((tokens, 1, 1))).astype(np.float32)
    out["uniform(-1, 1)"] = rng.uniform(-1, 1, size=shape).astype(np.float32)
    out["zeros (unwritten pages)"] = np.zeros(shape, dtype=np.float32)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--dim", type=int, default=128)
    a = ap.parse_args()
    rng = np.random.default_rng(0)
    data = cases(rng, a.tokens, a.heads, a.dim)
    data["random bit patterns (incompressible)"] = None
    for name, x in data.items():
        if x is None:
            bits = rng.integers(0, 1 << 16, size=a.tokens * a.heads * a.dim, dtype=np.uint16)
        else:
            bits = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16).reshape(-1)
        tiles = bits[:bits.size // TILE * TILE].reshape(-1, TILE)
        sizes = np.array([tile_bytes(t) for t in tiles])
        ref = K.reference_compress_tile(torch.from_numpy(tiles[0].view(np.int16).copy()).view(torch.bfloat16))
        assert ref.numel() == sizes[0], (name, ref.numel(), sizes[0])
        back = K.reference_decompress_tile(ref)
        assert torch.equal(back.view(torch.int16), torch.from_numpy(tiles[0].view(np.int16).copy())), name
        e = (bits >> 7) & 0xFF
        p = np.bincount(e, minlength=256) / e.size
        entropy = float(-(p[p > 0] * np.log2(p[p > 0])).sum())
        print(json.dumps({"case": name, "tiles": int(tiles.shape[0]),
                          "packed_over_raw": round(float(sizes.sum()) / (tiles.size * 2), 4),
                          "exponent_entropy_bits": round(entropy, 2),
                          "bound_if_exponents_at_entropy": round((8 + entropy) / 16, 4),
                          "tiles_stored_raw": int((sizes == 16 + 2 * TILE).sum())}))


if __name__ == "__main__":
    main()
