"""Synthetic fields for benchmarks and tests.

``block_normal`` is a block-addressable generator: the field is cut into 64-row blocks and every block is drawn
from its own generator seeded by a hash of (seed, sample, state, block), so a rank can produce only its own rows
and still match the rows of the global field bit for bit (the property the reference's fake datasets provide:
dataloader/glorys/loader_glorys_fake.py:13-81).
``blob_land_mask`` is a seeded land mask made of contiguous blobs covering about ``frac`` of the grid.
"""
from __future__ import annotations

import numpy as np
import torch

BLOCK_ROWS = 64
_MIX = 6364136223846793005
_INC = 1442695040888963407
_MASK64 = (1 << 64) - 1


def _hash_seed(seed: int, sample: int, state: int, block: int) -> int:
    h = seed & _MASK64
    for v in (sample, state, block):
        h = (h * _MIX + _INC + (v & _MASK64)) & _MASK64
        h ^= h >> 29
    return h & ((1 << 63) - 1)


def block_normal(seed, sample, state, row0, row1, width, channels, dtype=torch.float32):
    """Rows ``[row0, row1)`` of the N(0,1) field ``[H, W, C]`` of (seed, sample, state)."""
    out = torch.empty(row1 - row0, width, channels, dtype=dtype)
    b0, b1 = row0 // BLOCK_ROWS, (row1 - 1) // BLOCK_ROWS
    for b in range(b0, b1 + 1):
        g = torch.Generator().manual_seed(_hash_seed(seed, sample, state, b))
        blk = torch.randn(BLOCK_ROWS, width, channels, generator=g, dtype=torch.float32)
        lo, hi = max(row0, b * BLOCK_ROWS), min(row1, (b + 1) * BLOCK_ROWS)
        out[lo - row0:hi - row0] = blk[lo - b * BLOCK_ROWS:hi - b * BLOCK_ROWS].to(dtype)
    return out


def blob_land_mask(height, width, frac=0.3, seed=7, num_blobs=48):
    """[H, W] float mask, 0 on land, 1 on sea; land is a union of random ellipses grown until ``frac`` is covered."""
    rng = np.random.RandomState(seed)
    yy, xx = np.mgrid[0:height, 0:width]
    land = np.zeros((height, width), dtype=bool)
    scale = np.sqrt(frac * height * width / (np.pi * num_blobs))
    tries = 0
    while land.mean() < frac and tries < 50 * num_blobs:
        cy, cx = rng.randint(0, height), rng.randint(0, width)
        ry, rx = scale * rng.uniform(0.5, 1.6), scale * rng.uniform(0.5, 1.6)
        dy = yy - cy
        dx = np.minimum(np.abs(xx - cx), width - np.abs(xx - cx))     # periodic in longitude
        land |= (dy / ry) ** 2 + (dx / rx) ** 2 <= 1.0
        tries += 1
    return torch.from_numpy((~land).astype(np.float32))
