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


def block_normal(seed, sample, state, row0, row1, width, channels, dtype=torch.float32, device="cpu"):
    """Rows ``[row0, row1)`` of the N(0,1) field ``[H, W, C]`` of (seed, sample, state).

    ``device="cuda"`` draws the blocks with the GPU generator (much faster for benchmark-sized fields; the values
    differ from the CPU generator's but have the same block-addressable property) and returns a host tensor."""
    out = torch.empty(row1 - row0, width, channels, dtype=dtype)
    b0, b1 = row0 // BLOCK_ROWS, (row1 - 1) // BLOCK_ROWS
    dev = torch.device(device)
    for b in range(b0, b1 + 1):
        g = torch.Generator(device=dev).manual_seed(_hash_seed(seed, sample, state, b))
        blk = torch.randn(BLOCK_ROWS, width, channels, generator=g, dtype=torch.float32, device=dev)
        lo, hi = max(row0, b * BLOCK_ROWS), min(row1, (b + 1) * BLOCK_ROWS)
        out[lo - row0:hi - row0] = blk[lo - b * BLOCK_ROWS:hi - b * BLOCK_ROWS].to(dtype).cpu()
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


def patchify_hwc(x, p):
    """[B, H, W, C] -> [B, H/p, W/p, p*p*C] with (p1, p2, c) feature order."""
    Bn, H, W, C = x.shape
    return x.reshape(Bn, H // p, p, W // p, p, C).permute(0, 1, 3, 2, 4, 5).reshape(Bn, H // p, W // p, p * p * C)


def synthetic_batch(height, width, channels, patch_size, padded_shape, initial_padding, model_type, wp_size=1, wp_rank=0,
                    batch=1, sample=0, seed=2025, dtype=torch.float32, pin=False, gen_device="cpu"):
    """Seeded N(0,1) input / next-step label pair in the layout the model takes: the raw NHWC field for the
    sequential build, this rank's row stripe of the padded, patchified field for the parallel build."""
    out = {}
    for state, key in ((0, "input_tensor"), (1, "label_tensor")):
        if model_type == "sequential":
            t = torch.stack([block_normal(seed, sample * batch + b, state, 0, height, width, channels, dtype, gen_device)
                             for b in range(batch)])
        else:
            ph, pw = padded_shape
            left, right, top, bottom = initial_padding
            rows = ph // wp_size
            g0, g1 = wp_rank * rows - top, (wp_rank + 1) * rows - top          # rows of the unpadded field
            parts = []
            for b in range(batch):
                loc = torch.zeros(rows, pw, channels, dtype=dtype)
                lo, hi = max(g0, 0), min(g1, height)
                if hi > lo:
                    loc[lo - g0:hi - g0, left:left + width] = block_normal(seed, sample * batch + b, state, lo, hi, width, channels,
                                                                         dtype, gen_device)
                parts.append(patchify_hwc(loc[None], patch_size)[0])
            t = torch.stack(parts)
        t = t.to(dtype).contiguous()
        out[key] = t.pin_memory() if (pin and torch.cuda.is_available()) else t
    return out


def land_mask_for_rank(height, width, channels, patch_size, padded_shape, initial_padding, model_type, wp_size=1,
                       wp_rank=0, frac=0.3, seed=7, ones=False):
    """Mask in the model's output layout (no batch dimension) and ``padding_loss_scale`` = padded / real area."""
    m2 = torch.ones(height, width) if ones else blob_land_mask(height, width, frac, seed)
    if model_type == "sequential":
        return m2[:, :, None].expand(height, width, channels).contiguous(), 1.0
    ph, pw = padded_shape
    left, right, top, bottom = initial_padding
    mp = torch.nn.functional.pad(m2, (left, right, top, bottom))
    rows = ph // wp_size
    stripe = mp[wp_rank * rows:(wp_rank + 1) * rows]
    mask = patchify_hwc(stripe[None, :, :, None].expand(1, rows, pw, channels), patch_size)[0].contiguous()
    return mask, float(ph * pw) / float(height * width)
