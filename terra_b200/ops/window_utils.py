"""The explicit tensor forms of the window machinery that the attention kernels fold into their index arithmetic:
padding to whole windows, window partition / reverse, and the shifted-window attention mask.

Nothing on the training path calls these (the kernels locate every token of a shifted window in closed form and never
build a ``[windows, N, N]`` mask); they exist for pre- and post-processing code written against the reference's helper
names (models/utils.py:4-92), and as the plain statement of what the kernels' index arithmetic must reproduce: the
tests compare ``region_ids`` / ``shifted_window_sources`` of ``ops/attention.py`` with them. Windows may be rectangular
(``window_size`` an int or ``(wh, ww)``)."""
from __future__ import annotations

from typing import Sequence, Tuple, Union

import torch

Size2 = Union[int, Sequence[int]]


def _pair(v: Size2) -> Tuple[int, int]:
    return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))


def _split_pad(extent: int, window: int) -> Tuple[int, int]:
    """Padding (before, after) that brings ``extent`` up to a multiple of ``window``, the odd cell going behind."""
    short = (-extent) % window
    return short // 2, short - short // 2


def get_pad3d(input_resolution: Sequence[int], window_size: Sequence[int]):
    """``(left, right, top, bottom, front, back)`` for a ``(levels, lat, lon)`` grid and window."""
    (front, back), (top, bottom), (left, right) = (_split_pad(e, w) for e, w in zip(input_resolution, window_size))
    return left, right, top, bottom, front, back


def get_pad2d(input_resolution: Sequence[int], window_size: Sequence[int]):
    """``(left, right, top, bottom)`` for a ``(lat, lon)`` grid and window."""
    return get_pad3d([1] + list(input_resolution), [1] + list(window_size))[:4]


def window_partition(x: torch.Tensor, window_size: Size2) -> torch.Tensor:
    """``[B, H, W, C] -> [B * nWh * nWw, wh, ww, C]``, windows in row-major order within each sample."""
    wh, ww = _pair(window_size)
    B, H, W, C = x.shape
    tiles = x.reshape(B, H // wh, wh, W // ww, ww, C).transpose(2, 3)
    return tiles.reshape(-1, wh, ww, C)


def window_reverse(windows: torch.Tensor, window_size: Size2, H: int, W: int) -> torch.Tensor:
    """Inverse of ``window_partition``: ``[B * nWh * nWw, wh, ww, C] -> [B, H, W, C]``."""
    wh, ww = _pair(window_size)
    per_sample = (H // wh) * (W // ww)
    B = windows.shape[0] // per_sample
    tiles = windows.reshape(B, H // wh, W // ww, wh, ww, -1).transpose(2, 3)
    return tiles.reshape(B, H, W, -1)


def window_partition_HWBC(x: torch.Tensor, window_size: Size2) -> torch.Tensor:
    """``[H, W, B, C] -> [nWh * nWw * B, wh, ww, C]`` (window-major, the batch inside each window position)."""
    wh, ww = _pair(window_size)
    H, W, B, C = x.shape
    tiles = x.reshape(H // wh, wh, W // ww, ww, B, C).permute(0, 2, 4, 1, 3, 5)
    return tiles.reshape(-1, wh, ww, C)


def shift_region_map(H: int, W: int, window_size: Size2, shift_size: Size2) -> torch.Tensor:
    """``[H, W]`` region numbers 0..8 of the rolled frame: tokens of one window may attend to each other only inside
    one region (three bands per axis: untouched rows, the last window's rows before the seam, the rows wrapped around)."""
    (wh, ww), (sh, sw) = _pair(window_size), _pair(shift_size)

    def bands(extent, w, s):
        ids = torch.zeros(extent, dtype=torch.long)
        if s > 0:
            ids[extent - w:extent - s] = 1
            ids[extent - s:] = 2
        return ids

    return bands(H, wh, sh)[:, None] * 3 + bands(W, ww, sw)[None, :]


def get_swin_attention_mask(model_type, input_resolution, window_size: Size2, shift_size: Size2, manager=None) -> torch.Tensor:
    """``[windows, N, N]`` additive mask of shifted-window attention: 0 inside a region, -100 across regions. For
    ``model_type == 'parallel'`` the windows are cut into equal consecutive shares over the manager's model-parallel
    group and this rank's share is returned."""
    H, W = input_resolution
    wh, ww = _pair(window_size)
    regions = shift_region_map(H, W, window_size, shift_size).to(torch.float32)
    per_window = window_partition(regions[None, :, :, None], (wh, ww)).reshape(-1, wh * ww)
    mask = (per_window[:, None, :] != per_window[:, :, None]).to(torch.float32) * -100.0
    if model_type == "parallel" and manager is not None:
        n, r = manager.get_mp_group_size(), manager.get_mp_rank()
        share = mask.shape[0] // n
        mask = mask[r * share:(r + 1) * share]
    return mask
