"""Datasets: one ``.pt`` tensor per day (real data), and synthetic stand-ins that need no files.

Real (reference: dataloader/glorys/loader_glorys_seq.py, loader_glorys_parallel.py): files sorted by the number in
their name; train / test / validation are index ranges (first 9496 days, then 365, then 365); a sample is
``(state[t], state[t + lead])`` or the whole ``lead + 1`` sequence for rollout finetuning.
Synthetic (reference: dataloader/glorys/loader_glorys_fake.py): zeros or block-addressable N(0,1) so that a rank's
stripe equals the same rows of the global field.
"""
from __future__ import annotations

import os
import re
from glob import glob

import torch
from torch.utils import data

from .synthetic import block_normal, patchify_hwc

TRAIN_END_IDX = 9496
TEST_DAYS = 365


def _numeric_key(path):
    nums = re.findall(r"\d+", os.path.basename(path))
    return (int(nums[-1]) if nums else -1, path)


def split_bounds(total_files, status, train_end_idx=TRAIN_END_IDX, test_days=TEST_DAYS, lead_time=1):
    train_end_idx = min(train_end_idx, total_files)
    if status == 0:
        lo, hi = 0, train_end_idx
    elif status == 1:
        lo, hi = train_end_idx, min(total_files, train_end_idx + test_days)
    elif status == 2:
        lo, hi = min(total_files, train_end_idx + test_days), min(total_files, train_end_idx + 2 * test_days)
    else:
        raise ValueError(f"Unsupported GLORYS dataset status: {status}")
    return lo, max(lo, hi - lead_time)


class _DayFiles(data.Dataset):
    def __init__(self, root, status, norm_type, data_precision, lead_time, train_end_idx, test_days, return_sequence):
        if norm_type not in ("zs", "mm") or data_precision != "fp16":
            raise ValueError(f"Only GLORYS zs/mm fp16 data is supported, but got norm_type={norm_type}, "
                             f"data_precision={data_precision}")
        self.files_full = sorted(glob(os.path.join(root, "*.pt")), key=_numeric_key)
        if not self.files_full:
            raise FileNotFoundError(f"No GLORYS .pt files found under {root}")
        self.status, self.lead_time, self.return_sequence = status, lead_time, return_sequence
        self.start_idx, self.end_idx = split_bounds(len(self.files_full), status, train_end_idx, test_days, lead_time)
        self.length = max(0, self.end_idx - self.start_idx)

    def __len__(self):
        return self.length

    def _load_tensor(self, index):
        return torch.nan_to_num(torch.load(self.files_full[index], map_location="cpu"))

    def __getitem__(self, idx):
        i = self.start_idx + idx
        if self.return_sequence:
            return torch.stack([self._load_tensor(i + s) for s in range(self.lead_time + 1)], dim=0)
        return self._load_tensor(i), self._load_tensor(i + self.lead_time)


class GLORYSSequentialDataset(_DayFiles):
    """Whole fields, ``[C, H, W]`` or ``[H, W, C]`` fp16."""

    def __init__(self, root_full_path, status=0, norm_type="zs", data_precision="fp16", lead_time=1,
                 train_end_idx=TRAIN_END_IDX, test_days=TEST_DAYS, return_sequence=False):
        super().__init__(root_full_path, status, norm_type, data_precision, lead_time, train_end_idx, test_days,
                         return_sequence)


class GLORYSWindowLinearDataset(_DayFiles):
    """Fields pre-split per window-parallel rank: ``<root>/wp_rank_{r}/*.pt`` hold ``[h_loc, w, p*p*C]``."""

    def __init__(self, root_full_path, wp_rank, status=0, norm_type="zs", data_precision="fp16", lead_time=1,
                 train_end_idx=TRAIN_END_IDX, test_days=TEST_DAYS, return_sequence=False):
        super().__init__(os.path.join(root_full_path, f"wp_rank_{wp_rank}"), status, norm_type, data_precision, lead_time,
                         train_end_idx, test_days, return_sequence)


class FakeGLORYSSequentialDataset(data.Dataset):
    """Synthetic whole fields ``[H, W, C]`` fp16: zeros, or seeded N(0,1)."""

    def __init__(self, height=2041, width=4320, channels=93, length=64, lead_time=1, return_sequence=False, random=True,
                 seed=2025, dtype=torch.float16):
        self.h, self.w, self.c, self.length = height, width, channels, length
        self.lead_time, self.return_sequence, self.random, self.seed, self.dtype = lead_time, return_sequence, random, seed, dtype

    def __len__(self):
        return self.length

    def _state(self, sample, state):
        if not self.random:
            return torch.zeros(self.h, self.w, self.c, dtype=self.dtype)
        return block_normal(self.seed, sample, state, 0, self.h, self.w, self.c, self.dtype)

    def __getitem__(self, idx):
        if self.return_sequence:
            return torch.stack([self._state(idx, s) for s in range(self.lead_time + 1)], dim=0)
        return self._state(idx, 0), self._state(idx, self.lead_time)


class FakeGLORYSWindowLinearDataset(data.Dataset):
    """Synthetic stripes ``[h_loc, w, p*p*C]`` of the padded, patchified field of one window-parallel rank. Only the
    rank's rows are generated; they equal the same rows of ``FakeGLORYSSequentialDataset`` bit for bit."""

    def __init__(self, height, width, channels, patch_size, padded_shape, initial_padding, wp_size, wp_rank, length=64,
                 lead_time=1, return_sequence=False, random=True, seed=2025, dtype=torch.float16):
        self.h, self.w, self.c, self.p = height, width, channels, patch_size
        self.padded_shape, self.initial_padding = tuple(padded_shape), tuple(initial_padding)
        self.wp_size, self.wp_rank, self.length = wp_size, wp_rank, length
        self.lead_time, self.return_sequence, self.random, self.seed, self.dtype = lead_time, return_sequence, random, seed, dtype
        if self.padded_shape[0] // patch_size % wp_size != 0:
            raise ValueError(f"patch rows {self.padded_shape[0] // patch_size} must be divisible by wp size {wp_size}")

    def __len__(self):
        return self.length

    def _state(self, sample, state):
        ph, pw = self.padded_shape
        left, right, top, bottom = self.initial_padding
        rows = ph // self.wp_size
        g0, g1 = self.wp_rank * rows - top, (self.wp_rank + 1) * rows - top
        loc = torch.zeros(rows, pw, self.c, dtype=self.dtype)
        lo, hi = max(g0, 0), min(g1, self.h)
        if self.random and hi > lo:
            loc[lo - g0:hi - g0, left:left + self.w] = block_normal(self.seed, sample, state, lo, hi, self.w, self.c, self.dtype)
        return patchify_hwc(loc[None], self.p)[0]

    def __getitem__(self, idx):
        if self.return_sequence:
            return torch.stack([self._state(idx, s) for s in range(self.lead_time + 1)], dim=0)
        return self._state(idx, 0), self._state(idx, self.lead_time)
