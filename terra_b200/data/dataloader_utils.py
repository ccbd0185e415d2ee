"""Input pipeline (reference: dataloader/dataloader_utils.py:23-723).

* ``get_dataloader_for_task`` / ``get_finetune_dataloader_for_task``: dataset choice (real / synthetic, whole field /
  pre-split), ``DistributedSampler`` over the data-parallel group, pinned-memory ``DataLoader``.
* ``resolve_required_tensors_from_dataloader``: batch -> ``{'input_tensor', 'label_tensor'}`` on the device.
* ``resolve_required_tensors_online_split_for_parallel``: whole fields -> this rank's stripe, on the CPU, before the
  upload: pad rows/cols to the padded shape, take the stripe, patchify to ``[B, h_loc, w, p*p*C]``, pin, copy.
* ``GlorysLeadDoubleBuffer``: two-slot prefetch of the next lead's label during rollout finetuning.
"""
from __future__ import annotations

import time
from typing import Dict, Optional

import torch
from torch.utils.data import DataLoader
from torch.utils.data.distributed import DistributedSampler

from .datasets import (FakeGLORYSSequentialDataset, FakeGLORYSWindowLinearDataset, GLORYSSequentialDataset,
                       GLORYSWindowLinearDataset)
from .glorys_paths import get_glorys_parallel_file_path_prefix, resolve_glorys_sequential_root
from .synthetic import patchify_hwc


def _padded_shape(model_archi_params, other_params=None):
    spec = (other_params or {}).get("padding_spec") or model_archi_params.get("padding_spec")
    return tuple(spec["padded_shape"]) if spec else None


def get_dataset_for_task(manager, task_type, model_type, model_archi_params, other_params, status, for_pretrain=True,
                         lead_time=1):
    if task_type != "glorys":
        raise ValueError(f"Unsupported task_type={task_type!r}; only 'glorys' is supported")
    norm = other_params.get("norm_type", "zs")
    prec = other_params.get("data_precision", "fp16")
    if model_type == "sequential":
        root = resolve_glorys_sequential_root(norm, prec, other_params.get("glorys_data_root"))
        return GLORYSSequentialDataset(root, status, norm, prec, lead_time, return_sequence=not for_pretrain)
    if model_type in ("parallel", "hybrid"):
        root = get_glorys_parallel_file_path_prefix(
            other_params["embedding_parallel_type"], model_archi_params["height"], model_archi_params["width"],
            other_params["wp_topo"], model_archi_params["patch_size"], model_archi_params["window_size"],
            model_archi_params["padding_scale"], norm, prec,
            other_params.get("padding_spec", model_archi_params.get("padding_spec")))
        return GLORYSWindowLinearDataset(root, manager.get_wp_rank(), status, norm, prec, lead_time,
                                         return_sequence=not for_pretrain)
    raise ValueError(f"unsupported model_type {model_type} for glorys dataset")


def _fake_dataset(model_type, model_archi_params, other_params, manager, lead_time, return_sequence, use_splited_data,
                  random=True, seed=2025, length=64):
    a = model_archi_params
    if model_type == "sequential" or not use_splited_data:
        return FakeGLORYSSequentialDataset(a["height"], a["width"], a["num_channels"], length, lead_time, return_sequence,
                                           random, seed)
    return FakeGLORYSWindowLinearDataset(a["height"], a["width"], a["num_channels"], a["patch_size"], a["padded_shape"],
                                         a["initial_padding"], manager.get_wp_group_size(), manager.get_wp_rank(), length,
                                         lead_time, return_sequence, random, seed)


def _loader(dataset, manager, micro_batch_size, num_workers, pin_memory=True):
    sampler = DistributedSampler(dataset, num_replicas=manager.get_dp_group_size(), rank=manager.get_dp_rank(),
                                 shuffle=True, drop_last=False)
    return DataLoader(dataset, num_workers=num_workers, shuffle=False, pin_memory=pin_memory and torch.cuda.is_available(),
                      batch_size=micro_batch_size, drop_last=True, sampler=sampler)


def get_dataloader_for_task(task_type, micro_batch_size, use_splited_data=True, status=0, num_workers=1, simplified=True,
                            use_uv=True, manager=None, model_type="sequential", model_archi_params=None, other_params=None,
                            use_fake_input=False, fake_input_random=True, fake_input_seed=2025, fake_length=64):
    if task_type != "glorys":
        raise ValueError(f"Unsupported task_type={task_type!r}; only 'glorys' is supported")
    if use_fake_input:
        ds = _fake_dataset(model_type, model_archi_params, other_params, manager, 1, False, use_splited_data,
                           fake_input_random, fake_input_seed, fake_length)
    elif model_type == "sequential" or not use_splited_data:
        ds = get_dataset_for_task(manager, task_type, "sequential", model_archi_params, other_params, status, True)
    else:
        ds = get_dataset_for_task(manager, task_type, model_type, model_archi_params, other_params, status, True)
    return _loader(ds, manager, micro_batch_size, num_workers)


def get_finetune_dataloader_for_task(task_type, micro_batch_size, lead_time, use_splited_data=True, status=0,
                                     num_workers=1, manager=None, model_type="sequential", model_archi_params=None,
                                     other_params=None, use_fake_input=False, fake_input_random=True, fake_input_seed=2025,
                                     fake_length=64, pin_memory=True):
    """Batches are whole ``lead_time + 1`` sequences ``[B, L+1, ...]``."""
    if task_type != "glorys":
        raise ValueError(f"Unsupported task_type={task_type!r}; only 'glorys' is supported")
    if use_fake_input:
        ds = _fake_dataset(model_type, model_archi_params, other_params, manager, lead_time, True, use_splited_data,
                           fake_input_random, fake_input_seed, fake_length)
    elif model_type == "sequential" or not use_splited_data:
        ds = get_dataset_for_task(manager, task_type, "sequential", model_archi_params, other_params, status, False, lead_time)
    else:
        ds = get_dataset_for_task(manager, task_type, model_type, model_archi_params, other_params, status, False, lead_time)
    return _loader(ds, manager, micro_batch_size, num_workers, pin_memory)


# ------------------------------------------------------------------------------------------------ layout helpers
def patch_fy(x, patch_size):
    """``[B, H, W, C] -> [B, H/p, W/p, p*p*C]`` in (p1, p2, c) order (dataloader/dataloader_utils.py:483-487)."""
    return patchify_hwc(x, patch_size)


def pad_tensor(tensor, initial_padding, data_format="NHWC"):
    left, right, top, bottom = initial_padding
    if data_format == "NHWC":
        return torch.nn.functional.pad(tensor, (0, 0, left, right, top, bottom))
    return torch.nn.functional.pad(tensor, (left, right, top, bottom))


def to_nhwc(tensor, channels):
    """Accept ``[..., C, H, W]`` or ``[..., H, W, C]`` and return channels-last."""
    if tensor.shape[-1] == channels:
        return tensor
    if tensor.shape[-3] == channels:
        return tensor.movedim(-3, -1)
    raise ValueError(f"cannot find a channel dimension of size {channels} in {tuple(tensor.shape)}")


def get_patch_fy_slice_from_wp_rank(x, patch_size, wp_group_size, wp_rank):
    """Stripe of a padded NHWC field for one rank, patchified."""
    rows = x.shape[1] // wp_group_size
    if x.shape[1] % wp_group_size or rows % patch_size:
        raise ValueError(f"padded height {x.shape[1]} must split into {wp_group_size} stripes of whole patches")
    return patch_fy(x[:, wp_rank * rows:(wp_rank + 1) * rows], patch_size)


def _upload(t, device, dtype, non_blocking=True):
    if torch.device(device).type == "cuda":
        t = t.contiguous()
        if not t.is_pinned():
            t = t.pin_memory()
        return t.to(device=device, dtype=dtype, non_blocking=non_blocking)
    return t.to(dtype)


def resolve_required_tensors_from_dataloader(batch, device, my_dtype, model_type="sequential", channels=93,
                                             non_blocking=True) -> Dict[str, torch.Tensor]:
    """A ``(input, label)`` batch -> device tensors in the layout the model takes (whole fields are made NHWC)."""
    inp, lab = batch
    if model_type == "sequential":
        inp, lab = to_nhwc(inp, channels), to_nhwc(lab, channels)
    return {"input_tensor": _upload(inp, device, my_dtype, non_blocking), "label_tensor": _upload(lab, device, my_dtype, non_blocking)}


def online_split_one(tensor, device, my_dtype, model_archi_params, other_params, manager, non_blocking=True):
    """Whole field(s) ``[B, H, W, C]`` (or NCHW) -> this rank's padded, patchified stripe on the device."""
    a = model_archi_params
    x = to_nhwc(tensor, a["num_channels"])
    x = pad_tensor(x, a["initial_padding"], "NHWC")
    ph = a["padded_shape"][0] // a["patch_size"]
    if ph % manager.get_wp_group_size():
        raise ValueError(f"patch rows {ph} must be divisible by the window-parallel size {manager.get_wp_group_size()}")
    local = get_patch_fy_slice_from_wp_rank(x, a["patch_size"], manager.get_wp_group_size(), manager.get_wp_rank())
    return _upload(local, device, my_dtype, non_blocking)


def resolve_required_tensors_online_split_for_parallel(batch, device, my_dtype, model_archi_params, other_params, manager,
                                                       non_blocking=True):
    inp, lab = batch
    return {"input_tensor": online_split_one(inp, device, my_dtype, model_archi_params, other_params, manager, non_blocking),
            "label_tensor": online_split_one(lab, device, my_dtype, model_archi_params, other_params, manager, non_blocking)}


def manually_split_data_for_parallel_training(required_tensors, task_type, model_archi_params, my_dtype, other_params,
                                              manager, data_format="NHWC", padding_scale=1):
    """Device-side variant of the online split (tensors are already on the device)."""
    out = {}
    for k, v in required_tensors.items():
        x = pad_tensor(to_nhwc(v, model_archi_params["num_channels"]), model_archi_params["initial_padding"], "NHWC")
        out[k] = get_patch_fy_slice_from_wp_rank(x, model_archi_params["patch_size"], manager.get_wp_group_size(),
                                                 manager.get_wp_rank()).to(my_dtype).contiguous()
    return out


class GlorysLeadDoubleBuffer:
    """Frames of one rollout sequence, uploaded one lead ahead on a copy stream (two device slots).

    ``buf[i]`` returns frame ``i`` on the device and schedules frame ``i + 1``; frames must be requested in
    increasing order. ``sequence_tensor`` is a pinned CPU tensor ``[L + 1, ...]``."""

    def __init__(self, sequence_tensor, device, dtype, lead_time):
        self.seq = sequence_tensor if (not torch.cuda.is_available() or sequence_tensor.is_pinned()) else sequence_tensor.pin_memory()
        self.device, self.dtype, self.lead_time = torch.device(device), dtype, lead_time
        self.cuda = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.slots = [None, None]
        self.events = [None, None]
        self.scheduled = {}
        self._transfer_s = 0.0
        self._schedule(0)

    def __len__(self):
        return self.seq.shape[0]

    def _schedule(self, i):
        if i >= len(self) or i in self.scheduled:
            return
        slot = i % 2
        t0 = time.time()
        if self.cuda:
            with torch.cuda.stream(self.stream):
                if self.slots[slot] is None:
                    self.slots[slot] = torch.empty(self.seq.shape[1:], dtype=self.dtype, device=self.device)
                else:
                    self.stream.wait_stream(torch.cuda.current_stream(self.device))
                self.slots[slot].copy_(self.seq[i], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
                self.events[slot] = ev
        else:
            self.slots[slot] = self.seq[i].to(self.dtype)
        self.scheduled[i] = slot
        self._transfer_s += time.time() - t0

    def __getitem__(self, i):
        self._schedule(i)
        slot = self.scheduled[i]
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_event(self.events[slot])
        out = self.slots[slot]
        self.scheduled = {k: v for k, v in self.scheduled.items() if k >= i}
        self._schedule(i + 1)
        return out

    def transfer_time_s(self):
        return self._transfer_s

    def release(self):
        self.slots = [None, None]
        self.seq = None


class _WholeSequenceOnDevice(list):
    """Every frame uploaded at once (no double buffering); keeps the upload time for the metrics."""

    transfer_s = 0.0

    def transfer_time_s(self):
        return self.transfer_s


def resolve_glorys_finetune_double_buffer(sequence_batch, device, dtype, lead_time, enabled=True, non_blocking=True):
    """``[B, L+1, ...]`` pinned batch -> per-lead accessor (double buffered on CUDA when ``enabled``). ``non_blocking``
    (YAML ``input_transfer_non_blocking``) applies to the single upload of the path without double buffering; the
    double buffer is asynchronous by construction (reference: train_scripts/test_finetune.py:116-131,940-960)."""
    seq = sequence_batch.transpose(0, 1).contiguous()        # [L+1, B, ...]
    if enabled:
        return GlorysLeadDoubleBuffer(seq, device, dtype, lead_time)
    t0 = time.time()
    dev = seq.to(device=device, dtype=dtype, non_blocking=bool(non_blocking))
    if not non_blocking and torch.device(device).type == "cuda":
        torch.cuda.synchronize(device)
    frames = _WholeSequenceOnDevice(dev[i] for i in range(dev.shape[0]))
    frames.transfer_s = time.time() - t0
    return frames
