"""Per-task constants that travel with every step (reference: dataloader/task_specific_data.py:11-82,
dataloader/glorys_utils.py:19-38): the land-sea mask in the model's output layout and ``padding_loss_scale``."""
from __future__ import annotations

import os

import torch

from .glorys_paths import resolve_glorys_mask_path
from .synthetic import land_mask_for_rank, patchify_hwc


def get_land_sea_mask(height, width, channels, use_fake=True, mask_path=None, frac=0.0, seed=7):
    """``[H, W, C]`` mask. Synthetic: ones (``frac == 0``, like the reference's fake mask) or seeded blobs;
    real: the tensor at ``TERRA_GLORYS_MASK_PATH`` (``[C, H, W]`` or ``[H, W, C]``)."""
    if use_fake:
        from .synthetic import blob_land_mask

        m2 = torch.ones(height, width) if frac <= 0 else blob_land_mask(height, width, frac, seed)
        return m2[:, :, None].expand(height, width, channels).contiguous()
    m = torch.load(resolve_glorys_mask_path(mask_path), map_location="cpu").float()
    if m.shape[0] == channels and m.shape[-1] != channels:
        m = m.permute(1, 2, 0)
    return m.contiguous()


def get_task_specific_data(task_type, device, optimizer_state_tuple, model_archi_params, other_params, manager,
                           micro_batch_size, model_type="sequential", dataset_config=None):
    if task_type != "glorys":
        raise ValueError(f"Unsupported task_type={task_type!r}; only 'glorys' is supported")
    cfg = dataset_config or {}
    a = model_archi_params
    H, W, C, p = a["height"], a["width"], a["num_channels"], a["patch_size"]
    use_fake = bool(cfg.get("use_fake_input", os.environ.get("TERRA_USE_FAKE_INPUT", "0") == "1"))
    mask = get_land_sea_mask(H, W, C, use_fake, cfg.get("mask_path"), float(cfg.get("land_fraction", 0.0)),
                             int(cfg.get("land_mask_seed", 7)))
    dt = torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32
    out = {"test_iter_num": int(cfg.get("test_iter_num", -1)), "show_gradient_flag": bool(cfg.get("show_gradient_flag", False))}
    if model_type == "sequential":
        out["land_sea_mask"] = mask.to(device, dt)
        out["padding_loss_scale"] = 1.0
        return out
    ph, pw = a["padded_shape"]
    left, right, top, bottom = a["initial_padding"]
    mp = torch.nn.functional.pad(mask, (0, 0, left, right, top, bottom))
    rows = ph // manager.get_wp_group_size()
    r = manager.get_wp_rank()
    out["land_sea_mask"] = patchify_hwc(mp[None, r * rows:(r + 1) * rows], p)[0].contiguous().to(device, dt)
    out["padding_loss_scale"] = float(ph * pw) / float(H * W)
    return out
