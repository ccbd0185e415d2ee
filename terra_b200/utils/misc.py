"""Small helpers shared by the entry points (reference: utils.py:34-91)."""
from __future__ import annotations

import torch


def get_criterion(loss_func: str):
    """``L1`` -> mean absolute error, ``L2`` / ``MSE`` -> mean squared error."""
    if loss_func == "L1":
        return torch.nn.L1Loss(reduction="mean")
    if loss_func in ("L2", "MSE"):
        return torch.nn.MSELoss(reduction="mean")
    raise ValueError(f"unsupported loss_func {loss_func}")


def dtype_from_precision(precision: str):
    return {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[precision]


def count_parameters(model):
    total = sum(p.numel() for p in model.parameters())
    trainable = sum(p.numel() for p in model.parameters() if p.requires_grad)
    return total, trainable


def show_tensor_sum(description, tensor):
    print(description, f"{tensor.sum().item():.20f}", tensor.dtype)


def get_task_partition(rank: int, world_size: int, all_days: int = 331, div_10: bool = False):
    """``[start, end)`` of the items (days of a year of data, or tens of days with ``div_10``) that ``rank`` processes
    when ``world_size`` workers share them: the first ranks take ``n // world_size`` items, the last ``n % world_size``
    ranks one more (reference: utils.py:35-55)."""
    n = all_days // 10 + 1 if div_10 else all_days
    base, extra = divmod(n, world_size)
    small = world_size - extra                       # ranks that take `base` items
    if rank < small:
        start = rank * base
        return start, start + base
    start = small * base + (rank - small) * (base + 1)
    return start, start + base + 1


def sort_key(file_path: str) -> int:
    """Numeric sort key of files named ``<number>.<ext>``."""
    import os

    return int(os.path.splitext(os.path.basename(file_path))[0])


def all_reduce_and_print_rank0(x, rank, group, description) -> None:
    """Sum of ``x`` over ``group``, printed by rank 0 with full precision (a debugging aid for comparing layouts)."""
    import torch.distributed as dist

    t = x.detach().clone()
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    if rank == 0:
        print(description, f"{t.sum().item():.20f}", t.dtype)


def check_parallel_config(dp_size, mp_size, wp_topo, domain_topo, world_size, height, width, patch_size, window_size,
                          padding_scale=1) -> None:
    """The layout rules in one place: ``dp x mp x wp == world``, the padded window grid divides over the window-parallel
    grid, and the domain grid has ``mp`` cells. Raises ``ValueError`` with the offending numbers (reference:
    utils.py:121-150, which asserts)."""
    from .padding import get_padded_shape

    wh, ww = wp_topo
    if dp_size * mp_size * wh * ww != world_size:
        raise ValueError(f"dp_size * mp_size * wp_size ({dp_size * mp_size * wh * ww}) != world_size ({world_size})")
    _, _, padded = get_padded_shape(height, width, patch_size, window_size, padding_scale=padding_scale)
    win_h, win_w = (window_size, window_size) if isinstance(window_size, int) else window_size
    rows, cols = padded[0] // patch_size // win_h, padded[1] // patch_size // win_w
    if rows % wh or cols % ww:
        raise ValueError(f"window grid {rows} x {cols} does not divide over the window-parallel grid {wh} x {ww}")
    if domain_topo[0] * domain_topo[1] != mp_size:
        raise ValueError(f"domain grid {tuple(domain_topo)} does not have mp_size = {mp_size} cells")
