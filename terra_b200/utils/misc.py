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
