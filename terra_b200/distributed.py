"""Process bootstrap (reference: utils.py:10-32): environment contract ``RANK`` / ``LOCAL_RANK`` / ``WORLD_SIZE`` /
``MASTER_ADDR`` / ``MASTER_PORT``; NCCL on GPUs, gloo on CPU."""
from __future__ import annotations

import datetime
import os
import random

import numpy as np
import torch
import torch.distributed as dist


def set_random_seed(seed: int = 1234) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def init_distributed(backend: str = None, timeout_s: int = 1800):
    """Returns ``(rank, world_size, device)``. Without ``WORLD_SIZE`` in the environment nothing is initialised."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available() and backend != "gloo"
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = {}
        if use_cuda:
            kw["device_id"] = device
        dist.init_process_group(backend=backend or ("nccl" if use_cuda else "gloo"), init_method="env://",
                                rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return rank, world, device
