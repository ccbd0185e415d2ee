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


def bind_to_gpu_numa(device_index: int) -> bool:
    """Pin this process (and so its later pinned-memory allocations, by first touch) to the CPUs that NVML reports as
    local to the GPU. Host->device staging of multi-GB batches otherwise crosses the socket interconnect for the ranks
    whose GPU hangs off the other socket. Only the process's own CPU affinity is changed; no GPU setting is touched.
    ``TERRA_NUMA_BIND=0`` disables it. Returns whether a binding was applied."""
    if os.environ.get("TERRA_NUMA_BIND", "1") == "0" or not hasattr(os, "sched_setaffinity"):
        return False
    try:
        import pynvml

        pynvml.nvmlInit()
        try:
            handle = pynvml.nvmlDeviceGetHandleByIndex(_physical_gpu_index(device_index))
            words = (os.cpu_count() + 63) // 64
            mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        finally:
            pynvml.nvmlShutdown()
        cpus = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (int(m) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return False
        os.sched_setaffinity(0, cpus)
        return True
    except Exception:
        return False


def _physical_gpu_index(device_index: int) -> int:
    """Index of ``cuda:device_index`` in NVML's enumeration when CUDA_VISIBLE_DEVICES lists plain indices."""
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v.strip() for v in vis.split(",") if v.strip()]
        if device_index < len(ids) and ids[device_index].isdigit():
            return int(ids[device_index])
    return device_index


def init_distributed(backend: str = None, timeout_s: int = 1800):
    """Returns ``(rank, world_size, device)``. Without ``WORLD_SIZE`` in the environment nothing is initialised."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available() and backend != "gloo"
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
        bind_to_gpu_numa(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = {}
        if use_cuda:
            kw["device_id"] = device
        dist.init_process_group(backend=backend or ("nccl" if use_cuda else "gloo"), init_method="env://",
                                rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return rank, world, device
