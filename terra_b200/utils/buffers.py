"""Small buffer helpers for code written against the reference's names (core/buffer.py:29-50,
core/checkpoint/offload_utils.py:4-33). The training path of this repository does not use them: cross-rank staging lives
in the symmetric arenas (``parallel/nvlink.py``) and offload buffers in the C++ copy engine's pinned slab pool."""
from __future__ import annotations

from typing import Dict, Tuple

import torch

_BUFFERS: Dict[Tuple, torch.Tensor] = {}
_STREAMS: Dict[Tuple, "torch.cuda.Stream"] = {}


def get_preallocated_buffer(shape, dtype, device, key=0) -> torch.Tensor:
    """One cached tensor per ``(shape, dtype, device, key)``, allocated on first use and handed out again afterwards.
    Two users of the same key share the storage: give concurrent users different keys (the reference keys by rank only,
    which aliases the buffers of two live users of equal shape)."""
    k = (tuple(int(s) for s in shape), dtype, str(torch.device(device)), key)
    buf = _BUFFERS.get(k)
    if buf is None:
        buf = _BUFFERS[k] = torch.empty(k[0], dtype=dtype, device=device)
    return buf


def release_preallocated_buffers() -> None:
    _BUFFERS.clear()


def new_cpu_buffer_like(tensor: torch.Tensor, pin_memory: bool = True) -> torch.Tensor:
    """Host tensor with the shape, dtype and strides of ``tensor``, pinned when CUDA is available and asked for."""
    pin = bool(pin_memory) and torch.cuda.is_available()
    return torch.empty_strided(tensor.size(), tensor.stride(), dtype=tensor.dtype, device="cpu", pin_memory=pin)


def get_cuda_stream(device, name: str = "default"):
    """One side stream per ``(device, name)``; ``None`` without CUDA."""
    if not torch.cuda.is_available():
        return None
    k = (str(torch.device(device)), name)
    if k not in _STREAMS:
        _STREAMS[k] = torch.cuda.Stream(device=device)
    return _STREAMS[k]
