"""Checkpoint whose *inputs* are parked in pinned host memory until backward needs them.

Reference behaviour (core/checkpoint/boundary_offload.py:83-199,391-406): a non-reentrant ``torch`` checkpoint is
wrapped in ``saved_tensors_hooks`` so that only the tensors the checkpoint itself keeps - its inputs - are
intercepted; floating CUDA tensors of at least ``min_numel`` elements go to the host on a side stream and come back
when backward unpacks them, after which the segment is recomputed.

Here the copies run on the C++ copy engine (csrc/copy_engine.cpp): a pool of pinned slabs that is allocated once
and reused, one ``cudaMemcpyAsync`` per tensor on dedicated D2H / H2D streams, event fencing against the compute
stream. In addition ``prefetch_pending()`` lets the runtime queue the H2D copy of the most recently offloaded
boundaries *before* backward reaches them (look-ahead), instead of stalling on the copy at unpack time.

Modes (``offload.mode``): ``async_d2h_h2d`` (default; both directions on side streams), ``async_d2h`` (H2D waits on
the compute stream), ``sync`` / ``strict_sync`` (both on the compute stream). CPU tensors pass through unchanged.
"""
from __future__ import annotations

import threading
from typing import Any, Dict, List, Optional

import torch
from torch.utils.checkpoint import checkpoint as torch_checkpoint

OFFLOAD_MIN_NUMEL = 1024 * 1024
OFFLOAD_PIN_MEMORY = True
OFFLOAD_NON_BLOCKING = True
OFFLOAD_MODE = "async_d2h_h2d"

_STAT_KEYS = ("pack_calls", "unpack_calls", "offloaded_tensors", "restored_tensors", "d2h_bytes", "h2d_bytes",
              "inline_tensors", "cpu_tensors", "prefetched_tensors",
              "sampling_offloaded_tensors", "sampling_restored_tensors", "sampling_d2h_bytes", "sampling_h2d_bytes",
              "transformer_offloaded_tensors", "transformer_restored_tensors", "transformer_d2h_bytes",
              "transformer_h2d_bytes")
_STATS: Dict[str, int] = {k: 0 for k in _STAT_KEYS}
_ENGINES: Dict[int, Any] = {}
_PENDING: List["_Parked"] = []      # offloaded, not yet restored, most recent last
_LOCK = threading.Lock()


def get_boundary_offload_stats() -> Dict[str, int]:
    out = dict(_STATS)
    for idx, eng in _ENGINES.items():
        for k, v in eng.stats().items():
            out[f"engine{idx}_{k}"] = int(v)
    return out


def reset_boundary_offload_stats() -> None:
    for k in _STATS:
        _STATS[k] = 0


def _engine(device: torch.device):
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _ENGINES:
        from .. import _ext

        _ENGINES[idx] = _ext.load().CopyEngine(idx)
    return _ENGINES[idx]


def _is_boundary_activation(t, min_numel) -> bool:
    return (torch.is_tensor(t) and t.is_floating_point() and t.numel() >= min_numel
            and not getattr(t, "no_checkpointing", False))


class _Parked:
    """One tensor living in a pinned slab."""

    __slots__ = ("ticket", "engine", "shape", "stride", "dtype", "device", "requires_grad", "gpu", "nbytes", "scope",
                 "contiguous_shape")

    def __init__(self, ticket, engine, t: torch.Tensor, scope):
        self.ticket, self.engine = ticket, engine
        self.shape, self.stride, self.dtype, self.device = tuple(t.shape), tuple(t.stride()), t.dtype, t.device
        self.requires_grad = t.requires_grad
        self.gpu: Optional[torch.Tensor] = None      # set once the H2D copy has been queued
        self.nbytes = t.numel() * t.element_size()
        self.scope = scope

    def start_restore(self, wait: bool) -> torch.Tensor:
        if self.gpu is None:
            self.gpu = torch.empty(self.shape, dtype=self.dtype, device=self.device)
            self.engine.restore(self.ticket, self.gpu, wait)
            h2d = torch.cuda.ExternalStream(self.engine.h2d_stream(), device=self.device)
            self.gpu.record_stream(h2d)
        elif wait:
            self.engine.wait(self.ticket)
        return self.gpu

    def finish(self):
        self.engine.release(self.ticket)
        with _LOCK:
            if self in _PENDING:
                _PENDING.remove(self)


def prefetch_pending(max_tensors: int = 1) -> int:
    """Queue the host->device copies of the ``max_tensors`` most recently parked boundaries (those backward will
    need first). Returns how many copies were queued."""
    with _LOCK:
        todo = [p for p in reversed(_PENDING) if p.gpu is None][:max_tensors]
    for p in todo:
        p.start_restore(wait=False)
        _STATS["prefetched_tensors"] += 1
    return len(todo)


class _BoundaryTensorStore:
    def __init__(self, offload_config=None):
        cfg = offload_config or {}
        scope = str(cfg.get("scope", "other")).strip().lower()
        self.scope = scope if scope in ("sampling", "transformer") else "other"
        self.min_numel = int(cfg.get("min_numel", OFFLOAD_MIN_NUMEL))
        self.pin_memory = bool(cfg.get("pin_memory", OFFLOAD_PIN_MEMORY))
        self.non_blocking = bool(cfg.get("non_blocking", OFFLOAD_NON_BLOCKING))
        self.mode = cfg.get("mode", OFFLOAD_MODE)
        if self.mode not in ("async_d2h", "async_d2h_h2d", "sync", "strict_sync"):
            raise ValueError(f"Unsupported boundary offload mode={self.mode}")
        self.lookahead = int(cfg.get("prefetch_lookahead", 1))

    def _count(self, what, nbytes):
        _STATS[f"{what}_tensors"] += 1
        _STATS["d2h_bytes" if what == "offloaded" else "h2d_bytes"] += nbytes
        if self.scope != "other":
            _STATS[f"{self.scope}_{what}_tensors"] += 1
            _STATS[f"{self.scope}_{'d2h' if what == 'offloaded' else 'h2d'}_bytes"] += nbytes

    def pack(self, t):
        _STATS["pack_calls"] += 1
        if not _is_boundary_activation(t, self.min_numel):
            _STATS["inline_tensors"] += 1
            return ("inline", t.detach(), t.requires_grad)
        if not t.is_cuda:
            _STATS["cpu_tensors"] += 1
            return ("inline", t.detach(), t.requires_grad)
        src = t.detach()
        if not src.is_contiguous():
            src = src.contiguous()
        eng = _engine(t.device)
        if self.mode in ("sync", "strict_sync"):
            host = torch.empty(src.shape, dtype=src.dtype, device="cpu", pin_memory=self.pin_memory)
            host.copy_(src, non_blocking=self.non_blocking and self.mode == "sync")
            self._count("offloaded", src.numel() * src.element_size())
            return ("host", host, t.requires_grad, t.device)
        ticket = eng.offload(src)
        # the caching allocator must not hand the block to someone else while the D2H stream still reads it
        src.record_stream(torch.cuda.ExternalStream(eng.d2h_stream(), device=t.device))
        parked = _Parked(ticket, eng, src, self.scope)
        parked.requires_grad = t.requires_grad
        with _LOCK:
            _PENDING.append(parked)
        self._count("offloaded", parked.nbytes)
        return ("parked", parked)

    def unpack(self, packed):
        _STATS["unpack_calls"] += 1
        kind = packed[0]
        if kind == "inline":
            out, req = packed[1], packed[2]
        elif kind == "host":
            out = packed[1].to(packed[3], non_blocking=self.non_blocking)
            req = packed[2]
            self._count("restored", out.numel() * out.element_size())
        else:
            parked: _Parked = packed[1]
            out = parked.start_restore(wait=True)
            out.record_stream(torch.cuda.current_stream(parked.device))
            req = parked.requires_grad
            self._count("restored", parked.nbytes)
            parked.finish()
            if self.lookahead > 0 and self.mode == "async_d2h_h2d":
                prefetch_pending(self.lookahead)     # the next boundary backward will reach
        out = out.detach()
        out.requires_grad_(bool(req))
        return out


def _first_tensor_device(args):
    for a in args:
        if torch.is_tensor(a):
            return a.device
    return None


def checkpoint(function, *args, offload_config=None):
    """Recompute checkpoint whose saved inputs are offloaded as configured."""
    if _first_tensor_device(args) is None:
        return function(*args)
    store = _BoundaryTensorStore(offload_config)
    # The hooks are active while the checkpoint records its inputs; inside the body PyTorch's own checkpoint
    # hooks take precedence, so nothing produced by the body is intercepted here.
    with torch.autograd.graph.saved_tensors_hooks(store.pack, store.unpack):
        return torch_checkpoint(function, *args, use_reentrant=False, preserve_rng_state=True)
