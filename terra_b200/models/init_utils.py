"""Deterministic, layout-independent initialisation.

Every sub-module is created under a fixed seed with the global RNG state saved and restored, and tensor-parallel
shards are slices of the full seeded layer, so the sequential, window-parallel and TP-sharded builds start from
identical weights (reference: models/reference_model/init_utils.py:5-33, models/model_utils/init_weight.py:18-112).
The sequence of RNG draws per seed is part of that contract: ``nn.Linear(in, out)`` first, nothing else.
"""
from __future__ import annotations

import contextlib

import torch

REFERENCE_INIT_SEEDS = {
    "layers": 2026061001,
    "patch_embed": 2026061002,
    "patch_recovery": 2026061003,
    "down_blk": 2026061004,
    "up_blk": 2026061005,
    "attention": 2026061006,
    "mlp": 2026061007,
}


@contextlib.contextmanager
def deterministic_rng(seed):
    """Seed CPU (and CUDA, when present) generators for the body, then put the previous states back."""
    if seed is None:
        yield
        return
    cpu_state = torch.get_rng_state()
    cuda_states = torch.cuda.get_rng_state_all() if torch.cuda.is_available() else None
    torch.manual_seed(int(seed))
    if cuda_states is not None:
        torch.cuda.manual_seed_all(int(seed))
    try:
        yield
    finally:
        torch.set_rng_state(cpu_state)
        if cuda_states is not None:
            torch.cuda.set_rng_state_all(cuda_states)


def make_with_seed(seed, factory):
    with deterministic_rng(seed):
        return factory()


def run_with_seed(seed, fn):
    with deterministic_rng(seed):
        return fn()


def make_linear_with_seed(in_dim, out_dim, bias=True, init_seed=None):
    with deterministic_rng(init_seed):
        return torch.nn.Linear(in_dim, out_dim, bias=bias)


def linear_from_tensors(weight, bias=None):
    """An ``nn.Linear`` holding the given tensors; the global RNG does not advance."""
    with deterministic_rng(0):
        lin = torch.nn.Linear(weight.shape[1], weight.shape[0], bias=bias is not None)
    with torch.no_grad():
        lin.weight.copy_(weight)
        if bias is not None:
            lin.bias.copy_(bias)
    return lin


def sharded_linear_tensors(in_dim, out_dim, tp_rank=0, tp_size=1, split_dim=None, split_bias=True, init_seed=None):
    """Build the full seeded ``Linear(in_dim, out_dim)`` and return this TP rank's (weight, bias) slice.

    ``split_dim=0``: output features (column parallel), bias sliced alike; ``split_dim=-1``: input features
    (row parallel), bias kept whole unless ``split_bias``; ``None``: no sharding."""
    full = make_linear_with_seed(in_dim, out_dim, bias=True, init_seed=init_seed)
    w, b = full.weight.data, full.bias.data
    if split_dim is None or tp_size == 1:
        return w.clone(), b.clone()
    if split_dim == 0:
        if not split_bias:
            raise ValueError("column-parallel linears shard their bias")
        return w.chunk(tp_size, dim=0)[tp_rank].clone(), b.chunk(tp_size, dim=0)[tp_rank].clone()
    if split_dim == -1:
        wb = w.chunk(tp_size, dim=1)[tp_rank].contiguous().clone()
        bb = b.chunk(tp_size, dim=0)[tp_rank].clone() if split_bias else b.clone()
        return wb, bb
    raise ValueError(f"unrecognized split_dim {split_dim}")
