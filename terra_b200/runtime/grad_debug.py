"""Gradient inspection helpers of the test harness (reference: core/runtime/run_model.py:49-360).

* ``show_gradient``: after the backward pass of the last test iteration (``show_gradient_flag`` and
  ``test_iter_num`` in the task constants) print the sum of the gradient and of the value of a fixed list of parameters
  (first / last layers of every stage), reduced over the ranks that hold shards of a tensor-parallel parameter, so that
  serial and parallel runs can be compared line by line.
* ``install_grad_hooks`` (env ``DEBUG_GRAD_HOOK=1``): per-parameter hooks that print the gradient sum at the moment
  autograd produces it, at most ``DEBUG_GRAD_HOOK_PRINT_LIMIT`` lines. With the flat parameter arena the hook reads
  the arena's gradient view, which the fused kernels accumulate into directly.
* ``report_arena_gradients``: the CUDA form of the same switch. The fused kernels write parameter gradients into the
  flat gradient arena without autograd ever producing a leaf gradient, so no hook fires there; instead the step
  prints, right after the backward pass, the gradient sum of every parameter from the arena's views (one
  device-side reduction over the arena segments, one host transfer), under the same line limit."""
from __future__ import annotations

from typing import Iterable, List, Optional

import torch
import torch.distributed as dist

from .. import global_env_config as G

WATCHED_SUFFIXES = (
    "patch_embed.weight", "patch_embed.bias", "patch_embed.linear.weight", "patch_embed.linear.bias",
    "patch_recovery.weight", "patch_recovery.bias", "patch_recovery.linear.weight", "patch_recovery.linear.bias",
    "down_blk.conv.weight", "down_blk.conv.bias", "down_blk.conv.conv.weight", "down_blk.conv.conv.bias",
    "up_blk.conv.weight", "up_blk.conv.bias", "up_blk.conv.conv.weight", "up_blk.conv.conv.bias",
    "norm1.weight", "norm1.bias", "attn.q_linear.weight", "attn.q_linear.bias", "attn.proj.weight", "attn.proj.bias",
    "attn.relative_position_bias_table", "norm2.weight", "norm2.bias", "mlp.linear1.weight", "mlp.linear2.weight",
    "linear1.weight", "linear2.weight",
)


def watched_parameters(model) -> List[tuple]:
    """(name, parameter) of the watched tensors of the first and the last transformer block plus the embedding,
    recovery and sampling layers; ``module.`` prefixes of wrappers are ignored."""
    named = [(n[len("module."):] if n.startswith("module.") else n, p) for n, p in model.named_parameters()]
    block_names = sorted({n.split(".norm1.")[0] for n, _ in named if ".norm1." in n})
    keep_blocks = {block_names[0], block_names[-1]} if block_names else set()
    out = []
    for n, p in named:
        if not n.endswith(WATCHED_SUFFIXES):
            continue
        in_block = any(n.startswith(b + ".") for b in block_names)
        if in_block and not any(n.startswith(b + ".") for b in keep_blocks):
            continue
        out.append((n, p))
    return out


def _grad_of(p) -> Optional[torch.Tensor]:
    g = getattr(p, "grad", None)
    return g if g is not None else getattr(p, "main_grad", None)


def show_gradient(model, manager=None, tp_group=None, printer=print) -> List[str]:
    """Print (and return) one line per watched parameter: name, gradient sum, value sum. Sharded parameters are
    summed over ``tp_group``; only the group's first rank prints."""
    lines = []
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    for name, p in watched_parameters(model):
        g = _grad_of(p)
        vals = torch.stack([(g.detach().double().sum() if g is not None else torch.zeros((), dtype=torch.float64, device=p.device)),
                            p.detach().double().sum()])
        if tp_group is not None and getattr(p, "terra_grad_reduce_group", None) not in (None, "replicated"):
            dist.all_reduce(vals, group=tp_group)
        lines.append(f"[grad] rank {rank} {name}: grad_sum {vals[0].item():+.8e} param_sum {vals[1].item():+.8e}")
    if rank == 0 or manager is None:
        for ln in lines:
            printer(ln)
    return lines


def install_grad_hooks(model, limit: Optional[int] = None, printer=print):
    """Register the per-parameter debug hooks; returns the handles (``.remove()`` to uninstall)."""
    limit = G.DEBUG_GRAD_HOOK_PRINT_LIMIT if limit is None else limit
    state = {"n": 0}
    handles = []
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue

        def hook(grad, name=name, p=p):
            if state["n"] < limit:
                state["n"] += 1
                src = grad if grad is not None else _grad_of(p)
                printer(f"[grad hook] {name}: {src.detach().double().sum().item():+.8e}")
            return grad

        handles.append(p.register_hook(hook))
    return handles


_arena_lines = {"n": 0}


def report_named_gradients(named, limit: Optional[int] = None, printer=print) -> List[str]:
    """One ``[grad hook] name: sum`` line per ``(name, parameter)`` that has a gradient, at most ``limit`` lines over the
    run (shared with the other reports), with one device-to-host transfer."""
    limit = G.DEBUG_GRAD_HOOK_PRINT_LIMIT if limit is None else limit
    if _arena_lines["n"] >= limit:
        return []
    named = [(n, p) for n, p in named if p.requires_grad and _grad_of(p) is not None]
    if not named:
        return []
    sums = torch.stack([_grad_of(p).detach().double().sum() for _, p in named]).cpu()      # one transfer
    lines = []
    for (name, _), v in zip(named, sums.tolist()):
        if _arena_lines["n"] >= limit:
            break
        _arena_lines["n"] += 1
        lines.append(f"[grad hook] {name}: {v:+.8e}")
    for ln in lines:
        printer(ln)
    return lines


def report_arena_gradients(model, limit: Optional[int] = None, printer=print) -> List[str]:
    """Per-parameter gradient sums from the flat gradient arena (``DEBUG_GRAD_HOOK=1`` on CUDA, where gradients are
    accumulated in place by the kernels and autograd hooks do not fire). At most ``limit`` lines over the run."""
    return report_named_gradients(model.named_parameters(), limit, printer)


def report_unit_gradients(unit, limit: Optional[int] = None, printer=print) -> List[str]:
    """The same for one unit of sharded parameters, called when the backward pass leaves the unit: its whole-parameter
    gradients exist only until the reduce-scatter that follows (the reference prints per-parameter sums out of FSDP's
    flat shards at the same point: core/runtime/run_model.py:107-195)."""
    return report_named_gradients(zip(unit.arena.names, unit.arena.params), limit, printer)
