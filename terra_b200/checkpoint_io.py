"""Checkpoint files (reference layout: train_scripts/train.py:56-280, finetune.py:60-318).

``{train_path}/{description}/ckpt/<kind dir>/epoch{E}.pth`` (pretrain) and
``{train_path}/{description}/lead_{L}/ckpt/<kind dir>/{epoch{E}|step{N}}.pth`` (finetune), each holding
``model_state_dict, optimizer_state_dict, loss, epoch, global_step, ckpt_layout`` (+ ``scaler``).

Who writes what (``ckpt_layout``):
  ``single``      sequential build: rank 0 writes ``ckpt/``
  ``wp_rank``     parallel build with a replicated optimizer: the ranks of DP replica 0 write ``ckpt/wp_rank_{w}/``
  ``rank_local``  sharded optimizer: every rank writes ``ckpt/rank_{r}/`` (optimizer state exists only on its owner)
  ``fsdp_full``   ``optimizer_config`` 5 / 7 / 8 / 9 (the reference's FSDP configurations) with ``fsdp_checkpoint_type:
                  full`` (the default): rank 0 writes ``ckpt/`` with the whole model and the optimizer state gathered
                  into ``torch.optim.AdamW``'s per-parameter layout, so the file loads into any layout
  ``fsdp_sharded``  the same configurations with ``fsdp_checkpoint_type: sharded``: every rank writes
                  ``ckpt/fsdp_sharded/rank_{r}/`` with only what it owns - its contiguous ranges of the fp32 masters and
                  of the two moments; loading puts the ranges back together over the replica groups
(reference: train_scripts/train.py:60-84, 130-213).
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist


FSDP_OPTIMIZER_CONFIGS = (5, 7, 8, 9)


def checkpoint_kind(model_type: str, optimizer_state_tuple, model_config=None) -> str:
    use_ddp, use_fsdp, zero_stage, use_dist_opt = optimizer_state_tuple
    if model_config is not None and use_dist_opt and int(model_config.get("optimizer_config", -1)) in FSDP_OPTIMIZER_CONFIGS:
        kind = str(model_config.get("fsdp_checkpoint_type", "full"))
        if kind not in ("full", "sharded"):
            raise ValueError(f"fsdp_checkpoint_type must be 'full' or 'sharded', got {kind!r}")
        return "fsdp_" + kind
    if use_dist_opt:
        return "rank_local"
    if model_type in ("parallel", "hybrid"):
        return "wp_rank"
    return "single"


def checkpoint_dir(train_path, description, kind, manager, lead: Optional[int] = None) -> str:
    base = os.path.join(train_path, description)
    if lead is not None:
        base = os.path.join(base, f"lead_{lead}")
    base = os.path.join(base, "ckpt")
    if kind == "fsdp_sharded":
        return os.path.join(base, "fsdp_sharded", f"rank_{manager.get_rank()}")
    if kind == "rank_local":
        return os.path.join(base, f"rank_{manager.get_rank()}")
    if kind == "wp_rank":
        return os.path.join(base, f"wp_rank_{manager.get_wp_rank()}")
    return base


def should_write(kind, manager) -> bool:
    if kind in ("rank_local", "fsdp_sharded"):
        return True
    if kind == "wp_rank":
        return manager.get_dp_rank() == 0
    return manager.get_rank() == 0


def strip_module_prefix(state_dict):
    return {(k[len("module."):] if k.startswith("module.") else k): v for k, v in state_dict.items()}


def _non_parameters(real):
    names = {n for n, _ in real.named_parameters()}
    return {k: v.detach().cpu() for k, v in real.state_dict().items() if k not in names}


def _owned_ranges(real, optimizer):
    """This rank's contiguous ranges of the flat fp32 masters (one per optimizer shard), and everything in the state
    dict that is not a parameter (buffers such as the relative-position index)."""
    sharder = getattr(real, "_param_sharder", None)
    if sharder is not None:
        # sharded parameters: the owned slices are all a rank holds; ranges are positions within their unit's arena
        ranges = [dict(unit=u.name, label=r.label, rank=r.rank, size=r.size, start=r.start, end=r.end, lo=r.lo, hi=r.hi,
                       master=r.own_master.detach().cpu().clone()) for u in sharder.all_units() for r in u.ranges]
        return {"__flat_ranges__": ranges, "__numel__": int(sharder.total_numel()), "__non_parameters__": _non_parameters(real)}
    arena = real._param_arena
    names = {id(p): n for n, p in real.named_parameters()}
    param_keys = {names[id(p)] for p in arena.params if id(p) in names}
    ranges = [dict(label=sh.label, rank=sh.rank, size=sh.size, start=sh.start, end=sh.end, lo=sh.lo, hi=sh.hi,
                   master=arena.master[sh.lo:sh.hi].detach().cpu().clone()) for sh in optimizer.shards]
    extra = {k: v.detach().cpu() for k, v in real.state_dict().items() if k not in param_keys}
    return {"__flat_ranges__": ranges, "__numel__": int(arena.numel), "__non_parameters__": extra}


def _restore_owned_ranges(real, optimizer, saved):
    """Inverse of ``_owned_ranges``: own ranges from the file, the rest from their owners (every element of a shard's
    segment has exactly one owner in the shard's group, so a sum over the group puts the pieces together)."""
    sharder = getattr(real, "_param_sharder", None)
    if sharder is not None:
        if int(saved["__numel__"]) != int(sharder.total_numel()):
            raise ValueError("sharded checkpoint was written for a model with a different parameter count")
        mine = [(u, r) for u in sharder.all_units() for r in u.ranges]
        if len(mine) != len(saved["__flat_ranges__"]):
            raise ValueError("sharded checkpoint was written for a different unit layout")
        for (u, r), rg in zip(mine, saved["__flat_ranges__"]):
            if (rg.get("unit"), rg["label"], rg["rank"], rg["size"], rg["lo"], rg["hi"]) != (u.name, r.label, r.rank, r.size, r.lo, r.hi):
                raise ValueError("sharded checkpoint was written for a different layout (use fsdp_checkpoint_type: full "
                                 "to move between layouts)")
            with torch.no_grad():
                r.own_master.copy_(rg["master"])
                if r.own_work is not None:
                    r.own_work.copy_(r.own_master)
        if saved["__non_parameters__"]:
            real.load_state_dict(saved["__non_parameters__"], strict=False)
        return
    arena = real._param_arena
    if int(saved["__numel__"]) != int(arena.numel):
        raise ValueError("sharded checkpoint was written for a model with a different parameter count")
    for sh, rg in zip(optimizer.shards, saved["__flat_ranges__"]):
        if (rg["label"], rg["rank"], rg["size"], rg["lo"], rg["hi"]) != (sh.label, sh.rank, sh.size, sh.lo, sh.hi):
            raise ValueError("sharded checkpoint was written for a different layout (use fsdp_checkpoint_type: full "
                             "to move between layouts)")
        with torch.no_grad():
            seg = arena.master[sh.start:sh.end]
            if sh.size > 1:
                seg.zero_()
            arena.master[sh.lo:sh.hi] = rg["master"].to(arena.master.device)
            if sh.size > 1:
                dist.all_reduce(seg, group=sh.group)
    if saved["__non_parameters__"]:
        real.load_state_dict(saved["__non_parameters__"], strict=False)


def save_checkpoint(model, optimizer, loss, epoch, train_path, description, model_type, optimizer_state_tuple, manager,
                    scaler=None, lead=None, step=None, model_config=None) -> Optional[str]:
    kind = checkpoint_kind(model_type, optimizer_state_tuple, model_config)
    path = None
    if hasattr(optimizer, "sync_masters"):
        optimizer.sync_masters()
    real = model.module if hasattr(model, "module") else model
    sharder = getattr(real, "_param_sharder", None)
    # the gathered optimizer state is a collective: every rank takes part, rank 0 writes
    opt_state = optimizer.full_state_dict() if kind == "fsdp_full" else None
    # so is the gathered model of sharded parameters (every kind but the per-rank one stores whole tensors)
    full_model = sharder.full_state_dict() if (sharder is not None and kind != "fsdp_sharded") else None
    if should_write(kind, manager):
        d = checkpoint_dir(train_path, description, kind, manager, lead)
        os.makedirs(d, exist_ok=True)
        name = f"step{step}.pth" if step is not None else f"epoch{epoch}.pth"
        path = os.path.join(d, name)
        if kind == "fsdp_sharded":
            model_state = _owned_ranges(real, optimizer)
        elif full_model is not None:
            model_state = full_model
        else:
            model_state = {k: v.detach().cpu() for k, v in real.state_dict().items()}
        blob = {"model_state_dict": model_state,
                "optimizer_state_dict": opt_state if opt_state is not None else optimizer.state_dict(),
                "loss": float(loss) if loss is not None else None,
                "epoch": epoch, "global_step": int(getattr(optimizer, "global_step", 0)), "ckpt_layout": kind}
        if scaler is not None:
            blob["scaler"] = scaler.state_dict()
        torch.save(blob, path + ".tmp")
        os.replace(path + ".tmp", path)
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    return path


def load_checkpoint(model, optimizer, train_path, description, model_type, optimizer_state_tuple, manager, epoch=None,
                    step=None, scaler=None, lead=None, strict=True, model_config=None):
    """Returns ``(epoch, global_step, loss)`` of the loaded file."""
    kind = checkpoint_kind(model_type, optimizer_state_tuple, model_config)
    d = checkpoint_dir(train_path, description, kind, manager, lead)
    if kind == "wp_rank" and not os.path.isdir(d):
        d = checkpoint_dir(train_path, description, "single", manager, lead)
    name = f"step{step}.pth" if step is not None else f"epoch{epoch}.pth"
    blob = torch.load(os.path.join(d, name), map_location="cpu", weights_only=False)
    real = model.module if hasattr(model, "module") else model
    if kind == "fsdp_sharded":
        _restore_owned_ranges(real, optimizer, blob["model_state_dict"])
    elif getattr(real, "_param_sharder", None) is not None:
        real._param_sharder.load_full_state_dict(strip_module_prefix(blob["model_state_dict"]), strict=strict)
    else:
        real.load_state_dict(strip_module_prefix(blob["model_state_dict"]), strict=strict)
    arena = getattr(real, "_param_arena", None)
    if arena is not None:
        arena.sync_bf16()
    if optimizer is not None and blob.get("optimizer_state_dict") is not None:
        optimizer.load_state_dict(blob["optimizer_state_dict"])
        optimizer.global_step = int(blob.get("global_step", 0))
    if scaler is not None and "scaler" in blob:
        scaler.load_state_dict(blob["scaler"])
    return int(blob.get("epoch", 0)), int(blob.get("global_step", 0)), blob.get("loss")


def load_pretrained_weights(model, path, skip_suffixes=("attn_mask",), log=print):
    """Finetune import: keep the entries whose key exists with the same shape, drop the listed suffixes, load
    non-strictly (train_scripts/finetune.py:86-216)."""
    blob = torch.load(path, map_location="cpu", weights_only=False)
    sd = strip_module_prefix(blob.get("model_state_dict", blob) if isinstance(blob, dict) else blob)
    real = model.module if hasattr(model, "module") else model
    own = real.state_dict()
    keep, dropped = {}, []
    for k, v in sd.items():
        if any(k.endswith(s) for s in skip_suffixes):
            continue
        if k in own and tuple(own[k].shape) == tuple(v.shape):
            keep[k] = v
        else:
            dropped.append(k)
    missing = [k for k in own if k not in keep]
    if getattr(real, "_param_sharder", None) is not None:
        real._param_sharder.load_full_state_dict(keep, strict=False)      # collective: every rank loads the same file
    else:
        real.load_state_dict(keep, strict=False)
    arena = getattr(real, "_param_arena", None)
    if arena is not None:
        arena.sync_bf16()
    if log is not None:
        log(f"[pretrained] loaded {len(keep)} tensors, skipped {len(dropped)} (key/shape mismatch), {len(missing)} left at init")
    return keep.keys(), dropped, missing
