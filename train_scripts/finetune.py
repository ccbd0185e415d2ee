"""Rollout finetuning loop (reference: train_scripts/finetune.py:60-623).

Starts from pretrained weights (``trained_model_checkpoint_path`` or ``trained_model_config_path`` + ``trained_model_epoch``;
entries are kept by key and shape, ``attn_mask`` buffers are skipped, loading is non-strict), rolls the model out for
``finetune_lead_time`` steps per sample, and checkpoints under ``{train_path}/{description}/lead_{L}/ckpt/...`` by epoch
and, with ``save_interval_steps``, by step (``ckpt_step`` resumes from one).
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from train_scripts.common import FINETUNE_DEFAULTS, Session, base_parser  # noqa: E402
from terra_b200.checkpoint_io import (checkpoint_dir, checkpoint_kind, load_checkpoint, load_pretrained_weights,  # noqa: E402
                                      save_checkpoint)
from terra_b200.config import load_yaml  # noqa: E402
from terra_b200.data.dataloader_utils import resolve_glorys_finetune_double_buffer  # noqa: E402
from terra_b200.optim.utils import get_finetune_lr_by_global_step, set_lr  # noqa: E402
from terra_b200.runtime.finetune_one_step import one_step_finetune  # noqa: E402


def pretrained_path(s: Session):
    c = s.cfg
    if c.get("trained_model_checkpoint_path"):
        return c["trained_model_checkpoint_path"]
    if c.get("trained_model_config_path"):
        src = load_yaml(c["trained_model_config_path"])
        # the epoch to import: this run's key, else the epoch the pretraining config resumes from, else the
        # reference's default of 200 (train_scripts/test_finetune.py:309 there)
        epoch = c.get("trained_model_epoch")
        epoch = src.get("ckpt_epoch", 200) if epoch is None else epoch
        kind = checkpoint_kind(src.get("model_type", s.model_type), s.opt_state)

        class _Rank0:
            """Window-parallel replicas hold identical weights, so rank 0's file serves every rank."""

            def get_rank(self):
                return 0 if c.get("load_pretrained_from_wp_rank0", True) else s.manager.get_rank()

            def get_wp_rank(self):
                return 0 if c.get("load_pretrained_from_wp_rank0", True) else s.manager.get_wp_rank()

        d = checkpoint_dir(src.get("train_path", "./outputs"), src.get("description", "terra_run"), kind, _Rank0())
        return os.path.join(d, f"epoch{epoch}.pth")
    return None


def sequence_to_leads(s: Session, seq_batch, lead_time):
    """``[B, L+1, ...]`` host batch -> list of per-lead ``{'input_tensor', 'label_tensor'}`` (labels double buffered)."""
    if s.model_type == "sequential":
        from terra_b200.data.dataloader_utils import to_nhwc

        seq_batch = to_nhwc(seq_batch, s.archi["num_channels"])
    frames = resolve_glorys_finetune_double_buffer(seq_batch, s.device, s.data_dtype, lead_time,
                                                   enabled=s.cfg.get("input_double_buffer", True),
                                                   non_blocking=s.cfg.get("input_transfer_non_blocking", True))

    class _Leads:
        def __getitem__(self, lead):
            out = {"label_tensor": frames[lead + 1]}
            if lead == 0:
                out["input_tensor"] = frames[0]
            return out

    return _Leads(), frames


def main(argv=None):
    args = base_parser("terra_b200 rollout finetuning").parse_args(argv)
    s = Session(args.model_cfg, args.data_parallel_group_size, FINETUNE_DEFAULTS)
    c = s.cfg
    lead = int(c["finetune_lead_time"])
    path = pretrained_path(s)
    if path is not None and os.path.exists(path):
        load_pretrained_weights(s.model, path, tuple(c.get("skip_pretrained_state_suffixes", ["attn_mask"])),
                                log=print if s.is_log_rank() else None)
    loader = s.finetune_loader(lead, status=0)
    if s.is_log_rank():
        print("[TERRA finetune config]", "description=", c["description"], "task_type=", s.task_type, "model_type=",
              s.model_type, "optimizer_config=", c["optimizer_config"], "precision=", s.precision, "norm_type=",
              c.get("norm_type"), "data_precision=", c.get("data_precision"), "use_splited_data=", c["use_splited_data"],
              "lead_time=", lead, "wp_topo=", c.get("wp_topo"), "xfmr_wp_topo=", c.get("xfmr_wp_topo"), "xfmr_sp_size=",
              c.get("xfmr_sp_size", 1), "tensor_parallel_size=", c.get("tensor_parallel_size", 1), flush=True)
    start_epoch, skip_steps = int(c.get("start_epoch", 0)), 0
    if c.get("ckpt_start", False):
        epoch, gstep, ckpt_loss = load_checkpoint(s.model, s.optimizer, c["train_path"], c["description"], s.model_type,
                                                  s.opt_state, s.manager, epoch=c.get("ckpt_epoch"), step=c.get("ckpt_step"),
                                                  scaler=s.gscaler, lead=lead, model_config=c)
        if c.get("ckpt_step") is not None:
            # a step checkpoint resumes inside its epoch: the steps already taken are skipped, so the sampler's order
            # for that epoch continues where it stopped (reference: train_scripts/finetune.py:259-265, 541-543)
            per_epoch = len(loader)
            if c.get("max_train_steps_per_epoch") is not None:
                per_epoch = min(per_epoch, int(c["max_train_steps_per_epoch"]))
            if per_epoch <= 0:
                raise RuntimeError(f"invalid steps_per_epoch for finetune step resume: {per_epoch}")
            start_epoch, skip_steps = gstep // per_epoch, gstep % per_epoch
        else:
            start_epoch = epoch + 1
        if s.is_log_rank():
            print("resume start_epoch:", start_epoch)
            print("resume skip_steps_in_epoch:", skip_steps)
            print("resume global_step:", gstep)
            print("ckpt loss:", ckpt_loss, flush=True)
    log_file = None
    if s.is_log_rank():
        d = os.path.join(c["train_path"], c["description"], f"lead_{lead}", "loss")
        os.makedirs(d, exist_ok=True)
        log_file = open(os.path.join(d, f"rank{s.rank}.txt"), "a", buffering=1)
    last = None
    for epoch in range(start_epoch, int(c["num_finetune_epochs"])):
        if hasattr(loader.sampler, "set_epoch"):
            loader.sampler.set_epoch(epoch)
        for step, seq in enumerate(loader):
            if epoch == start_epoch and step < skip_steps:
                continue
            limit = c.get("max_train_steps_per_epoch")
            if limit is not None and step >= int(limit):
                break
            lr = get_finetune_lr_by_global_step(s.optimizer.global_step, c["learning_rate"], c["warmup_steps"])
            set_lr(s.optimizer, lr)
            leads, frames = sequence_to_leads(s, seq, lead)
            _, loss, step_time, _ = one_step_finetune(
                s.task_type, s.model_type, s.model, s.engine, s.optimizer, leads, s.task_data, s.other, s.precision,
                c["half_model"], s.my_dtype, s.loss_fn, s.gscaler, s.manager, s.opt_state, lead_time=lead,
                loss_reduction=c["finetune_loss_reduction"], clip_grad=c["clip_grad"], sync_for_timing=False,
                barrier_for_timing=False)
            last = float(loss.item())
            s.guard.after_step(s.optimizer.global_step)      # raises on a lost peer or a timed-out device wait
            if hasattr(frames, "release"):
                frames.release()
            if log_file is not None:
                # the reference's line (train_scripts/finetune.py:588-601: train_gs counts the steps before this one),
                # then this framework's additions
                parts = [c["description"], "epoch", epoch, "finetune step:", step, "loss", last, "lr:", f"{lr:.8f}",
                         "train_gs", s.optimizer.global_step - 1]
                if s.gscaler is not None and hasattr(s.gscaler, "get_scale"):
                    parts += ["scale", s.gscaler.get_scale()]
                parts += ["lead", lead, "step_time_s", f"{step_time:.4f}"]
                print(*parts, flush=True)
                print(*parts, file=log_file)
            every = int(c.get("save_interval_steps") or 0)
            if every > 0 and s.optimizer.global_step % every == 0:
                save_checkpoint(s.model, s.optimizer, last, epoch, c["train_path"], c["description"], s.model_type,
                                s.opt_state, s.manager, s.gscaler, lead=lead, step=s.optimizer.global_step,
                                model_config=c)
        if (epoch + 1) % int(c["save_interval_epochs"]) == 0:
            save_checkpoint(s.model, s.optimizer, last, epoch, c["train_path"], c["description"], s.model_type, s.opt_state,
                            s.manager, s.gscaler, lead=lead, model_config=c)
    if log_file is not None:
        log_file.close()
    s.close()
    return last


if __name__ == "__main__":
    main()
