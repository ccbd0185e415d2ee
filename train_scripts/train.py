"""Production pretraining loop (CLI and files as in the reference's train_scripts/train.py:40-592).

    torchrun --nproc-per-node N train_scripts/train.py --data_parallel_group_size D --model_cfg X.yaml

Per step: LR schedule (linear warm-up, cosine decay) -> batch to this rank's layout -> one optimisation step -> rank-0
log line in ``{train_path}/{description}/loss/rank0.txt``. Checkpoints every ``save_interval_epochs`` under
``{train_path}/{description}/ckpt/...``; ``ckpt_start: True`` + ``ckpt_epoch`` resumes.
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from train_scripts.common import PRETRAIN_DEFAULTS, Session, base_parser  # noqa: E402
from terra_b200.checkpoint_io import load_checkpoint, save_checkpoint  # noqa: E402
from terra_b200.optim.utils import get_lr_by_global_step, set_lr  # noqa: E402
from terra_b200.runtime.run_model import one_step_train_production  # noqa: E402


def main(argv=None):
    args = base_parser("terra_b200 pretraining").parse_args(argv)
    s = Session(args.model_cfg, args.data_parallel_group_size, PRETRAIN_DEFAULTS)
    c = s.cfg
    if s.is_log_rank():
        use_ddp, use_fsdp, zero_stage, use_dist_opt = s.opt_state
        print("training description:", c["description"])
        print("task/model:", s.task_type, c.get("model_architecture"), s.model_type)
        print("optimizer_config:", c["optimizer_config"], "DDP/FSDP/Zero/DistOpt:", use_ddp, use_fsdp, zero_stage, use_dist_opt)
        print("parallel:", "wp_topo=", s.other.get("wp_topo"), "xfmr_wp_topo=", s.other.get("xfmr_wp_topo"), "sp=",
              s.other.get("xfmr_sp_size"), "tp=", s.other.get("tensor_parallel_size"), flush=True)
    loader = s.pretrain_loader(status=0)
    start_epoch = int(c.get("start_epoch", 0))
    if c.get("ckpt_start", False):
        epoch, gstep, ckpt_loss = load_checkpoint(s.model, s.optimizer, c["train_path"], c["description"], s.model_type,
                                                  s.opt_state, s.manager, epoch=c["ckpt_epoch"], scaler=s.gscaler,
                                                  model_config=c)
        start_epoch = epoch + 1
        if s.is_log_rank():
            print("resumed epoch:", start_epoch)
            print("resumed global_step:", gstep)
            print("resumed loss:", ckpt_loss, flush=True)
    log_file = None
    if s.is_log_rank():
        d = os.path.join(c["train_path"], c["description"], "loss")
        os.makedirs(d, exist_ok=True)
        log_file = open(os.path.join(d, "rank0.txt"), "a", buffering=1)
    last_loss = None
    for epoch in range(start_epoch, int(c["num_pre_train_epochs"])):
        if hasattr(loader.sampler, "set_epoch"):
            loader.sampler.set_epoch(epoch)
        for step, batch in enumerate(loader):
            limit = c.get("max_train_steps_per_epoch")
            if limit is not None and step >= int(limit):
                break
            lr = get_lr_by_global_step(s.task_type, s.optimizer.global_step, c["learning_rate"], c["warmup_steps"],
                                       c["num_pre_train_epochs"])
            set_lr(s.optimizer, lr)
            tensors = s.to_required_tensors(batch)
            _, loss, step_time, fwd_time = one_step_train_production(
                s.task_type, s.model_type, s.model, s.engine, s.optimizer, tensors, s.task_data, s.other, s.precision,
                c["half_model"], s.my_dtype, s.loss_fn, s.gscaler, s.manager, s.opt_state, clip_grad=c["clip_grad"])
            last_loss = float(loss.item())
            s.guard.after_step(s.optimizer.global_step)      # raises on a lost peer or a timed-out device wait
            if log_file is not None:
                # the reference's line (train_scripts/train.py:552-571), on stdout and appended to loss/rank0.txt
                parts = [c["description"], "epoch", epoch, "train step:", step, "loss", last_loss, "lr:", f"{lr:.8f}",
                         "train_gs", s.optimizer.global_step, "step_time_s", f"{step_time:.4f}", "forward_time_s",
                         f"{fwd_time:.4f}"]
                if s.gscaler is not None and hasattr(s.gscaler, "get_scale"):
                    parts += ["scale", s.gscaler.get_scale()]
                print(*parts, flush=True)
                print(*parts, file=log_file)
        if (epoch + 1) % int(c["save_interval_epochs"]) == 0:
            path = save_checkpoint(s.model, s.optimizer, last_loss, epoch, c["train_path"], c["description"], s.model_type,
                                   s.opt_state, s.manager, s.gscaler, model_config=c)
            if path is not None and s.is_log_rank():
                print(f"saved checkpoint: {path}", flush=True)
    if log_file is not None:
        log_file.close()
    s.close()
    return last_loss


if __name__ == "__main__":
    main()
