"""Optimizer factory and learning-rate schedules (reference: optimizer/utils.py:8-123)."""
from __future__ import annotations

import math

STEPS_PER_EPOCH = 594   # the reference's cosine schedule assumes this many steps per epoch (optimizer/utils.py:104)


def get_optimizer(model, model_config, manager=None, use_dist_opt=None):
    """AdamW(betas=(0.9, 0.95), weight_decay=0.1) at the YAML learning rate; ``optimizer_config == 6`` selects the
    sharded ``DistributedAdamW``. The returned optimizer carries ``global_step = 0``."""
    from .adamw import FusedAdamW
    from .distributed_adamw import DistributedAdamW

    lr = float(model_config.get("learning_rate", 1e-4))
    if use_dist_opt is None:
        use_dist_opt = int(model_config.get("optimizer_config", 4)) == 6
    if use_dist_opt:
        opt = DistributedAdamW(model.parameters(), lr=lr, betas=(0.9, 0.95), weight_decay=0.1, manager=manager, model=model)
    else:
        opt = FusedAdamW(model.parameters(), lr=lr, betas=(0.9, 0.95), weight_decay=0.1, model=model)
    opt.global_step = 0
    return opt


def get_lr_by_global_step(task_type, step, base_lr, warmup_steps, num_pre_train_epochs=None, min_lr=1e-6,
                          steps_per_epoch=STEPS_PER_EPOCH):
    """Linear warm-up ``base_lr * step / warmup``, then cosine decay to ``min_lr`` over
    ``num_pre_train_epochs * steps_per_epoch`` steps."""
    if task_type != "glorys":
        raise ValueError(f"Unsupported task_type: {task_type}; only GLORYS reference workload is available")
    if step < warmup_steps:
        return base_lr * step / max(1, warmup_steps)
    total = num_pre_train_epochs * steps_per_epoch
    progress = (step - warmup_steps) / (total - warmup_steps)
    return min_lr + (base_lr - min_lr) * 0.5 * (1.0 + math.cos(math.pi * progress))


def get_finetune_lr_by_global_step(step, base_lr, warmup_steps):
    """Linear warm-up, then constant."""
    if step < warmup_steps:
        return base_lr * step / max(1, warmup_steps)
    return base_lr


def set_lr(optimizer, lr):
    for group in optimizer.param_groups:
        group["lr"] = lr
