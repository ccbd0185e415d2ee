"""Optimizers and LR schedules."""
from .adamw import FusedAdamW
from .distributed_adamw import DistributedAdamW
from .utils import get_finetune_lr_by_global_step, get_lr_by_global_step, get_optimizer, set_lr

__all__ = ["FusedAdamW", "DistributedAdamW", "get_optimizer", "get_lr_by_global_step",
           "get_finetune_lr_by_global_step", "set_lr"]
