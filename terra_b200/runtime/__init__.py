"""Step runtime: forward / loss / backward / gradient reduction / optimizer step, pretrain and rollout finetune."""
from .run_model import one_step_train, one_step_train_production, make_global_report_loss
from .run_one_step import backbone_run, cal_loss, grad_post_process, loss_post_process

__all__ = ["one_step_train", "one_step_train_production", "make_global_report_loss", "backbone_run", "cal_loss",
           "grad_post_process", "loss_post_process"]
