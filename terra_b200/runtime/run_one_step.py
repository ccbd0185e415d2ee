"""Pieces of one training step (reference: core/runtime/run_one_step.py:3-127).

* ``backbone_run`` / ``cal_loss``: ``criterion(model(x) * land_sea_mask, label)``; on CUDA the mask multiply, the
  loss reduction and the loss gradient are one kernel (``fused_forward_loss``).
* ``loss_post_process``: parallel builds divide by the window-parallel size (each rank holds the mean over its own
  stripe) and multiply by ``padding_loss_scale`` (padded area / real area).
* ``grad_post_process``: gradients of replicated parameters are summed over the window-parallel group, those of
  TP shards over the ranks that hold the same shard - here as ONE collective per arena segment instead of one
  per parameter.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops.loss import masked_loss
from ..utils.flat_params import get_arena


def _unwrap(model):
    return model.module if hasattr(model, "module") else model


def criterion_name(loss_fn) -> str:
    if isinstance(loss_fn, str):
        return "L2" if loss_fn in ("L2", "MSE") else "L1"
    if isinstance(loss_fn, torch.nn.MSELoss):
        return "L2"
    return "L1"


def backbone_run(task_type, model, required_tensors, task_specific_data_dict):
    if task_type != "glorys":
        raise ValueError("Unsupported task_type; only glorys is supported")
    out = model(required_tensors["input_tensor"])
    mask = task_specific_data_dict["land_sea_mask"]
    return [out * mask.to(out.dtype)]


def cal_loss(task_type, output_tensor_list, required_tensors, task_specific_data_dict, loss_fn, output_info=None):
    if task_type != "glorys":
        raise ValueError("Unsupported task_type; only glorys is supported")
    out, label = output_tensor_list[0], required_tensors["label_tensor"]
    if callable(loss_fn) and not isinstance(loss_fn, str):
        return loss_fn(out.float(), label.float()).float()
    return masked_loss(out, label.to(out.dtype), None, criterion_name(loss_fn))


def loss_scale_factor(model_type, embedding_parallel_type, manager, task_specific_data_dict, USE_FSDP) -> float:
    scale = 1.0
    if model_type in ("parallel", "hybrid"):
        if embedding_parallel_type in ("window_embedding", "window_linear", None):
            if not USE_FSDP:
                scale /= manager.get_wp_group_size()
        elif embedding_parallel_type == "window_domain":
            scale /= manager.get_mp_group_size() * manager.get_wp_group_size()
        else:
            raise ValueError(f"loss scaling is undefined for embedding_parallel_type={embedding_parallel_type}")
        scale *= float(task_specific_data_dict.get("padding_loss_scale", 1.0))
    return scale


def loss_post_process(loss, model_type, embedding_parallel_type, manager, task_specific_data_dict, USE_FSDP):
    return loss * loss_scale_factor(model_type, embedding_parallel_type, manager, task_specific_data_dict, USE_FSDP)


def fused_forward_loss(task_type, model, required_tensors, task_specific_data_dict, loss_fn, post_scale):
    """Forward + masked loss with the post-processing scale folded in. Returns ``(output, scaled_loss)``."""
    if task_type != "glorys":
        raise ValueError("Unsupported task_type; only glorys is supported")
    out = model(required_tensors["input_tensor"])
    loss = masked_loss(out, required_tensors["label_tensor"], task_specific_data_dict.get("land_sea_mask"),
                       criterion_name(loss_fn), post_scale)
    return out, loss


def grad_post_process(model_type, optimizer_state_tuple, model, manager, dp_average=False):
    """Sum gradients over the ranks that replicate each parameter. With ``dp_average`` the DP replicas are
    included in the same collective and the result is divided by the DP size (the role DDP plays in the
    reference's ``optimizer_config: 4``)."""
    USE_DDP, USE_FSDP, ZERO_STAGE_NUMBER, USE_DIST_OPT = optimizer_state_tuple
    if USE_FSDP or USE_DIST_OPT or manager is None or not (dist.is_available() and dist.is_initialized()):
        return
    real = _unwrap(model)
    parallel = model_type in ("parallel", "hybrid")
    arena = get_arena(real)
    dp = manager.get_dp_group_size()

    def pick(label):
        if label == "xfmr_tp_param_group":
            return manager.xfmr_tp_param_replica_group if dp_average else manager.xfmr_tp_param_group
        if not parallel:
            return manager.data_parallel_group if dp_average else None
        return manager.full_param_replica_group if dp_average else manager.window_parallel_group

    if arena is not None:
        for seg in arena.segments:
            group = pick(seg.label)
            if group is None or dist.get_world_size(group) == 1:
                continue
            dist.all_reduce(arena.grad[seg.start:seg.end], group=group)
            if dp_average and dp > 1:
                arena.grad[seg.start:seg.end].div_(dp)
        return
    for p in real.parameters():
        if p.grad is None:
            continue
        group = pick(getattr(p, "terra_grad_reduce_group", None) or "full")
        if group is None or dist.get_world_size(group) == 1:
            continue
        dist.all_reduce(p.grad, group=group)
        if dp_average and dp > 1:
            p.grad.div_(dp)


def loss_scale_of(gscaler, precision, on_cuda) -> float:
    """Factor folded into the loss gradient on CUDA when ``precision: fp16`` runs with the dynamic loss scaler
    (``terra_b200.optim.grad_scaler.LossScaler``); 1.0 otherwise."""
    if on_cuda and precision == "fp16" and gscaler is not None and hasattr(gscaler, "get_scale") and gscaler.is_enabled():
        return float(gscaler.get_scale())
    return 1.0


def optimizer_step(model, optimizer, gscaler, precision, clip_grad, on_cuda, scale) -> bool:
    """The optimizer step of both training loops (reference: core/runtime/run_model.py:512-514, 571-593): with loss
    scaling, inspect the gradients once (inf / nan flag shared by all ranks, squared norm for the fp16-only clipping at
    max-norm 1.0), fold un-scaling and clipping into the optimizer kernel, skip the step on overflow and update the
    scale; without it, clip (fp16 only) and step. Returns ``True`` when the parameters were updated."""
    if scale != 1.0 or (on_cuda and precision == "fp16" and gscaler is not None and hasattr(gscaler, "inspect")):
        group = dist.group.WORLD if (dist.is_available() and dist.is_initialized()) else None
        if hasattr(optimizer, "gradient_stats"):
            # sharded parameters: the gradients live in the owned slices; the optimizer reports their statistics
            ran = gscaler.step_with_stats(optimizer, *optimizer.gradient_stats(), clip_max_norm=1.0 if clip_grad else None)
        else:
            arena = get_arena(_unwrap(model))
            ran = gscaler.step(optimizer, arena.grad, clip_max_norm=1.0 if clip_grad else None, group=group)
        gscaler.update()
        return ran
    if clip_grad and precision == "fp16":
        if hasattr(optimizer, "clip_grad_norm_"):
            optimizer.clip_grad_norm_(1.0)
        else:
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
    optimizer.step()
    return True
