"""Autoregressive rollout finetuning (reference: core/runtime/finetune_one_step.py:15-233, run_model.py:625-862).

For ``lead_time`` steps the masked output of one step is the input of the next, with the graph kept; the per-lead
losses are summed and (``loss_reduction='mean'``) divided by the number of leads. ``lead_callback(event, lead, loss)``
fires ``"before_forward"`` and ``"after_loss"`` so that a harness can switch activation-checkpoint plans per lead.
``required_tensors`` is indexable by lead (a list of dicts or a double buffer of label frames).
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist

from ..ops.loss import masked_loss
from ..profiler.memory_timeline import mark_memory_timeline, set_memory_timeline_context
from .run_model import make_global_report_loss
from .run_one_step import criterion_name, grad_post_process, loss_scale_factor, loss_scale_of, optimizer_step


def _lead_scale(lead_time, loss_reduction):
    if loss_reduction == "sum":
        return 1.0
    if loss_reduction == "mean":
        return 1.0 / max(1, int(lead_time))
    raise ValueError(f"unsupported finetune_loss_reduction: {loss_reduction}")


def finetune_run(task_type, model, required_tensors, task_specific_data_dict, loss_fn, lead_time=1, loss_reduction="mean",
                 lead_callback=None, post_scale=1.0):
    """Returns ``([last_output], total_loss)``; ``total_loss`` already carries ``post_scale`` and the reduction."""
    if task_type != "glorys":
        raise ValueError("Unsupported task_type; only glorys is supported")
    mask = task_specific_data_dict["land_sea_mask"]
    scale = post_scale * _lead_scale(lead_time, loss_reduction)
    total, cur_input, cur_output = None, None, None
    for lead in range(lead_time):
        cur = required_tensors[lead]
        set_memory_timeline_context(lead_idx=lead)
        if lead_callback is not None:
            lead_callback("before_forward", lead, None)
        if lead == 0:
            cur_input = cur["input_tensor"]
        cur_output = model(cur_input)
        cur_output = cur_output * mask.to(cur_output.dtype)
        if callable(loss_fn) and not isinstance(loss_fn, (str, torch.nn.L1Loss, torch.nn.MSELoss)):
            cur_loss = loss_fn(cur_output.float(), cur["label_tensor"].float()).float() * scale
        else:
            cur_loss = masked_loss(cur_output, cur["label_tensor"].to(cur_output.dtype), None, criterion_name(loss_fn), scale)
        total = cur_loss if total is None else total + cur_loss
        if lead_callback is not None:
            lead_callback("after_loss", lead, cur_loss)
        cur_input = cur_output
    if total is None:
        raise RuntimeError("finetune loss is None; check lead_time and required_tensors")
    return [cur_output], total


funetune_run = finetune_run   # historical spelling kept as an alias


def run_one_step_for_finetune_train(task_type, model_type, model, optimizer, engine, gscaler, precision, my_dtype,
                                    required_tensors, task_specific_data_dict, other_params, loss_fn, manager,
                                    optimizer_state_tuple, lead_time=1, loss_reduction="mean", lead_callback=None,
                                    clip_grad=False):
    USE_DDP, USE_FSDP, ZERO_STAGE_NUMBER, USE_DIST_OPT = optimizer_state_tuple
    post = loss_scale_factor(model_type, (other_params or {}).get("embedding_parallel_type"), manager,
                             task_specific_data_dict, USE_FSDP)
    optimizer.zero_grad()
    mark_memory_timeline("before_forward")
    on_cuda = next(model.parameters()).is_cuda
    scale = loss_scale_of(gscaler, precision, on_cuda)
    outs, loss = finetune_run(task_type, model, required_tensors, task_specific_data_dict, loss_fn, lead_time,
                              loss_reduction, lead_callback, post * scale)
    mark_memory_timeline("after_forward")
    set_memory_timeline_context(execution_phase="backward")
    mark_memory_timeline("before_backward")
    loss.backward()
    mark_memory_timeline("after_backward")
    grad_post_process(model_type, optimizer_state_tuple, model, manager, dp_average=not hasattr(model, "module"))
    optimizer_step(model, optimizer, gscaler, precision, clip_grad, on_cuda, scale)
    optimizer.global_step += 1
    mark_memory_timeline("after_optimizer")
    return outs[0], (loss.detach() / scale if scale != 1.0 else loss)


@torch.no_grad()
def run_one_step_for_finetune_eval(task_type, model_type, model, precision, my_dtype, required_tensors,
                                   task_specific_data_dict, other_params, loss_fn, manager, optimizer_state_tuple,
                                   lead_time=1, loss_reduction="mean"):
    USE_FSDP = optimizer_state_tuple[1]
    post = loss_scale_factor(model_type, (other_params or {}).get("embedding_parallel_type"), manager,
                             task_specific_data_dict, USE_FSDP)
    outs, loss = finetune_run(task_type, model, required_tensors, task_specific_data_dict, loss_fn, lead_time,
                              loss_reduction, None, post)
    return outs[0], loss


def one_step_finetune(task_type, model_type, model, engine, optimizer, required_tensors, task_specific_data_dict,
                      other_params, precision, half_model, my_dtype, loss_fn, gscaler, manager=None,
                      optimizer_state_tuple=None, lead_time=1, loss_reduction="mean", lead_callback=None,
                      memory_timeline=None, clip_grad=False, sync_for_timing=True, barrier_for_timing=True):
    """Timed rollout step: ``(output, report_loss, step_time_s, forward_time_s)``."""
    on_cuda = torch.cuda.is_available() and next(model.parameters()).is_cuda
    live = dist.is_available() and dist.is_initialized()
    if on_cuda and sync_for_timing:
        torch.cuda.synchronize()
    if live and barrier_for_timing:
        dist.barrier()
    t0 = time.time()
    ev0 = ev1 = None
    if on_cuda:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
    out, loss = run_one_step_for_finetune_train(task_type, model_type, model, optimizer, engine, gscaler, precision,
                                                my_dtype, required_tensors, task_specific_data_dict, other_params, loss_fn,
                                                manager, optimizer_state_tuple or (False, False, -1, False), lead_time,
                                                loss_reduction, lead_callback, clip_grad)
    if on_cuda:
        ev1.record()
        if sync_for_timing:
            torch.cuda.synchronize()
    if live and barrier_for_timing:
        dist.barrier()
    step_time = ev0.elapsed_time(ev1) * 1e-3 if (on_cuda and sync_for_timing) else time.time() - t0
    return out, make_global_report_loss(loss, manager, model_type), step_time, 0.0
