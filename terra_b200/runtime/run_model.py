"""One optimisation step (reference: core/runtime/run_model.py:362-622).

``one_step_train`` returns ``(output, report_loss, step_time_s, forward_time_s)`` like the reference. Differences
that matter: on CUDA the step time is measured with CUDA events on the launching stream (device time, not host
wall time), forward+loss are fused, and gradient reduction is one collective per parameter class.
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist

from .. import global_env_config as G
from ..profiler.memory_timeline import mark_memory_timeline
from .run_one_step import (backbone_run, cal_loss, fused_forward_loss, grad_post_process, loss_post_process,
                           loss_scale_factor, loss_scale_of, optimizer_step)


def make_global_report_loss(loss, manager, model_type):
    """Loss for logging: summed over the window-parallel group (each rank holds loss / wp), averaged over DP."""
    rep = loss.detach().float().clone()
    if manager is None or not (dist.is_available() and dist.is_initialized()):
        return rep
    if model_type in ("parallel", "hybrid") and manager.get_wp_group_size() > 1:
        dist.all_reduce(rep, group=manager.window_parallel_group)
    if manager.get_dp_group_size() > 1:
        dist.all_reduce(rep, group=manager.data_parallel_group)
        rep /= manager.get_dp_group_size()
    return rep


def _autocast(precision, device_type, enabled):
    dt = {"fp16": torch.float16, "bf16": torch.bfloat16}.get(precision)
    return torch.autocast(device_type=device_type, dtype=dt, enabled=bool(enabled and dt is not None and device_type == "cuda"))


def one_step_train(task_type, model_type, model, engine, optimizer, required_tensors, task_specific_data_dict,
                   other_params, precision, half_model, my_dtype, loss_fn, gscaler, manager=None,
                   optimizer_state_tuple=None, memory_timeline=None, clip_grad=False, sync_for_timing=True,
                   barrier_for_timing=True):
    USE_DDP, USE_FSDP, ZERO_STAGE_NUMBER, USE_DIST_OPT = optimizer_state_tuple or (False, False, -1, False)
    x = required_tensors["input_tensor"]
    on_cuda = x.is_cuda
    live = dist.is_available() and dist.is_initialized()

    if on_cuda and sync_for_timing:
        torch.cuda.synchronize()
    if live and barrier_for_timing:
        dist.barrier()
    t0 = time.time()
    ev0 = ev1 = evf = None
    if on_cuda:
        ev0, evf, ev1 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        ev0.record()

    pctx = getattr(model.module if hasattr(model, "module") else model, "pctx", None)
    for arena_name in ("attn_arena", "tp_arena", "dom_arena"):
        arena = getattr(pctx, arena_name, None)
        if arena is not None:
            arena.reset()      # per-step symmetric buffers of the previous step are dead
    mark_memory_timeline("before_forward")
    post_scale = loss_scale_factor(model_type, other_params.get("embedding_parallel_type") if other_params else None,
                                   manager, task_specific_data_dict, USE_FSDP)
    optimizer.zero_grad()
    scale = loss_scale_of(gscaler, precision, on_cuda)
    if on_cuda:
        # The sm_100a kernels take bf16 activations and fp32 masters directly, so no autocast context is needed and
        # `precision` selects only the loss-scaling behaviour: "bf16" none, "fp16" the dynamic scaler (bf16 arithmetic,
        # GradScaler semantics), "fp32" is refused when the model is built (terra_b200.models.get_model).
        output, loss = fused_forward_loss(task_type, model, required_tensors, task_specific_data_dict, loss_fn,
                                          post_scale * scale)
    else:
        outs = backbone_run(task_type, model, required_tensors, task_specific_data_dict)
        output = outs[0]
        loss = cal_loss(task_type, outs, required_tensors, task_specific_data_dict, loss_fn) * post_scale
    mark_memory_timeline("after_forward")
    t_fwd = time.time() - t0
    if on_cuda:
        evf.record()

    mark_memory_timeline("before_backward")
    if gscaler is not None and precision == "fp16" and not on_cuda:
        gscaler.scale(loss).backward()
    else:
        loss.backward()
    mark_memory_timeline("after_backward")

    grad_post_process(model_type, optimizer_state_tuple or (False, False, -1, False), model, manager,
                      dp_average=not hasattr(model, "module"))
    tsd = task_specific_data_dict or {}
    sharded = getattr(model.module if hasattr(model, "module") else model, "_param_sharder", None) is not None
    if sharded and tsd.get("show_gradient_flag") and not getattr(one_step_train, "_told", False):
        one_step_train._told = True
        print("[grad debug] parameters are sharded: whole-parameter gradients exist only inside the backward pass; "
              "show_gradient_flag is skipped (DEBUG_GRAD_HOOK reports them unit by unit)", flush=True)
    if not sharded and tsd.get("show_gradient_flag") and getattr(optimizer, "global_step", 0) == int(tsd.get("test_iter_num", -1)) - 1:
        from .grad_debug import show_gradient

        show_gradient(model, manager, getattr(manager, "xfmr_tp_group", None) if manager is not None else None)
    if on_cuda and G.DEBUG_GRAD_HOOK and not sharded:
        from .grad_debug import report_arena_gradients

        report_arena_gradients(model)
    mark_memory_timeline("before_optimizer")
    optimizer_step(model, optimizer, gscaler, precision, clip_grad, on_cuda, scale)
    optimizer.global_step += 1
    if scale != 1.0:
        loss = loss.detach() / scale
    mark_memory_timeline("after_optimizer")

    if on_cuda:
        ev1.record()
        if sync_for_timing:
            torch.cuda.synchronize()
    if live and barrier_for_timing:
        dist.barrier()
    if on_cuda and sync_for_timing:
        step_time = ev0.elapsed_time(ev1) * 1e-3
        t_fwd = ev0.elapsed_time(evf) * 1e-3
    else:
        step_time = time.time() - t0
    report_loss = make_global_report_loss(loss, manager, model_type)
    return output, report_loss, step_time, t_fwd


def one_step_train_production(*args, **kwargs):
    """The same step without synchronisation or barriers around it."""
    kwargs["sync_for_timing"] = False
    kwargs["barrier_for_timing"] = False
    return one_step_train(*args, **kwargs)
