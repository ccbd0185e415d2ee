"""Benchmark / correctness harness for rollout finetuning (reference: train_scripts/test_finetune.py:60-1270).

Per step: loss, output sum, peak memory, step time, input-transfer time, offload statistics; ``--memory_timeline_csv``
writes one row per (iteration, lead). Activation plans can change per lead (``activation.lead_checkpoint_schedule`` and
``activation.lead_sampling_checkpoint_schedule``, leads numbered from 1; formats in
``terra_b200/memory/lead_schedule.py``):

    activation:
      lead_checkpoint_schedule:
        "1": []
        "2": ['0-3']
        "3-4": {checkpoint_layers: ['0-7'], mode: cpu_boundary_offload_recompute, offload: {min_numel: 1048576}}
      lead_sampling_checkpoint_schedule:
        "3-4": {down: D1, up: U1}
"""
from __future__ import annotations

import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from train_scripts.common import FINETUNE_DEFAULTS, Session, base_parser  # noqa: E402
from train_scripts.finetune import pretrained_path, sequence_to_leads  # noqa: E402
from train_scripts.metrics import finetune_row, gather_run_facts, write_finetune_metrics  # noqa: E402
from terra_b200 import global_env_config as G  # noqa: E402
from terra_b200.checkpoint_io import load_pretrained_weights  # noqa: E402
from terra_b200.logging_utils import debug_log_wp_ranks, set_dp_rank_print_redirect  # noqa: E402
from terra_b200.profiler.flops_profiler import TorchFlopsProfiler, analytic_step_flops  # noqa: E402
from terra_b200.memory.lead_schedule import LeadScheduler  # noqa: E402
from terra_b200.memory.boundary_offload import get_boundary_offload_stats, reset_boundary_offload_stats  # noqa: E402
from terra_b200.profiler.memory_timeline import (CudaMemoryTimeline, get_memory_timeline_peak_mib,  # noqa: E402
                                                 mark_memory_timeline, set_memory_timeline_context)
from terra_b200.runtime.finetune_one_step import one_step_finetune  # noqa: E402


def make_lead_callback(model, cfg, records, timeline_rows_wanted=False, device=None):
    """Applies the per-lead activation plans before each lead's forward and records one row per lead (the fields of
    the reference's ``--memory_timeline_csv``: train_scripts/test_finetune.py:671-800)."""
    sched = LeadScheduler(model, cfg.get("activation") or {})
    if not (sched.active or timeline_rows_wanted):
        return None, sched

    def callback(event, lead, loss):
        if event == "before_forward":
            set_memory_timeline_context(lead_idx=int(lead) + 1)
            sched.before_lead(lead)
            mark_memory_timeline("rollout_lead_pre", f"lead_{int(lead) + 1}", lead_idx=int(lead) + 1)
        elif event == "after_loss":
            mark_memory_timeline("rollout_lead_post", f"lead_{int(lead) + 1}", lead_idx=int(lead) + 1)
            row = sched.describe(lead)
            on_gpu = device is not None and device.type == "cuda"
            if on_gpu:
                torch.cuda.synchronize(device)
            row.update(allocated_memory_mb=torch.cuda.memory_allocated(device) / 2 ** 20 if on_gpu else 0.0,
                       reserved_memory_mb=torch.cuda.memory_reserved(device) / 2 ** 20 if on_gpu else 0.0,
                       peak_memory_mb=get_memory_timeline_peak_mib(),
                       loss=float(loss.detach().float().item()) if loss is not None else "")
            records.append(row)

    return callback, sched


def main(argv=None):
    ap = base_parser("terra_b200 finetuning test harness")
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--metrics_csv", default=None)
    ap.add_argument("--metrics_json", default=None)
    ap.add_argument("--memory_timeline_csv", default=None)
    ap.add_argument("--metrics_no_json", action="store_true")
    ap.add_argument("--disable_torch_prof", action="store_true")
    ap.add_argument("--quiet_metrics", action="store_true")
    ap.add_argument("--disable_rank_log_redirect", action="store_true")
    ap.add_argument("--mem_prof", type=int, default=None)
    args = ap.parse_args(argv)
    if args.steps is not None and args.steps <= 0:
        raise ValueError(f"--steps must be positive, got {args.steps}")
    steps = args.steps or 2
    # synthetic fields unless the config says otherwise; TERRA_USE_FAKE_INPUT (the reference's switch) sets the default
    fake_default = G.USE_FAKE_INPUT if os.environ.get("TERRA_USE_FAKE_INPUT") else True
    s = Session(args.model_cfg, args.data_parallel_group_size, dict(FINETUNE_DEFAULTS, use_fake_input=fake_default))
    c = s.cfg
    lead = int(c["finetune_lead_time"])
    # data-path switches of the reference harness (train_scripts/test_finetune.py:107-160)
    non_blocking = bool(c.get("input_transfer_non_blocking", True))
    count_transfer = bool(c.get("include_input_transfer_in_step_time", False))
    release_cpu = bool(c.get("release_cpu_batch_after_transfer", False))
    if c.get("input_double_buffer", True) and not non_blocking:
        raise ValueError("input_double_buffer requires input_transfer_non_blocking=true")
    if non_blocking and not c.get("dataloader_pin_memory", True) and s.is_log_rank():
        print("warning: input_transfer_non_blocking=true without dataloader_pin_memory: the copies are synchronous", flush=True)
    if c.get("fake_input_dmp_local", False):
        # the fake datasets here always generate only the rows a rank owns (block-addressable generator), which is
        # what this switch asks for; it keeps the reference's preconditions
        if not c.get("use_fake_input", False):
            raise ValueError("fake_input_dmp_local requires use_fake_input=true")
        if s.model_type not in ("parallel", "hybrid"):
            raise ValueError("fake_input_dmp_local only supports parallel/hybrid GLORYS finetune")
    # start from pretrained weights when the config names them (train_scripts/test_finetune.py:297-315 in the reference)
    weights = pretrained_path(s)
    if weights:
        load_pretrained_weights(s.model, weights, tuple(c.get("skip_pretrained_state_suffixes", ["attn_mask"])),
                                log=print if (s.is_log_rank() and not args.quiet_metrics) else None)
    elif s.is_log_rank() and not args.quiet_metrics:
        print("No trained_model_config_path is provided; finetune starts from current model initialization.", flush=True)
    log_ranks = debug_log_wp_ranks(s.manager, s.model_type, s.other)
    set_dp_rank_print_redirect(s.manager, s.model_type, s.opt_state, s.other.get("embedding_parallel_type"),
                               quiet=args.quiet_metrics, disable=args.disable_rank_log_redirect or s.world == 1,
                               only_wp_ranks=log_ranks)
    if s.manager.get_wp_rank() in log_ranks and not args.quiet_metrics:
        o = s.other
        print("[TERRA parallel config]", "task_type=", s.task_type, "model_architecture=", c.get("model_architecture"),
              "model_type=", s.model_type, "dp_size=", s.dp, "ranks_per_dp=", s.world // max(1, s.dp), "wp_topo=", o["wp_topo"],
              "xfmr_wp_topo=", o["xfmr_wp_topo"], "xfmr_sp_size=", o.get("xfmr_sp_size", 1), "tensor_parallel_size=",
              o.get("tensor_parallel_size", 1), "sp_tp_placement=", o.get("sp_tp_placement", "tp_first"),
              "embedding_parallel_type=", o.get("embedding_parallel_type"), "optimizer_config=", c["optimizer_config"],
              "optimizer_state_tuple=", s.opt_state, flush=True)
    reset_boundary_offload_stats()
    mem_prof = args.mem_prof if args.mem_prof is not None else int(os.environ.get("MEM_PROF", G.MEM_PROF))
    timeline = CudaMemoryTimeline(s.device if s.device.type == "cuda" else None, enabled=mem_prof > 0)
    use_prof = G.ENABLE_TORCH_PROF and not args.disable_torch_prof and not G.DISABLE_TORCH_PROF
    prof = TorchFlopsProfiler(G.TORCH_PROF_STEP_LIST, enabled=use_prof, rank=s.rank,
                              trace_dir="./log/profiler/rank0" if G.TORCH_PROF_WRITE_TRACE else None)
    prof.__enter__()
    analytic_flops = analytic_step_flops(s.archi, c["micro_batch_size"])      # one lead's forward and backward
    loader = s.finetune_loader(lead, status=0)
    rows, lead_rows = [], []
    it = iter(loader)
    for i in range(steps):
        t_load = time.time()
        try:
            seq = next(it)
        except StopIteration:
            it = iter(loader)
            seq = next(it)
        load_time = time.time() - t_load
        leads, frames = sequence_to_leads(s, seq, lead)
        records = []
        cb, _ = make_lead_callback(s.model, c, records, args.memory_timeline_csv is not None, s.device)
        if s.device.type == "cuda":
            torch.cuda.reset_peak_memory_stats(s.device)
        set_memory_timeline_context(iter=i)
        with timeline.iteration(i):
            out, loss, step_time, fwd_time = one_step_finetune(
                s.task_type, s.model_type, s.model, s.engine, s.optimizer, leads, s.task_data, s.other, s.precision,
                c["half_model"], s.my_dtype, s.loss_fn, s.gscaler, s.manager, s.opt_state, lead_time=lead,
                loss_reduction=c["finetune_loss_reduction"], lead_callback=cb, memory_timeline=timeline,
                clip_grad=c["clip_grad"])
        transfer = frames.transfer_time_s() if hasattr(frames, "transfer_time_s") else 0.0
        if count_transfer:
            step_time += transfer
        if release_cpu:
            if hasattr(frames, "release"):
                frames.release()               # pinned source and device slots of the double buffer
            del seq
        out_sum = out.detach().float().sum()
        if dist.is_available() and dist.is_initialized() and s.model_type != "sequential":
            dist.all_reduce(out_sum, group=s.manager.window_parallel_group)
        peak = torch.cuda.max_memory_allocated(s.device) / 2 ** 20 if s.device.type == "cuda" else 0.0
        peak = max(peak, timeline.iteration_peak_allocated_mib)      # peaks the timeline's interval resets folded away
        off = get_boundary_offload_stats()
        rows.append(finetune_row(i, lead, c["finetune_loss_reduction"], float(loss.item()), float(out_sum.item()), out.dtype,
                                 peak, step_time, fwd_time, load_time, local_flops_per_step=analytic_flops * lead,
                                 input_transfer_time_s=transfer, offloaded_tensors=off["offloaded_tensors"],
                                 d2h_bytes=off["d2h_bytes"], h2d_bytes=off["h2d_bytes"]))
        prof.step()
        for r in records:
            lead_rows.append(dict(iter=i, **{k: (str(v) if isinstance(v, list) else v) for k, v in r.items()}))
        if s.is_log_rank() and not args.quiet_metrics:
            print(f"iter {i} loss {rows[-1]['loss']:.8f} peak_memory_mb {peak:.1f} step_time_s {step_time:.4f} "
                  f"offloaded {off['offloaded_tensors']}", flush=True)
    prof.__exit__(None, None, None)
    flops_summary = prof.summarize()                      # collective: every rank
    facts = gather_run_facts(s, rows, get_boundary_offload_stats())
    if s.is_log_rank():
        data_path = dict(fake_input_dmp_local=bool(c.get("fake_input_dmp_local", False)),
                         release_cpu_batch_after_transfer=release_cpu,
                         dataloader_pin_memory=bool(c.get("dataloader_pin_memory", True)),
                         input_transfer_non_blocking=non_blocking,
                         include_input_transfer_in_step_time=count_transfer,
                         input_double_buffer=bool(c.get("input_double_buffer", True)))
        write_finetune_metrics(s, args, rows, lead_rows, facts, flops_summary, lead, c["finetune_loss_reduction"],
                               data_path, extra=dict(
                                   description=c.get("description"), offload=get_boundary_offload_stats(),
                                   final_loss=rows[-1]["loss"], analytic_flops_per_step=analytic_flops * lead,
                                   recompute=s.model.recompute_scheduler.summary()))
        if mem_prof > 0 and timeline.events:
            timeline.write_outputs(os.environ.get("MEMORY_TIMELINE_OUTPUT_DIR", "./log/memory_timeline"), "finetune_rank0")
        if not args.quiet_metrics:
            # the closing report of the reference's harness (train_scripts/test_finetune.py:1240-1267)
            print("all_parameters", facts["parameter_count"]["post_wrap_local_parameter_counts_by_rank"])
            print("all_mem_peak_last", facts["peak_memory_last_by_rank"])
            print("all_time_peak", facts["step_time_last_by_rank"])
            if flops_summary.enabled:
                prof.print_top_ops(20)
                print("local_FLOPs_per_step", flops_summary.local_flops_per_step)
                print("world_FLOPs_per_step", flops_summary.world_flops_per_step)
                print("world_avg_FLOPs_per_step", flops_summary.world_avg_flops_per_step)
            per_step = flops_summary.local_flops_per_step if flops_summary.enabled else analytic_flops * lead / max(1, s.world // max(1, s.dp))
            print("-----------------------------Accuracy------------------------------")
            for r in rows:
                print("iter", r["iter"], r["output_dtype"], "sum:", r["output_sum"], "loss", r["loss"])
            print("-----------------------------Per-step memory------------------------------")
            for r in rows:
                print("iter", r["iter"], "peak_memory", r["peak_memory_mb"])
            print("-----------------------------Per-step time and FLOPS------------------------------")
            for r in rows:
                print("iter", r["iter"], f"Total Time  : {r['step_time_s'] * 1000:.3f} ms",
                      f"FLOPS : {per_step / r['step_time_s'] / 1e12:.3f} TFLOPS",
                      f"forward Time  : {(r['forward_time_s'] or 0.0) * 1000:.3f} ms",
                      f"load data time {(r['load_data_time_s'] or 0.0) * 1000:.3f} ms")
            print("-----------------------------Per-step time break down------------------------------")
            for r in rows:
                fwd = r["forward_time_s"] or 0.0
                print("iter", r["iter"], f"Total Time  : {r['step_time_s'] * 1000:.3f} ms", f"forward Time  : {fwd * 1000:.3f} ms",
                      f"Rest Time  : {(r['step_time_s'] - fwd) * 1000:.3f} ms", flush=True)
    s.close()
    return rows


if __name__ == "__main__":
    main()
