"""Benchmark / correctness harness for pretraining (reference: train_scripts/test_pretrain.py:61-699).

Runs ``--steps`` optimisation steps and records, per step, the loss, the output sum, the peak memory and the step time
(``--metrics_csv``), plus run metadata, parameter counts and FLOPs (``--metrics_json``). ``MEM_PROF`` = 1 / 2 turns
the memory timeline on (2 adds the per-primitive summary).
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from train_scripts.common import PRETRAIN_DEFAULTS, Session, base_parser  # noqa: E402
from train_scripts.metrics import gather_run_facts, write_pretrain_metrics  # noqa: E402
from terra_b200 import global_env_config as G  # noqa: E402
from terra_b200.logging_utils import debug_log_wp_ranks, set_dp_rank_print_redirect  # noqa: E402
from terra_b200.memory.boundary_offload import get_boundary_offload_stats, reset_boundary_offload_stats  # noqa: E402
from terra_b200.profiler.flops_profiler import TorchFlopsProfiler, analytic_step_flops  # noqa: E402
from terra_b200.profiler.memory_timeline import CudaMemoryTimeline  # noqa: E402
from terra_b200.runtime.run_model import one_step_train  # noqa: E402
from terra_b200.utils.misc import count_parameters  # noqa: E402


def main(argv=None):
    ap = base_parser("terra_b200 pretraining test harness")
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--metrics_csv", default=None)
    ap.add_argument("--metrics_json", default=None)
    ap.add_argument("--metrics_no_json", action="store_true")
    ap.add_argument("--disable_torch_prof", action="store_true")
    ap.add_argument("--quiet_metrics", action="store_true")
    ap.add_argument("--disable_rank_log_redirect", action="store_true")
    ap.add_argument("--mem_prof", type=int, default=None)
    args = ap.parse_args(argv)
    if args.steps is not None and args.steps <= 0:
        raise ValueError(f"--steps must be positive, got {args.steps}")
    steps = args.steps or 4

    # synthetic fields unless the config says otherwise; TERRA_USE_FAKE_INPUT (the reference's switch) sets the default
    fake_default = G.USE_FAKE_INPUT if os.environ.get("TERRA_USE_FAKE_INPUT") else True
    s = Session(args.model_cfg, args.data_parallel_group_size, dict(PRETRAIN_DEFAULTS, use_fake_input=fake_default))
    c = s.cfg
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
    loader = s.pretrain_loader(status=0)
    rows = []
    it = iter(loader)
    with prof:
        for i in range(steps):
            try:
                batch = next(it)
            except StopIteration:
                it = iter(loader)
                batch = next(it)
            tensors = s.to_required_tensors(batch)
            if s.device.type == "cuda":
                torch.cuda.reset_peak_memory_stats(s.device)
            with timeline.iteration(i):
                out, loss, step_time, fwd_time = one_step_train(
                    s.task_type, s.model_type, s.model, s.engine, s.optimizer, tensors, s.task_data, s.other, s.precision,
                    c["half_model"], s.my_dtype, s.loss_fn, s.gscaler, s.manager, s.opt_state, memory_timeline=timeline,
                    clip_grad=c["clip_grad"])
            prof.step()
            out_sum = out.detach().float().sum()
            if dist.is_available() and dist.is_initialized() and s.model_type != "sequential":
                dist.all_reduce(out_sum, group=s.manager.window_parallel_group)
            peak = torch.cuda.max_memory_allocated(s.device) / 2 ** 20 if s.device.type == "cuda" else 0.0
            peak = max(peak, timeline.iteration_peak_allocated_mib)      # peaks the timeline's interval resets folded away
            rows.append(dict(iter=i, loss=float(loss.item()), output_sum=float(out_sum.item()), output_dtype=str(out.dtype),
                             peak_memory_mb=peak, step_time_s=step_time, forward_time_s=fwd_time))
            if s.is_log_rank() and not args.quiet_metrics:
                print(f"iter {i} loss {rows[-1]['loss']:.8f} output_sum {rows[-1]['output_sum']:.6f} "
                      f"peak_memory_mb {peak:.1f} step_time_s {step_time:.4f}", flush=True)
    flops_summary = prof.summarize()                      # collective: every rank
    facts = gather_run_facts(s, rows)
    if s.is_log_rank():
        flops = analytic_step_flops(s.archi, c["micro_batch_size"])
        times = [r["step_time_s"] for r in rows[1:]] or [rows[0]["step_time_s"]]
        avg = sum(times) / len(times)
        total, trainable = count_parameters(s.model)
        write_pretrain_metrics(s, args, rows, facts, flops_summary, extra=dict(
            description=c.get("description"), parameters=total, trainable_parameters=trainable,
            analytic_flops_per_step=flops, avg_step_time_s=avg, tflops=flops / avg / 1e12,
            offload=get_boundary_offload_stats(), final_loss=rows[-1]["loss"]))
        if mem_prof > 0 and timeline.events:
            # CSV, summary, event table and plot as the MEMORY_TIMELINE_WRITE_* switches ask
            timeline.write_outputs(os.environ.get("MEMORY_TIMELINE_OUTPUT_DIR", "./log/memory_timeline"), "rank0")
        if not args.quiet_metrics:
            # the closing report of the reference's harness (train_scripts/test_pretrain.py:671-696)
            counts = facts["parameter_count"]
            print("all_parameters", counts["post_wrap_local_parameter_counts_by_rank"])
            print("all_pre_wrap_parameters", counts["pre_wrap_parameter_counts_by_rank"])
            print("parameter_count_summary", counts)
            print("all_mem_peak_last", facts["peak_memory_last_by_rank"])
            print("all_time_peak", facts["step_time_last_by_rank"])
            # the profiler's count where it ran; the kernels' FLOPs are invisible to it, so the closed form otherwise
            per_step = flops_summary.local_flops_per_step if flops_summary.enabled else flops / max(1, s.world // max(1, s.dp))
            print("-----------------------------Accuracy------------------------------")
            for r in rows:
                print("iter", r["iter"], r["output_dtype"], "sum:", r["output_sum"], "loss", r["loss"])
            print("-----------------------------Per-step memory------------------------------")
            for r in rows:
                print("iter", r["iter"], "peak_memory", r["peak_memory_mb"])
            print("-----------------------------Per-step time and FLOPS------------------------------")
            for r in rows:
                print("iter", r["iter"], f"Total Time  : {r['step_time_s'] * 1000:.3f} ms",
                      f"FLOPS : {per_step / r['step_time_s'] / 1e12:.3f} TFLOPS", flush=True)
    s.close()
    return rows


if __name__ == "__main__":
    main()
