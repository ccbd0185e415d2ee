"""Reference arm of ``bench.py``: runs the UNMODIFIED reference installed under ``baseline/_ref`` through its own
model classes, process-group manager and ``one_step_train``, on the same metric, config and synthetic data as the
framework's own arm. Nothing from ``terra_b200``'s models, kernels or engine is on this path; only the synthetic
data generator is shared so that both arms see the same fields.

What has to differ from the framework's arm, because the reference cannot express it (recorded in the JSON line):
  * one ``num_heads`` for every layer (12) and ``num_layers = sum(depths)``: the reference is single-stage;
  * the grid size is passed to the model constructors directly, because the reference's config resolver hard-codes
    2041 x 4320;
  * ``timm`` is replaced by a two-function shim (``to_2tuple``, ``trunc_normal_``);
  * 1 GPU runs the sequential build (the reference's 1-GPU mode), N > 1 the window-parallel build with
    ``wp_topo = (N, 1)`` and ``terra_m1_ragged_auto``; bf16 autocast with fp32 parameters, DDP over the (size-1) data
    parallel group, ``grad_post_process`` all-reduces over the window-parallel group, ``torch.optim.AdamW``.

With an extra layout ``(wg, sp, tp)`` (the 2 x 2 x 2 layout on 8 GPUs) the same model and data are timed a second time
in the reference's factorised build: ``xfmr_wp_topo = (wg, 1)``, ``xfmr_sp_size = sp``, ``tensor_parallel_size = tp``,
its own ``DistributedAdamW`` (``optimizer_config: 6``, which the reference requires for TP > 1) under bf16 autocast,
exactly the objects its ``get_model_for_train`` builds for that configuration. The result is reported under
``layout_<wg>x<sp>x<tp>`` of the same JSON line.
"""
from __future__ import annotations

import json
import os
import sys
import time


def _emit(obj):
    print(json.dumps(obj), flush=True)


def main(args, cfg, ClockSampler, metric, layout=None):
    from baseline import ref_import

    if not ref_import.available():
        _emit({"impl": "reference", "unavailable": "reference is not installed under baseline/_ref"})
        return
    try:
        import torch
        import torch.distributed as dist

        if not torch.cuda.is_available():
            _emit({"impl": "reference", "unavailable": "no CUDA device (the reference's parallel model needs CUDA + NCCL)"})
            return
        ref_import.enable()
        _run(args, cfg, ClockSampler, metric, layout)
    except Exception as exc:  # the reference arm must never take the driver down
        import traceback

        traceback.print_exc(file=sys.stderr)
        _emit({"impl": "reference", "unavailable": f"reference run failed: {type(exc).__name__}: {exc}"[:400]})


def _run(args, cfg, ClockSampler, metric, layout=None):
    import torch
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    from core.rank_manager import ParallelManager                      # reference
    from core.runtime.run_model import one_step_train                  # reference
    from models.reference_model.parallel_hierarchical_swin import ParallelHierarchicalSwin          # reference
    from models.reference_model.sequential_hierarchical_swin import SequentialHierarchicalSwin      # reference
    from optimizer.utils import get_optimizer as ref_get_optimizer     # reference

    from terra_b200.config import resolve_padding_spec                 # padding arithmetic only
    from terra_b200.data.synthetic import land_mask_for_rank, synthetic_batch   # shared synthetic data

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29531")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", "0")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group(backend="nccl", init_method="env://", rank=rank, world_size=world)
    torch.manual_seed(1234)

    H, W, C, p, D = cfg["height"], cfg["width"], cfg["num_channels"], cfg["patch_size"], cfg["embedding_dim"]
    ws = cfg["window_size"]
    layers, heads = sum(cfg["depths"]), 12 if D % 12 == 0 else cfg["num_heads"][0]
    n = args.gpus
    mode = "terra_m1_ragged_auto"
    loss_fn = torch.nn.L1Loss(reduction="mean")
    model_type = "sequential" if n == 1 else "parallel"

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def build(lay):
        """(step function, padding spec) of the reference's own objects for the main layout (``lay is None``) or the
        factorised one."""
        wg, sp, tp = lay if lay is not None else (n, 1, 1)
        spec = resolve_padding_spec({"padding_policy": "auto"}, "credit_hierarchical_swin", H, W, p, ws, (n, 1), (wg, 1), mode)
        manager = ParallelManager(dp_size=1, mp_size=1, wp_topo=(n, 1), xfmr_wp_topo=(wg, 1), rank=rank, world_size=world,
                                  device=dev, window_assignment_mode=mode, xfmr_sp_size=sp, tensor_parallel_size=tp)
        if n == 1:
            model = SequentialHierarchicalSwin(padding_scale=1, num_channels=C, patch_size=p, window_size=ws, height=H,
                                               width=W, embedding_dim=D, num_heads=heads, num_layers=layers,
                                               recompute_config=None, manager=manager, padding_spec=spec)
        else:
            model = ParallelHierarchicalSwin(height=H, width=W, num_channels=C, patch_size=p, embedding_dim=D,
                                             num_layers=layers, num_heads=heads, window_size=ws, manager=manager,
                                             device=dev, padding_scale=1, embedding_parallel_type="window_linear",
                                             recompute_config=None, padding_spec=spec)
        model = model.to(dev)
        if lay is None:
            model = DDP(model, device_ids=[local], process_group=manager.data_parallel_group)
            optimizer = torch.optim.AdamW(model.parameters(), lr=cfg["learning_rate"], betas=(0.9, 0.95), weight_decay=0.1)
            optimizer.global_step = 0
            state = (True, False, None, False)   # USE_DDP, USE_FSDP, ZERO_STAGE_NUMBER, USE_DIST_OPT
        else:
            model.train()
            _, optimizer = ref_get_optimizer("bf16", model, cfg["learning_rate"], manager=manager, model_type=model_type,
                                             zero_stage_number=None, use_distributed_optimizer=True)
            state = (False, False, None, True)
        mask, pad_scale = land_mask_for_rank(H, W, C, p, spec["padded_shape"], spec["initial_padding"], model_type, n, rank)
        task = {"land_sea_mask": mask.to(dev, torch.bfloat16), "padding_loss_scale": pad_scale, "test_iter_num": -1,
                "show_gradient_flag": False}
        other = {"embedding_parallel_type": "window_linear" if n > 1 else None}

        def step(batch):
            _, loss, _, _ = one_step_train("glorys", model_type, model, None, optimizer, batch, task, other, "bf16", False,
                                           torch.bfloat16, loss_fn, None, manager=manager, optimizer_state_tuple=state,
                                           memory_timeline=None, clip_grad=False, sync_for_timing=False,
                                           barrier_for_timing=False)
            return loss

        return step, spec

    def time_device(step, batches):
        for i in range(args.warmup):
            step(batches[i % 2])
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for i in range(args.steps):
            loss = step(batches[i % 2])
        ev1.record()
        barrier()
        ms = torch.tensor([ev0.elapsed_time(ev1) / args.steps], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item(), float(loss.item())

    step, spec = build(None)
    host = [synthetic_batch(H, W, C, p, spec["padded_shape"], spec["initial_padding"], model_type, n, rank, 1, i, 2025,
                            torch.bfloat16, pin=True, gen_device="cuda") for i in range(2)]
    devb = [{k: v.to(dev, non_blocking=True) for k, v in b.items()} for b in host]
    h2d_bytes = sum(v.numel() * v.element_size() for v in host[0].values())

    sampler = ClockSampler(local)
    sampler.start()
    ms, last_loss = time_device(step, devb)

    # end to end the way the reference's own loop does it: pinned host batch -> .to(device, non_blocking) -> step -> .item()
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        b = {k: v.to(dev, non_blocking=True) for k, v in host[i % 2].items()}
        e2e_loss = float(step(b).item())
    barrier()
    e2e_ms = torch.tensor([(time.perf_counter() - t0) * 1e3 / args.steps], device=dev)
    dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop()

    line = {
        "metric": metric, "value": 1.0 / (ms * 1e-3), "unit": "samples/s", "n_gpus": n, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16 autocast, fp32 parameters", "data": "synthetic", "impl": "reference",
        "config": {"model": f"credit_hierarchical_swin {H}x{W}x{C} p{p} D{D} layers {layers} heads {heads} ws{ws}",
                   "global_batch": 1, "parallelism": f"wp{n}" if n > 1 else "sequential",
                   "deviations": "single num_heads (reference is single-stage); grid passed to constructors; timm shim",
                   "l2_policy": "inputs (3.3 GB each) larger than L2, two batches alternated"},
        "clocks": clocks,
        "e2e": {"value": 1.0 / (e2e_ms.item() * 1e-3), "unit": "samples/s", "ms_per_step": e2e_ms.item(),
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4},
        "loss": last_loss, "e2e_loss": e2e_loss,
    }
    if layout is not None:
        # The main number is measured; the factorised build must not be able to lose it. An exception is reported in
        # the line; a rank that stops answering is turned into an orderly exit of every rank by the deadline.
        import gc
        import threading

        key = "layout_" + "x".join(str(v) for v in layout)
        name = "wg{}xsp{}xtp{}".format(*layout)
        deadline = float(getattr(args, "extra_deadline", 420.0))
        printed = threading.Lock()

        def give_up():
            if printed.acquire(blocking=False):
                line[key] = {"layout": name, "unavailable": f"no result within {deadline} s"}
                if rank == 0:
                    _emit(line)
                os._exit(0)

        timer = threading.Timer(deadline, give_up)
        timer.daemon = True
        timer.start()
        del step
        gc.collect()
        torch.cuda.empty_cache()
        failed = False
        try:
            step2, _ = build(layout)
            ms2, loss2 = time_device(step2, devb)
            extra = {"layout": name, "ms_per_step": ms2, "samples_per_s": 1.0 / (ms2 * 1e-3),
                     "loss": loss2, "optimizer": "reference DistributedAdamW (optimizer_config 6)"}
        except Exception as exc:   # the main number stands even if the factorised build cannot run
            import traceback

            traceback.print_exc(file=sys.stderr)
            extra = {"layout": name, "unavailable": f"{type(exc).__name__}: {exc}"[:300]}
            failed = True
        if not printed.acquire(blocking=False):
            return
        timer.cancel()
        line[key] = extra
        if failed:                 # other ranks may sit in a collective: leave without another one
            if rank == 0:
                _emit(line)
            os._exit(0)
    if rank == 0:
        _emit(line)
    dist.destroy_process_group()
