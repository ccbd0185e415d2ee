"""Headline benchmark: training samples/s of the high-resolution hierarchical Swin step on N B200 GPUs of one node.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref, same metric and config

One sample (B = 1, 2 x 93 channels, 2048 x 4320 grid; patch 4, embed 384, depths [2,6,6,2], heads [6,12,24,12], window
8 x 8 with shift, conv down/up block) is split over the N GPUs (row stripes for the conv stage, row-major ragged window
ownership for the Swin stage), so scaling is strong. Synthetic N(0,1) fields with a seeded ~30 % blob land mask, random
initial weights, bf16 compute with fp32 master weights, masked L1 loss, AdamW step inside the timed region.

Rank 0 prints ONE JSON line. ``value`` is device-timed (CUDA events, max over ranks) on device-resident inputs
(each 3.3 GB, far larger than L2); ``e2e`` times the same step through ``terra_b200.api.Trainer.step`` including the
per-step host->device copy of input and label from pinned memory and the device->host read of the loss.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "train_samples_per_s"


def parse_layout(text, n_gpus):
    """``"wg,sp,tp"`` -> tuple; the default is the 2 x 2 x 2 layout on 8 GPUs and nothing elsewhere."""
    if text in (None, "", "none"):
        return (2, 2, 2) if (text is None and n_gpus == 8) else None
    wg, sp, tp = (int(v) for v in text.split(","))
    if wg * sp * tp != n_gpus:
        raise SystemExit(f"--extra-layout {text}: wg x sp x tp must equal --gpus {n_gpus}")
    return wg, sp, tp


def flagship_config(n_gpus: int, small: bool = False, layout=None) -> dict:
    """``layout = (window groups, sequence-parallel size, tensor-parallel size)``: the factorised layout of the same
    model (conv stage still split in ``n_gpus`` row stripes); ``None``: window parallel over all GPUs."""
    cfg = _flagship_config(n_gpus, small)
    if layout is not None:
        wg, sp, tp = layout
        if small:                         # head counts every sp x tp of the smoke layouts divides
            cfg.update(embedding_dim=128, num_heads=[4, 8])
        cfg.update(xfmr_wp_topo=f"({wg}, 1)", xfmr_sp_size=sp, tensor_parallel_size=tp, optimizer_config=6)
    return cfg


def _flagship_config(n_gpus: int, small: bool = False) -> dict:
    cfg = dict(
        task_type="glorys", model_architecture="credit_hierarchical_swin", model_type="parallel",
        height=2048, width=4320, num_channels=186, patch_size=4, embedding_dim=384, depths=[2, 6, 6, 2],
        num_heads=[6, 12, 24, 12], num_layers=16, window_size=8, padding_policy="auto",
        window_assignment_mode="terra_m1_ragged_auto", wp_topo=f"({n_gpus}, 1)", xfmr_wp_topo=f"({n_gpus}, 1)",
        xfmr_sp_size=1, tensor_parallel_size=1, optimizer_config=6 if n_gpus > 1 else 4, precision="bf16",
        half_model=False, loss_func="L1", learning_rate=1e-4, micro_batch_size=1, use_attn_mask=True,
        use_relative_position_bias=True, comm_backend=os.environ.get("TERRA_COMM_BACKEND", "nvlink"))
    if small:
        cfg.update(height=256, width=512, num_channels=64, embedding_dim=96, depths=[2, 2], num_heads=[3, 6], num_layers=4)
    return cfg


class ClockSampler:
    """Samples SM clocks / throttle reasons of this process's GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()     # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        try:
            rows = [ln.strip().split(", ") for ln in open(self.path) if ln.strip()]
            os.unlink(self.path)
        except Exception:
            return out
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.strip().lower().startswith("active"):
                    reasons.add(name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def _time_device_steps(trainer, devb, steps, warmup, barrier):
    """W untimed + K timed steps on device-resident batches: (ms per step as the max over ranks, launches, last loss)."""
    import torch
    import torch.distributed as dist

    from terra_b200 import _ext

    on_gpu = trainer.device.type == "cuda"
    ext = _ext.load() if on_gpu else None          # the kernels (and their launch counter) exist on a GPU only
    for i in range(warmup):
        trainer.step_on_device(devb[i % 2])
    barrier()
    launches0 = ext.launch_count() if on_gpu else 0
    if on_gpu:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
    t0 = time.perf_counter()
    for i in range(steps):
        loss = trainer.step_on_device(devb[i % 2])
    if on_gpu:
        ev1.record()
    barrier()
    launches = ext.launch_count() - launches0 if on_gpu else 0
    # the host clock only where there is no device (the harness's own test on CPU ranks)
    elapsed = ev0.elapsed_time(ev1) if on_gpu else (time.perf_counter() - t0) * 1e3
    ms = torch.tensor([elapsed / steps], device=trainer.device)
    if dist.is_initialized():
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item(), int(launches), float(loss.item())


def run_ours(args):
    import gc

    import torch
    import torch.distributed as dist

    from terra_b200.api import Trainer
    from terra_b200.ops.gemm import check_status

    cfg = flagship_config(args.gpus, args.small)
    trainer = Trainer(cfg, data_parallel_group_size=1)
    rank, world, dev = trainer.rank, trainer.world, trainer.device
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    live = dist.is_initialized()

    def barrier():
        if live:
            dist.barrier()
        if dev.type == "cuda":
            torch.cuda.synchronize()

    host = [trainer.synthetic_batch(sample=i) for i in range(2)]
    devb = [{k: v.to(dev, non_blocking=True) for k, v in b.items()} for b in host]
    h2d_bytes = sum(v.numel() * v.element_size() for v in host[0].values())

    # ---- device-timed kernel-only number (the clock sampler runs from the warm-up on: nvidia-smi needs a moment to
    #      start, and a multi-GPU timed region lasts only tens of milliseconds)
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    ms_per_step, launches, last_loss = _time_device_steps(trainer, devb, args.steps, args.warmup, barrier)

    # ---- end to end through the public API: staged H2D of every step's batch + D2H of the loss
    e2e_loss, e2e_ms = None, torch.tensor([float("nan")], device=dev)
    if not args.skip_e2e:
        staged = trainer.stage(host[0])
        for i in range(max(1, args.warmup // 2)):
            nxt = trainer.stage(host[(i + 1) % 2])
            trainer.step(host[i % 2], staged)
            staged = nxt
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            nxt = trainer.stage(host[(i + 1) % 2])       # next step's upload overlaps this step's compute
            e2e_loss = trainer.step(host[i % 2], staged)
            staged = nxt
        barrier()
        e2e_ms = torch.tensor([(time.perf_counter() - t0) * 1e3 / args.steps], device=dev)
        if live:
            dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop()
    if dev.type == "cuda":
        check_status(dev)
    seq_len = trainer.archi["padded_shape"][0] // 8 * (trainer.archi["padded_shape"][1] // 8)

    gb = 1
    par = f"wp{args.gpus}" if args.gpus > 1 else "single"
    line = {
        "metric": METRIC, "value": gb / (ms_per_step * 1e-3), "unit": "samples/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "terra_b200",
        "config": {"model": "credit_hierarchical_swin 2048x4320x186 p4 D384 depths[2,6,6,2] heads[6,12,24,12] ws8"
                   if not args.small else "credit_hierarchical_swin small (smoke)",
                   "global_batch": gb, "seq_len": seq_len,
                   "parallelism": par, "l2_policy": "inputs (3.3 GB each) larger than L2, two batches alternated",
                   "optimizer": "AdamW fp32 master, sharded over ranks when N>1"},
        "clocks": clocks,
        "e2e": None if args.skip_e2e else {"value": gb / (e2e_ms.item() * 1e-3), "unit": "samples/s",
                                           "ms_per_step": e2e_ms.item(), "h2d_bytes_per_step": h2d_bytes,
                                           "d2h_bytes_per_step": 4},
        "gpu_launches": int(launches), "loss": last_loss, "e2e_loss": e2e_loss,
    }

    # ---- the factorised layout of the same model and data (window groups x sequence parallel x tensor parallel, sharded
    #      AdamW): the step in which the fused tensor-parallel GEMMs and the sequence-parallel K/V gather run. Every rank
    #      runs it in a child process of its own (a fresh CUDA context, process group and rendezvous port, as a separate
    #      launch would have) and waits for it no longer than the deadline; the headline above is already measured and is
    #      printed whatever the child does.
    layout = parse_layout(args.extra_layout, args.gpus)
    child_port = [None]
    if layout is not None:
        if rank == 0:                     # a port that is free now, agreed on while the ranks can still talk
            import socket

            with socket.socket() as sock:
                sock.bind(("127.0.0.1", 0))
                child_port[0] = sock.getsockname()[1]
        if live:
            dist.broadcast_object_list(child_port, src=0)
    trainer.close()                       # frees the model; destroys the process group
    del trainer, devb
    gc.collect()
    if dev.type == "cuda":
        torch.cuda.empty_cache()
    if layout is not None:
        line["layout_" + "x".join(str(v) for v in layout)] = _extra_layout_in_child(args, layout, rank, child_port[0])
    if rank == 0:
        print(json.dumps(line), flush=True)


def _extra_layout_in_child(args, layout, rank, port):
    """Runs ``bench.py --only-layout`` as a child of this rank; returns rank 0's result (or the reason there is none).
    ``port``: the rendezvous port of the children (the same on every rank)."""
    text = ",".join(str(v) for v in layout)
    out = os.path.join(tempfile.gettempdir(), f"terra_bench_layout_{port}_{text.replace(',', 'x')}.json")
    if rank == 0 and os.path.exists(out):
        os.unlink(out)
    env = dict(os.environ)
    env["MASTER_ADDR"] = os.environ.get("MASTER_ADDR", "127.0.0.1")
    env["MASTER_PORT"] = str(port)                                                  # a rendezvous of its own
    for name in [k for k in env if k.startswith("TORCHELASTIC_")]:
        # without TORCHELASTIC_USE_AGENT_STORE the child of rank 0 hosts the store on the new port itself (the launcher's
        # agent store listens on the old one only)
        env.pop(name)
    cmd = [sys.executable, os.path.abspath(__file__), "--gpus", str(args.gpus), "--steps", str(args.steps), "--warmup",
           str(args.warmup), "--only-layout", text, "--result-file", out] + (["--small"] if args.small else [])
    try:
        child = subprocess.Popen(cmd, env=env, stdout=subprocess.DEVNULL, stderr=subprocess.PIPE, text=True)
    except Exception as exc:
        return {"error": f"could not start: {exc!r}"[:300]}
    try:
        _, err = child.communicate(timeout=args.extra_deadline)
    except subprocess.TimeoutExpired:
        child.kill()                      # the exact child started above
        child.communicate()
        return {"error": f"no result within {args.extra_deadline} s"}
    if rank != 0:
        return None
    try:
        with open(out) as f:
            result = json.load(f)
        os.unlink(out)
        return result
    except Exception:
        return {"error": f"child exit code {child.returncode}: {(err or '').strip()[-300:]}"}


def run_layout_only(args):
    """Child of ``run_ours``: the device-timed loop of one factorised layout; rank 0 writes the result file."""
    import torch
    import torch.distributed as dist

    from terra_b200.api import Trainer
    from terra_b200.ops.gemm import check_status

    layout = parse_layout(args.only_layout, args.gpus)
    trainer = Trainer(flagship_config(args.gpus, args.small, layout), data_parallel_group_size=1)
    dev = trainer.device

    def barrier():
        if dist.is_initialized():
            dist.barrier()
        if dev.type == "cuda":
            torch.cuda.synchronize()

    devb = [{k: v.to(dev, non_blocking=True) for k, v in trainer.synthetic_batch(sample=i).items()} for i in range(2)]
    ms, launches, loss = _time_device_steps(trainer, devb, args.steps, args.warmup, barrier)
    if dev.type == "cuda":
        check_status(dev)
    pc = trainer.model.pctx
    if trainer.rank == 0:
        result = {"layout": "wg{}xsp{}xtp{}".format(*layout), "ms_per_step": ms, "samples_per_s": 1.0 / (ms * 1e-3),
                  "gpu_launches": launches, "loss": loss, "optimizer": "DistributedAdamW (optimizer_config 6)",
                  "fused_tp": getattr(pc, "tp_comm", None) is not None, "fused_attn": pc.fused_comm is not None}
        with open(args.result_file + ".tmp", "w") as f:
            json.dump(result, f)
        os.replace(args.result_file + ".tmp", args.result_file)
    trainer.close()


def run_reference(args):
    try:
        from baseline import ref_harness
    except Exception as exc:  # pragma: no cover
        print(json.dumps({"impl": "reference", "unavailable": f"harness import failed: {exc!r}"[:300]}), flush=True)
        return
    ref_harness.main(args, flagship_config(args.gpus, args.small), ClockSampler, METRIC,
                     parse_layout(args.extra_layout, args.gpus))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--small", action="store_true", help="tiny model (smoke test of the harness, not a benchmark)")
    ap.add_argument("--skip-e2e", action="store_true", help="only the device-timed loop (used when profiling)")
    ap.add_argument("--only-layout", default=None, help=argparse.SUPPRESS)     # child mode, see run_ours
    ap.add_argument("--result-file", default=None, help=argparse.SUPPRESS)
    ap.add_argument("--extra-deadline", type=float, default=200.0,
                    help="seconds after which the extra layout is given up and the headline printed without it")
    ap.add_argument("--extra-layout", default=None,
                    help='also time the factorised layout "wg,sp,tp" of the same model (default: 2,2,2 on 8 GPUs; "none")')
    args = ap.parse_args()
    if args.warmup < 3 and not args.small:
        args.warmup = 3
    if args.only_layout:
        run_layout_only(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
