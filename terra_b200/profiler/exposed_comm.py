"""Exposed-communication accounting for one training step.

A step's device timeline is split into compute kernels and communication kernels (NCCL kernels, the peer barrier /
signal / halo / small all-reduce / relayout kernels; kernels that compute and communicate at once, such as the window-attention kernel reading peer rows or
the peer-scattering GEMM, count as compute). ``exposed`` is the part of the step during which no compute kernel runs:
time the GPU spends waiting for peers or moving data with nothing to overlap it, plus launch gaps; ``comm_busy`` is the
union of the communication kernels' intervals, of which ``comm_hidden`` overlaps compute.

    python -m torch.distributed.run --nproc-per-node N -m terra_b200.profiler.exposed_comm [--small]

prints one JSON line from rank 0 (max over ranks of every figure). The reference has no such accounting (its profiler
reports FLOPs and memory: profiler/flops_profiler.py:27-152, profiler/memory_timeline.py:172-727); the figure answers
the "exposed communication per step" target of the benchmark plan."""
from __future__ import annotations

import json
from typing import Iterable, List, Sequence, Tuple

# pure communication kernels: NCCL, the flag barrier / signal kernels, the halo push, the small all-reduce, the indexed
# relayout gather, peer row copies, and peer-to-peer copies of the copy engines
COMM_KERNEL_MARKERS = ("nccl", "peer_barrier", "peer_signal", "halo_push", "peer_allreduce_small", "peer_gather_indexed",
                       "peer_copy_rows", "peer_sum_small", "Memcpy PtoP", "Memcpy DtoD (Peer")


def is_comm_kernel(name: str) -> bool:
    low = name.lower()
    return any(m.lower() in low for m in COMM_KERNEL_MARKERS)


def union_length(intervals: Iterable[Tuple[float, float]]) -> float:
    total, end = 0.0, None
    for s, e in sorted(intervals):
        if end is None or s > end:
            total += e - s
            end = e
        elif e > end:
            total += e - end
            end = e
    return total


def _intersection_with_union(a: Sequence[Tuple[float, float]], b: Sequence[Tuple[float, float]]) -> float:
    """Length of (union of a) ∩ (union of b)."""
    return union_length(a) + union_length(b) - union_length(list(a) + list(b))


def account(kernels: Sequence[Tuple[str, float, float]]) -> dict:
    """``kernels``: (name, start, end) in any one time unit. Returns span, compute_busy, comm_busy, comm_hidden,
    exposed (= span - compute_busy) in the same unit."""
    if not kernels:
        return {"span": 0.0, "compute_busy": 0.0, "comm_busy": 0.0, "comm_hidden": 0.0, "exposed": 0.0}
    comp = [(s, e) for n, s, e in kernels if not is_comm_kernel(n)]
    comm = [(s, e) for n, s, e in kernels if is_comm_kernel(n)]
    span = max(e for _, _, e in kernels) - min(s for _, s, _ in kernels)
    cb, mb = union_length(comp), union_length(comm)
    return {"span": span, "compute_busy": cb, "comm_busy": mb, "comm_hidden": _intersection_with_union(comp, comm),
            "exposed": span - cb}


def profile_step(trainer, dev_batch, warmup: int = 3) -> dict:
    """Runs ``warmup`` steps, then one step under ``torch.profiler`` and accounts its device timeline (milliseconds)."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    for _ in range(warmup):
        trainer.step_on_device(dev_batch)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        trainer.step_on_device(dev_batch)
        torch.cuda.synchronize()
    ks: List[Tuple[str, float, float]] = []
    for ev in prof.events():
        if ev.device_type == torch.autograd.DeviceType.CUDA and ev.time_range.end > ev.time_range.start:
            if ev.name.startswith("nccl:"):          # annotation ranges duplicate the NCCL kernels
                continue
            ks.append((ev.name, ev.time_range.start / 1e3, ev.time_range.end / 1e3))
    return account(ks)


def main(argv=None):
    import argparse
    import os
    import sys

    import torch
    import torch.distributed as dist

    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    if here not in sys.path:
        sys.path.insert(0, here)
    from bench import flagship_config          # the benchmark's configuration lives beside the repository root
    from terra_b200.api import Trainer

    ap = argparse.ArgumentParser()
    ap.add_argument("--small", action="store_true")
    a = ap.parse_args(argv)
    n = int(os.environ.get("WORLD_SIZE", "1"))
    t = Trainer(flagship_config(n, a.small), 1)
    batch = {k: v.to(t.device) for k, v in t.synthetic_batch(0).items()}
    res = profile_step(t, batch)
    vals = torch.tensor([res[k] for k in sorted(res)], device=t.device, dtype=torch.float64)
    if dist.is_initialized():
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    if t.rank == 0:
        out = {k: round(float(v), 3) for k, v in zip(sorted(res), vals.tolist())}
        out.update(n_gpus=n, unit="ms", exposed_fraction=round(out["exposed"] / max(out["span"], 1e-9), 4))
        print(json.dumps(out), flush=True)
    t.close()


if __name__ == "__main__":
    main()
