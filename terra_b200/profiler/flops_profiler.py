"""FLOP and kernel-time profiling (reference: profiler/flops_profiler.py:27-152).

``TorchFlopsProfiler`` wraps ``torch.profiler`` with a ``[wait, warmup, active, repeat]`` schedule
(``TORCH_PROF_STEP_LIST``), sums ``evt.flops`` over the active steps, reduces to world sum / average, lists the top
operators by device time and can write a TensorBoard trace. Because the hot operators here are custom kernels whose
FLOPs the profiler cannot see, ``analytic_step_flops`` supplies the model's FLOP count in closed form.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List

import torch
import torch.distributed as dist


@dataclass
class FlopsSummary:
    """What the profiler counted (reference: profiler/flops_profiler.py:7-24). ``enabled`` False: nothing was profiled
    and every figure is zero."""
    enabled: bool
    local_flops_per_step: float = 0.0
    world_flops_per_step: float = 0.0
    world_avg_flops_per_step: float = 0.0
    active_steps: int = 0
    event_count: int = 0

    def local_tflops(self, step_time_s: float) -> float:
        return self.local_flops_per_step / step_time_s / 1e12 if step_time_s > 0 else 0.0

    def world_tflops(self, step_time_s: float) -> float:
        return self.world_flops_per_step / step_time_s / 1e12 if step_time_s > 0 else 0.0

    def as_metadata(self) -> Dict[str, float]:
        """The ``flops_profiler_*`` keys of the harnesses' JSON records."""
        return {"flops_profiler_enabled": self.enabled, "flops_profiler_active_steps": self.active_steps,
                "flops_profiler_event_count": self.event_count,
                "flops_profiler_local_flops_per_step": self.local_flops_per_step,
                "flops_profiler_world_flops_per_step": self.world_flops_per_step,
                "flops_profiler_world_avg_flops_per_step": self.world_avg_flops_per_step}


class TorchFlopsProfiler:
    def __init__(self, step_list=(1, 1, 3, 1), enabled=True, trace_dir=None, rank=0):
        self.wait, self.warmup, self.active, self.repeat = (int(v) for v in step_list)
        self.enabled = enabled
        self.rank = rank
        self.trace_dir = trace_dir
        self.prof = None
        self._summary = None

    def __enter__(self):
        if not self.enabled:
            return self
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        handler = None
        if self.trace_dir and self.rank == 0:
            os.makedirs(self.trace_dir, exist_ok=True)
            handler = torch.profiler.tensorboard_trace_handler(self.trace_dir)
        self.prof = torch.profiler.profile(
            activities=acts, with_flops=True, on_trace_ready=handler,
            schedule=torch.profiler.schedule(wait=self.wait, warmup=self.warmup, active=self.active, repeat=self.repeat))
        self.prof.__enter__()
        return self

    def __exit__(self, *exc):
        if self.prof is not None:
            self.prof.__exit__(*exc)
        return False

    def step(self):
        if self.prof is not None:
            self.prof.step()

    def total_steps(self) -> int:
        return (self.wait + self.warmup + self.active) * max(1, self.repeat)

    def summarize(self) -> "FlopsSummary":
        """FLOPs per active step on this rank, summed and averaged over the ranks. Collective when a process group is
        up, so every rank calls it; the result is kept, later calls return it without communicating."""
        if self._summary is not None:
            return self._summary
        if self.prof is None:
            self._summary = FlopsSummary(enabled=False)
            return self._summary
        counted = [getattr(e, "flops", 0) or 0 for e in self.prof.key_averages()]
        steps = max(1, self.active * max(1, self.repeat))
        local = float(sum(counted)) / steps
        world_sum = world_avg = local
        if dist.is_available() and dist.is_initialized():
            t = torch.tensor([local], dtype=torch.float64, device="cuda" if torch.cuda.is_available() else "cpu")
            dist.all_reduce(t)
            world_sum = float(t.item())
            world_avg = world_sum / dist.get_world_size()
        self._summary = FlopsSummary(enabled=True, local_flops_per_step=local, world_flops_per_step=world_sum,
                                     world_avg_flops_per_step=world_avg, active_steps=steps,
                                     event_count=sum(1 for f in counted if f > 0))
        return self._summary

    def top_ops(self, n=20) -> List[Dict[str, float]]:
        if self.prof is None:
            return []
        evts = sorted(self.prof.key_averages(), key=lambda e: getattr(e, "device_time_total", 0), reverse=True)[:n]
        return [{"name": e.key, "device_time_us": float(getattr(e, "device_time_total", 0)), "calls": int(e.count)}
                for e in evts]

    def print_top_ops(self, n=20):
        for row in self.top_ops(n):
            print(f"{row['device_time_us']:12.1f} us  x{row['calls']:<6d} {row['name']}")


def analytic_step_flops(archi: dict, batch: int = 1, training: bool = True) -> float:
    """Multiply-add FLOPs (2 per MAC) of one step of the hierarchical Swin on the whole padded grid."""
    p, C, D = archi["patch_size"], archi["num_channels"], archi["embedding_dim"]
    ph, pw = archi["padded_shape"]
    sampling = archi.get("model_architecture", "credit_hierarchical_swin") == "credit_hierarchical_swin"
    hp, wp = ph // p, pw // p
    ds = 2 if sampling else 1
    tok = (hp // ds) * (wp // ds)
    ws = archi["window_size"]
    N = ws[0] * ws[1] if isinstance(ws, (list, tuple)) else ws * ws
    layers = archi["num_layers"]
    macs = 2 * hp * wp * (p * p * C) * D                       # patch embed + recovery
    macs += layers * tok * (12 * D * D + 2 * N * D)            # qkv, proj, mlp, attention
    if sampling:
        macs += tok * 9 * D * D * 3                            # down conv + 2 residual convs at token resolution
        macs += tok * 4 * D * D                                # transposed conv
        macs += hp * wp * 9 * D * D * 2                        # 2 residual convs at patch resolution
    return 2.0 * macs * batch * (3.0 if training else 1.0)
