"""FLOP and kernel-time profiling (reference: profiler/flops_profiler.py:27-152).

``TorchFlopsProfiler`` wraps ``torch.profiler`` with a ``[wait, warmup, active, repeat]`` schedule
(``TORCH_PROF_STEP_LIST``), sums ``evt.flops`` over the active steps, reduces to world sum / average, lists the top
operators by device time and can write a TensorBoard trace. Because the hot operators here are custom kernels whose
FLOPs the profiler cannot see, ``analytic_step_flops`` supplies the model's FLOP count in closed form.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


class TorchFlopsProfiler:
    def __init__(self, step_list=(1, 1, 2, 1), enabled=True, trace_dir=None, rank=0):
        self.wait, self.warmup, self.active, self.repeat = (int(v) for v in step_list)
        self.enabled = enabled
        self.rank = rank
        self.trace_dir = trace_dir
        self.prof = None

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

    def summarize(self) -> Dict[str, float]:
        if self.prof is None:
            return {}
        flops = sum(getattr(e, "flops", 0) or 0 for e in self.prof.key_averages())
        per_step = flops / max(1, self.active * max(1, self.repeat))
        out = {"flops_per_step_local": float(per_step)}
        if dist.is_available() and dist.is_initialized():
            t = torch.tensor([per_step], dtype=torch.float64, device="cuda" if torch.cuda.is_available() else "cpu")
            dist.all_reduce(t)
            out["flops_per_step_world_sum"] = float(t.item())
            out["flops_per_step_world_avg"] = float(t.item() / dist.get_world_size())
        else:
            out["flops_per_step_world_sum"] = out["flops_per_step_world_avg"] = float(per_step)
        return out

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
