"""Optional NVTX ranges around the framework's kernel launches (``TERRA_NVTX=1``): timelines captured by an external
profiler then show ``terra.gemm``, ``terra.window_attn.fwd`` ... instead of bare kernel names. Off by default: the
decorator returns the function unchanged, so the hot path pays nothing."""
from __future__ import annotations

import functools
import os

ENABLED = os.environ.get("TERRA_NVTX", "0") == "1"


def nvtx_range(name: str):
    def deco(fn):
        if not ENABLED:
            return fn

        @functools.wraps(fn)
        def wrapped(*args, **kwargs):
            import torch

            if not torch.cuda.is_available():
                return fn(*args, **kwargs)
            torch.cuda.nvtx.range_push(name)
            try:
                return fn(*args, **kwargs)
            finally:
                torch.cuda.nvtx.range_pop()

        return wrapped

    return deco
