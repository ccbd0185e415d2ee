"""Kernel microbenchmarks: ``python -m terra_b200.ops.microbench <case> [options]``.

Each case times one sm_100a kernel with CUDA events on the launching stream (warm-up, synchronise on both sides,
an L2 flush between timed launches unless ``--no-flush``) and prints one JSON line with the achieved rate and its
fraction of the measured peaks (``MEASURED_PEAKS.json`` next to the repository root when present, otherwise the
fallback figures 6.65 TB/s / 1.59 PFLOP/s). ``--launches N --no-time`` just runs the kernel N times, which is the form
used under ``ncu`` (the capture then picks the kernel by name).

Cases: ``gemm`` (``--epilogue none|bias|gelu|residual|dgelu|wgrad``), ``attn`` (``--bwd``), ``conv`` (``--stride``,
``--wgrad``), ``layernorm`` (``--bwd``), ``groupnorm``, ``adamw``, ``colsum``.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from .. import _ext
from . import _flags as F
from .attention import WindowGeometry
from .gemm import check_status, gemm, status_word


def peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


_FLUSH = None


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def time_kernel(fn, iters=10, warmup=3, flush=True):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def case_gemm(a):
    M, N, K = a.m, a.n, a.k
    flops = 2.0 * M * N * K
    if a.epilogue == "wgrad":
        dy, x = _rand(M, N, scale=0.1), _rand(M, K, scale=0.1)
        out = torch.zeros(N, K, device="cuda")
        bn = a.bn if a.bn else 128
        width = bn % 1000
        rows = 256 if bn >= 1000 else 128
        tiles = ((N + rows - 1) // rows) * ((K + width - 1) // width)
        units = 74 if bn >= 1000 else 148
        split = max(1, min((M + 63) // 64, units // max(1, tiles)))
        if a.bn:
            fn = lambda: gemm(dy, x, a_mn=True, b_mn=True, out=out, accumulate=True, split_k=split, bn=bn)
        else:       # tile width and split as the model's linears choose them
            from .blocks import wgrad_accumulate
            gb = torch.zeros(N, device="cuda") if a.colsum else None      # bias gradient from the same kernel
            fn = lambda: wgrad_accumulate(dy, x, out, gb)
        nbytes = (M * N + M * K) * 2 + N * K * 4
    else:
        x = _rand(M, K)
        w = _rand(K, N, scale=0.05) if a.b_mn else _rand(N, K, scale=0.05)
        bias = _rand(N)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        res = _rand(M, N) if a.epilogue in ("residual",) else None
        aux = _rand(M, N) if a.epilogue == "dgelu" else None
        kw = dict(out=out, bn=a.bn, b_mn=a.b_mn)
        if a.epilogue in ("bias", "gelu", "residual"):
            kw["bias"] = bias
        if a.epilogue == "gelu":
            kw.update(gelu=True, save_pre=True)
        if a.epilogue == "residual":
            kw["residual"] = res
        if a.epilogue == "dgelu":
            kw["dgelu_aux"] = aux
        fn = lambda: gemm(x, w, **kw)
        nbytes = (M * K + N * K + M * N * (2 if a.epilogue == "gelu" else 1)) * 2
        nbytes += M * N * 2 if a.epilogue in ("residual", "dgelu") else 0
    return fn, flops, nbytes


def case_attn(a):
    ext = _ext.load()
    geo = WindowGeometry(1, a.nwh, a.nww, a.ws, a.ws)
    C, heads = a.c, a.heads
    rows = geo.nWh * geo.nWw * geo.N
    qkv = _rand(rows, 3 * C, scale=0.5)
    out = torch.empty(rows, C, device="cuda", dtype=torch.bfloat16)
    dqkv = torch.empty_like(qkv)
    table = torch.randn((2 * a.ws - 1) ** 2, heads, device="cuda") * 0.1
    dtable = torch.zeros_like(table)
    sh = a.ws // 2 if a.shifted else 0
    args = (list(geo.win_start), 0, 1, 0, geo.N, 1, geo.nWh, geo.nWw, C, heads, a.ws, a.ws, sh, sh, bool(a.shifted),
            (C // heads) ** -0.5, 1)
    if a.bwd:
        if a.impl == "tc":
            fn = lambda: ext.window_attn_tc_bwd([qkv.data_ptr()], [out.data_ptr()], [dqkv.data_ptr()], table, dtable, *args,
                                                status_word("cuda"), [], [])
        else:
            fn = lambda: ext.window_attn_bwd([qkv.data_ptr()], [out.data_ptr()], [dqkv.data_ptr()], table, dtable, *args)
        flops = 2.0 * rows * geo.N * C * 5
        nbytes = rows * C * 2 * (3 + 1 + 3)
    else:
        if a.impl == "tc":
            fn = lambda: ext.window_attn_tc_fwd([qkv.data_ptr()], [out.data_ptr()], table, *args, status_word("cuda"), [])
        else:
            fn = lambda: ext.window_attn_fwd([qkv.data_ptr()], [out.data_ptr()], table, *args)
        flops = 2.0 * rows * geo.N * C * 2
        nbytes = rows * C * 2 * (3 + 1)
    return fn, flops, nbytes


def case_conv(a):
    ext = _ext.load()
    from .conv import pack_conv3x3_weight

    B, H, W, C = 1, a.h, a.w, a.c
    x = _rand(B, H, W, C)
    w = _rand(C, C, 3, 3, scale=0.05)
    Ho, Wo = (H, W) if a.stride == 1 else ((H + 1) // 2, W // 2)
    flops = 2.0 * B * Ho * Wo * 9 * C * C
    if a.wgrad:
        dy = _rand(B, Ho, Wo, C, scale=0.1)
        dw = torch.zeros(9, C, C, device="cuda")
        from .conv import _wgrad_split
        split = a.split if a.split else _wgrad_split(B, H, W, a.stride, C, C)      # the model's choice
        fn = lambda: ext.conv3x3_wgrad(x, dy, dw, a.stride, split, status_word("cuda"), None, None)
        nbytes = (x.numel() + dy.numel()) * 2
    else:
        wp = pack_conv3x3_weight(w)
        y = torch.empty(B, Ho, Wo, C, device="cuda", dtype=torch.bfloat16)
        bias = _rand(C)
        fn = lambda: ext.conv3x3_fwd(x, wp, y, a.stride, F.EPI_BIAS, bias, None, status_word("cuda"), None, None)
        nbytes = (x.numel() + y.numel()) * 2
    return fn, flops, nbytes


def case_layernorm(a):
    ext = _ext.load()
    rows, C = a.m, a.c
    x, g, b = _rand(rows, C), _rand(C), _rand(C)
    y = torch.empty_like(x)
    mean, rstd = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    ext.layernorm_fwd(x, g, b, y, mean, rstd, 1e-5)
    if a.bwd:
        dy, dx = _rand(rows, C), torch.empty_like(x)
        dg, db = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
        return (lambda: ext.layernorm_bwd(dy, x, g, mean, rstd, dx, dg, db, None)), 0.0, rows * C * 2 * 3
    return (lambda: ext.layernorm_fwd(x, g, b, y, mean, rstd, 1e-5)), 0.0, rows * C * 2 * 2


def case_groupnorm(a):
    ext = _ext.load()
    B, HW, C, G = 1, a.m, a.c, 32
    x, g, b = _rand(B, HW, C), _rand(C), _rand(C)
    y = torch.empty_like(x)
    sums = torch.zeros(B, G, 2, device="cuda")
    stats = torch.tensor([[0.0, 1.0]] * G, device="cuda").reshape(B, G, 2).contiguous()

    def fn():
        ext.groupnorm_stats(x, sums, G)
        ext.groupnorm_silu_apply(x, stats, g, b, None, y, G)

    return fn, 0.0, B * HW * C * 2 * 3


def case_colsum(a):
    ext = _ext.load()
    x = _rand(a.m, a.c)
    out = torch.zeros(a.c, device="cuda")
    return (lambda: ext.colsum(x, out)), 0.0, a.m * a.c * 2


def case_adamw(a):
    ext = _ext.load()
    n = a.m
    p, m, v, g = (torch.randn(n, device="cuda") for _ in range(4))
    v.abs_()
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    return (lambda: ext.adamw_step(p, m, v, g, pb, 1e-4, 0.9, 0.95, 1e-8, 0.1, 3, 1.0)), 0.0, n * (4 * 7 + 2)


CASES = {"gemm": case_gemm, "attn": case_attn, "conv": case_conv, "layernorm": case_layernorm,
         "groupnorm": case_groupnorm, "adamw": case_adamw, "colsum": case_colsum}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--m", type=int, default=65536)
    ap.add_argument("--n", type=int, default=1536)
    ap.add_argument("--k", type=int, default=384)
    ap.add_argument("--c", type=int, default=384)
    ap.add_argument("--bn", type=int, default=0, help="tile width; 1000 + width selects CTA-pair mode")
    ap.add_argument("--b-mn", action="store_true", help="B given as [K, N] (input-gradient form)")
    ap.add_argument("--epilogue", default="none", choices=["none", "bias", "gelu", "residual", "dgelu", "wgrad"])
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--ws", type=int, default=8)
    ap.add_argument("--nwh", type=int, default=32)
    ap.add_argument("--nww", type=int, default=68)
    ap.add_argument("--shifted", action="store_true")
    ap.add_argument("--impl", default="tc", choices=["tc", "mma"], help="attention forward kernel: tcgen05 or mma.sync")
    ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--h", type=int, default=256)
    ap.add_argument("--w", type=int, default=544)
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--wgrad", action="store_true")
    ap.add_argument("--colsum", action="store_true", help="weight-gradient GEMM: also produce the bias gradient")
    ap.add_argument("--split", type=int, default=0, help="split-K factor of the convolution weight gradient (0: the model's choice)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--launches", type=int, default=0)
    ap.add_argument("--no-time", action="store_true")
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args(argv)
    torch.manual_seed(0)
    fn, flops, nbytes = CASES[a.case](a)
    if a.no_time:
        for _ in range(max(1, a.launches)):
            fn()
        torch.cuda.synchronize()
        check_status("cuda")
        print(json.dumps({"case": a.case, "launches": max(1, a.launches)}))
        return
    ext = _ext.load()
    ms = time_kernel(fn, a.iters, 3, not a.no_flush)
    check_status("cuda")
    stalls = None
    if a.case == "gemm":
        # share of each role's time spent waiting (cycle counters summed over CTAs), one extra launch
        torch.cuda.synchronize()
        ext.gemm_stall_counters(True)
        fn()
        torch.cuda.synchronize()
        c = ext.gemm_stall_counters(True)
        stalls = {"mma_wait_accumulator": c[1] / max(1, c[0]), "mma_wait_operands": c[2] / max(1, c[0]),
                  "tma_wait_stage": c[4] / max(1, c[3]), "epilogue_wait_tile": c[6] / max(1, c[5])}
    pk = peaks()
    out = {"case": a.case, "args": {k: v for k, v in vars(a).items() if k not in ("case",)}, "ms": ms,
           "tflops": flops / ms / 1e9, "gbs": nbytes / ms / 1e6,
           "frac_of_" + pk["source"] + "_bf16": flops / ms / 1e9 / pk["bf16_tflops"],
           "frac_of_" + pk["source"] + "_hbm": nbytes / ms / 1e6 / pk["hbm_gbs"]}
    if a.case == "attn" and a.impl == "tc" and not a.bwd:
        torch.cuda.synchronize()
        ext.window_attn_tc_stalls(True)
        fn()
        c = ext.window_attn_tc_stalls(True)
        stalls = {"producer_wait_buffer": c[1] / max(1, c[0]), "mma_wait_operands": c[3] / max(1, c[2]),
                  "mma_wait_probabilities": c[4] / max(1, c[2]), "softmax_wait_scores": c[6] / max(1, c[5]),
                  "softmax_wait_outputs": c[7] / max(1, c[5]),
                  "softmax_segments": {k: c[8 + i] / max(1, c[5]) for i, k in enumerate(
                      ("prologue", "score_load", "math", "store_signal", "fold_output", "row_store"))}}
    if stalls is not None:
        out["wait_fractions"] = stalls
    print(json.dumps(out))


if __name__ == "__main__":
    main()
