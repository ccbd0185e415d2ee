"""Microbenchmarks of the fused compute + communication kernels against the library sequence they replace.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m terra_b200.ops.microbench_comm <case> [options]

One rank per GPU of one node. Every number is device time (CUDA events on the launching stream, warm-up first, the
maximum over ranks). Rank 0 prints one JSON line per configuration with the fused time, the library time and the
roofline: the slower of FLOPs / measured bf16 peak and NVLink bytes / 770 GB/s (the measured peer-copy bandwidth per
direction and GPU), and of HBM bytes / measured copy bandwidth where the kernel is memory bound.

Cases
  ``halo``       boundary strips ``[1, rows, W, C]`` bf16 to both row-stripe neighbours: one ``halo_push`` kernel over
                 peer memory against NCCL ``batch_isend_irecv`` (what the reference's HaloExchange issues)
  ``ag_gemm``    all-gather -> GEMM (``M`` rows over the ranks, ``N = K``): fused (copy-engine and direct transports)
                 against NCCL all-gather + GEMM
  ``gemm_rs``    GEMM -> reduce-scatter: fused against GEMM + NCCL reduce-scatter
  ``dist_adamw`` sharded AdamW over a flat buffer: one peer-memory kernel (reduce + update + store to every replica)
                 against NCCL reduce-scatter + the AdamW kernel + NCCL all-gather
  ``small_sum``  all-reduce of a few hundred floats (GroupNorm statistics): single-block peer kernel against NCCL
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

from .. import _ext
from ..distributed import init_distributed
from ..parallel.nvlink import BARRIER_SPIN_LIMIT, PeerDomain, SymmetricArena
from .gemm import check_status, gemm
from .microbench import peaks

NVLINK_GBS = 770.0


def timed(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def emit(rank, **kw):
    if rank == 0:
        print(json.dumps(kw), flush=True)


def case_halo(a, rank, world, dev):
    prev, nxt = (rank - 1 if rank > 0 else None), (rank + 1 if rank < world - 1 else None)
    for W in a.widths:
        for C in a.channels:
            shape = (1, a.rows, W, C)
            nbytes = a.rows * W * C * 2
            arena = SymmetricArena(dist.group.WORLD, 64 * nbytes + (32 << 20), dev)
            peer = PeerDomain(arena)
            top = torch.randn(shape, device=dev).to(torch.bfloat16)
            bot = torch.randn(shape, device=dev).to(torch.bfloat16)

            def fused():
                arena.reset()
                return peer.exchange_rows(top, bot)

            def nccl():
                ops, rp, rn = [], torch.empty_like(bot), torch.empty_like(top)
                if prev is not None:
                    ops += [dist.P2POp(dist.isend, top, prev), dist.P2POp(dist.irecv, rp, prev)]
                if nxt is not None:
                    ops += [dist.P2POp(dist.isend, bot, nxt), dist.P2POp(dist.irecv, rn, nxt)]
                for r in dist.batch_isend_irecv(ops):
                    r.wait()

            lo, hi = fused()
            torch.cuda.synchronize()
            dist.barrier()
            # what arrived is the neighbour's strip: compare against an NCCL exchange of the same data
            ok = True
            if prev is not None or nxt is not None:
                rp, rn = torch.empty_like(bot), torch.empty_like(top)
                ops = []
                if prev is not None:
                    ops += [dist.P2POp(dist.isend, top, prev), dist.P2POp(dist.irecv, rp, prev)]
                if nxt is not None:
                    ops += [dist.P2POp(dist.isend, bot, nxt), dist.P2POp(dist.irecv, rn, nxt)]
                for r in dist.batch_isend_irecv(ops):
                    r.wait()
                ok = (prev is None or torch.equal(lo, rp)) and (nxt is None or torch.equal(hi, rn))
            t_f, t_n = timed(fused, a.iters), timed(nccl, a.iters)
            roof = nbytes / (NVLINK_GBS * 1e9) * 1e3            # each direction moves one strip
            emit(rank, case="halo", ranks=world, W=W, C=C, rows=a.rows, strip_mb=nbytes / 2 ** 20, fused_ms=t_f, nccl_ms=t_n,
                 roofline_ms=roof, fused_of_roofline=roof / t_f, speedup_vs_nccl=t_n / t_f, correct=bool(ok))
            check_status(dev)
            del peer, arena


def case_tp_gemm(a, rank, world, dev, which):
    from .tp_fused import TpFusedComm

    pk = peaks()
    for nk in a.width:
        for M in a.tokens:
            rows = M // world
            Ns = nk // world
            arena = SymmetricArena(dist.group.WORLD, rows * nk * 2 * 2 + world * rows * nk * 2 * 2 + (64 << 20), dev)
            comm = TpFusedComm(arena)
            torch.manual_seed(1)
            if which == "ag_gemm":
                x = arena.alloc((rows, nk), torch.bfloat16, persistent=True)
                x.copy_((torch.randn(rows, nk, device=dev) * 0.1).to(torch.bfloat16))
                w = (torch.randn(Ns, nk, device=dev) * 0.02).to(torch.bfloat16)          # column shard [N / tp, K]
                gathered = torch.empty(M, nk, dtype=torch.bfloat16, device=dev)

                def lib():
                    dist.all_gather_into_tensor(gathered, x)
                    return gemm(gathered, w)

                def fused_ce():
                    arena.reset()
                    return comm.ag_gemm(x, w, via_copy_engine=True)

                def fused_direct():
                    arena.reset()
                    return comm.ag_gemm(x, w, via_copy_engine=False)

                flops = 2.0 * M * Ns * nk
                link = (world - 1) * rows * nk * 2
                res = {"fused_copy_engine_ms": timed(fused_ce, a.iters), "fused_direct_ms": timed(fused_direct, a.iters),
                       "library_ms": timed(lib, a.iters), "local_gemm_ms": timed(lambda: gemm(gathered, w), a.iters)}
                best = min(res["fused_copy_engine_ms"], res["fused_direct_ms"])
            else:
                h = (torch.randn(M, Ns, device=dev) * 0.1).to(torch.bfloat16)            # [M, K / tp]
                w = (torch.randn(nk, Ns, device=dev) * 0.02).to(torch.bfloat16)          # row shard [N, K / tp]
                scat = torch.empty(rows, nk, dtype=torch.bfloat16, device=dev)

                def lib():
                    dist.reduce_scatter_tensor(scat, gemm(h, w))
                    return scat

                def fused():
                    arena.reset()
                    return comm.gemm_rs(h, w)

                flops = 2.0 * M * Ns * nk
                link = (world - 1) * rows * nk * 2
                res = {"fused_ms": timed(fused, a.iters), "library_ms": timed(lib, a.iters),
                       "local_gemm_ms": timed(lambda: gemm(h, w), a.iters)}
                best = res["fused_ms"]
            roof = max(flops / (pk["bf16_tflops"] * 1e12), link / (NVLINK_GBS * 1e9)) * 1e3
            emit(rank, case=which, ranks=world, M=M, N=nk if which == "gemm_rs" else Ns, K=nk if which == "ag_gemm" else Ns,
                 roofline_ms=roof, fused_of_roofline=roof / best, speedup_vs_library=res["library_ms"] / best, **res)
            check_status(dev)
            if comm.watchdog is not None:
                comm.watchdog.close()
            arena.release_waits()
            del comm, arena


def case_dist_adamw(a, rank, world, dev):
    ext = _ext.load()
    pk = peaks()
    for mb in a.mb:
        n = (mb << 20) // 4 // (world * 64) * (world * 64)          # fp32 gradient elements
        per = n // world
        arena = SymmetricArena(dist.group.WORLD, n * 6 + (16 << 20), dev)
        grad = arena.alloc((n,), torch.float32, persistent=True)
        bf16 = arena.alloc((n,), torch.bfloat16, persistent=True)
        grad.normal_(0, 1e-3)
        master = torch.randn(n, device=dev)
        m, v = torch.zeros(per, device=dev), torch.zeros(per, device=dev)
        lo = rank * per

        def fused():
            arena.barrier()
            ext.dist_adamw_step(arena.peer_ptrs(grad), arena.peer_ptrs(bf16), master, m, v, lo, per, 1e-4, 0.9, 0.95, 1e-8,
                                0.1, 3, 1.0)
            arena.barrier()

        shard = torch.empty(per, device=dev)

        def lib():
            dist.reduce_scatter_tensor(shard, grad)
            ext.adamw_step(master[lo:lo + per], m, v, shard, bf16[lo:lo + per], 1e-4, 0.9, 0.95, 1e-8, 0.1, 3, 1.0)
            dist.all_gather_into_tensor(bf16, bf16[lo:lo + per])

        t_f, t_l = timed(fused, a.iters), timed(lib, a.iters)
        link = (world - 1) * per * 4 + (world - 1) * per * 2        # gradients in (fp32), working copy out (bf16), per GPU
        hbm = per * (4 + 4 * 6 + 2)                                  # own gradient, master + moments read and written, bf16
        roof = max(link / (NVLINK_GBS * 1e9), hbm / (pk["hbm_gbs"] * 1e9)) * 1e3
        emit(rank, case="dist_adamw", ranks=world, grad_mb=n * 4 / 2 ** 20, fused_ms=t_f, library_ms=t_l, roofline_ms=roof,
             fused_of_roofline=roof / t_f, speedup_vs_library=t_l / t_f)
        check_status(dev)
        del grad, bf16, arena


def case_small_sum(a, rank, world, dev):
    arena = SymmetricArena(dist.group.WORLD, 4 << 20, dev)
    peer = PeerDomain(arena)
    for n in (64, 768, 4096):
        x = torch.randn(n, device=dev)
        ref = x.clone()
        dist.all_reduce(ref)
        err = float((peer.all_reduce_small(x) - ref).abs().max().item())
        t_f = timed(lambda: peer.all_reduce_small(x), 50)
        t_n = timed(lambda: dist.all_reduce(x.clone()), 50)
        emit(rank, case="small_sum", ranks=world, n=n, fused_us=t_f * 1e3, nccl_us=t_n * 1e3, max_err=err)
    check_status(dev)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["halo", "ag_gemm", "gemm_rs", "dist_adamw", "small_sum"])
    ap.add_argument("--widths", type=int, nargs="+", default=[1440, 4320])
    ap.add_argument("--channels", type=int, nargs="+", default=[192, 384, 768])
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--tokens", type=int, nargs="+", default=[4096, 16384, 65536, 262144])
    ap.add_argument("--width", type=int, nargs="+", default=[1536, 3072])
    ap.add_argument("--mb", type=int, nargs="+", default=[16, 64, 256, 1024, 4096])
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    rank, world, dev = init_distributed(timeout_s=300)
    if world < 2:
        raise SystemExit("the communication microbenchmarks need at least two ranks (torch.distributed.run)")
    if a.case == "halo":
        case_halo(a, rank, world, dev)
    elif a.case in ("ag_gemm", "gemm_rs"):
        case_tp_gemm(a, rank, world, dev, a.case)
    elif a.case == "dist_adamw":
        case_dist_adamw(a, rank, world, dev)
    else:
        case_small_sum(a, rank, world, dev)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
