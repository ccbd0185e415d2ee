"""Worker of the fused tensor-parallel tests (torch.distributed.run, one rank per GPU): all-gather -> GEMM,
GEMM -> reduce-scatter and the sequence-sharded MLP (forward and backward) against plain PyTorch collectives + fp32
matmuls. (Timings of the same kernels: ``python -m terra_b200.ops.microbench_comm ag_gemm|gemm_rs``.)"""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    from terra_b200.distributed import init_distributed
    from terra_b200.ops.gemm import check_status, gemm
    from terra_b200.ops.tp_fused import TpFusedComm, tp_mlp
    from terra_b200.parallel.nvlink import SymmetricArena

    rank, world, dev = init_distributed(timeout_s=120)     # a rank that fails must not keep the others waiting long
    arena = SymmetricArena(dist.group.WORLD, 256 << 20, dev)
    comm = TpFusedComm(arena)
    x_sym = None
    torch.manual_seed(5)                      # same weights and global activations on every rank
    rows, C, F = 328, 256, 512    # rows per rank; 328 is not a tile multiple
    Fs = F // world
    x_full = (torch.randn(rows * world, C, device=dev) * 0.5).to(torch.bfloat16)
    w1 = (torch.randn(F, C, device=dev) * 0.05).to(torch.bfloat16)
    b1 = (torch.randn(F, device=dev) * 0.1).to(torch.bfloat16)
    w2 = (torch.randn(C, F, device=dev) * 0.05).to(torch.bfloat16)
    x = x_full[rank * rows:(rank + 1) * rows].contiguous()
    x_sym = arena.alloc((rows, C), torch.bfloat16, persistent=True)      # an activation produced in symmetric memory
    x_sym.copy_(x)
    w1s, b1s, w2s = w1[rank * Fs:(rank + 1) * Fs].contiguous(), b1[rank * Fs:(rank + 1) * Fs].contiguous(), \
        w2[:, rank * Fs:(rank + 1) * Fs].contiguous()
    res = {}

    def rel(a, b):
        return float((a.detach().float() - b.detach().float()).abs().max() / (b.detach().float().abs().max() + 1e-6))

    # ---- all-gather -> GEMM
    ag_ref = x_full.float() @ w1s.float().t() + b1s.float()
    res["ag_gemm"] = rel(comm.ag_gemm(x, w1s, bias=b1s, via_copy_engine=False), ag_ref)
    res["ag_gemm_copy_engine"] = rel(comm.ag_gemm(x, w1s, bias=b1s, via_copy_engine=True), ag_ref)
    # ---- GEMM -> reduce-scatter
    h_full = (torch.randn(rows * world, F, device=dev) * 0.3).to(torch.bfloat16)
    hs = h_full[:, rank * Fs:(rank + 1) * Fs].contiguous()
    ref = (h_full.float() @ w2.float().t())[rank * rows:(rank + 1) * rows]
    res["gemm_rs"] = rel(comm.gemm_rs(hs, w2s), ref)
    res["gemm_rs_exact"] = rel(comm.gemm_rs(hs, w2s, exact=True), ref)
    arena.reset()
    # ---- MLP forward / backward
    xr = x.clone().requires_grad_(True)
    p = [t.clone().requires_grad_(True) for t in (w1s, b1s, w2s)]
    out = tp_mlp(xr, p[0], p[1], p[2], comm)
    dout = (torch.randn(rows * world, C, device=dev) * 0.2).to(torch.bfloat16)
    out.backward(dout[rank * rows:(rank + 1) * rows].contiguous())
    xf = x_full.float().requires_grad_(True)
    pf = [t.float().requires_grad_(True) for t in (w1, b1, w2)]
    full = torch.nn.functional.gelu(xf @ pf[0].t() + pf[1]) @ pf[2].t()
    full.backward(dout.float())
    res["mlp_out"] = rel(out, full[rank * rows:(rank + 1) * rows])
    res["mlp_dx"] = rel(xr.grad, xf.grad[rank * rows:(rank + 1) * rows])
    res["mlp_dw1"] = rel(p[0].grad, pf[0].grad[rank * Fs:(rank + 1) * Fs])
    res["mlp_db1"] = rel(p[1].grad, pf[1].grad[rank * Fs:(rank + 1) * Fs])
    res["mlp_dw2"] = rel(p[2].grad, pf[2].grad[:, rank * Fs:(rank + 1) * Fs])
    check_status(dev)

    if rank == 0:
        print("RESULT " + json.dumps(res), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except BaseException:
        import traceback

        traceback.print_exc()
        sys.stdout.flush()
        os._exit(1)          # leave at once: the peers' collectives then end with the process-group timeout
