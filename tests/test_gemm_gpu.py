"""tcgen05 GEMM family against fp32 PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


def _close(got, ref, rtol=2e-2, atol=2e-2):
    got = got.float()
    ref = ref.float()
    err = (got - ref).abs().max().item()
    denom = ref.abs().max().item() + 1e-6
    assert err <= atol + rtol * denom, f"max abs err {err} vs ref max {denom}"


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 384, 384), (1000, 1152, 384), (515, 200, 1000), (4096, 1536, 384)])
def test_gemm_kmajor(M, N, K):
    from terra_b200.ops.gemm import gemm, check_status

    torch.manual_seed(0)
    a, b = _rand(M, K), _rand(N, K, scale=0.05)
    c = gemm(a, b)
    check_status("cuda")
    _close(c, a.float() @ b.float().t())


@pytest.mark.parametrize("bn", [64, 128, 192, 256])
def test_gemm_tile_widths(bn):
    from terra_b200.ops.gemm import gemm, check_status

    torch.manual_seed(1)
    a, b = _rand(777, 512), _rand(520, 512, scale=0.05)
    c = gemm(a, b, bn=bn)
    check_status("cuda")
    _close(c, a.float() @ b.float().t())


def test_gemm_epilogues():
    from terra_b200.ops.gemm import gemm, check_status

    torch.manual_seed(2)
    M, N, K = 900, 768, 384
    a, b = _rand(M, K), _rand(N, K, scale=0.05)
    bias = _rand(N)
    res = _rand(M, N)
    ref = a.float() @ b.float().t() + bias.float()
    out, pre = gemm(a, b, bias=bias, gelu=True, save_pre=True)
    check_status("cuda")
    _close(pre, ref)
    _close(out, torch.nn.functional.gelu(ref))
    out2 = gemm(a, b, bias=bias, residual=res)
    _close(out2, ref + res.float())
    aux = _rand(M, N)
    out3 = gemm(a, b, dgelu_aux=aux)
    x = aux.float().requires_grad_(True)
    torch.nn.functional.gelu(x).sum().backward()
    _close(out3, (a.float() @ b.float().t()) * x.grad)
    check_status("cuda")


@pytest.mark.parametrize("M,N,K,bn", [(40000, 800, 128, 128), (33001, 384, 384, 192), (20010, 1536, 384, 256),
                                      (3000, 64, 64, 0), (29000, 416, 256, 192)])
def test_gemm_epilogues_over_many_tiles(M, N, K, bn):
    """Every CTA runs several tiles (the epilogue's operand prefetch crosses tile boundaries), the last row tile is
    ragged and, where N is not a multiple of the tile width, the last column tile is narrow."""
    from terra_b200.ops.gemm import gemm, check_status

    torch.manual_seed(5)
    a, b = _rand(M, K), _rand(N, K, scale=0.05)
    bias, res, aux = _rand(N), _rand(M, N), _rand(M, N)
    acc = a.float() @ b.float().t()
    ref = acc + bias.float()
    out, pre = gemm(a, b, bias=bias, gelu=True, save_pre=True, bn=bn)
    _close(pre, ref)
    _close(out, torch.nn.functional.gelu(ref))
    _close(gemm(a, b, bias=bias, residual=res, bn=bn), ref + res.float())
    _close(gemm(a, b, bias=bias, bn=bn), ref)
    x = aux.float().requires_grad_(True)
    torch.nn.functional.gelu(x).sum().backward()
    _close(gemm(a, b, dgelu_aux=aux, bn=bn), acc * x.grad)
    view = torch.zeros(M, N + 64, device="cuda", dtype=torch.bfloat16)      # output rows with a pitch wider than N
    gemm(a, b, bias=bias, out=view[:, 32:32 + N], bn=bn)
    _close(view[:, 32:32 + N], ref)
    assert float(view[:, :32].abs().max()) == 0.0 and float(view[:, 32 + N:].abs().max()) == 0.0
    check_status("cuda")


def test_gemm_dgrad_b_mnmajor():
    from terra_b200.ops.gemm import gemm, check_status

    torch.manual_seed(3)
    M, N, K = 1030, 1536, 384   # dx[M,K] = dy[M,N] @ W[N,K]
    dy, w = _rand(M, N), _rand(N, K, scale=0.05)
    dx = gemm(dy, w, b_mn=True)
    check_status("cuda")
    _close(dx, dy.float() @ w.float())


@pytest.mark.parametrize("split_k", [1, 7, 64])
def test_gemm_wgrad_both_mnmajor(split_k):
    from terra_b200.ops.gemm import gemm, check_status

    torch.manual_seed(4)
    M, N, K = 5000, 384, 1536   # dW[N,K] = dy[M,N]^T @ x[M,K]
    dy, x = _rand(M, N, scale=0.1), _rand(M, K, scale=0.1)
    dw = gemm(dy, x, a_mn=True, b_mn=True, split_k=split_k, out_f32=True)
    check_status("cuda")
    _close(dw, dy.float().t() @ x.float())


@pytest.mark.parametrize("M,N,K,bn,split_k", [(5000, 384, 1536, 192, 7), (3000, 1152, 384, 192, 1), (4100, 200, 96, 128, 5),
                                              (2000, 48, 64, 64, 3)])
def test_gemm_wgrad_with_fused_column_sums(M, N, K, bn, split_k):
    """dW = dy^T x and, from the same kernel, db = column sums of dy (a 16-column MMA of the dy tiles against ones)."""
    from terra_b200.ops.gemm import gemm, check_status

    torch.manual_seed(6)
    dy, x = _rand(M, N, scale=0.1), _rand(M, K, scale=0.1)
    dw = torch.zeros(N, K, device="cuda")
    db = torch.full((N,), 0.5, device="cuda")          # accumulated into, not overwritten
    gemm(dy, x, a_mn=True, b_mn=True, out=dw, accumulate=True, split_k=split_k, bn=bn, colsum=db)
    check_status("cuda")
    _close(dw, dy.float().t() @ x.float())
    _close(db, 0.5 + dy.float().sum(0))


def test_gemm_large_matches_and_times():
    from terra_b200.ops.gemm import gemm, check_status

    torch.manual_seed(5)
    M, N, K = 8192, 8192, 8192
    a, b = _rand(M, K, scale=0.05), _rand(N, K, scale=0.05)
    c = gemm(a, b, bn=256)
    check_status("cuda")
    ref = a @ b.t()
    _close(c, ref, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("bn", [128, 192, 256])
def test_gemm_mn_major_operands_tile_widths(bn):
    """Input-gradient form (B read untransposed) and weight-gradient form (both operands MN-major, split-K fp32
    accumulation) at every tile width."""
    from terra_b200.ops.gemm import gemm, check_status

    torch.manual_seed(7)
    M, N, K = 1000, 384, 768
    dy, w = _rand(M, K, scale=0.2), _rand(K, N, scale=0.05)      # dx[M, N] = dy[M, K] @ w[K, N]
    dx = gemm(dy, w, b_mn=True, bn=bn)
    check_status("cuda")
    _close(dx, dy.float() @ w.float())
    x = _rand(M, N, scale=0.2)
    gw = torch.zeros(K, N, device="cuda")                        # gw[K, N] = dy^T x
    gemm(dy, x, a_mn=True, b_mn=True, out=gw, accumulate=True, split_k=4, bn=bn)
    check_status("cuda")
    _close(gw, dy.float().t() @ x.float())


@pytest.mark.parametrize("bn", [1128, 1256])
def test_gemm_cta_pair(bn):
    """Pair mode (a cluster of two CTAs drives one 256-row MMA): forward, input-gradient and weight-gradient forms and
    the fused epilogues, with M not a multiple of 256 and N not a multiple of the tile width."""
    from terra_b200.ops.gemm import gemm, check_status

    torch.manual_seed(11)
    M, N, K = 1000, 640, 448
    a, w = _rand(M, K, scale=0.3), _rand(N, K, scale=0.05)
    bias, res = _rand(N), _rand(M, N)
    c = gemm(a, w, bn=bn)
    check_status("cuda")
    _close(c, a.float() @ w.float().t())
    c = gemm(a, w, bias=bias, residual=res, bn=bn)
    check_status("cuda")
    _close(c, a.float() @ w.float().t() + bias.float() + res.float())
    act, pre = gemm(a, w, bias=bias, gelu=True, save_pre=True, bn=bn)
    check_status("cuda")
    ref = a.float() @ w.float().t() + bias.float()
    _close(pre, ref)
    _close(act, torch.nn.functional.gelu(ref))
    dy = _rand(M, N, scale=0.2)
    dx = gemm(dy, w, b_mn=True, bn=bn)                      # dx[M, K] = dy[M, N] @ w[N, K]
    check_status("cuda")
    _close(dx, dy.float() @ w.float())
    gw = torch.zeros(N, K, device="cuda")
    gemm(dy, a, a_mn=True, b_mn=True, out=gw, accumulate=True, split_k=3, bn=bn)
    check_status("cuda")
    _close(gw, dy.float().t() @ a.float())
