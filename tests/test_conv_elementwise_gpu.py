"""Implicit-GEMM convolution and the memory-bound kernels against fp32 PyTorch references."""
import pytest
import torch
import torch.nn.functional as TF

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


def _close(got, ref, rtol=2e-2, atol=2e-2):
    got, ref = got.float(), ref.float()
    err = (got - ref).abs().max().item()
    denom = ref.abs().max().item() + 1e-6
    assert err <= atol + rtol * denom, f"max abs err {err} vs ref max {denom}"


def _pack_w(w):
    """(Cout, Cin, 3, 3) -> [Cout, 9 * Cin_pad] tap-major bf16."""
    cout, cin = w.shape[:2]
    cpad = (cin + 63) // 64 * 64
    wp = torch.zeros(cout, 9, cpad, device=w.device, dtype=torch.bfloat16)
    wp[:, :, :cin] = w.permute(0, 2, 3, 1).reshape(cout, 9, cin).to(torch.bfloat16)
    return wp.reshape(cout, 9 * cpad).contiguous()


@pytest.mark.parametrize("B,H,W,Cin,Cout,stride", [(1, 16, 32, 64, 128, 1), (2, 13, 200, 96, 96, 1), (1, 32, 64, 384, 384, 1),
                                                    (1, 16, 32, 64, 64, 2), (1, 33, 272, 96, 96, 2), (1, 64, 128, 384, 384, 2)])
def test_conv3x3_fwd(B, H, W, Cin, Cout, stride):
    from terra_b200 import _ext
    from terra_b200.ops import _flags as F
    from terra_b200.ops.gemm import status_word, check_status

    torch.manual_seed(0)
    ext = _ext.load()
    x = _rand(B, H, W, Cin)
    w = _rand(Cout, Cin, 3, 3, scale=0.05)
    bias = _rand(Cout)
    Ho, Wo = (H, W) if stride == 1 else ((H + 1) // 2, W // 2)
    y = torch.empty(B, Ho, Wo, Cout, device="cuda", dtype=torch.bfloat16)
    ext.conv3x3_fwd(x, _pack_w(w), y, stride, F.EPI_BIAS, bias, None, status_word("cuda"), None, None)
    check_status("cuda")
    ref = TF.conv2d(x.float().permute(0, 3, 1, 2), w.float(), bias.float(), stride=stride, padding=1).permute(0, 2, 3, 1)
    _close(y, ref)


@pytest.mark.parametrize("B,H,W,Cin,Cout,stride", [(1, 16, 64, 64, 128, 1), (2, 13, 200, 96, 96, 1), (1, 16, 64, 128, 64, 2),
                                                    (1, 33, 272, 96, 96, 2), (1, 20, 136, 384, 384, 1), (1, 21, 144, 192, 128, 2)])
def test_conv3x3_wgrad(B, H, W, Cin, Cout, stride):
    from terra_b200 import _ext
    from terra_b200.ops.gemm import status_word, check_status

    torch.manual_seed(1)
    ext = _ext.load()
    x = _rand(B, H, W, Cin, scale=0.3)
    Ho, Wo = (H, W) if stride == 1 else ((H + 1) // 2, W // 2)
    dy = _rand(B, Ho, Wo, Cout, scale=0.3)
    dw = torch.zeros(9, Cout, Cin, device="cuda", dtype=torch.float32)
    db = torch.zeros(Cout, device="cuda")
    ext.conv3x3_wgrad(x, dy, dw, stride, 16, status_word("cuda"), None, None, bias_grad=db)
    check_status("cuda")
    _close(db, dy.float().sum((0, 1, 2)))
    xr = x.float().permute(0, 3, 1, 2).requires_grad_(False)
    wr = torch.zeros(Cout, Cin, 3, 3, device="cuda", requires_grad=True)
    TF.conv2d(xr, wr, None, stride=stride, padding=1).backward(dy.float().permute(0, 3, 1, 2))
    ref = wr.grad.permute(2, 3, 0, 1).reshape(9, Cout, Cin)
    _close(dw, ref)


@pytest.mark.parametrize("rows,C", [(1000, 96), (4097, 384), (300, 1536), (64, 192)])
def test_layernorm(rows, C):
    from terra_b200 import _ext

    torch.manual_seed(2)
    ext = _ext.load()
    x = _rand(rows, C) + 0.5
    g, b = _rand(C), _rand(C)
    y = torch.empty_like(x)
    mean = torch.empty(rows, device="cuda")
    rstd = torch.empty(rows, device="cuda")
    ext.layernorm_fwd(x, g, b, y, mean, rstd, 1e-5)
    xr = x.float().requires_grad_(True)
    gr, br = g.float().requires_grad_(True), b.float().requires_grad_(True)
    ref = TF.layer_norm(xr, (C,), gr, br, 1e-5)
    _close(y, ref)
    dy = _rand(rows, C)
    ref.backward(dy.float())
    dx = torch.empty_like(x)
    dg = torch.zeros(C, device="cuda")
    db = torch.zeros(C, device="cuda")
    ext.layernorm_bwd(dy, x, g, mean, rstd, dx, dg, db, None)
    _close(dx, xr.grad)
    _close(dg, gr.grad, rtol=3e-2, atol=5e-2)
    _close(db, br.grad, rtol=3e-2, atol=5e-2)


@pytest.mark.parametrize("B,HW,C", [(1, 5000, 96), (2, 3000, 384)])
def test_groupnorm_silu(B, HW, C):
    from terra_b200 import _ext

    torch.manual_seed(3)
    ext = _ext.load()
    G = 32
    x = _rand(B, HW, C) + 0.3
    g, b = _rand(C), _rand(C)
    sums = torch.zeros(B, G, 2, device="cuda")
    ext.groupnorm_stats(x, sums, G)
    n = HW * (C // G)
    mean = sums[..., 0] / n
    var = sums[..., 1] / n - mean * mean
    stats = torch.stack([mean, torch.rsqrt(var + 1e-5)], dim=-1).contiguous()
    y = torch.empty_like(x)
    ext.groupnorm_silu_apply(x, stats, g, b, None, y, G)
    xr = x.float().requires_grad_(True)
    gr, br = g.float().requires_grad_(True), b.float().requires_grad_(True)
    ref = TF.silu(TF.group_norm(xr.permute(0, 2, 1), G, gr, br, 1e-5)).permute(0, 2, 1)
    _close(y, ref)
    dy = _rand(B, HW, C)
    ref.backward(dy.float())
    red = torch.zeros(B, C, 2, device="cuda")
    ext.groupnorm_silu_bwd_reduce(dy, x, stats, g, b, red, G)
    dx = torch.empty_like(x)
    ext.groupnorm_silu_bwd_apply(dy, x, stats, red, g, b, dx, G, 1.0 / n)
    _close(dx, xr.grad, rtol=3e-2, atol=3e-2)
    _close(red[..., 0].sum(0), br.grad, rtol=3e-2, atol=1e-1)
    _close(red[..., 1].sum(0), gr.grad, rtol=3e-2, atol=1e-1)


def test_colsum_loss_adamw():
    from terra_b200 import _ext

    torch.manual_seed(4)
    ext = _ext.load()
    x = _rand(3001, 384)
    out = torch.zeros(384, device="cuda")
    ext.colsum(x, out)
    _close(out, x.float().sum(0), rtol=1e-2, atol=1e-1)

    pred, label = _rand(2, 64, 128), _rand(2, 64, 128)
    mask = (torch.rand(64, 128, device="cuda") > 0.3).to(torch.bfloat16)
    for kind in (0, 1):
        loss = torch.zeros(1, device="cuda")
        grad = torch.empty_like(pred)
        n = pred.numel()
        ext.masked_loss(pred, label, mask, kind, 1.0 / n, loss, grad)
        pr = pred.float().requires_grad_(True)
        d = pr * mask.float() - label.float()
        ref = d.abs().mean() if kind == 0 else (d * d).mean()
        ref.backward()
        _close(loss / n, ref.detach().reshape(1), rtol=1e-3, atol=1e-4)
        _close(grad, pr.grad, rtol=2e-2, atol=1e-6)

    n = 10007
    p = torch.randn(n, device="cuda")
    ref_p = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref_p], lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    for step in range(1, 4):
        gr = torch.randn(n, device="cuda")
        ref_p.grad = gr.clone()
        opt.step()
        ext.adamw_step(p, m, v, gr, pb, 1e-3, 0.9, 0.95, 1e-8, 0.1, step, 1.0)
    assert (p - ref_p.detach()).abs().max().item() < 1e-5
    _close(pb, p, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("stride", [1, 2])
def test_conv3x3_row_stripe_with_halo_rows(stride):
    """A stripe of a taller image convolved with its neighbours' boundary rows passed separately must equal the
    same rows of the whole-image convolution (forward and weight gradient)."""
    from terra_b200 import _ext
    from terra_b200.ops import _flags as F
    from terra_b200.ops.gemm import status_word, check_status

    torch.manual_seed(5)
    ext = _ext.load()
    B, H, W, Cin, Cout = 1, 24, 72, 64, 64
    x = _rand(B, H, W, Cin, scale=0.5)
    w = _rand(Cout, Cin, 3, 3, scale=0.05)
    bias = _rand(Cout)
    r0, r1 = 8, 16                                   # the middle stripe
    xs = x[:, r0:r1].contiguous()
    lo, hi = x[:, r0 - 1:r0].contiguous(), x[:, r1:r1 + 1].contiguous()
    ho = (r1 - r0) // stride
    y = torch.empty(B, ho, W // stride, Cout, device="cuda", dtype=torch.bfloat16)
    ext.conv3x3_fwd(xs, _pack_w(w), y, stride, F.EPI_BIAS, bias, None, status_word("cuda"), lo, hi)
    check_status("cuda")
    xr = x.float().permute(0, 3, 1, 2)
    ref = TF.conv2d(xr, w.float(), bias.float(), stride=stride, padding=1).permute(0, 2, 3, 1)
    _close(y, ref[:, r0 // stride:r1 // stride])

    dy_full = torch.zeros(B, H // stride, W // stride, Cout, device="cuda")
    dy = _rand(B, ho, W // stride, Cout, scale=0.3)
    dy_full[:, r0 // stride:r1 // stride] = dy.float()
    dw = torch.zeros(9, Cout, Cin, device="cuda")
    ext.conv3x3_wgrad(xs, dy, dw, stride, 4, status_word("cuda"), lo, hi)
    check_status("cuda")
    wr = torch.zeros(Cout, Cin, 3, 3, device="cuda", requires_grad=True)
    TF.conv2d(xr, wr, None, stride=stride, padding=1).backward(dy_full.permute(0, 3, 1, 2))
    _close(dw, wr.grad.permute(2, 3, 0, 1).reshape(9, Cout, Cin))
