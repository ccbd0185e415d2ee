"""Window attention kernels (forward and backward) against the PyTorch fp32 reference of the same op: the mma.sync
kernel (windows of at most 128 tokens) and the tcgen05 / TMEM kernels (any window size: two small windows per tile, or
flash-style K/V streaming with a two-pass backward for large windows)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(got, ref, rtol=3e-2, atol=3e-2):
    got, ref = got.float(), ref.float()
    err = (got - ref).abs().max().item()
    denom = ref.abs().max().item() + 1e-6
    assert err <= atol + rtol * denom, f"max abs err {err} vs ref max {denom}"


@pytest.mark.parametrize("B,nWh,nWw,wh,ww,C,heads,shifted,use_bias", [
    (1, 2, 4, 8, 8, 96, 3, False, True),
    (1, 2, 4, 8, 8, 96, 3, True, True),
    (2, 3, 5, 8, 8, 192, 12, True, True),
    (1, 3, 4, 8, 12, 192, 6, True, True),
    (1, 4, 4, 8, 8, 384, 6, True, False),
    (1, 2, 3, 8, 8, 256, 2, True, True),
    (1, 3, 3, 7, 7, 64, 2, True, True),
])
def test_window_attention_fwd_bwd(B, nWh, nWw, wh, ww, C, heads, shifted, use_bias):
    from terra_b200.ops.attention import WindowGeometry, window_attention, window_attention_reference

    torch.manual_seed(0)
    geo = WindowGeometry(B, nWh, nWw, wh, ww)
    N, nW = wh * ww, nWh * nWw
    qkv = (torch.randn(B * nW * N, 3 * C, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    table = (torch.randn((2 * wh - 1) * (2 * ww - 1), heads, device="cuda") * 0.2).requires_grad_(True) if use_bias else None
    scale = (C // heads) ** -0.5
    out = window_attention(qkv, geo, heads, shifted, table, True, scale)
    dout = (torch.randn_like(out.float()) * 0.5).to(torch.bfloat16)
    out.backward(dout)

    q32 = qkv.detach().float().requires_grad_(True)
    t32 = table.detach().clone().requires_grad_(True) if use_bias else None
    ref = window_attention_reference(q32.reshape(B, nW, N, 3 * C), geo, heads, shifted, t32, True, scale).reshape(-1, C)
    ref.backward(dout.float())
    _close(out, ref)
    _close(qkv.grad, q32.grad)
    if use_bias:
        _close(table.grad, t32.grad, rtol=3e-2, atol=5e-2)


def _run_case(B, nWh, nWw, wh, ww, C, heads, shifted, use_bias):
    from terra_b200.ops.attention import WindowGeometry, window_attention, window_attention_reference

    torch.manual_seed(0)
    geo = WindowGeometry(B, nWh, nWw, wh, ww)
    N, nW = wh * ww, nWh * nWw
    qkv = (torch.randn(B * nW * N, 3 * C, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    table = (torch.randn((2 * wh - 1) * (2 * ww - 1), heads, device="cuda") * 0.2).requires_grad_(True) if use_bias else None
    scale = (C // heads) ** -0.5
    out = window_attention(qkv, geo, heads, shifted, table, True, scale)
    dout = (torch.randn_like(out.float()) * 0.5).to(torch.bfloat16)
    out.backward(dout)
    q32 = qkv.detach().float().requires_grad_(True)
    t32 = table.detach().clone().requires_grad_(True) if use_bias else None
    ref = window_attention_reference(q32.reshape(B, nW, N, 3 * C), geo, heads, shifted, t32, True, scale).reshape(-1, C)
    ref.backward(dout.float())
    _close(out, ref)
    _close(qkv.grad, q32.grad)
    if use_bias:
        _close(table.grad, t32.grad, rtol=3e-2, atol=5e-2)


@pytest.mark.parametrize("B,nWh,nWw,wh,ww,C,heads,shifted,use_bias", [
    (1, 3, 3, 7, 7, 64, 2, True, True),          # N = 49: padded keys inside a 64-key slot
    (1, 2, 4, 8, 8, 128, 4, False, True),        # N = 64, unshifted
    (2, 3, 5, 8, 8, 192, 12, True, True),        # N = 64, head dim 16, odd window count (a tile with one window)
    (1, 2, 3, 8, 8, 128, 2, True, False),        # head dim 64, no bias
])
def test_tensor_core_kernels_on_small_windows(monkeypatch, B, nWh, nWw, wh, ww, C, heads, shifted, use_bias):
    """The tcgen05 forward and backward (two windows per 128-row tile), selected instead of the default mma.sync path."""
    monkeypatch.setenv("TERRA_ATTN_FWD", "tc")
    monkeypatch.setenv("TERRA_ATTN_BWD", "tc")
    _run_case(B, nWh, nWw, wh, ww, C, heads, shifted, use_bias)


@pytest.mark.parametrize("B,nWh,nWw,wh,ww,C,heads,shifted,use_bias", [
    (1, 2, 2, 8, 12, 64, 2, True, True),         # N = 96: forward on tensor cores, backward on the mma.sync kernel
    (1, 2, 3, 12, 12, 64, 4, True, True),        # N = 144: two query blocks, three key slots, ragged tail
    (1, 1, 2, 32, 32, 64, 2, True, True),        # N = 1024 (window size of the reference's correctness config)
    (1, 2, 1, 32, 32, 64, 1, False, False),      # N = 1024, head dim 64, no bias, unshifted
])
def test_large_windows_forward_and_two_pass_backward(monkeypatch, B, nWh, nWw, wh, ww, C, heads, shifted, use_bias):
    monkeypatch.setenv("TERRA_ATTN_FWD", "tc")
    _run_case(B, nWh, nWw, wh, ww, C, heads, shifted, use_bias)


def test_large_window_attention_on_cuda():
    """144-token windows (above the shared-memory kernel's 128) run on the tensor-core kernels, forward and backward."""
    from terra_b200.ops.attention import WindowGeometry, window_attention, window_attention_reference

    torch.manual_seed(3)
    B, nWh, nWw, w, C, heads = 1, 2, 3, 12, 64, 4
    geo = WindowGeometry(B, nWh, nWw, w, w)
    N, nW = w * w, nWh * nWw
    qkv = (torch.randn(B * nW * N, 3 * C, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    table = (torch.randn((2 * w - 1) ** 2, heads, device="cuda") * 0.2).requires_grad_(True)
    out = window_attention(qkv, geo, heads, True, table, True, (C // heads) ** -0.5)
    dout = (torch.randn_like(out.float()) * 0.5).to(torch.bfloat16)
    out.backward(dout)
    q32 = qkv.detach().float().requires_grad_(True)
    t32 = table.detach().clone().requires_grad_(True)
    ref = window_attention_reference(q32.reshape(B, nW, N, 3 * C), geo, heads, True, t32, True, (C // heads) ** -0.5).reshape(-1, C)
    ref.backward(dout.float())
    _close(out, ref)
    _close(qkv.grad, q32.grad)
    _close(table.grad, t32.grad, rtol=3e-2, atol=5e-2)
