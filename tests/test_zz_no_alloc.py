"""The allocation-free GroupNorm+SiLU entry point, called through its exported C symbol.

Some users of the library run where device allocation is forbidden (inside another framework's memory pool, in a
loop that bans cudaMalloc after start-up); ``terra_groupnorm_silu_noalloc`` serves them with a scratch array built
into the library. This test loads the shared object with ctypes, calls the symbol twice in a row on different
inputs (the scratch keeps the previous call's contents, so the second call checks that it is cleared) and compares
with the regular two-kernel path of the extension.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular(ext, x, g, b, groups, eps):
    B, HW, C = x.shape
    sums = torch.zeros(B, groups, 2, device="cuda")
    ext.groupnorm_stats(x, sums, groups)
    n = HW * (C // groups)
    mean = sums[..., 0] / n
    var = (sums[..., 1] / n - mean * mean).clamp_min(0)
    stats = torch.stack([mean, torch.rsqrt(var + eps)], dim=-1).contiguous()
    y = torch.empty_like(x)
    ext.groupnorm_silu_apply(x, stats, g, b, None, y, groups)
    return y


def test_noalloc_groupnorm_silu_matches_regular_path_twice():
    from terra_b200 import _ext

    ext = _ext.load()
    lib = ctypes.CDLL(ext.__file__)
    fn = lib.terra_groupnorm_silu_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong,
                   ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p]
    torch.manual_seed(0)
    groups, eps = 32, 1e-5
    stream = torch.cuda.current_stream().cuda_stream
    for call, (B, HW, C, shift) in enumerate([(2, 3000, 384, 0.3), (1, 5000, 96, -1.5)]):
        x = (torch.randn(B, HW, C, device="cuda") * (1.0 + call) + shift).to(torch.bfloat16)
        g = torch.randn(C, device="cuda").to(torch.bfloat16)
        b = torch.randn(C, device="cuda").to(torch.bfloat16)
        y = torch.empty_like(x)
        before = torch.cuda.memory_allocated()
        rc = fn(x.data_ptr(), g.data_ptr(), b.data_ptr(), y.data_ptr(), B, HW, C, groups, eps, stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        ref = _regular(ext, x, g, b, groups, eps)
        err = (y.float() - ref.float()).abs().max().item()
        assert err <= 2e-2 + 2e-2 * ref.float().abs().max().item(), (call, err)
    # sizes beyond the built-in scratch are refused, nothing is launched
    big = torch.empty(200, 8, 32, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(32, device="cuda", dtype=torch.bfloat16)
    assert fn(big.data_ptr(), w.data_ptr(), w.data_ptr(), big.data_ptr(), 200, 8, 32, 32, eps, stream) == -2
