"""The allocation-free GroupNorm+SiLU entry point, called through its exported C symbol.

Some users of the library run where device allocation is forbidden (inside another framework's memory pool, in a
loop that bans cudaMalloc after start-up); ``terra_groupnorm_silu_noalloc`` serves them with a scratch array built
into the library. This test loads the shared object with ctypes, calls the symbol twice in a row on different
inputs (the scratch keeps the previous call's contents, so the second call checks that it is cleared) and compares
with the regular two-kernel path of the extension and with PyTorch's fp32 ``group_norm`` + ``silu``. "Allocates
nothing" is checked twice: PyTorch's caching allocator saw no request, and the driver's free-memory figure
(``cudaMemGetInfo``, which a raw ``cudaMalloc`` inside the library would move) is unchanged.
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
        if call == 0:
            # the very first call on a device resolves the scratch address; take the driver's figure after it
            assert fn(x.data_ptr(), g.data_ptr(), b.data_ptr(), y.data_ptr(), B, HW, C, groups, eps, stream) == 0
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(x.data_ptr(), g.data_ptr(), b.data_ptr(), y.data_ptr(), B, HW, C, groups, eps, stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] == free_before
        ref = _regular(ext, x, g, b, groups, eps)
        err = (y.float() - ref.float()).abs().max().item()
        assert err <= 2e-2 + 2e-2 * ref.float().abs().max().item(), (call, err)
        xt = x.float().permute(0, 2, 1)                                   # [B, C, HW]
        ref32 = torch.nn.functional.silu(torch.nn.functional.group_norm(xt, groups, g.float(), b.float(), eps)).permute(0, 2, 1)
        err32 = (y.float() - ref32).abs().max().item()
        assert err32 <= 2e-2 + 2e-2 * ref32.abs().max().item(), (call, err32)
    # sizes beyond the built-in scratch are refused, nothing is launched
    big = torch.empty(200, 8, 32, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(32, device="cuda", dtype=torch.bfloat16)
    assert fn(big.data_ptr(), w.data_ptr(), w.data_ptr(), big.data_ptr(), 200, 8, 32, 32, eps, stream) == -2
