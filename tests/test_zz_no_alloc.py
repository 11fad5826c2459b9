"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some users of the library run in places where device allocation is forbidden (inside another
framework's allocator callback, or in a plugin hook invoked while the allocator is locked), so
``b200_rmsnorm_bwd_noalloc`` keeps its fp32 staging rows in a fixed device array of the library
image.  This test calls the symbol directly with ctypes, twice in a row (the second call reuses the
staging rows the first one left behind), and compares against the regular entry point, which takes
a caller-allocated staging buffer.  This file sorts last so a run that stops at the first failure
has already run everything else.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from aws_ofi_nccl_b200.ops import _lib as L

    lib = C.CDLL(str(L.lib_path()))
    vp, i = C.c_void_p, C.c_int
    lib.b200_rmsnorm_bwd_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, i, vp]
    lib.b200_rmsnorm_bwd_noalloc.restype = i
    lib.b200_rmsnorm_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, vp]
    lib.b200_rmsnorm_bwd.restype = i
    lib.b200_rmsnorm_bwd_partial_rows.restype = i
    return lib


def _reference(dy, x, w, rstd, dres, dw_before):
    """The same backward in plain fp32 PyTorch: y = x * rstd * w."""
    dy32, x32, w32 = dy.float(), x.float(), w.float()
    xhat = x32 * rstd[:, None]
    g = dy32 * w32
    dx = rstd[:, None] * (g - xhat * (g * xhat).mean(-1, keepdim=True))
    if dres is not None:
        dx = dx + dres.float()
    dw = (dy32 * xhat).sum(0)
    if dw_before is not None:
        dw = dw + dw_before.float()
    return dx, dw


def _case(lib, T, H, with_res, seed, accumulate=False):
    torch.manual_seed(seed)
    dev = "cuda"
    dy = torch.randn(T, H, device=dev).bfloat16()
    x = torch.randn(T, H, device=dev).bfloat16()
    w = (1 + 0.1 * torch.randn(H, device=dev)).bfloat16()
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
    dres = torch.randn(T, H, device=dev).bfloat16() if with_res else None
    stream = torch.cuda.current_stream().cuda_stream
    # existing entry point: caller allocates the staging rows
    partial = torch.empty(lib.b200_rmsnorm_bwd_partial_rows(), H, device=dev, dtype=torch.float32)
    dw_start = (0.5 * torch.randn(H, device=dev)).bfloat16()   # what dw holds before an accumulating call
    dx_ref, dw_ref = torch.empty_like(x), dw_start.clone()
    rc = lib.b200_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                              dres.data_ptr() if with_res else None, dx_ref.data_ptr(), partial.data_ptr(),
                              dw_ref.data_ptr(), int(accumulate), T, H, stream)
    assert rc == 0
    dx, dw = torch.empty_like(x), dw_start.clone()
    before = torch.cuda.memory_allocated()
    rc = lib.b200_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                      dres.data_ptr() if with_res else None, dx.data_ptr(), dw.data_ptr(),
                                      int(accumulate), T, H, stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    # against the entry point that takes a caller-allocated staging buffer ...
    for got, ref in ((dx, dx_ref), (dw, dw_ref)):
        err = (got.float() - ref.float()).abs().max().item()
        assert err <= 2e-2 * ref.float().abs().max().item() + 2e-2, err
    # ... and against the same maths in plain fp32 PyTorch (a mistake shared by both kernels would pass the first)
    dx32, dw32 = _reference(dy, x, w, rstd, dres, dw_start if accumulate else None)
    for got, ref in ((dx, dx32), (dw, dw32)):
        err = (got.float() - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item() + 2e-2, err


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    lib = _lib()
    _case(lib, 300, 4096, True, 1)    # first call: performs the per-device address lookup
    _case(lib, 64, 1024, False, 2)    # second call: smaller shape over the rows the first one left
    _case(lib, 1000, 8192, True, 3)   # largest hidden size the fixed area serves
    _case(lib, 200, 2048, False, 4, accumulate=True)   # dw += instead of dw =


def test_noalloc_rejects_sizes_beyond_the_fixed_area():
    lib = _lib()
    t = torch.zeros(16, device="cuda")
    p = t.data_ptr()
    assert lib.b200_rmsnorm_bwd_noalloc(p, p, p, p, None, p, p, 0, 4, 8192 + 8, None) == 10004
    assert lib.b200_rmsnorm_bwd_noalloc(p, p, p, p, None, p, p, 0, 4, 100, None) == 10001
    # a pointer that is not 16-byte aligned is refused on the host instead of faulting on the device
    assert lib.b200_rmsnorm_bwd_noalloc(p + 2, p, p, p, None, p, p, 0, 2, 8, None) == 10001
