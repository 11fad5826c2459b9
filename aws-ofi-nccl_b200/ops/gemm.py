"""tcgen05 GEMM bindings and the autograd ``linear`` built on them.

``gemm`` exposes the kernel's storage flags directly (see csrc/kernels/gemm.cu); ``linear`` maps
a linear layer's forward, input-gradient and weight-gradient products onto them so no transpose
is ever materialised.
"""
from __future__ import annotations

import torch

from . import _lib


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16,
         accumulate: bool = False, bn: int = 0, max_ctas: int = 0) -> torch.Tensor:
    """C[M,N] (+)= op(A) op(B) with bf16 operands and fp32 accumulation.

    a is [M,K] (a_mn=False) or [K,M] (a_mn=True); b is [N,K] (b_mn=False) or [K,N] (b_mn=True).
    Rows may be strided (last dim contiguous).
    """
    assert a.is_cuda and b.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"reduction dims differ: {K} vs {Kb}"
    if out is None:
        assert not accumulate
        out = torch.empty((M, N), device=a.device, dtype=out_dtype)
    assert out.shape == (M, N) and out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    rc = _lib.load().b200_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
        int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate), bn, max_ctas, _lib.stream_ptr())
    _lib.check(rc, "b200_gemm_bf16")
    return out


def quantize_rows_fp8(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 [R, K] -> (e4m3 [R, K], fp32 scale [R]) with one scale per row: x ~= q * scale[:, None]."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    R, K = x.shape
    q = torch.empty((R, K), device=x.device, dtype=torch.float8_e4m3fn)
    scale = torch.empty(R, device=x.device, dtype=torch.float32)
    _lib.check(_lib.load().b200_quant_rows_fp8(x.data_ptr(), q.data_ptr(), scale.data_ptr(), R, K, x.stride(0), q.stride(0),
                                               _lib.stream_ptr()), "b200_quant_rows_fp8")
    return q, scale


def gemm_fp8(a8: torch.Tensor, b8: torch.Tensor, a_scale: torch.Tensor, b_scale: torch.Tensor,
             out: torch.Tensor | None = None) -> torch.Tensor:
    """C[M,N] (bf16) = (a8[M,K] @ b8[N,K]^T) * a_scale[:, None] * b_scale[None, :] with e4m3 operands,
    fp32 accumulation in TMEM and the dequantisation fused into the epilogue (M >= 256, N >= 128)."""
    assert a8.dtype == torch.float8_e4m3fn and b8.dtype == torch.float8_e4m3fn
    assert a8.stride(1) == 1 and b8.stride(1) == 1 and a8.shape[1] == b8.shape[1]
    M, K = a8.shape
    N = b8.shape[0]
    assert a_scale.shape == (M,) and b_scale.shape == (N,) and a_scale.dtype == b_scale.dtype == torch.float32
    if out is None:
        out = torch.empty((M, N), device=a8.device, dtype=torch.bfloat16)
    assert out.shape == (M, N) and out.dtype == torch.bfloat16 and out.stride(1) == 1
    _lib.check(_lib.load().b200_gemm_fp8(a8.data_ptr(), b8.data_ptr(), a_scale.data_ptr(), b_scale.data_ptr(),
                                         out.data_ptr(), M, N, K, a8.stride(0), b8.stride(0), out.stride(0),
                                         _lib.stream_ptr()), "b200_gemm_fp8")
    return out


class _Linear(torch.autograd.Function):
    """y = x W^T.  The weight gradient is written straight into ``weight.main_grad`` when the
    parameter has one (a view of the flat gradient buffer), and the ``grad_ready`` hook of the
    parameter is called so a data-parallel engine can start reducing that bucket at once."""

    @staticmethod
    def forward(ctx, x, weight):
        ctx.save_for_backward(x, weight)
        x2 = x.reshape(-1, x.shape[-1])
        # allocate with the final shape: a custom Function must not return a view it created,
        # or later in-place ops on the output (RoPE) are refused by autograd
        y = torch.empty((*x.shape[:-1], weight.shape[0]), device=x.device, dtype=torch.bfloat16)
        gemm(x2, weight, out=y.view(-1, weight.shape[0]))
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).view_as(x)
        dw = None
        if ctx.needs_input_grad[1]:
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                fresh = not getattr(weight, "grad_written", False)
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main_grad, accumulate=not fresh)
                weight.grad_written = True
                hook = getattr(weight, "grad_ready", None)
                if hook is not None:
                    hook(weight)
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True)
        return dx, dw


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    return _Linear.apply(x, weight)
