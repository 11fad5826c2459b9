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
