"""Autograd wrappers of the bandwidth-bound Llama kernels (csrc/kernels/llm_ops.cu)."""
from __future__ import annotations

import torch

from . import _lib

_scratch: dict = {}


def _dw_partial(device, H: int) -> torch.Tensor:
    rows = _lib.load().b200_rmsnorm_bwd_partial_rows()
    key = (device, H)
    buf = _scratch.get(key)
    if buf is None or buf.shape[0] < rows:
        buf = torch.empty((rows, H), device=device, dtype=torch.float32)
        _scratch[key] = buf
    return buf


def _write_param_grad(weight: torch.Tensor, producer) -> torch.Tensor | None:
    """Run ``producer(out, accumulate)`` into weight.main_grad when present, else into a new tensor."""
    main_grad = getattr(weight, "main_grad", None)
    if main_grad is not None:
        producer(main_grad, getattr(weight, "grad_written", False))
        weight.grad_written = True
        hook = getattr(weight, "grad_ready", None)
        if hook is not None:
            hook(weight)
        return None
    out = torch.empty_like(weight)
    producer(out, False)
    return out


class _RMSNorm(torch.autograd.Function):
    """y = rmsnorm(h) * w with h = x (+ res).  Returns (y, h); with a residual, h is a new tensor
    produced in the same pass as the normalisation."""

    @staticmethod
    def forward(ctx, x, res, weight, eps):
        H = x.shape[-1]
        T = x.numel() // H
        assert x.is_contiguous() and (res is None or res.is_contiguous())
        y = torch.empty_like(x)
        h = torch.empty_like(x) if res is not None else x
        rstd = torch.empty(T, device=x.device, dtype=torch.float32)
        rc = _lib.load().b200_rmsnorm_fwd(x.data_ptr(), res.data_ptr() if res is not None else None,
                                          h.data_ptr() if res is not None else None, weight.data_ptr(),
                                          y.data_ptr(), rstd.data_ptr(), T, H, eps, _lib.stream_ptr())
        _lib.check(rc, "b200_rmsnorm_fwd")
        ctx.save_for_backward(h, weight, rstd)
        ctx.has_res = res is not None
        return y, (h if res is not None else None)

    @staticmethod
    def backward(ctx, dy, dh):
        x, weight, rstd = ctx.saved_tensors
        H = x.shape[-1]
        T = x.numel() // H
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dres_in = dh.contiguous() if dh is not None else None
        partial = _dw_partial(x.device, H)
        lib = _lib.load()

        def produce(out, acc):
            rc = lib.b200_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), weight.data_ptr(), rstd.data_ptr(),
                                      dres_in.data_ptr() if dres_in is not None else None, dx.data_ptr(),
                                      partial.data_ptr(), out.data_ptr(), int(acc), T, H, _lib.stream_ptr())
            _lib.check(rc, "b200_rmsnorm_bwd")

        dw = _write_param_grad(weight, produce)
        return dx, (dx if ctx.has_res else None), dw, None


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, residual: torch.Tensor | None = None):
    """Returns (normed, h) where h = x + residual (or x itself when residual is None)."""
    y, h = _RMSNorm.apply(x, residual, weight, eps)
    return y, (h if residual is not None else x)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        F = gu.shape[-1] // 2
        T = gu.numel() // (2 * F)
        assert gu.is_contiguous()
        out = torch.empty((*gu.shape[:-1], F), device=gu.device, dtype=gu.dtype)
        _lib.check(_lib.load().b200_swiglu_fwd(gu.data_ptr(), out.data_ptr(), T, F, _lib.stream_ptr()), "swiglu_fwd")
        ctx.save_for_backward(gu)
        return out

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        F = gu.shape[-1] // 2
        T = gu.numel() // (2 * F)
        dout = dout.contiguous()
        dgu = torch.empty_like(gu)
        _lib.check(_lib.load().b200_swiglu_bwd(dout.data_ptr(), gu.data_ptr(), dgu.data_ptr(), T, F,
                                               _lib.stream_ptr()), "swiglu_bwd")
        return dgu


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for a fused [..., 2F] tensor laid out as gate | up."""
    return _SwiGLU.apply(gate_up)


class _RoPE(torch.autograd.Function):
    """In-place rotary embedding on a [T, nheads, hd] view (token pitch may exceed nheads*hd)."""

    @staticmethod
    def forward(ctx, x, cos, sin, seq):
        T, nh, hd = x.shape
        assert x.stride(2) == 1 and x.stride(1) == hd
        _lib.check(_lib.load().b200_rope(x.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, nh, hd, x.stride(0), seq, 0,
                                         _lib.stream_ptr()), "rope")
        ctx.save_for_backward(cos, sin)
        ctx.seq = seq
        ctx.mark_dirty(x)
        return x

    @staticmethod
    def backward(ctx, dx):
        cos, sin = ctx.saved_tensors
        dx = dx.clone(memory_format=torch.contiguous_format)  # never rotate the caller's gradient in place
        T, nh, hd = dx.shape
        _lib.check(_lib.load().b200_rope(dx.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, nh, hd, dx.stride(0),
                                         ctx.seq, 1, _lib.stream_ptr()), "rope_bwd")
        return dx, None, None, None


def rope_(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq: int) -> torch.Tensor:
    return _RoPE.apply(x, cos, sin, seq)


class _CrossEntropy(torch.autograd.Function):
    """Mean token cross-entropy.  The logits tensor is overwritten with its own gradient in the
    forward pass (one fused kernel), so backward only rescales by the incoming scalar."""

    @staticmethod
    def forward(ctx, logits, targets):
        T, V = logits.shape
        assert logits.stride(1) == 1
        loss = torch.empty(T, device=logits.device, dtype=torch.float32)
        _lib.check(_lib.load().b200_cross_entropy(logits.data_ptr(), targets.data_ptr(), loss.data_ptr(), T, V,
                                                  logits.stride(0), 1.0 / T, _lib.stream_ptr()), "cross_entropy")
        ctx.save_for_backward(logits)
        ctx.mark_dirty(logits)
        return loss.mean(), logits

    @staticmethod
    def backward(ctx, dloss, _unused):
        (dlogits,) = ctx.saved_tensors
        # dloss is 1.0 in the training loop; avoid a 1 GB multiply in that case
        if dloss.numel() == 1 and getattr(_CrossEntropy, "assume_unit_grad", True):
            return dlogits, None
        return dlogits * dloss, None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    loss, _ = _CrossEntropy.apply(logits, targets)
    return loss


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        T = ids.numel()
        H = table.shape[1]
        out = torch.empty((*ids.shape, H), device=table.device, dtype=table.dtype)
        _lib.check(_lib.load().b200_embedding_fwd(ids.data_ptr(), table.data_ptr(), out.data_ptr(), T, H,
                                                  _lib.stream_ptr()), "embedding_fwd")
        ctx.save_for_backward(ids, table)
        return out

    @staticmethod
    def backward(ctx, dout):
        ids, table = ctx.saved_tensors
        dout = dout.contiguous()
        T = ids.numel()
        H = table.shape[1]
        lib = _lib.load()

        def produce(out, acc):
            if not acc:
                out.zero_()
            _lib.check(lib.b200_embedding_bwd(ids.data_ptr(), dout.data_ptr(), out.data_ptr(), T, H,
                                              _lib.stream_ptr()), "embedding_bwd")

        return None, _write_param_grad(table, produce)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    return _Embedding.apply(ids, table)


def adamw_step(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, master: torch.Tensor | None,
               *, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
               grad_scale: float = 1.0, zero_grad: bool = True) -> None:
    """One fused AdamW update over flat buffers (bf16 p/g, fp32 m/v, optional fp32 master)."""
    n = p.numel()
    assert g.numel() == n and m.numel() == n and v.numel() == n and n % 8 == 0
    rc = _lib.load().b200_adamw(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(),
                                master.data_ptr() if master is not None else None, n, lr, beta1, beta2, eps,
                                weight_decay, step, grad_scale, int(zero_grad), _lib.stream_ptr())
    _lib.check(rc, "b200_adamw")


def sumsq(x: torch.Tensor) -> torch.Tensor:
    out = torch.zeros(1, device=x.device, dtype=torch.float32)
    _lib.check(_lib.load().b200_sumsq(x.data_ptr(), x.numel(), out.data_ptr(), _lib.stream_ptr()), "sumsq")
    return out
