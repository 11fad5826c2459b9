"""Expert parallelism: MoE token dispatch / combine over NVLink, device-initiated.

``ExpertParallel`` owns the window layout (receive rows, scales, per-row records, combine cells,
histogram matrix) and the small device-side state of ``csrc/kernels/moe.cu`` and exposes

    route(topk_idx)                      -> per-expert row offsets of this rank's receive buffer
    dispatch(x, topk_idx, topk_w)        -> received rows, packed expert-major (bf16, or fp8 + scales)
    combine(y_rows, topk_w)              -> gate-weighted sum back in token order

``dispatch`` and ``combine`` are differentiable (each one's backward is the other's forward on
the gradients), so an MoE layer trains end to end through them.

The reference has no model-level code; its GIN layer offers the put / signal / wait primitives
such a dispatch is built from (reference: src/rdma/gin/nccl_ofi_gin.cpp,
include/rdma/gin/nccl_ofi_gin_types.h).
"""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import _lib
from .symm import Communicator

_vp, _i, _sz = C.c_void_p, C.c_int, C.c_size_t
_lib.register("b200_moe_route", [_i, _vp, _i, _i, _i, _sz, _vp, _vp, _vp, _vp, _vp, _vp], _i)
_lib.register("b200_moe_dispatch", [_i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _sz, _sz, _sz, _i, _vp,
                                    _vp], _i)
_lib.register("b200_moe_combine", [_i, _vp, _vp, _i, _sz, _sz, _vp, _vp, _i, _i, _i, _vp, _vp, _vp], _i)
_lib.register("b200_moe_combine_wgrad", [_vp, _vp, _vp, _vp, _i, _i, _i, _vp], _i)
_lib.register("b200_fp8_dequant_rows", [_vp, _vp, _vp, _vp, _i, _i, _vp], _i)


def _align(x: int, a: int = 1024) -> int:
    return (x + a - 1) // a * a


class ExpertParallel:
    """State and window layout for one MoE layer shape (tokens per rank, hidden, experts, top-k)."""

    def __init__(self, comm: Communicator, tokens: int, hidden: int, experts: int, topk: int, *,
                 capacity_factor: float = 2.0, window_offset: int = 0):
        assert experts % comm.world == 0 and hidden % 256 == 0
        self.comm, self.T, self.H, self.E, self.k = comm, tokens, hidden, experts, topk
        self.experts_local = experts // comm.world
        worst = comm.world * tokens * topk
        self.capacity = min(worst, max(1024, int(capacity_factor * tokens * topk)))
        self.cnt_off = _align(window_offset)
        self.recv_off = _align(self.cnt_off + 2 * comm.world * experts * 4)
        self.scale_off = _align(self.recv_off + self.capacity * hidden * 2)
        self.meta_off = _align(self.scale_off + self.capacity * (hidden // 128) * 4)
        self.comb_off = _align(self.meta_off + self.capacity * 16)
        self.window_end = self.comb_off + tokens * topk * hidden * 2
        assert self.window_end <= comm.window.chunk, (
            f"communicator window too small: need {self.window_end} bytes, have {comm.window.chunk}")
        dev = comm.device
        self.cnt_local = torch.zeros(experts, device=dev, dtype=torch.int32)
        self.dest_base = torch.zeros(experts, device=dev, dtype=torch.int32)
        self.cursor = torch.zeros(experts, device=dev, dtype=torch.int32)
        self.expert_offsets = torch.zeros(self.experts_local + 1, device=dev, dtype=torch.int32)
        self.row_of = torch.full((tokens, topk), -1, device=dev, dtype=torch.int32)
        self._done = torch.zeros(4, device=dev, dtype=torch.int32)
        self._last_topk_idx = None

    @staticmethod
    def window_bytes(world: int, tokens: int, hidden: int, experts: int, topk: int, capacity_factor: float = 2.0) -> int:
        cap = min(world * tokens * topk, max(1024, int(capacity_factor * tokens * topk)))
        return (_align(2 * world * experts * 4) + _align(cap * hidden * 2) + _align(cap * (hidden // 128) * 4) +
                _align(cap * 16) + _align(tokens * topk * hidden * 2) + 8192)

    # ---- views of the receive side
    def recv_rows(self, fp8: bool) -> torch.Tensor:
        if fp8:
            return self.comm.local[self.recv_off:self.recv_off + self.capacity * self.H].view(self.capacity, self.H)
        return self.comm.view(self.recv_off, self.capacity * self.H, torch.bfloat16).view(self.capacity, self.H)

    def recv_scales(self) -> torch.Tensor:
        g = self.H // 128
        return self.comm.view(self.scale_off, self.capacity * g, torch.float32).view(self.capacity, g)

    def recv_meta(self) -> torch.Tensor:
        """int32 [capacity, 4]: token, slot, weight bits, source rank."""
        return self.comm.view(self.meta_off, self.capacity * 4, torch.int32).view(self.capacity, 4)

    def combine_cells(self) -> torch.Tensor:
        return self.comm.view(self.comb_off, self.T * self.k * self.H, torch.bfloat16).view(self.T, self.k, self.H)

    # ---- raw collectives (stream-ordered, no autograd)
    def route(self, topk_idx: torch.Tensor) -> torch.Tensor:
        assert topk_idx.shape == (self.T, self.k) and topk_idx.dtype == torch.int32 and topk_idx.is_contiguous()
        rc = _lib.load().b200_moe_route(self.comm.id, topk_idx.data_ptr(), self.T, self.k, self.E, self.cnt_off,
                                        self.cnt_local.data_ptr(), self.dest_base.data_ptr(),
                                        self.expert_offsets.data_ptr(), self.cursor.data_ptr(),
                                        self._done[0:].data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "b200_moe_route")
        return self.expert_offsets

    def dispatch_raw(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor | None, *, fp8: bool,
                     use_saved_rows: bool = False, scale_by_weight: bool = False) -> None:
        assert x.shape == (self.T, self.H) and x.dtype == torch.bfloat16 and x.is_contiguous()
        rc = _lib.load().b200_moe_dispatch(
            self.comm.id, x.data_ptr(), topk_idx.data_ptr(), topk_w.data_ptr() if topk_w is not None else None,
            self.T, self.k, self.H, self.E, int(fp8), int(use_saved_rows), int(scale_by_weight),
            self.dest_base.data_ptr(), self.cursor.data_ptr(), self.row_of.data_ptr(), self.recv_off, self.scale_off,
            self.meta_off, self.capacity, self._done[1:].data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "b200_moe_dispatch")

    def combine_raw(self, y_rows: torch.Tensor, topk_w: torch.Tensor | None, out: torch.Tensor) -> None:
        assert y_rows.dtype == torch.bfloat16 and y_rows.is_contiguous() and y_rows.shape[1] == self.H
        assert out.shape == (self.T, self.H) and out.dtype == torch.bfloat16 and out.is_contiguous()
        rc = _lib.load().b200_moe_combine(
            self.comm.id, y_rows.data_ptr(), self.expert_offsets.data_ptr(), self.experts_local, self.meta_off,
            self.comb_off, topk_w.data_ptr() if topk_w is not None else None, self.row_of.data_ptr(), self.T, self.k,
            self.H, out.data_ptr(), self._done[2:].data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "b200_moe_combine")

    def dequant(self, out: torch.Tensor | None = None) -> torch.Tensor:
        """fp8 receive rows + scales -> bf16 [capacity, H] (only the rows actually received are written)."""
        if out is None:
            out = torch.zeros(self.capacity, self.H, device=self.comm.device, dtype=torch.bfloat16)
        rc = _lib.load().b200_fp8_dequant_rows(self.recv_rows(True).data_ptr(), self.recv_scales().data_ptr(),
                                               out.data_ptr(), self.expert_offsets[self.experts_local:].data_ptr(),
                                               self.capacity, self.H, _lib.stream_ptr())
        _lib.check(rc, "b200_fp8_dequant_rows")
        return out

    # ---- differentiable forms
    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, fp8: bool = False) -> torch.Tensor:
        """Route + dispatch.  Returns bf16 rows [capacity, H]; rows [expert_offsets[e], expert_offsets[e+1])
        belong to local expert e, rows past expert_offsets[-1] are unspecified."""
        return _Dispatch.apply(x, self, topk_idx, topk_w, fp8)

    def combine(self, y_rows: torch.Tensor, topk_w: torch.Tensor) -> torch.Tensor:
        return _Combine.apply(y_rows, topk_w, self)


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ep, topk_idx, topk_w, fp8):
        ep.route(topk_idx)
        ep.dispatch_raw(x.contiguous(), topk_idx, topk_w, fp8=fp8)
        ep._last_topk_idx = topk_idx
        ctx.ep = ep
        if fp8:
            return ep.dequant()
        return ep.recv_rows(False).clone()

    @staticmethod
    def backward(ctx, d_rows):
        ep = ctx.ep
        dx = torch.empty(ep.T, ep.H, device=d_rows.device, dtype=torch.bfloat16)
        ep.combine_raw(d_rows.contiguous(), None, dx)   # unweighted sum of the k row gradients of each token
        return dx, None, None, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_rows, topk_w, ep):
        out = torch.empty(ep.T, ep.H, device=y_rows.device, dtype=torch.bfloat16)
        w = topk_w.detach().float().contiguous()
        ep.combine_raw(y_rows.contiguous(), w, out)
        ctx.ep = ep
        ctx.n_rows = y_rows.shape[0]
        ctx.save_for_backward(w, ep.combine_cells().clone())
        return out

    @staticmethod
    def backward(ctx, d_out):
        ep = ctx.ep
        w, cells = ctx.saved_tensors
        d_out = d_out.contiguous()
        dw = torch.empty(ep.T, ep.k, device=d_out.device, dtype=torch.float32)
        _lib.check(_lib.load().b200_moe_combine_wgrad(d_out.data_ptr(), cells.data_ptr(), ep.row_of.data_ptr(),
                                                      dw.data_ptr(), ep.T, ep.k, ep.H, _lib.stream_ptr()),
                   "b200_moe_combine_wgrad")
        # d(y_row) = weight * d_out[token]: the forward dispatch again, on the same rows, weighted
        idx = ep._last_topk_idx
        ep.dispatch_raw(d_out, idx, w, fp8=False, use_saved_rows=True, scale_by_weight=True)
        return ep.recv_rows(False)[:ctx.n_rows].clone(), dw, None
