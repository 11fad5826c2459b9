"""Tensor parallelism over NVLink: GEMMs fused with their collectives.

``ag_gemm`` and ``gemm_rs`` bind the single-kernel all-gather->GEMM(->SwiGLU) and
GEMM->reduce-scatter of ``csrc/kernels/fused_tp.cu``.  ``TensorParallelMLP`` is a
sequence-parallel SwiGLU MLP (activations sharded along tokens between layers, weights sharded
along the hidden FFN dimension) whose forward and backward are four fused kernels plus two local
weight-gradient GEMMs.  ``FsdpLinear`` keeps a weight sharded along its output rows and gathers
it inside the GEMM kernel that consumes it.

The transport plugin this framework replaces only moves bytes for NCCL
(reference: src/nccl_ofi_net.cpp, src/rdma/nccl_ofi_rdma.cpp); on an NVSwitch node the same
bytes move inside the compute kernel instead.
"""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import _lib
from ..ops.gemm import gemm
from .symm import Communicator

_vp, _i, _sz, _f, _ll = C.c_void_p, C.c_int, C.c_size_t, C.c_float, C.c_longlong
_lib.register("b200_ag_gemm", [_i, _sz, _i, _i, _i, _i, _vp, _ll, _i, _vp, _ll, _vp, _ll, _i, _i, _i, _vp], _i)
_lib.register("b200_gemm_rs", [_i, _vp, _ll, _vp, _ll, _i, _i, _i, _i, _sz, _vp, _ll, _f, _vp], _i)
_lib.register("b200_gemm_rs_staging_bytes", [_i, _i, _i], _sz)
_lib.set_kernels_per_call("b200_gemm_rs_staging_bytes", 0)

TP_CHANNEL = 2  # barrier slots used by the fused kernels (0: default collectives, 1: gradient reducer)


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """[F,H] gate and up projections -> [2F,H] with rows alternating in blocks of 32 (32 gate rows,
    then the matching 32 up rows), the layout the fused SwiGLU epilogue expects."""
    F, H = w_gate.shape
    assert w_up.shape == (F, H) and F % 32 == 0
    return torch.stack((w_gate.view(F // 32, 32, H), w_up.view(F // 32, 32, H)), dim=1).reshape(2 * F, H).contiguous()


def deinterleave_gate_up(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    F2, H = w.shape
    v = w.view(F2 // 64, 2, 32, H)
    return v[:, 0].reshape(F2 // 2, H), v[:, 1].reshape(F2 // 2, H)


def ag_gemm(comm: Communicator, gathered_off: int, rows: int, k: int, other: torch.Tensor, *, b_mn: bool = False,
            gather_b: bool = False, out: torch.Tensor | None = None, act: torch.Tensor | None = None,
            swiglu: bool = False, n_movers: int = 0, channel: int = TP_CHANNEL) -> None:
    """One kernel: all-gather the operand whose shards sit at ``gathered_off`` in every rank's
    window (``rows`` x ``k`` bf16 in total, this rank's shard already written in place), and
    multiply.  gather_b=False: C = gathered[rows,k] @ op(other), ``other`` is [N,k] (or [k,N] with
    b_mn).  gather_b=True: C = other[M,k] @ gathered[rows=N,k]^T.  With ``swiglu`` the product's
    interleaved gate|up columns are reduced to ``act`` [M,N/2]; ``out`` (optional then) keeps the
    raw product for the backward pass."""
    assert other.dtype == torch.bfloat16 and other.stride(1) == 1
    if gather_b:
        M, N = other.shape[0], rows
        assert other.shape[1] == k and not b_mn
    else:
        M = rows
        N = other.shape[1] if b_mn else other.shape[0]
        assert (other.shape[0] if b_mn else other.shape[1]) == k
    if out is not None:
        assert out.shape == (M, N) and out.dtype == torch.bfloat16 and out.stride(1) == 1
    if swiglu:
        assert act is not None and act.shape == (M, N // 2) and act.stride(1) == 1
    rc = _lib.load().b200_ag_gemm(
        comm.id, gathered_off, int(gather_b), M, N, k, other.data_ptr(), other.stride(0), int(b_mn),
        out.data_ptr() if out is not None else None, out.stride(0) if out is not None else 0,
        act.data_ptr() if act is not None else None, act.stride(0) if act is not None else 0,
        int(swiglu), n_movers, channel, _lib.stream_ptr())
    _lib.check(rc, "b200_ag_gemm")


def gemm_rs_staging_bytes(world: int, m: int, n: int) -> int:
    """Window bytes ``gemm_rs`` needs at ``staging_off`` on every rank (two call parities of the
    world-1 ring hops)."""
    return 0 if world <= 1 else 2 * (world - 1) * (m // world) * n * 2


def gemm_rs(comm: Communicator, a: torch.Tensor, b: torch.Tensor, staging_off: int, out: torch.Tensor, *,
            b_mn: bool = False, scale: float = 1.0) -> None:
    """One kernel: partial = a[M,K] @ op(b), ring reduce-scatter over ranks along M inside the GEMM
    epilogue; out[M/world, N] = scale * sum_r partial_r[rows of this rank].  ``staging_off`` names
    ``gemm_rs_staging_bytes`` of window space on every rank."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.stride(1) == 1 and b.stride(1) == 1
    M, K = a.shape
    N = b.shape[1] if b_mn else b.shape[0]
    assert (b.shape[0] if b_mn else b.shape[1]) == K
    assert out.shape == (M // comm.world, N) and out.dtype == torch.bfloat16 and out.stride(1) == 1
    rc = _lib.load().b200_gemm_rs(comm.id, a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), int(b_mn), M, N, K,
                                  staging_off, out.data_ptr(), out.stride(0), scale, _lib.stream_ptr())
    _lib.check(rc, "b200_gemm_rs")


def _align(x: int, a: int = 1024) -> int:
    return (x + a - 1) // a * a


class _TPMlpFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, w_gu, w_down, mlp):
        comm, T, H, Fl = mlp.comm, mlp.tokens, mlp.hidden, mlp.ffn_local
        Ts = T // comm.world
        # this rank's token shard goes into its slot of the gathered activation
        mlp.x_full[comm.rank * Ts:(comm.rank + 1) * Ts].copy_(x_shard)
        gu = torch.empty((T, 2 * Fl), device=x_shard.device, dtype=torch.bfloat16)
        act = torch.empty((T, Fl), device=x_shard.device, dtype=torch.bfloat16)
        ag_gemm(comm, mlp.x_off, T, H, w_gu, out=gu, act=act, swiglu=True, n_movers=mlp.n_helpers)
        y_shard = torch.empty((Ts, H), device=x_shard.device, dtype=torch.bfloat16)
        gemm_rs(comm, act, w_down, mlp.stage_off, y_shard)
        ctx.mlp = mlp
        ctx.save_for_backward(gu, act, w_gu, w_down)
        return y_shard

    @staticmethod
    def backward(ctx, dy_shard):
        mlp = ctx.mlp
        gu, act, w_gu, w_down = ctx.saved_tensors
        comm, T, H, Fl = mlp.comm, mlp.tokens, mlp.hidden, mlp.ffn_local
        Ts = T // comm.world
        mlp.dy_full[comm.rank * Ts:(comm.rank + 1) * Ts].copy_(dy_shard)
        # dact[T,Fl] = gather(dy)[T,H] @ w_down[H,Fl]   (w_down is stored [K=H][N=Fl])
        dact = torch.empty((T, Fl), device=dy_shard.device, dtype=torch.bfloat16)
        ag_gemm(comm, mlp.dy_off, T, H, w_down, b_mn=True, out=dact, n_movers=mlp.n_helpers)
        # dW_down[H,Fl] = dy_full^T @ act
        _accumulate_wgrad(w_down, mlp.dy_full, act)
        dgu = torch.empty_like(gu)
        _lib.check(_lib.load().b200_swiglu_bwd_interleaved(dact.data_ptr(), gu.data_ptr(), dgu.data_ptr(), T, Fl,
                                                           _lib.stream_ptr()), "swiglu_bwd_interleaved")
        # dx[T/n,H] = reduce_scatter(dgu[T,2Fl] @ w_gu[2Fl,H])   (w_gu is stored [K=2Fl][N=H])
        dx_shard = torch.empty((Ts, H), device=dy_shard.device, dtype=torch.bfloat16)
        gemm_rs(comm, dgu, w_gu, mlp.stage_off, dx_shard, b_mn=True)
        # dW_gu[2Fl,H] = dgu^T @ x_full
        _accumulate_wgrad(w_gu, dgu, mlp.x_full)
        return dx_shard, None, None, None


def _accumulate_wgrad(w: torch.Tensor, a_km: torch.Tensor, b_kn: torch.Tensor) -> None:
    """w.main_grad (or w.grad) (+)= a_km^T @ b_kn, both operands stored with the reduction (token)
    dimension outermost."""
    target = getattr(w, "main_grad", None)
    if target is not None:
        gemm(a_km, b_kn, a_mn=True, b_mn=True, out=target, accumulate=True)
    elif w.grad is None:
        w.grad = gemm(a_km, b_kn, a_mn=True, b_mn=True)
    else:
        gemm(a_km, b_kn, a_mn=True, b_mn=True, out=w.grad, accumulate=True)
    hook = getattr(w, "grad_ready", None)
    if hook is not None:
        hook()


class TensorParallelMLP(torch.nn.Module):
    """SwiGLU MLP with sequence-parallel activations: takes this rank's [tokens/world, hidden]
    shard and returns the same shard of the output.  ``w_gate_up`` holds this rank's slice of the
    FFN dimension in the interleaved layout of ``interleave_gate_up``; ``w_down`` is [hidden,
    ffn/world]."""

    def __init__(self, comm: Communicator, tokens: int, hidden: int, ffn: int, window_offset: int = 0,
                 n_helpers: int = 16, seed: int = 0):
        super().__init__()
        assert ffn % (32 * comm.world) == 0 and tokens % (128 * comm.world) == 0
        self.comm, self.tokens, self.hidden, self.ffn = comm, tokens, hidden, ffn
        self.ffn_local = ffn // comm.world
        self.n_helpers = n_helpers
        act_bytes = tokens * hidden * 2
        self.x_off = _align(window_offset)
        self.dy_off = _align(self.x_off + act_bytes)
        self.stage_off = _align(self.dy_off + act_bytes)
        self.window_end = self.stage_off + gemm_rs_staging_bytes(comm.world, tokens, hidden)
        assert self.window_end <= comm.window.chunk, "communicator window too small for this layer"
        self.x_full = comm.view(self.x_off, tokens * hidden, torch.bfloat16).view(tokens, hidden)
        self.dy_full = comm.view(self.dy_off, tokens * hidden, torch.bfloat16).view(tokens, hidden)
        g = torch.Generator(device="cpu").manual_seed(seed)
        wg = torch.randn(ffn, hidden, generator=g) * hidden ** -0.5
        wu = torch.randn(ffn, hidden, generator=g) * hidden ** -0.5
        wd = torch.randn(hidden, ffn, generator=g) * ffn ** -0.5
        lo, hi = comm.rank * self.ffn_local, (comm.rank + 1) * self.ffn_local
        dev = comm.device
        self.w_gate_up = torch.nn.Parameter(interleave_gate_up(wg[lo:hi], wu[lo:hi]).to(dev, torch.bfloat16))
        self.w_down = torch.nn.Parameter(wd[:, lo:hi].contiguous().to(dev, torch.bfloat16))
        self._full = (wg, wu, wd)  # CPU fp32 copies of the unsharded weights (reference checks only)

    @staticmethod
    def window_bytes(tokens: int, hidden: int) -> int:
        return 4 * _align(tokens * hidden * 2) + 1024

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        return _TPMlpFn.apply(x_shard, self.w_gate_up, self.w_down, self)


class FsdpLinear(torch.nn.Module):
    """y = x W^T with W [out, in] sharded along its rows over the ranks; each rank keeps only its
    shard (inside the communicator window) and the forward GEMM gathers the other shards while it
    runs.  The backward pass computes dx with the already gathered weight and reduce-scatters the
    weight gradient so every rank ends with the gradient of its own shard."""

    def __init__(self, comm: Communicator, in_features: int, out_features: int, window_offset: int = 0,
                 n_helpers: int = 8, seed: int = 0):
        super().__init__()
        assert out_features % (256 * comm.world) == 0
        self.comm, self.inf, self.outf = comm, in_features, out_features
        self.n_helpers = n_helpers
        self.w_off = _align(window_offset)
        self.window_end = self.w_off + out_features * in_features * 2
        assert self.window_end <= comm.window.chunk
        self.w_full = comm.view(self.w_off, out_features * in_features, torch.bfloat16).view(out_features, in_features)
        rows = out_features // comm.world
        g = torch.Generator(device="cpu").manual_seed(seed)
        w = torch.randn(out_features, in_features, generator=g) * in_features ** -0.5
        self._full = w
        self.shard = self.w_full[comm.rank * rows:(comm.rank + 1) * rows]
        self.shard.copy_(w[comm.rank * rows:(comm.rank + 1) * rows].to(torch.bfloat16))
        self.shard_grad = torch.zeros((rows, in_features), device=comm.device, dtype=torch.float32)
        # staging for the weight-gradient reduce-scatter sits right behind the weight
        self.grad_off = _align(self.window_end)
        self.window_end = self.grad_off + out_features * in_features * 2
        assert self.window_end <= comm.window.chunk

    @staticmethod
    def window_bytes(in_features: int, out_features: int) -> int:
        return 2 * _align(in_features * out_features * 2) + 2048

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _FsdpLinearFn.apply(x, self)


class _FsdpLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, layer):
        x2 = x.reshape(-1, layer.inf)
        y = torch.empty((*x.shape[:-1], layer.outf), device=x.device, dtype=torch.bfloat16)
        ag_gemm(layer.comm, layer.w_off, layer.outf, layer.inf, x2, gather_b=True, out=y.view(-1, layer.outf),
                n_movers=layer.n_helpers)
        ctx.layer = layer
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy):
        layer = ctx.layer
        (x,) = ctx.saved_tensors
        comm = layer.comm
        x2 = x.reshape(-1, layer.inf)
        dy2 = dy.reshape(-1, layer.outf)
        # the gathered weight is still in the window: dx = dy @ W  (W stored [K=out][N=in])
        dx = gemm(dy2, layer.w_full, b_mn=True)
        # full dW = dy^T @ x, then each rank keeps the sum of its rows
        dw = gemm(dy2, x2, a_mn=True, b_mn=True)
        rows = layer.outf // comm.world
        if comm.world == 1:
            layer.shard_grad += dw.float()
        else:
            stage = comm.view(layer.grad_off, layer.outf * layer.inf, torch.bfloat16)
            stage.copy_(dw.view(-1))
            part = torch.empty((rows, layer.inf), device=x.device, dtype=torch.float32)
            comm.reduce_scatter(layer.grad_off, rows * layer.inf * 2, torch.bfloat16, part, channel=TP_CHANNEL)
            layer.shard_grad += part
        return dx.view_as(x), None
