"""Llama-3 decoder for training on B200: every GEMM runs on the tcgen05 kernel, every bandwidth
op on the kernels of llm_ops.cu; attention uses torch SDPA (a library kernel).

Parameters live in ONE flat bf16 buffer and their gradients in ONE flat bf16 buffer
(``weight.main_grad`` views), so the optimizer is a single fused launch and a data-parallel
engine can reduce contiguous gradient ranges as soon as backward has produced them.
"""
from __future__ import annotations

import dataclasses
import math

import torch
import torch.nn.functional as F

from ..ops import gemm as gemm_ops
from ..ops import llm as llm_ops


@dataclasses.dataclass
class LlamaConfig:
    vocab_size: int = 128256
    hidden: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn: int = 14336
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5
    max_seq: int = 4096

    @property
    def head_dim(self) -> int:
        return self.hidden // self.n_heads

    @staticmethod
    def llama3_8b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def tiny() -> "LlamaConfig":
        return LlamaConfig(vocab_size=1024, hidden=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn=512, max_seq=128)

    def param_shapes(self) -> list[tuple[str, tuple[int, ...]]]:
        hd = self.head_dim
        qkv = (self.n_heads + 2 * self.n_kv_heads) * hd
        shapes: list[tuple[str, tuple[int, ...]]] = [("embed", (self.vocab_size, self.hidden))]
        for i in range(self.n_layers):
            shapes += [
                (f"l{i}.norm1", (self.hidden,)),
                (f"l{i}.wqkv", (qkv, self.hidden)),
                (f"l{i}.wo", (self.hidden, self.n_heads * hd)),
                (f"l{i}.norm2", (self.hidden,)),
                (f"l{i}.wgu", (2 * self.ffn, self.hidden)),
                (f"l{i}.wdown", (self.hidden, self.ffn)),
            ]
        shapes += [("normf", (self.hidden,)), ("lm_head", (self.vocab_size, self.hidden))]
        return shapes

    def num_params(self) -> int:
        return sum(math.prod(s) for _, s in self.param_shapes())


class _QKRope(torch.autograd.Function):
    """Rotary embedding applied in place to the q and k heads of a fused [T, (nq+2nkv)*hd] tensor."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, n_rot_heads, hd, seq):
        T = qkv.shape[0]
        view = qkv.as_strided((T, n_rot_heads, hd), (qkv.stride(0), hd, 1))
        from ..ops import _lib
        _lib.check(_lib.load().b200_rope(view.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, n_rot_heads, hd,
                                         qkv.stride(0), seq, 0, _lib.stream_ptr()), "rope")
        ctx.save_for_backward(cos, sin)
        ctx.meta = (n_rot_heads, hd, seq)
        ctx.mark_dirty(qkv)
        return qkv

    @staticmethod
    def backward(ctx, d):
        from ..ops import _lib
        cos, sin = ctx.saved_tensors
        n_rot_heads, hd, seq = ctx.meta
        d = d.clone(memory_format=torch.contiguous_format)
        _lib.check(_lib.load().b200_rope(d.data_ptr(), cos.data_ptr(), sin.data_ptr(), d.shape[0], n_rot_heads, hd,
                                         d.stride(0), seq, 1, _lib.stream_ptr()), "rope_bwd")
        return d, None, None, None, None, None


class Llama:
    """Functional model over a flat parameter buffer (no nn.Module: the buffers are the state)."""

    def __init__(self, cfg: LlamaConfig, device="cuda", grad_buffer: torch.Tensor | None = None, seed: int = 0,
                 init_std: float = 0.02):
        self.cfg = cfg
        self.device = torch.device(device)
        n = 0
        self.offsets: dict[str, tuple[int, tuple[int, ...]]] = {}
        for name, shape in cfg.param_shapes():
            self.offsets[name] = (n, shape)
            n += (math.prod(shape) + 127) // 128 * 128  # 256-byte aligned views
        self.numel = n
        self.flat_params = torch.empty(n, device=self.device, dtype=torch.bfloat16)
        if grad_buffer is None:
            grad_buffer = torch.zeros(n, device=self.device, dtype=torch.bfloat16)
        assert grad_buffer.numel() >= n and grad_buffer.dtype == torch.bfloat16
        self.flat_grads = grad_buffer[:n]
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed)
        self.flat_params.normal_(0.0, init_std, generator=gen)
        self.params: dict[str, torch.Tensor] = {}
        for name, (off, shape) in self.offsets.items():
            p = self.flat_params[off:off + math.prod(shape)].view(shape)
            if "norm" in name:
                p.fill_(1.0)
            p.requires_grad_(True)
            p.main_grad = self.flat_grads[off:off + math.prod(shape)].view(shape)
            p.grad_written = False
            p.param_name = name
            self.params[name] = p
        hd = cfg.head_dim
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, device=self.device, dtype=torch.float32) / hd))
        ang = torch.outer(torch.arange(cfg.max_seq, device=self.device, dtype=torch.float32), inv)
        self.cos, self.sin = ang.cos().contiguous(), ang.sin().contiguous()

    # ------------------------------------------------------------------ hooks for data parallelism
    def set_grad_ready_hook(self, fn) -> None:
        for p in self.params.values():
            p.grad_ready = fn

    def reset_grad_flags(self) -> None:
        for p in self.params.values():
            p.grad_written = False

    # ------------------------------------------------------------------ forward
    def _attention(self, qkv: torch.Tensor, B: int, S: int) -> torch.Tensor:
        cfg = self.cfg
        hd, nq, nkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
        qkv = _QKRope.apply(qkv, self.cos, self.sin, nq + nkv, hd, S)
        q = qkv[:, : nq * hd].view(B, S, nq, hd).transpose(1, 2)
        k = qkv[:, nq * hd:(nq + nkv) * hd].view(B, S, nkv, hd).transpose(1, 2)
        v = qkv[:, (nq + nkv) * hd:].view(B, S, nkv, hd).transpose(1, 2)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=(nq != nkv))
        return o.transpose(1, 2).reshape(B * S, nq * hd)

    def forward_loss(self, ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        """ids, labels: int64 [B, S] on the device.  Returns the mean next-token loss (labels are
        already the shifted targets)."""
        cfg, P = self.cfg, self.params
        B, S = ids.shape
        x = llm_ops.embedding(ids.reshape(-1), P["embed"])
        h, delta = x, None
        for i in range(cfg.n_layers):
            n1, h = llm_ops.rmsnorm(h if delta is None else delta, P[f"l{i}.norm1"], cfg.rms_eps,
                                    residual=None if delta is None else h)
            qkv = gemm_ops.linear(n1, P[f"l{i}.wqkv"])
            attn = self._attention(qkv, B, S)
            o = gemm_ops.linear(attn, P[f"l{i}.wo"])
            n2, h = llm_ops.rmsnorm(o, P[f"l{i}.norm2"], cfg.rms_eps, residual=h)
            gu = gemm_ops.linear(n2, P[f"l{i}.wgu"])
            act = llm_ops.swiglu(gu)
            delta = gemm_ops.linear(act, P[f"l{i}.wdown"])
        nf, _ = llm_ops.rmsnorm(delta, P["normf"], cfg.rms_eps, residual=h)
        logits = gemm_ops.linear(nf, P["lm_head"])
        return llm_ops.cross_entropy(logits, labels.reshape(-1))


def reference_forward_loss(model: Llama, ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Plain-PyTorch fp32 restatement of forward_loss over the same parameters (test oracle)."""
    cfg = model.cfg
    P = {k: v.detach().float() for k, v in model.params.items()}
    B, S = ids.shape
    hd, nq, nkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads

    def norm(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * w

    def rope(t):  # [B,S,n,hd]
        c = model.cos[:S].view(1, S, 1, hd // 2)
        s = model.sin[:S].view(1, S, 1, hd // 2)
        a, b = t[..., : hd // 2], t[..., hd // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], -1)

    h = P["embed"][ids]
    for i in range(cfg.n_layers):
        n1 = norm(h, P[f"l{i}.norm1"])
        qkv = n1 @ P[f"l{i}.wqkv"].T
        q = rope(qkv[..., : nq * hd].view(B, S, nq, hd)).transpose(1, 2)
        k = rope(qkv[..., nq * hd:(nq + nkv) * hd].view(B, S, nkv, hd)).transpose(1, 2)
        v = qkv[..., (nq + nkv) * hd:].view(B, S, nkv, hd).transpose(1, 2)
        k = k.repeat_interleave(nq // nkv, 1)
        v = v.repeat_interleave(nq // nkv, 1)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, nq * hd)
        h = h + o @ P[f"l{i}.wo"].T
        n2 = norm(h, P[f"l{i}.norm2"])
        gu = n2 @ P[f"l{i}.wgu"].T
        g, u = gu[..., : cfg.ffn], gu[..., cfg.ffn:]
        h = h + (F.silu(g) * u) @ P[f"l{i}.wdown"].T
    logits = norm(h, P["normf"]) @ P["lm_head"].T
    return F.cross_entropy(logits.view(B * S, -1), labels.reshape(-1))
