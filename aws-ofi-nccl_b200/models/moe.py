"""Expert-parallel mixture-of-experts layer: softmax top-k router, device-initiated dispatch of the
token rows to the ranks that own their experts (optionally as block-scaled fp8), SwiGLU experts
on the tcgen05 GEMM, gate-weighted combine back to token order."""
from __future__ import annotations

import torch

from ..ops.gemm import linear
from ..ops.llm import swiglu
from ..parallel.expert_parallel import ExpertParallel
from ..parallel.symm import Communicator


class MoELayer(torch.nn.Module):
    def __init__(self, comm: Communicator, tokens: int, hidden: int, ffn: int, experts: int, topk: int, *,
                 fp8_dispatch: bool = False, capacity_factor: float = 2.0, window_offset: int = 0, seed: int = 0):
        super().__init__()
        self.ep = ExpertParallel(comm, tokens, hidden, experts, topk, capacity_factor=capacity_factor,
                                 window_offset=window_offset)
        self.hidden, self.ffn, self.experts, self.topk, self.fp8 = hidden, ffn, experts, topk, fp8_dispatch
        el = experts // comm.world
        g = torch.Generator(device="cpu").manual_seed(seed)
        router = torch.randn(experts, hidden, generator=g) * hidden ** -0.5
        w_gu = torch.randn(experts, 2 * ffn, hidden, generator=g) * hidden ** -0.5
        w_dn = torch.randn(experts, hidden, ffn, generator=g) * ffn ** -0.5
        lo = comm.rank * el
        dev = comm.device
        self.router = torch.nn.Parameter(router.to(dev))   # fp32, replicated
        self.w_gate_up = torch.nn.ParameterList(
            [torch.nn.Parameter(w_gu[lo + e].to(dev, torch.bfloat16)) for e in range(el)])
        self.w_down = torch.nn.ParameterList(
            [torch.nn.Parameter(w_dn[lo + e].to(dev, torch.bfloat16)) for e in range(el)])
        self._full = (router, w_gu, w_dn)  # CPU fp32 copies of all experts (reference checks only)

    def route(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        probs = torch.softmax(x.float() @ self.router.t(), dim=-1)
        w, idx = torch.topk(probs, self.topk, dim=-1)
        return idx.to(torch.int32).contiguous(), w.contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        idx, w = self.route(x)
        rows = self.ep.dispatch(x, idx, w, self.fp8)
        # The per-expert row ranges live on the device; slicing the rows for the per-expert GEMM
        # calls needs them on the host.
        off = self.ep.expert_offsets.tolist()
        outs = []
        for e in range(len(self.w_gate_up)):
            if off[e + 1] > off[e]:
                seg = rows[off[e]:off[e + 1]]
                outs.append(linear(swiglu(linear(seg, self.w_gate_up[e])), self.w_down[e]))
        if outs:
            y = torch.cat(outs, dim=0)
        else:
            y = rows[:0]
        return self.ep.combine(y, w)
