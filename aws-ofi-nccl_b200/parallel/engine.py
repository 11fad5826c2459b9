"""Training engine: the public entry point a user calls for a Llama training step.

``Trainer.step(ids_host, labels_host)`` runs one full optimizer step — host-to-device copy of the
batch from pinned memory, forward, backward (with the gradient all-reduce of a data-parallel job
overlapped behind it), fused AdamW — and returns the loss as a Python float (device-to-host read).
"""
from __future__ import annotations

import dataclasses

import torch

from ..models.llama import Llama, LlamaConfig
from ..ops import llm as llm_ops


@dataclasses.dataclass
class OptimConfig:
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    master_weights: bool = True


class Trainer:
    def __init__(self, cfg: LlamaConfig, optim: OptimConfig | None = None, device="cuda", dp=None, seed: int = 0):
        """dp: an optional ``parallel.data_parallel.GradReducer`` (owns the symmetric gradient buffer)."""
        self.cfg = cfg
        self.optim = optim or OptimConfig()
        self.device = torch.device(device)
        self.dp = dp
        grad_buffer = dp.allocate_grad_buffer(self._padded_numel(cfg)) if dp is not None else None
        self.model = Llama(cfg, device=self.device, grad_buffer=grad_buffer, seed=seed)
        n = self.model.numel
        # a reducer in "zero" mode leaves each rank the optimizer state of its own shard only
        self.shard = dp.shard_range(n) if getattr(dp, "mode", "") == "zero" else (0, n)
        lo, hi = self.shard
        self.m = torch.zeros(hi - lo, device=self.device, dtype=torch.float32)
        self.v = torch.zeros(hi - lo, device=self.device, dtype=torch.float32)
        self.master = self.model.flat_params[lo:hi].float() if self.optim.master_weights else None
        self.step_count = 0
        self.kernel_launches = 0
        if dp is not None:
            dp.attach(self.model)
        self._ids_dev = None
        self._labels_dev = None

    @staticmethod
    def _padded_numel(cfg: LlamaConfig) -> int:
        import math
        return sum((math.prod(s) + 127) // 128 * 128 for _, s in cfg.param_shapes())

    # ------------------------------------------------------------------ one optimizer step, device tensors in
    def step_device(self, ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        model, oc = self.model, self.optim
        model.reset_grad_flags()
        if self.dp is not None:
            self.dp.begin_step()
        loss = model.forward_loss(ids, labels)
        loss.backward()
        if self.dp is not None:
            self.dp.finish_step()  # all buckets reduced (averaged) in place in the flat gradient buffer
        self.step_count += 1
        lo, hi = self.shard
        grad_scale = float(getattr(self.dp, "grad_scale", 1.0))   # reducers that sum leave the 1/N to the optimizer
        llm_ops.adamw_step(model.flat_params[lo:hi], model.flat_grads[lo:hi], self.m, self.v, self.master, lr=oc.lr,
                           beta1=oc.beta1, beta2=oc.beta2, eps=oc.eps, weight_decay=oc.weight_decay,
                           step=self.step_count, grad_scale=grad_scale, zero_grad=True)
        if (lo, hi) != (0, model.numel):
            if lo > 0:
                model.flat_grads[:lo].zero_()
            if hi < model.numel:
                model.flat_grads[hi:].zero_()
            self.dp.gather_params(model.flat_params)
        return loss.detach()

    # ------------------------------------------------------------------ end to end: pinned host batch in, float out
    def step(self, ids_host: torch.Tensor, labels_host: torch.Tensor) -> float:
        if self._ids_dev is None or self._ids_dev.shape != ids_host.shape:
            self._ids_dev = torch.empty(ids_host.shape, device=self.device, dtype=torch.int64)
            self._labels_dev = torch.empty(labels_host.shape, device=self.device, dtype=torch.int64)
        self._ids_dev.copy_(ids_host, non_blocking=True)
        self._labels_dev.copy_(labels_host, non_blocking=True)
        loss = self.step_device(self._ids_dev, self._labels_dev)
        return float(loss.item())

    def launches_per_step(self) -> int:
        """Number of this library's kernels launched by one step (GEMMs + bandwidth kernels)."""
        L = self.cfg.n_layers
        fwd = 1 + L * (2 + 4 + 1 + 1) + 1 + 1 + 1  # embed; per layer 2 norms, 4 GEMMs, rope, swiglu; final norm, lm_head, CE
        bwd = 1 + L * (2 * 2 + 8 + 1 + 1) + 2 + 2  # embed bwd; per layer norm bwd(2 kernels each), 8 GEMMs, rope, swiglu
        opt = 1
        dp = self.dp.launches_per_step() if self.dp is not None else 0
        return fwd + bwd + opt + dp

    # ------------------------------------------------------------------ checkpoint / resume
    def state_dict(self) -> dict:
        return {
            "params": self.model.flat_params, "m": self.m, "v": self.v, "master": self.master,
            "step": self.step_count, "rng_cpu": torch.get_rng_state(),
            "rng_cuda": torch.cuda.get_rng_state(self.device) if self.device.type == "cuda" else None,
        }

    def load_state_dict(self, sd: dict) -> None:
        self.model.flat_params.copy_(sd["params"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        if self.master is not None and sd.get("master") is not None:
            self.master.copy_(sd["master"])
        self.step_count = int(sd["step"])
        torch.set_rng_state(sd["rng_cpu"])
        if sd.get("rng_cuda") is not None and self.device.type == "cuda":
            torch.cuda.set_rng_state(sd["rng_cuda"], self.device)
