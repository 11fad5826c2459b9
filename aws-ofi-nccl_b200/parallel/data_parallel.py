"""Data parallelism over NVLink: gradient averaging fused with its scale, overlapped with backward.

The model's flat bf16 gradient buffer IS the symmetric window of an NVLink communicator, so the
backward GEMMs write weight gradients straight into memory that peers (and the NVSwitch multicast
object) can address.  As soon as every parameter of a bucket has its gradient, the bucket is
all-reduced in place on a side stream by ``all_reduce_kernel`` (sum in the switch, multiplied by
1/N before the single rounding back to bf16) while backward continues with the next layer.
"""
from __future__ import annotations

import math
import os

import torch
import torch.distributed as dist

from .symm import Communicator


class GradReducer:
    def __init__(self, group: dist.ProcessGroup, device: torch.device, bucket_bytes: int | None = None,
                 nblocks: int | None = None, nvls: bool | None = None, channel: int = 1):
        self.group, self.device = group, device
        self.world = dist.get_world_size(group)
        self.bucket_bytes = bucket_bytes or int(os.environ.get("B200NET_DP_BUCKET_MB", "512")) << 20
        self.nblocks = nblocks or int(os.environ.get("B200NET_DP_BLOCKS", "48"))
        self.nvls = nvls
        self.channel = channel
        self.comm: Communicator | None = None
        self.stream = torch.cuda.Stream(device=device)
        self.buckets: list[dict] = []
        self._launched = 0

    # ------------------------------------------------------------------ setup
    def allocate_grad_buffer(self, numel: int) -> torch.Tensor:
        self.comm = Communicator(self.group, numel * 2, self.device, multicast=self.nvls)
        return self.comm.view(0, numel, torch.bfloat16)

    def attach(self, model) -> None:
        """Cut the flat buffer into contiguous buckets, walking parameters in backward order."""
        items = sorted(((off, math.prod(shape), name) for name, (off, shape) in model.offsets.items()), reverse=True)
        self.buckets = []
        cur = None
        for off, n, name in items:
            end = off + (n + 127) // 128 * 128
            if cur is None or (cur["end"] - off) * 2 > self.bucket_bytes:
                cur = {"start": off, "end": end, "pending": 0, "names": []}
                self.buckets.append(cur)
            cur["start"] = off
            cur["names"].append(name)
        self._bucket_of = {}
        for i, b in enumerate(self.buckets):
            for name in b["names"]:
                self._bucket_of[name] = i
        model.set_grad_ready_hook(self._on_grad_ready)

    # ------------------------------------------------------------------ per step
    def begin_step(self) -> None:
        for b in self.buckets:
            b["pending"] = len(b["names"])
        self._launched = 0

    def _on_grad_ready(self, param) -> None:
        b = self.buckets[self._bucket_of[param.param_name]]
        b["pending"] -= 1
        if b["pending"] == 0:
            self._reduce(b)

    def _reduce(self, b: dict) -> None:
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self.stream.wait_event(ev)
        with torch.cuda.stream(self.stream):
            self.comm.all_reduce(b["start"] * 2, (b["end"] - b["start"]) * 2, torch.bfloat16,
                                 scale=1.0 / self.world, nvls=self.nvls, nblocks=self.nblocks, channel=self.channel)
        self._launched += 1

    def finish_step(self) -> None:
        for b in self.buckets:  # parameters that took no part in this backward still need reducing
            if b["pending"] > 0:
                b["pending"] = 0
                self._reduce(b)
        torch.cuda.current_stream(self.device).wait_stream(self.stream)

    def launches_per_step(self) -> int:
        return len(self.buckets)

    def close(self) -> None:
        if self.comm is not None:
            self.comm.close()
            self.comm = None


class NcclGradReducer:
    """The same bucketed, overlapped gradient averaging, issued through ``torch.distributed`` (NCCL)
    instead of this library's own kernels.  With NCCL_NET_PLUGIN pointing at this repository's
    plugin and NCCL's intra-node transports off, every bucket crosses the plugin's isend / irecv and
    the tuner it carries; with stock settings it is the NVLink baseline.

    mode "allreduce": each bucket is all-reduced as soon as its last gradient is written (data
    parallel).  mode "zero": gradients are reduce-scattered, every rank runs AdamW on its own
    contiguous shard only, and the updated parameters are all-gathered (sharded optimizer state, the
    traffic pattern of FSDP / ZeRO: reduce-scatter + all-gather instead of all-reduce)."""

    def __init__(self, group: dist.ProcessGroup, device: torch.device, bucket_bytes: int | None = None, mode: str = "allreduce"):
        assert mode in ("allreduce", "zero")
        self.group, self.device, self.mode = group, device, mode
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.bucket_bytes = bucket_bytes or int(os.environ.get("B200NET_DP_BUCKET_MB", "512")) << 20
        self.stream = torch.cuda.Stream(device=device)
        self.buckets: list[dict] = []
        self.grads: torch.Tensor | None = None
        self.grad_scale = 1.0 / self.world   # the optimizer applies it (NCCL sums)
        # The first steps allocate device memory and load kernels for the first time. When NCCL's
        # traffic crosses a transport whose proxy thread has to launch device work for the collective
        # to finish (this repository's plugin), such a call can wait for the device while the
        # collective waits for the proxy, so these steps keep collectives apart from everything
        # else: reductions run after backward, with the device idle before and after.
        self.settle_steps = int(os.environ.get("B200NET_DP_SETTLE_STEPS", "2"))
        self._steps_done = 0

    def allocate_grad_buffer(self, numel: int) -> torch.Tensor:
        pad = (numel + 128 * self.world - 1) // (128 * self.world) * (128 * self.world)
        self.grads = torch.zeros(pad, device=self.device, dtype=torch.bfloat16)
        return self.grads[:numel]

    def attach(self, model) -> None:
        items = sorted(((off, math.prod(shape), name) for name, (off, shape) in model.offsets.items()), reverse=True)
        self.buckets, cur = [], None
        for off, n, name in items:
            end = off + (n + 127) // 128 * 128
            if cur is None or (cur["end"] - off) * 2 > self.bucket_bytes:
                cur = {"start": off, "end": end, "pending": 0, "names": []}
                self.buckets.append(cur)
            cur["start"] = off
            cur["names"].append(name)
        self._bucket_of = {name: i for i, b in enumerate(self.buckets) for name in b["names"]}
        if self.mode == "allreduce":
            model.set_grad_ready_hook(self._on_grad_ready)

    def begin_step(self) -> None:
        for b in self.buckets:
            b["pending"] = len(b["names"])

    def _settling(self) -> bool:
        return self._steps_done < self.settle_steps

    def _on_grad_ready(self, param) -> None:
        b = self.buckets[self._bucket_of[param.param_name]]
        b["pending"] -= 1
        if b["pending"] == 0 and not self._settling():
            self._reduce(b)
        elif b["pending"] == 0:
            b["pending"] = -1   # reduced in finish_step

    def _reduce(self, b: dict) -> None:
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            dist.all_reduce(self.grads[b["start"]:b["end"]], group=self.group)

    def finish_step(self) -> None:
        settling = self._settling()
        if settling:
            torch.cuda.synchronize(self.device)
        if self.mode == "allreduce":
            for b in self.buckets:
                if b["pending"] != 0:
                    b["pending"] = 0
                    self._reduce(b)
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
        else:
            shard = self.grads.numel() // self.world
            dist.reduce_scatter_tensor(self.grads[self.rank * shard:(self.rank + 1) * shard], self.grads, group=self.group)
        if settling:
            torch.cuda.synchronize(self.device)
        self._steps_done += 1

    # ---- sharded optimizer support (mode "zero")
    def shard_range(self, numel: int) -> tuple[int, int]:
        shard = self.grads.numel() // self.world
        return min(self.rank * shard, numel), min((self.rank + 1) * shard, numel)

    def gather_params(self, flat_params: torch.Tensor) -> None:
        """All ranks receive every shard of the updated parameters (in place)."""
        shard = self.grads.numel() // self.world
        n = flat_params.numel()
        settling = self._steps_done <= self.settle_steps
        if n == shard * self.world:
            mine = flat_params[self.rank * shard:(self.rank + 1) * shard].clone()
            if settling:
                torch.cuda.synchronize(self.device)
            dist.all_gather_into_tensor(flat_params, mine, group=self.group)
            if settling:
                torch.cuda.synchronize(self.device)
            return
        full = torch.empty(shard * self.world, device=self.device, dtype=flat_params.dtype)
        mine = torch.zeros(shard, device=self.device, dtype=flat_params.dtype)
        lo, hi = self.shard_range(n)
        mine[:hi - lo].copy_(flat_params[lo:hi])
        dist.all_gather_into_tensor(full, mine, group=self.group)
        flat_params.copy_(full[:n])

    def launches_per_step(self) -> int:
        return 0   # NCCL's kernels, not this library's

    def close(self) -> None:
        self.grads = None
