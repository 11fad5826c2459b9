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
