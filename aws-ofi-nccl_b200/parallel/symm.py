"""Symmetric memory and the NVLink communicator.

``SymmetricMemory`` allocates one VMM chunk per rank, exchanges the chunks' file descriptors
between the ranks' processes (unix sockets), maps every peer chunk locally and, when the GPUs
support it, binds an NVSwitch multicast object over them.  ``Communicator`` pairs a data window
with a control pad (barrier flags, signals, counters) and exposes the device collectives of
``csrc/kernels/collectives.cu``.

torch.distributed is used only as the bootstrap (exchange of socket names, host barriers).
"""
from __future__ import annotations

import ctypes as C
import os
import uuid

import torch
import torch.distributed as dist

from ..ops import _lib

_vp, _i, _sz, _f, _ull = C.c_void_p, C.c_int, C.c_size_t, C.c_float, C.c_ulonglong
_P = C.POINTER

_lib.register("b200_symm_multicast_supported", [_i], _i)
_lib.register("b200_symm_alloc", [_sz, _i, _i, _i, _i, _P(_i), _P(_sz)], _i)
_lib.register("b200_symm_export_fd", [_i, _i, _P(_i)], _i)
_lib.register("b200_fd_server_start", [C.c_char_p, _P(_i), _i, _i, _i, _P(_i)], _i)
_lib.register("b200_fd_server_join", [_i], _i)
_lib.register("b200_fd_fetch", [C.c_char_p, _i, _i, _P(_i)], _i)
_lib.register("b200_symm_map", [_i, _P(_i), _P(_vp)], _i)
_lib.register("b200_symm_mc_create", [_i], _i)
_lib.register("b200_symm_mc_import", [_i, _i], _i)
_lib.register("b200_symm_mc_add_device", [_i], _i)
_lib.register("b200_symm_mc_bind_map", [_i, _P(_vp)], _i)
_lib.register("b200_symm_free", [_i], _i)
_lib.register("b200_comm_create", [_i, _i, _vp, _sz, _vp, _vp, _sz, _ull, _P(_i)], _i)
_lib.register("b200_comm_destroy", [_i], _i)
_lib.register("b200_comm_set_wait_limit", [_i, _ull], _i)
_lib.register("b200_all_reduce", [_i, _sz, _sz, _i, _f, _i, _i, _i, _vp], _i)
_lib.register("b200_all_reduce_oneshot", [_i, _sz, _sz, _i, _f, _i, _vp, _i, _i, _vp], _i)
_lib.register("b200_reduce_scatter", [_i, _sz, _sz, _i, _f, _i, _vp, _i, _i, _i, _vp], _i)
_lib.register("b200_all_gather", [_i, _sz, _sz, _i, _i, _i, _vp], _i)
_lib.register("b200_all_to_all", [_i, _sz, _sz, _sz, _i, _i, _vp], _i)
_lib.register("b200_barrier", [_i, _i, _vp], _i)
_lib.register("b200_gin_pingpong", [_i, _sz, _sz, _i, _i, _vp, _vp], _i)
_lib.register("b200_gin_wait_timeout_probe", [_i, _i, _vp, _vp], _i)
for _n in ("b200_symm_multicast_supported", "b200_symm_alloc", "b200_symm_export_fd", "b200_fd_server_start",
           "b200_fd_server_join", "b200_fd_fetch", "b200_symm_map", "b200_symm_mc_create", "b200_symm_mc_import",
           "b200_symm_mc_add_device", "b200_symm_mc_bind_map", "b200_symm_free", "b200_comm_create",
           "b200_comm_destroy", "b200_comm_set_wait_limit"):
    _lib.set_kernels_per_call(_n, 0)

PAD_BYTES = 2 << 20
_DTYPE_CODE = {torch.bfloat16: 0, torch.float32: 1}


class _RawCudaBuffer:
    """Exposes a raw device pointer through __cuda_array_interface__ so torch can alias it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def tensor_from_ptr(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    return torch.as_tensor(_RawCudaBuffer(ptr, nbytes), device=device)


class SymmetricMemory:
    """`nbytes` per rank, identical on all ranks.  `local` is this rank's chunk as a uint8 tensor,
    `peer_ptr(i)` the local address of rank i's chunk, `mc_ptr` the multicast alias (0 if none)."""

    def __init__(self, group: dist.ProcessGroup, nbytes: int, device: torch.device, multicast: bool | None = None,
                 timeout_ms: int = 60000):
        lib = _lib.load()
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.device = device
        dev = device.index if device.index is not None else torch.cuda.current_device()
        if multicast is None:
            multicast = os.environ.get("B200NET_NVLS_ENABLE", "1") != "0" and self.world > 1
        if multicast and lib.b200_symm_multicast_supported(dev) != 1:
            multicast = False
        flags = [None] * self.world
        dist.all_gather_object(flags, bool(multicast), group=group)
        multicast = all(flags)
        idc, chunk = _i(-1), _sz(0)
        _lib.check(lib.b200_symm_alloc(nbytes, dev, self.world, self.rank, int(multicast), C.byref(idc), C.byref(chunk)),
                   "symm_alloc")
        self.id, self.chunk = idc.value, chunk.value
        # ---- exchange the chunk descriptors: every rank serves its fd to world-1 peers
        tag = [None]
        if self.rank == 0:
            tag[0] = uuid.uuid4().hex[:16]
        dist.broadcast_object_list(tag, src=dist.get_global_rank(group, 0), group=group)
        names = [f"b200symm-{tag[0]}-{r}".encode() for r in range(self.world)]
        fd = _i(-1)
        _lib.check(lib.b200_symm_export_fd(self.id, 0, C.byref(fd)), "export_fd")
        own_fds = [fd.value]
        if multicast and self.rank == 0:
            _lib.check(lib.b200_symm_mc_create(self.id), "mc_create")
            mfd = _i(-1)
            _lib.check(lib.b200_symm_export_fd(self.id, 1, C.byref(mfd)), "export mc fd")
            own_fds.append(mfd.value)
        nclients = (self.world - 1) * (2 if (multicast and self.rank == 0) else 1)
        server = _i(-1)
        arr = (_i * len(own_fds))(*own_fds)
        if self.world > 1:
            _lib.check(lib.b200_fd_server_start(names[self.rank], arr, len(own_fds), nclients, timeout_ms,
                                                C.byref(server)), "fd_server_start")
        dist.barrier(group=group)
        fds = (_i * self.world)(*([-1] * self.world))
        for r in range(self.world):
            if r == self.rank:
                continue
            got = _i(-1)
            _lib.check(lib.b200_fd_fetch(names[r], 0, timeout_ms, C.byref(got)), f"fd_fetch from rank {r}")
            fds[r] = got.value
        mc_fd = -1
        if multicast and self.rank != 0:
            got = _i(-1)
            _lib.check(lib.b200_fd_fetch(names[0], 1, timeout_ms, C.byref(got)), "fd_fetch multicast")
            mc_fd = got.value
        if self.world > 1:
            left = lib.b200_fd_server_join(server.value)
            if left != 0:
                raise RuntimeError(f"fd server: {left} peers never fetched their descriptor")
        for f in own_fds:
            os.close(f)
        base = _vp(0)
        _lib.check(lib.b200_symm_map(self.id, fds, C.byref(base)), "symm_map")
        self.base = base.value
        self.mc_ptr = 0
        if multicast:
            if self.rank != 0:
                _lib.check(lib.b200_symm_mc_import(self.id, mc_fd), "mc_import")
            _lib.check(lib.b200_symm_mc_add_device(self.id), "mc_add_device")
            dist.barrier(group=group)
            mp = _vp(0)
            _lib.check(lib.b200_symm_mc_bind_map(self.id, C.byref(mp)), "mc_bind_map")
            self.mc_ptr = mp.value
        dist.barrier(group=group)
        self.local = tensor_from_ptr(self.base + self.rank * self.chunk, self.chunk, device)
        self.local.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        self._freed = False

    def peer_ptr(self, r: int) -> int:
        return self.base + r * self.chunk

    def free(self) -> None:
        if self._freed:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self.local = None
        _lib.load().b200_symm_free(self.id)
        self._freed = True


class Communicator:
    """A data window of `window_bytes` per rank plus the control pad; device collectives act on
    byte ranges of the window.  `channel` selects an independent set of barrier slots, so two
    streams may run collectives of the same communicator concurrently on different channels."""

    def __init__(self, group: dist.ProcessGroup, window_bytes: int, device: torch.device,
                 multicast: bool | None = None, wait_limit_s: float = 20.0):
        self.group, self.device = group, device
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.window = SymmetricMemory(group, window_bytes, device, multicast)
        self.pad = SymmetricMemory(group, PAD_BYTES, device, multicast=False)
        cid = _i(-1)
        _lib.check(_lib.load().b200_comm_create(self.rank, self.world, self.window.base, self.window.chunk,
                                                self.window.mc_ptr or None, self.pad.base, self.pad.chunk,
                                                int(wait_limit_s * 1e9), C.byref(cid)), "comm_create")
        self.id = cid.value
        dist.barrier(group=group)
        self.nvls = bool(self.window.mc_ptr)
        self.local = self.window.local  # uint8 view of this rank's window

    # ---- views
    def view(self, offset: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        return self.local[offset:offset + nbytes].view(dtype)

    def set_wait_limit(self, seconds: float) -> None:
        _lib.check(_lib.load().b200_comm_set_wait_limit(self.id, int(seconds * 1e9)), "set_wait_limit")

    # ---- collectives on byte ranges of the window (stream-ordered on the current stream)
    def all_reduce(self, offset: int, nbytes: int, dtype: torch.dtype, scale: float = 1.0, nvls: bool | None = None,
                   nblocks: int = 0, channel: int = 0) -> None:
        use = self.nvls if nvls is None else (nvls and self.nvls)
        _lib.check(_lib.load().b200_all_reduce(self.id, offset, nbytes, _DTYPE_CODE[dtype], scale, int(use), nblocks,
                                               channel, _lib.stream_ptr()), "all_reduce")

    def all_reduce_oneshot(self, offset: int, nbytes: int, dtype: torch.dtype, out: torch.Tensor, scale: float = 1.0,
                           nvls: bool | None = None, nblocks: int = 0, channel: int = 0) -> None:
        use = self.nvls if nvls is None else (nvls and self.nvls)
        _lib.check(_lib.load().b200_all_reduce_oneshot(self.id, offset, nbytes, _DTYPE_CODE[dtype], scale, int(use),
                                                       out.data_ptr(), nblocks, channel, _lib.stream_ptr()),
                   "all_reduce_oneshot")

    def reduce_scatter(self, offset: int, bytes_per_rank: int, dtype: torch.dtype, out: torch.Tensor,
                       scale: float = 1.0, nvls: bool | None = None, nblocks: int = 0, channel: int = 0) -> None:
        use = self.nvls if nvls is None else (nvls and self.nvls)
        out_fp32 = int(dtype == torch.bfloat16 and out.dtype == torch.float32)
        _lib.check(_lib.load().b200_reduce_scatter(self.id, offset, bytes_per_rank, _DTYPE_CODE[dtype], scale, int(use),
                                                   out.data_ptr(), out_fp32, nblocks, channel, _lib.stream_ptr()),
                   "reduce_scatter")

    def all_gather(self, offset: int, bytes_per_rank: int, nvls: bool | None = None, nblocks: int = 0,
                   channel: int = 0) -> None:
        use = self.nvls if nvls is None else (nvls and self.nvls)
        _lib.check(_lib.load().b200_all_gather(self.id, offset, bytes_per_rank, int(use), nblocks, channel,
                                               _lib.stream_ptr()), "all_gather")

    def all_to_all(self, send_offset: int, recv_offset: int, bytes_per_peer: int, nblocks: int = 0,
                   channel: int = 0) -> None:
        _lib.check(_lib.load().b200_all_to_all(self.id, send_offset, recv_offset, bytes_per_peer, nblocks, channel,
                                               _lib.stream_ptr()), "all_to_all")

    def barrier(self, channel: int = 0) -> None:
        _lib.check(_lib.load().b200_barrier(self.id, channel, _lib.stream_ptr()), "barrier")

    def pingpong_ns(self, nbytes: int, iters: int = 1000, offset: int = 0, signal: int = 0) -> float:
        """Device-timed put+signal round trips between ranks 0 and 1; returns ns per one-way hop."""
        out = torch.zeros(1, device=self.device, dtype=torch.int64)
        _lib.check(_lib.load().b200_gin_pingpong(self.id, offset, nbytes, iters, signal, out.data_ptr(),
                                                 _lib.stream_ptr()), "gin_pingpong")
        torch.cuda.synchronize(self.device)
        return float(out.item()) / (2.0 * iters)

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        _lib.load().b200_comm_destroy(self.id)
        self.local = None
        self.window.free()
        self.pad.free()
