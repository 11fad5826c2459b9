"""CPU worker (gloo): every rank serves a memory file descriptor to every other rank through the
library's unix-socket descriptor server (the bootstrap step of the symmetric-memory allocator)
and checks what it can read through the descriptors it fetched."""
import ctypes as C
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    from aws_ofi_nccl_b200.ops import _lib
    from aws_ofi_nccl_b200.parallel import symm  # noqa: F401  (registers the signatures)

    lib = _lib.load()
    tag = [os.urandom(6).hex() if rank == 0 else None]
    dist.broadcast_object_list(tag, src=0)
    names = [f"b200fdtest-{tag[0]}-{r}".encode() for r in range(world)]
    # two descriptors per rank: distinct contents so index mix-ups show
    fds = []
    for idx in range(2):
        fd = os.memfd_create(f"rank{rank}-{idx}")
        os.write(fd, f"payload of rank {rank} index {idx}".encode())
        fds.append(fd)
    arr = (C.c_int * 2)(*fds)
    server = C.c_int(-1)
    nclients = (world - 1) * 2
    _lib.check(lib.b200_fd_server_start(names[rank], arr, 2, nclients, 20000, C.byref(server)), "fd_server_start")
    dist.barrier()
    ok = True
    for r in range(world):
        if r == rank:
            continue
        for idx in range(2):
            got = C.c_int(-1)
            _lib.check(lib.b200_fd_fetch(names[r], idx, 20000, C.byref(got)), f"fd_fetch {r}/{idx}")
            os.lseek(got.value, 0, os.SEEK_SET)
            text = os.read(got.value, 200).decode()
            if text != f"payload of rank {r} index {idx}":
                ok = False
                print(f"[{rank}] descriptor {idx} of rank {r} reads {text!r}", flush=True)
            os.close(got.value)
    left = lib.b200_fd_server_join(server.value)
    if left != 0:
        ok = False
        print(f"[{rank}] {left} clients never fetched", flush=True)
    # a fetch from a name nobody serves must time out with an error, not hang
    got = C.c_int(-1)
    rc = lib.b200_fd_fetch(f"b200fdtest-{tag[0]}-nobody".encode(), 0, 300, C.byref(got))
    if rc == 0:
        ok = False
        print(f"[{rank}] fetch from an unknown server succeeded", flush=True)
    for fd in fds:
        os.close(fd)
    flags = [None] * world
    dist.all_gather_object(flags, ok)
    dist.destroy_process_group()
    if not all(flags):
        sys.exit(1)
    if rank == 0:
        print("FD_EXCHANGE_OK", flush=True)


if __name__ == "__main__":
    main()
