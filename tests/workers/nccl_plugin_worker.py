"""Multi-GPU worker: stock NCCL (torch.distributed) with its intra-node transports disabled, so all
traffic crosses this repository's net plugin.  Checks all_reduce / all_gather / reduce_scatter /
all_to_all / send-recv results against host references and prints NCCL's own view of the plugin."""
import os
import sys

import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ok = True
    for dtype in (torch.float32, torch.bfloat16):
        for numel in (8, 1024, 1 << 16, 1 << 20, (1 << 22) + 40):
            torch.manual_seed(7 + rank)
            x = torch.randn(numel, device=dev).to(dtype)
            xs = [torch.empty_like(x) for _ in range(world)]
            ref_in = x.clone()
            dist.all_reduce(x)
            dist.all_gather(xs, ref_in)
            ref = sum(t.double() for t in xs)
            tol = 1e-5 if dtype == torch.float32 else 5e-2
            if not torch.allclose(x.double(), ref, rtol=tol, atol=tol * 4):
                ok = False
                print(f"[{rank}] all_reduce mismatch {dtype} {numel}: {(x.double() - ref).abs().max().item()}")
            for r in range(world):
                torch.manual_seed(7 + r)
                want = torch.randn(numel, device=dev).to(dtype)
                if not torch.equal(xs[r], want):
                    ok = False
                    print(f"[{rank}] all_gather mismatch {dtype} {numel} from {r}")
            if numel % world == 0:
                out = torch.empty(numel // world, device=dev, dtype=dtype)
                dist.reduce_scatter_tensor(out, ref_in)
                if not torch.allclose(out.double(), ref[rank * (numel // world):(rank + 1) * (numel // world)],
                                      rtol=tol, atol=tol * 4):
                    ok = False
                    print(f"[{rank}] reduce_scatter mismatch {dtype} {numel}")
                a2a = torch.empty_like(ref_in)
                dist.all_to_all_single(a2a, ref_in)
                per = numel // world
                want = torch.cat([xs[s][rank * per:(rank + 1) * per] for s in range(world)])
                if not torch.equal(a2a, want):
                    ok = False
                    print(f"[{rank}] all_to_all mismatch {dtype} {numel}")
    # point-to-point ring
    t = torch.full((1 << 18,), float(rank), device=dev)
    r = torch.empty_like(t)
    ops = [dist.P2POp(dist.isend, t, (rank + 1) % world), dist.P2POp(dist.irecv, r, (rank - 1) % world)]
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    if not torch.all(r == float((rank - 1) % world)):
        ok = False
        print(f"[{rank}] send/recv ring mismatch")
    # a quick bandwidth figure through the plugin
    big = torch.randn(64 << 20, device=dev)
    for _ in range(3):
        dist.all_reduce(big)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(5):
        dist.all_reduce(big)
    b.record()
    b.synchronize()
    ms = a.elapsed_time(b) / 5
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        busbw = big.numel() * 4 * 2 * (world - 1) / world / ms / 1e6
        print(f"plugin all_reduce 256 MiB fp32: {ms:.2f} ms, busbw {busbw:.1f} GB/s")
    dist.destroy_process_group()
    if flag.item() != 1:
        sys.exit(1)
    if rank == 0:
        print("nccl plugin worker OK")


if __name__ == "__main__":
    main()
