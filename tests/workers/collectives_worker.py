"""Multi-GPU worker (launched by torchrun): device collectives vs an fp64 host reference."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from aws_ofi_nccl_b200.ops import _lib
    from aws_ofi_nccl_b200.parallel.symm import Communicator

    nvls_modes = [False, True] if os.environ.get("B200NET_NVLS_ENABLE", "1") != "0" else [False]
    comm = Communicator(dist.group.WORLD, 64 << 20, dev)
    if not comm.nvls:
        nvls_modes = [False]
    ok = True

    def gather_host(t):
        out = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(out, t)
        return [o.double().cpu() for o in out]

    for dtype in (torch.bfloat16, torch.float32):
        es = 2 if dtype == torch.bfloat16 else 4
        for numel in (8 * world, 4096, 1 << 20, (1 << 20) + 8 * world * 3):
            nbytes = numel * es
            for nvls in nvls_modes:
                # ---------------- all-reduce (scaled)
                torch.manual_seed(1234 + rank)
                x = torch.randn(numel, device=dev).to(dtype)
                comm.view(0, numel, dtype).copy_(x)
                ref = sum(gather_host(x)) / world
                comm.all_reduce(0, nbytes, dtype, scale=1.0 / world, nvls=nvls)
                torch.cuda.synchronize()
                got = comm.view(0, numel, dtype).double().cpu()
                tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
                if not torch.allclose(got, ref, rtol=tol, atol=tol):
                    ok = False
                    print(f"[{rank}] all_reduce mismatch dtype={dtype} n={numel} nvls={nvls} "
                          f"err={(got - ref).abs().max().item()}")
                # ---------------- one-shot all-reduce into a local buffer
                comm.view(0, numel, dtype).copy_(x)
                dist.barrier()
                out = torch.empty(numel, device=dev, dtype=dtype)
                comm.all_reduce_oneshot(0, nbytes, dtype, out, scale=1.0 / world, nvls=nvls)
                torch.cuda.synchronize()
                if not torch.allclose(out.double().cpu(), ref, rtol=tol, atol=tol):
                    ok = False
                    print(f"[{rank}] oneshot mismatch dtype={dtype} n={numel} nvls={nvls}")
                # ---------------- reduce-scatter (bf16 -> fp32 upcast fused)
                if numel % (8 * world) == 0:
                    per = numel // world
                    comm.view(0, numel, dtype).copy_(x)
                    dist.barrier()
                    o = torch.empty(per, device=dev, dtype=torch.float32)
                    comm.reduce_scatter(0, per * es, dtype, o, scale=1.0, nvls=nvls)
                    torch.cuda.synchronize()
                    rs_ref = (ref * world)[rank * per:(rank + 1) * per]
                    if not torch.allclose(o.double().cpu(), rs_ref, rtol=tol, atol=tol * 4):
                        ok = False
                        print(f"[{rank}] reduce_scatter mismatch dtype={dtype} n={numel} nvls={nvls}")
                    # ---------------- all-gather (byte exact)
                    comm.view(0, numel, dtype).zero_()
                    comm.view(0, numel, dtype)[rank * per:(rank + 1) * per].copy_(x[:per])
                    dist.barrier()
                    comm.all_gather(0, per * es, nvls=nvls)
                    torch.cuda.synchronize()
                    parts = gather_host(x[:per].contiguous())
                    ag_ref = torch.cat(parts)
                    if not torch.equal(comm.view(0, numel, dtype).double().cpu(), ag_ref):
                        ok = False
                        print(f"[{rank}] all_gather mismatch dtype={dtype} n={numel} nvls={nvls}")
            # ---------------- all-to-all (byte exact)
            if numel % (8 * world) == 0:
                per = numel // world
                send_off, recv_off = 0, 32 << 20
                comm.view(send_off, numel, dtype).copy_(x)
                comm.view(recv_off, numel, dtype).zero_()
                dist.barrier()
                comm.all_to_all(send_off, recv_off, per * es)
                torch.cuda.synchronize()
                allx = gather_host(x)
                a2a_ref = torch.cat([allx[s][rank * per:(rank + 1) * per] for s in range(world)])
                if not torch.equal(comm.view(recv_off, numel, dtype).double().cpu(), a2a_ref):
                    ok = False
                    print(f"[{rank}] all_to_all mismatch dtype={dtype} n={numel}")
            dist.barrier()

    # ---------------- GIN put+signal latency between ranks 0 and 1 (device timed)
    lat = comm.pingpong_ns(64, iters=200)
    if rank == 0:
        print(f"gin put+signal one-way latency (64 B): {lat:.0f} ns")
        if not (0 < lat < 1e6):
            ok = False

    # ---------------- bounded wait: a signal nobody sets must time out and report, not hang
    comm.set_wait_limit(0.2)
    out = torch.ones(1, device=dev, dtype=torch.int64)
    _lib.check(_lib.load().b200_gin_wait_timeout_probe(comm.id, 7, out.data_ptr(), _lib.stream_ptr()), "probe")
    torch.cuda.synchronize()
    status = _lib.read_status(clear=True)
    if out.item() != 0 or status != 201:
        ok = False
        print(f"[{rank}] timeout probe: waited={out.item()} status={status}")
    comm.set_wait_limit(20.0)

    t = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    final_status = _lib.read_status()
    comm.close()
    dist.destroy_process_group()
    if t.item() != 1 or final_status != 0:
        print(f"[{rank}] FAILED ok={ok} status={final_status}")
        sys.exit(1)
    if rank == 0:
        print("collectives worker OK")


if __name__ == "__main__":
    main()
