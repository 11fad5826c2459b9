"""Collective sweep: this library's NVLink kernels vs stock NCCL, bus bandwidth per size.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m aws_ofi_nccl_b200.utils.bench_collectives [--max-bytes 1073741824] [--json out.json]

all_reduce (sum), reduce_scatter, all_gather and all_to_all on bf16 (and fp32 for all_reduce)
N(0,1) buffers, sizes doubling from 8 B (rounded up to the 16-byte vector the kernels use) to
--max-bytes, warm-up + timed iterations measured with CUDA events, maximum over ranks.  Bus
bandwidth uses the usual factors: 2(n-1)/n for all_reduce, (n-1)/n for the others.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..parallel.symm import Communicator


def _time(fn, warmup: int, iters: int, dev) -> float:
    """ms per call: the iterations are timed in five batches and the median batch is reported, so a
    single stall (another tenant, a clock change) does not distort a whole size; max over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(dev)
    batches = 5 if iters >= 10 else 1
    per = max(1, iters // batches)
    means = []
    for _ in range(batches):
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(per):
            fn()
        b.record()
        b.synchronize()
        means.append(a.elapsed_time(b) / per)
    means.sort()
    t = torch.tensor([means[len(means) // 2]], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--min-bytes", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--json")
    ap.add_argument("--nblocks", type=int, default=0, help="CTAs per collective kernel (0 = size based)")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    align = 16 * world
    max_bytes = (args.max_bytes + align - 1) // align * align
    comm = Communicator(dist.group.WORLD, 2 * max_bytes, dev)
    rows = []
    torch.manual_seed(rank)
    size = args.min_bytes
    while size <= args.max_bytes:
        nbytes = (size + align - 1) // align * align
        iters = args.iters if nbytes <= (64 << 20) else max(10, args.iters // 5)
        warm = args.warmup if nbytes <= (64 << 20) else 5
        nb = args.nblocks or (4 if nbytes <= (64 << 10) else 16 if nbytes <= (1 << 20) else 64 if nbytes <= (32 << 20) else 128)
        for dtype in (torch.bfloat16, torch.float32):
            es = 2 if dtype == torch.bfloat16 else 4
            numel = nbytes // es
            x = torch.randn(numel, device=dev).to(dtype)
            comm.view(0, numel, dtype).copy_(x)
            y = x.clone()
            ours = _time(lambda: comm.all_reduce(0, nbytes, dtype, nblocks=nb), warm, iters, dev)
            ref = _time(lambda: dist.all_reduce(y), warm, iters, dev)
            f = 2 * (world - 1) / world
            rows.append({"coll": "all_reduce", "dtype": str(dtype).split(".")[-1], "bytes": nbytes, "ours_us": ours * 1e3,
                         "nccl_us": ref * 1e3, "ours_busbw_GBs": nbytes * f / ours / 1e6,
                         "nccl_busbw_GBs": nbytes * f / ref / 1e6})
            if dtype == torch.float32:
                continue
            # small sizes: one-shot latency form
            if nbytes <= (256 << 10):
                out = torch.empty(numel, device=dev, dtype=dtype)
                one = _time(lambda: comm.all_reduce_oneshot(0, nbytes, dtype, out, nblocks=min(nb, 8)), warm, iters, dev)
                rows.append({"coll": "all_reduce_oneshot", "dtype": "bfloat16", "bytes": nbytes, "ours_us": one * 1e3,
                             "nccl_us": ref * 1e3, "ours_busbw_GBs": nbytes * f / one / 1e6,
                             "nccl_busbw_GBs": nbytes * f / ref / 1e6})
            per = nbytes // world
            g = (world - 1) / world
            o = torch.empty(per // es, device=dev, dtype=dtype)
            ours = _time(lambda: comm.reduce_scatter(0, per, dtype, o, nblocks=nb), warm, iters, dev)
            ref = _time(lambda: dist.reduce_scatter_tensor(o, y), warm, iters, dev)
            rows.append({"coll": "reduce_scatter", "dtype": "bfloat16", "bytes": nbytes, "ours_us": ours * 1e3,
                         "nccl_us": ref * 1e3, "ours_busbw_GBs": nbytes * g / ours / 1e6,
                         "nccl_busbw_GBs": nbytes * g / ref / 1e6})
            ours = _time(lambda: comm.all_gather(0, per, nblocks=nb), warm, iters, dev)
            ref = _time(lambda: dist.all_gather_into_tensor(y, o), warm, iters, dev)
            rows.append({"coll": "all_gather", "dtype": "bfloat16", "bytes": nbytes, "ours_us": ours * 1e3,
                         "nccl_us": ref * 1e3, "ours_busbw_GBs": nbytes * g / ours / 1e6,
                         "nccl_busbw_GBs": nbytes * g / ref / 1e6})
            z = torch.empty_like(y)
            ours = _time(lambda: comm.all_to_all(0, max_bytes, per, nblocks=nb), warm, iters, dev)
            ref = _time(lambda: dist.all_to_all_single(z, y), warm, iters, dev)
            rows.append({"coll": "all_to_all", "dtype": "bfloat16", "bytes": nbytes, "ours_us": ours * 1e3,
                         "nccl_us": ref * 1e3, "ours_busbw_GBs": nbytes * g / ours / 1e6,
                         "nccl_busbw_GBs": nbytes * g / ref / 1e6})
        if rank == 0:
            for r in rows[-6:]:
                if r["bytes"] == nbytes:
                    print(json.dumps(r), flush=True)
        size *= 2
    lat = comm.pingpong_ns(8, iters=2000) if world >= 2 else 0.0
    if rank == 0:
        print(json.dumps({"gin_put_signal_one_way_ns": lat, "payload_bytes": 8, "nvls": comm.nvls, "world": world}))
        if args.json:
            with open(args.json, "w") as fjs:
                json.dump({"world": world, "nvls": comm.nvls, "gin_put_signal_one_way_ns": lat, "rows": rows}, fjs, indent=1)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
