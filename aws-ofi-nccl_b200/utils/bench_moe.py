"""MoE expert-parallel dispatch / combine: device-initiated kernels vs an NCCL all_to_all baseline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m aws_ofi_nccl_b200.utils.bench_moe [--tokens 4096] [--hidden 7168] [--experts 256] [--topk 8] [--json out.json]

Per rank: `tokens` bf16 N(0,1) rows, top-k routing from the softmax of N(0,1) gate logits.  Timed
on the device with CUDA events, L2 flushed between iterations, maximum over ranks:

  dispatch_bf16 / dispatch_fp8 : route + dispatch (fp8: e4m3 payload with one fp32 scale per 128 elements)
  combine                      : expert rows back to their tokens + gate-weighted sum
  baseline_*                   : argsort + index_select + NCCL all_to_all_single with split sizes
                                 (and the reverse + index_add for the combine)

Roofline: bytes that must leave each GPU over NVLink / measured peer-copy bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..parallel.expert_parallel import ExpertParallel
from ..parallel.symm import Communicator
from .timing import flush_l2

NVLINK_GBS_MEASURED = 770.0


def _time(fn, warmup: int, iters: int, dev) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(dev)
    total = 0.0
    for _ in range(iters):
        flush_l2()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        total += a.elapsed_time(b)
    t = torch.tensor([total / iters], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    T, H, E, k = args.tokens, args.hidden, args.experts, args.topk
    el = E // world
    comm = Communicator(dist.group.WORLD, ExpertParallel.window_bytes(world, T, H, E, k, 2.0) + (1 << 20), dev)
    ep = ExpertParallel(comm, T, H, E, k, capacity_factor=2.0)
    torch.manual_seed(rank)
    x = torch.randn(T, H, device=dev).bfloat16()
    w, idx = torch.topk(torch.softmax(torch.randn(T, E, device=dev), -1), k, dim=-1)
    idx = idx.to(torch.int32).contiguous()
    w = w.contiguous()
    remote_frac = (world - 1) / world
    rows = []

    def report(name, ms, base_ms, link_bytes):
        bound = link_bytes / (NVLINK_GBS_MEASURED * 1e9) * 1e3
        row = {"op": name, "world": world, "ours_ms": ms, "baseline_ms": base_ms,
               "speedup": (base_ms / ms) if base_ms else None, "nvlink_GBs_per_gpu": link_bytes / ms / 1e6,
               "roofline_ms": bound, "frac_of_measured_roofline": (bound / ms) if bound else None}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    # ---- baseline: sort by expert, exchange split sizes on the host, all_to_all_single
    def base_dispatch():
        flat = idx.flatten().long()
        order = torch.argsort(flat, stable=True)
        send = x[order // k]
        counts = torch.bincount(flat // el, minlength=world)
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts)
        in_split, out_split = counts.tolist(), recv_counts.tolist()
        recv = torch.empty(sum(out_split), H, device=dev, dtype=torch.bfloat16)
        dist.all_to_all_single(recv, send, out_split, in_split)
        return recv, order, in_split, out_split

    state = {}

    def base_dispatch_keep():
        state["d"] = base_dispatch()

    def base_combine():
        recv, order, in_split, out_split = state["d"]
        back = torch.empty(T * k, H, device=dev, dtype=torch.bfloat16)
        dist.all_to_all_single(back, recv, in_split, out_split)
        out = torch.zeros(T, H, device=dev, dtype=torch.float32)
        out.index_add_(0, order // k, back.float() * w.flatten()[order][:, None])
        return out.bfloat16()

    base_d = _time(base_dispatch_keep, args.warmup, args.iters, dev)
    base_c = _time(base_combine, args.warmup, args.iters, dev)

    def ours_dispatch(fp8):
        ep.route(idx)
        ep.dispatch_raw(x, idx, w, fp8=fp8)

    d16 = _time(lambda: ours_dispatch(False), args.warmup, args.iters, dev)
    report("dispatch_bf16", d16, base_d, T * k * H * 2 * remote_frac)
    # combine needs matching dispatch state: rows of the last bf16 dispatch are in place
    n_rows = int(ep.expert_offsets[-1].item())
    y = ep.recv_rows(False)[:n_rows].clone()
    out = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    c16 = _time(lambda: ep.combine_raw(y, w, out), args.warmup, args.iters, dev)
    report("combine_bf16", c16, base_c, T * k * H * 2 * remote_frac)
    d8 = _time(lambda: ours_dispatch(True), args.warmup, args.iters, dev)
    report("dispatch_fp8", d8, base_d, T * k * (H + H // 128 * 4) * remote_frac)
    ref = x.float() * w.sum(-1, keepdim=True)
    err = ((out.float() - ref).norm() / ref.norm()).item()
    if rank == 0:
        print(json.dumps({"check": "combine(dispatch(x)) == x * sum(w)", "rel_err": err, "rows_received": n_rows,
                          "capacity_rows": ep.capacity}), flush=True)
        if args.json:
            with open(args.json, "w") as f:
                json.dump({"world": world, "tokens": T, "hidden": H, "experts": E, "topk": k,
                           "nvlink_gbs": NVLINK_GBS_MEASURED, "rows": rows, "roundtrip_rel_err": err}, f, indent=1)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
