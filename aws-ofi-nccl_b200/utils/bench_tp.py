"""Fused compute+collective kernels vs the unfused library baseline, with roofline fractions.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m aws_ofi_nccl_b200.utils.bench_tp [--tokens 8192] [--hidden 4096] [--ffn 14336] [--json out.json]

For a sequence-parallel SwiGLU MLP of the given size (defaults: Llama-3-8B, 8192 tokens per step)
this times, on the device with CUDA events and as the maximum over ranks:

  ag_gemm_swiglu : all-gather(x) -> x W_gu^T -> SwiGLU      fused kernel  vs  NCCL all_gather + matmul + silu*mul
  gemm_rs        : act W_down^T -> reduce-scatter            fused kernel  vs  matmul + NCCL reduce_scatter
  mlp_fwd_bwd    : TensorParallelMLP forward + backward      fused         vs  the same with NCCL + matmul

Roofline per fused kernel: the slower of FLOPs / measured bf16 GEMM peak and NVLink bytes (per
direction, per GPU) / measured peer-copy bandwidth.  Inputs and outputs together exceed the L2, and
the L2 is flushed between timed iterations.
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch
import torch.distributed as dist

from ..parallel import tensor_parallel as tp
from ..parallel.symm import Communicator
from .timing import flush_l2

NVLINK_GBS_MEASURED = 770.0   # peer copy, per direction per GPU, measured on this hardware generation
FALLBACK_TFLOPS = 1590.0


def _peak_tflops() -> tuple[float, str]:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    try:
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), "measured"
    except (OSError, KeyError, ValueError):
        return FALLBACK_TFLOPS, "fallback"


def _time(fn, warmup: int, iters: int, dev) -> float:
    """ms per call: every iteration is timed on its own after an L2 flush; max over ranks of the mean."""
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
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--helpers", type=int, default=16, help="mover CTAs of the all-gather kernels")
    ap.add_argument("--json")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    T, H, F = args.tokens, args.hidden, args.ffn
    Fl, Ts = F // world, T // world
    comm = Communicator(dist.group.WORLD, tp.TensorParallelMLP.window_bytes(T, H), dev)
    mlp = tp.TensorParallelMLP(comm, T, H, F, n_helpers=args.helpers)
    peak, peak_src = _peak_tflops()
    torch.manual_seed(rank)
    x_shard = torch.randn(Ts, H, device=dev).bfloat16()
    dy_shard = torch.randn(Ts, H, device=dev).bfloat16()
    w_gu, w_down = mlp.w_gate_up.detach(), mlp.w_down.detach()
    gu = torch.empty(T, 2 * Fl, device=dev, dtype=torch.bfloat16)
    act = torch.empty(T, Fl, device=dev, dtype=torch.bfloat16)
    y_shard = torch.empty(Ts, H, device=dev, dtype=torch.bfloat16)
    x_full = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    y_full = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    rows = []

    def report(name, ours_ms, base_ms, flops, link_bytes):
        t_math = flops / (peak * 1e12) * 1e3
        t_link = link_bytes / (NVLINK_GBS_MEASURED * 1e9) * 1e3
        bound = max(t_math, t_link)
        row = {"op": name, "world": world, "ours_ms": ours_ms, "baseline_ms": base_ms, "speedup": base_ms / ours_ms,
               "tflops": flops / ours_ms / 1e9, "roofline_ms": bound, "roofline_bound": "math" if t_math >= t_link else "nvlink",
               f"frac_of_{peak_src}_roofline": bound / ours_ms}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    # ---- all-gather -> GEMM -> SwiGLU
    def fused_up():
        mlp.x_full[rank * Ts:(rank + 1) * Ts].copy_(x_shard)
        tp.ag_gemm(comm, mlp.x_off, T, H, w_gu, out=gu, act=act, swiglu=True, n_movers=args.helpers)

    def base_up():
        dist.all_gather_into_tensor(x_full, x_shard)
        g = x_full @ w_gu.t()   # timing only: the baseline reads the product as gate | up halves
        torch.mul(torch.nn.functional.silu(g[:, :Fl]), g[:, Fl:], out=act)

    flops_up = 2.0 * T * H * 2 * Fl
    report("ag_gemm_swiglu", _time(fused_up, args.warmup, args.iters, dev), _time(base_up, args.warmup, args.iters, dev),
           flops_up, (world - 1) * Ts * H * 2)

    # ---- GEMM -> reduce-scatter
    def fused_down():
        tp.gemm_rs(comm, act, w_down, mlp.stage_off, y_shard)

    def base_down():
        torch.matmul(act, w_down.t(), out=y_full)
        dist.reduce_scatter_tensor(y_shard, y_full)

    flops_down = 2.0 * T * H * Fl
    report("gemm_rs", _time(fused_down, args.warmup, args.iters, dev), _time(base_down, args.warmup, args.iters, dev),
           flops_down, (world - 1) * Ts * H * 2)

    # ---- whole MLP, forward + backward
    xs = x_shard.clone().requires_grad_(True)

    def fused_mlp():
        mlp.w_gate_up.grad = None
        mlp.w_down.grad = None
        mlp(xs).backward(dy_shard)

    wgu_b = w_gu.clone().requires_grad_(True)
    wd_b = w_down.clone().requires_grad_(True)

    class _AG(torch.autograd.Function):
        @staticmethod
        def forward(ctx, t):
            out = torch.empty(T, H, device=dev, dtype=t.dtype)
            dist.all_gather_into_tensor(out, t.contiguous())
            return out

        @staticmethod
        def backward(ctx, g):
            out = torch.empty(Ts, H, device=dev, dtype=g.dtype)
            dist.reduce_scatter_tensor(out, g.contiguous())
            return out

    class _RS(torch.autograd.Function):
        @staticmethod
        def forward(ctx, t):
            out = torch.empty(Ts, H, device=dev, dtype=t.dtype)
            dist.reduce_scatter_tensor(out, t.contiguous())
            return out

        @staticmethod
        def backward(ctx, g):
            out = torch.empty(T, H, device=dev, dtype=g.dtype)
            dist.all_gather_into_tensor(out, g.contiguous())
            return out

    def base_mlp():
        wgu_b.grad = None
        wd_b.grad = None
        xf = _AG.apply(xs)
        g = xf @ wgu_b.t()
        a = torch.nn.functional.silu(g[:, :Fl]) * g[:, Fl:]
        _RS.apply(a @ wd_b.t()).backward(dy_shard)

    flops_mlp = 3.0 * (flops_up + flops_down)
    report("mlp_fwd_bwd", _time(fused_mlp, args.warmup, args.iters, dev), _time(base_mlp, args.warmup, args.iters, dev),
           flops_mlp, 4 * (world - 1) * Ts * H * 2)

    if rank == 0 and args.json:
        with open(args.json, "w") as f:
            json.dump({"world": world, "tokens": T, "hidden": H, "ffn": F, "peak_tflops": peak, "peak_source": peak_src,
                       "nvlink_gbs": NVLINK_GBS_MEASURED, "rows": rows}, f, indent=1)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
