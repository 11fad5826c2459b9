"""GEMM micro-benchmark: the tcgen05 kernel vs torch.matmul (cuBLAS) on the Llama-3-8B shapes.

    python -m aws_ofi_nccl_b200.utils.bench_gemm [--json out.json] [--small] [--shape M N K]

Times each shape with CUDA events (warm-up, L2 flushed between iterations) and reports TFLOP/s and
the fraction of the measured cuBLAS peak from MEASURED_PEAKS.json when that file is present.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..ops.gemm import gemm
from .timing import time_cuda

# (name, M, N, K, a_mn, b_mn): forward, input-gradient and weight-gradient products of one layer
LLAMA_SHAPES = [
    ("qkv_fwd", 4096, 6144, 4096, False, False),
    ("wo_fwd", 4096, 4096, 4096, False, False),
    ("gate_up_fwd", 4096, 28672, 4096, False, False),
    ("down_fwd", 4096, 4096, 14336, False, False),
    ("gate_up_dgrad", 4096, 4096, 28672, False, True),
    ("down_dgrad", 4096, 14336, 4096, False, True),
    ("gate_up_wgrad", 28672, 4096, 4096, True, True),
    ("down_wgrad", 4096, 14336, 4096, True, True),
    ("lm_head_fwd", 4096, 128256, 4096, False, False),
]
SMALL_SHAPES = [("small_fwd", 4096, 4096, 4096, False, False), ("small_wgrad", 4096, 4096, 4096, True, True)]


def measured_peak_tflops() -> float | None:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f).get("bf16_tflops", 0)) or None
    return None


def run(shapes, iters: int = 10, bn: int = 0) -> list[dict]:
    peak = measured_peak_tflops()
    rows = []
    for name, M, N, K, a_mn, b_mn in shapes:
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        A = a.T if a_mn else a
        B = b if b_mn else b.T
        ms_ours = time_cuda(lambda: gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, bn=bn), iters=iters)
        ms_lib = time_cuda(lambda: torch.matmul(A, B, out=out), iters=iters)
        fl = 2.0 * M * N * K
        row = {"shape": name, "M": M, "N": N, "K": K, "a_mn": a_mn, "b_mn": b_mn, "ms": ms_ours,
               "tflops": fl / ms_ours / 1e9, "cublas_ms": ms_lib, "cublas_tflops": fl / ms_lib / 1e9,
               "vs_cublas": ms_lib / ms_ours}
        if peak:
            row["frac_of_measured_peak"] = row["tflops"] / peak
        rows.append(row)
        print(json.dumps(row), flush=True)
        del a, b, out
    return rows


def run_fp8(shapes, iters: int = 10) -> list[dict]:
    """e4m3 x e4m3 -> bf16 with per-row scales; torch._scaled_mm (cuBLASLt) is the library reference."""
    from ..ops.gemm import gemm_fp8, quantize_rows_fp8

    rows = []
    for name, M, N, K, _, _ in shapes:
        x = torch.randn(M, K, device="cuda").bfloat16()
        w = (torch.randn(N, K, device="cuda") * K ** -0.5).bfloat16()
        xq, xs = quantize_rows_fp8(x)
        wq, ws = quantize_rows_fp8(w)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = time_cuda(lambda: gemm_fp8(xq, wq, xs, ws, out=out), iters=iters)
        row = {"shape": name + "_fp8", "M": M, "N": N, "K": K, "ms": ms, "tflops": 2.0 * M * N * K / ms / 1e9}
        try:
            sa, sb = xs[:, None].contiguous(), ws[None, :].contiguous()
            ms_lib = time_cuda(lambda: torch._scaled_mm(xq, wq.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16),
                               iters=iters)
            row.update(cublaslt_ms=ms_lib, cublaslt_tflops=2.0 * M * N * K / ms_lib / 1e9, vs_cublaslt=ms_lib / ms)
        except (RuntimeError, TypeError, AttributeError) as e:   # not offered by this torch build for these scales
            row["cublaslt"] = f"unavailable: {type(e).__name__}"
        rows.append(row)
        print(json.dumps(row), flush=True)
    return rows


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--json")
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--shape", type=int, nargs=3, metavar=("M", "N", "K"), help="time this one shape only")
    ap.add_argument("--fp8", action="store_true", help="also time the e4m3 kernel (row / column scales) on the forward shapes")
    args = ap.parse_args()
    if args.shape:
        shapes = [("custom", *args.shape, False, False)]
    else:
        shapes = SMALL_SHAPES if args.small else LLAMA_SHAPES
    rows = run(shapes, iters=args.iters, bn=args.bn)
    if args.fp8:
        rows += run_fp8([s for s in shapes if not s[4] and not s[5]], iters=args.iters)
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
