"""Multi-GPU worker (launched by torchrun): fused all-gather->GEMM / GEMM->reduce-scatter kernels,
the tensor-parallel MLP and the FSDP linear layer against fp32 references built from NCCL
collectives and plain matmuls."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist


def rel_err(got, ref):
    return ((got.float() - ref.float()).norm() / ref.float().norm().clamp_min(1e-6)).item()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from aws_ofi_nccl_b200.ops import _lib
    from aws_ofi_nccl_b200.parallel.symm import Communicator
    from aws_ofi_nccl_b200.parallel import tensor_parallel as tp

    comm = Communicator(dist.group.WORLD, 96 << 20, dev, wait_limit_s=5.0)
    ok = True

    def check(name, got, ref, tol=2e-2):
        nonlocal ok
        e = rel_err(got, ref)
        if not (e < tol):
            ok = False
            print(f"[{rank}] {name}: rel err {e:.4g} (tol {tol})", flush=True)

    def all_gather_rows(t):
        out = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(out, t.contiguous())
        return torch.cat(out, dim=0)

    torch.manual_seed(100 + rank)
    for (Ts, N, K) in ((128, 256, 64), (256, 512 * world, 1024), (384, 1024, 4096 + 64)):
        M = Ts * world
        # ---------------- all-gather(A) -> GEMM, both weight layouts
        a_shard = torch.randn(Ts, K, device=dev).bfloat16()
        a_full_ref = all_gather_rows(a_shard)
        w = (torch.randn(N, K, device=dev) * K ** -0.5).bfloat16()
        gathered = comm.view(0, M * K, torch.bfloat16).view(M, K)
        for rep in range(2):  # twice: the second call exercises flag / epoch reuse
            gathered.zero_()
            gathered[rank * Ts:(rank + 1) * Ts].copy_(a_shard)
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            tp.ag_gemm(comm, 0, M, K, w, out=out, n_movers=4)
            torch.cuda.synchronize()
            check(f"ag_gemm {M}x{N}x{K} rep{rep}", out, a_full_ref.float() @ w.float().t())
            if not torch.equal(gathered, a_full_ref):
                ok = False
                print(f"[{rank}] ag_gemm left a wrong gathered operand", flush=True)
        wt = w.t().contiguous()
        gathered.zero_()
        gathered[rank * Ts:(rank + 1) * Ts].copy_(a_shard)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        tp.ag_gemm(comm, 0, M, K, wt, b_mn=True, out=out, n_movers=4)
        torch.cuda.synchronize()
        check(f"ag_gemm b_mn {M}x{N}x{K}", out, a_full_ref.float() @ w.float().t())
        # ---------------- ... with the SwiGLU epilogue
        if N % 64 == 0:
            gathered.zero_()
            gathered[rank * Ts:(rank + 1) * Ts].copy_(a_shard)
            act = torch.empty(M, N // 2, device=dev, dtype=torch.bfloat16)
            gu = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            tp.ag_gemm(comm, 0, M, K, w, out=gu, act=act, swiglu=True, n_movers=4)
            torch.cuda.synchronize()
            wg, wu = tp.deinterleave_gate_up(w)
            g = a_full_ref.float() @ wg.float().t()
            u = a_full_ref.float() @ wu.float().t()
            check(f"ag_gemm swiglu {M}x{N}x{K}", act, torch.nn.functional.silu(g) * u, tol=3e-2)
            check(f"ag_gemm swiglu raw {M}x{N}x{K}", gu, a_full_ref.float() @ w.float().t())
        # ---------------- GEMM -> reduce-scatter
        a = torch.randn(M, K, device=dev).bfloat16()
        stage_off = tp._align(M * K * 2)
        ref_full = a.float() @ w.float().t()
        dist.all_reduce(ref_full)
        for rep in range(2):
            o = torch.empty(Ts, N, device=dev, dtype=torch.bfloat16)
            tp.gemm_rs(comm, a, w, stage_off, o)
            torch.cuda.synchronize()
            check(f"gemm_rs {M}x{N}x{K} rep{rep}", o, ref_full[rank * Ts:(rank + 1) * Ts])
        o = torch.empty(Ts, N, device=dev, dtype=torch.bfloat16)
        tp.gemm_rs(comm, a, wt, stage_off, o, b_mn=True, scale=0.5)
        torch.cuda.synchronize()
        check(f"gemm_rs b_mn {M}x{N}x{K}", o, 0.5 * ref_full[rank * Ts:(rank + 1) * Ts])
        dist.barrier()

    # ---------------- all-gather(B) -> GEMM (weights sharded along their rows)
    for (M, N, K) in ((128, 256 * world, 256), (300, 512 * world, 1024)):
        rows = N // world
        w_shard = (torch.randn(rows, K, device=dev) * K ** -0.5).bfloat16()
        w_full_ref = all_gather_rows(w_shard)
        x = torch.randn(M, K, device=dev).bfloat16()
        gathered = comm.view(0, N * K, torch.bfloat16).view(N, K)
        gathered.zero_()
        gathered[rank * rows:(rank + 1) * rows].copy_(w_shard)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        tp.ag_gemm(comm, 0, N, K, x, gather_b=True, out=out, n_movers=2)
        torch.cuda.synchronize()
        check(f"ag_gemm gather_b {M}x{N}x{K}", out, x.float() @ w_full_ref.float().t())
        dist.barrier()

    # ---------------- tensor-parallel MLP, forward and backward
    T, H, F = 256 * world, 512, 1024 * world
    mlp = tp.TensorParallelMLP(comm, T, H, F, n_helpers=4, seed=7)
    Ts = T // world
    g = torch.Generator(device="cpu").manual_seed(99)
    x_all = torch.randn(T, H, generator=g).bfloat16()
    dy_all = torch.randn(T, H, generator=g).bfloat16()
    x_shard = x_all[rank * Ts:(rank + 1) * Ts].to(dev).requires_grad_(True)
    for rep in range(2):
        mlp.w_gate_up.grad = None
        mlp.w_down.grad = None
        x_shard.grad = None
        y = mlp(x_shard)
        y.backward(dy_all[rank * Ts:(rank + 1) * Ts].to(dev))
        torch.cuda.synchronize()
        wg, wu, wd = (t.bfloat16().float().to(dev) for t in mlp._full)
        xr = x_all.float().to(dev).requires_grad_(True)
        wg.requires_grad_(True), wu.requires_grad_(True), wd.requires_grad_(True)
        yr = (torch.nn.functional.silu(xr @ wg.t()) * (xr @ wu.t())) @ wd.t()
        yr.backward(dy_all.float().to(dev))
        lo, hi = rank * mlp.ffn_local, (rank + 1) * mlp.ffn_local
        check(f"tp mlp y rep{rep}", y, yr[rank * Ts:(rank + 1) * Ts], tol=3e-2)
        check(f"tp mlp dx rep{rep}", x_shard.grad, xr.grad[rank * Ts:(rank + 1) * Ts], tol=3e-2)
        dg, du = tp.deinterleave_gate_up(mlp.w_gate_up.grad)
        check(f"tp mlp dWgate rep{rep}", dg, wg.grad[lo:hi], tol=3e-2)
        check(f"tp mlp dWup rep{rep}", du, wu.grad[lo:hi], tol=3e-2)
        check(f"tp mlp dWdown rep{rep}", mlp.w_down.grad, wd.grad[:, lo:hi], tol=3e-2)
    dist.barrier()

    # ---------------- FSDP linear
    inf, outf = 512, 256 * world * 2
    layer = tp.FsdpLinear(comm, inf, outf, window_offset=0, n_helpers=2, seed=3)
    xs = torch.randn(192, inf, device=dev).bfloat16().requires_grad_(True)
    y = layer(xs)
    dy = torch.randn_like(y)
    y.backward(dy)
    torch.cuda.synchronize()
    wf = layer._full.bfloat16().float().to(dev)
    check("fsdp y", y, xs.float() @ wf.t())
    check("fsdp dx", xs.grad, dy.float() @ wf)
    dw_ref = dy.float().t() @ xs.detach().float()
    dist.all_reduce(dw_ref)
    rows = outf // world
    check("fsdp dW shard", layer.shard_grad, dw_ref[rank * rows:(rank + 1) * rows], tol=3e-2)

    status = _lib.read_status(clear=True)
    if status != 0:
        ok = False
        print(f"[{rank}] device status word = {status}", flush=True)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    comm.close()
    dist.destroy_process_group()
    if flag.item() != 1:
        sys.exit(1)
    if rank == 0:
        print("TP_WORKER_OK", flush=True)


if __name__ == "__main__":
    main()
