"""Multi-GPU worker (launched by torchrun): MoE route / dispatch / combine kernels (bf16 and
block-scaled fp8) and the expert-parallel MoE layer, forward and backward, against fp32 references."""
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
    from aws_ofi_nccl_b200.parallel.expert_parallel import ExpertParallel
    from aws_ofi_nccl_b200.models.moe import MoELayer

    T, H, E, k = 384, 512, 4 * world, 3
    comm = Communicator(dist.group.WORLD, ExpertParallel.window_bytes(world, T, H, E, k, 8.0) + (1 << 20), dev,
                        wait_limit_s=5.0)
    ok = True

    def check(name, got, ref, tol):
        nonlocal ok
        e = rel_err(got, ref)
        if not (e < tol):
            ok = False
            print(f"[{rank}] {name}: rel err {e:.4g} (tol {tol})", flush=True)

    ep = ExpertParallel(comm, T, H, E, k, capacity_factor=8.0)
    el = E // world
    for rep in range(3):
        torch.manual_seed(1000 * rep + rank)
        x = torch.randn(T, H, device=dev).bfloat16()
        logits = torch.randn(T, E, device=dev)
        if rep == 2:
            logits[:, 0] += 10.0   # every token picks expert 0: one hot segment, others nearly empty
        w, idx = torch.topk(torch.softmax(logits, -1), k, dim=-1)
        idx = idx.to(torch.int32).contiguous()
        w = w.contiguous()
        for fp8 in (False, True):
            off = ep.route(idx)
            ep.dispatch_raw(x, idx, w, fp8=fp8)
            torch.cuda.synchronize()
            off_h = off.tolist()
            # per-expert totals must equal the global histogram of the choices
            counts = torch.bincount(idx.flatten().long(), minlength=E)
            dist.all_reduce(counts)
            mine = counts[rank * el:(rank + 1) * el].tolist()
            got = [off_h[i + 1] - off_h[i] for i in range(el)]
            if got != mine or off_h[0] != 0:
                ok = False
                print(f"[{rank}] rep{rep} fp8={fp8}: expert row counts {got} != {mine}", flush=True)
            rows = ep.dequant() if fp8 else ep.recv_rows(False)
            total = off_h[-1]
            # every received row must equal the source token named by its record
            meta = ep.recv_meta()[:total].cpu()
            xs = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(xs, x)
            x_all = torch.stack(xs).cpu()
            ref_rows = x_all[meta[:, 3].long(), meta[:, 0].long()]
            check(f"dispatch rows rep{rep} fp8={fp8}", rows[:total].cpu(), ref_rows, 4e-2 if fp8 else 1e-6)
            idxs = [torch.empty_like(idx) for _ in range(world)]
            dist.all_gather(idxs, idx)
            idx_all = torch.stack(idxs).cpu()
            row_expert = torch.repeat_interleave(torch.arange(el), torch.tensor(got)) + rank * el
            named = idx_all[meta[:, 3].long(), meta[:, 0].long(), meta[:, 1].long()]
            if not torch.equal(named.long(), row_expert.long()):
                ok = False
                print(f"[{rank}] rep{rep} fp8={fp8}: rows landed in the wrong expert segment", flush=True)
            # "experts" that scale by (expert id + 1): the combine result has a closed form
            y = (rows[:total].float() * (row_expert.to(dev).float() + 1)[:, None]).bfloat16().contiguous()
            out = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
            ep.combine_raw(y, w, out)
            torch.cuda.synchronize()
            ref = x.float() * (w * (idx.float() + 1)).sum(-1, keepdim=True)
            check(f"combine rep{rep} fp8={fp8}", out, ref, 4e-2 if fp8 else 1.5e-2)
        dist.barrier()

    # ---------------- MoE layer, forward and backward, vs a dense fp32 evaluation of all experts
    F = 256
    for fp8 in (False, True):
        layer = MoELayer(comm, T, H, F, E, k, fp8_dispatch=fp8, capacity_factor=8.0, seed=5)
        torch.manual_seed(77 + rank)
        x = torch.randn(T, H, device=dev).bfloat16().requires_grad_(True)
        dy = torch.randn(T, H, device=dev).bfloat16()
        out = layer(x)
        out.backward(dy)
        torch.cuda.synchronize()
        router, w_gu, w_dn = (t.to(dev) for t in layer._full)
        w_gu = w_gu.bfloat16().float().requires_grad_(True)
        w_dn = w_dn.bfloat16().float().requires_grad_(True)
        xr = x.detach().float().requires_grad_(True)
        router_r = router.clone().requires_grad_(True)
        probs = torch.softmax(xr @ router_r.t(), -1)
        wr, ir = torch.topk(probs, k, dim=-1)
        ref = torch.zeros(T, H, device=dev)
        for s in range(k):
            e_s = ir[:, s]
            gu = torch.einsum("th,tfh->tf", xr, w_gu[e_s])
            h = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
            ref = ref + wr[:, s:s + 1] * torch.einsum("tf,thf->th", h, w_dn[e_s])
        ref.backward(dy.float())
        tol = 6e-2 if fp8 else 3e-2
        check(f"moe layer out fp8={fp8}", out, ref, tol)
        check(f"moe layer dx fp8={fp8}", x.grad, xr.grad, 8e-2 if fp8 else 4e-2)
        check(f"moe layer d(router) fp8={fp8}", _allreduce(layer.router.grad), _allreduce(router_r.grad), 8e-2 if fp8 else 4e-2)
        lo = rank * el
        g_gu = w_gu.grad.clone()
        g_dn = w_dn.grad.clone()
        dist.all_reduce(g_gu)
        dist.all_reduce(g_dn)
        for e in range(el):
            if layer.w_gate_up[e].grad is not None and g_gu[lo + e].abs().sum() > 0:
                check(f"moe layer dWgu[{e}] fp8={fp8}", layer.w_gate_up[e].grad, g_gu[lo + e], 8e-2 if fp8 else 4e-2)
                check(f"moe layer dWdown[{e}] fp8={fp8}", layer.w_down[e].grad, g_dn[lo + e], 8e-2 if fp8 else 4e-2)
        dist.barrier()

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
        print("MOE_WORKER_OK", flush=True)


def _allreduce(t):
    t = t.clone()
    dist.all_reduce(t)
    return t


if __name__ == "__main__":
    main()
