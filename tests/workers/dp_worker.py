"""Multi-GPU worker: data-parallel tiny Llama — gradients after the fused all-reduce must equal the
average of the per-rank gradients, the ranks must stay bit-identical after optimizer steps, and N
ranks fed identical batches must reproduce the loss curve of a single replica step for step (with
this library's reducer and with the NCCL-based one in both of its modes)."""
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
    from aws_ofi_nccl_b200.models.llama import Llama, LlamaConfig
    from aws_ofi_nccl_b200.ops import _lib
    from aws_ofi_nccl_b200.parallel.data_parallel import GradReducer
    from aws_ofi_nccl_b200.parallel.engine import Trainer

    cfg = LlamaConfig.tiny()
    dp = GradReducer(dist.group.WORLD, dev, bucket_bytes=256 << 10)
    tr = Trainer(cfg, device=dev, dp=dp, seed=7)
    gen = torch.Generator().manual_seed(100 + rank)
    ids = torch.randint(0, cfg.vocab_size, (2, 128), generator=gen).to(dev)
    lbl = torch.randint(0, cfg.vocab_size, (2, 128), generator=gen).to(dev)

    # reference: local gradients of an identical replica, averaged with NCCL
    ref = Llama(cfg, device=dev, seed=7)
    ref.forward_loss(ids, lbl).backward()
    g_ref = ref.flat_grads.float()
    dist.all_reduce(g_ref)
    g_ref /= world

    tr.model.reset_grad_flags()
    dp.begin_step()
    tr.model.forward_loss(ids, lbl).backward()
    dp.finish_step()
    torch.cuda.synchronize()
    g = tr.model.flat_grads.float()
    err = (g - g_ref).abs().max().item()
    scale = g_ref.abs().max().item()
    ok = err <= 2e-2 * scale + 1e-6
    if not ok:
        print(f"[{rank}] DP gradient mismatch: err {err} scale {scale}")
    tr.model.flat_grads.zero_()

    losses = [tr.step_device(ids, lbl).item() for _ in range(4)]
    ok = ok and losses[-1] < losses[0]
    # replicas must hold identical parameters
    p = tr.model.flat_params.float()
    pmax, pmin = p.clone(), p.clone()
    dist.all_reduce(pmax, op=dist.ReduceOp.MAX)
    dist.all_reduce(pmin, op=dist.ReduceOp.MIN)
    if not torch.equal(pmax, pmin):
        ok = False
        print(f"[{rank}] replicas diverged: {(pmax - pmin).abs().max().item()}")
    # ---- loss parity: the same batches on every rank, so the averaged gradient equals one
    # replica's gradient and the loss curve has to match a run without any reducer
    from aws_ofi_nccl_b200.parallel.data_parallel import NcclGradReducer
    from aws_ofi_nccl_b200.parallel.engine import OptimConfig

    gen2 = torch.Generator().manual_seed(4242)
    batches = [(torch.randint(0, cfg.vocab_size, (2, 128), generator=gen2).to(dev),
                torch.randint(0, cfg.vocab_size, (2, 128), generator=gen2).to(dev)) for _ in range(3)]

    def curve(reducer):
        trainer = Trainer(cfg, OptimConfig(lr=1e-3), device=dev, dp=reducer, seed=11)
        out = [trainer.step_device(*batches[i % 3]).item() for i in range(6)]
        torch.cuda.synchronize()
        return out

    single = curve(None)
    for name, make in (("fused", lambda: GradReducer(dist.group.WORLD, dev, bucket_bytes=256 << 10, channel=3)),
                       ("nccl all-reduce", lambda: NcclGradReducer(dist.group.WORLD, dev, bucket_bytes=256 << 10)),
                       ("nccl reduce-scatter + all-gather", lambda: NcclGradReducer(dist.group.WORLD, dev, mode="zero"))):
        red = make()
        got = curve(red)
        red.close()
        worst = max(abs(a - b) / max(abs(b), 1e-6) for a, b in zip(got, single))
        if worst > 2e-2:
            ok = False
            print(f"[{rank}] loss curve with the {name} reducer differs from the single replica: {got} vs {single}")
    t = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    status = _lib.read_status()
    dp.close()
    dist.destroy_process_group()
    if t.item() != 1 or status != 0:
        print(f"[{rank}] FAILED status={status}")
        sys.exit(1)
    if rank == 0:
        print("dp worker OK", losses)


if __name__ == "__main__":
    main()
