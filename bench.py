#!/usr/bin/env python
"""Headline benchmark: Llama-3-8B training step (bf16, seq 4096, micro-batch 1 per GPU), tokens/s.

  python bench.py --gpus 1 --steps 5 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
      --master-port P bench.py --gpus N --steps K --warmup W

For N > 1 the job is data parallel: every rank holds a replica, gradients are averaged by this
repository's own NVLink all-reduce kernels (fused with the 1/N scale) overlapped behind backward;
that number is the headline ``value``.  At N > 1 the same JSON line also carries

  collectives       bus bandwidth of this repository's collective kernels next to stock NCCL
                    (NVLink / NVLS) on the same buffers, every size checked against an fp64 sum
  gin_put_signal_us one-way latency of a device-initiated 8-byte put + signal between two GPUs
  nccl_over_plugin  the same collectives issued through unmodified NCCL with NCCL_P2P_DISABLE=1 and
                    NCCL_SHM_DISABLE=1, so that every byte crosses this repository's net plugin
                    (libnccl-net-ofi-b200.so, loaded through NCCL_NET_PLUGIN, tuner self-registered)
  through_plugin    the training step with its gradient traffic issued through NCCL over the plugin:
                    all-reduce per bucket (data parallel) and reduce-scatter + sharded AdamW +
                    parameter all-gather (ZeRO / FSDP pattern)

The last two run as child processes (NCCL picks its transport once per process); a child that does
not finish within its limit is ended with all its ranks and reported as such.
``--impl reference`` reports why the reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "llama3_8b_train_tokens_per_sec"
PLUGIN_LIB = os.path.join(ROOT, "aws-ofi-nccl_b200", "lib")


def reference_arm() -> None:
    why = ("aws-ofi-nccl is a C++ autotools NCCL plugin, not a Python package: pip cannot build it, and its "
           "configure step needs libfabric>=1.18, hwloc and autoconf/automake/libtool, none of which exist in "
           "this offline image")
    print(json.dumps({"impl": "reference", "unavailable": why}))


def plugin_env(base: dict) -> dict:
    """Environment of a process whose NCCL traffic has to cross this repository's net plugin."""
    env = dict(base)
    env.update(NCCL_NET_PLUGIN="ofi-b200", NCCL_P2P_DISABLE="1", NCCL_SHM_DISABLE="1", NCCL_NVLS_ENABLE="0",
               LD_LIBRARY_PATH=f"{PLUGIN_LIB}:" + base.get("LD_LIBRARY_PATH", ""))
    # The plugin's proxy thread launches copy kernels that NCCL's kernel waits for: nothing in the
    # process may make the device wait for that kernel first (a lazy kernel load synchronises the
    # context), and the device should offer all its hardware work queues.
    env.setdefault("CUDA_MODULE_LOADING", "EAGER")
    env.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")
    # point-to-point calls (all_to_all): eight channels per peer instead of NCCL's two for a network.
    # NCCL reads this before it initialises the plugin, so the plugin's own environment defaults come
    # too late for it. Measured on two GPUs only (256 MiB all_to_all 45 -> 166 GB/s), so larger jobs
    # keep NCCL's default here.
    if int(base.get("WORLD_SIZE", "1")) <= 2:
        env.setdefault("NCCL_NCHANNELS_PER_NET_PEER", "8")
    # gradient traffic through the plugin runs after backward, not behind it: with compute kernels
    # and their stream waits queued on the device while the proxy thread launches copies, the first
    # overlapped step stopped moving (both ranks waiting for data, nothing left to send)
    env.setdefault("B200NET_DP_SETTLE_STEPS", "1000000000")
    env.pop("NCCL_TUNER_PLUGIN", None)   # the plugin registers its own tuner
    return env


def run_child(argv: list[str], env: dict, port_offset: int, limit: float, tag: str):
    """One child per rank (each rank of this job starts its own, with the same rank numbers and a
    rendezvous port of its own). Returns (json dict | None, note)."""
    from aws_ofi_nccl_b200.utils.proc import run_job

    env = dict(env)
    env["MASTER_PORT"] = str(int(os.environ.get("MASTER_PORT", "29500")) + port_offset)
    env["MASTER_ADDR"] = "127.0.0.1"
    for k in ("TORCHELASTIC_RUN_ID", "TORCHELASTIC_USE_AGENT_STORE", "TORCHELASTIC_RESTART_COUNT", "TORCHELASTIC_MAX_RESTARTS",
              "TORCH_NCCL_ASYNC_ERROR_HANDLING"):
        env.pop(k, None)
    rc, out, err = run_job([sys.executable] + argv, env=env, cwd=ROOT, timeout=limit)
    if rc is None:
        warns = [ln.split("NCCL WARN")[-1].strip()[:200] for ln in (out + err).splitlines() if "NCCL WARN" in ln][:6]
        return None, f"{tag}: did not finish within {limit:.0f} s" + ("; " + " | ".join(warns) if warns else "")
    lines = [ln for ln in out.splitlines() if ln.startswith(tag + " ")]
    if rc != 0 or not lines:
        tail = (err or out).strip().splitlines()[-3:]
        return None, f"{tag}: exit {rc}: " + " | ".join(t[:160] for t in tail)
    return json.loads(lines[-1][len(tag) + 1:]), ""


# ---------------------------------------------------------------------------------------------- collectives
def collective_rows(fn_ours, fn_nccl, world: int, sizes, device, check: bool):
    """Times ours / NCCL per size and collective with CUDA events (max over ranks); every size is
    checked once against an fp64 reduction on the device."""
    import torch
    import torch.distributed as dist

    def timed(fn, warm, iters):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize(device)
        dist.barrier()
        # the waiting thread sleeps instead of spinning: with traffic through a net plugin every rank also has a
        # proxy thread that has to run, and a box may have no more cores than that
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True, blocking=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        b.synchronize()
        t = torch.tensor([a.elapsed_time(b) / iters], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    rows = []
    for nbytes in sizes:
        warm, iters = (20, 100) if nbytes <= (64 << 20) else (5, 20)
        for coll in ("all_reduce", "reduce_scatter", "all_gather", "all_to_all"):
            factor = 2 * (world - 1) / world if coll == "all_reduce" else (world - 1) / world
            row = {"coll": coll, "bytes": nbytes}
            for arm, make in (("ours", fn_ours), ("nccl", fn_nccl)):
                if make is None:
                    continue
                fn, ok = make(coll, nbytes, check)
                ms = timed(fn, warm, iters)
                row[f"{arm}_us"] = round(ms * 1e3, 2)
                row[f"{arm}_busbw_GBs"] = round(nbytes * factor / ms / 1e6, 2)
                row[f"{arm}_fp64_check"] = ok
            rows.append(row)
    return rows


def nccl_maker(world: int, rank: int, device):
    """torch.distributed (NCCL) calls on bf16 N(0,1) buffers plus their fp64 check."""
    import torch
    import torch.distributed as dist

    def make(coll, nbytes, check):
        numel = nbytes // 2
        torch.manual_seed(7 + rank)
        x = torch.randn(numel, device=device).bfloat16()
        per = numel // world
        ok = None
        if check:
            xs = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(xs, x)
            torch.cuda.synchronize(device)
            ref = sum(t.double() for t in xs)
            tol = dict(rtol=5e-2, atol=5e-2 * world)
            if coll == "all_reduce":
                y = x.clone()
                dist.all_reduce(y)
                torch.cuda.synchronize(device)   # nothing else is queued while the collective is in flight
                ok = bool(torch.allclose(y.double(), ref, **tol))
            elif coll == "reduce_scatter":
                o = torch.empty(per, device=device, dtype=torch.bfloat16)
                dist.reduce_scatter_tensor(o, x)
                torch.cuda.synchronize(device)   # nothing else is queued while the collective is in flight
                ok = bool(torch.allclose(o.double(), ref[rank * per:(rank + 1) * per], **tol))
            elif coll == "all_gather":
                y = torch.empty(numel, device=device, dtype=torch.bfloat16)
                dist.all_gather_into_tensor(y, x[:per].contiguous())
                torch.cuda.synchronize(device)   # nothing else is queued while the collective is in flight
                ok = bool(torch.equal(y, torch.cat([t[:per] for t in xs])))
            else:
                y = torch.empty_like(x)
                dist.all_to_all_single(y, x)
                torch.cuda.synchronize(device)   # nothing else is queued while the collective is in flight
                ok = bool(torch.equal(y, torch.cat([t[rank * per:(rank + 1) * per] for t in xs])))
            del xs, ref
            torch.cuda.synchronize(device)
        y = torch.empty_like(x)
        part = torch.empty(per, device=device, dtype=torch.bfloat16)
        fn = {"all_reduce": lambda: dist.all_reduce(x), "reduce_scatter": lambda: dist.reduce_scatter_tensor(part, y),
              "all_gather": lambda: dist.all_gather_into_tensor(y, part), "all_to_all": lambda: dist.all_to_all_single(y, x)}[coll]
        return fn, ok

    return make


def ours_maker(comm, world: int, rank: int, device, max_bytes: int):
    """This repository's collective kernels on the communicator's symmetric window."""
    import torch
    import torch.distributed as dist

    def make(coll, nbytes, check):
        numel = nbytes // 2
        per_b = nbytes // world
        per = numel // world
        nb = 4 if nbytes <= (64 << 10) else 16 if nbytes <= (1 << 20) else 64 if nbytes <= (32 << 20) else 128
        torch.manual_seed(7 + rank)
        x = torch.randn(numel, device=device).bfloat16()
        win = comm.view(0, numel, torch.bfloat16)
        out = torch.empty(per, device=device, dtype=torch.bfloat16)
        ok = None
        if check:
            xs = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(xs, x)
            torch.cuda.synchronize(device)
            ref = sum(t.double() for t in xs)
            tol = dict(rtol=5e-2, atol=5e-2 * world)
            win.copy_(x)
            if coll == "all_gather":
                win.zero_()
                win[rank * per:(rank + 1) * per].copy_(x[:per])
            dist.barrier()   # every rank's window is filled before a peer reads or writes it
            if coll == "all_reduce":
                comm.all_reduce(0, nbytes, torch.bfloat16, nblocks=nb)
                ok = bool(torch.allclose(win.double(), ref, **tol))
            elif coll == "reduce_scatter":
                comm.reduce_scatter(0, per_b, torch.bfloat16, out, nblocks=nb)
                ok = bool(torch.allclose(out.double(), ref[rank * per:(rank + 1) * per], **tol))
            elif coll == "all_gather":
                comm.all_gather(0, per_b, nblocks=nb)
                ok = bool(torch.equal(win, torch.cat([t[:per] for t in xs])))
            else:
                comm.all_to_all(0, max_bytes, per_b, nblocks=nb)
                got = comm.view(max_bytes, numel, torch.bfloat16)
                ok = bool(torch.equal(got, torch.cat([t[rank * per:(rank + 1) * per] for t in xs])))
            del xs, ref
            torch.cuda.synchronize(device)
            dist.barrier()
            win.copy_(x)
        fn = {"all_reduce": lambda: comm.all_reduce(0, nbytes, torch.bfloat16, nblocks=nb),
              "reduce_scatter": lambda: comm.reduce_scatter(0, per_b, torch.bfloat16, out, nblocks=nb),
              "all_gather": lambda: comm.all_gather(0, per_b, nblocks=nb),
              "all_to_all": lambda: comm.all_to_all(0, max_bytes, per_b, nblocks=nb)}[coll]
        return fn, ok

    return make


def collectives_child(args) -> None:
    """Child process: stock NCCL collectives with whatever transport the environment selects (the
    parent selects this repository's plugin)."""
    import torch
    import torch.distributed as dist

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    rows = collective_rows(None, nccl_maker(world, rank, device), world, args.sizes, device, check=True)
    if rank == 0:
        print("COLL_CHILD " + json.dumps(rows), flush=True)
    dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------- training
def train_measure(args, world: int, rank: int, local_rank: int, device):
    import torch
    import torch.distributed as dist

    from aws_ofi_nccl_b200.models.llama import LlamaConfig
    from aws_ofi_nccl_b200.ops import _lib
    from aws_ofi_nccl_b200.parallel.engine import OptimConfig, Trainer
    from aws_ofi_nccl_b200.utils.timing import ClockSampler

    dp = None
    if world > 1:
        if args.comm == "fused":
            from aws_ofi_nccl_b200.parallel.data_parallel import GradReducer
            dp = GradReducer(dist.group.WORLD, device)
        else:
            from aws_ofi_nccl_b200.parallel.data_parallel import NcclGradReducer
            dp = NcclGradReducer(dist.group.WORLD, device, mode="zero" if args.comm == "nccl-zero" else "allreduce")

    cfg = LlamaConfig.llama3_8b() if args.model == "llama3_8b" else LlamaConfig.tiny()
    seq = min(args.seq, cfg.max_seq)
    master = not args.no_master
    try:
        trainer = Trainer(cfg, OptimConfig(master_weights=master, lr=args.lr), device=device, dp=dp, seed=1234)
    except torch.OutOfMemoryError:
        if world > 1:
            raise
        torch.cuda.empty_cache()
        master = False
        trainer = Trainer(cfg, OptimConfig(master_weights=False, lr=args.lr), device=device, dp=dp, seed=1234)

    gen = torch.Generator().manual_seed(1000 + rank)
    n_batches = 4
    host_ids = [torch.randint(0, cfg.vocab_size, (1, seq), generator=gen).pin_memory() for _ in range(n_batches)]
    host_lbl = [torch.randint(0, cfg.vocab_size, (1, seq), generator=gen).pin_memory() for _ in range(n_batches)]
    dev_ids = [t.to(device) for t in host_ids]
    dev_lbl = [t.to(device) for t in host_lbl]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed region
    for i in range(args.warmup):
        trainer.step_device(dev_ids[i % n_batches], dev_lbl[i % n_batches])
    barrier()
    launches0 = _lib.launch_count
    with ClockSampler(gpu_index=local_rank) as clocks:
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        loss = None
        for i in range(args.steps):
            loss = trainer.step_device(dev_ids[i % n_batches], dev_lbl[i % n_batches])
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1)
    launches = _lib.launch_count - launches0
    final_loss = float(loss.item())

    # ---- end-to-end region (public API: pinned host batch in, float loss out)
    trainer.step(host_ids[0], host_lbl[0])
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        trainer.step(host_ids[i % n_batches], host_lbl[i % n_batches])
    barrier()
    e2e_s = time.perf_counter() - t0

    t = torch.tensor([ms, e2e_s * 1e3], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    status = _lib.read_status()
    tokens = world * seq * args.steps
    res = {"tokens_per_s": tokens / (ms / 1e3), "ms_per_step": ms / args.steps, "e2e_tokens_per_s": tokens / (e2e_ms / 1e3),
           "launches": launches, "final_loss": final_loss, "device_status": status, "seq": seq, "master": master,
           "clocks": {k: v for k, v in clocks.summary().items() if k in ("sm_mhz", "sm_max_mhz", "reasons")}}
    if dp is not None:
        dp.close()
    del trainer
    torch.cuda.empty_cache()
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3_8b", choices=["llama3_8b", "tiny"])
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--no-master", action="store_true", help="bf16 parameters only (no fp32 master copy)")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl", "nccl-zero"],
                    help="gradient traffic: this repository's fused NVLink kernels, or torch.distributed (NCCL) all-reduce / "
                         "reduce-scatter + sharded optimizer + all-gather")
    ap.add_argument("--extras", default="auto", choices=["auto", "none"],
                    help="at N > 1 also measure the collectives, the GIN latency and the plugin arms (auto) or only the step (none)")
    ap.add_argument("--child", default="", choices=["", "train", "collectives"], help=argparse.SUPPRESS)
    ap.add_argument("--sizes", type=int, nargs="+", default=[65536, 1 << 20, 16 << 20, 256 << 20], help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return
    args.warmup = max(args.warmup, 3)
    if args.child == "collectives":
        collectives_child(args)
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    res = train_measure(args, world, rank, local_rank, device)
    if args.child == "train":
        if rank == 0:
            print("TRAIN_CHILD " + json.dumps({k: res[k] for k in ("tokens_per_s", "ms_per_step", "e2e_tokens_per_s", "final_loss")}),
                  flush=True)
        dist.destroy_process_group()
        return

    extras = {}
    if world > 1 and args.extras == "auto":
        from aws_ofi_nccl_b200.parallel.symm import Communicator

        max_bytes = max(args.sizes)
        comm = Communicator(dist.group.WORLD, 2 * max_bytes, device)
        extras["collectives"] = collective_rows(ours_maker(comm, world, rank, device, max_bytes), nccl_maker(world, rank, device),
                                                world, args.sizes, device, check=True)
        extras["gin_put_signal_us"] = round(comm.pingpong_ns(8, iters=2000) / 1e3, 3)
        comm.close()
        torch.cuda.synchronize()
        dist.barrier()
        # ---- arms whose NCCL traffic crosses this repository's net plugin (child processes)
        penv = plugin_env(os.environ)
        rows, note = run_child([os.path.abspath(__file__), "--child", "collectives", "--sizes"] + [str(s) for s in args.sizes],
                               penv, 101, 120, "COLL_CHILD")
        extras["nccl_over_plugin"] = rows if rows is not None else {"unavailable": note}
        dist.barrier()
        through = {}
        for i, comm_mode in enumerate(("nccl", "nccl-zero")):
            r, note = run_child([os.path.abspath(__file__), "--child", "train", "--comm", comm_mode, "--steps", str(args.steps),
                                 "--warmup", str(args.warmup), "--model", args.model, "--seq", str(args.seq), "--gpus", str(world)],
                                penv, 102 + i, 150, "TRAIN_CHILD")
            through["all_reduce" if comm_mode == "nccl" else "reduce_scatter_all_gather"] = r if r is not None else {"unavailable": note}
            dist.barrier()
        extras["through_plugin"] = through

    if rank == 0:
        seq = res["seq"]
        out = {
            "metric": METRIC, "value": res["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init weights)",
            "config": {"model": "Llama-3-8B" if args.model == "llama3_8b" else "tiny", "global_batch": world,
                       "seq_len": seq, "parallelism": f"dp{world}", "gradient_traffic": args.comm,
                       "optimizer": "AdamW fp32 m/v" + (" + fp32 master" if res["master"] else ", bf16 params"),
                       "l2": "working set (16 GB of weights per step) exceeds the 126 MB L2; no flush needed"},
            "clocks": res["clocks"],
            "e2e": {"value": res["e2e_tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 2 * seq * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": res["launches"], "final_loss": res["final_loss"], "device_status": res["device_status"],
        }
        out.update(extras)
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
