"""NCCL collective sweep with the traffic forced through this repository's net plugin, against
stock NCCL's built-in socket transport under the same restriction.

    python -m aws_ofi_nccl_b200.utils.bench_plugin --gpus 2 [--arms plugin socket] [--max-bytes 268435456] [--json out.json]

Both arms run with NCCL_P2P_DISABLE=1 and NCCL_SHM_DISABLE=1, so every byte between the GPUs
crosses a network transport: `plugin` loads libnccl-net-ofi-b200.so through NCCL_NET_PLUGIN,
`socket` uses NCCL's own NET/Socket.  all_reduce, all_gather, reduce_scatter and all_to_all on
bf16 buffers, sizes doubling from --min-bytes, warm-up + timed iterations with CUDA events, maximum
over ranks, checked on the first iteration against a host fp64 reduction.  Each arm is a torchrun
job of its own because NCCL picks its transport once per process.
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import sys
from pathlib import Path

from .proc import run_job

LIB = Path(__file__).resolve().parent.parent / "lib"


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(args) -> None:
    import torch
    import torch.distributed as dist

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    verbose = bool(int(os.environ.get("BENCH_PLUGIN_VERBOSE", "0")))
    if verbose:   # where every rank stands, should the job stop moving
        import faulthandler
        faulthandler.dump_traceback_later(int(os.environ.get("BENCH_PLUGIN_DUMP_AFTER", "25")), exit=False)

    def say(msg):
        if verbose:
            print(f"[bench_plugin rank {rank}] {msg}", file=sys.stderr, flush=True)

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    say("process group up")
    rows = []
    size = args.min_bytes
    while size <= args.max_bytes:
        numel = max(world, (size // 2 + world - 1) // world * world)
        torch.manual_seed(1 + rank)
        x = torch.randn(numel, device=dev).bfloat16()
        part = torch.empty(numel // world, device=dev, dtype=torch.bfloat16)
        y = torch.empty_like(x)
        # correctness once per size: all_reduce against an fp64 sum of the gathered inputs
        xs = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(xs, x)
        torch.cuda.synchronize(dev)
        say(f"{numel * 2} bytes: all_gather for the check done")
        z = x.clone()
        dist.all_reduce(z)
        if os.environ.get("BENCH_PLUGIN_SYNC_AFTER_CHECK") == "1":
            torch.cuda.synchronize(dev)
        ref = sum(t.double() for t in xs)
        ok = bool(torch.allclose(z.double(), ref, rtol=5e-2, atol=5e-2 * world))
        say(f"{numel * 2} bytes: check {ok}")
        calls = {"all_reduce": (lambda: dist.all_reduce(x), 2 * (world - 1) / world),
                 "all_gather": (lambda: dist.all_gather_into_tensor(y, part), (world - 1) / world),
                 "reduce_scatter": (lambda: dist.reduce_scatter_tensor(part, y), (world - 1) / world),
                 "all_to_all": (lambda: dist.all_to_all_single(y, x), (world - 1) / world)}
        iters = args.iters if size <= (8 << 20) else max(3, args.iters // 4)
        for name, (fn, factor) in calls.items():
            for _ in range(args.warmup if size <= (8 << 20) else 2):
                fn()
            torch.cuda.synchronize(dev)
            dist.barrier()
            # the waiting thread sleeps instead of spinning: with traffic through a net plugin every rank also has a
            # proxy thread that has to run, and a box may have no more cores than that
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True, blocking=True)
            a.record()
            for _ in range(iters):
                fn()
            b.record()
            b.synchronize()
            t = torch.tensor([a.elapsed_time(b) / iters], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            say(f"{numel * 2} bytes: {name} {ms * 1e3:.1f} us")
            rows.append({"coll": name, "bytes": numel * 2, "us": ms * 1e3, "busbw_GBs": numel * 2 * factor / ms / 1e6,
                         "correct": ok})
        if rank == 0:
            print(f"[bench_plugin] {numel * 2} bytes done", file=sys.stderr, flush=True)
        size *= 2
    if rank == 0:
        print("PLUGIN_BENCH_ROWS " + json.dumps(rows), flush=True)
    dist.destroy_process_group()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--min-bytes", type=int, default=8)
    ap.add_argument("--max-bytes", type=int, default=256 << 20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    # the socket arm is opt-in: on a box whose loopback NCCL cannot use for NET/Socket it waits until the timeout
    ap.add_argument("--arms", nargs="+", default=["plugin"], choices=["plugin", "socket"])
    ap.add_argument("--timeout", type=int, default=240, help="seconds per arm")
    ap.add_argument("--json")
    ap.add_argument("--worker", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args(argv)
    if args.worker:
        _worker(args)
        return 0
    result = {"gpus": args.gpus}
    for arm in args.arms:
        env = dict(os.environ, NCCL_P2P_DISABLE="1", NCCL_SHM_DISABLE="1", NCCL_NVLS_ENABLE="0")
        # The plugin's proxy thread launches copy kernels while NCCL's kernel waits for them, so
        # nothing in the process may make the device wait for that kernel first: kernels are loaded
        # when the process starts (a lazy load synchronises the context) and the device gets its
        # full set of hardware work queues (fewer queues shared by more streams).
        env.setdefault("CUDA_MODULE_LOADING", "EAGER")
        env.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")
        # all_to_all: eight channels per peer (NCCL reads this before it loads the plugin, whose own
        # environment defaults therefore cannot supply it); measured on two GPUs only, larger jobs keep
        # NCCL's default unless the caller exports the variable
        if arm == "plugin" and args.gpus <= 2:
            env.setdefault("NCCL_NCHANNELS_PER_NET_PEER", "8")
        if arm == "plugin":
            env.update(NCCL_NET_PLUGIN="ofi-b200", LD_LIBRARY_PATH=f"{LIB}:" + env.get("LD_LIBRARY_PATH", ""))
        else:
            env.update(NCCL_NET="Socket", NCCL_NET_PLUGIN="none", NCCL_SOCKET_IFNAME="lo")
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), "-m",
               "aws_ofi_nccl_b200.utils.bench_plugin", "--worker", "--min-bytes", str(args.min_bytes), "--max-bytes",
               str(args.max_bytes), "--warmup", str(args.warmup), "--iters", str(args.iters)]
        rc, out, err = run_job(cmd, env=env, timeout=args.timeout)   # ends every rank when the limit passes
        if rc is None:
            print(f"{arm}: timed out\n{out[-3000:]}\n{err[-3000:]}", flush=True)
            continue
        got = [ln for ln in out.splitlines() if ln.startswith("PLUGIN_BENCH_ROWS ")]
        if rc != 0 or not got:
            print(f"{arm}: failed\n{err[-1500:]}", flush=True)
            continue
        result[arm] = json.loads(got[-1][len("PLUGIN_BENCH_ROWS "):])
    if "plugin" in result:
        other = {(r["coll"], r["bytes"]): r for r in result.get("socket", [])}
        print(f"{'coll':<15}{'bytes':>12}{'plugin us':>12}{'plugin GB/s':>13}{'socket us':>12}{'socket GB/s':>13}  ok")
        for r in result["plugin"]:
            o = other.get((r["coll"], r["bytes"]))
            print(f"{r['coll']:<15}{r['bytes']:>12}{r['us']:>12.1f}{r['busbw_GBs']:>13.2f}"
                  + (f"{o['us']:>12.1f}{o['busbw_GBs']:>13.2f}" if o else f"{'-':>12}{'-':>13}") + f"  {r['correct']}")
    if args.json:
        with open(args.json, "w") as f:
            json.dump(result, f, indent=1)
    return 0 if "plugin" in result else 1


if __name__ == "__main__":
    sys.exit(main())
