"""Calibration run for the measured-bandwidth tuner: times NCCL's own (algorithm, protocol) choices
on this machine and writes the table that ``B200NET_TUNER_TYPE=Measured`` loads.

    python -m aws_ofi_nccl_b200.utils.tuner_calibrate --gpus 8 --out measured.json \
        [--algos Ring Tree NVLS NVLSTree PAT] [--protos LL LL128 Simple] [--min-bytes 8] [--max-bytes 1073741824]
    python -m aws_ofi_nccl_b200.utils.tuner_calibrate --gpus 8 --plugin-channels 1 2 4 8 16 --out channels.json

The second form times NCCL with all traffic routed through this repository's net plugin, once per
forced channel count (``B200NET_TUNER_FORCE_CHANNELS``), algorithm and protocol left to NCCL; its rows
carry ``algo`` / ``proto`` -1 and decide channels only (``data/transport_channels_b200_x2.json`` is
such a table, measured on two B200).

NCCL reads NCCL_ALGO / NCCL_PROTO once per process, so every (algorithm, protocol) pair is timed by
a torchrun job of its own; pairs NCCL refuses for a collective are simply absent from the table.
Rows: {"coll", "algo", "proto", "nchannels", "bytes", "time_us"} with NCCL's numeric ids, times on
the device with CUDA events, maximum over ranks.  (The reference ships fixed tables measured by its
authors, src/tuner/nccl_ofi_regions.cpp; this produces them on the machine at hand.)
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import sys

from .proc import run_job

ALGOS = {"Tree": 0, "Ring": 1, "NVLS": 4, "NVLSTree": 5, "PAT": 6}
PROTOS = {"LL": 0, "LL128": 1, "Simple": 2}
COLLS = {"all_gather": 2, "reduce_scatter": 3, "all_reduce": 4}


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(args) -> None:
    import torch
    import torch.distributed as dist

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rows = []
    size = args.min_bytes
    while size <= args.max_bytes:
        numel = max(world, (size // 2 + world - 1) // world * world)   # bf16 elements, divisible by the world
        x = torch.randn(numel, device=dev).bfloat16()
        part = torch.empty(numel // world, device=dev, dtype=torch.bfloat16)
        calls = {"all_reduce": lambda: dist.all_reduce(x),
                 "all_gather": lambda: dist.all_gather_into_tensor(x, part),
                 "reduce_scatter": lambda: dist.reduce_scatter_tensor(part, x)}
        iters = args.iters if size <= (16 << 20) else max(3, args.iters // 4)
        for name, fn in calls.items():
            try:
                for _ in range(3):
                    fn()
                torch.cuda.synchronize(dev)
                dist.barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(iters):
                    fn()
                b.record()
                b.synchronize()
                t = torch.tensor([a.elapsed_time(b) / iters * 1e3], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                rows.append({"coll": COLLS[name], "bytes": numel * 2, "time_us": float(t.item())})
            except RuntimeError:   # this algorithm / protocol does not implement the collective
                break
        size *= args.step
    if rank == 0:
        print("CALIBRATION_ROWS " + json.dumps(rows), flush=True)
    dist.destroy_process_group()


def plugin_rows_to_table(world: int, per_channel: dict[int, list[dict]]) -> dict:
    """bench_plugin rows per forced channel count -> the measured tuner's table (rows that failed
    their fp64 check are dropped; all_to_all is point-to-point traffic and not the tuner's call)."""
    rows = []
    for ch, got in sorted(per_channel.items()):
        for r in got:
            if r["coll"] in COLLS and r.get("correct", True):
                rows.append({"coll": COLLS[r["coll"]], "algo": -1, "proto": -1, "nchannels": ch, "bytes": r["bytes"],
                             "time_us": round(r["us"], 1)})
    return {"world": world, "rows": rows}


def _sweep_plugin_channels(args) -> int:
    import tempfile

    per_channel = {}
    for ch in args.plugin_channels:
        with tempfile.NamedTemporaryFile(suffix=".json") as tmp:
            env = dict(os.environ, B200NET_TUNER_FORCE_CHANNELS=str(ch))
            cmd = [sys.executable, "-m", "aws_ofi_nccl_b200.utils.bench_plugin", "--gpus", str(args.gpus), "--min-bytes",
                   str(max(args.min_bytes, 8)), "--max-bytes", str(args.max_bytes), "--iters", str(args.iters), "--timeout",
                   str(args.timeout), "--json", tmp.name]
            rc, out, err = run_job(cmd, env=env, timeout=args.timeout + 30)
            if rc != 0:
                print(f"{ch} channels: no result ({'timed out' if rc is None else 'failed'})", flush=True)
                continue
            per_channel[ch] = json.load(open(tmp.name)).get("plugin", [])
            print(f"{ch} channels: {len(per_channel[ch])} measurements", flush=True)
    table = plugin_rows_to_table(args.gpus, per_channel)
    with open(args.out, "w") as f:
        json.dump(table, f, indent=1)
    print(f"wrote {len(table['rows'])} rows to {args.out}")
    return 0 if table["rows"] else 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--out", default="measured.json")
    ap.add_argument("--algos", nargs="+", default=list(ALGOS), choices=list(ALGOS))
    ap.add_argument("--protos", nargs="+", default=list(PROTOS), choices=list(PROTOS))
    ap.add_argument("--min-bytes", type=int, default=8)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--step", type=int, default=4, help="size multiplier between measurements")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--timeout", type=int, default=300, help="seconds per (algorithm, protocol) job")
    ap.add_argument("--plugin-channels", nargs="+", type=int, default=None,
                    help="sweep these channel counts with the traffic routed through this repository's net plugin")
    ap.add_argument("--worker", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args(argv)
    if args.worker:
        _worker(args)
        return 0
    if args.plugin_channels:
        return _sweep_plugin_channels(args)
    rows = []
    for algo in args.algos:
        for proto in args.protos:
            env = dict(os.environ, NCCL_ALGO=algo, NCCL_PROTO=proto)
            env.pop("NCCL_TUNER_PLUGIN", None)   # measure NCCL's kernels, not an earlier table's choices
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), "-m",
                   "aws_ofi_nccl_b200.utils.tuner_calibrate", "--worker", "--min-bytes", str(args.min_bytes),
                   "--max-bytes", str(args.max_bytes), "--step", str(args.step), "--iters", str(args.iters)]
            rc, out, _ = run_job(cmd, env=env, timeout=args.timeout)   # ends every rank when the limit passes
            if rc is None:
                print(f"{algo}/{proto}: timed out, skipped", flush=True)
                continue
            got = [ln for ln in out.splitlines() if ln.startswith("CALIBRATION_ROWS ")]
            if rc != 0 or not got:
                print(f"{algo}/{proto}: not available here", flush=True)
                continue
            part = json.loads(got[-1][len("CALIBRATION_ROWS "):])
            for r in part:
                r.update(algo=ALGOS[algo], proto=PROTOS[proto], nchannels=0)
            rows += part
            print(f"{algo}/{proto}: {len(part)} measurements", flush=True)
    with open(args.out, "w") as f:
        json.dump({"world": args.gpus, "rows": rows}, f, indent=1)
    print(f"wrote {len(rows)} rows to {args.out}")
    return 0 if rows else 1


if __name__ == "__main__":
    sys.exit(main())
