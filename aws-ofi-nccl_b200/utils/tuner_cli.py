"""show-tuner-decisions: print where the tuner plugin changes its (algorithm, protocol, channels)
choice as the message size grows, per collective, for one or more platforms.

    python -m aws_ofi_nccl_b200.utils.tuner_cli --platform p6-b200.48xlarge --nodes 16 --ranks-per-node 8
    python -m aws_ofi_nccl_b200.utils.tuner_cli --platform "DGX B200" --nodes 1 --table measured.json

The plugin is loaded with ctypes through its exported ``ncclTunerPlugin_v3`` table.  The platform
is detected once per process, so every platform is queried in a subprocess of its own with
``OFI_NCCL_FORCE_PRODUCT_NAME`` set (reference: contrib/python/ofi_nccl/tuner/cli).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
from pathlib import Path

ALGOS = ["Tree", "Ring", "CollNetDirect", "CollNetChain", "NVLS", "NVLSTree", "PAT"]
PROTOS = ["LL", "LL128", "Simple"]
COLLS = {"broadcast": 0, "reduce": 1, "all_gather": 2, "reduce_scatter": 3, "all_reduce": 4}
LIB = Path(__file__).resolve().parent.parent / "lib" / "libnccl-net-ofi-b200.so"

_LOGFN = C.CFUNCTYPE(None, C.c_int, C.c_ulong, C.c_char_p, C.c_int, C.c_char_p)


class _TunerV3(C.Structure):
    _fields_ = [("name", C.c_char_p),
                ("init", C.CFUNCTYPE(C.c_int, C.c_size_t, C.c_size_t, C.c_void_p, C.POINTER(C.c_void_p))),
                ("getCollInfo", C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_size_t, C.c_int, C.c_void_p, C.c_int, C.c_int,
                                            C.POINTER(C.c_int))),
                ("destroy", C.CFUNCTYPE(C.c_int, C.c_void_p))]


class Tuner:
    def __init__(self, n_ranks: int, n_nodes: int, lib_path: Path = LIB):
        self.lib = C.CDLL(str(lib_path))
        self.table = _TunerV3.in_dll(self.lib, "ncclTunerPlugin_v3")
        self.ctx = C.c_void_p(None)
        rc = self.table.init(n_ranks, n_nodes, None, C.byref(self.ctx))
        if rc != 0:
            raise RuntimeError(f"tuner init failed: {rc}")

    @property
    def active(self) -> bool:
        return bool(self.ctx.value)

    def decide(self, coll: int, nbytes: int, pipe_ops: int = 1):
        """Returns (algo, proto, channels), (None, None, channels) when only the channel count is set,
        or None when the tuner leaves everything to NCCL."""
        cost = ((C.c_float * len(PROTOS)) * len(ALGOS))()
        for a in range(len(ALGOS)):
            for p in range(len(PROTOS)):
                cost[a][p] = 1.0e9
        nch = C.c_int(0)
        rc = self.table.getCollInfo(self.ctx, coll, nbytes, pipe_ops, C.cast(cost, C.c_void_p), len(ALGOS), len(PROTOS),
                                    C.byref(nch))
        if rc != 0:
            raise RuntimeError(f"getCollInfo failed: {rc}")
        for a in range(len(ALGOS)):
            for p in range(len(PROTOS)):
                if cost[a][p] == 0.0:
                    return ALGOS[a], PROTOS[p], nch.value
        if nch.value > 0:   # channels only: algorithm and protocol stay NCCL's choice
            return None, None, nch.value
        return None

    def close(self) -> None:
        if self.ctx.value:
            self.table.destroy(self.ctx)
            self.ctx = C.c_void_p(None)


def decision_edges(tuner: Tuner, coll: int, lo: int = 8, hi: int = 8 << 30) -> list[dict]:
    """Walk sizes by doubling, then bisect every interval whose ends disagree, down to 1 byte."""
    rows = []
    size = lo
    prev_size, prev = lo, tuner.decide(coll, lo)
    rows.append({"from_bytes": lo, "decision": prev})
    while size < hi:
        size *= 2
        cur = tuner.decide(coll, size)
        if cur != prev:
            a, b = prev_size, size
            while b - a > 1:
                mid = (a + b) // 2
                if tuner.decide(coll, mid) == prev:
                    a = mid
                else:
                    b = mid
            rows.append({"from_bytes": b, "decision": tuner.decide(coll, b)})
            prev = tuner.decide(coll, b)
            if prev != cur:  # more than one change inside the interval: keep walking from b
                size = b
        prev_size = size
    return rows


def _query(args) -> dict:
    n_ranks = args.nodes * args.ranks_per_node
    t = Tuner(n_ranks, args.nodes)
    out = {"platform": args.platform, "nodes": args.nodes, "ranks": n_ranks, "active": t.active, "collectives": {}}
    if t.active:
        for name in args.collectives:
            out["collectives"][name] = decision_edges(t, COLLS[name], args.min_bytes, args.max_bytes)
    t.close()
    return out


def _fmt_bytes(n: int) -> str:
    for unit, sh in (("GiB", 30), ("MiB", 20), ("KiB", 10)):
        if n >= 1 << sh:
            return f"{n / (1 << sh):.4g} {unit}"
    return f"{n} B"


def _print(result: dict) -> None:
    print(f"== platform {result['platform'] or '(detected)'}: {result['nodes']} node(s), {result['ranks']} ranks, "
          f"tuner {'active' if result['active'] else 'passive (NCCL decides)'}")
    try:
        import pandas as pd
    except ImportError:
        pd = None
    for coll, rows in result["collectives"].items():
        table = [{"from": _fmt_bytes(r["from_bytes"]),
                  "algorithm": (r["decision"][0] or "NCCL's") if r["decision"] else "-",
                  "protocol": (r["decision"][1] or "NCCL's") if r["decision"] else "-",
                  "channels": (r["decision"][2] or "-") if r["decision"] else "-"} for r in rows]
        print(f"-- {coll}")
        if pd is not None:
            print(pd.DataFrame(table).to_string(index=False))
        else:
            for row in table:
                print("   ", row)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--platform", action="append", default=None, help="product name to impersonate (repeatable)")
    ap.add_argument("--nodes", type=int, default=16)
    ap.add_argument("--ranks-per-node", type=int, default=8)
    ap.add_argument("--collectives", nargs="+", default=["all_reduce", "all_gather", "reduce_scatter"], choices=list(COLLS))
    ap.add_argument("--min-bytes", type=int, default=8)
    ap.add_argument("--max-bytes", type=int, default=8 << 30)
    ap.add_argument("--tuner-type", default=None, choices=["Region", "Model", "Measured", "Internal"])
    ap.add_argument("--table", default=None, help="measured-bandwidth JSON for --tuner-type Measured")
    ap.add_argument("--json", action="store_true", help="print JSON instead of tables")
    ap.add_argument("--worker", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args(argv)
    if args.worker:
        args.platform = os.environ.get("OFI_NCCL_FORCE_PRODUCT_NAME", "")
        print(json.dumps(_query(args)))
        return 0
    results = []
    for plat in (args.platform or [""]):
        env = dict(os.environ)
        if plat:
            env["OFI_NCCL_FORCE_PRODUCT_NAME"] = plat
        if args.tuner_type:
            env["B200NET_TUNER_TYPE"] = args.tuner_type
        if args.table:
            env["B200NET_TUNER_TABLE"] = args.table
            env.setdefault("B200NET_TUNER_TYPE", "Measured")
        cmd = [sys.executable, "-m", "aws_ofi_nccl_b200.utils.tuner_cli", "--worker", "--nodes", str(args.nodes),
               "--ranks-per-node", str(args.ranks_per_node), "--min-bytes", str(args.min_bytes), "--max-bytes",
               str(args.max_bytes), "--collectives", *args.collectives]
        root = Path(__file__).resolve().parent.parent.parent
        env["PYTHONPATH"] = f"{root}:" + env.get("PYTHONPATH", "")
        res = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if res.returncode != 0:
            sys.stderr.write(res.stderr)
            return 1
        results.append(json.loads(res.stdout.strip().splitlines()[-1]))
    if args.json:
        print(json.dumps(results, indent=1))
    else:
        for r in results:
            _print(r)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
