"""The tuner inspection CLI against the built plugin (CPU only)."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _cli(*args):
    res = subprocess.run([sys.executable, "-m", "aws_ofi_nccl_b200.utils.tuner_cli", "--json", *args],
                         capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert res.returncode == 0, res.stderr
    return json.loads(res.stdout)


def test_decision_edges_per_platform(built):
    out = _cli("--platform", "p6-b200.48xlarge", "--platform", "m5.large", "--nodes", "16", "--collectives", "all_reduce")
    b200, unknown = out
    assert b200["active"] and not unknown["active"]
    rows = b200["collectives"]["all_reduce"]
    assert rows[0]["decision"][:2] == ["Tree", "LL"]
    assert rows[-1]["decision"][:2] == ["NVLSTree", "Simple"]
    edges = [r["from_bytes"] for r in rows]
    assert edges == sorted(edges) and 384 * 1024 + 1 in edges  # 384 KiB itself is still LL (edges are inclusive)


def test_single_node_nvswitch_box_is_tuned(built):
    (out,) = _cli("--platform", "DGX B200", "--nodes", "1", "--collectives", "all_reduce", "all_gather")
    assert out["active"]
    assert out["collectives"]["all_reduce"][-1]["decision"][:2] == ["NVLS", "Simple"]


def test_measured_table_drives_decisions(built, tmp_path):
    table = {"world": 8, "rows": [
        {"coll": 4, "algo": 1, "proto": 0, "nchannels": 2, "bytes": 1024, "time_us": 5.0},
        {"coll": 4, "algo": 0, "proto": 0, "nchannels": 2, "bytes": 1024, "time_us": 9.0},
        {"coll": 4, "algo": 4, "proto": 2, "nchannels": 16, "bytes": 1 << 26, "time_us": 100.0},
        {"coll": 4, "algo": 1, "proto": 2, "nchannels": 16, "bytes": 1 << 26, "time_us": 300.0}]}
    path = tmp_path / "measured.json"
    path.write_text(json.dumps(table))
    (out,) = _cli("--platform", "DGX B200", "--nodes", "1", "--table", str(path), "--collectives", "all_reduce")
    rows = out["collectives"]["all_reduce"]
    assert rows[0]["decision"] == ["Ring", "LL", 2]
    assert rows[-1]["decision"] == ["NVLS", "Simple", 16]


def test_transport_tuner_and_channel_sweep_show_channel_only_decisions(built):
    """Ranks that only reach each other through the plugin (one per "node"): the tuner sets channel
    counts and leaves algorithm and protocol to NCCL; the shipped sweep of two B200 does the same
    through the measured tuner."""
    (out,) = _cli("--platform", "DGX B200", "--nodes", "8", "--ranks-per-node", "1", "--collectives", "all_reduce",
                  "all_gather")
    assert out["active"]
    for coll in ("all_reduce", "all_gather"):
        rows = out["collectives"][coll]
        assert all(r["decision"][0] is None and r["decision"][1] is None for r in rows)
        chans = [r["decision"][2] for r in rows]
        assert chans[0] == 1 and chans[-1] == 16 and chans == sorted(chans)
    # an all_gather of 8 MiB over 8 ranks moves 1 MiB per step: 8 channels, as a 1 MiB step of all_reduce would not (2)
    ag = {r["from_bytes"]: r["decision"][2] for r in out["collectives"]["all_gather"]}
    assert max(c for b, c in ag.items() if b <= 8 << 20) == 8
    table = ROOT / "aws-ofi-nccl_b200" / "data" / "transport_channels_b200_x2.json"
    (swept,) = _cli("--platform", "DGX B200", "--nodes", "2", "--ranks-per-node", "1", "--tuner-type", "Measured", "--table",
                    str(table), "--collectives", "all_reduce")
    rows = swept["collectives"]["all_reduce"]
    assert rows[0]["decision"] == [None, None, 1] and rows[-1]["decision"][2] >= 16
