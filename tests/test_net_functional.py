"""Functional tests of the net plugin through its exported ABI (two host processes, no GPU)."""
import ctypes
import os
import subprocess

import pytest


def _run(built, env_extra, scenario=None, timeout=400):
    env = dict(os.environ, FUNC_NET_BW_MAX=str(4 << 20))   # the throughput scenario is run for its checks here
    env.update(env_extra)
    cmd = [str(built / "tests" / "func_net"), str(built / "libnccl-net-ofi-b200.so")]
    if scenario:
        cmd.append(scenario)
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=built)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]


@pytest.mark.parametrize("env", [
    {"B200NET_PROTOCOL": "SENDRECV"},
    {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "4"},
    {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "1"},
    {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "4", "B200NET_DISABLE_CMA": "1"},
    {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "4", "B200NET_EAGER_MAX_SIZE": "0"},
    {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "3", "B200NET_MIN_STRIPE_SIZE": "4096",
     "B200NET_MR_CACHE_DISABLE": "1"},
], ids=["sendrecv", "rdma4", "rdma1", "rdma4-staged-writes", "rdma4-no-eager", "rdma3-small-stripes-nocache"])
def test_two_process_scenarios(built, env):
    _run(built, env)


@pytest.mark.parametrize("threads", ["0", "4"])
def test_proxy_pattern_with_many_channels_in_flight(built, threads):
    """Eight channels, eight chunk-sized sends in flight each, one driving thread per process (the
    way NCCL's proxy uses a net plugin), with and without the host copy workers: this is the pattern
    that exposed queued retries naming a recycled request address."""
    env = {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "4", "B200NET_HOST_COPY_THREADS": threads,
           "FUNC_NET_PROXY_CHUNK": str(4 << 20)}
    for _ in range(3):
        _run(built, env, "proxy_pattern")


@pytest.mark.parametrize("proto,rails,ranks", [("RDMA", "4", 4), ("RDMA", "1", 3), ("SENDRECV", "1", 4), ("RDMA", "1", 8)])
def test_ring_of_processes(built, proto, rails, ranks):
    """N ranks in a ring, 32 sends and 32 receives in flight per rank and round, flush, byte-exact."""
    env = dict(os.environ, B200NET_PROTOCOL=proto, B200NET_FORCE_NUM_RAILS=rails)
    cmd = [str(built / "tests" / "func_ring"), str(built / "libnccl-net-ofi-b200.so"), str(ranks)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=built)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]


def test_compat_env_prefix_is_honoured(built):
    # the reference's variable names keep working
    _run(built, {"OFI_NCCL_PROTOCOL": "RDMA", "OFI_NCCL_FORCE_NUM_RAILS": "2"}, "pingpong")


def test_exported_symbols_and_names(built):
    lib = ctypes.CDLL(str(built / "libnccl-net-ofi-b200.so"))
    for v in range(6, 13):
        assert hasattr(lib, f"ncclNetPlugin_v{v}")
    for alias in ("libnccl-net.so", "libnccl-net-b200.so"):
        assert (built / alias).exists()


def test_c_program_can_dlopen_plugin(built):
    res = subprocess.run([str(built / "tests" / "dlopen_c_test"), str(built / "libnccl-net-ofi-b200.so")],
                         capture_output=True, text=True, timeout=60, cwd=built)
    assert res.returncode == 0 and res.stdout.startswith("ok"), res.stdout + res.stderr


def test_plugin_name_follows_nccl_net(built):
    code = ("import ctypes,sys;l=ctypes.CDLL(sys.argv[1]);"
            "p=ctypes.c_char_p.in_dll(l,'ncclNetPlugin_v11');print(p.value.decode())")
    import sys
    so = str(built / "libnccl-net-ofi-b200.so")
    out = subprocess.run([sys.executable, "-c", code, so], capture_output=True, text=True,
                         env={**os.environ, "NCCL_NET": "MyFabric"}).stdout.strip()
    assert out == "MyFabric"
    out = subprocess.run([sys.executable, "-c", code, so], capture_output=True, text=True,
                         env={k: v for k, v in os.environ.items() if k != "NCCL_NET"}).stdout.strip()
    assert out == "B200NVL"


@pytest.mark.parametrize("nranks,env", [
    (2, {"B200NET_PROTOCOL": "SENDRECV"}),
    (3, {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "4"}),
    (4, {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "2", "B200NET_DISABLE_CMA": "1"}),
], ids=["2-sendrecv", "3-rdma", "4-rdma-staged"])
def test_rma_gin_tables_n_processes(built, nranks, env):
    e = dict(os.environ)
    e.update(env)
    res = subprocess.run([str(built / "tests" / "func_rma"), str(built / "libnccl-net-ofi-b200.so"), str(nranks)],
                         capture_output=True, text=True, timeout=300, env=e, cwd=built)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]


def test_gin_trace_ranges_are_closed(built, tmp_path):
    """Every put, put + signal, get and flush that opens a range in the trace closes it, also the
    gets that are served by the owner (staged fabric) and end when the response arrives."""
    import collections
    import json

    e = dict(os.environ)
    e.update({"B200NET_PROTOCOL": "RDMA", "B200NET_DISABLE_CMA": "1", "B200NET_TRACE": "ring",
              "B200NET_TRACE_FILE": str(tmp_path / "trace.%p.json")})
    res = subprocess.run([str(built / "tests" / "func_rma"), str(built / "libnccl-net-ofi-b200.so"), "3"],
                         capture_output=True, text=True, timeout=300, env=e, cwd=built)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    files = sorted(tmp_path.glob("trace.*.json"))
    assert len(files) == 3, files
    for f in files:
        n = collections.Counter(ev["name"] for ev in json.loads(f.read_text())["traceEvents"])
        for kind in ("gin_put", "gin_put_signal", "gin_get", "gin_flush"):
            assert n[kind + "_begin"] == n[kind + "_end"] > 0, (kind, n)


def test_gin_rma_tuner_symbols_exported(built):
    lib = ctypes.CDLL(str(built / "libnccl-net-ofi-b200.so"))
    for sym in ("ncclGinPlugin_v11", "ncclGinPlugin_v13", "ncclGinPlugin_v14", "ncclRmaPlugin_v14", "ncclRmaPlugin_v15",
                "ncclTunerPlugin_v2", "ncclTunerPlugin_v3", "ncclTunerPlugin_v4", "ncclTunerPlugin_v5",
                "ncclTunerPlugin_v6"):
        assert hasattr(lib, sym), sym
    assert (built / "libnccl-tuner-ofi-b200.so").exists()


def test_trace_file_at_finalize(built, tmp_path):
    """B200NET_TRACE=all + B200NET_TRACE_FILE: the ring of tracepoints leaves the process as Chrome
    trace-event JSON, every Send has its SendEnd and every Recv its RecvEnd (the pairs NVTX shows as
    ranges; with no profiler attached the NVTX calls do nothing)."""
    import collections
    import json

    _run(built, {"B200NET_PROTOCOL": "RDMA", "B200NET_TRACE": "all",
                 "B200NET_TRACE_FILE": str(tmp_path / "trace.%p.json")}, "message_transfer")
    files = sorted(tmp_path.glob("trace.*.json"))
    assert len(files) == 2, files
    for f in files:
        ev = json.loads(f.read_text())["traceEvents"]
        n = collections.Counter(e["name"] for e in ev)
        assert n["Send"] == n["SendEnd"] > 0 and n["Recv"] == n["RecvEnd"] > 0, n
        assert n["Send_eager_start"] == n["Send_eager_complete"], n
        assert n["Send_write_segment_start"] == n["Send_write_segment_complete"] > 0, n
        assert n["Write_ctrl_start"] == n["Write_ctrl_end"] > 0, n
        assert n["ProcessCompletionsRdma"] < len(ev) // 2    # polls that found nothing are not traced
        ts = [e["ts"] for e in ev]
        assert ts == sorted(ts)


def test_statistics_file_at_finalize(built, tmp_path):
    """B200NET_STATS_FILE: one JSON object per process with the counters (posts, back-offs, bytes by
    path) and the histograms (sizes, stripes per send, request latencies)."""
    import json

    _run(built, {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "4",
                 "B200NET_STATS_FILE": str(tmp_path / "stats.%p.json")}, "message_transfer")
    files = sorted(tmp_path.glob("stats.*.json"))
    assert len(files) == 2, files
    for f in files:
        d = json.loads(f.read_text())
        c = d["counters"]
        assert c["sends"] == c["recvs"] > 0 and c["connects"] == c["accepts"] == 1
        assert c["eager_sends"] + c["rendezvous_sends"] == c["sends"]
        assert c["send_bytes"] >= c["recv_bytes"] > 0          # sends larger than the posted receive are cut
        assert c["bytes_host_writes"] + c["bytes_eager"] == c["recv_bytes"]
        assert c["flushes"] > 0 and c["requests_failed"] == 0 and c["endpoints_aborted"] == 0
        h = {x["name"]: x for x in d["histograms"]}
        assert h["send_message_size"]["samples"] == c["sends"]
        assert h["stripes_per_send"]["max"] <= 4
        assert h["send_request_latency"]["unit"] == "ns"


def test_a_removed_setting_stops_the_plugin_at_init(built):
    """A script that still carries a setting the reference removed must not run with something else
    silently: init fails and the log says which variable; a deprecated one only warns."""
    exe = [str(built / "tests" / "func_net"), str(built / "libnccl-net-ofi-b200.so"), "connection"]
    env = dict(os.environ, OFI_NCCL_RDMA_MIN_POSTED_BOUNCE_BUFFERS="8", FUNC_NET_VERBOSE="1")
    res = subprocess.run(exe, capture_output=True, text=True, timeout=120, env=env, cwd=built)
    assert res.returncode != 0
    assert "RDMA_MIN_POSTED_BOUNCE_BUFFERS is no longer supported" in res.stderr
    env = dict(os.environ, B200NET_ENDPOINT_PER_COMM="1", FUNC_NET_VERBOSE="1")
    res = subprocess.run(exe, capture_output=True, text=True, timeout=120, env=env, cwd=built)
    assert res.returncode == 0, res.stderr[-2000:]
    assert "ENDPOINT_PER_COMM is deprecated" in res.stderr
