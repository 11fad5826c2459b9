"""The plugin's device-buffer paths on real GPUs, through the public ncclNet table: two processes,
payloads in device memory (one GPU per rank where there are two), the plugin's own copy and
eager-pack kernels, IPC mapping of the peer's buffers, byte-exact checks through host mirrors.
The same binaries run on CPU against a stand-in driver (test_net_device_paths_cpu.py)."""
import json
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu


# legacy: cuMemAlloc buffers (small ones share a backing block); vmm: cuMemCreate buffers, as NCCL's own are
ALLOCATORS = {"legacy": {}, "vmm": {"FUNC_NET_VMM": "1"}}


@pytest.mark.parametrize("allocator", list(ALLOCATORS))
@pytest.mark.parametrize("scenario", ["device_transfer", "proxy_pattern"])
def test_functional_scenarios_on_device_memory(built, tmp_path, scenario, allocator):
    env = dict(os.environ, FUNC_NET_DEVICE="1", B200NET_PROTOCOL="RDMA", B200NET_FORCE_NUM_RAILS="4",
               B200NET_STATS_FILE=str(tmp_path / "stats.%p.json"), **ALLOCATORS[allocator])
    res = subprocess.run([str(built / "tests" / "func_net"), str(built / "libnccl-net-ofi-b200.so"), scenario],
                         capture_output=True, text=True, timeout=180, env=env, cwd=built)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "host buffers" not in res.stderr, "the test fell back to host memory:\n" + res.stderr[-2000:]
    files = sorted(tmp_path.glob("stats.*.json"))
    assert len(files) == 2, files
    for f in files:
        c = json.loads(f.read_text())["counters"]
        # device payloads leave through the plugin's copy kernel, never as a host write
        assert c["bytes_copy_kernel"] > 0, c
        assert c["bytes_host_writes"] == 0 and c["requests_failed"] == 0, c


@pytest.mark.parametrize("allocator", list(ALLOCATORS))
@pytest.mark.parametrize("exe,ranks", [("func_ring", 4), ("func_rma", 3)])
def test_ring_and_rma_on_device_memory(built, tmp_path, exe, ranks, allocator):
    """N processes (spread over the visible GPUs): a ring with 32 sends and 32 receives of device
    memory in flight per rank, and the RMA / GIN tables with windows, sources and signal words in
    device memory."""
    env = dict(os.environ, FUNC_NET_DEVICE="1", B200NET_PROTOCOL="RDMA", B200NET_FORCE_NUM_RAILS="4",
               B200NET_STATS_FILE=str(tmp_path / "stats.%p.json"), **ALLOCATORS[allocator])
    res = subprocess.run([str(built / "tests" / exe), str(built / "libnccl-net-ofi-b200.so"), str(ranks)],
                         capture_output=True, text=True, timeout=180, env=env, cwd=built)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "host buffers" not in res.stderr, "the test fell back to host memory:\n" + res.stderr[-2000:]
    stats = [json.loads(f.read_text())["counters"] for f in sorted(tmp_path.glob("stats.*.json"))]
    assert len(stats) == ranks, stats
    for c in stats:
        assert c["requests_failed"] == 0 and c["endpoints_aborted"] == 0, c
        if exe == "func_rma":
            assert c["gin_puts"] > 0 and c["gin_bytes_host_writes"] == 0, c
