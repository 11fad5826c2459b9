"""The plugin's device-buffer paths (IPC mapping of a peer's registration, the copy-and-flag and
eager-pack kernels, copy-engine fallback, staging when a peer cannot be mapped) run here without a
GPU: the test binary and the plugin load a stand-in ``libcuda.so.1`` whose "device memory" is
shared host memory and whose "kernels" are host functions that finish after a chosen delay.  The
addresses it hands out as device memory are mapped without access rights, so any place where the
plugin touches a device buffer with the CPU (instead of going through a copy or a kernel) faults
here, as it would on a GPU.  The stand-in is test code only; the plugin itself is the unmodified
shipped library."""
import os
import re
import subprocess

import pytest


def _run(built, env_extra, scenario=None, timeout=400):
    fake = built / "tests" / "fake_cuda"
    assert (fake / "libcuda.so.1").exists(), "the stand-in driver was not built"
    # the throughput scenario stops at 1 MiB messages here: it is run for its checks, not its figures
    env = dict(os.environ, FUNC_NET_DEVICE="1", FUNC_NET_VERBOSE="1", FUNC_NET_BW_MAX=str(1 << 20))
    env["LD_LIBRARY_PATH"] = f"{fake}:" + env.get("LD_LIBRARY_PATH", "")
    env.update(env_extra)
    cmd = [str(built / "tests" / "func_net"), str(built / "libnccl-net-ofi-b200.so")]
    if scenario:
        cmd.append(scenario)
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=built)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    return res.stderr


_COUNTERS = re.compile(r"copy kernel (\d+), copy engine (\d+), staged through host (\d+), host writes (\d+), eager (\d+)")


def _payload_counters(log):
    """Sums the per-endpoint byte counters the plugin logs when an endpoint closes (lines of the
    two ranks can interleave on the shared stderr; a torn line is skipped)."""
    names = ("copy kernel", "copy engine", "staged through host", "host writes", "eager")
    total = dict.fromkeys(names, 0)
    for m in _COUNTERS.finditer(log):
        for n, v in zip(names, m.groups()):
            total[n] += int(v)
    return total


def test_bursts_of_stripes_share_launches_of_the_batch_kernel(built, tmp_path):
    """NCCL's proxy pattern (many channels, one driving thread) with kernels that take a while: the
    stripes posted while earlier launches run leave in launches of the batch kernel, several per
    launch, and every byte still arrives (the scenario checks them). With B200NET_COPY_BATCH=0
    every stripe is a launch of its own."""
    import json

    def counters(extra, tag):
        env = {"B200NET_PROTOCOL": "RDMA", "FAKE_CUDA_LAUNCH_DELAY_US": "300",
               "B200NET_STATS_FILE": str(tmp_path / f"{tag}.%p.json")}
        env.update(extra)
        _run(built, env, "proxy_pattern")
        total = {}
        for f in tmp_path.glob(f"{tag}.*.json"):
            for k, v in json.loads(f.read_text())["counters"].items():
                total[k] = total.get(k, 0) + v
        return total

    on = counters({}, "on")
    assert on["bytes_copy_kernel"] > 0
    assert on["copy_batch_launches"] > 0, on
    assert on["copy_batched_stripes"] >= 2 * on["copy_batch_launches"]
    off = counters({"B200NET_COPY_BATCH": "0"}, "off")
    assert off["bytes_copy_kernel"] == on["bytes_copy_kernel"]
    assert off["copy_batch_launches"] == 0
    assert off["copy_kernel_launches"] > on["copy_kernel_launches"]


@pytest.mark.parametrize("delay_us", ["0", "300"], ids=["sync-kernels", "async-kernels"])
@pytest.mark.parametrize("proto", ["RDMA", "SENDRECV"])
def test_every_scenario_with_device_buffers(built, proto, delay_us):
    _run(built, {"B200NET_PROTOCOL": proto, "B200NET_FORCE_NUM_RAILS": "4", "FAKE_CUDA_LAUNCH_DELAY_US": delay_us})


def test_device_payloads_take_the_kernel_and_eager_pack_paths(built):
    log = _run(built, {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "4", "FAKE_CUDA_LAUNCH_DELAY_US": "100"},
               "device_transfer")
    c = _payload_counters(log)
    assert c["copy kernel"] > 0 and c["eager"] > 0, c
    assert c["staged through host"] == 0 and c["host writes"] == 0, c


def test_copy_engine_path_when_the_kernels_are_switched_off(built):
    log = _run(built, {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "2", "B200NET_COPY_KERNEL": "0",
                       "FAKE_CUDA_LAUNCH_DELAY_US": "100"}, "device_transfer")
    c = _payload_counters(log)
    assert c["copy engine"] > 0 and c["copy kernel"] == 0, c


def test_unmappable_peer_memory_falls_back_to_staged_fragments(built):
    """cuIpcOpenMemHandle fails (as between containers): payloads must still arrive, through host
    fragments that the receiver copies to its device, and the plugin says so once."""
    log = _run(built, {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "4", "FAKE_CUDA_FAIL_IPC_OPEN": "1"},
               "device_transfer")
    c = _payload_counters(log)
    assert c["staged through host"] > 0 and c["copy kernel"] == 0 and c["copy engine"] == 0, c
    assert "cannot be mapped here" in log


def test_slow_peer_mapping_does_not_stall_the_sender(built):
    """cuIpcOpenMemHandle can wait for the device to go idle, and the device may be running a
    collective kernel that waits for this very data.  The open therefore runs on a helper thread:
    with an open that takes 300 ms the payloads leave as host fragments after the grace period."""
    log = _run(built, {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "4", "FAKE_CUDA_IPC_OPEN_DELAY_MS": "300",
                       "B200NET_IPC_MAP_WAIT_US": "2000", "FAKE_CUDA_LAUNCH_DELAY_US": "100"}, "device_transfer")
    c = _payload_counters(log)
    assert c["staged through host"] > 0, c
    assert "still in progress" in log
    # the same buffers used again and again: later chunks find the mapping and go direct
    log = _run(built, {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "4", "FAKE_CUDA_IPC_OPEN_DELAY_MS": "20",
                       "B200NET_IPC_MAP_WAIT_US": "100"}, "proxy_pattern")
    c = _payload_counters(log)
    assert c["staged through host"] > 0 and c["copy kernel"] > 0, c


def test_allocations_without_ipc_handles_are_staged(built):
    """Memory of the virtual-memory API has no legacy IPC handle: such registrations are published
    as reachable through host fragments only, and every scenario still passes."""
    log = _run(built, {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "4", "FAKE_CUDA_FAIL_IPC_GET": "1"})
    c = _payload_counters(log)
    assert c["staged through host"] > 0 and c["copy kernel"] == 0 and c["copy engine"] == 0, c


@pytest.mark.parametrize("delay_us", ["0", "200"])
def test_proxy_pattern_on_device_buffers(built, delay_us):
    """NCCL's proxy pattern with device chunks and kernels that complete asynchronously: many
    requests per channel wait on their own completion words while new ones are posted."""
    env = {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "4", "FAKE_CUDA_LAUNCH_DELAY_US": delay_us}
    for _ in range(3):
        _run(built, env, "proxy_pattern")


@pytest.mark.parametrize("nranks,env", [
    (2, {}),
    (3, {"FAKE_CUDA_LAUNCH_DELAY_US": "100"}),
    (4, {"B200NET_DISABLE_CMA": "1"}),
    (3, {"FUNC_RMA_HOST_TARGETS": "1"}),
    (3, {"FUNC_RMA_HOST_TARGETS": "1", "B200NET_DISABLE_CMA": "1"}),
    (3, {"FUNC_RMA_HOST_SOURCES": "1"}),
    (3, {"FUNC_RMA_HOST_SOURCES": "2"}),
    (3, {"FUNC_RMA_HOST_SOURCES": "2", "B200NET_DISABLE_CMA": "1"}),
    (3, {"FAKE_CUDA_FAIL_IPC_GET": "1"}),
    (3, {"FAKE_CUDA_FAIL_IPC_OPEN": "1", "B200NET_DISABLE_CMA": "1"}),
    (3, {"FAKE_CUDA_FAIL_IPC_GET": "1", "FUNC_RMA_HOST_SOURCES": "2"}),
], ids=["2", "3-async", "4-staged", "dev-to-host", "dev-to-host-staged", "host-to-dev", "host-read-into-dev",
        "host-read-into-dev-served", "no-ipc-handles", "ipc-open-fails-staged", "no-ipc-handles-host-sources"])
def test_rma_and_gin_tables_on_device_buffers(built, nranks, env):
    """Puts, signalled puts, gets and flushes with windows, sources and signal words in device
    memory, every host / device pairing of source and target, and device windows that peers cannot
    map (allocations without IPC handles, as the virtual-memory API makes them; handles that cannot
    be opened): those travel as fragments that the owner copies to its device, reads are served by
    the owner, and a kernel-initiated context is refused."""
    fake = built / "tests" / "fake_cuda"
    e = dict(os.environ, FUNC_NET_DEVICE="1")
    e["LD_LIBRARY_PATH"] = f"{fake}:" + e.get("LD_LIBRARY_PATH", "")
    e.update(env)
    res = subprocess.run([str(built / "tests" / "func_rma"), str(built / "libnccl-net-ofi-b200.so"), str(nranks)],
                         capture_output=True, text=True, timeout=300, env=e, cwd=built)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]


@pytest.mark.parametrize("proto,ranks", [("RDMA", 4), ("SENDRECV", 3), ("RDMA", 8)])
def test_ring_of_processes_on_device_buffers(built, proto, ranks):
    """N ranks in a ring, 32 sends and 32 receives of device memory in flight per rank, flush."""
    fake = built / "tests" / "fake_cuda"
    e = dict(os.environ, FUNC_NET_DEVICE="1", B200NET_PROTOCOL=proto, B200NET_FORCE_NUM_RAILS="4",
             FAKE_CUDA_LAUNCH_DELAY_US="100", FAKE_CUDA_DEVICES=str(max(2, ranks)))
    e["LD_LIBRARY_PATH"] = f"{fake}:" + e.get("LD_LIBRARY_PATH", "")
    res = subprocess.run([str(built / "tests" / "func_ring"), str(built / "libnccl-net-ofi-b200.so"), str(ranks)],
                         capture_output=True, text=True, timeout=300, env=e, cwd=built)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]


def test_mapping_helper_thread_hands_over_or_cleans_up(built):
    fake = built / "tests" / "fake_cuda"
    e = dict(os.environ)
    e["LD_LIBRARY_PATH"] = f"{fake}:" + e.get("LD_LIBRARY_PATH", "")
    res = subprocess.run([str(built / "tests" / "drv_ipc_mapper")], capture_output=True, text=True, timeout=120, env=e, cwd=built)
    assert res.returncode == 0 and res.stdout.strip().endswith("ok"), res.stdout[-2000:] + res.stderr[-3000:]


@pytest.mark.parametrize("proto", ["RDMA", "SENDRECV"])
def test_mirror_mode_of_the_test_buffers(built, proto):
    """The buffer mode a GPU box uses (device memory plus a host mirror with explicit copies), run
    here against the stand-in driver so that every copy call in the scenarios is exercised."""
    _run(built, {"B200NET_PROTOCOL": proto, "B200NET_FORCE_NUM_RAILS": "4", "FUNC_NET_MIRROR": "1",
                 "FAKE_CUDA_LAUNCH_DELAY_US": "100"}, "device_transfer")
    _run(built, {"B200NET_PROTOCOL": proto, "B200NET_FORCE_NUM_RAILS": "4", "FUNC_NET_MIRROR": "1"}, "proxy_pattern")
    # the same with buffers made through the plugin's own cuMemCreate wrapper (FUNC_NET_VMM=1 on a GPU box)
    _run(built, {"B200NET_PROTOCOL": proto, "B200NET_FORCE_NUM_RAILS": "4", "FUNC_NET_MIRROR": "1", "FUNC_NET_VMM": "1"},
         "device_transfer")
    fake = built / "tests" / "fake_cuda"
    e = dict(os.environ, FUNC_NET_DEVICE="1", FUNC_NET_MIRROR="1", B200NET_PROTOCOL=proto)
    e["LD_LIBRARY_PATH"] = f"{fake}:" + e.get("LD_LIBRARY_PATH", "")
    for exe, arg in (("func_ring", "3"), ("func_rma", "3")):
        res = subprocess.run([str(built / "tests" / exe), str(built / "libnccl-net-ofi-b200.so"), arg],
                             capture_output=True, text=True, timeout=300, env=e, cwd=built)
        assert res.returncode == 0, exe + res.stdout[-2000:] + res.stderr[-4000:]


def test_buffers_of_the_virtual_memory_api_are_imported_through_a_descriptor(built):
    """NCCL allocates its own buffers with cuMemCreate: no legacy IPC handle exists for them.  The
    owner exports the allocation as a file descriptor, the peer duplicates it (pidfd_getfd), imports
    and maps it, and payloads then take the same copy-kernel path as legacy allocations."""
    log = _run(built, {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "4", "FAKE_CUDA_VMM": "1",
                       "FAKE_CUDA_LAUNCH_DELAY_US": "100"})
    c = _payload_counters(log)
    # (on a loaded machine a mapping can miss its grace period; those few payloads go through host fragments)
    assert c["copy kernel"] > 0 and c["staged through host"] < c["copy kernel"] // 20, c
    # an import that fails degrades to host fragments
    log = _run(built, {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "4", "FAKE_CUDA_VMM": "1",
                       "FAKE_CUDA_FAIL_VMM_IMPORT": "1"}, "device_transfer")
    c = _payload_counters(log)
    assert c["staged through host"] > 0 and c["copy kernel"] == 0, c
    assert "cannot be mapped here" in log
    # buffers registered, released and replaced: descriptor numbers recur, mappings must not
    for _ in range(2):
        _run(built, {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "2", "FAKE_CUDA_VMM": "1"}, "proxy_pattern")


@pytest.mark.parametrize("env,direct", [({}, True), ({"FAKE_CUDA_FAIL_VMM_IMPORT": "1"}, False),
                                        ({"FUNC_RMA_HOST_SOURCES": "2", "B200NET_DISABLE_CMA": "1"}, True)],
                         ids=["imported", "import-fails", "imported-mixed-staged"])
def test_rma_windows_of_the_virtual_memory_api(built, tmp_path, env, direct):
    """Symmetric registrations of cuMemCreate memory (what NCCL's windows are): every peer imports
    the allocation through the exported descriptor at registration; when that fails, puts travel
    as fragments and reads are served by the owner."""
    fake = built / "tests" / "fake_cuda"
    e = dict(os.environ, FUNC_NET_DEVICE="1", FUNC_NET_VERBOSE="1", FAKE_CUDA_VMM="1",
             B200NET_STATS_FILE=str(tmp_path / "stats.%p.json"))
    e["LD_LIBRARY_PATH"] = f"{fake}:" + e.get("LD_LIBRARY_PATH", "")
    e.update(env)
    res = subprocess.run([str(built / "tests" / "func_rma"), str(built / "libnccl-net-ofi-b200.so"), "3"],
                         capture_output=True, text=True, timeout=300, env=e, cwd=built)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "exported as a descriptor" in res.stderr
    assert ("2 of 2 peers mapped directly" in res.stderr) == direct
    # the counters say the same: payload for device windows went direct, or as fragments
    import json
    stats = [json.loads(f.read_text())["counters"] for f in sorted(tmp_path.glob("stats.*.json"))]
    assert len(stats) == 3
    for c in stats:
        assert c["gin_puts"] == 2 * 129 and c["gin_gets"] == 1 and c["gin_signals_applied"] == 2 * 65, c
        assert (c["gin_bytes_direct"] > 0) == direct and (c["gin_bytes_fragments"] > 0) == (not direct), c


@pytest.mark.parametrize("vmm", ["0", "1"])
def test_signal_words_in_a_range_backed_by_several_allocations(built, vmm):
    """One address range, two cuMemCreate allocations behind it, ranks signalling into different
    ones (the reference's rma_multiseg_signal): no single handle covers the registration, so it is
    published without one and signals still land, applied by their owner."""
    fake = built / "tests" / "fake_cuda"
    e = dict(os.environ, FUNC_NET_DEVICE="1", FUNC_NET_VERBOSE="1", FUNC_RMA_MULTISEG="1", FAKE_CUDA_VMM=vmm)
    e["LD_LIBRARY_PATH"] = f"{fake}:" + e.get("LD_LIBRARY_PATH", "")
    res = subprocess.run([str(built / "tests" / "func_rma"), str(built / "libnccl-net-ofi-b200.so"), "4"],
                         capture_output=True, text=True, timeout=300, env=e, cwd=built)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "131072 bytes of device memory: 0 of 3 peers mapped directly" in res.stderr
