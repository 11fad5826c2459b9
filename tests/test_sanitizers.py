"""The host code under ASAN + UBSAN and under TSAN: every C++ unit test, the two-process functional
test of both protocols and the multi-threaded connection scenario run against sanitizer builds of
the plugin.  Skipped when the toolchain has no sanitizer runtimes (B200NET_SKIP_SANITIZERS=1 skips
it by hand)."""
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "aws-ofi-nccl_b200" / "build" / "san"

pytestmark = pytest.mark.skipif(os.environ.get("B200NET_SKIP_SANITIZERS") == "1", reason="disabled by environment")


def _build(kind: str):
    from aws_ofi_nccl_b200 import build
    try:
        build.build_host(sanitize=kind)
        build.build_tests(sanitize=kind)
    except RuntimeError as e:
        pytest.skip(f"no {kind} sanitizer build on this toolchain: {e}")
    return LIB / f"tests-{kind}", LIB / f"libnccl-net-ofi-b200-{kind}.so"


def _run(cmd, env_extra=None, timeout=600):
    env = dict(os.environ)
    env.update(env_extra or {})
    res = subprocess.run([str(c) for c in cmd], capture_output=True, text=True, timeout=timeout, env=env, cwd=LIB)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-6000:]
    assert "runtime error" not in res.stderr, res.stderr[-6000:]


def test_address_and_undefined_behaviour():
    tests, so = _build("address,undefined")
    for exe in sorted(tests.glob("unit_*")):
        _run([exe])
    scenarios = ["connection", "message_transfer", "pingpong", "grouped_recv", "eager", "reuse_listen", "threads", "bandwidth", "proxy_pattern", "eager_multirecv"]
    for proto in ("SENDRECV", "RDMA"):
        for sc in scenarios:
            # leak checking stays on for the single-process unit tests only: LeakSanitizer's report
            # on a forked two-process run was not reproducible from one run to the next
            _run([tests / "func_net", so, sc],
                 {"B200NET_PROTOCOL": proto, "B200NET_FORCE_NUM_RAILS": "2", "ASAN_OPTIONS": "detect_leaks=0"})
        # a communicator closed with requests in flight abandons those requests by design
        _run([tests / "func_net", so, "inflight_close"],
             {"B200NET_PROTOCOL": proto, "ASAN_OPTIONS": "detect_leaks=0"})
    for sc in ("drop_conn", "peer_exit"):
        _run([tests / "func_fault", so, sc], {"ASAN_OPTIONS": "detect_leaks=0"})
    # device payloads against the stand-in driver: IPC mappings, copy / pack "kernels" that finish
    # later, and the staged fallback when the peer's memory cannot be mapped
    from aws_ofi_nccl_b200 import build
    build.build_fake_cuda()
    fake = f"{build.LIB / 'tests' / 'fake_cuda'}:" + os.environ.get("LD_LIBRARY_PATH", "")
    for extra in ({}, {"FUNC_RMA_HOST_TARGETS": "1"}, {"FUNC_RMA_HOST_SOURCES": "2", "B200NET_DISABLE_CMA": "1"},
                  {"FAKE_CUDA_VMM": "1"}, {"FAKE_CUDA_FAIL_IPC_GET": "1"}, {"FUNC_RMA_MULTISEG": "1"}):
        _run([tests / "func_rma", so, 3],
             {"ASAN_OPTIONS": "detect_leaks=0", "FUNC_NET_DEVICE": "1", "LD_LIBRARY_PATH": fake, **extra})
    # a copy-kernel launch that fails: the error path through the completion word of a queued stripe
    _run([tests / "func_fault", so, "kernel_launch_failure"], {"ASAN_OPTIONS": "detect_leaks=0", "LD_LIBRARY_PATH": fake})
    for extra in ({"FAKE_CUDA_LAUNCH_DELAY_US": "200"}, {"FAKE_CUDA_FAIL_IPC_OPEN": "1"}, {"FAKE_CUDA_VMM": "1"}):
        for sc in ("device_transfer", "grouped_recv", "eager", "proxy_pattern"):
            _run([tests / "func_net", so, sc],
                 {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "2", "ASAN_OPTIONS": "detect_leaks=0",
                  "FUNC_NET_DEVICE": "1", "LD_LIBRARY_PATH": fake, **extra})


def test_thread_sanitizer():
    tests, so = _build("thread")
    for exe in sorted(tests.glob("unit_*")):
        _run([exe])
    _run([tests / "func_net", so, "threads"], {"B200NET_PROTOCOL": "RDMA"})
    # the copy workers and the proxy thread share stripes' status words
    _run([tests / "func_net", so, "bandwidth"], {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "4",
                                                  "B200NET_HOST_COPY_THREADS": "4"})
    _run([tests / "func_net", so, "proxy_pattern"], {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "4",
                                                      "B200NET_HOST_COPY_THREADS": "4"})
    # the helper thread that maps peers' device memory hands its result to the proxy thread
    # (against a copy of the stand-in driver built with the same instrumentation, so that the
    # release / acquire pairs between its "kernels" and the plugin are visible to the detector)
    from aws_ofi_nccl_b200 import build
    fake = f"{build.build_fake_cuda(sanitize='thread').parent}:" + os.environ.get("LD_LIBRARY_PATH", "")
    _run([tests / "func_net", so, "proxy_pattern"],
         {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "2", "FUNC_NET_DEVICE": "1", "LD_LIBRARY_PATH": fake,
          "FAKE_CUDA_IPC_OPEN_DELAY_MS": "20", "B200NET_IPC_MAP_WAIT_US": "100", "FAKE_CUDA_LAUNCH_DELAY_US": "100"})
    # device payloads with "kernels" that finish on another thread: completion words, eager slots
    for sc in ("device_transfer", "eager_multirecv"):
        _run([tests / "func_net", so, sc],
             {"B200NET_PROTOCOL": "RDMA", "B200NET_FORCE_NUM_RAILS": "2", "FUNC_NET_DEVICE": "1", "LD_LIBRARY_PATH": fake,
              "FAKE_CUDA_LAUNCH_DELAY_US": "100"})
    # GIN / RMA: the proxy thread, the device-signal worker and (for served reads) the peers' requests
    _run([tests / "func_rma", so, 3])
    for extra in ({}, {"FAKE_CUDA_VMM": "1"}, {"FUNC_RMA_HOST_SOURCES": "2", "B200NET_DISABLE_CMA": "1"}):
        _run([tests / "func_rma", so, 3], {"FUNC_NET_DEVICE": "1", "LD_LIBRARY_PATH": fake, **extra})
