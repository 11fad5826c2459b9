"""Failure handling of the net plugin with faults made on the host: a dropped connect request, a
dropped write completion, a peer process that exits. No GPU is involved and nothing is made to
hang: every plugin call has to return promptly with a status."""
import subprocess

import pytest


@pytest.mark.parametrize("scenario", ["drop_conn", "drop_completion", "peer_exit"])
def test_host_fault_scenarios(built, scenario):
    cmd = [str(built / "tests" / "func_fault"), str(built / "libnccl-net-ofi-b200.so"), scenario]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=120, cwd=built)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "ok" in res.stdout


def test_failed_copy_to_the_device_is_reported_by_test(built):
    """The stand-in driver makes the receiver's cuMemcpyAsync fail: the receive must end with an error
    from test(), never with a success status and no data."""
    import os
    # the copy engine delivers the payload in this run (with the copy kernels there is no cuMemcpyAsync to fail)
    env = dict(os.environ, B200NET_COPY_KERNEL="0",
               LD_LIBRARY_PATH=f"{built / 'tests' / 'fake_cuda'}:" + os.environ.get("LD_LIBRARY_PATH", ""))
    cmd = [str(built / "tests" / "func_fault"), str(built / "libnccl-net-ofi-b200.so"), "device_copy_failure"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=120, cwd=built, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "ok" in res.stdout


def test_a_failed_copy_kernel_launch_fails_the_send(built):
    """The stand-in driver refuses the launch that carries a queued stripe: the send's test() reports
    an error (it must neither hang nor claim the bytes were delivered)."""
    import os
    env = dict(os.environ, LD_LIBRARY_PATH=f"{built / 'tests' / 'fake_cuda'}:" + os.environ.get("LD_LIBRARY_PATH", ""))
    cmd = [str(built / "tests" / "func_fault"), str(built / "libnccl-net-ofi-b200.so"), "kernel_launch_failure"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=120, cwd=built, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "ok" in res.stdout
