"""Kernel-initiated GIN through the plugin's own handles, on real GPUs: two processes connect through
``ncclGinPlugin_v14``, and a one-thread kernel puts 64 bytes and raises a signal using the
``GinDevHandle`` / ``GinDevWindow`` that ``createContext`` / ``regMrSym`` uploaded; a bounded wait on
a signal nobody raises must give up and set the status word."""
import subprocess

import pytest

pytestmark = pytest.mark.gpu


def test_put_and_signal_from_a_kernel_through_plugin_built_handles(built):
    exe = built / "tests" / "gpu_gin_plugin"
    assert exe.exists(), "the CUDA test program was not built"
    res = subprocess.run([str(exe), str(built / "libnccl-net-ofi-b200.so")], capture_output=True, text=True, timeout=180, cwd=built)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "ok" in res.stdout
