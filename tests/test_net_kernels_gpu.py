"""The plugin's own device kernels (copy with completion flag, eager pack) driven through the
plugin's driver shim by a C++ program; byte-exact against host memcpy."""
import subprocess

import pytest

pytestmark = pytest.mark.gpu


def test_plugin_copy_and_eager_pack_kernels(built):
    exe = built / "tests" / "gpu_net_kernels"
    assert exe.exists(), f"{exe} was not built"
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, cwd=built)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "ok" in res.stdout
