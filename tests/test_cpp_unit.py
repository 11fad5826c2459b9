"""Runs every C++ unit-test program (csrc/tests/*.cpp|.c); each reports through its exit status."""
import os
import subprocess
from pathlib import Path

import pytest

CSRC_TESTS = Path(__file__).resolve().parent.parent / "aws-ofi-nccl_b200" / "csrc" / "tests"
NAMES = sorted(p.stem for p in CSRC_TESTS.glob("unit_*.cpp"))


@pytest.mark.parametrize("name", NAMES)
def test_cpp_unit(built, name):
    exe = built / "tests" / name
    assert exe.exists(), f"{exe} was not built"
    # the tuner test also reads the channel table that ships with the package
    env = dict(os.environ, B200NET_TEST_CHANNEL_TABLE=str(built.parent / "data" / "transport_channels_b200_x2.json"))
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, cwd=built, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
