"""Multi-process CPU test (gloo, world size 3) of the descriptor exchange that the symmetric-memory
allocator uses to pass CUDA VMM handles between the ranks' processes."""
import os
import socket
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_descriptor_exchange_between_three_processes(built):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(ROOT / "tests" / "workers" / "fd_exchange_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT, env=dict(os.environ))
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "FD_EXCHANGE_OK" in res.stdout
