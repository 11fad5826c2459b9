"""Multi-GPU tests: each launches a torchrun job over the visible GPUs (2..8) and checks its exit code."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from aws_ofi_nccl_b200.utils.proc import run_job  # noqa: E402


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(worker: str, nproc: int, env_extra: dict | None = None, timeout: int = 600):
    env = dict(os.environ)
    env.update(env_extra or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(ROOT / "tests" / "workers" / worker)]
    # when the limit passes, the launcher AND every worker it started are ended (a worker left
    # behind would keep its kernels spinning on the GPU)
    rc, out, err = run_job(cmd, env=env, cwd=ROOT, timeout=timeout)
    assert rc is not None, f"{worker} on {nproc} ranks did not finish within {timeout} s\n" + out[-3000:] + err[-3000:]
    assert rc == 0, out[-4000:] + err[-4000:]
    return out


def _ngpus() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_ngpus() < 2, reason="needs at least 2 GPUs")
def test_device_collectives_all_gpus():
    out = _run("collectives_worker.py", min(_ngpus(), 8))
    assert "collectives worker OK" in out


@pytest.mark.skipif(_ngpus() < 2, reason="needs at least 2 GPUs")
def test_device_collectives_p2p_only():
    out = _run("collectives_worker.py", 2, {"B200NET_NVLS_ENABLE": "0"})
    assert "collectives worker OK" in out


@pytest.mark.skipif(_ngpus() < 2, reason="needs at least 2 GPUs")
def test_data_parallel_gradients_and_replicas():
    out = _run("dp_worker.py", min(_ngpus(), 4))
    assert "dp worker OK" in out


@pytest.mark.skipif(_ngpus() < 2, reason="needs at least 2 GPUs")
def test_unmodified_nccl_runs_over_the_net_plugin(tmp_path):
    """NCCL loads the plugin through NCCL_NET_PLUGIN; P2P and SHM transports are off, so every byte
    between the two GPUs crosses isend/irecv/test of this repository's plugin."""
    lib = ROOT / "aws-ofi-nccl_b200" / "lib"
    log = tmp_path / "nccl.log"
    env = {
        "NCCL_NET_PLUGIN": "ofi-b200", "LD_LIBRARY_PATH": f"{lib}:" + os.environ.get("LD_LIBRARY_PATH", ""),
        "NCCL_P2P_DISABLE": "1", "NCCL_SHM_DISABLE": "1", "NCCL_DEBUG": "INFO", "NCCL_DEBUG_SUBSYS": "INIT,NET",
        "NCCL_DEBUG_FILE": str(log) + ".%p", "NCCL_NVLS_ENABLE": "0", "NCCL_CUMEM_ENABLE": "0",
    }
    # a job that stalls is cut off after three minutes and fails the test; it is never run again
    out = _run("nccl_plugin_worker.py", 2, env, timeout=180)
    assert "nccl plugin worker OK" in out
    text = "".join(p.read_text() for p in tmp_path.glob("nccl.log.*"))
    assert "B200NVL" in text, text[-3000:]


@pytest.mark.skipif(_ngpus() < 1, reason="needs a GPU")
def test_fused_tp_kernels_single_rank():
    """World size 1: the fused kernels degenerate to a gated GEMM and a local reduction."""
    out = _run("tp_worker.py", 1)
    assert "TP_WORKER_OK" in out


@pytest.mark.skipif(_ngpus() < 2, reason="needs at least 2 GPUs")
def test_fused_tp_kernels_all_gpus():
    out = _run("tp_worker.py", min(_ngpus(), 8))
    assert "TP_WORKER_OK" in out


@pytest.mark.skipif(_ngpus() < 1, reason="needs a GPU")
def test_moe_dispatch_combine_single_rank():
    out = _run("moe_worker.py", 1)
    assert "MOE_WORKER_OK" in out


@pytest.mark.skipif(_ngpus() < 2, reason="needs at least 2 GPUs")
def test_moe_dispatch_combine_all_gpus():
    out = _run("moe_worker.py", min(_ngpus(), 8))
    assert "MOE_WORKER_OK" in out
