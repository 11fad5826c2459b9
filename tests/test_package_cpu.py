"""CPU-only checks of the package layout, the build and the model bookkeeping."""
import math


def test_import_and_layout():
    import aws_ofi_nccl_b200
    import aws_ofi_nccl_b200.models
    import aws_ofi_nccl_b200.ops
    import aws_ofi_nccl_b200.parallel
    import aws_ofi_nccl_b200.utils

    assert aws_ofi_nccl_b200.__version__


def test_llama3_8b_parameter_count():
    from aws_ofi_nccl_b200.models.llama import LlamaConfig

    cfg = LlamaConfig.llama3_8b()
    n = cfg.num_params()
    assert abs(n - 8.03e9) < 0.01e9, n
    assert math.prod(dict(cfg.param_shapes())["l0.wqkv"]) == 6144 * 4096


def test_kernel_library_builds_for_sm100a(built):
    assert (built / "libb200ops.so").exists()
    import ctypes

    lib = ctypes.CDLL(str(built / "libb200ops.so"))
    for sym in ("b200_gemm_bf16", "b200_rmsnorm_fwd", "b200_adamw", "b200_cross_entropy"):
        assert hasattr(lib, sym)


def test_bench_reference_arm_reports_unavailable():
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    out = subprocess.run([sys.executable, str(root / "bench.py"), "--impl", "reference"], capture_output=True,
                         text=True, check=True).stdout.strip().splitlines()[-1]
    d = json.loads(out)
    assert d["impl"] == "reference" and "unavailable" in d
