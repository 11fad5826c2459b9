"""CPU checks of the host-side arithmetic of the parallel layers: weight interleaving, window
layouts and staging sizes, and the numeric ids the tuner tools share with the plugin's ABI header."""
import re
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent


def test_gate_up_interleave_round_trip_and_block_layout():
    from aws_ofi_nccl_b200.parallel import tensor_parallel as tp

    F, H = 96, 8
    g = torch.arange(F * H, dtype=torch.float32).view(F, H)
    u = -g
    w = tp.interleave_gate_up(g, u)
    assert w.shape == (2 * F, H)
    # 32 gate rows, then the matching 32 up rows, and so on
    assert torch.equal(w[0:32], g[0:32]) and torch.equal(w[32:64], u[0:32]) and torch.equal(w[64:96], g[32:64])
    g2, u2 = tp.deinterleave_gate_up(w)
    assert torch.equal(g2, g) and torch.equal(u2, u)


def test_gemm_rs_staging_is_two_parities_of_the_ring_hops():
    from aws_ofi_nccl_b200.parallel import tensor_parallel as tp

    assert tp.gemm_rs_staging_bytes(1, 4096, 4096) == 0
    assert tp.gemm_rs_staging_bytes(2, 8192, 4096) == 2 * 1 * 4096 * 4096 * 2
    assert tp.gemm_rs_staging_bytes(8, 8192, 4096) == 2 * 7 * 1024 * 4096 * 2
    # the MLP reserves room for the gathered input, the gathered output gradient and the staging
    for world in (1, 2, 8):
        need = 2 * tp._align(8192 * 4096 * 2) + tp.gemm_rs_staging_bytes(world, 8192, 4096)
        assert tp.TensorParallelMLP.window_bytes(8192, 4096) >= need


def test_expert_parallel_window_layout_is_aligned_and_disjoint():
    from aws_ofi_nccl_b200.parallel.expert_parallel import ExpertParallel, _align

    world, T, H, E, k = 8, 4096, 7168, 256, 8
    total = ExpertParallel.window_bytes(world, T, H, E, k, 2.0)
    cap = min(world * T * k, max(1024, int(2.0 * T * k)))
    parts = [2 * world * E * 4, cap * H * 2, cap * (H // 128) * 4, cap * 16, T * k * H * 2]
    assert total >= sum(_align(p) for p in parts)
    assert total < 4 << 30   # 4096 tokens per rank, hidden 7168, top-8: fits a 4 GiB window per rank
    # a capacity factor above the worst case is clamped to the worst case
    assert ExpertParallel.window_bytes(2, 128, 256, 8, 2, 100.0) == ExpertParallel.window_bytes(2, 128, 256, 8, 2, 1e9)


def test_tool_ids_match_the_abi_header():
    from aws_ofi_nccl_b200.utils import tuner_calibrate, tuner_cli

    hdr = (ROOT / "aws-ofi-nccl_b200" / "csrc" / "include" / "nccl_abi.h").read_text()
    algo = {m.group(1): int(m.group(2)) for m in re.finditer(r"#define NCCL_ALGO_(\w+) (\d+)", hdr)}
    proto = {m.group(1): int(m.group(2)) for m in re.finditer(r"#define NCCL_PROTO_(\w+) (\d+)", hdr)}
    funcs = {m.group(1): int(m.group(2)) for m in re.finditer(r"ncclFunc(\w+) = (\d+)", hdr)}
    assert tuner_calibrate.ALGOS == {"Tree": algo["TREE"], "Ring": algo["RING"], "NVLS": algo["NVLS"],
                                     "NVLSTree": algo["NVLS_TREE"], "PAT": algo["PAT"]}
    assert tuner_calibrate.PROTOS == {"LL": proto["LL"], "LL128": proto["LL128"], "Simple": proto["SIMPLE"]}
    assert tuner_calibrate.COLLS == {"all_gather": funcs["AllGather"], "reduce_scatter": funcs["ReduceScatter"],
                                     "all_reduce": funcs["AllReduce"]}
    assert tuner_cli.ALGOS[algo["NVLS_TREE"]] == "NVLSTree" and tuner_cli.PROTOS[proto["SIMPLE"]] == "Simple"
    for name, idx in tuner_cli.COLLS.items():
        assert funcs["".join(p.capitalize() for p in name.split("_"))] == idx


def test_roofline_denominator_falls_back_when_no_measurement_file(tmp_path, monkeypatch):
    from aws_ofi_nccl_b200.utils import bench_tp

    tflops, source = bench_tp._peak_tflops()
    assert tflops > 0 and source in ("measured", "fallback")
    if source == "fallback":
        assert tflops == bench_tp.FALLBACK_TFLOPS
