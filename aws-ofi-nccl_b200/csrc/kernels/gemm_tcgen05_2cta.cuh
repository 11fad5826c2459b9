// Persistent bf16 GEMM mainloop on CTA pairs: one 256 x 256 (or 256 x 128) output tile per cluster
// of two CTAs, computed by `tcgen05.mma.cta_group::2` issued from the even ("leader") CTA.
//
// Each CTA loads its own 128 rows of A and its own half of the B tile (32 KB per 64-deep k-block
// instead of the 48 KB a lone CTA needs for a 128 x 256 tile), so six stages fit where the one-CTA
// kernel has four (eight instead of six for the narrow tile) and the L2 traffic per flop drops by
// a third. Each CTA's TMEM holds its
// 128 rows of the accumulator (all 256 columns, double-buffered) and its own epilogue warps store
// them.
//
// Synchronisation (all barriers are mbarriers in shared memory, every wait is bounded):
//   full[s]   leader only : both CTAs' TMA loads report their bytes here
//   empty[s]  both CTAs   : the leader's tcgen05.commit arrives on both (multicast commit)
//   tfull[b]  both CTAs   : accumulator b complete (multicast commit)
//   tempty[b] leader only : all eight epilogue warps of the pair have drained accumulator b
// None of the loads uses cluster multicast; only tcgen05.commit does.
#pragma once
#include "gemm_tcgen05.cuh"

namespace b200 {

template <int BN>   // 256 or 128 output columns per cluster tile
struct Gemm2Smem {
  static constexpr int A_BYTES = 128 * GEMM_BK * 2;
  static constexpr int B_BYTES = (BN / 2) * GEMM_BK * 2;   // this CTA's half of the B tile
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 6 : 8;
  static constexpr int BAR_BYTES = 256;
  static constexpr int TOTAL = 1024 + STAGES * STAGE_BYTES + BAR_BYTES;
};
constexpr int GEMM2_BM = 256;  // rows per cluster tile

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tiled load into this CTA's shared memory whose byte count is reported to a barrier of the pair's
// leader (`bar_cluster` is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const CUtensorMap* m, int x, int y,
                                                 uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// fp8 (e4m3 / e5m2) operands: kind::f8f6f4, K = 32 per instruction.
__device__ __forceinline__ void umma_f8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` (same offset) in both CTAs of the pair once every MMA issued so far has finished.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(mask)
               : "memory");
}

// Launch with cluster dimension (2,1,1), 192 threads, Gemm2Smem<BN>::TOTAL (+ epilogue extras)
// bytes of dynamic shared memory and an even grid. shape.tiles_m counts 256-row tiles here.
// The gate and the epilogue hooks (tile_begin / tile_end) are called with the index of this CTA's
// 128-row tile (2 * pair tile + rank in the pair), so gates and epilogues written for the one-CTA
// mainloop work unchanged. shape.cta_first / num_ctas (both even) restrict the GEMM to a part of
// the grid.
// FP8: both operands are 1-byte e4m3, K-major only; a k-block is then 128 elements (the same 128
// bytes per row, so stages, swizzle and descriptors do not change) and one MMA covers K = 32.
template <int BN, bool A_MN, bool B_MN, class Epilogue, class LoadGate, bool FP8 = false>
__device__ __forceinline__ void gemm_mainloop_2cta(const CUtensorMap* tmA, const CUtensorMap* tmB, GemmShape shape,
                                                   Epilogue& epi, LoadGate& gate, int* err_word, uint8_t* smem_raw) {
  using S = Gemm2Smem<BN>;
  static_assert(BN == 128 || BN == 256, "cluster tile is 256 x 128 or 256 x 256");
  static_assert(!FP8 || (!A_MN && !B_MN), "fp8 operands are K-major");
  constexpr int BK_ELEMS = FP8 ? 2 * GEMM_BK : GEMM_BK;   // elements per 128-byte row of a stage
  constexpr int HALF_N = BN / 2;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();   // 0 = leader
  const bool leader = rank == 0;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + S::STAGES * S::STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (S::STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * S::STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * S::STAGES + 2 + b); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * S::STAGES + 4);
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(smem_raw + (bar_base - smem_u32(smem_raw)) + 8u * (2 * S::STAGES + 4) + 8);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 8);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(tmA);
    tma_prefetch_desc(tmB);
  }
  constexpr uint32_t TMEM_COLS = 2 * BN;
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int num_tiles = shape.tiles_m * shape.tiles_n;
  const int num_kb = (shape.K + BK_ELEMS - 1) / BK_ELEMS;
  const int pair_id = (static_cast<int>(blockIdx.x) - shape.cta_first) >> 1;
  const int pair_stride = (shape.num_ctas > 0 ? shape.num_ctas : static_cast<int>(gridDim.x)) >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one_sync()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += pair_stride) {
        int tm, tn;
        tile_coords(shape, tile, tm, tn);
        const int row0 = tm * GEMM2_BM + static_cast<int>(rank) * 128;   // this CTA's rows of A
        const int col0 = tn * BN + static_cast<int>(rank) * HALF_N;   // this CTA's half of B
        if (!gate.wait_tile(2 * tm + static_cast<int>(rank), tn, abort_flag, err_word)) break;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1, abort_flag, err_word, DEV_ERR_EMPTY_BAR_TIMEOUT,
                                 GEMM_WAIT_LIMIT_NS)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * S::STAGE_BYTES;
          const uint32_t b_dst = a_dst + S::A_BYTES;
          const uint32_t bar = map_to_cta(full_bar(stage), 0);
          if (leader) mbar_expect_tx(full_bar(stage), 2 * S::STAGE_BYTES);  // both CTAs' bytes
          if constexpr (!A_MN) {
            tma_load_2d_pair(a_dst, tmA, kb * BK_ELEMS, row0, bar);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_2d_pair(a_dst + j * 8192, tmA, row0 + j * 64, kb * GEMM_BK, bar);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(b_dst, tmB, kb * BK_ELEMS, col0, bar);
          } else {
#pragma unroll
            for (int j = 0; j < HALF_N / 64; ++j) tma_load_2d_pair(b_dst + j * 8192, tmB, col0 + j * 64, kb * GEMM_BK, bar);
          }
          if (++stage == S::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && elect_one_sync()) {
      // operand format field: 1 = bf16 for kind::f16, 0 = e4m3 for kind::f8f6f4
      constexpr uint32_t idesc = make_instr_desc(FP8 ? 0 : 1, FP8 ? 0 : 1, GEMM2_BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc_buf = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += pair_stride) {
        if (!mbar_wait_bounded(tempty_bar(acc_buf), acc_phase ^ 1, abort_flag, err_word, DEV_ERR_TMEM_EMPTY_TIMEOUT,
                               GEMM_WAIT_LIMIT_NS))
          break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc_buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(full_bar(stage), phase, abort_flag, err_word, DEV_ERR_FULL_BAR_TIMEOUT,
                                 GEMM_WAIT_LIMIT_NS)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_src = smem_base + stage * S::STAGE_BYTES;
          const uint32_t b_src = a_src + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(a_src + k * 2048, 8192, 1024)
                                        : make_smem_desc_sw128(a_src + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(b_src + k * 2048, 8192, 1024)
                                        : make_smem_desc_sw128(b_src + k * 32, 16, 1024);
            if constexpr (FP8)
              umma_f8_pair(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            else
              umma_f16_pair(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(stage));  // frees the stage in both CTAs once these MMAs have read it
          if (++stage == S::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit_pair(tfull_bar(acc_buf));  // accumulator complete -> both epilogues
        acc_buf ^= 1;
        if (acc_buf == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quarter = warp & 3;
    int acc_buf = 0;
    uint32_t acc_phase = 0;
    for (int tile = pair_id; tile < num_tiles; tile += pair_stride) {
      int tm, tn;
      tile_coords(shape, tile, tm, tn);
      if (!mbar_wait_bounded(tfull_bar(acc_buf), acc_phase, abort_flag, err_word, DEV_ERR_TMEM_FULL_TIMEOUT,
                             GEMM_WAIT_LIMIT_NS))
        break;
      tc_fence_after();
      epi.tile_begin(2 * tm + static_cast<int>(rank), tn);
      const int row = tm * GEMM2_BM + static_cast<int>(rank) * 128 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc_buf * BN;
      if constexpr (Epilogue::kPair) {
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t acc0[32], acc1[32];
          tmem_ld_32x32(taddr + c * 64, acc0);
          tmem_ld_32x32(taddr + c * 64 + 32, acc1);
          tmem_ld_wait();
          epi(row, tn * BN + c * 64, acc0, acc1, shape);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t acc[32];
          tmem_ld_32x32(taddr + c * 32, acc);
          tmem_ld_wait();
          epi(row, tn * BN + c * 32, acc, shape);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(map_to_cta(tempty_bar(acc_buf), 0));
      epi.tile_end(2 * tm + static_cast<int>(rank), tn);
      acc_buf ^= 1;
      if (acc_buf == 0) acc_phase ^= 1;
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // Give copies that may still be in flight time to land before shared memory is released.
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  cluster_sync_all();   // neither CTA leaves while the other may still signal its barriers or read its tiles
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace b200
