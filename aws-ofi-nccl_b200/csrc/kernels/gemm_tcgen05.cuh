// Persistent warp-specialised bf16 GEMM mainloop for sm_100a: TMA -> shared memory -> tcgen05.mma
// with the accumulator in TMEM, double-buffered so the epilogue of tile i overlaps the MMAs of
// tile i+1. The epilogue is a functor, so the same mainloop serves the plain GEMM, the fused
// SwiGLU GEMM and the GEMMs that push their tiles to peer GPUs.
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (+ TMEM owner),
// warps 2..5 = epilogue (each reads the TMEM lane quarter `warp_id % 4`).
#pragma once
#include "sm100_common.cuh"

namespace b200 {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int GEMM_THREADS = 192;
constexpr uint64_t GEMM_WAIT_LIMIT_NS = 2000000000ull;  // 2 s per wait, then the kernel gives up

template <int BN>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int BAR_BYTES = 256;
  static constexpr int TOTAL = 1024 + STAGES * STAGE_BYTES + BAR_BYTES;
};

struct GemmShape {
  int M, N, K;
  int tiles_m, tiles_n;
  // Fused kernels run the GEMM on a subset of the grid and may want a rotated M order:
  int cta_first = 0;   // first CTA (blockIdx.x) that takes part in the GEMM
  int num_ctas = 0;    // number of GEMM CTAs (0 = the whole grid)
  int m_rot = 0;       // tile_m = (raw + m_rot) % tiles_m
  int m_major = 0;     // 1: walk all N tiles of an M tile before the next M tile
  int n_rot = 0;       // tile_n = (raw + n_rot) % tiles_n
  int group_m = 0;     // default order only: M tiles are walked in groups of this many (0 = all)
};

// The tile id -> (tile_m, tile_n) map. Default: M fastest inside a group of group_m M tiles, so
// the CTAs that run together cover a roughly square patch of C and share both their A and their B
// tiles in L2. m_major: N fastest, so that M tiles finish (or are needed) one after another.
__device__ __forceinline__ void tile_coords(const GemmShape& s, int tile, int& tm, int& tn) {
  int raw_m;
  if (s.m_major) {
    raw_m = tile / s.tiles_n;
    tn = tile % s.tiles_n;
  } else if (s.group_m > 0 && s.group_m < s.tiles_m) {
    const int per_group = s.group_m * s.tiles_n;
    const int g = tile / per_group;
    const int first_m = g * s.group_m;
    const int gsize = min(s.group_m, s.tiles_m - first_m);
    const int in = tile - g * per_group;
    tn = in / gsize;
    raw_m = first_m + (in - tn * gsize);
  } else {
    raw_m = tile % s.tiles_m;
    tn = tile / s.tiles_m;
  }
  tm = raw_m + s.m_rot;
  if (tm >= s.tiles_m) tm -= s.tiles_m;
  tn += s.n_rot;
  if (tn >= s.tiles_n) tn -= s.tiles_n;
}

// Epilogue functor contract:
//   __device__ void operator()(int row, int col0, const uint32_t (&acc)[32], const GemmShape&)
// called by one thread per accumulator row for 32 consecutive columns starting at col0 (fp32 bits).
// Optional hooks: tile_begin(tm, tn) / tile_end(tm, tn) called by every epilogue thread.

template <int BN, bool A_MN, bool B_MN, class Epilogue, class LoadGate>
__device__ __forceinline__ void gemm_mainloop(const CUtensorMap* tmA, const CUtensorMap* tmB, GemmShape shape,
                                              Epilogue& epi, LoadGate& gate, int* err_word, uint8_t* smem_raw) {
  using S = GemmSmem<BN>;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // 1024-byte aligned tile area (required by the 128-byte swizzle).
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
      mbar_init(tempty_bar(b), 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(tmA);
    tma_prefetch_desc(tmB);
  }
  constexpr uint32_t TMEM_COLS = 2 * BN;  // 256 or 512: a power of two >= 32
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int num_tiles = shape.tiles_m * shape.tiles_n;
  const int num_kb = (shape.K + GEMM_BK - 1) / GEMM_BK;
  const int cta_id = static_cast<int>(blockIdx.x) - shape.cta_first;
  const int cta_stride = shape.num_ctas > 0 ? shape.num_ctas : static_cast<int>(gridDim.x);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one_sync()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cta_id; tile < num_tiles && ok; tile += cta_stride) {
        int tm, tn;
        tile_coords(shape, tile, tm, tn);
        if (!gate.wait_tile(tm, tn, abort_flag, err_word)) break;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1, abort_flag, err_word, DEV_ERR_EMPTY_BAR_TIMEOUT,
                                 GEMM_WAIT_LIMIT_NS)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * S::STAGE_BYTES;
          const uint32_t b_dst = a_dst + S::A_BYTES;
          mbar_expect_tx(full_bar(stage), S::STAGE_BYTES);
          if constexpr (!A_MN) {
            tma_load_2d(a_dst, tmA, kb * GEMM_BK, tm * GEMM_BM, full_bar(stage));
          } else {
#pragma unroll
            for (int j = 0; j < GEMM_BM / 64; ++j)
              tma_load_2d(a_dst + j * 8192, tmA, tm * GEMM_BM + j * 64, kb * GEMM_BK, full_bar(stage));
          }
          if constexpr (!B_MN) {
            tma_load_2d(b_dst, tmB, kb * GEMM_BK, tn * BN, full_bar(stage));
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_dst + j * 8192, tmB, tn * BN + j * 64, kb * GEMM_BK, full_bar(stage));
          }
          if (++stage == S::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one_sync()) {
      constexpr uint32_t idesc = make_instr_desc(1, 1, GEMM_BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc_buf = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cta_id; tile < num_tiles && ok; tile += cta_stride) {
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
            umma_f16(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
          if (++stage == S::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(tfull_bar(acc_buf));  // accumulator complete -> epilogue
        acc_buf ^= 1;
        if (acc_buf == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;
    int acc_buf = 0;
    uint32_t acc_phase = 0;
    for (int tile = cta_id; tile < num_tiles; tile += cta_stride) {
      int tm, tn;
      tile_coords(shape, tile, tm, tn);
      if (!mbar_wait_bounded(tfull_bar(acc_buf), acc_phase, abort_flag, err_word, DEV_ERR_TMEM_FULL_TIMEOUT,
                             GEMM_WAIT_LIMIT_NS))
        break;
      tc_fence_after();
      epi.tile_begin(tm, tn);
      const int row = tm * GEMM_BM + quarter * 32 + lane;
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
      if (lane == 0) mbar_arrive(tempty_bar(acc_buf));
      epi.tile_end(tm, tn);
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
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Gate that never waits (all operand rows are local and ready).
struct NoGate {
  __device__ __forceinline__ bool wait_tile(int, int, volatile int*, int*) { return true; }
};

}  // namespace b200
