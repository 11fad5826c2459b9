// Tensor-parallel GEMMs fused with their collectives, each as ONE kernel:
//
//  ag_gemm  : all-gather(A over ranks, along M or B along N) -> tcgen05 GEMM (-> SwiGLU). A few
//             "mover" CTAs pull the peers' shards over NVLink into this GPU's copy of the
//             gathered operand and publish one flag per 128-row chunk; the GEMM CTAs walk the tiles
//             in the order the chunks arrive (own shard first) and their TMA producer waits on the
//             flag of the chunk it is about to load. Remote data crosses NVLink exactly once and
//             is always TMA-loaded from local memory.
//  gemm_rs  : tcgen05 GEMM -> reduce-scatter as a ring inside the epilogue: every finished tile is
//             added to the running sum received from the next rank and stored straight into the
//             previous rank's staging slot (peer stores + a release-ordered flag); the last hop
//             writes the result. All SMs run the GEMM, the traffic is spread over the whole
//             kernel, and no GPU's NVLink ingress is hit by everyone at once.
//
// Every wait is bounded (status word + early exit), none of the loads uses cluster multicast.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "gemm_epilogues.cuh"
#include "gemm_tcgen05.cuh"
#include "gemm_tcgen05_2cta.cuh"
#include "gin_device.cuh"
#include "host_util.h"

namespace b200 {

const GinDevHandle* comm_handle(int id);  // collectives.cu

// Scratch words inside the control pad used by these kernels (u32 each).
// Every flag holds the number of the call (per communicator, counted on the host) that last set
// it, so nothing is ever reset and calls of different shapes can follow one another.
constexpr size_t TP_READY_OFF = GIN_PAD_SCRATCH_OFF;                    // [4096] chunk-ready flags (ag_gemm)
constexpr size_t TP_ARRIVED_OFF = GIN_PAD_SCRATCH_OFF + 4096 * 4;       // [ring step][tile of a shard] arrival flags (gemm_rs)
constexpr int TP_MAX_CHUNKS = 4096;
constexpr int TP_MAX_TILES = 16384;
static_assert(TP_ARRIVED_OFF + size_t(TP_MAX_TILES) * GIN_MAX_RANKS * 4 <= GIN_PAD_BYTES, "pad too small");

__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// ------------------------------------------------------------------------------------------ ag_gemm
// Gate on the gathered operand: chunk index = tile index along the gathered dimension.
struct ChunkGate {
  const uint32_t* ready;   // local flags
  uint32_t target;         // value a flag reaches when its chunk has landed in this call
  int chunks_per_shard;
  int my_shard;
  int on_b;                // 0: A rows are gathered (gate on tm), 1: B rows are gathered (gate on tn)
  uint64_t limit_ns;
  __device__ __forceinline__ bool wait_tile(int tm, int tn, volatile int* abort_flag, int* err_word) {
    const int chunk = on_b ? tn : tm;
    if (chunk / chunks_per_shard == my_shard) return true;
    const uint32_t* f = ready + chunk;
    if (static_cast<int32_t>(ld_acquire_gpu_u32(f) - target) >= 0) {
      fence_proxy_async_global();
      return true;
    }
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t spins = 1;; ++spins) {
      if (static_cast<int32_t>(ld_acquire_gpu_u32(f) - target) >= 0) {
        fence_proxy_async_global();  // the chunk was written with ordinary stores; TMA reads it next
        return true;
      }
      if ((spins & 0xFF) == 0) {
        if (*abort_flag) return false;
        if (globaltimer_ns() - t0 > limit_ns) {
          *abort_flag = 1;
          if (err_word) atomicCAS(err_word, 0, DEV_ERR_SIGNAL_TIMEOUT);
          return false;
        }
      }
    }
  }
};

struct AgGemmArgs {
  GinDevHandle h;
  size_t gathered_off;      // byte offset of the gathered operand inside the window
  size_t shard_bytes;       // bytes of one rank's shard (contiguous rows)
  size_t chunk_bytes;       // bytes of one gate chunk (tile rows x row bytes)
  int chunks_per_shard;
  int n_movers;
  int channel;
  uint32_t epoch;
};

// Untiled bulk copies (no multicast): global -> shared with an mbarrier, shared -> global in a bulk group.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
               : "memory");
}

constexpr uint32_t MOVER_PIECE = 32768;
constexpr int MOVER_STAGES = 5;   // 160 KiB of the CTA's shared memory; four loads in flight
static_assert(MOVER_STAGES * MOVER_PIECE + 1024 + 64 <= GemmSmem<256>::TOTAL, "mover buffers exceed the kernel's smem");

// Mover CTAs: fetch the peers' shards, nearest rank first, chunk by chunk. One thread drives the
// copy engine: pieces of 32 KiB travel peer memory -> shared memory -> this GPU's copy of the
// gathered operand, several loads in flight, and the chunk's flag is published once its last
// store has completed.
__device__ __forceinline__ void ag_mover(const AgGemmArgs& a, uint8_t* smem_raw) {
  const GinDevHandle& h = a.h;
  if (!gin_barrier(h, a.channel, blockIdx.x)) return;  // every rank's shard is in place
  if (threadIdx.x == 0 && h.nranks > 1) {
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + MOVER_STAGES * MOVER_PIECE;
    for (int s = 0; s < MOVER_STAGES; ++s) mbar_init(bars + 8u * s, 1);
    fence_barrier_init();
    uint32_t* ready = reinterpret_cast<uint32_t*>(h.pad[h.rank] + TP_READY_OFF);
    const uint32_t pieces_per_chunk = static_cast<uint32_t>((a.chunk_bytes + MOVER_PIECE - 1) / MOVER_PIECE);
    const int my_chunks = (a.chunks_per_shard - static_cast<int>(blockIdx.x) + a.n_movers - 1) / a.n_movers;
    const uint32_t total = static_cast<uint32_t>(h.nranks - 1) * my_chunks * pieces_per_chunk;
    // piece index -> (peer, chunk, offset in chunk, bytes)
    auto locate = [&](uint32_t i, int& peer, int& chunk, size_t& off, uint32_t& bytes) {
      const uint32_t pc = i / pieces_per_chunk, pi = i - pc * pieces_per_chunk;
      const int s = 1 + static_cast<int>(pc) / my_chunks;
      peer = (h.rank + s) % h.nranks;
      chunk = static_cast<int>(blockIdx.x) + (static_cast<int>(pc) % my_chunks) * a.n_movers;
      const size_t in_chunk = static_cast<size_t>(pi) * MOVER_PIECE;
      off = a.gathered_off + peer * a.shard_bytes + chunk * a.chunk_bytes + in_chunk;
      const size_t left = a.chunk_bytes - in_chunk;
      bytes = left < MOVER_PIECE ? static_cast<uint32_t>(left) : MOVER_PIECE;
    };
    auto issue = [&](uint32_t i) {
      int peer, chunk;
      size_t off;
      uint32_t bytes;
      locate(i, peer, chunk, off, bytes);
      const uint32_t st = i % MOVER_STAGES;
      mbar_expect_tx(bars + 8u * st, bytes);
      bulk_load(base + st * MOVER_PIECE, h.window[peer] + off, bytes, bars + 8u * st);
    };
    int abort_local = 0;
    for (uint32_t i = 0; i < total && i < MOVER_STAGES - 1; ++i) issue(i);
    for (uint32_t i = 0; i < total; ++i) {
      const uint32_t st = i % MOVER_STAGES;
      if (!mbar_wait_bounded(bars + 8u * st, (i / MOVER_STAGES) & 1u, &abort_local, h.status, DEV_ERR_SIGNAL_TIMEOUT,
                             h.wait_limit_ns))
        break;
      int peer, chunk;
      size_t off;
      uint32_t bytes;
      locate(i, peer, chunk, off, bytes);
      bulk_store(h.window[h.rank] + off, base + st * MOVER_PIECE, bytes);
      tma_store_commit();
      if (i + MOVER_STAGES - 1 < total) {
        // the stage about to be refilled was read by the store issued one step ago
        tma_store_wait_read<1>();
        issue(i + MOVER_STAGES - 1);
      }
      if ((i + 1) % pieces_per_chunk == 0) {
        tma_store_wait<0>();           // the chunk is complete in this GPU's memory
        fence_proxy_async_global();
        __threadfence();
        st_release_gpu_u32(ready + peer * a.chunks_per_shard + chunk, a.epoch);
      }
    }
    tma_store_wait<0>();
  }
  gin_barrier(h, a.channel, blockIdx.x);  // nobody overwrites a shard that a peer is still reading
}

template <int BN, bool B_MN, class Epi>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    ag_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmShape shape,
                   AgGemmArgs args, Epi epi, int gate_on_b) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if (static_cast<int>(blockIdx.x) < args.n_movers) {
    ag_mover(args, smem_raw);
    return;
  }
  ChunkGate gate{reinterpret_cast<const uint32_t*>(args.h.pad[args.h.rank] + TP_READY_OFF), args.epoch,
                 args.chunks_per_shard, args.h.rank, gate_on_b, args.h.wait_limit_ns};
  gemm_mainloop<BN, false, B_MN>(&tmA, &tmB, shape, epi, gate, args.h.status, smem_raw);
}

// The same kernel on CTA pairs (256-row cluster tiles, tcgen05.mma.cta_group::2). Movers come in
// pairs too (n_movers is even), so every cluster is either two movers or two GEMM CTAs.
template <bool B_MN, class Epi>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
    ag_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmShape shape,
                        AgGemmArgs args, Epi epi, int gate_on_b) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if (static_cast<int>(blockIdx.x) < args.n_movers) {
    ag_mover(args, smem_raw);
    return;
  }
  ChunkGate gate{reinterpret_cast<const uint32_t*>(args.h.pad[args.h.rank] + TP_READY_OFF), args.epoch,
                 args.chunks_per_shard, args.h.rank, gate_on_b, args.h.wait_limit_ns};
  gemm_mainloop_2cta<256, false, B_MN>(&tmA, &tmB, shape, epi, gate, args.h.status, smem_raw);
}

// B200_TP_2CTA=0 keeps the fused kernels on single CTAs.
static bool tp_pairs_enabled() {
  static int mode = -2;
  if (mode == -2) {
    const char* e = getenv("B200_TP_2CTA");
    mode = e ? atoi(e) : 1;
  }
  return mode != 0;
}

// ------------------------------------------------------------------------------------------ gemm_rs
// Ring reduce-scatter carried by the GEMM epilogue. Rank r walks the shards r+1, r+2, ..., r
// (its own last). At step k it computes its partial tile of shard r+1+k, adds the running sum that
// rank r+1 pushed for the same tile one step earlier, and either pushes the new sum to rank r-1
// (peer stores + a release-ordered flag) or, at the last step, scales and writes the result.
// Neighbours run one step apart, so an incoming tile has normally landed long before it is
// needed; the wait on its flag is bounded all the same. The staging area is double-buffered by
// call parity, which makes the kernel free of cross-GPU barriers: a rank can run at most one call
// ahead of its ring neighbour.
struct RsArgs {
  GinDevHandle h;
  size_t staging_off;       // window offset: [parity 2][step n-1][rows_per_shard][N] bf16
  int rows_per_shard;       // M / nranks
  int tiles_per_shard_m;
  uint32_t epoch;
  __nv_bfloat16* out;       // [rows_per_shard][N] on this rank
  int64_t ld_out;
  float scale;
};

template <int BN>
struct RingEpilogue {
  static constexpr bool kPair = true;   // called with 64 consecutive columns per row
  RsArgs a;
  int N, tiles_n;
  // Shared-memory counters of epilogue warps that finished a tile, indexed by (tile sequence & 3):
  // with two accumulator buffers a warp can run at most two tiles ahead of the slowest one, so
  // four counters never mix tiles.
  unsigned int* warp_count;
  uint8_t* stage;  // 4 KiB of shared memory per epilogue warp: 32 rows x 128 B, 16-byte chunks XOR-swizzled by row
  unsigned int seq;
  int step, row_base, tile_in_shard;
  bool have_in;

  __device__ __forceinline__ size_t slot_elems() const { return static_cast<size_t>(a.rows_per_shard) * N; }
  __device__ __forceinline__ __nv_bfloat16* staging(int rank, int slot) const {
    const size_t parity_elems = static_cast<size_t>(a.h.nranks - 1) * slot_elems();
    return reinterpret_cast<__nv_bfloat16*>(a.h.window[rank] + a.staging_off) + (a.epoch & 1u) * parity_elems +
           static_cast<size_t>(slot) * slot_elems();
  }
  __device__ __forceinline__ uint32_t* flag(int rank, int slot) const {
    return reinterpret_cast<uint32_t*>(a.h.pad[rank] + TP_ARRIVED_OFF) +
           static_cast<size_t>(slot) * a.tiles_per_shard_m * tiles_n + tile_in_shard;
  }

  __device__ __forceinline__ void tile_begin(int tm, int tn) {
    const int n = a.h.nranks;
    const int shard = tm / a.tiles_per_shard_m;
    step = (shard - a.h.rank - 1 + 2 * n) % n;
    row_base = shard * a.rows_per_shard;
    tile_in_shard = (tm - shard * a.tiles_per_shard_m) * tiles_n + tn;
    have_in = false;
    if (step > 0) {
      int ok = 1;
      if ((threadIdx.x & 31) == 0) ok = gin_spin_u32_ge(a.h, flag(a.h.rank, step - 1), a.epoch, DEV_ERR_SIGNAL_TIMEOUT) ? 1 : 0;
      have_in = __shfl_sync(0xffffffffu, ok, 0) != 0;  // on a timeout the tile goes on without the missing sum
    }
  }

  __device__ __forceinline__ void operator()(int row, int col0, uint32_t (&a0)[32], uint32_t (&a1)[32], const GemmShape& s) {
    if (col0 >= s.N) return;  // uniform over the warp
    const int lane = threadIdx.x & 31;
    uint8_t* buf = stage + ((threadIdx.x >> 5) - 2) * 4096;
    const int row0 = row - lane;  // first row of this warp's 32-row slab
    const size_t slab = static_cast<size_t>(row0 - row_base) * N + col0;
    const int c = lane & 7;
    if (have_in) {
      // coalesced read of the incoming 32 x 64 slab (four full 128-byte row segments per load)
      const __nv_bfloat16* in = staging(a.h.rank, step - 1) + slab;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = 4 * i + (lane >> 3);
        const uint4 v = *reinterpret_cast<const uint4*>(in + static_cast<size_t>(r) * N + c * 8);
        *reinterpret_cast<uint4*>(buf + r * 128 + ((c ^ (r & 7)) << 4)) = v;
      }
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 v = *reinterpret_cast<const uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4));
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
        uint32_t* acc = j < 4 ? &a0[8 * j] : &a1[8 * (j - 4)];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          acc[2 * q] = __float_as_uint(__uint_as_float(acc[2 * q]) + __low2float(p[q]));
          acc[2 * q + 1] = __float_as_uint(__uint_as_float(acc[2 * q + 1]) + __high2float(p[q]));
        }
      }
      __syncwarp();
    }
    const bool last = step == a.h.nranks - 1;
    const float sc = last ? a.scale : 1.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t* acc = j < 4 ? &a0[8 * j] : &a1[8 * (j - 4)];
      const uint4 v = make_uint4(pack_bf16x2(__uint_as_float(acc[0]) * sc, __uint_as_float(acc[1]) * sc),
                                 pack_bf16x2(__uint_as_float(acc[2]) * sc, __uint_as_float(acc[3]) * sc),
                                 pack_bf16x2(__uint_as_float(acc[4]) * sc, __uint_as_float(acc[5]) * sc),
                                 pack_bf16x2(__uint_as_float(acc[6]) * sc, __uint_as_float(acc[7]) * sc));
      *reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
    }
    __syncwarp();
    __nv_bfloat16* dst;
    int64_t ld;
    if (last) {
      dst = a.out + static_cast<int64_t>(row0 - row_base) * a.ld_out + col0;
      ld = a.ld_out;
    } else {
      const int prev = (a.h.rank + a.h.nranks - 1) % a.h.nranks;
      dst = staging(prev, step) + slab;
      ld = N;
    }
    // every store instruction writes four complete 128-byte row segments
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = 4 * i + (lane >> 3);
      const uint4 v = *reinterpret_cast<const uint4*>(buf + r * 128 + ((c ^ (r & 7)) << 4));
      *reinterpret_cast<uint4*>(dst + static_cast<int64_t>(r) * ld + c * 8) = v;
    }
    __syncwarp();
  }

  // Called by every epilogue thread. The warp that arrives last (no warp ever waits for another,
  // so a warp that gave up on a timeout cannot block the rest) tells the previous rank that the
  // running sum of this tile is complete in its staging slot.
  __device__ __forceinline__ void tile_end(int, int) {
    __syncwarp();
    if (step != a.h.nranks - 1 && (threadIdx.x & 31) == 0) {
      fence_acq_rel_sys();  // this warp's peer stores are performed before the count moves
      const unsigned int prev_count = atomicAdd(warp_count + (seq & 3u), 1u);
      if ((prev_count & 3u) == 3u) {
        const int prev = (a.h.rank + a.h.nranks - 1) % a.h.nranks;
        st_release_sys_u32(flag(prev, step), a.epoch);
      }
    }
    ++seq;
  }
};

template <int BN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_rs_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmShape shape,
                   RsArgs args) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ unsigned int epi_warp_count[4];
  if (threadIdx.x < 4) epi_warp_count[threadIdx.x] = 0;
  __syncthreads();
  RingEpilogue<BN> epi{args, shape.N, shape.tiles_n, epi_warp_count, smem_raw + GemmSmem<BN>::TOTAL, 0, 0, 0, 0, false};
  NoGate gate;
  gemm_mainloop<BN, false, B_MN>(&tmA, &tmB, shape, epi, gate, args.h.status, smem_raw);
}

template <bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
    gemm_rs_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmShape shape,
                        RsArgs args) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ unsigned int epi_warp_count[4];
  if (threadIdx.x < 4) epi_warp_count[threadIdx.x] = 0;
  __syncthreads();
  RingEpilogue<256> epi{args, shape.N, shape.tiles_n, epi_warp_count, smem_raw + Gemm2Smem<256>::TOTAL, 0, 0, 0, 0, false};
  NoGate gate;
  gemm_mainloop_2cta<256, false, B_MN>(&tmA, &tmB, shape, epi, gate, args.h.status, smem_raw);
}

// per-communicator call counters (flags and counters only ever grow; the expected value is
// derived from the number of calls made so far)
static uint32_t g_ag_epoch[64] = {0};
static uint32_t g_rs_epoch[64] = {0};

template <typename K>
static int set_smem(K kern, int bytes) {
  return static_cast<int>(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
}

}  // namespace b200

extern "C" {
using namespace b200;

// C[M,N] = gather(A)[M,K] * B^T, A gathered along M from all ranks' shards (rows rank*M/n ...),
// which live at `gathered_off` in every rank's window (own shard already in place); the local
// operand B is passed in `other`.
//   b_mn     : B stored [K][N] instead of [N][K]
//   epilogue : 0 = store C (bf16, ldc), 1 = SwiGLU on interleaved gate|up columns -> act [M][N/2]
//              (ld_act), also storing the raw gate|up into C when C is non-null
// M must be a multiple of 128 * nranks.
// gather_b = 1 gathers B instead (FSDP: the weight [N][K] is sharded over ranks along N, the
// activation A [M][K] is local and passed in `other`); then N must be a multiple of 256 * nranks
// and b_mn must be 0.
int b200_ag_gemm(int comm, size_t gathered_off, int gather_b, int M, int N, int K, const void* other, long long ld_other,
                 int b_mn, void* C, long long ldc, void* act, long long ld_act, int epilogue, int n_movers, int channel,
                 void* stream) {
  ensure_context();
  const GinDevHandle* hp = comm_handle(comm);
  if (!hp || comm < 0 || comm >= 64 || !other) return B200_ERR_BAD_ARG;
  GinDevHandle h = *hp;
  constexpr int BN = 256;
  if (K % 8 || N % 64 || (epilogue == 1 && !act) || (epilogue == 0 && !C)) return B200_ERR_BAD_ARG;
  if (!gather_b && M % (GEMM_BM * h.nranks)) return B200_ERR_BAD_ARG;
  if (gather_b && (N % (BN * h.nranks) || b_mn)) return B200_ERR_BAD_ARG;
  const size_t shard_bytes = static_cast<size_t>((gather_b ? N : M) / h.nranks) * K * 2;
  if (gathered_off % 1024 || gathered_off + shard_bytes * h.nranks > h.window_bytes) return B200_ERR_BAD_ARG;
  GemmShape shape{M, N, K, (M + GEMM_BM - 1) / GEMM_BM, (N + BN - 1) / BN};
  const int chunks_total = gather_b ? shape.tiles_n : shape.tiles_m;
  const int chunks_per_shard = chunks_total / h.nranks;
  if (chunks_total > TP_MAX_CHUNKS) return B200_ERR_TOO_LARGE;
  if (n_movers <= 0) n_movers = 16;
  if (n_movers > chunks_per_shard) n_movers = chunks_per_shard;
  const int sms = sm_count();
  shape.cta_first = n_movers;
  shape.num_ctas = sms - n_movers;
  if (shape.num_ctas > shape.tiles_m * shape.tiles_n) shape.num_ctas = shape.tiles_m * shape.tiles_n;
  // own shard first, then rank+1, rank+2, ... along the gathered dimension
  if (gather_b) {
    shape.n_rot = h.rank * chunks_per_shard;
    shape.m_major = 0;
  } else {
    // groups of M tiles that never straddle a shard, M fastest inside a group: the CTAs of a wave
    // share their weight tiles in L2 and still consume the shards in arrival order
    shape.m_rot = h.rank * chunks_per_shard;
    int gm = chunks_per_shard < 16 ? chunks_per_shard : 16;
    while (chunks_per_shard % gm) --gm;
    shape.group_m = gm;
    if (gm >= shape.tiles_m) shape.m_major = 1;  // a single group: walk the N tiles of each M tile instead
  }
  // CTA pairs when every 256-row (A gathered) cluster tile lies inside one shard and the B tile is full width
  const bool pairs = tp_pairs_enabled() && M >= 256 && N >= 256 && (gather_b || chunks_per_shard % 2 == 0) && sms >= 4;
  if (pairs) {
    n_movers = (n_movers + 1) & ~1;
    shape.tiles_m = (M + GEMM2_BM - 1) / GEMM2_BM;
    shape.cta_first = n_movers;
    shape.num_ctas = (sms - n_movers) & ~1;
    if (shape.num_ctas > 2 * shape.tiles_m * shape.tiles_n) shape.num_ctas = 2 * shape.tiles_m * shape.tiles_n;
    if (gather_b) {
      shape.n_rot = h.rank * chunks_per_shard;
      shape.m_major = 0;
      shape.group_m = 0;
    } else {
      const int cps2 = chunks_per_shard / 2;   // 256-row tiles per shard
      shape.m_rot = h.rank * cps2;
      int gm = cps2 < 8 ? cps2 : 8;
      while (cps2 % gm) --gm;
      shape.group_m = gm;
      shape.m_major = gm >= shape.tiles_m ? 1 : 0;
    }
  }
  CUtensorMap tmA, tmB;
  int rc;
  const void* gathered = h.window[h.rank] + gathered_off;
  const int b_box_rows = pairs ? BN / 2 : BN;
  if (gather_b) {
    rc = make_tmap_2d(&tmA, other, M, K, ld_other, GEMM_BM, GEMM_BK, 2, true);
    if (rc) return rc;
    rc = make_tmap_2d(&tmB, gathered, N, K, K, b_box_rows, GEMM_BK, 2, true);
  } else {
    rc = make_tmap_2d(&tmA, gathered, M, K, K, GEMM_BM, GEMM_BK, 2, true);
    if (rc) return rc;
    rc = b_mn ? make_tmap_2d(&tmB, other, K, N, ld_other, GEMM_BK, 64, 2, true)
              : make_tmap_2d(&tmB, other, N, K, ld_other, b_box_rows, GEMM_BK, 2, true);
  }
  if (rc) return rc;
  AgGemmArgs args{h, gathered_off, shard_bytes, static_cast<size_t>(gather_b ? BN : GEMM_BM) * K * 2, chunks_per_shard,
                  n_movers, channel, ++g_ag_epoch[comm]};
  const int grid = n_movers + shape.num_ctas;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int smem = pairs ? Gemm2Smem<BN>::TOTAL : GemmSmem<BN>::TOTAL;
#define B200_AG_LAUNCH(KERNEL, EPI)                                             \
  do {                                                                          \
    auto k = KERNEL;                                                            \
    if (set_smem(k, smem)) return B200_ERR_BAD_ARG;                             \
    k<<<grid, GEMM_THREADS, smem, s>>>(tmA, tmB, shape, args, EPI, gather_b);   \
  } while (0)
  if (epilogue == 1) {
    SwiGluEpilogue epi{static_cast<__nv_bfloat16*>(act), ld_act, static_cast<__nv_bfloat16*>(C), ldc};
    if (pairs) {
      if (b_mn) B200_AG_LAUNCH((ag_gemm_pair_kernel<true, SwiGluEpilogue>), epi);
      else B200_AG_LAUNCH((ag_gemm_pair_kernel<false, SwiGluEpilogue>), epi);
    } else {
      if (b_mn) B200_AG_LAUNCH((ag_gemm_kernel<BN, true, SwiGluEpilogue>), epi);
      else B200_AG_LAUNCH((ag_gemm_kernel<BN, false, SwiGluEpilogue>), epi);
    }
  } else {
    StoreEpilogue<__nv_bfloat16> epi{static_cast<__nv_bfloat16*>(C), ldc, 0};
    if (pairs) {
      if (b_mn) B200_AG_LAUNCH((ag_gemm_pair_kernel<true, StoreEpilogue<__nv_bfloat16>>), epi);
      else B200_AG_LAUNCH((ag_gemm_pair_kernel<false, StoreEpilogue<__nv_bfloat16>>), epi);
    } else {
      if (b_mn) B200_AG_LAUNCH((ag_gemm_kernel<BN, true, StoreEpilogue<__nv_bfloat16>>), epi);
      else B200_AG_LAUNCH((ag_gemm_kernel<BN, false, StoreEpilogue<__nv_bfloat16>>), epi);
    }
  }
#undef B200_AG_LAUNCH
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

// out[M/n, N] (this rank's rows) = scale * sum over ranks of (A_r[M,K] * B_r^T)[rows of this rank].
// staging_off: window offset of 2 * (nranks-1) * (M/nranks) * N bf16 of staging space on every rank
// (b200_gemm_rs_staging_bytes). The running sums are rounded to bf16 at every hop of the ring.
size_t b200_gemm_rs_staging_bytes(int nranks, int M, int N) {
  return nranks <= 1 ? 0 : 2ull * (nranks - 1) * (static_cast<size_t>(M) / nranks) * N * 2;
}

int b200_gemm_rs(int comm, const void* A, long long lda, const void* B, long long ldb, int b_mn, int M, int N, int K,
                 size_t staging_off, void* out, long long ld_out, float scale, void* stream) {
  ensure_context();
  const GinDevHandle* hp = comm_handle(comm);
  if (!hp || comm < 0 || comm >= 64) return B200_ERR_BAD_ARG;
  GinDevHandle h = *hp;
  constexpr int BN = 256;
  if (M % (GEMM_BM * h.nranks) || K % 8 || N % 64 || !A || !B || !out || ld_out % 8) return B200_ERR_BAD_ARG;
  if (staging_off % 16 || staging_off + b200_gemm_rs_staging_bytes(h.nranks, M, N) > h.window_bytes) return B200_ERR_BAD_ARG;
  GemmShape shape{M, N, K, M / GEMM_BM, (N + BN - 1) / BN};
  const int tiles_per_shard_m = shape.tiles_m / h.nranks;
  if (static_cast<size_t>(h.nranks - 1) * tiles_per_shard_m * shape.tiles_n > static_cast<size_t>(TP_MAX_TILES) * GIN_MAX_RANKS)
    return B200_ERR_TOO_LARGE;
  const int sms = sm_count();
  const bool pairs = tp_pairs_enabled() && tiles_per_shard_m % 2 == 0 && N >= 256 && sms >= 2;
  if (pairs) {
    shape.tiles_m = M / GEMM2_BM;
    shape.num_ctas = (sms & ~1) < 2 * shape.tiles_m * shape.tiles_n ? (sms & ~1) : 2 * shape.tiles_m * shape.tiles_n;
    shape.m_rot = ((h.rank + 1) % h.nranks) * (tiles_per_shard_m / 2);
  } else {
    shape.num_ctas = sms < shape.tiles_m * shape.tiles_n ? sms : shape.tiles_m * shape.tiles_n;
    shape.m_rot = ((h.rank + 1) % h.nranks) * tiles_per_shard_m;  // next rank's rows first, own rows last
  }
  shape.m_major = 1;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, M, K, lda, GEMM_BM, GEMM_BK, 2, true);
  if (rc) return rc;
  rc = b_mn ? make_tmap_2d(&tmB, B, K, N, ldb, GEMM_BK, 64, 2, true)
            : make_tmap_2d(&tmB, B, N, K, ldb, pairs ? BN / 2 : BN, GEMM_BK, 2, true);
  if (rc) return rc;
  RsArgs args{h, staging_off, M / h.nranks, tiles_per_shard_m, ++g_rs_epoch[comm], static_cast<__nv_bfloat16*>(out), ld_out,
              scale};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // + one transpose buffer per epilogue warp
  const int smem = (pairs ? Gemm2Smem<BN>::TOTAL : GemmSmem<BN>::TOTAL) + 4 * 4096;
#define B200_RS_LAUNCH(KERNEL)                                                  \
  do {                                                                          \
    auto k = KERNEL;                                                            \
    if (set_smem(k, smem)) return B200_ERR_BAD_ARG;                             \
    k<<<shape.num_ctas, GEMM_THREADS, smem, s>>>(tmA, tmB, shape, args);        \
  } while (0)
  if (pairs) {
    if (b_mn) B200_RS_LAUNCH((gemm_rs_pair_kernel<true>));
    else B200_RS_LAUNCH((gemm_rs_pair_kernel<false>));
  } else {
    if (b_mn) B200_RS_LAUNCH((gemm_rs_kernel<BN, true>));
    else B200_RS_LAUNCH((gemm_rs_kernel<BN, false>));
  }
#undef B200_RS_LAUNCH
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // extern "C"
