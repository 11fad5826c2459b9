// Expert-parallel MoE dispatch / combine, device-initiated over the GIN primitives (peer stores,
// release-ordered remote atomics, bounded waits), fused with the routing permute and the
// block-scaled fp8 (e4m3, 1x128 groups) quantisation:
//
//  moe_route    : histogram of this rank's top-k choices per expert, all ranks exchange their
//                 histograms (puts + signals), and every rank derives from the full matrix where
//                 each (source rank, expert) segment starts in the owner's receive buffer. The
//                 receive buffer therefore comes out packed expert-major with no padding and is
//                 directly usable as the row-segmented operand of the expert GEMMs.
//  moe_dispatch : one warp per token: quantise (or copy) the row once, then store it into the
//                 receive buffer of every rank that owns one of its k experts, with its scales
//                 and a 16-byte record (token, slot, weight, source rank) used on the way back.
//  moe_combine  : every expert-output row travels back to its source token's (token, slot) cell;
//                 when all ranks have delivered, the source sums its k cells, gate-weighted.
//
// The reference moves such traffic as host-proxied RDMA writes with immediate data and signal
// atomics (reference: src/rdma/gin/nccl_ofi_gin.cpp, nccl_ofi_gin_resources.cpp); here the GPU
// threads that produce the bytes also put them.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "gin_device.cuh"
#include "host_util.h"

namespace b200 {

const GinDevHandle* comm_handle(int id);  // collectives.cu

constexpr int MOE_SIG_BASE = 3072;  // GIN signal slots [3072, 3072 + 3 * 8): phase x source rank
constexpr int MOE_MAX_EXPERTS = 1024;
constexpr int MOE_THREADS = 256;

struct MoeMeta {  // one per received row
  int32_t token, slot;
  float weight;
  int32_t src_rank;
};

__device__ __forceinline__ bool moe_wait_all(const GinDevHandle& h, int phase, uint64_t epoch) {
  // threads 0..nranks-1 each wait for one source
  bool ok = true;
  if (static_cast<int>(threadIdx.x) < h.nranks)
    ok = gin_spin_u64_ge(h, gin_signal_ptr(h, h.rank, MOE_SIG_BASE + phase * GIN_MAX_RANKS + threadIdx.x), 0, epoch,
                         DEV_ERR_SIGNAL_TIMEOUT);
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// The CTA that finishes last returns true (and rearms the counter for the next launch).
__device__ __forceinline__ bool last_cta_done(unsigned int* counter) {
  __shared__ int is_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(counter, 1u);
    is_last = prev == gridDim.x - 1;
    if (is_last) *counter = 0;
    __threadfence();
  }
  __syncthreads();
  return is_last != 0;
}

// ------------------------------------------------------------------------------------------ route
struct RouteArgs {
  GinDevHandle h;
  const int32_t* topk_idx;  // [T][k]
  int T, k, E;
  size_t cnt_off;           // window: int32 [2][nranks][E] (call parity), row r written by rank r
  int32_t* cnt_local;       // [E] zero on entry, zero again on exit
  int32_t* dest_base;       // [E] out: first row, in the owner's receive buffer, of this rank's tokens for expert e
  int32_t* expert_offsets;  // [E/nranks + 1] out: row ranges of the local experts in this rank's receive buffer
  int32_t* cursor;          // [E] out: zeroed (next free position inside each of this rank's segments)
  unsigned int* done;
  uint64_t epoch;
};

__global__ void __launch_bounds__(MOE_THREADS) moe_route_kernel(RouteArgs a) {
  __shared__ int32_t hist[MOE_MAX_EXPERTS];
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int total = a.T * a.k;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int e = a.topk_idx[i];
    if (e >= 0 && e < a.E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < a.E; e += blockDim.x)
    if (hist[e]) atomicAdd(&a.cnt_local[e], hist[e]);
  if (!last_cta_done(a.done)) return;
  const GinDevHandle& h = a.h;
  // publish this rank's histogram in everybody's matrix, then signal
  for (int p = 0; p < h.nranks; ++p) {
    int32_t* row = reinterpret_cast<int32_t*>(h.window[p] + a.cnt_off) + ((a.epoch & 1) * h.nranks + h.rank) * a.E;
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) row[e] = a.cnt_local[e];
  }
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < h.nranks)
    gin_signal(h, threadIdx.x, MOE_SIG_BASE + 0 * GIN_MAX_RANKS + h.rank, 1, GIN_SIGNAL_INC);
  const bool ok = moe_wait_all(h, 0, a.epoch);
  const int32_t* mat = reinterpret_cast<const int32_t*>(h.window[h.rank] + a.cnt_off) + (a.epoch & 1) * h.nranks * a.E;
  const int el = a.E / h.nranks;  // experts per rank
  // totals per expert, then the exclusive prefix over the experts of one owner
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) {
    int tot = 0;
    for (int s = 0; s < h.nranks; ++s) tot += ok ? mat[s * a.E + e] : 0;
    hist[e] = tot;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) {
    const int owner_first = (e / el) * el;
    int base = 0;
    for (int j = owner_first; j < e; ++j) base += hist[j];
    int before_me = 0;
    for (int s = 0; s < h.rank; ++s) before_me += ok ? mat[s * a.E + e] : 0;
    a.dest_base[e] = base + before_me;
    a.cursor[e] = 0;
    a.cnt_local[e] = 0;
    if (e / el == h.rank) {
      a.expert_offsets[e - owner_first] = base;
      if (e - owner_first == el - 1) a.expert_offsets[el] = base + hist[e];
    }
  }
}

// ------------------------------------------------------------------------------------------ dispatch
struct DispatchArgs {
  GinDevHandle h;
  const __nv_bfloat16* x;    // [T][H]
  const int32_t* topk_idx;   // [T][k]
  const float* topk_w;       // [T][k]
  int T, k, H, E;
  int fp8;                   // 1: payload e4m3 + fp32 scale per 128 elements; 0: payload bf16
  int use_saved_rows;        // 1: rows come from row_of (backward pass); 0: assigned here and saved there
  int scale_by_weight;       // 1: the row is multiplied by its gate weight before it is sent
  const int32_t* dest_base;  // [E]
  int32_t* cursor;           // [E]
  int32_t* row_of;           // [T][k] receive-buffer row of every (token, slot); -1 = dropped
  size_t recv_off, scale_off, meta_off;  // window offsets on the receiving side
  int capacity_rows;
  unsigned int* done;
  uint64_t epoch;
};

__device__ __forceinline__ float warp_half_max(float v) {  // max over each group of 16 lanes
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

constexpr int MOE_MAX_TOPK = 16;

// Eight values of one lane (16 lanes share a 128-element scale group) -> eight e4m3 bytes.
__device__ __forceinline__ uint2 quantize8(const float (&v)[8], float w, float& scale) {
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j] * w));
  amax = warp_half_max(amax);
  scale = fmaxf(amax, 1e-12f) * (1.f / 448.f);
  const float m = w / scale;
  uint2 q;
  q.x = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(v[0] * m, v[1] * m), __NV_SATFINITE, __NV_E4M3)) |
        (static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(v[2] * m, v[3] * m), __NV_SATFINITE, __NV_E4M3)) << 16);
  q.y = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(v[4] * m, v[5] * m), __NV_SATFINITE, __NV_E4M3)) |
        (static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(v[6] * m, v[7] * m), __NV_SATFINITE, __NV_E4M3)) << 16);
  return q;
}

__global__ void __launch_bounds__(MOE_THREADS) moe_dispatch_kernel(DispatchArgs a) {
  const GinDevHandle& h = a.h;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int el = a.E / h.nranks;
  const int chunks = a.H / 256;      // 256 elements (two scale groups) per warp pass
  const int groups = a.H / 128;
  const size_t row_bytes = a.fp8 ? static_cast<size_t>(a.H) : static_cast<size_t>(a.H) * 2;
  __shared__ float scale_buf[MOE_THREADS / 32][64];
  for (int t = blockIdx.x * warps + warp; t < a.T; t += gridDim.x * warps) {
    // ---- where do the k copies go
    int my_rank = -1, my_row = -1;   // lane s (< k) holds the destination of slot s
    float my_w = 0.f;
    if (lane < a.k) {
      const int e = a.topk_idx[t * a.k + lane];
      my_w = a.topk_w ? a.topk_w[t * a.k + lane] : 1.f;
      if (e >= 0 && e < a.E) {
        my_rank = e / el;
        if (a.use_saved_rows) {
          my_row = a.row_of[t * a.k + lane];
        } else {
          my_row = a.dest_base[e] + atomicAdd(&a.cursor[e], 1);
          if (my_row >= a.capacity_rows) {
            gin_record_error(h, DEV_ERR_CAPACITY);
            my_row = -1;
          }
          a.row_of[t * a.k + lane] = my_row;
        }
        if (my_row >= 0) {
          MoeMeta m{t, lane, my_w, h.rank};
          *reinterpret_cast<int4*>(h.window[my_rank] + a.meta_off + static_cast<size_t>(my_row) * sizeof(MoeMeta)) =
              *reinterpret_cast<const int4*>(&m);
        }
      } else if (!a.use_saved_rows) {
        a.row_of[t * a.k + lane] = -1;
      }
    }
    // ---- the row itself, 256 elements (two scale groups) per pass; an unweighted row is
    // quantised once and stored k times, a weighted one is scaled and quantised per slot
    const uint4* src = reinterpret_cast<const uint4*>(a.x + static_cast<size_t>(t) * a.H);
    const bool weighted = a.scale_by_weight != 0;
    for (int c = 0; c < chunks; ++c) {
      const uint4 raw = src[c * 32 + lane];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
      float v[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[2 * j] = __low2float(p[j]);
        v[2 * j + 1] = __high2float(p[j]);
      }
      uint2 q = make_uint2(0, 0);
      float scale = 1.f;
      if (a.fp8 && !weighted) {
        q = quantize8(v, 1.f, scale);
        if ((lane & 15) == 0) scale_buf[warp][2 * c + (lane >> 4)] = scale;
      }
      for (int s = 0; s < a.k; ++s) {
        const int drank = __shfl_sync(0xffffffffu, my_rank, s);
        const int drow = __shfl_sync(0xffffffffu, my_row, s);
        const float w = __shfl_sync(0xffffffffu, my_w, s);
        if (drow < 0) continue;  // uniform over the warp
        uint8_t* dst = h.window[drank] + a.recv_off + static_cast<size_t>(drow) * row_bytes;
        if (a.fp8) {
          if (weighted) {
            q = quantize8(v, w, scale);
            if ((lane & 15) == 0)
              reinterpret_cast<float*>(h.window[drank] + a.scale_off)[static_cast<size_t>(drow) * groups + 2 * c + (lane >> 4)] = scale;
          }
          reinterpret_cast<uint2*>(dst)[c * 32 + lane] = q;
        } else if (!weighted) {
          reinterpret_cast<uint4*>(dst)[c * 32 + lane] = raw;
        } else {
          __nv_bfloat162 r[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) r[j] = __floats2bfloat162_rn(v[2 * j] * w, v[2 * j + 1] * w);
          reinterpret_cast<uint4*>(dst)[c * 32 + lane] = *reinterpret_cast<const uint4*>(r);
        }
      }
    }
    if (a.fp8 && !weighted) {
      __syncwarp();
      for (int s = 0; s < a.k; ++s) {
        const int drank = __shfl_sync(0xffffffffu, my_rank, s);
        const int drow = __shfl_sync(0xffffffffu, my_row, s);
        if (drow < 0) continue;
        float* sd = reinterpret_cast<float*>(h.window[drank] + a.scale_off) + static_cast<size_t>(drow) * groups;
        for (int g = lane; g < groups; g += 32) sd[g] = scale_buf[warp][g];
      }
      __syncwarp();
    }
  }
  if (!last_cta_done(a.done)) return;
  // every row of this rank is on its way: tell all ranks, then wait until everybody's rows are here
  if (static_cast<int>(threadIdx.x) < h.nranks) {
    fence_acq_rel_sys();
    gin_signal(h, threadIdx.x, MOE_SIG_BASE + 1 * GIN_MAX_RANKS + h.rank, 1, GIN_SIGNAL_INC);
  }
  moe_wait_all(h, 1, a.epoch);
}

// ------------------------------------------------------------------------------------------ combine
struct CombineArgs {
  GinDevHandle h;
  const __nv_bfloat16* y;          // [rows][H] expert outputs in receive-buffer row order
  const int32_t* expert_offsets;   // [E/nranks + 1]; the last entry is the number of rows
  int experts_local;
  size_t meta_off, comb_off;       // window offsets: MoeMeta [rows] (local), bf16 [T][k][H] (on the source)
  const float* topk_w;             // [T][k] on the source, or null for an unweighted sum
  const int32_t* row_of;           // [T][k] on the source: cells whose row is < 0 were never sent
  int T, k, H;
  __nv_bfloat16* out;              // [T][H]
  unsigned int* done;
  uint64_t epoch;
};

__global__ void __launch_bounds__(MOE_THREADS) moe_combine_kernel(CombineArgs a) {
  const GinDevHandle& h = a.h;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int rows = a.expert_offsets[a.experts_local];
  const int vec = a.H / 8;
  const MoeMeta* meta = reinterpret_cast<const MoeMeta*>(h.window[h.rank] + a.meta_off);
  for (int r = blockIdx.x * warps + warp; r < rows; r += gridDim.x * warps) {
    const MoeMeta m = meta[r];
    if (m.src_rank < 0 || m.src_rank >= h.nranks || m.token < 0 || m.token >= a.T || m.slot < 0 || m.slot >= a.k) {
      if (lane == 0) gin_record_error(h, DEV_ERR_BOUNDS);
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(a.y + static_cast<size_t>(r) * a.H);
    uint4* dst = reinterpret_cast<uint4*>(h.window[m.src_rank] + a.comb_off) +
                 (static_cast<size_t>(m.token) * a.k + m.slot) * vec;
    constexpr int U = 4;
    for (int v0 = lane; v0 < vec; v0 += 32 * U) {
      uint4 tmp[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (v0 + 32 * u < vec) tmp[u] = src[v0 + 32 * u];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (v0 + 32 * u < vec) dst[v0 + 32 * u] = tmp[u];
    }
  }
  // ---- all of this rank's rows are out: signal every source (one CTA does it) ...
  if (last_cta_done(a.done)) {
    if (static_cast<int>(threadIdx.x) < h.nranks) {
      fence_acq_rel_sys();
      gin_signal(h, threadIdx.x, MOE_SIG_BASE + 2 * GIN_MAX_RANKS + h.rank, 1, GIN_SIGNAL_INC);
    }
  }
  // ---- ... and every CTA waits for all ranks' rows before it reduces its share of the tokens
  if (!moe_wait_all(h, 2, a.epoch)) return;
  const uint4* comb = reinterpret_cast<const uint4*>(h.window[h.rank] + a.comb_off);
  for (int t = blockIdx.x * warps + warp; t < a.T; t += gridDim.x * warps) {
    float w = 0.f;
    int live = 0;
    if (lane < a.k) {
      live = a.row_of[t * a.k + lane] >= 0;
      w = a.topk_w ? a.topk_w[t * a.k + lane] : 1.f;
    }
    for (int v0 = lane; v0 < vec; v0 += 32) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int s = 0; s < a.k; ++s) {
        const float ws = __shfl_sync(0xffffffffu, w, s);
        if (!__shfl_sync(0xffffffffu, live, s)) continue;
        const uint4 q = comb[(static_cast<size_t>(t) * a.k + s) * vec + v0];
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] += ws * __low2float(p[j]);
          acc[2 * j + 1] += ws * __high2float(p[j]);
        }
      }
      __nv_bfloat162 o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      reinterpret_cast<uint4*>(a.out + static_cast<size_t>(t) * a.H)[v0] = *reinterpret_cast<const uint4*>(o);
    }
  }
}

// d(weight)[t][s] = <d_out[t], cell[t][s]> over the combine buffer kept from the forward pass.
__global__ void __launch_bounds__(MOE_THREADS)
    moe_combine_wgrad_kernel(const __nv_bfloat16* dout, const __nv_bfloat16* comb, const int32_t* row_of, float* dw, int T,
                             int k, int H) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int vec = H / 8;
  for (int i = blockIdx.x * warps + warp; i < T * k; i += gridDim.x * warps) {
    const int t = i / k;
    float acc = 0.f;
    if (row_of[i] >= 0) {
      const uint4* a = reinterpret_cast<const uint4*>(dout + static_cast<size_t>(t) * H);
      const uint4* b = reinterpret_cast<const uint4*>(comb + static_cast<size_t>(i) * H);
      for (int v = lane; v < vec; v += 32) {
        const uint4 x = a[v], y = b[v];
        const __nv_bfloat162* px = reinterpret_cast<const __nv_bfloat162*>(&x);
        const __nv_bfloat162* py = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          acc += __low2float(px[j]) * __low2float(py[j]) + __high2float(px[j]) * __high2float(py[j]);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) dw[i] = acc;
  }
}

// fp8 (e4m3) rows with one fp32 scale per 128 elements -> bf16.
__global__ void __launch_bounds__(MOE_THREADS)
    fp8_dequant_rows_kernel(const uint8_t* q, const float* scales, __nv_bfloat16* out, const int32_t* rows_ptr, int rows_max,
                            int H) {
  const int rows = rows_ptr ? min(*rows_ptr, rows_max) : rows_max;
  const int64_t nvec = static_cast<int64_t>(rows) * H / 8;
  const int groups = H / 128;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t e0 = i * 8;
    const int64_t r = e0 / H;
    const int g = static_cast<int>((e0 - r * H) / 128);
    const float s = scales[r * groups + g];
    const uint2 raw = reinterpret_cast<const uint2*>(q)[i];
    const __nv_fp8x2_storage_t* p = reinterpret_cast<const __nv_fp8x2_storage_t*>(&raw);
    __nv_bfloat162 o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(p[j], __NV_E4M3);
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
      o[j] = __floats2bfloat162_rn(f.x * s, f.y * s);
    }
    reinterpret_cast<uint4*>(out)[i] = *reinterpret_cast<const uint4*>(o);
  }
}

static uint64_t g_moe_epoch[64][3] = {};

static int moe_grid(int work_warps) {
  const int per_cta = MOE_THREADS / 32;
  int grid = (work_warps + per_cta - 1) / per_cta;
  const int cap = sm_count() * 4;
  if (grid > cap) grid = cap;
  return grid < 1 ? 1 : grid;
}

}  // namespace b200

extern "C" {
using namespace b200;

// Collective over the communicator. `done` is a zero-initialised device word private to this call
// site; cnt_local must be zero on the first call (the kernel leaves it zero).
int b200_moe_route(int comm, const void* topk_idx, int T, int k, int E, size_t cnt_off, void* cnt_local, void* dest_base,
                   void* expert_offsets, void* cursor, void* done, void* stream) {
  ensure_context();
  const GinDevHandle* hp = comm_handle(comm);
  if (!hp || comm < 0 || comm >= 64) return B200_ERR_BAD_ARG;
  GinDevHandle h = *hp;
  if (E <= 0 || E > MOE_MAX_EXPERTS || E % h.nranks || k <= 0 || k > MOE_MAX_TOPK || T <= 0) return B200_ERR_BAD_ARG;
  if (cnt_off % 16 || cnt_off + 2ull * h.nranks * E * 4 > h.window_bytes) return B200_ERR_BAD_ARG;
  RouteArgs a{h, static_cast<const int32_t*>(topk_idx), T, k, E, cnt_off, static_cast<int32_t*>(cnt_local),
              static_cast<int32_t*>(dest_base), static_cast<int32_t*>(expert_offsets), static_cast<int32_t*>(cursor),
              static_cast<unsigned int*>(done), ++g_moe_epoch[comm][0]};
  int grid = (T * k + MOE_THREADS * 8 - 1) / (MOE_THREADS * 8);
  if (grid > 64) grid = 64;
  moe_route_kernel<<<grid, MOE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(a);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

// Collective. Window layout on every rank: payload rows at recv_off (H bytes per row for fp8, 2H
// for bf16), fp32 scales at scale_off (H/128 per row, fp8 only), 16-byte records at meta_off.
int b200_moe_dispatch(int comm, const void* x, const void* topk_idx, const void* topk_w, int T, int k, int H, int E, int fp8,
                      int use_saved_rows, int scale_by_weight, const void* dest_base, void* cursor, void* row_of,
                      size_t recv_off, size_t scale_off, size_t meta_off, int capacity_rows, void* done, void* stream) {
  ensure_context();
  const GinDevHandle* hp = comm_handle(comm);
  if (!hp || comm < 0 || comm >= 64) return B200_ERR_BAD_ARG;
  GinDevHandle h = *hp;
  if (E <= 0 || E % h.nranks || k <= 0 || k > MOE_MAX_TOPK || H % 256 || T <= 0) return B200_ERR_BAD_ARG;
  if (H / 128 > 64) return B200_ERR_TOO_LARGE;
  const size_t row_bytes = fp8 ? static_cast<size_t>(H) : static_cast<size_t>(H) * 2;
  if (recv_off % 16 || meta_off % 16 || scale_off % 16) return B200_ERR_BAD_ARG;
  if (recv_off + row_bytes * capacity_rows > h.window_bytes || meta_off + 16ull * capacity_rows > h.window_bytes ||
      (fp8 && scale_off + 4ull * (H / 128) * capacity_rows > h.window_bytes))
    return B200_ERR_BAD_ARG;
  DispatchArgs a{h, static_cast<const __nv_bfloat16*>(x), static_cast<const int32_t*>(topk_idx),
                 static_cast<const float*>(topk_w), T, k, H, E, fp8, use_saved_rows, scale_by_weight,
                 static_cast<const int32_t*>(dest_base), static_cast<int32_t*>(cursor), static_cast<int32_t*>(row_of),
                 recv_off, scale_off, meta_off, capacity_rows, static_cast<unsigned int*>(done), ++g_moe_epoch[comm][1]};
  moe_dispatch_kernel<<<moe_grid(T), MOE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(a);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

// Collective. Every CTA of this kernel waits for the other ranks, so the grid is limited to what
// is resident at once.
int b200_moe_combine(int comm, const void* y, const void* expert_offsets, int experts_local, size_t meta_off, size_t comb_off,
                     const void* topk_w, const void* row_of, int T, int k, int H, void* out, void* done, void* stream) {
  ensure_context();
  const GinDevHandle* hp = comm_handle(comm);
  if (!hp || comm < 0 || comm >= 64) return B200_ERR_BAD_ARG;
  GinDevHandle h = *hp;
  if (H % 8 || k <= 0 || k > MOE_MAX_TOPK || T <= 0) return B200_ERR_BAD_ARG;
  if (comb_off % 16 || comb_off + static_cast<size_t>(T) * k * H * 2 > h.window_bytes) return B200_ERR_BAD_ARG;
  CombineArgs a{h, static_cast<const __nv_bfloat16*>(y), static_cast<const int32_t*>(expert_offsets), experts_local, meta_off,
                comb_off, static_cast<const float*>(topk_w), static_cast<const int32_t*>(row_of), T, k, H,
                static_cast<__nv_bfloat16*>(out), static_cast<unsigned int*>(done), ++g_moe_epoch[comm][2]};
  int per_sm = 0;
  B200_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_combine_kernel, MOE_THREADS, 0));
  if (per_sm < 1) return B200_ERR_BAD_ARG;
  if (per_sm > 4) per_sm = 4;
  moe_combine_kernel<<<sm_count() * per_sm, MOE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(a);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

int b200_moe_combine_wgrad(const void* dout, const void* comb, const void* row_of, void* dw, int T, int k, int H, void* stream) {
  ensure_context();
  if (H % 8) return B200_ERR_BAD_ARG;
  moe_combine_wgrad_kernel<<<moe_grid(T * k), MOE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(comb), static_cast<const int32_t*>(row_of),
      static_cast<float*>(dw), T, k, H);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

// rows_ptr (device int32, may be null) limits the work to the rows actually received.
int b200_fp8_dequant_rows(const void* q, const void* scales, void* out, const void* rows_ptr, int rows_max, int H, void* stream) {
  ensure_context();
  if (H % 128) return B200_ERR_BAD_ARG;
  int grid = sm_count() * 8;
  fp8_dequant_rows_kernel<<<grid, MOE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(q), static_cast<const float*>(scales), static_cast<__nv_bfloat16*>(out),
      static_cast<const int32_t*>(rows_ptr), rows_max, H);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // extern "C"
