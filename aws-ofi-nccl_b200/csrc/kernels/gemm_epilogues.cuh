// Epilogue functors for the tcgen05 GEMM mainloop: plain store (bf16 / fp32, optional accumulate)
// and the fused SwiGLU store used by the tensor-parallel MLP.
#pragma once
#include "gemm_tcgen05.cuh"

namespace b200 {

template <typename OutT>
struct StoreEpilogue {
  static constexpr bool kPair = false;
  OutT* C;
  int64_t ldc;
  int accumulate;
  __device__ __forceinline__ void tile_begin(int, int) {}
  __device__ __forceinline__ void tile_end(int, int) {}
  __device__ __forceinline__ void operator()(int row, int col0, const uint32_t (&acc)[32], const GemmShape& s) {
    if (row >= s.M || col0 >= s.N) return;
    OutT* dst = C + static_cast<int64_t>(row) * ldc + col0;
    const int ncols = min(32, s.N - col0);
    if constexpr (sizeof(OutT) == 2) {
      if (ncols == 32) {
        uint32_t packed[16];
        if (accumulate) {
          const uint4* old = reinterpret_cast<const uint4*>(dst);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o = old[v];
            const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __nv_bfloat162 ob = *reinterpret_cast<const __nv_bfloat162*>(&ow[j]);
              packed[v * 4 + j] = pack_bf16x2(__uint_as_float(acc[v * 8 + 2 * j]) + __low2float(ob),
                                              __uint_as_float(acc[v * 8 + 2 * j + 1]) + __high2float(ob));
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            packed[j] = pack_bf16x2(__uint_as_float(acc[2 * j]), __uint_as_float(acc[2 * j + 1]));
        }
        uint4* out = reinterpret_cast<uint4*>(dst);
#pragma unroll
        for (int v = 0; v < 4; ++v)
          out[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
      } else {
        for (int j = 0; j < ncols; ++j) {
          float v = __uint_as_float(acc[j]);
          if (accumulate) v += __bfloat162float(reinterpret_cast<__nv_bfloat16*>(dst)[j]);
          reinterpret_cast<__nv_bfloat16*>(dst)[j] = __float2bfloat16(v);
        }
      }
    } else {
      if (ncols == 32) {
        float4* out = reinterpret_cast<float4*>(dst);
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          float4 o = accumulate ? out[v] : make_float4(0.f, 0.f, 0.f, 0.f);
          out[v] = make_float4(o.x + __uint_as_float(acc[4 * v]), o.y + __uint_as_float(acc[4 * v + 1]),
                               o.z + __uint_as_float(acc[4 * v + 2]), o.w + __uint_as_float(acc[4 * v + 3]));
        }
      } else {
        for (int j = 0; j < ncols; ++j) {
          float v = __uint_as_float(acc[j]);
          if (accumulate) v += reinterpret_cast<float*>(dst)[j];
          reinterpret_cast<float*>(dst)[j] = v;
        }
      }
    }
  }
};


// bf16 store of acc * row_scale[row] * col_scale[col]: the dequantisation of an fp8 product whose
// operands were quantised per row (activations: one scale per token, weights: one per output
// channel).
struct ScaledStoreEpilogue {
  static constexpr bool kPair = false;
  __nv_bfloat16* C;
  int64_t ldc;
  const float* row_scale;   // [M]
  const float* col_scale;   // [N]
  __device__ __forceinline__ void tile_begin(int, int) {}
  __device__ __forceinline__ void tile_end(int, int) {}
  __device__ __forceinline__ void operator()(int row, int col0, const uint32_t (&acc)[32], const GemmShape& s) {
    if (row >= s.M || col0 >= s.N) return;
    const float rs = row_scale[row];
    __nv_bfloat16* dst = C + static_cast<int64_t>(row) * ldc + col0;
    const int ncols = min(32, s.N - col0);
    if (ncols == 32) {
      uint32_t packed[16];
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        const float4 cs = *reinterpret_cast<const float4*>(col_scale + col0 + 4 * v);
        packed[2 * v] = pack_bf16x2(__uint_as_float(acc[4 * v]) * rs * cs.x, __uint_as_float(acc[4 * v + 1]) * rs * cs.y);
        packed[2 * v + 1] = pack_bf16x2(__uint_as_float(acc[4 * v + 2]) * rs * cs.z, __uint_as_float(acc[4 * v + 3]) * rs * cs.w);
      }
      uint4* out = reinterpret_cast<uint4*>(dst);
#pragma unroll
      for (int v = 0; v < 4; ++v) out[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
    } else {
      for (int j = 0; j < ncols; ++j) dst[j] = __float2bfloat16(__uint_as_float(acc[j]) * rs * col_scale[col0 + j]);
    }
  }
};

// SwiGLU fused into the up/gate GEMM. The weight rows are interleaved in blocks of 64 output
// columns: 32 gate columns followed by their 32 up columns, so one call sees a gate chunk and the
// matching up chunk and writes act = silu(gate) * up (and, optionally, the raw gate|up pair that
// the backward pass needs).
struct SwiGluEpilogue {
  static constexpr bool kPair = true;
  __nv_bfloat16* act;   // [M][N/2]
  int64_t ld_act;
  __nv_bfloat16* gu;    // [M][N] interleaved as computed, or null
  int64_t ld_gu;
  __device__ __forceinline__ void tile_begin(int, int) {}
  __device__ __forceinline__ void tile_end(int, int) {}
  // col0 is the first column of the 64-wide (gate|up) block
  __device__ __forceinline__ void operator()(int row, int col0, const uint32_t (&g)[32], const uint32_t (&u)[32],
                                             const GemmShape& s) {
    if (row >= s.M || col0 >= s.N) return;
    uint32_t packed[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
      const float a0 = g0 / (1.f + __expf(-g0)) * __uint_as_float(u[2 * j]);
      const float a1 = g1 / (1.f + __expf(-g1)) * __uint_as_float(u[2 * j + 1]);
      packed[j] = pack_bf16x2(a0, a1);
    }
    uint4* out = reinterpret_cast<uint4*>(act + static_cast<int64_t>(row) * ld_act + col0 / 2);
#pragma unroll
    for (int v = 0; v < 4; ++v) out[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
    if (gu) {
      uint4* o2 = reinterpret_cast<uint4*>(gu + static_cast<int64_t>(row) * ld_gu + col0);
#pragma unroll
      for (int v = 0; v < 4; ++v)
        o2[v] = make_uint4(pack_bf16x2(__uint_as_float(g[8 * v]), __uint_as_float(g[8 * v + 1])),
                           pack_bf16x2(__uint_as_float(g[8 * v + 2]), __uint_as_float(g[8 * v + 3])),
                           pack_bf16x2(__uint_as_float(g[8 * v + 4]), __uint_as_float(g[8 * v + 5])),
                           pack_bf16x2(__uint_as_float(g[8 * v + 6]), __uint_as_float(g[8 * v + 7])));
#pragma unroll
      for (int v = 0; v < 4; ++v)
        o2[4 + v] = make_uint4(pack_bf16x2(__uint_as_float(u[8 * v]), __uint_as_float(u[8 * v + 1])),
                               pack_bf16x2(__uint_as_float(u[8 * v + 2]), __uint_as_float(u[8 * v + 3])),
                               pack_bf16x2(__uint_as_float(u[8 * v + 4]), __uint_as_float(u[8 * v + 5])),
                               pack_bf16x2(__uint_as_float(u[8 * v + 6]), __uint_as_float(u[8 * v + 7])));
    }
  }
};

}  // namespace b200
