// RMSNorm backward for callers that cannot allocate: the partial-sum rows sit in a file-scope
// device array instead of a caller-provided buffer. See noalloc.h for the contract.
#include "noalloc.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <stdint.h>
#include <stdio.h>

namespace {

using bf16 = __nv_bfloat16;
using bf162 = __nv_bfloat162;
constexpr int THREADS = 256;

// Fixed staging area. In host code this name is only a stand-in for the symbol — never a device
// address — so the host asks the runtime for the address (below) and hands that to the kernels.
static __device__ __align__(256) float g_dw_partial[B200_NOALLOC_MAX_ROWS * B200_NOALLOC_MAX_H];

struct alignas(16) Vec8 {
  bf162 v[4];
};
__device__ __forceinline__ void unpack(const Vec8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __low2float(p.v[i]);
    f[2 * i + 1] = __high2float(p.v[i]);
  }
}
__device__ __forceinline__ Vec8 pack(const float (&f)[8]) {
  Vec8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

// Each CTA walks rows blockIdx.x, +gridDim.x, ...; its slice of dw stays in registers and is
// written once, completely, to row blockIdx.x of `partial` (row pitch H).
template <int VPT>
__global__ void __launch_bounds__(THREADS)
    bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
               const float* __restrict__ rstd, const bf16* __restrict__ dres, bf16* __restrict__ dx,
               float* __restrict__ partial, int T, int H) {
  __shared__ float red[32];
  float acc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  const Vec8* wr = reinterpret_cast<const Vec8*>(w);
  for (int64_t row = blockIdx.x; row < T; row += gridDim.x) {
    const Vec8* dyr = reinterpret_cast<const Vec8*>(dy + row * H);
    const Vec8* xr = reinterpret_cast<const Vec8*>(x + row * H);
    const float r = rstd[row];
    float g[VPT][8], xv[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * THREADS;
      if (idx * 8 < H) {
        float d[8], wv[8];
        unpack(dyr[idx], d);
        unpack(xr[idx], xv[i]);
        unpack(wr[idx], wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc[i][j] += d[j] * xv[i][j] * r;
          g[i][j] = d[j] * wv[j];
          dot += g[i][j] * xv[i][j];
        }
      }
    }
    dot = block_sum(dot, red);
    const float c = dot * r * r / H;
    Vec8* dxr = reinterpret_cast<Vec8*>(dx + row * H);
    const Vec8* drr = dres ? reinterpret_cast<const Vec8*>(dres + row * H) : nullptr;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * THREADS;
      if (idx * 8 < H) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = r * (g[i][j] - xv[i][j] * c);
        if (drr) {
          float e[8];
          unpack(drr[idx], e);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += e[j];
        }
        dxr[idx] = pack(o);
      }
    }
  }
  float* out = partial + static_cast<int64_t>(blockIdx.x) * H;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (idx * 8 < H) {
#pragma unroll
      for (int j = 0; j < 8; ++j) out[idx * 8 + j] = acc[i][j];
    }
  }
}

__global__ void colsum_kernel(const float* __restrict__ partial, bf16* __restrict__ dw, int nrows, int H, int accumulate) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  float s = 0.f;
  for (int r = 0; r < nrows; ++r) s += partial[static_cast<int64_t>(r) * H + h];
  if (accumulate) s += __bfloat162float(dw[h]);
  dw[h] = __float2bfloat16(s);
}

// Device address of the staging array and SM count, looked up once per device (index = device
// ordinal). The address is published last, with release ordering, and read with acquire ordering:
// a thread that sees it also sees the SM count. Two threads making the first call at once both do
// the look-up and store the same values. The address belongs to the device's current context: it
// does not survive a cudaDeviceReset (the next call after one would use a stale address).
std::atomic<float*> g_partial_addr[64];
int g_sm_count[64] = {0};

}  // namespace

extern "C" int b200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                        const void* dres, void* dx, void* dw, int accumulate_dw, int T, int H,
                                        void* stream) {
  if (!dy || !x || !w || !rstd || !dx || !dw || T <= 0 || H <= 0 || H % 8) return 10001;
  // the kernels move rows as 16-byte vectors: a misaligned pointer would fault on the device
  const uintptr_t all = reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) |
                        reinterpret_cast<uintptr_t>(dres) | reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(dw);
  if ((all & 15) || (reinterpret_cast<uintptr_t>(rstd) & 3)) return 10001;
  if (H > B200_NOALLOC_MAX_H) {
    fprintf(stderr, "[b200ops] rmsnorm_bwd_noalloc: H=%d exceeds the fixed staging area (max %d)\n", H,
            B200_NOALLOC_MAX_H);
    return 10004;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) return e != cudaSuccess ? static_cast<int>(e) : 10001;
  float* partial = g_partial_addr[dev].load(std::memory_order_acquire);
  if (!partial) {
    // set-up, once per device, with that device current
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_dw_partial);
    if (e != cudaSuccess) {
      fprintf(stderr, "[b200ops] cudaGetSymbolAddress(staging rows) failed: %s\n", cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_sm_count[dev] = sms;
    g_partial_addr[dev].store(p, std::memory_order_release);
    partial = p;
  }
  int grid = 2 * g_sm_count[dev];
  if (grid > B200_NOALLOC_MAX_ROWS) grid = B200_NOALLOC_MAX_ROWS;
  if (grid > T) grid = T;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto DY = static_cast<const bf16*>(dy);
  auto X = static_cast<const bf16*>(x);
  auto W = static_cast<const bf16*>(w);
  auto DR = static_cast<const bf16*>(dres);
  auto DX = static_cast<bf16*>(dx);
  const int vpt = (H + THREADS * 8 - 1) / (THREADS * 8);
  switch (vpt) {
    case 1: bwd_kernel<1><<<grid, THREADS, 0, s>>>(DY, X, W, rstd, DR, DX, partial, T, H); break;
    case 2: bwd_kernel<2><<<grid, THREADS, 0, s>>>(DY, X, W, rstd, DR, DX, partial, T, H); break;
    case 3: bwd_kernel<3><<<grid, THREADS, 0, s>>>(DY, X, W, rstd, DR, DX, partial, T, H); break;
    default: bwd_kernel<4><<<grid, THREADS, 0, s>>>(DY, X, W, rstd, DR, DX, partial, T, H); break;
  }
  colsum_kernel<<<(H + 255) / 256, 256, 0, s>>>(partial, static_cast<bf16*>(dw), grid, H, accumulate_dw);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
