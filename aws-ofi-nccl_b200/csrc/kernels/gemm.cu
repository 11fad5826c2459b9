// bf16 GEMM entry points built on the tcgen05 mainloop.
//
//   C[M,N] (+)= op(A) * op(B)     fp32 accumulation in TMEM, bf16 or fp32 output
//
// Operand storage is described by two flags instead of BLAS transposes:
//   a_mn = 0 : A stored [M][K] (K contiguous)      a_mn = 1 : A stored [K][M] (M contiguous)
//   b_mn = 0 : B stored [N][K] (K contiguous)      b_mn = 1 : B stored [K][N] (N contiguous)
// so a linear layer's forward (x W^T), input gradient (dy W) and weight gradient (dy^T x) all run
// on the same kernel without materialising a transpose.
#include <cuda_fp8.h>

#include "gemm_epilogues.cuh"
#include "gemm_tcgen05.cuh"
#include "gemm_tcgen05_2cta.cuh"
#include "host_util.h"

namespace b200 {

int* device_status_word() {
  static int* words[16] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) dev = 0;
  if (!words[dev]) {
    if (cudaMalloc(&words[dev], 256) != cudaSuccess) return nullptr;
    cudaMemset(words[dev], 0, 256);
  }
  return words[dev];
}

template <int BN, bool A_MN, bool B_MN, typename OutT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, OutT* C,
                     int64_t ldc, GemmShape shape, int accumulate, int* err_word) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  StoreEpilogue<OutT> epi{C, ldc, accumulate};
  NoGate gate;
  gemm_mainloop<BN, A_MN, B_MN>(&tmA, &tmB, shape, epi, gate, err_word, smem_raw);
}

// M tiles per raster group: the CTAs of one wave (one per SM) then cover a patch of about
// group_m x (SMs / group_m) tiles, which is close to square in elements for the default value.
// B200_GEMM_GROUP_M overrides it (0 = plain column-major walk).
static int gemm_group_m(int bn) {
  static int override_value = -2;
  if (override_value == -2) {
    const char* e = getenv("B200_GEMM_GROUP_M");
    override_value = e ? atoi(e) : -1;
  }
  if (override_value >= 0) return override_value;
  return bn == 256 ? 16 : 12;
}

template <int BN, bool A_MN, bool B_MN, typename OutT>
static int launch_gemm(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                       int64_t ldc, int accumulate, int max_ctas, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN)
    rc = make_tmap_2d(&tmA, A, M, K, lda, GEMM_BM, GEMM_BK, 2, true);
  else
    rc = make_tmap_2d(&tmA, A, K, M, lda, GEMM_BK, 64, 2, true);
  if (rc) return rc;
  if (!B_MN)
    rc = make_tmap_2d(&tmB, B, N, K, ldb, BN, GEMM_BK, 2, true);
  else
    rc = make_tmap_2d(&tmB, B, K, N, ldb, GEMM_BK, 64, 2, true);
  if (rc) return rc;
  GemmShape shape{M, N, K, (M + GEMM_BM - 1) / GEMM_BM, (N + BN - 1) / BN};
  shape.group_m = gemm_group_m(BN);
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, OutT>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN>::TOTAL));
    attr_set = true;
  }
  int grid = shape.tiles_m * shape.tiles_n;
  int cap = sm_count();
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  if (grid > cap) grid = cap;
  int* err = device_status_word();
  kern<<<grid, GEMM_THREADS, GemmSmem<BN>::TOTAL, stream>>>(tmA, tmB, static_cast<OutT*>(C), ldc, shape, accumulate,
                                                           err);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

// ---------------------------------------------------------------- CTA-pair variant (256 x 256 tile per cluster)
template <int BN, bool A_MN, bool B_MN, typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
    gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, OutT* C,
                          int64_t ldc, GemmShape shape, int accumulate, int* err_word) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  StoreEpilogue<OutT> epi{C, ldc, accumulate};
  NoGate gate;
  gemm_mainloop_2cta<BN, A_MN, B_MN>(&tmA, &tmB, shape, epi, gate, err_word, smem_raw);
}

template <int BN, bool A_MN, bool B_MN, typename OutT>
static int launch_gemm_2cta(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                            int64_t ldc, int accumulate, int max_ctas, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  int rc;
  // every CTA loads 128 rows of A and BN/2 rows (its half) of B per k-block
  if (!A_MN)
    rc = make_tmap_2d(&tmA, A, M, K, lda, 128, GEMM_BK, 2, true);
  else
    rc = make_tmap_2d(&tmA, A, K, M, lda, GEMM_BK, 64, 2, true);
  if (rc) return rc;
  if (!B_MN)
    rc = make_tmap_2d(&tmB, B, N, K, ldb, BN / 2, GEMM_BK, 2, true);
  else
    rc = make_tmap_2d(&tmB, B, K, N, ldb, GEMM_BK, 64, 2, true);
  if (rc) return rc;
  GemmShape shape{M, N, K, (M + GEMM2_BM - 1) / GEMM2_BM, (N + BN - 1) / BN};
  shape.group_m = (gemm_group_m(BN) + 1) / 2;
  auto kern = gemm_bf16_2cta_kernel<BN, A_MN, B_MN, OutT>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Gemm2Smem<BN>::TOTAL));
    attr_set = true;
  }
  int cap = sm_count();
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  int grid = 2 * shape.tiles_m * shape.tiles_n;
  if (grid > cap) grid = cap & ~1;
  int* err = device_status_word();
  kern<<<grid, GEMM_THREADS, Gemm2Smem<BN>::TOTAL, stream>>>(tmA, tmB, static_cast<OutT*>(C), ldc, shape, accumulate, err);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

template <int BN, typename OutT>
static int dispatch_major_2cta(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                               int64_t ldc, int a_mn, int b_mn, int accumulate, int max_ctas, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch_gemm_2cta<BN, false, false, OutT>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, max_ctas, stream);
  if (!a_mn && b_mn) return launch_gemm_2cta<BN, false, true, OutT>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, max_ctas, stream);
  if (a_mn && !b_mn) return launch_gemm_2cta<BN, true, false, OutT>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, max_ctas, stream);
  return launch_gemm_2cta<BN, true, true, OutT>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, max_ctas, stream);
}

// ---------------------------------------------------------------- fp8 (e4m3) x fp8 -> bf16 with row / column scales
template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
    gemm_fp8_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         ScaledStoreEpilogue epi, GemmShape shape, int* err_word) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  NoGate gate;
  gemm_mainloop_2cta<BN, false, false, ScaledStoreEpilogue, NoGate, true>(&tmA, &tmB, shape, epi, gate, err_word, smem_raw);
}

template <int BN>
static int launch_gemm_fp8(const void* A, const void* B, const float* a_scale, const float* b_scale, void* C, int M, int N,
                           int K, int64_t lda, int64_t ldb, int64_t ldc, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, M, K, lda, 128, 2 * GEMM_BK, 1, true);   // 128 one-byte elements = 128 B per row
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, B, N, K, ldb, BN / 2, 2 * GEMM_BK, 1, true);
  if (rc) return rc;
  GemmShape shape{M, N, K, (M + GEMM2_BM - 1) / GEMM2_BM, (N + BN - 1) / BN};
  shape.group_m = (gemm_group_m(BN) + 1) / 2;
  auto kern = gemm_fp8_2cta_kernel<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Gemm2Smem<BN>::TOTAL));
    attr_set = true;
  }
  int grid = 2 * shape.tiles_m * shape.tiles_n;
  const int cap = sm_count() & ~1;
  if (grid > cap) grid = cap;
  ScaledStoreEpilogue epi{static_cast<__nv_bfloat16*>(C), ldc, a_scale, b_scale};
  kern<<<grid, GEMM_THREADS, Gemm2Smem<BN>::TOTAL, stream>>>(tmA, tmB, epi, shape, device_status_word());
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

// One e4m3 row per bf16 row: scale = amax / 448 (fp32), q = x / scale.
__global__ void __launch_bounds__(256) quant_rows_fp8_kernel(const __nv_bfloat16* x, uint8_t* q, float* scale, int rows,
                                                            int K, int64_t ldx, int64_t ldq) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (int r = blockIdx.x * warps + warp; r < rows; r += gridDim.x * warps) {
    const uint4* src = reinterpret_cast<const uint4*>(x + r * ldx);
    const int nvec = K / 8;
    float amax = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      const uint4 raw = src[v];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fmaxf(fabsf(__low2float(p[j])), fabsf(__high2float(p[j]))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = fmaxf(amax, 1e-12f) * (1.f / 448.f);
    const float inv = 1.f / s;
    if (lane == 0) scale[r] = s;
    uint2* dst = reinterpret_cast<uint2*>(q + r * ldq);
    for (int v = lane; v < nvec; v += 32) {
      const uint4 raw = src[v];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
      uint32_t w[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float2 f0 = __bfloat1622float2(p[2 * h]), f1 = __bfloat1622float2(p[2 * h + 1]);
        w[h] = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(f0.x * inv, f0.y * inv), __NV_SATFINITE, __NV_E4M3)) |
               (static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(f1.x * inv, f1.y * inv), __NV_SATFINITE, __NV_E4M3)) << 16);
      }
      dst[v] = make_uint2(w[0], w[1]);
    }
  }
}

// B200_GEMM_2CTA=0 keeps every GEMM on the one-CTA kernel; by default CTA pairs are used wherever
// they apply (M >= 256, N >= 128).
static int gemm_pair_mode() {
  static int mode = -2;
  if (mode == -2) {
    const char* e = getenv("B200_GEMM_2CTA");
    mode = e ? atoi(e) : -1;
  }
  return mode;
}

template <int BN, typename OutT>
static int dispatch_major(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                          int64_t ldc, int a_mn, int b_mn, int accumulate, int max_ctas, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch_gemm<BN, false, false, OutT>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, max_ctas, stream);
  if (!a_mn && b_mn) return launch_gemm<BN, false, true, OutT>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, max_ctas, stream);
  if (a_mn && !b_mn) return launch_gemm<BN, true, false, OutT>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, max_ctas, stream);
  return launch_gemm<BN, true, true, OutT>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, max_ctas, stream);
}

}  // namespace b200

extern "C" {

// Returns 0 on success. Alignment: base pointers and row pitches must be multiples of 16 bytes.
// out_fp32 selects an fp32 C; accumulate adds to the existing C. bn is 128 or 256 (0 = choose).
int b200_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                   long long ldc, int a_mn, int b_mn, int out_fp32, int accumulate, int bn, int max_ctas,
                   void* stream) {
  b200::ensure_context();
  using namespace b200;
  if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return B200_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return B200_ERR_BAD_ARG;
  if ((lda % 8) || (ldb % 8) || (ldc % (out_fp32 ? 4 : 8))) return B200_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool pairs = gemm_pair_mode() != 0 && M >= 256 && N >= 128 && (max_ctas == 0 || max_ctas >= 2);
  if (bn == 0) {
    // Wider tiles re-read A less; fall back to the narrower tile when that fills the SMs better.
    // With CTA pairs the tile is 256 rows tall and a wave is one tile per pair of SMs.
    const int units = pairs ? sm_count() / 2 : sm_count();
    const long rows = pairs ? (M + 255) / 256 : (M + 127) / 128;
    const long t256 = rows * ((N + 255) / 256);
    const long t128 = rows * ((N + 127) / 128);
    const double eff256 = static_cast<double>(t256) / (((t256 + units - 1) / units) * units);
    const double eff128 = static_cast<double>(t128) / (((t128 + units - 1) / units) * units);
    bn = (N >= 256 && eff256 + 0.08 >= eff128) ? 256 : 128;
  }
  if (pairs) {
    if (bn == 256)
      return out_fp32 ? dispatch_major_2cta<256, float>(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, accumulate, max_ctas, s)
                      : dispatch_major_2cta<256, __nv_bfloat16>(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, accumulate, max_ctas, s);
    if (bn == 128)
      return out_fp32 ? dispatch_major_2cta<128, float>(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, accumulate, max_ctas, s)
                      : dispatch_major_2cta<128, __nv_bfloat16>(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, accumulate, max_ctas, s);
  }
  if (bn == 256) {
    return out_fp32 ? dispatch_major<256, float>(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, accumulate, max_ctas, s)
                    : dispatch_major<256, __nv_bfloat16>(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, accumulate,
                                                         max_ctas, s);
  }
  return out_fp32 ? dispatch_major<128, float>(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, accumulate, max_ctas, s)
                  : dispatch_major<128, __nv_bfloat16>(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, accumulate,
                                                       max_ctas, s);
}

// C[M,N] (bf16) = (A8[M,K] * B8[N,K]^T) * a_scale[M] x b_scale[N]; A8, B8 e4m3, K-major, K % 16 == 0.
// CTA pairs only: M >= 256 and N >= 128.
int b200_gemm_fp8(const void* A, const void* B, const float* a_scale, const float* b_scale, void* C, int M, int N, int K,
                  long long lda, long long ldb, long long ldc, void* stream) {
  b200::ensure_context();
  using namespace b200;
  if (!A || !B || !C || !a_scale || !b_scale || M < 256 || N < 128 || K <= 0) return B200_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) |
       reinterpret_cast<uintptr_t>(b_scale)) & 15)
    return B200_ERR_BAD_ARG;
  if ((lda % 16) || (ldb % 16) || (ldc % 8) || (K % 16) || (N % 4)) return B200_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int units = sm_count() / 2;
  const long rows = (M + 255) / 256;
  const long t256 = rows * ((N + 255) / 256), t128 = rows * ((N + 127) / 128);
  const double eff256 = static_cast<double>(t256) / (((t256 + units - 1) / units) * units);
  const double eff128 = static_cast<double>(t128) / (((t128 + units - 1) / units) * units);
  if (N >= 256 && eff256 + 0.08 >= eff128) return launch_gemm_fp8<256>(A, B, a_scale, b_scale, C, M, N, K, lda, ldb, ldc, s);
  return launch_gemm_fp8<128>(A, B, a_scale, b_scale, C, M, N, K, lda, ldb, ldc, s);
}

// q[rows,K] (e4m3) and scale[rows] (fp32) from x[rows,K] (bf16); K % 8 == 0, 16-byte aligned rows.
int b200_quant_rows_fp8(const void* x, void* q, float* scale, int rows, int K, long long ldx, long long ldq, void* stream) {
  b200::ensure_context();
  if (!x || !q || !scale || rows <= 0 || K <= 0 || K % 8 || ldx % 8 || ldq % 8) return b200::B200_ERR_BAD_ARG;
  int grid = (rows + 7) / 8;
  const int cap = b200::sm_count() * 8;
  if (grid > cap) grid = cap;
  b200::quant_rows_fp8_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), scale, rows, K, ldx, ldq);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

// Reads and clears the device status word (0 = no kernel gave up on a wait). Synchronises the device.
int b200_read_status(int clear) {
  b200::ensure_context();
  int* w = b200::device_status_word();
  if (!w) return -1;
  int v = 0;
  if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (clear && v) cudaMemset(w, 0, sizeof(int));
  return v;
}

}  // extern "C"
