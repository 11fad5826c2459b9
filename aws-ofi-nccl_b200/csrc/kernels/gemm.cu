// bf16 GEMM entry points built on the tcgen05 mainloop.
//
//   C[M,N] (+)= op(A) * op(B)     fp32 accumulation in TMEM, bf16 or fp32 output
//
// Operand storage is described by two flags instead of BLAS transposes:
//   a_mn = 0 : A stored [M][K] (K contiguous)      a_mn = 1 : A stored [K][M] (M contiguous)
//   b_mn = 0 : B stored [N][K] (K contiguous)      b_mn = 1 : B stored [K][N] (N contiguous)
// so a linear layer's forward (x W^T), input gradient (dy W) and weight gradient (dy^T x) all run
// on the same kernel without materialising a transpose.
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
