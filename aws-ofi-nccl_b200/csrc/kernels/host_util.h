// Host-side helpers shared by the kernel launchers: driver entry points resolved through the
// runtime (no link-time dependency on libcuda), tensor-map encoding, device status word.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace b200 {

#define B200_CUDA_OK(expr)                                                                      \
  do {                                                                                          \
    cudaError_t _e = (expr);                                                                    \
    if (_e != cudaSuccess) {                                                                    \
      fprintf(stderr, "[b200ops] %s:%d %s -> %s\n", __FILE__, __LINE__, #expr, cudaGetErrorString(_e)); \
      return static_cast<int>(_e);                                                              \
    }                                                                                           \
  } while (0)

// Library-specific return codes (above the CUDA error range).
enum HostErr : int {
  B200_ERR_BAD_ARG = 10001,
  B200_ERR_NO_DRIVER = 10002,
  B200_ERR_TENSORMAP = 10003,
  B200_ERR_TOO_LARGE = 10004,
};

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major tensor [rows][cols] of `elem_bytes` elements, row pitch `ld` elements.
// Box = [box_rows][box_cols]; box_cols * elem_bytes must equal the swizzle span (128 B) when swizzled.
inline int make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                        uint32_t box_rows, uint32_t box_cols, int elem_bytes, bool swizzle128) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return B200_ERR_NO_DRIVER;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                             : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[b200ops] cuTensorMapEncodeTiled failed: %d (base=%p rows=%llu cols=%llu ld=%llu box=%ux%u)\n",
            static_cast<int>(r), base, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld,
            box_rows, box_cols);
    return B200_ERR_TENSORMAP;
  }
  return 0;
}

// Worker threads (PyTorch's autograd threads) may enter the library with no CUDA context bound
// to the thread. One process drives one GPU, so remember the device of the first call that had
// a context and bind later context-less threads to it.
inline void ensure_context() {
  static int g_dev = -1;
  using GetCurFn = CUresult (*)(CUcontext*);
  static GetCurFn get_cur = nullptr;
  if (!get_cur) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      get_cur = reinterpret_cast<GetCurFn>(p);
  }
  CUcontext ctx = nullptr;
  if (get_cur) get_cur(&ctx);
  if (ctx) {
    if (g_dev < 0) cudaGetDevice(&g_dev);
  } else {
    cudaSetDevice(g_dev >= 0 ? g_dev : 0);
    cudaFree(0);
  }
}

// Per-device status word that kernels write on a bounded-wait timeout. Allocated once per device.
int* device_status_word();

inline int sm_count() {
  static int n[16] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) dev = 0;
  if (!n[dev]) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
  return n[dev] ? n[dev] : 148;
}

}  // namespace b200
