// Device code of the network plugin's data path, loaded by the plugin through the driver API from
// an image embedded at build time (the plugin links no CUDA library).
//
//  b200net_copy_flag  : payload of an isend whose source and destination are both device-visible
//                       (the peer's buffer is mapped through CUDA IPC / VMM): 16-byte vector copy
//                       over NVLink by however many CTAs the host chose for the stripe, then ONE
//                       release-ordered store of a completion word in pinned host memory, so the
//                       proxy thread polls a cache line instead of calling into the driver.
//  b200net_eager_pack : small device payload -> one pinned host slot laid out as
//                       [header 16 B][payload][flag 8 B]: payload and header first, the flag last
//                       with release ordering, so a reader that sees the flag sees the whole slot.
//
// The reference's data path is the NIC's DMA engine driven by fi_write / fi_writedata
// (reference: src/rdma/nccl_ofi_rdma.cpp, post_rdma_write / post_rdma_eager_send); on an NVLink
// box the SMs are the engine.
#include <cuda_runtime.h>

#include <cstdint>

namespace {

__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// All threads of all CTAs call it; returns true in every thread of the CTA that finished last.
__device__ __forceinline__ bool last_cta(unsigned int* counter) {
  __shared__ int is_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(counter, 1u);
    is_last = prev == gridDim.x - 1;
    if (is_last) *counter = 0;  // rearm for the next launch that uses this slot
  }
  __syncthreads();
  return is_last != 0;
}

}  // namespace

extern "C" __global__ void __launch_bounds__(512)
    b200net_copy_flag(unsigned char* dst, const unsigned char* src, unsigned long long bytes, unsigned int* counter,
                      unsigned long long* flag, unsigned long long flag_value) {
  const unsigned long long tid = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x;
  const unsigned long long nthreads = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0) {
    const unsigned long long nvec = bytes >> 4;
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    constexpr int U = 4;
    for (unsigned long long v = tid; v < nvec; v += nthreads * U) {
      uint4 tmp[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (v + u * nthreads < nvec) tmp[u] = s[v + u * nthreads];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (v + u * nthreads < nvec) d[v + u * nthreads] = tmp[u];
    }
    for (unsigned long long b = (nvec << 4) + tid; b < bytes; b += nthreads) dst[b] = src[b];
  } else {
    for (unsigned long long b = tid; b < bytes; b += nthreads) dst[b] = src[b];
  }
  if (last_cta(counter) && threadIdx.x == 0) st_release_sys_u64(flag, flag_value);
}

// One CTA. slot: [hdr0 u64][hdr1 u64][payload ...][pad to 8][flag u64 at slot + flag_off].
extern "C" __global__ void __launch_bounds__(256)
    b200net_eager_pack(unsigned char* slot, const unsigned char* payload, unsigned int bytes, unsigned long long hdr0,
                       unsigned long long hdr1, unsigned int flag_off, unsigned long long flag_value) {
  unsigned char* body = slot + 16;
  if (((reinterpret_cast<uintptr_t>(payload)) & 15) == 0) {
    const unsigned int nvec = bytes >> 4;
    for (unsigned int v = threadIdx.x; v < nvec; v += blockDim.x)
      reinterpret_cast<uint4*>(body)[v] = reinterpret_cast<const uint4*>(payload)[v];
    for (unsigned int b = (nvec << 4) + threadIdx.x; b < bytes; b += blockDim.x) body[b] = payload[b];
  } else {
    for (unsigned int b = threadIdx.x; b < bytes; b += blockDim.x) body[b] = payload[b];
  }
  if (threadIdx.x == 0) {
    reinterpret_cast<unsigned long long*>(slot)[0] = hdr0;
    reinterpret_cast<unsigned long long*>(slot)[1] = hdr1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    st_release_sys_u64(reinterpret_cast<unsigned long long*>(slot + flag_off), flag_value);
  }
}
