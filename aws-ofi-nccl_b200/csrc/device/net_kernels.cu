// Device code of the network plugin's data path, loaded by the plugin through the driver API from
// an image embedded at build time (the plugin links no CUDA library).
//
//  b200net_copy_flag  : payload of an isend whose source and destination are both device-visible
//                       (the peer's buffer is mapped through CUDA IPC / VMM): 16-byte vector copy
//                       over NVLink by however many CTAs the host chose for the stripe, then ONE
//                       release-ordered store of a completion word in pinned host memory, so the
//                       proxy thread polls a cache line instead of calling into the driver.
//  b200net_copy_bulk  : the same transfer for 16-byte aligned stripes, driven by the bulk-copy (TMA)
//                       unit: one thread per CTA keeps four 32 KiB pieces in flight, global ->
//                       shared memory -> the peer's memory, so a handful of CTAs with one warp each
//                       hold megabytes in flight over NVLink and leave the SMs' issue slots to the
//                       collective kernel that is running beside it. No load is multicast.
//  b200net_copy_batch : up to 16 such transfers in one launch, each with its own completion word: the
//                       stripes that piled up while earlier launches were running share one launch
//                       latency instead of paying it one after the other on the plugin's one stream.
//  b200net_signal_add : a GIN signal applied by the host for a peer: one atomic add on the word.
//  b200net_eager_pack : small device payload -> one pinned host slot laid out as
//                       [header 16 B][payload][flag 8 B]: payload and header first, the flag last
//                       with release ordering, so a reader that sees the flag sees the whole slot.
//
// The reference's data path is the NIC's DMA engine driven by fi_write / fi_writedata
// (reference: src/rdma/nccl_ofi_rdma.cpp, post_rdma_write / post_rdma_eager_send); on an NVLink
// box the SMs are the engine.
#include <cuda_runtime.h>

#include <cstdint>

#include "b200net/net_kernel_args.h"

namespace {

__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

constexpr unsigned int kCtaFailed = 0x80000000u;   // set in the slot's counter by a CTA whose wait ran out

// All threads of all CTAs call it; returns non-zero in every thread of the CTA that finished last:
// 1 when every CTA copied its share, 2 when one of them gave up.
__device__ __forceinline__ int last_cta(unsigned int* counter, unsigned int total, bool failed = false) {
  __shared__ int is_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (failed) atomicOr(counter, kCtaFailed);
    const unsigned int prev = atomicAdd(counter, 1u);
    is_last = (prev & ~kCtaFailed) == total - 1 ? (((prev & kCtaFailed) || failed) ? 2 : 1) : 0;
    if (is_last) *counter = 0;  // rearm for the next launch that uses this slot
  }
  __syncthreads();
  return is_last;
}

__device__ __forceinline__ unsigned int smem_u32(const void* p) { return static_cast<unsigned int>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Waits for the phase of an mbarrier; gives up (false) once `deadline_ns` of the global timer has passed.
__device__ __forceinline__ bool mbar_wait_bounded(unsigned int bar, unsigned int parity, unsigned long long deadline_ns) {
  for (unsigned int spins = 0;; ++spins) {
    unsigned int ok;
    asm volatile(
        "{\n .reg .pred P;\n mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n selp.u32 %0, 1, 0, P;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((spins & 1023u) == 1023u && global_ns() > deadline_ns) return false;
  }
}

}  // namespace

// CTA `cta` of `nctas` copies its share of [0, bytes) with every thread of the block.
__device__ __forceinline__ void copy_vector(unsigned char* dst, const unsigned char* src, unsigned long long bytes,
                                            unsigned int cta, unsigned int nctas) {
  const unsigned long long tid = cta * static_cast<unsigned long long>(blockDim.x) + threadIdx.x;
  const unsigned long long nthreads = static_cast<unsigned long long>(nctas) * blockDim.x;
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
}

extern "C" __global__ void __launch_bounds__(512)
    b200net_copy_flag(unsigned char* dst, const unsigned char* src, unsigned long long bytes, unsigned int* counter,
                      unsigned long long* flag, unsigned long long flag_value) {
  copy_vector(dst, src, bytes, blockIdx.x, gridDim.x);
  if (last_cta(counter, gridDim.x) && threadIdx.x == 0) st_release_sys_u64(flag, flag_value);
}

// dst, src and bytes are multiples of 16 (the host checks). One warp per CTA; lane 0 does the work.
// Dynamic shared memory: kBulkStages pieces of kBulkChunk bytes, then one mbarrier per stage.
// The completion word receives flag_value, or flag_value | 1 << 63 when a wait ran out (the host
// then fails the request instead of reporting bytes that may not have landed).
constexpr unsigned int kBulkChunk = 32768;
constexpr int kBulkStages = 4;

// Called by ONE thread of CTA `cta` of `nctas`: moves the pieces cta, cta + nctas, ... of [0, bytes)
// through the CTA's shared memory. `bars` are kBulkStages initialised mbarriers whose phase count
// starts at `phase0` pieces (a CTA that runs several transfers keeps counting). Returns false when a
// wait ran out; in every case no copy of this CTA is in flight when it returns.
__device__ __forceinline__ bool copy_bulk_cta(unsigned char* dst, const unsigned char* src, unsigned long long bytes,
                                              unsigned int cta, unsigned int nctas, unsigned char* smem,
                                              unsigned long long* bars, unsigned long long wait_limit_ns) {
  bool failed = false;
  const unsigned long long nchunks = (bytes + kBulkChunk - 1) / kBulkChunk;
  const unsigned long long mine = nchunks > cta ? (nchunks - cta + nctas - 1) / nctas : 0;
  const unsigned long long deadline = global_ns() + wait_limit_ns;
  auto chunk_off = [&](unsigned long long k) { return (cta + k * nctas) * static_cast<unsigned long long>(kBulkChunk); };
  auto chunk_len = [&](unsigned long long k) {
    const unsigned long long off = chunk_off(k);
    return static_cast<unsigned int>(bytes - off < kBulkChunk ? bytes - off : kBulkChunk);
  };
  auto load = [&](unsigned long long k) {
    const int s = static_cast<int>(k % kBulkStages);
    const unsigned int len = chunk_len(k);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&bars[s])), "r"(len) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem + s * kBulkChunk)),
                 "l"(src + chunk_off(k)), "r"(len), "r"(smem_u32(&bars[s]))
                 : "memory");
  };
  unsigned long long loaded = 0;
  for (; loaded < mine && loaded < kBulkStages; ++loaded) load(loaded);
  unsigned long long k = 0;
  for (; k < mine; ++k) {
    const int s = static_cast<int>(k % kBulkStages);
    if (!mbar_wait_bounded(smem_u32(&bars[s]), static_cast<unsigned int>((k / kBulkStages) & 1), deadline)) {
      failed = true;
      break;
    }
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst + chunk_off(k)),
                 "r"(smem_u32(smem + s * kBulkChunk)), "r"(chunk_len(k))
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    // the stage of the piece before this one is free once its store has read shared memory
    if (k >= 1 && loaded < mine) {
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      load(loaded++);
    }
  }
  if (failed) {
    // loads already issued may still write this CTA's shared memory: give each one more bounded wait
    const unsigned long long again = global_ns() + wait_limit_ns;
    for (unsigned long long j = k; j < loaded; ++j)
      mbar_wait_bounded(smem_u32(&bars[j % kBulkStages]), static_cast<unsigned int>((j / kBulkStages) & 1), again);
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  return !failed;
}

__device__ __forceinline__ void bulk_barriers_init(unsigned long long* bars) {
  for (int s = 0; s < kBulkStages; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bars[s])));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

extern "C" __global__ void __launch_bounds__(32)
    b200net_copy_bulk(unsigned char* dst, const unsigned char* src, unsigned long long bytes, unsigned int* counter,
                      unsigned long long* flag, unsigned long long flag_value, unsigned long long wait_limit_ns) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + kBulkStages * kBulkChunk);
  bool failed = false;
  if (threadIdx.x == 0) {
    bulk_barriers_init(bars);
    failed = !copy_bulk_cta(dst, src, bytes, blockIdx.x, gridDim.x, smem, bars, wait_limit_ns);
  }
  const int last = last_cta(counter, gridDim.x, failed);
  if (last && threadIdx.x == 0) st_release_sys_u64(flag, last == 2 ? (flag_value | (1ull << 63)) : flag_value);
}

// Several transfers in one launch. CTA b works on the job whose [cta_begin, cta_begin + ctas) holds
// b: with the bulk-copy unit when the job's bit in bulk_mask is set (one thread drives it), else with
// all 128 threads. Every job has its own counter and completion word, so each request completes on
// its own, as if it had been launched alone. Same shared-memory layout as b200net_copy_bulk.
extern "C" __global__ void __launch_bounds__(128) b200net_copy_batch(const __grid_constant__ B200NetBatchArgs args) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + kBulkStages * kBulkChunk);
  unsigned int j = 0;
  while (j + 1 < args.njobs && blockIdx.x >= args.job[j].cta_begin + args.job[j].ctas) ++j;
  const B200NetBatchJob& job = args.job[j];
  if (blockIdx.x < job.cta_begin || blockIdx.x >= job.cta_begin + job.ctas) return;   // a table that does not cover the grid
  const unsigned int cta = blockIdx.x - job.cta_begin;
  bool failed = false;
  if ((args.bulk_mask >> j) & 1u) {
    if (threadIdx.x == 0) {
      bulk_barriers_init(bars);
      failed = !copy_bulk_cta(job.dst, job.src, job.bytes, cta, job.ctas, smem, bars, args.wait_limit_ns);
    }
  } else {
    copy_vector(job.dst, job.src, job.bytes, cta, job.ctas);
  }
  const int last = last_cta(job.counter, job.ctas, failed);
  if (last && threadIdx.x == 0) st_release_sys_u64(job.flag, last == 2 ? (job.flag_value | (1ull << 63)) : job.flag_value);
}

// A signal raised by the host on behalf of a peer: one release-ordered atomic add on the signal
// word in device memory. An atomic, not a store of a value computed on the host: kernels that
// raise the same signal from the device (red.release.sys) and this one compose.
extern "C" __global__ void b200net_signal_add(unsigned long long* word, unsigned long long value) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(word), "l"(value) : "memory");
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
