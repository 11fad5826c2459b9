// GIN device API for NVLink: put / put_value / signal / wait_signal / counters / flush / reset,
// plus the multimem (NVSwitch in-fabric reduction / broadcast) primitives and the cross-GPU
// barrier, all callable from inside any kernel of this library.
//
// It plays the role of the kernel-initiated GIN path of the reference, where the GPU builds NIC
// work-queue entries and rings a doorbell (reference: include/rdma/gin/nccl_ofi_gin_gdaki_dev.h
// :302-382 for the handle, 3rd-party/efa-gda/CUDA/device/efa_cuda_dp_impl.cuh for the queue
// operations). On one NVSwitch box a "put" is a peer store, a "signal" is a release-ordered
// remote atomic add on the peer's signal word, and a "wait" is a bounded acquire spin on local
// memory. Signal reset is offset based, as in the reference, so a remote writer never races a reset.
//
// Every wait is bounded by `wait_limit_ns`; on expiry the waiter records an error code in the
// device status word and returns false.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

#include "b200net/gin_dev_handle.h"
#include "sm100_common.cuh"

namespace b200 {

enum GinSignalOp : uint32_t { GIN_SIGNAL_INC = 1, GIN_SIGNAL_ADD = 2 };

// ---------------------------------------------------------------- raw memory-model primitives
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t ld_acquire_sys_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add_u32(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add_u64(uint64_t* p, uint64_t v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

__device__ __forceinline__ void gin_record_error(const GinDevHandle& h, int code) {
  if (h.status) atomicCAS(h.status, 0, code);
}

// ---------------------------------------------------------------- multimem (NVSwitch) primitives, 16 bytes each
__device__ __forceinline__ uint4 mc_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}
__device__ __forceinline__ uint4 mc_ld_reduce_f32x4(const void* mc_addr) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}
__device__ __forceinline__ void mc_st_16(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// ---------------------------------------------------------------- bounded waits
__device__ __forceinline__ bool gin_spin_u32_ge(const GinDevHandle& h, const uint32_t* p, uint32_t target, int code) {
  if (static_cast<int32_t>(ld_acquire_sys_u32(p) - target) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t spins = 1;; ++spins) {
    if (static_cast<int32_t>(ld_acquire_sys_u32(p) - target) >= 0) return true;
    if ((spins & 0xFF) == 0 && globaltimer_ns() - t0 > h.wait_limit_ns) {
      gin_record_error(h, code);
      return false;
    }
  }
}
__device__ __forceinline__ bool gin_spin_u64_ge(const GinDevHandle& h, const uint64_t* p, uint64_t base,
                                                uint64_t target, int code) {
  if (ld_acquire_sys_u64(p) - base >= target) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t spins = 1;; ++spins) {
    if (ld_acquire_sys_u64(p) - base >= target) return true;
    if ((spins & 0xFF) == 0 && globaltimer_ns() - t0 > h.wait_limit_ns) {
      gin_record_error(h, code);
      return false;
    }
  }
}

// ---------------------------------------------------------------- cross-GPU barrier (all threads of the CTA call it)
// Block `slot` of every rank meets block `slot` of every other rank on channel `ch`. Writes made
// by any thread of the CTA before the barrier are visible to every rank after it.
__device__ __forceinline__ bool gin_barrier(const GinDevHandle& h, int ch, int slot) {
  __shared__ int ok_flag;
  __syncthreads();
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  const size_t idx = (static_cast<size_t>(ch) * GIN_MAX_BLOCKS + slot);
  uint32_t* epoch = reinterpret_cast<uint32_t*>(h.pad[h.rank] + GIN_PAD_EPOCH_OFF) + idx;
  const uint32_t target = *epoch + 1;
  if (threadIdx.x < h.nranks) {
    const int peer = threadIdx.x;
    uint32_t* remote = reinterpret_cast<uint32_t*>(h.pad[peer] + GIN_PAD_FLAGS_OFF) + idx * GIN_MAX_RANKS + h.rank;
    fence_acq_rel_sys();
    red_release_sys_add_u32(remote, 1);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(h.pad[h.rank] + GIN_PAD_FLAGS_OFF) + idx * GIN_MAX_RANKS + peer;
    if (!gin_spin_u32_ge(h, mine, target, DEV_ERR_BARRIER_TIMEOUT)) ok_flag = 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) *epoch = target;
  const bool ok = ok_flag != 0;
  __syncthreads();
  return ok;
}

// Two-rank form: only this rank and `peer` meet (both must use the same channel and slot, and that
// slot must not be used for full barriers).
__device__ __forceinline__ bool gin_barrier_pair(const GinDevHandle& h, int ch, int slot, int peer) {
  __shared__ int ok_pair;
  __syncthreads();
  if (threadIdx.x == 0) {
    const size_t idx = (static_cast<size_t>(ch) * GIN_MAX_BLOCKS + slot);
    uint32_t* epoch = reinterpret_cast<uint32_t*>(h.pad[h.rank] + GIN_PAD_EPOCH_OFF) + idx;
    const uint32_t target = *epoch + 1;
    uint32_t* remote = reinterpret_cast<uint32_t*>(h.pad[peer] + GIN_PAD_FLAGS_OFF) + idx * GIN_MAX_RANKS + h.rank;
    fence_acq_rel_sys();
    red_release_sys_add_u32(remote, 1);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(h.pad[h.rank] + GIN_PAD_FLAGS_OFF) + idx * GIN_MAX_RANKS + peer;
    ok_pair = gin_spin_u32_ge(h, mine, target, DEV_ERR_BARRIER_TIMEOUT) ? 1 : 0;
    *epoch = target;
  }
  __syncthreads();
  return ok_pair != 0;
}

// ---------------------------------------------------------------- put
// Copy `bytes` from local `src` into peer's window at dst_off; all `nthreads` threads with index
// `tid` take part (a warp: 32/lane, a CTA: blockDim/threadIdx). 16-byte vectors when both sides
// are 16-byte aligned, bytes otherwise. Out-of-window offsets are refused and recorded.
__device__ __forceinline__ bool gin_put(const GinDevHandle& h, int peer, size_t dst_off, const void* src, size_t bytes,
                                        int tid, int nthreads) {
  if (dst_off + bytes > h.window_bytes || peer < 0 || peer >= h.nranks) {
    gin_record_error(h, DEV_ERR_BOUNDS);
    return false;
  }
  uint8_t* dst = h.window[peer] + dst_off;
  const uint8_t* s = static_cast<const uint8_t*>(src);
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(s)) & 15) == 0) {
    const size_t nvec = bytes >> 4;
    const uint4* sv = reinterpret_cast<const uint4*>(s);
    uint4* dv = reinterpret_cast<uint4*>(dst);
    for (size_t i = tid; i < nvec; i += nthreads) dv[i] = sv[i];
    for (size_t i = (nvec << 4) + tid; i < bytes; i += nthreads) dst[i] = s[i];
  } else {
    for (size_t i = tid; i < bytes; i += nthreads) dst[i] = s[i];
  }
  return true;
}

// The same put into a registration of its own (a window that regMrSym of the plugin's
// kernel-initiated table described): the handle supplies the rank count and the status word.
__device__ __forceinline__ bool gin_put_window(const GinDevHandle& h, const GinDevWindow& w, int peer, size_t dst_off,
                                               const void* src, size_t bytes, int tid, int nthreads) {
  if (dst_off + bytes > w.bytes || peer < 0 || peer >= h.nranks || !w.base[peer]) {
    gin_record_error(h, DEV_ERR_BOUNDS);
    return false;
  }
  uint8_t* dst = w.base[peer] + dst_off;
  const uint8_t* s = static_cast<const uint8_t*>(src);
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(s)) & 15) == 0) {
    const size_t nvec = bytes >> 4;
    const uint4* sv = reinterpret_cast<const uint4*>(s);
    uint4* dv = reinterpret_cast<uint4*>(dst);
    for (size_t i = tid; i < nvec; i += nthreads) dv[i] = sv[i];
    for (size_t i = (nvec << 4) + tid; i < bytes; i += nthreads) dst[i] = s[i];
  } else {
    for (size_t i = tid; i < bytes; i += nthreads) dst[i] = s[i];
  }
  return true;
}

// One thread stores a value of up to 8 bytes.
template <typename T>
__device__ __forceinline__ bool gin_put_value(const GinDevHandle& h, int peer, size_t dst_off, T value) {
  static_assert(sizeof(T) <= 8, "put_value carries at most 8 bytes");
  if (dst_off + sizeof(T) > h.window_bytes) {
    gin_record_error(h, DEV_ERR_BOUNDS);
    return false;
  }
  *reinterpret_cast<volatile T*>(h.window[peer] + dst_off) = value;
  return true;
}

// ---------------------------------------------------------------- signals and counters
__device__ __forceinline__ uint64_t* gin_signal_ptr(const GinDevHandle& h, int rank, int sig) {
  return reinterpret_cast<uint64_t*>(h.pad[rank] + GIN_PAD_SIGNAL_OFF) + sig;
}
// Release-ordered: everything this THREAD wrote (and, after a __syncthreads(), everything its CTA
// wrote) to the peer is visible there before the signal value changes.
__device__ __forceinline__ void gin_signal(const GinDevHandle& h, int peer, int sig, uint64_t value, uint32_t op) {
  // the release on the atomic orders it after this thread's earlier writes and, through a preceding
  // __syncthreads(), after its CTA's writes: no separate fence is needed
  red_release_sys_add_u64(gin_signal_ptr(h, peer, sig), op == GIN_SIGNAL_INC ? 1ull : value);
}
__device__ __forceinline__ uint64_t gin_read_signal(const GinDevHandle& h, int sig) {
  const uint64_t base = reinterpret_cast<const uint64_t*>(h.pad[h.rank] + GIN_PAD_SIGBASE_OFF)[sig];
  return ld_acquire_sys_u64(gin_signal_ptr(h, h.rank, sig)) - base;
}
// Wait until the local signal (since its last reset) has reached `target`.
__device__ __forceinline__ bool gin_wait_signal(const GinDevHandle& h, int sig, uint64_t target) {
  const uint64_t base = reinterpret_cast<const uint64_t*>(h.pad[h.rank] + GIN_PAD_SIGBASE_OFF)[sig];
  return gin_spin_u64_ge(h, gin_signal_ptr(h, h.rank, sig), base, target, DEV_ERR_SIGNAL_TIMEOUT);
}
// Offset-based reset: remember the current raw value; remote adds that race the reset are kept.
__device__ __forceinline__ void gin_reset_signal(const GinDevHandle& h, int sig) {
  reinterpret_cast<uint64_t*>(h.pad[h.rank] + GIN_PAD_SIGBASE_OFF)[sig] =
      ld_acquire_sys_u64(gin_signal_ptr(h, h.rank, sig));
}
// Local completion counters: bumped by the issuer once its puts are globally performed.
__device__ __forceinline__ void gin_counter_add(const GinDevHandle& h, int counter, uint64_t v) {
  fence_acq_rel_sys();
  atomicAdd(reinterpret_cast<unsigned long long*>(h.pad[h.rank] + GIN_PAD_COUNTER_OFF) + counter,
            static_cast<unsigned long long>(v));
}
__device__ __forceinline__ bool gin_wait_counter(const GinDevHandle& h, int counter, uint64_t target) {
  return gin_spin_u64_ge(h, reinterpret_cast<const uint64_t*>(h.pad[h.rank] + GIN_PAD_COUNTER_OFF) + counter, 0, target,
                         DEV_ERR_SIGNAL_TIMEOUT);
}
__device__ __forceinline__ void gin_flush() { fence_acq_rel_sys(); }

// CTA-wide put followed by a signal from one thread (data first, then the flag).
__device__ __forceinline__ bool gin_put_signal_cta(const GinDevHandle& h, int peer, size_t dst_off, const void* src,
                                                   size_t bytes, int sig, uint64_t value, uint32_t op) {
  const bool ok = gin_put(h, peer, dst_off, src, bytes, threadIdx.x, blockDim.x);
  __syncthreads();
  if (threadIdx.x == 0 && ok) gin_signal(h, peer, sig, value, op);
  return ok;
}

}  // namespace b200
