// NVLink collectives on symmetric memory, built on the GIN device API: all-reduce, reduce-scatter,
// all-gather, all-to-all, a device put+signal ping-pong (latency probe), plus the communicator
// registry that the other fused kernels use. Two data paths per collective:
//   NVLS : multimem.ld_reduce / multimem.st — the reduction and the broadcast happen in the switch
//   P2P  : plain peer loads / stores — needs no multicast object (used when NVLS is off)
// The reduce-type kernels take a scale and an output type, so a gradient average (sum * 1/N) and
// the cast of the result are part of the same pass over the data.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <string.h>

#include <mutex>
#include <vector>

#include "gin_device.cuh"
#include "host_util.h"

namespace b200 {

struct Comm {
  GinDevHandle h;
  size_t pad_bytes;
};
static std::mutex g_comm_mu;
static std::vector<Comm*> g_comms;

const GinDevHandle* comm_handle(int id) {
  std::lock_guard<std::mutex> g(g_comm_mu);
  if (id < 0 || id >= static_cast<int>(g_comms.size()) || !g_comms[id]) return nullptr;
  return &g_comms[id]->h;
}

// ---------------------------------------------------------------- helpers
__device__ __forceinline__ void bf16x8_to_f32(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __low2float(p[i]);
    f[2 * i + 1] = __high2float(p[i]);
  }
}
__device__ __forceinline__ uint4 f32_to_bf16x8(const float (&f)[8]) {
  uint4 v;
  uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) w[i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
  return v;
}

// Reduce one 16-byte vector at byte offset `off` of the window across all ranks.
template <bool BF16, bool NVLS>
__device__ __forceinline__ void reduce_vec(const GinDevHandle& h, size_t off, float scale, float (&acc)[8], int& n) {
  if constexpr (BF16) {
    n = 8;
    if constexpr (NVLS) {
      bf16x8_to_f32(mc_ld_reduce_bf16x8(h.mc_window + off), acc);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int p = 0; p < h.nranks; ++p) {
        // start with the own rank and go round, so the ranks do not all hit the same peer at once
        const int peer = (h.rank + p) % h.nranks;
        float f[8];
        bf16x8_to_f32(*reinterpret_cast<const uint4*>(h.window[peer] + off), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
    }
  } else {
    n = 4;
    if constexpr (NVLS) {
      const uint4 r = mc_ld_reduce_f32x4(h.mc_window + off);
      acc[0] = __uint_as_float(r.x); acc[1] = __uint_as_float(r.y); acc[2] = __uint_as_float(r.z); acc[3] = __uint_as_float(r.w);
    } else {
      acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
      for (int p = 0; p < h.nranks; ++p) {
        const int peer = (h.rank + p) % h.nranks;
        const float4 f = *reinterpret_cast<const float4*>(h.window[peer] + off);
        acc[0] += f.x; acc[1] += f.y; acc[2] += f.z; acc[3] += f.w;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] *= scale;
}

template <bool BF16>
__device__ __forceinline__ uint4 pack_vec(const float (&acc)[8]) {
  if constexpr (BF16) return f32_to_bf16x8(acc);
  return make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
}

template <bool NVLS>
__device__ __forceinline__ void broadcast_vec(const GinDevHandle& h, size_t off, uint4 v) {
  if constexpr (NVLS) {
    mc_st_16(h.mc_window + off, v);
  } else {
    for (int p = 0; p < h.nranks; ++p) {
      const int peer = (h.rank + p) % h.nranks;
      *reinterpret_cast<uint4*>(h.window[peer] + off) = v;
    }
  }
}

// Register budget: with U = 4 the NVLS all-reduce needs 68 registers, so a 512-thread CTA of it and
// a 192-thread GEMM CTA (90 registers) fit one SM together and the gradient all-reduce really does
// overlap the backward GEMMs; U = 8 (96 registers) pushed the pair over the 64 K register file and
// the collective then waited for whole SMs.
// Walk vectors [v0, v1) of the window range starting at byte `off` with the whole grid, U vectors
// per thread per trip: the U reductions (multimem loads, or nranks peer loads each) are issued
// before any result is consumed, which keeps enough bytes in flight to cover the NVLink latency.
template <bool BF16, bool NVLS, int U, class Sink>
__device__ __forceinline__ void reduce_range(const GinDevHandle& h, size_t off, size_t v0, size_t v1, float scale,
                                             Sink&& sink) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t v = v0 + blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v < v1; v += stride * U) {
    float acc[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t idx = v + u * stride;
      int n;
      if (idx < v1) reduce_vec<BF16, NVLS>(h, off + (idx << 4), scale, acc[u], n);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t idx = v + u * stride;
      if (idx < v1) sink(idx, acc[u]);
    }
  }
}

// ---------------------------------------------------------------- all-reduce (in place in the window)
// Two-shot: rank r reduces slice r of the range and broadcasts the result to every rank.
template <bool BF16, bool NVLS>
__global__ void __launch_bounds__(512) all_reduce_kernel(GinDevHandle h, size_t off, size_t nvec, float scale,
                                                        int ch) {
  if (!gin_barrier(h, ch, blockIdx.x)) return;
  const size_t per = (nvec + h.nranks - 1) / h.nranks;
  const size_t v0 = min(nvec, per * h.rank);
  const size_t v1 = min(nvec, v0 + per);
  reduce_range<BF16, NVLS, NVLS ? 4 : 2>(h, off, v0, v1, scale, [&](size_t idx, const float(&acc)[8]) {
    broadcast_vec<NVLS>(h, off + (idx << 4), pack_vec<BF16>(acc));
  });
  gin_barrier(h, ch, blockIdx.x);
}

// One-shot (latency form): every rank reduces the whole range into a local output buffer. It
// cannot run in place, because a fast rank would overwrite inputs a slow rank still has to read.
template <bool BF16, bool NVLS>
__global__ void __launch_bounds__(512) all_reduce_oneshot_kernel(GinDevHandle h, size_t off, size_t nvec, float scale,
                                                                void* out, int ch) {
  if (!gin_barrier(h, ch, blockIdx.x)) return;
  reduce_range<BF16, NVLS, NVLS ? 4 : 2>(h, off, 0, nvec, scale, [&](size_t idx, const float(&acc)[8]) {
    reinterpret_cast<uint4*>(out)[idx] = pack_vec<BF16>(acc);
  });
  gin_barrier(h, ch, blockIdx.x);
}

// ---------------------------------------------------------------- reduce-scatter: out = scale * sum_r window_r[slice(rank)]
// OUT_MODE 0: same type as the input; 1: bf16 input -> fp32 output (gradient upcast fused in).
template <bool BF16, bool NVLS, int OUT_MODE>
__global__ void __launch_bounds__(512) reduce_scatter_kernel(GinDevHandle h, size_t off, size_t nvec_per_rank,
                                                            float scale, void* out, int ch) {
  if (!gin_barrier(h, ch, blockIdx.x)) return;
  const size_t base = off + ((nvec_per_rank * h.rank) << 4);
  reduce_range<BF16, NVLS, NVLS ? 4 : 2>(h, base, 0, nvec_per_rank, scale, [&](size_t idx, const float(&acc)[8]) {
    if constexpr (OUT_MODE == 1 && BF16) {
      float4* o = reinterpret_cast<float4*>(out) + 2 * idx;
      o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else {
      reinterpret_cast<uint4*>(out)[idx] = pack_vec<BF16>(acc);
    }
  });
  gin_barrier(h, ch, blockIdx.x);
}

// ---------------------------------------------------------------- all-gather: slice(rank) of the window -> every rank
template <bool NVLS>
__global__ void __launch_bounds__(512) all_gather_kernel(GinDevHandle h, size_t off, size_t nvec_per_rank, int ch) {
  if (!gin_barrier(h, ch, blockIdx.x)) return;
  const size_t base = off + ((nvec_per_rank * h.rank) << 4);
  constexpr int U = 4;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t v = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v < nvec_per_rank; v += stride * U) {
    uint4 val[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (v + u * stride < nvec_per_rank)
        val[u] = *reinterpret_cast<const uint4*>(h.window[h.rank] + base + ((v + u * stride) << 4));
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (v + u * stride >= nvec_per_rank) continue;
      const size_t o = base + ((v + u * stride) << 4);
      if constexpr (NVLS) {
        mc_st_16(h.mc_window + o, val[u]);
      } else {
        for (int p = 1; p < h.nranks; ++p) {
          const int peer = (h.rank + p) % h.nranks;
          *reinterpret_cast<uint4*>(h.window[peer] + o) = val[u];
        }
      }
    }
  }
  gin_barrier(h, ch, blockIdx.x);
}

// ---------------------------------------------------------------- all-to-all: send chunk p -> peer p's recv chunk `rank`
__global__ void __launch_bounds__(512) all_to_all_kernel(GinDevHandle h, size_t send_off, size_t recv_off,
                                                        size_t nvec_per_peer, int ch) {
  if (!gin_barrier(h, ch, blockIdx.x)) return;
  // gridDim.x is a multiple of nranks: block b serves destination (rank + 1 + b % nranks), so at any
  // moment the ranks target different peers
  const int per_peer = static_cast<int>(gridDim.x) / h.nranks;
  const int peer = (h.rank + 1 + static_cast<int>(blockIdx.x) % h.nranks) % h.nranks;
  const int sub = static_cast<int>(blockIdx.x) / h.nranks;
  const uint4* src = reinterpret_cast<const uint4*>(h.window[h.rank] + send_off) + nvec_per_peer * peer;
  uint4* dst = reinterpret_cast<uint4*>(h.window[peer] + recv_off) + nvec_per_peer * h.rank;
  constexpr int U = 4;
  const size_t stride = static_cast<size_t>(per_peer) * blockDim.x;
  for (size_t v = sub * static_cast<size_t>(blockDim.x) + threadIdx.x; v < nvec_per_peer; v += stride * U) {
    uint4 val[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (v + u * stride < nvec_per_peer) val[u] = src[v + u * stride];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (v + u * stride < nvec_per_peer) dst[v + u * stride] = val[u];
  }
  gin_barrier(h, ch, blockIdx.x);
}

// ---------------------------------------------------------------- barrier-only kernel
__global__ void barrier_kernel(GinDevHandle h, int ch) { gin_barrier(h, ch, blockIdx.x); }

// ---------------------------------------------------------------- GIN put+signal ping-pong between rank 0 and rank 1
// Rank 0 puts `bytes` to rank 1 and signals; rank 1 waits, puts back and signals; `iters` round
// trips. out_ns[0] = total device time of the loop on this rank.
__global__ void __launch_bounds__(256) gin_pingpong_kernel(GinDevHandle h, size_t off, size_t bytes, int iters,
                                                          int sig, unsigned long long* out_ns) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 1;
    gin_reset_signal(h, sig);
  }
  const int peer = h.rank ^ 1;
  if (!gin_barrier_pair(h, GIN_NUM_CHANNELS - 1, GIN_MAX_BLOCKS - 1, peer)) return;  // ranks 0 and 1 only
  const uint64_t t0 = globaltimer_ns();
  for (int i = 1; i <= iters && ok; ++i) {
    if (h.rank == 0) {
      gin_put_signal_cta(h, peer, off, h.window[h.rank] + off, bytes, sig, 1, GIN_SIGNAL_INC);
      if (threadIdx.x == 0 && !gin_wait_signal(h, sig, i)) ok = 0;
    } else {
      if (threadIdx.x == 0 && !gin_wait_signal(h, sig, i)) ok = 0;
      __syncthreads();
      if (ok) gin_put_signal_cta(h, peer, off, h.window[h.rank] + off, bytes, sig, 1, GIN_SIGNAL_INC);
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) out_ns[0] = globaltimer_ns() - t0;
}

// Waits on a signal nobody sets: exercises the bounded-wait path (status word gets the code).
__global__ void gin_wait_timeout_kernel(GinDevHandle h, int sig, unsigned long long* out) {
  gin_reset_signal(h, sig);
  const bool ok = gin_wait_signal(h, sig, 1);
  out[0] = ok ? 1ull : 0ull;
}

static int clamp_blocks(int nblocks) {
  if (nblocks <= 0) nblocks = 32;
  if (nblocks > GIN_MAX_BLOCKS) nblocks = GIN_MAX_BLOCKS;
  return nblocks;
}

}  // namespace b200

extern "C" {
using namespace b200;

// Register a communicator over an already mapped symmetric data window and control pad.
// window_base/pad_base: peer i at base + i*chunk. mc_window may be null (no NVLS).
int b200_comm_create(int rank, int nranks, void* window_base, size_t window_chunk, void* mc_window, void* pad_base,
                     size_t pad_chunk, unsigned long long wait_limit_ns, int* comm_out) {
  ensure_context();
  if (nranks < 1 || nranks > GIN_MAX_RANKS || rank < 0 || rank >= nranks || pad_chunk < GIN_PAD_BYTES)
    return B200_ERR_BAD_ARG;
  auto* c = new Comm();
  memset(&c->h, 0, sizeof(c->h));
  c->h.rank = rank;
  c->h.nranks = nranks;
  for (int i = 0; i < nranks; ++i) {
    c->h.window[i] = static_cast<uint8_t*>(window_base) + i * window_chunk;
    c->h.pad[i] = static_cast<uint8_t*>(pad_base) + i * pad_chunk;
  }
  c->h.mc_window = static_cast<uint8_t*>(mc_window);
  c->h.window_bytes = window_chunk;
  c->h.status = device_status_word();
  c->h.wait_limit_ns = wait_limit_ns ? wait_limit_ns : 10000000000ull;
  c->pad_bytes = pad_chunk;
  // the own pad starts zeroed (flags, epochs, signals, counters); peers do the same before the
  // host-side barrier that must follow this call
  B200_CUDA_OK(cudaMemset(c->h.pad[rank], 0, GIN_PAD_BYTES));
  B200_CUDA_OK(cudaDeviceSynchronize());
  std::lock_guard<std::mutex> g(g_comm_mu);
  g_comms.push_back(c);
  *comm_out = static_cast<int>(g_comms.size()) - 1;
  return 0;
}

int b200_comm_destroy(int comm) {
  std::lock_guard<std::mutex> g(g_comm_mu);
  if (comm < 0 || comm >= static_cast<int>(g_comms.size()) || !g_comms[comm]) return B200_ERR_BAD_ARG;
  delete g_comms[comm];
  g_comms[comm] = nullptr;
  return 0;
}

int b200_comm_set_wait_limit(int comm, unsigned long long ns) {
  std::lock_guard<std::mutex> g(g_comm_mu);
  if (comm < 0 || comm >= static_cast<int>(g_comms.size()) || !g_comms[comm]) return B200_ERR_BAD_ARG;
  g_comms[comm]->h.wait_limit_ns = ns;
  return 0;
}

#define GET_COMM(h, comm)                         \
  ensure_context();                               \
  const GinDevHandle* _hp = comm_handle(comm);    \
  if (!_hp) return B200_ERR_BAD_ARG;              \
  GinDevHandle h = *_hp;

// dtype: 0 = bf16, 1 = fp32. use_nvls: 1 = multimem path (needs mc_window). `bytes` multiple of 16.
int b200_all_reduce(int comm, size_t off, size_t bytes, int dtype, float scale, int use_nvls, int nblocks, int ch,
                    void* stream) {
  GET_COMM(h, comm);
  if ((off | bytes) & 15 || off + bytes > h.window_bytes || (use_nvls && !h.mc_window) || ch < 0 || ch >= GIN_NUM_CHANNELS)
    return B200_ERR_BAD_ARG;
  const size_t nvec = bytes >> 4;
  const int nb = clamp_blocks(nblocks);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0) {
    if (use_nvls) all_reduce_kernel<true, true><<<nb, 512, 0, s>>>(h, off, nvec, scale, ch);
    else all_reduce_kernel<true, false><<<nb, 512, 0, s>>>(h, off, nvec, scale, ch);
  } else {
    if (use_nvls) all_reduce_kernel<false, true><<<nb, 512, 0, s>>>(h, off, nvec, scale, ch);
    else all_reduce_kernel<false, false><<<nb, 512, 0, s>>>(h, off, nvec, scale, ch);
  }
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

// Latency form: every rank reduces the whole range into its own `out` (local memory, not the window).
int b200_all_reduce_oneshot(int comm, size_t off, size_t bytes, int dtype, float scale, int use_nvls, void* out,
                            int nblocks, int ch, void* stream) {
  GET_COMM(h, comm);
  if ((off | bytes) & 15 || off + bytes > h.window_bytes || (use_nvls && !h.mc_window) || !out) return B200_ERR_BAD_ARG;
  const size_t nvec = bytes >> 4;
  const int nb = clamp_blocks(nblocks);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0) {
    if (use_nvls) all_reduce_oneshot_kernel<true, true><<<nb, 512, 0, s>>>(h, off, nvec, scale, out, ch);
    else all_reduce_oneshot_kernel<true, false><<<nb, 512, 0, s>>>(h, off, nvec, scale, out, ch);
  } else {
    if (use_nvls) all_reduce_oneshot_kernel<false, true><<<nb, 512, 0, s>>>(h, off, nvec, scale, out, ch);
    else all_reduce_oneshot_kernel<false, false><<<nb, 512, 0, s>>>(h, off, nvec, scale, out, ch);
  }
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

// out (local) = scale * sum over ranks of the window slice [off + rank*bytes_per_rank, +bytes_per_rank).
// out_fp32 with dtype bf16 upcasts in the same pass.
int b200_reduce_scatter(int comm, size_t off, size_t bytes_per_rank, int dtype, float scale, int use_nvls, void* out,
                        int out_fp32, int nblocks, int ch, void* stream) {
  GET_COMM(h, comm);
  if ((off | bytes_per_rank) & 15 || off + bytes_per_rank * h.nranks > h.window_bytes || (use_nvls && !h.mc_window) || !out)
    return B200_ERR_BAD_ARG;
  const size_t nvec = bytes_per_rank >> 4;
  const int nb = clamp_blocks(nblocks);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0 && out_fp32) {
    if (use_nvls) reduce_scatter_kernel<true, true, 1><<<nb, 512, 0, s>>>(h, off, nvec, scale, out, ch);
    else reduce_scatter_kernel<true, false, 1><<<nb, 512, 0, s>>>(h, off, nvec, scale, out, ch);
  } else if (dtype == 0) {
    if (use_nvls) reduce_scatter_kernel<true, true, 0><<<nb, 512, 0, s>>>(h, off, nvec, scale, out, ch);
    else reduce_scatter_kernel<true, false, 0><<<nb, 512, 0, s>>>(h, off, nvec, scale, out, ch);
  } else {
    if (use_nvls) reduce_scatter_kernel<false, true, 0><<<nb, 512, 0, s>>>(h, off, nvec, scale, out, ch);
    else reduce_scatter_kernel<false, false, 0><<<nb, 512, 0, s>>>(h, off, nvec, scale, out, ch);
  }
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

int b200_all_gather(int comm, size_t off, size_t bytes_per_rank, int use_nvls, int nblocks, int ch, void* stream) {
  GET_COMM(h, comm);
  if ((off | bytes_per_rank) & 15 || off + bytes_per_rank * h.nranks > h.window_bytes || (use_nvls && !h.mc_window))
    return B200_ERR_BAD_ARG;
  const int nb = clamp_blocks(nblocks);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (use_nvls) all_gather_kernel<true><<<nb, 512, 0, s>>>(h, off, bytes_per_rank >> 4, ch);
  else all_gather_kernel<false><<<nb, 512, 0, s>>>(h, off, bytes_per_rank >> 4, ch);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

int b200_all_to_all(int comm, size_t send_off, size_t recv_off, size_t bytes_per_peer, int nblocks, int ch,
                    void* stream) {
  GET_COMM(h, comm);
  if ((send_off | recv_off | bytes_per_peer) & 15 || send_off + bytes_per_peer * h.nranks > h.window_bytes ||
      recv_off + bytes_per_peer * h.nranks > h.window_bytes)
    return B200_ERR_BAD_ARG;
  int nb = clamp_blocks(nblocks);
  nb = nb < h.nranks ? h.nranks : nb / h.nranks * h.nranks;
  all_to_all_kernel<<<nb, 512, 0, static_cast<cudaStream_t>(stream)>>>(h, send_off, recv_off, bytes_per_peer >> 4, ch);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

int b200_barrier(int comm, int ch, void* stream) {
  GET_COMM(h, comm);
  barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(h, ch);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

int b200_gin_pingpong(int comm, size_t off, size_t bytes, int iters, int sig, unsigned long long* out_ns_dev,
                      void* stream) {
  GET_COMM(h, comm);
  if (h.nranks < 2 || off + bytes > h.window_bytes || sig < 0 || sig >= GIN_MAX_SIGNALS) return B200_ERR_BAD_ARG;
  if (h.rank > 1) return 0;
  gin_pingpong_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(h, off, bytes, iters, sig, out_ns_dev);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

int b200_gin_wait_timeout_probe(int comm, int sig, unsigned long long* out_dev, void* stream) {
  GET_COMM(h, comm);
  gin_wait_timeout_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(h, sig, out_dev);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // extern "C"
