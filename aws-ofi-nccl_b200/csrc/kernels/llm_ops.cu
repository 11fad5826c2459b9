// Memory-bound kernels of the Llama training step: RMSNorm (+residual), SwiGLU, RoPE, fused
// softmax-cross-entropy forward+backward, embedding gather/scatter, fused AdamW over flat buffers.
// All are bandwidth kernels: 16-byte vector accesses, one pass where the maths allows it.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_util.h"

namespace b200 {

using bf16 = __nv_bfloat16;
using bf162 = __nv_bfloat162;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : -INFINITY;
  if (w == 0) {
    t = warp_max(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

struct alignas(16) Bf16x8 {
  bf162 v[4];
};
__device__ __forceinline__ void unpack8(const Bf16x8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __low2float(p.v[i]);
    f[2 * i + 1] = __high2float(p.v[i]);
  }
}
__device__ __forceinline__ Bf16x8 pack8(const float (&f)[8]) {
  Bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

// ------------------------------------------------------------------ RMSNorm
// One CTA per row. If `res` is given: h = x + res is written to h_out (the new residual stream)
// and normalised in the same pass, so the residual add costs no extra pass.
constexpr int NORM_THREADS = 256;
template <int VEC_PER_THREAD>  // H = NORM_THREADS * 8 * VEC_PER_THREAD
__global__ void __launch_bounds__(NORM_THREADS)
    rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res, bf16* __restrict__ h_out,
                       const bf16* __restrict__ w, bf16* __restrict__ y, float* __restrict__ rstd, int H,
                       float eps) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const Bf16x8* xr = reinterpret_cast<const Bf16x8*>(x + row * H);
  Bf16x8* hr = reinterpret_cast<Bf16x8*>(h_out + row * H);
  const Bf16x8* rr = res ? reinterpret_cast<const Bf16x8*>(res + row * H) : nullptr;
  const Bf16x8* wr = reinterpret_cast<const Bf16x8*>(w);
  float vals[VEC_PER_THREAD][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VEC_PER_THREAD; ++i) {
    const int idx = threadIdx.x + i * NORM_THREADS;
    if (idx * 8 < H) {
      unpack8(xr[idx], vals[i]);
      if (rr) {
        float r[8];
        unpack8(rr[idx], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[i][j] += r[j];
        Bf16x8 h = pack8(vals[i]);
        hr[idx] = h;
        unpack8(h, vals[i]);  // normalise exactly what was stored
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
    }
  }
  ss = block_sum<NORM_THREADS>(ss, red);
  const float r = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
  Bf16x8* yr = reinterpret_cast<Bf16x8*>(y + row * H);
#pragma unroll
  for (int i = 0; i < VEC_PER_THREAD; ++i) {
    const int idx = threadIdx.x + i * NORM_THREADS;
    if (idx * 8 < H) {
      float wv[8], o[8];
      unpack8(wr[idx], wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * r * wv[j];
      yr[idx] = pack8(o);
    }
  }
}

// dx = rstd * (dy*w - x * rstd^2 * mean(dy*w*x)); optionally dx += dres (gradient arriving through
// the residual branch). Each CTA walks rows blockIdx.x, +gridDim.x, ... and keeps its slice of
// dw in registers, written once to `dw_partial[gridDim.x][H]`.
template <int VEC_PER_THREAD>
__global__ void __launch_bounds__(NORM_THREADS)
    rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                       const float* __restrict__ rstd, const bf16* __restrict__ dres, bf16* __restrict__ dx,
                       float* __restrict__ dw_partial, int T, int H) {
  __shared__ float red[32];
  float dw_acc[VEC_PER_THREAD][8];
#pragma unroll
  for (int i = 0; i < VEC_PER_THREAD; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[i][j] = 0.f;
  const Bf16x8* wr = reinterpret_cast<const Bf16x8*>(w);
  for (int64_t row = blockIdx.x; row < T; row += gridDim.x) {
    const Bf16x8* dyr = reinterpret_cast<const Bf16x8*>(dy + row * H);
    const Bf16x8* xr = reinterpret_cast<const Bf16x8*>(x + row * H);
    const float r = rstd[row];
    float g[VEC_PER_THREAD][8], xv[VEC_PER_THREAD][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VEC_PER_THREAD; ++i) {
      const int idx = threadIdx.x + i * NORM_THREADS;
      if (idx * 8 < H) {
        float d[8], wv[8];
        unpack8(dyr[idx], d);
        unpack8(xr[idx], xv[i]);
        unpack8(wr[idx], wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dw_acc[i][j] += d[j] * xv[i][j] * r;
          g[i][j] = d[j] * wv[j];
          dot += g[i][j] * xv[i][j];
        }
      }
    }
    dot = block_sum<NORM_THREADS>(dot, red);
    const float c = dot * r * r / H;
    Bf16x8* dxr = reinterpret_cast<Bf16x8*>(dx + row * H);
    const Bf16x8* drr = dres ? reinterpret_cast<const Bf16x8*>(dres + row * H) : nullptr;
#pragma unroll
    for (int i = 0; i < VEC_PER_THREAD; ++i) {
      const int idx = threadIdx.x + i * NORM_THREADS;
      if (idx * 8 < H) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = r * (g[i][j] - xv[i][j] * c);
        if (drr) {
          float e[8];
          unpack8(drr[idx], e);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += e[j];
        }
        dxr[idx] = pack8(o);
      }
    }
  }
  float* out = dw_partial + static_cast<int64_t>(blockIdx.x) * H;
#pragma unroll
  for (int i = 0; i < VEC_PER_THREAD; ++i) {
    const int idx = threadIdx.x + i * NORM_THREADS;
    if (idx * 8 < H) {
#pragma unroll
      for (int j = 0; j < 8; ++j) out[idx * 8 + j] = dw_acc[i][j];
    }
  }
}

// dw[h] (+)= sum over partial rows.
__global__ void colsum_partial_kernel(const float* __restrict__ partial, bf16* __restrict__ dw, int nrows, int H,
                                      int accumulate) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  float s = 0.f;
  for (int r = 0; r < nrows; ++r) s += partial[static_cast<int64_t>(r) * H + h];
  if (accumulate) s += __bfloat162float(dw[h]);
  dw[h] = __float2bfloat16(s);
}

// ------------------------------------------------------------------ SwiGLU on a fused [T, 2F] gate|up tensor
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int64_t T, int F) {
  const int64_t nvec = T * F / 8;
  const int fv = F / 8;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / fv;
    const int c = static_cast<int>(i - t * fv);
    const Bf16x8* row = reinterpret_cast<const Bf16x8*>(gu + t * 2 * F);
    float g[8], u[8], o[8];
    unpack8(row[c], g);
    unpack8(row[fv + c], u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    reinterpret_cast<Bf16x8*>(out + t * F)[c] = pack8(o);
  }
}
// dgu[T,2F] from dout[T,F] and the saved gate|up. INTERLEAVED: gate and up alternate in blocks of
// 32 columns (the layout the fused GEMM+SwiGLU epilogue produces) instead of two halves.
template <bool INTERLEAVED>
__global__ void swiglu_bwd_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ gu, bf16* __restrict__ dgu,
                                  int64_t T, int F) {
  const int64_t nvec = T * F / 8;
  const int fv = F / 8;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / fv;
    const int c = static_cast<int>(i - t * fv);
    const int gi = INTERLEAVED ? (c >> 2) * 8 + (c & 3) : c;       // in 8-element vectors
    const int ui = INTERLEAVED ? gi + 4 : fv + c;
    const Bf16x8* row = reinterpret_cast<const Bf16x8*>(gu + t * 2 * F);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(row[gi], g);
    unpack8(row[ui], u);
    unpack8(reinterpret_cast<const Bf16x8*>(dout + t * F)[c], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * s;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (s + silu * (1.f - s));
    }
    Bf16x8* orow = reinterpret_cast<Bf16x8*>(dgu + t * 2 * F);
    orow[gi] = pack8(dg);
    orow[ui] = pack8(du);
  }
}

// ------------------------------------------------------------------ RoPE (rotate-half convention), in place.
// x: [T, nheads, hd] with row pitch `pitch` elements between tokens; cos/sin: [T_pos, hd/2] fp32;
// position of token t is t % seq. sign = +1 forward, -1 backward (the inverse rotation).
__global__ void rope_kernel(bf16* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn, int64_t T,
                            int nheads, int hd, int64_t pitch, int seq, float sign) {
  const int half = hd / 2;
  const int64_t total = T * nheads * (half / 2);  // each thread rotates two adjacent pairs (bf162 loads)
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int p2 = static_cast<int>(i % (half / 2));
    const int64_t th = i / (half / 2);
    const int h = static_cast<int>(th % nheads);
    const int64_t t = th / nheads;
    const int pos = static_cast<int>(t % seq);
    bf16* base = x + t * pitch + static_cast<int64_t>(h) * hd;
    bf162* lo = reinterpret_cast<bf162*>(base) + p2;
    bf162* hi = reinterpret_cast<bf162*>(base + half) + p2;
    const float2 c = reinterpret_cast<const float2*>(cs + static_cast<int64_t>(pos) * half)[p2];
    float2 s = reinterpret_cast<const float2*>(sn + static_cast<int64_t>(pos) * half)[p2];
    s.x *= sign;
    s.y *= sign;
    const bf162 a = *lo, b = *hi;
    const float a0 = __low2float(a), a1 = __high2float(a), b0 = __low2float(b), b1 = __high2float(b);
    *lo = __floats2bfloat162_rn(a0 * c.x - b0 * s.x, a1 * c.y - b1 * s.y);
    *hi = __floats2bfloat162_rn(b0 * c.x + a0 * s.x, b1 * c.y + a1 * s.y);
  }
}

// ------------------------------------------------------------------ softmax cross-entropy, forward + backward fused
// One CTA per token row. Pass 1: online max/sum. Pass 2: overwrite the logits with
// dlogits = (softmax - onehot) * grad_scale. loss[row] = logsumexp - logit[target].
constexpr int CE_THREADS = 1024;
__global__ void __launch_bounds__(CE_THREADS)
    cross_entropy_fwd_bwd_kernel(bf16* __restrict__ logits, const int64_t* __restrict__ targets,
                                 float* __restrict__ loss, int V, int64_t ld, float grad_scale) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  bf16* lr = logits + row * ld;
  const int nvec = V / 8;
  const Bf16x8* lv = reinterpret_cast<const Bf16x8*>(lr);
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float f[8];
    unpack8(lv[i], f);
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    if (lm > m) {
      s *= __expf(m - lm);
      m = lm;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += CE_THREADS) {
    const float f = __bfloat162float(lr[i]);
    if (f > m) {
      s *= __expf(m - f);
      m = f;
    }
    s += __expf(f - m);
  }
  const float gm = block_max<CE_THREADS>(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum<CE_THREADS>(s, red);
  const int64_t tgt = targets[row];
  if (threadIdx.x == 0) {
    const float lt = (tgt >= 0 && tgt < V) ? __bfloat162float(lr[tgt]) : 0.f;
    loss[row] = (tgt >= 0 && tgt < V) ? (logf(gs) + gm - lt) : 0.f;
  }
  __syncthreads();
  const float inv = (tgt >= 0 && tgt < V) ? grad_scale / gs : 0.f;  // ignored rows get zero gradient
  const float gsc = (tgt >= 0 && tgt < V) ? grad_scale : 0.f;
  Bf16x8* ov = reinterpret_cast<Bf16x8*>(lr);
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float f[8];
    unpack8(ov[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      f[j] = __expf(f[j] - gm) * inv;
      if (i * 8 + j == tgt) f[j] -= gsc;
    }
    ov[i] = pack8(f);
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += CE_THREADS) {
    float f = __expf(__bfloat162float(lr[i]) - gm) * inv;
    if (i == tgt) f -= gsc;
    lr[i] = __float2bfloat16(f);
  }
}

// ------------------------------------------------------------------ embedding
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ ids, const bf16* __restrict__ table,
                                     bf16* __restrict__ out, int64_t T, int H) {
  const int hv = H / 8;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < T * hv;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / hv;
    const int c = static_cast<int>(i - t * hv);
    reinterpret_cast<Bf16x8*>(out + t * H)[c] = reinterpret_cast<const Bf16x8*>(table + ids[t] * H)[c];
  }
}
// dtable[ids[t]] += dout[t]  (bf16x2 atomics: repeated tokens accumulate)
__global__ void embedding_bwd_kernel(const int64_t* __restrict__ ids, const bf16* __restrict__ dout,
                                     bf16* __restrict__ dtable, int64_t T, int H) {
  const int hv = H / 2;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < T * hv;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / hv;
    const int c = static_cast<int>(i - t * hv);
    atomicAdd(reinterpret_cast<bf162*>(dtable + ids[t] * H) + c, reinterpret_cast<const bf162*>(dout + t * H)[c]);
  }
}

// ------------------------------------------------------------------ fused AdamW over flat buffers
// p (bf16) and g (bf16) are the model's flat parameter/gradient buffers; m, v (fp32) and the optional
// fp32 master copy are the optimizer state. One launch updates every parameter. The gradient is
// multiplied by grad_scale (loss scaling / clipping factor) on the way in and zeroed on the way out
// when zero_grad is set, so no separate memset pass is needed.
__global__ void adamw_kernel(bf16* __restrict__ p, bf16* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                             float* __restrict__ master, int64_t n, float lr, float beta1, float beta2, float eps,
                             float wd, float bc1, float bc2, float grad_scale, int zero_grad) {
  const int64_t nvec = n / 8;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float gf[8], pf[8];
    unpack8(reinterpret_cast<const Bf16x8*>(g)[i], gf);
    if (master) {
      const float4 a = reinterpret_cast<const float4*>(master)[2 * i], b = reinterpret_cast<const float4*>(master)[2 * i + 1];
      pf[0] = a.x; pf[1] = a.y; pf[2] = a.z; pf[3] = a.w; pf[4] = b.x; pf[5] = b.y; pf[6] = b.z; pf[7] = b.w;
    } else {
      unpack8(reinterpret_cast<const Bf16x8*>(p)[i], pf);
    }
    float4 m0 = reinterpret_cast<float4*>(m)[2 * i], m1 = reinterpret_cast<float4*>(m)[2 * i + 1];
    float4 v0 = reinterpret_cast<float4*>(v)[2 * i], v1 = reinterpret_cast<float4*>(v)[2 * i + 1];
    float mf[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vf[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gr = gf[j] * grad_scale;
      mf[j] = beta1 * mf[j] + (1.f - beta1) * gr;
      vf[j] = beta2 * vf[j] + (1.f - beta2) * gr * gr;
      const float mh = mf[j] / bc1, vh = vf[j] / bc2;
      pf[j] = pf[j] * (1.f - lr * wd) - lr * mh / (sqrtf(vh) + eps);
    }
    reinterpret_cast<float4*>(m)[2 * i] = make_float4(mf[0], mf[1], mf[2], mf[3]);
    reinterpret_cast<float4*>(m)[2 * i + 1] = make_float4(mf[4], mf[5], mf[6], mf[7]);
    reinterpret_cast<float4*>(v)[2 * i] = make_float4(vf[0], vf[1], vf[2], vf[3]);
    reinterpret_cast<float4*>(v)[2 * i + 1] = make_float4(vf[4], vf[5], vf[6], vf[7]);
    if (master) {
      reinterpret_cast<float4*>(master)[2 * i] = make_float4(pf[0], pf[1], pf[2], pf[3]);
      reinterpret_cast<float4*>(master)[2 * i + 1] = make_float4(pf[4], pf[5], pf[6], pf[7]);
    }
    reinterpret_cast<Bf16x8*>(p)[i] = pack8(pf);
    if (zero_grad) reinterpret_cast<uint4*>(g)[i] = make_uint4(0, 0, 0, 0);
  }
}

// sum of squares of a bf16 buffer -> out[0] (fp32 atomics; out must be zeroed by the caller)
__global__ void sumsq_kernel(const bf16* __restrict__ x, int64_t n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  const int64_t nvec = n / 8;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const Bf16x8*>(x)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += f[j] * f[j];
  }
  s = block_sum<256>(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

static inline int grid_for(int64_t work_items, int threads) {
  int64_t b = (work_items + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace b200

extern "C" {
using namespace b200;

int b200_rmsnorm_fwd(const void* x, const void* res, void* h_out, const void* w, void* y, float* rstd, int T, int H,
                     float eps, void* stream) {
  b200::ensure_context();
  if (H % 8 || H > NORM_THREADS * 8 * 4) return B200_ERR_BAD_ARG;
  if (res && !h_out) return B200_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int vpt = (H + NORM_THREADS * 8 - 1) / (NORM_THREADS * 8);
  auto X = static_cast<const bf16*>(x);
  auto R = static_cast<const bf16*>(res);
  auto HO = static_cast<bf16*>(h_out);
  auto W = static_cast<const bf16*>(w);
  auto Y = static_cast<bf16*>(y);
  switch (vpt) {
    case 1: rmsnorm_fwd_kernel<1><<<T, NORM_THREADS, 0, s>>>(X, R, HO, W, Y, rstd, H, eps); break;
    case 2: rmsnorm_fwd_kernel<2><<<T, NORM_THREADS, 0, s>>>(X, R, HO, W, Y, rstd, H, eps); break;
    case 3: rmsnorm_fwd_kernel<3><<<T, NORM_THREADS, 0, s>>>(X, R, HO, W, Y, rstd, H, eps); break;
    default: rmsnorm_fwd_kernel<4><<<T, NORM_THREADS, 0, s>>>(X, R, HO, W, Y, rstd, H, eps); break;
  }
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

// Number of fp32 rows the caller must provide in dw_partial.
int b200_rmsnorm_bwd_partial_rows() {
  b200::ensure_context(); return sm_count() * 2; }

int b200_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                     float* dw_partial, void* dw, int accumulate_dw, int T, int H, void* stream) {
  b200::ensure_context();
  if (H % 8 || H > NORM_THREADS * 8 * 4) return B200_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int vpt = (H + NORM_THREADS * 8 - 1) / (NORM_THREADS * 8);
  int grid = sm_count() * 2;
  if (grid > T) grid = T;
  auto DY = static_cast<const bf16*>(dy);
  auto X = static_cast<const bf16*>(x);
  auto W = static_cast<const bf16*>(w);
  auto DR = static_cast<const bf16*>(dres);
  auto DX = static_cast<bf16*>(dx);
  switch (vpt) {
    case 1: rmsnorm_bwd_kernel<1><<<grid, NORM_THREADS, 0, s>>>(DY, X, W, rstd, DR, DX, dw_partial, T, H); break;
    case 2: rmsnorm_bwd_kernel<2><<<grid, NORM_THREADS, 0, s>>>(DY, X, W, rstd, DR, DX, dw_partial, T, H); break;
    case 3: rmsnorm_bwd_kernel<3><<<grid, NORM_THREADS, 0, s>>>(DY, X, W, rstd, DR, DX, dw_partial, T, H); break;
    default: rmsnorm_bwd_kernel<4><<<grid, NORM_THREADS, 0, s>>>(DY, X, W, rstd, DR, DX, dw_partial, T, H); break;
  }
  colsum_partial_kernel<<<(H + 255) / 256, 256, 0, s>>>(dw_partial, static_cast<bf16*>(dw), grid, H, accumulate_dw);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

int b200_swiglu_fwd(const void* gu, void* out, long long T, int F, void* stream) {
  b200::ensure_context();
  if (F % 8) return B200_ERR_BAD_ARG;
  swiglu_fwd_kernel<<<grid_for(T * F / 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf16*>(gu), static_cast<bf16*>(out), T, F);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}
int b200_swiglu_bwd(const void* dout, const void* gu, void* dgu, long long T, int F, void* stream) {
  b200::ensure_context();
  if (F % 8) return B200_ERR_BAD_ARG;
  swiglu_bwd_kernel<false><<<grid_for(T * F / 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf16*>(dout), static_cast<const bf16*>(gu), static_cast<bf16*>(dgu), T, F);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}
int b200_swiglu_bwd_interleaved(const void* dout, const void* gu, void* dgu, long long T, int F, void* stream) {
  b200::ensure_context();
  if (F % 32) return B200_ERR_BAD_ARG;
  swiglu_bwd_kernel<true><<<grid_for(T * F / 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf16*>(dout), static_cast<const bf16*>(gu), static_cast<bf16*>(dgu), T, F);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

int b200_rope(void* x, const float* cs, const float* sn, long long T, int nheads, int hd, long long pitch, int seq,
              int backward, void* stream) {
  b200::ensure_context();
  if (hd % 4) return B200_ERR_BAD_ARG;
  rope_kernel<<<grid_for(T * nheads * (hd / 4), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<bf16*>(x), cs, sn, T, nheads, hd, pitch, seq, backward ? -1.f : 1.f);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

int b200_cross_entropy(void* logits, const long long* targets, float* loss, int T, int V, long long ld,
                       float grad_scale, void* stream) {
  b200::ensure_context();
  if (ld % 8) return B200_ERR_BAD_ARG;
  cross_entropy_fwd_bwd_kernel<<<T, CE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<bf16*>(logits), reinterpret_cast<const int64_t*>(targets), loss, V, ld, grad_scale);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

int b200_embedding_fwd(const long long* ids, const void* table, void* out, long long T, int H, void* stream) {
  b200::ensure_context();
  if (H % 8) return B200_ERR_BAD_ARG;
  embedding_fwd_kernel<<<grid_for(T * H / 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const int64_t*>(ids), static_cast<const bf16*>(table), static_cast<bf16*>(out), T, H);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}
int b200_embedding_bwd(const long long* ids, const void* dout, void* dtable, long long T, int H, void* stream) {
  b200::ensure_context();
  if (H % 2) return B200_ERR_BAD_ARG;
  embedding_bwd_kernel<<<grid_for(T * H / 2, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const int64_t*>(ids), static_cast<const bf16*>(dout), static_cast<bf16*>(dtable), T, H);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

int b200_adamw(void* p, void* g, float* m, float* v, float* master, long long n, float lr, float beta1, float beta2,
               float eps, float wd, int step, float grad_scale, int zero_grad, void* stream) {
  b200::ensure_context();
  if (n % 8) return B200_ERR_BAD_ARG;
  const float bc1 = 1.f - powf(beta1, static_cast<float>(step));
  const float bc2 = 1.f - powf(beta2, static_cast<float>(step));
  adamw_kernel<<<grid_for(n / 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<bf16*>(p), static_cast<bf16*>(g), m, v, master, n, lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale,
      zero_grad);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

int b200_sumsq(const void* x, long long n, float* out, void* stream) {
  b200::ensure_context();
  if (n % 8) return B200_ERR_BAD_ARG;
  sumsq_kernel<<<grid_for(n / 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const bf16*>(x), n, out);
  B200_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // extern "C"
