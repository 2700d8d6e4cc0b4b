// Shared host/device helpers for libmodiff_b200.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "modiff_b200.h"

namespace modiff {

// Thread-local message buffer behind modiff_last_error().
char* error_buffer();
int set_error(int code, const char* fmt, ...);

#define MODIFF_CHECK_ARG(cond, ...)                                   \
  do {                                                                \
    if (!(cond)) return ::modiff::set_error(MODIFF_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define MODIFF_CUDA(call)                                                         \
  do {                                                                            \
    cudaError_t e__ = (call);                                                     \
    if (e__ != cudaSuccess)                                                       \
      return ::modiff::set_error(MODIFF_ERR_CUDA, "%s failed: %s (%s:%d)", #call, \
                                 cudaGetErrorString(e__), __FILE__, __LINE__);    \
  } while (0)

#define MODIFF_LAUNCH_CHECK(name)                                                 \
  do {                                                                            \
    cudaError_t e__ = cudaGetLastError();                                         \
    if (e__ != cudaSuccess)                                                       \
      return ::modiff::set_error(MODIFF_ERR_CUDA, "launch of %s failed: %s", name, \
                                 cudaGetErrorString(e__));                        \
  } while (0)

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ inline int round_up(int a, int b) { return ceil_div(a, b) * b; }

// Derived quantities of a layer geometry (host and device).
struct Derived {
  int ho, wo;        // output spatial size
  int hp, wp;        // code-plane rows / columns
  int cp;            // channels stored per code pixel (multiple of 16)
  int kp;            // weight K stride per tap (multiple of 128)
  int nplanes;       // stride * stride
  int taps;          // kh * kw
  int nseg;          // 1, or 2 with split
};

__host__ __device__ inline Derived derive(const modiff_conv_geom& g) {
  Derived d;
  d.ho = (g.h + g.pad_t + g.pad_b - g.kh) / g.stride + 1;
  d.wo = (g.w + g.pad_l + g.pad_r - g.kw) / g.stride + 1;
  d.hp = ceil_div(g.h + g.pad_t + g.pad_b, g.stride);
  d.wp = ceil_div(g.w + g.pad_l + g.pad_r, g.stride);
  d.cp = round_up(g.cin, 16);
  d.kp = round_up(g.cin, 128);
  d.nplanes = g.stride * g.stride;
  d.taps = g.kh * g.kw;
  d.nseg = g.split > 0 ? 2 : 1;
  return d;
}

int validate_geom(const modiff_conv_geom* g);

// Division of 0 <= x < 2^31 by a divisor fixed at launch: one wide multiply and a shift instead
// of the ~20-instruction software division.  m = floor(2^k / d) + 1 with k = 31 + ceil(log2 d)
// gives floor(x * m / 2^k) == floor(x / d) for every such x.
struct FastDiv {
  uint32_t d, m;
  int k;
  FastDiv() : d(1), m(0x80000001u), k(31) {}
  explicit FastDiv(int div) : d((uint32_t)div) {
    int s = 0;
    while ((1u << s) < d) ++s;
    k = 31 + s;
    m = (uint32_t)((((uint64_t)1) << k) / d + 1);
  }
  __host__ __device__ inline int div(int x) const {
    return (int)(((uint64_t)(uint32_t)x * m) >> k);
  }
  // quotient and remainder
  __host__ __device__ inline int divmod(int x, int& r) const {
    const int q = div(x);
    r = x - q * (int)d;
    return q;
  }
};

#ifdef __CUDACC__
// x * sigmoid(x), shared by every kernel that applies the UNet's nonlinearity, so that a value
// is the same wherever it is (re)computed.  Hardware exp2 / reciprocal: about 2 ulp, a few
// instructions (the quantiser kernels evaluate it twice per element and are otherwise
// memory-bound).
__device__ inline float silu_f(float y) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(y * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return y * r;   // five instructions; -0 for y far below zero
}
// GroupNorm affine step, one fused multiply-add everywhere it is evaluated.
__device__ inline float gn_apply(float v, float mean, float ga, float be) {
  return fmaf(v - mean, ga, be);
}
// Sum over the block; every thread gets the total.  `sh` holds 32 floats.
__device__ inline float block_sum(float v, float* sh) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (lane < nw) ? sh[lane] : 0.0f;
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}
// Two sums at once (each with exactly the operations of block_sum, so the same bits) for
// half the barriers.  `sh` holds 64 floats.
__device__ inline void block_sum2(float& a, float& b, float* sh) {
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) {
    sh[warp] = a;
    sh[32 + warp] = b;
  }
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  a = (lane < nw) ? sh[lane] : 0.0f;
  b = (lane < nw) ? sh[32 + lane] : 0.0f;
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
}
#endif

#ifdef __CUDACC__
// Raises a kernel's dynamic shared-memory limit to `bytes` on the CURRENT device, once per
// device and size (function attributes belong to a device; one SmemLimit per kernel).
struct SmemLimit {
  size_t done[64] = {};
};
template <typename K>
inline cudaError_t raise_smem_limit(K kernel, size_t bytes, SmemLimit& st) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (bytes > st.done[dev]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) st.done[dev] = bytes;
  }
  return e;
}
#endif

// Launch shape of the GroupNorm kernels for one (image, group) slab of `count` elements.  The
// statistics are summed per thread and then over the block, so two kernels agree on the last
// bit of mean and variance only when they use the same thread count.
// Slabs under 1024 elements are summed by ONE warp (no block barrier on the critical path).
inline int groupnorm_threads(int count) { return count >= 8192 ? 512 : (count >= 1024 ? 256 : 32); }
// log2(hw / 4) when hw / 4 is a power of two, else -1
inline int groupnorm_lg_hw4(int hw) {
  if (hw % 4 != 0) return -1;
  const int hw4 = hw / 4;
  if ((hw4 & (hw4 - 1)) != 0) return -1;
  int lg = 0;
  while ((1 << lg) < hw4) ++lg;
  return lg;
}

// LayerNorm of one row by one warp, the row held in registers: lane l owns the 16-byte chunks
// l, l + 32, ... (NV of them, c4 = c / 4 chunks in the row); sums run chunk by chunk, element by
// element, then a butterfly reduction.  Every kernel that normalises rows goes through these
// functions with the same NV, so they agree to the bit.
constexpr int kLnMaxChannels = 1280;
inline int ln_chunks_per_lane(int c) { return c <= 384 ? 3 : (c <= 640 ? 5 : 10); }

template <int NV>
__device__ inline void ln_row_load(const float* __restrict__ row, int c4, int lane, float4 (&v)[NV]) {
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int idx = lane + 32 * k;
    v[k] = idx < c4 ? __ldg(reinterpret_cast<const float4*>(row) + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}
template <int NV>
__device__ inline void ln_row_stats(const float4 (&v)[NV], int c4, int lane, float eps, float& mean,
                                    float& rstd) {
  const float n = (float)(4 * c4);
  float s = 0.0f;
#pragma unroll
  for (int k = 0; k < NV; ++k)
    if (lane + 32 * k < c4) { s += v[k].x; s += v[k].y; s += v[k].z; s += v[k].w; }
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  mean = s / n;
  float q = 0.0f;
#pragma unroll
  for (int k = 0; k < NV; ++k)
    if (lane + 32 * k < c4) {
      float d = v[k].x - mean; q += d * d;
      d = v[k].y - mean; q += d * d;
      d = v[k].z - mean; q += d * d;
      d = v[k].w - mean; q += d * d;
    }
  for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
  rstd = 1.0f / sqrtf(q / n + eps);
}
__device__ inline float ln_value(float x, float mean, float rstd, float gamma, float beta) {
  return fmaf((x - mean) * rstd, gamma, beta);
}
__device__ inline float4 ln_value4(float4 x, float mean, float rstd, float4 g, float4 b) {
  return make_float4(ln_value(x.x, mean, rstd, g.x, b.x), ln_value(x.y, mean, rstd, g.y, b.y),
                     ln_value(x.z, mean, rstd, g.z, b.z), ln_value(x.w, mean, rstd, g.w, b.w));
}

// GEGLU with the exact (erf) gelu: a * gelu(g) (ldm/modules/attention.py:37-44).  One function for
// every kernel that evaluates it, so they agree to the bit.
__device__ inline float geglu_value(float a, float g) {
  return a * (0.5f * g * (1.0f + erff(g * 0.70710678118654752440f)));
}

// Symmetric activation code range of an n-bit quantiser
// (n_levels = 2^(b-1) - 1; clamp(-n_levels - 1, n_levels)).
__host__ __device__ inline int sym_levels(int n_bits) { return (1 << (n_bits - 1)) - 1; }

}  // namespace modiff
