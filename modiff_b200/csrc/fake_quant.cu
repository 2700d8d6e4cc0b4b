// Stand-alone fake quantiser: y = (clamp(rne(x / delta) + zp) - zp) * delta with the scale
// rules of UniformAffineQuantizer (qdiff/quant_layer.py:70-111):
//   per-tensor 'max'  (:191-214): Python-float (double) arithmetic for delta / zero point,
//                                 min/max extended with 0 for the symmetric range;
//   per dim-0 slice   (:160-190): fp32 tensor arithmetic, raw min/max.
#include "common.cuh"

namespace modiff {

namespace {

// Order-preserving map float -> uint32 (and back) so that atomicMax works on signed floats.
__device__ inline unsigned int f2ord(float f) {
  unsigned int b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ inline float ord2f(unsigned int o) {
  return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
}

struct FqScratch {
  unsigned int counter;
  unsigned int pad[3];
  // per slice: [2*s] = ordered max, [2*s+1] = ~ordered min; zero means "unset"
  unsigned int mm[2];
};

constexpr int kThreads = 256;
constexpr int kChunk = 256 * 16;  // elements per block

__global__ void __launch_bounds__(kThreads)
fq_minmax_kernel(const float* __restrict__ x, int64_t slices, int64_t slice_len, int blocks_per_slice,
                 int n_bits, int symmetric, int always_zero, int channel_wise,
                 FqScratch* __restrict__ scratch, float* __restrict__ delta_out,
                 float* __restrict__ zp_out) {
  const int64_t s = blockIdx.x / blocks_per_slice;
  const int64_t b = blockIdx.x % blocks_per_slice;
  const float* xs = x + s * slice_len;
  const int64_t beg = b * kChunk;
  const int64_t end = (beg + kChunk < slice_len) ? beg + kChunk : slice_len;
  float mn = INFINITY, mx = -INFINITY;
  for (int64_t i = beg + threadIdx.x; i < end; i += kThreads) {
    const float v = __ldg(xs + i);
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  __shared__ float smn[kThreads / 32], smx[kThreads / 32];
  __shared__ bool is_last;
  if ((threadIdx.x & 31) == 0) {
    smn[threadIdx.x >> 5] = mn;
    smx[threadIdx.x >> 5] = mx;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < kThreads / 32; ++i) {
      mn = fminf(mn, smn[i]);
      mx = fmaxf(mx, smx[i]);
    }
    if (beg < end) {
      atomicMax(&scratch->mm[2 * s], f2ord(mx));
      atomicMax(&scratch->mm[2 * s + 1], ~f2ord(mn));
    }
    __threadfence();
    const unsigned int ticket = atomicAdd(&scratch->counter, 1u);
    is_last = (ticket == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int64_t i = threadIdx.x; i < slices; i += kThreads) {
    const float xmax = ord2f(atomicExch(&scratch->mm[2 * i], 0u));
    const float xmin = ord2f(~atomicExch(&scratch->mm[2 * i + 1], 0u));
    float delta, zp;
    if (!channel_wise) {
      const int n_levels = symmetric ? (1 << (n_bits - 1)) - 1 : (1 << n_bits);
      const double dmin = fmin((double)xmin, 0.0), dmax = fmax((double)xmax, 0.0);
      double d;
      if (symmetric) d = fmax(fabs(dmin), dmax) / (double)n_levels;
      else d = ((double)xmax - (double)xmin) / (double)(n_levels - 1);
      if (d < 1e-8) d = 1e-8;
      zp = (symmetric || always_zero) ? 0.0f : (float)rint(-(double)xmin / d);
      delta = (float)d;
    } else {
      const int n_levels = symmetric ? (1 << (n_bits - 1)) - 1 : (1 << n_bits);
      if (symmetric) delta = __fdiv_rn(fmaxf(fabsf(xmin), xmax), (float)n_levels);
      else delta = __fdiv_rn(__fsub_rn(xmax, xmin), (float)(n_levels - 1));
      if (delta < 1e-8f) delta = 1e-8f;
      zp = (symmetric || always_zero) ? 0.0f : rintf(__fdiv_rn(-xmin, delta));
    }
    delta_out[i] = delta;
    zp_out[i] = zp;
  }
  if (threadIdx.x == 0) scratch->counter = 0u;
}

__global__ void __launch_bounds__(kThreads)
fq_apply_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t slice_len,
                int blocks_per_slice, int n_bits, int symmetric, const float* __restrict__ delta,
                const float* __restrict__ zp) {
  const int64_t s = blockIdx.x / blocks_per_slice;
  const int64_t b = blockIdx.x % blocks_per_slice;
  const float d = delta[s], z = zp[s];
  const int n_levels = symmetric ? (1 << (n_bits - 1)) - 1 : (1 << n_bits);
  const float lo = symmetric ? (float)(-n_levels - 1) : 0.0f;
  const float hi = symmetric ? (float)n_levels : (float)(n_levels - 1);
  const int64_t beg = b * kChunk;
  const int64_t end = (beg + kChunk < slice_len) ? beg + kChunk : slice_len;
  for (int64_t i = beg + threadIdx.x; i < end; i += kThreads) {
    const float v = __ldg(x + s * slice_len + i);
    float q = __fadd_rn(rintf(__fdiv_rn(v, d)), z);
    q = fminf(fmaxf(q, lo), hi);
    y[s * slice_len + i] = __fmul_rn(__fsub_rn(q, z), d);
  }
}

}  // namespace
}  // namespace modiff

using namespace modiff;

extern "C" int modiff_fake_quant(const float* x, float* y, int64_t slices, int64_t slice_len,
                                 int n_bits, int symmetric, int always_zero, int channel_wise,
                                 int recompute, float* delta, float* zp, void* scratch,
                                 void* stream) {
  MODIFF_CHECK_ARG(x && y && delta && zp, "NULL pointer argument");
  MODIFF_CHECK_ARG(slices > 0 && slice_len > 0, "empty tensor");
  MODIFF_CHECK_ARG(channel_wise || slices == 1, "per-tensor mode takes exactly one slice");
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 16, "n_bits %d outside [2, 16]", n_bits);
  const int bps = (int)ceil_div64(slice_len, kChunk);
  MODIFF_CHECK_ARG(slices * bps < (1ll << 31), "tensor too large");
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned int grid = (unsigned int)(slices * bps);
  if (recompute) {
    MODIFF_CHECK_ARG(scratch != nullptr, "scratch is NULL");
    fq_minmax_kernel<<<grid, kThreads, 0, s>>>(x, slices, slice_len, bps, n_bits, symmetric,
                                               always_zero, channel_wise, (FqScratch*)scratch, delta, zp);
    MODIFF_LAUNCH_CHECK("fq_minmax_kernel");
  }
  fq_apply_kernel<<<grid, kThreads, 0, s>>>(x, y, slice_len, bps, n_bits, symmetric, delta, zp);
  MODIFF_LAUNCH_CHECK("fq_apply_kernel");
  return MODIFF_OK;
}
