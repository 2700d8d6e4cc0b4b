// HBM-bound fp32 NCHW kernels of the UNet graph between the quantised layers:
// GroupNorm(+SiLU) with fused channel concat, SiLU, broadcast add, nearest 2x upsample,
// channel concat, sinusoidal timestep embedding, the DDIM update and int4 nibble packing.
// Reference: ddim/models/diffusion.py:6-52, 121-128, 345-357; ddim/functions/denoising.py:30-48;
// qdiff/quant_layer_int4.py:341-366 (nibble order).
#include "common.cuh"

namespace modiff {

namespace {

// One block per (image, group).  Sweeps over the group's elements: mean, centred variance and
// (unless only the statistics are wanted) normalise; sweeps 2 and 3 hit L1/L2.
// Input = channel concat [x0 | x1] plus an optional per-(image, channel) bias.
__global__ void __launch_bounds__(512)
groupnorm_silu_kernel(const float* __restrict__ x0, const float* __restrict__ x1, int c0,
                      const float* __restrict__ chan_bias, const float* __restrict__ film,
                      float* __restrict__ y, float* __restrict__ affine,
                      const float* __restrict__ gamma,
                      const float* __restrict__ beta, int c, int hw, int groups, float eps,
                      int silu, int lg_hw4) {
  __shared__ float sh[32];
  const int n = blockIdx.x / groups;
  const int grp = blockIdx.x % groups;
  const int cpg = c / groups;
  const int cbeg = grp * cpg;
  const int count = cpg * hw;
  const int c1 = c - c0;
  const bool vec = (hw % 4 == 0);

  auto src = [&](int ch) -> const float* {
    return (ch < c0) ? x0 + ((size_t)n * c0 + ch) * hw : x1 + ((size_t)n * c1 + (ch - c0)) * hw;
  };
  auto bias_of = [&](int ch) -> float { return chan_bias ? chan_bias[(size_t)n * c + ch] : 0.0f; };

  // One sweep: sums of (v - shift) and (v - shift)^2 with shift = the group's first element,
  // which keeps the variance free of cancellation when the mean is far from zero.
  const float shift = __fadd_rn(__ldg(src(cbeg)), bias_of(cbeg));
  float s = 0.0f, q = 0.0f;
  if (vec && lg_hw4 >= 0) {
    // flat sweep over the group, channel = i >> lg_hw4: no divisions, four loads in flight
    const int total4 = cpg << lg_hw4;
    const int mask = (1 << lg_hw4) - 1;
#pragma unroll 4
    for (int i = threadIdx.x; i < total4; i += blockDim.x) {
      const int ch = cbeg + (i >> lg_hw4);
      float4 v = __ldg(reinterpret_cast<const float4*>(src(ch)) + (i & mask));
      const float b = bias_of(ch);
      const float a = __fadd_rn(v.x, b) - shift, bb = __fadd_rn(v.y, b) - shift,
                  cc = __fadd_rn(v.z, b) - shift, dd = __fadd_rn(v.w, b) - shift;
      s += (a + bb) + (cc + dd);
      q += (a * a + bb * bb) + (cc * cc + dd * dd);
    }
  } else {
    for (int k = 0; k < cpg; ++k) {
      const int ch = cbeg + k;
      const float* sp = src(ch);
      const float b = bias_of(ch);
      for (int i = threadIdx.x; i < hw; i += blockDim.x) {
        const float a = __fadd_rn(__ldg(sp + i), b) - shift;
        s += a;
        q += a * a;
      }
    }
  }
  const float ms = block_sum(s, sh) / (float)count;          // mean - shift
  const float mean = shift + ms;
  const float var = fmaxf(block_sum(q, sh) / (float)count - ms * ms, 0.0f);
  const float rstd = 1.0f / sqrtf(var + eps);
  if (affine) {
    // per-(image, channel) scale / shift with the bias folded in:
    // gn(x + b) = x * (gamma*rstd) + (beta + (b - mean) * gamma*rstd)
    for (int k = threadIdx.x; k < cpg; k += blockDim.x) {
      const int ch = cbeg + k;
      float ga = gamma[ch] * rstd;
      float sh = fmaf(bias_of(ch) - mean, ga, beta[ch]);
      if (film) {   // gn(x) * (1 + scale) + shift
        const float f = 1.0f + film[(size_t)n * 2 * c + ch];
        ga *= f;
        sh = fmaf(sh, f, film[(size_t)n * 2 * c + c + ch]);
      }
      affine[2 * ((size_t)n * c + ch)] = ga;
      affine[2 * ((size_t)n * c + ch) + 1] = sh;
    }
  }
  if (!y) return;

  float* yn = y + (size_t)n * c * hw;
  if (vec) {
    const int hw4 = hw >> 2;
    for (int i = threadIdx.x; i < cpg * hw4; i += blockDim.x) {
      const int ch = cbeg + i / hw4;
      float4 v = __ldg(reinterpret_cast<const float4*>(src(ch)) + i % hw4);
      const float b = bias_of(ch);
      const float ga = gamma[ch] * rstd, be = beta[ch];
      float4 o;
      o.x = gn_apply(__fadd_rn(v.x, b), mean, ga, be);
      o.y = gn_apply(__fadd_rn(v.y, b), mean, ga, be);
      o.z = gn_apply(__fadd_rn(v.z, b), mean, ga, be);
      o.w = gn_apply(__fadd_rn(v.w, b), mean, ga, be);
      if (film) {
        const float f = 1.0f + film[(size_t)n * 2 * c + ch], sh = film[(size_t)n * 2 * c + c + ch];
        o.x = fmaf(o.x, f, sh); o.y = fmaf(o.y, f, sh); o.z = fmaf(o.z, f, sh); o.w = fmaf(o.w, f, sh);
      }
      if (silu) { o.x = silu_f(o.x); o.y = silu_f(o.y); o.z = silu_f(o.z); o.w = silu_f(o.w); }
      reinterpret_cast<float4*>(yn + (size_t)ch * hw)[i % hw4] = o;
    }
  } else {
    for (int i = threadIdx.x; i < count; i += blockDim.x) {
      const int ch = cbeg + i / hw;
      float o = gn_apply(__fadd_rn(__ldg(src(ch) + i % hw), bias_of(ch)), mean, gamma[ch] * rstd,
                         beta[ch]);
      if (film) o = fmaf(o, 1.0f + film[(size_t)n * 2 * c + ch], film[(size_t)n * 2 * c + c + ch]);
      if (silu) o = silu_f(o);
      yn[(size_t)ch * hw + i % hw] = o;
    }
  }
}

// Attention for small token counts (t, tk <= 64): one block per image, fp32 on CUDA cores.
// q [c][t], k [c][tk], v [c][tk], out [c][t]  (qdiff/quant_block.py:344-360).
__global__ void __launch_bounds__(256)
attention_small_kernel(const float* __restrict__ q, const float* __restrict__ k,
                       const float* __restrict__ v, float* __restrict__ out, int c, int t, int tk,
                       float scale) {
  __shared__ float sc[64][65];
  const int b = blockIdx.x;
  const float* qb = q + (size_t)b * c * t;
  const float* kb = k + (size_t)b * c * tk;
  const float* vb = v + (size_t)b * c * tk;
  for (int e = threadIdx.x; e < t * tk; e += blockDim.x) {
    const int i = e / tk, j = e % tk;
    float acc = 0.0f;
    for (int ch = 0; ch < c; ++ch) acc = fmaf(__ldg(qb + (size_t)ch * t + i), __ldg(kb + (size_t)ch * tk + j), acc);
    sc[i][j] = acc * scale;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < t; i += blockDim.x) {
    float mx = -INFINITY;
    for (int j = 0; j < tk; ++j) mx = fmaxf(mx, sc[i][j]);
    float sum = 0.0f;
    for (int j = 0; j < tk; ++j) { const float e = expf(sc[i][j] - mx); sc[i][j] = e; sum += e; }
    const float inv = 1.0f / sum;
    for (int j = 0; j < tk; ++j) sc[i][j] *= inv;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < c * t; e += blockDim.x) {
    const int ch = e / t, i = e % t;
    float acc = 0.0f;
    for (int j = 0; j < tk; ++j) acc = fmaf(__ldg(vb + (size_t)ch * tk + j), sc[i][j], acc);
    out[(size_t)b * c * t + e] = acc;
  }
}

// LayerNorm over the last dimension: one warp per row (ldm/modules/attention.py:229-231).  Rows of
// up to 1280 channels (a multiple of 4, 16-byte aligned) are held in registers (layernorm_kernel);
// anything else takes the scalar kernel.
template <int NV>
__global__ void __launch_bounds__(256)
layernorm_kernel(const float* __restrict__ x, float* __restrict__ y, const float* __restrict__ gamma,
                 const float* __restrict__ beta, int64_t rows, int c, float eps) {
  const int lane = threadIdx.x & 31;
  const int c4 = c >> 2;
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
       row += (int64_t)gridDim.x * (blockDim.x >> 5)) {
    float4 v[NV];
    ln_row_load<NV>(x + row * c, c4, lane, v);
    float mean, rstd;
    ln_row_stats<NV>(v, c4, lane, eps, mean, rstd);
    float4* yr = reinterpret_cast<float4*>(y + row * c);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int idx = lane + 32 * k;
      if (idx < c4)
        yr[idx] = ln_value4(v[k], mean, rstd, __ldg(reinterpret_cast<const float4*>(gamma) + idx),
                            __ldg(reinterpret_cast<const float4*>(beta) + idx));
    }
  }
}

__global__ void __launch_bounds__(256)
layernorm_scalar_kernel(const float* __restrict__ x, float* __restrict__ y,
                        const float* __restrict__ gamma, const float* __restrict__ beta, int64_t rows,
                        int c, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float* xr = x + row * c;
  float s = 0.0f;
  for (int i = lane; i < c; i += 32) s += xr[i];
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const float mean = s / (float)c;
  float q = 0.0f;
  for (int i = lane; i < c; i += 32) { const float d = xr[i] - mean; q += d * d; }
  for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
  const float rstd = 1.0f / sqrtf(q / (float)c + eps);
  float* yr = y + row * c;
  for (int i = lane; i < c; i += 32) yr[i] = ln_value(xr[i], mean, rstd, gamma[i], beta[i]);
}

// GEGLU: y[r][j] = x[r][j] * gelu(x[r][n + j]), exact (erf) gelu (ldm/modules/attention.py:37-44).
__global__ void geglu_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t rows, int n) {
  const int64_t total = rows * n;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const int64_t r = i / n;
    const int j = (int)(i % n);
    const float a = x[r * 2 * n + j], g = x[r * 2 * n + n + j];
    y[i] = geglu_value(a, g);
  }
}

// Batched 2-D transpose x[b][r][c] -> y[b][c][r] through a padded shared-memory tile.
__global__ void transpose_kernel(const float* __restrict__ x, float* __restrict__ y, int r, int c) {
  __shared__ float tile[32][33];
  const float* xb = x + (size_t)blockIdx.z * r * c;
  float* yb = y + (size_t)blockIdx.z * r * c;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int rr = r0 + i, cc = c0 + threadIdx.x;
    if (rr < r && cc < c) tile[i][threadIdx.x] = xb[(size_t)rr * c + cc];
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int cc = c0 + i, rr = r0 + threadIdx.x;
    if (rr < r && cc < c) yb[(size_t)cc * r + rr] = tile[threadIdx.x][i];
  }
}

__global__ void silu_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) y[i] = silu_f(x[i]);
}

__global__ void add_kernel(const float* __restrict__ a, const float* __restrict__ b,
                           float* __restrict__ out, int64_t n, int hw, int per_channel) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = __fadd_rn(a[i], per_channel ? b[i / hw] : b[i]);
}

__global__ void add4_kernel(const float4* __restrict__ a, const float4* __restrict__ b,
                            float4* __restrict__ out, int64_t n4) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n4; i += stride) {
    float4 u = a[i], v = b[i];
    out[i] = make_float4(__fadd_rn(u.x, v.x), __fadd_rn(u.y, v.y), __fadd_rn(u.z, v.z),
                         __fadd_rn(u.w, v.w));
  }
}

__global__ void upsample2x_kernel(const float* __restrict__ x, float* __restrict__ y,
                                  int64_t planes, int h, int w) {
  // one thread per input element, writes a 2x2 block
  const int64_t total = planes * h * w;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const int xx = (int)(i % w);
    const int yy = (int)((i / w) % h);
    const int64_t pl = i / ((int64_t)w * h);
    const float v = x[i];
    float* o = y + (pl * 2 * h + 2 * yy) * 2 * w + 2 * xx;
    *reinterpret_cast<float2*>(o) = make_float2(v, v);
    *reinterpret_cast<float2*>(o + 2 * w) = make_float2(v, v);
  }
}

__global__ void avgpool2x_kernel(const float* __restrict__ x, float* __restrict__ y,
                                 int64_t planes, int h, int w) {
  const int ho = h / 2, wo = w / 2;
  const int64_t total = planes * ho * wo;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const int xx = (int)(i % wo);
    const int yy = (int)((i / wo) % ho);
    const int64_t pl = i / ((int64_t)wo * ho);
    const float* p = x + (pl * h + 2 * yy) * w + 2 * xx;
    y[i] = (((p[0] + p[1]) + p[w]) + p[w + 1]) * 0.25f;
  }
}

__global__ void concat_c_kernel(const float* __restrict__ a, int64_t ea, const float* __restrict__ b,
                                int64_t eb, float* __restrict__ y, int64_t total) {
  // per image: ea elements of a followed by eb elements of b
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t per = ea + eb;
  for (; i < total; i += stride) {
    const int64_t n = i / per, r = i % per;
    y[i] = (r < ea) ? a[n * ea + r] : b[n * eb + (r - ea)];
  }
}

__global__ void timestep_embedding_kernel(const float* __restrict__ t,
                                          const float* __restrict__ freq,
                                          float* __restrict__ emb, int batch, int dim,
                                          int cos_first) {
  const int half = dim / 2;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= batch * dim) return;
  const int b = i / dim, j = i % dim;
  if (j >= 2 * half) { emb[i] = 0.0f; return; }  // odd dim: zero pad
  const int f = (j < half) ? j : j - half;
  const float arg = __fmul_rn(t[b], freq[f]);
  emb[i] = ((j < half) != (cos_first != 0)) ? sinf(arg) : cosf(arg);
}

__global__ void ddim_step_kernel(const float* __restrict__ x, const float* __restrict__ e,
                                 const float* __restrict__ noise, float* __restrict__ x_next,
                                 float* __restrict__ x0_out, int64_t n, float s1, float s2,
                                 float s3, float c1, float c2) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const float ev = e[i];
    const float x0 = __fdiv_rn(__fsub_rn(x[i], __fmul_rn(ev, s1)), s2);
    float acc = __fmul_rn(s3, x0);
    acc = __fadd_rn(acc, noise ? __fmul_rn(c1, noise[i]) : 0.0f);
    acc = __fadd_rn(acc, __fmul_rn(c2, ev));
    x_next[i] = acc;
    if (x0_out) x0_out[i] = x0;
  }
}

__global__ void cfg_combine_kernel(const float* __restrict__ eu, const float* __restrict__ ec,
                                   float* __restrict__ out, int64_t n, float scale) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride)
    out[i] = __fadd_rn(eu[i], __fmul_rn(scale, __fsub_rn(ec[i], eu[i])));
}

__global__ void pack_int4_kernel(const int8_t* __restrict__ codes, uint8_t* __restrict__ packed,
                                 int64_t n) {
  const int64_t nb = (n + 1) / 2;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < nb; i += stride) {
    const int lo = codes[2 * i] & 0xf;
    const int hi = (2 * i + 1 < n) ? (codes[2 * i + 1] & 0xf) : 0;
    packed[i] = (uint8_t)(lo | (hi << 4));
  }
}

__global__ void unpack_int4_kernel(const uint8_t* __restrict__ packed, int8_t* __restrict__ codes,
                                   int64_t n, int is_signed) {
  const int64_t nb = (n + 1) / 2;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < nb; i += stride) {
    const int v = packed[i];
    int lo = v & 0xf, hi = (v >> 4) & 0xf;
    if (is_signed) {
      if (lo > 7) lo -= 16;
      if (hi > 7) hi -= 16;
    }
    codes[2 * i] = (int8_t)lo;
    if (2 * i + 1 < n) codes[2 * i + 1] = (int8_t)hi;
  }
}

inline int grid_for(int64_t n, int block) {
  int64_t b = ceil_div64(n, block);
  const int64_t cap = 148 * 32;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace
}  // namespace modiff

using namespace modiff;

extern "C" {

int modiff_groupnorm_silu(const float* x0, const float* x1, int c0, const float* chan_bias,
                          const float* film, float* y, float* affine, const float* gamma,
                          const float* beta, int batch, int c, int hw, int groups, float eps,
                          int silu, void* stream) {
  MODIFF_CHECK_ARG(x0 && (y || affine) && gamma && beta, "NULL pointer argument");
  MODIFF_CHECK_ARG(batch > 0 && c > 0 && hw > 0 && groups > 0 && c % groups == 0,
                   "bad GroupNorm shape: c=%d groups=%d", c, groups);
  MODIFF_CHECK_ARG(c0 > 0 && c0 <= c && (c0 == c || x1 != nullptr), "bad concat split c0=%d", c0);
  MODIFF_CHECK_ARG((((uintptr_t)x0 | (uintptr_t)y | (uintptr_t)x1) & 15) == 0,
                   "GroupNorm tensors must be 16-byte aligned");
  const int count = (c / groups) * hw;
  const int threads = groupnorm_threads(count);
  const int lg_hw4 = groupnorm_lg_hw4(hw);
  groupnorm_silu_kernel<<<batch * groups, threads, 0, (cudaStream_t)stream>>>(
      x0, x1, c0, chan_bias, film, y, affine, gamma, beta, c, hw, groups, eps, silu, lg_hw4);
  MODIFF_LAUNCH_CHECK("groupnorm_silu_kernel");
  return MODIFF_OK;
}

int modiff_attention_small(const float* q, const float* k, const float* v, float* out, int batch,
                           int c, int t, int tk, float scale, void* stream) {
  MODIFF_CHECK_ARG(q && k && v && out && batch > 0 && c > 0, "bad argument");
  MODIFF_CHECK_ARG(t > 0 && tk > 0 && t <= 64 && tk <= 64, "token counts %d x %d exceed 64", t, tk);
  attention_small_kernel<<<batch, 256, 0, (cudaStream_t)stream>>>(q, k, v, out, c, t, tk, scale);
  MODIFF_LAUNCH_CHECK("attention_small_kernel");
  return MODIFF_OK;
}

int modiff_layernorm(const float* x, float* y, const float* gamma, const float* beta, int64_t rows,
                     int c, float eps, void* stream) {
  MODIFF_CHECK_ARG(x && y && gamma && beta && rows > 0 && c > 0, "bad argument");
  const int64_t blocks = ceil_div64(rows, 8);
  MODIFF_CHECK_ARG(blocks < (1ll << 31), "too many rows");
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec = c % 4 == 0 && c <= kLnMaxChannels &&
                   ((((uintptr_t)x | (uintptr_t)y | (uintptr_t)gamma | (uintptr_t)beta) & 15) == 0);
  if (vec) {
    const unsigned grid = (unsigned)(blocks < 148 * 8 ? blocks : 148 * 8);
    switch (ln_chunks_per_lane(c)) {
      case 3: layernorm_kernel<3><<<grid, 256, 0, s>>>(x, y, gamma, beta, rows, c, eps); break;
      case 5: layernorm_kernel<5><<<grid, 256, 0, s>>>(x, y, gamma, beta, rows, c, eps); break;
      default: layernorm_kernel<10><<<grid, 256, 0, s>>>(x, y, gamma, beta, rows, c, eps); break;
    }
  } else {
    layernorm_scalar_kernel<<<(unsigned)blocks, 256, 0, s>>>(x, y, gamma, beta, rows, c, eps);
  }
  MODIFF_LAUNCH_CHECK("layernorm_kernel");
  return MODIFF_OK;
}

int modiff_geglu(const float* x, float* y, int64_t rows, int n, void* stream) {
  MODIFF_CHECK_ARG(x && y && rows > 0 && n > 0, "bad argument");
  geglu_kernel<<<grid_for(rows * n, 256), 256, 0, (cudaStream_t)stream>>>(x, y, rows, n);
  MODIFF_LAUNCH_CHECK("geglu_kernel");
  return MODIFF_OK;
}

int modiff_transpose(const float* x, float* y, int batch, int r, int c, void* stream) {
  MODIFF_CHECK_ARG(x && y && batch > 0 && r > 0 && c > 0 && batch <= 65535, "bad argument");
  dim3 grid(ceil_div(c, 32), ceil_div(r, 32), batch);
  MODIFF_CHECK_ARG(grid.y <= 65535, "too many rows");
  transpose_kernel<<<grid, dim3(32, 8), 0, (cudaStream_t)stream>>>(x, y, r, c);
  MODIFF_LAUNCH_CHECK("transpose_kernel");
  return MODIFF_OK;
}

int modiff_silu(const float* x, float* y, int64_t n, void* stream) {
  MODIFF_CHECK_ARG(x && y && n >= 0, "bad argument");
  if (n == 0) return MODIFF_OK;
  silu_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(x, y, n);
  MODIFF_LAUNCH_CHECK("silu_kernel");
  return MODIFF_OK;
}

int modiff_add(const float* a, const float* b, float* out, int batch, int c, int hw,
               int b_per_channel, void* stream) {
  MODIFF_CHECK_ARG(a && b && out && batch > 0 && c > 0 && hw > 0, "bad argument");
  const int64_t n = (int64_t)batch * c * hw;
  const bool al = ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15) == 0) && (n % 4 == 0);
  if (!b_per_channel && al) {
    add4_kernel<<<grid_for(n / 4, 256), 256, 0, (cudaStream_t)stream>>>(
        (const float4*)a, (const float4*)b, (float4*)out, n / 4);
  } else {
    add_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(a, b, out, n, hw, b_per_channel);
  }
  MODIFF_LAUNCH_CHECK("add_kernel");
  return MODIFF_OK;
}

int modiff_upsample2x(const float* x, float* y, int batch, int c, int h, int w, void* stream) {
  MODIFF_CHECK_ARG(x && y && batch > 0 && c > 0 && h > 0 && w > 0, "bad argument");
  MODIFF_CHECK_ARG(((uintptr_t)y & 7) == 0, "output must be 8-byte aligned");
  const int64_t planes = (int64_t)batch * c;
  upsample2x_kernel<<<grid_for(planes * h * w, 256), 256, 0, (cudaStream_t)stream>>>(x, y, planes, h, w);
  MODIFF_LAUNCH_CHECK("upsample2x_kernel");
  return MODIFF_OK;
}

int modiff_avgpool2x(const float* x, float* y, int batch, int c, int h, int w, void* stream) {
  MODIFF_CHECK_ARG(x && y && batch > 0 && c > 0 && h >= 2 && w >= 2 && h % 2 == 0 && w % 2 == 0,
                   "bad argument");
  const int64_t planes = (int64_t)batch * c;
  avgpool2x_kernel<<<grid_for(planes * (h / 2) * (w / 2), 256), 256, 0, (cudaStream_t)stream>>>(
      x, y, planes, h, w);
  MODIFF_LAUNCH_CHECK("avgpool2x_kernel");
  return MODIFF_OK;
}

int modiff_concat_c(const float* a, int ca, const float* b, int cb, float* y, int batch, int hw,
                    void* stream) {
  MODIFF_CHECK_ARG(a && b && y && ca > 0 && cb > 0 && batch > 0 && hw > 0, "bad argument");
  const int64_t ea = (int64_t)ca * hw, eb = (int64_t)cb * hw;
  const int64_t total = (ea + eb) * batch;
  concat_c_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(a, ea, b, eb, y, total);
  MODIFF_LAUNCH_CHECK("concat_c_kernel");
  return MODIFF_OK;
}

int modiff_timestep_embedding(const float* t, const float* freq, float* emb, int batch, int dim,
                              int cos_first, void* stream) {
  MODIFF_CHECK_ARG(t && freq && emb && batch > 0 && dim >= 4, "bad argument");
  timestep_embedding_kernel<<<ceil_div(batch * dim, 256), 256, 0, (cudaStream_t)stream>>>(t, freq, emb, batch, dim, cos_first);
  MODIFF_LAUNCH_CHECK("timestep_embedding_kernel");
  return MODIFF_OK;
}

int modiff_ddim_step(const float* x, const float* e, const float* noise, float* x_next, float* x0,
                     int64_t n, float s1, float s2, float s3, float c1, float c2, void* stream) {
  MODIFF_CHECK_ARG(x && e && x_next && n > 0, "bad argument");
  ddim_step_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(x, e, noise, x_next, x0, n, s1,
                                                                      s2, s3, c1, c2);
  MODIFF_LAUNCH_CHECK("ddim_step_kernel");
  return MODIFF_OK;
}

int modiff_cfg_combine(const float* e_uncond, const float* e_cond, float* out, int64_t n,
                       float scale, void* stream) {
  MODIFF_CHECK_ARG(e_uncond && e_cond && out && n > 0, "bad argument");
  cfg_combine_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(e_uncond, e_cond, out, n,
                                                                        scale);
  MODIFF_LAUNCH_CHECK("cfg_combine_kernel");
  return MODIFF_OK;
}

int modiff_pack_int4(const int8_t* codes, uint8_t* packed, int64_t n, void* stream) {
  MODIFF_CHECK_ARG(codes && packed && n >= 0, "bad argument");
  if (n == 0) return MODIFF_OK;
  pack_int4_kernel<<<grid_for((n + 1) / 2, 256), 256, 0, (cudaStream_t)stream>>>(codes, packed, n);
  MODIFF_LAUNCH_CHECK("pack_int4_kernel");
  return MODIFF_OK;
}

int modiff_unpack_int4(const uint8_t* packed, int8_t* codes, int64_t n, int is_signed, void* stream) {
  MODIFF_CHECK_ARG(codes && packed && n >= 0, "bad argument");
  if (n == 0) return MODIFF_OK;
  unpack_int4_kernel<<<grid_for((n + 1) / 2, 256), 256, 0, (cudaStream_t)stream>>>(packed, codes, n,
                                                                                 is_signed);
  MODIFF_LAUNCH_CHECK("unpack_int4_kernel");
  return MODIFF_OK;
}

}  // extern "C"
