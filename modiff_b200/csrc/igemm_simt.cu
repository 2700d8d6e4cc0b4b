// CUDA-core (dp4a) int8 implicit-GEMM conv / linear with the modulation epilogue.
// Handles every geometry the C ABI accepts; the tensor-core kernel covers the hot
// shapes and this one covers the rest (3-channel input conv, odd sizes) and serves
// as the on-device cross-check of the tensor-core path.
//
// Reference arithmetic: F.conv2d(rq, wq) + o_hat with rq = codes * delta_x and
// wq = (q - zp) * delta_w[c] (qdiff/quant_layer.py:345-365).  Here the integer
// accumulator sum codes * (q - zp) is exact and is scaled once in the epilogue.
#include "common.cuh"

namespace modiff {

namespace {

constexpr int BM = 64, BN = 64, BK = 64;  // BK in bytes (int8 elements)
constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
igemm_simt_kernel(const int8_t* __restrict__ codes, const int8_t* __restrict__ wcodes,
                  int with_sum_rows, const float* __restrict__ x_scale,
                  const float* __restrict__ w_scale, const int32_t* __restrict__ w_corr,
                  float* __restrict__ o_hat, int accumulate, const float* __restrict__ bias,
                  modiff_conv_geom g, Derived d, int per_sample, int32_t* __restrict__ acc_out,
                  const float* __restrict__ x_zp, const int32_t* __restrict__ w_csum) {
  __shared__ uint32_t As[BM][BK / 4 + 1];
  __shared__ uint32_t Bs[BN][BK / 4 + 1];

  const int howo = d.ho * d.wo;
  const int M = g.batch * howo;
  const int m0 = blockIdx.x * BM;
  const int n0 = blockIdx.y * BN;
  const int tx = threadIdx.x & 15;
  const int ty = threadIdx.x >> 4;

  // loader role: one 16-byte piece of one row
  const int lrow = threadIdx.x >> 2;
  const int lpiece = threadIdx.x & 3;
  const int lm = m0 + lrow;
  int l_n = 0, l_ho = 0, l_wo = 0;
  const bool lm_valid = lm < M;
  if (lm_valid) {
    l_n = lm / howo;
    const int r = lm % howo;
    l_ho = r / d.wo;
    l_wo = r % d.wo;
  }
  const int lco = n0 + lrow;
  const bool lco_valid = lco < g.cout;
  const size_t wrow = with_sum_rows ? (size_t)(lco / 128) * 144 + (lco % 128) : (size_t)lco;

  float facc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) facc[i][j] = 0.0f;

  for (int seg = 0; seg < d.nseg; ++seg) {
    const int cb = (seg == 0) ? 0 : g.split;
    const int ce = (d.nseg == 1 || seg == 1) ? g.cin : g.split;
    int acc[4][4];
    int rsum[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      rsum[i] = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0;
    }
    for (int tap = 0; tap < d.taps; ++tap) {
      const int r = tap / g.kw, sx = tap % g.kw;
      const int plane = (r % g.stride) * g.stride + (sx % g.stride);
      const int dh = r / g.stride, dw = sx / g.stride;
      const int8_t* arow = nullptr;
      if (lm_valid) {
        const size_t pix = (((size_t)l_n * d.nplanes + plane) * d.hp + (l_ho + dh)) * d.wp + (l_wo + dw);
        arow = codes + pix * d.cp;
      }
      const int8_t* brow = wcodes + (wrow * d.taps + tap) * d.kp;
      for (int c0 = cb; c0 < ce; c0 += BK) {
        // ---- load tiles (16 bytes per thread per operand), zero outside [cb, ce)
        {
          const int c = c0 + 16 * lpiece;
          uint32_t va[4] = {0, 0, 0, 0}, vb[4] = {0, 0, 0, 0};
          if (c < ce) {
            const bool full = (c + 16 <= ce) && ((c & 15) == 0);
            if (lm_valid) {
              if (full) {
                int4 t = __ldg(reinterpret_cast<const int4*>(arow + c));
                va[0] = t.x; va[1] = t.y; va[2] = t.z; va[3] = t.w;
              } else {
                for (int b = 0; b < 16; ++b)
                  if (c + b < ce)
                    va[b >> 2] |= (uint32_t)(uint8_t)arow[c + b] << (8 * (b & 3));
              }
            }
            if (lco_valid) {
              if (full) {
                int4 t = __ldg(reinterpret_cast<const int4*>(brow + c));
                vb[0] = t.x; vb[1] = t.y; vb[2] = t.z; vb[3] = t.w;
              } else {
                for (int b = 0; b < 16; ++b)
                  if (c + b < ce)
                    vb[b >> 2] |= (uint32_t)(uint8_t)brow[c + b] << (8 * (b & 3));
              }
            }
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            As[lrow][4 * lpiece + k] = va[k];
            Bs[lrow][4 * lpiece + k] = vb[k];
          }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK / 4; ++kk) {
          int a[4], b[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) a[i] = (int)As[tx + 16 * i][kk];
#pragma unroll
          for (int j = 0; j < 4; ++j) b[j] = (int)Bs[ty * 4 + j][kk];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (w_corr) rsum[i] = __dp4a(a[i], 0x01010101, rsum[i]);
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = __dp4a(a[i], b[j], acc[i][j]);
          }
        }
        __syncthreads();
      }
    }
    // fold this segment into the fp32 result
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int co = n0 + ty * 4 + j;
      if (co >= g.cout) continue;
      const float ws = w_scale[seg * g.cout + co];
      const int corr = w_corr ? w_corr[seg * g.cout + co] : 0;
      // offset (8-bit asymmetric) activation codes: take (zp - 128) * sum(w) back out
      const int off = x_zp ? -((int)x_zp[seg] - 128) * w_csum[seg * g.cout + co] : 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = m0 + tx + 16 * i;
        if (m >= M) continue;
        const int a = acc[i][j] + corr * rsum[i] + off;
        const float xs = per_sample ? x_scale[m / howo] : x_scale[seg];
        facc[i][j] += (float)a * __fmul_rn(xs, ws);
        if (acc_out) acc_out[((size_t)seg * M + m) * g.cout + co] = a;
      }
    }
  }

#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int co = n0 + ty * 4 + j;
    if (co >= g.cout) continue;
    const float bv = bias ? bias[co] : 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = m0 + tx + 16 * i;
      if (m >= M) continue;
      const int n = m / howo, r = m % howo;
      const size_t idx = ((size_t)n * g.cout + co) * howo + r;
      float v = facc[i][j];
      if (accumulate) v += o_hat[idx];
      o_hat[idx] = v + bv;
    }
  }
}

}  // namespace

int launch_igemm_simt(const int8_t* codes, const int8_t* wcodes, int with_sum_rows,
                      const float* x_scale, const float* w_scale, const int32_t* w_corr,
                      float* o_hat, int accumulate, const float* bias, const modiff_conv_geom* g,
                      int per_sample, int32_t* acc_out, cudaStream_t s, const float* x_zp,
                      const int32_t* w_csum) {
  Derived d = derive(*g);
  const int M = g->batch * d.ho * d.wo;
  dim3 grid(ceil_div(M, BM), ceil_div(g->cout, BN));
  igemm_simt_kernel<<<grid, kThreads, 0, s>>>(codes, wcodes, with_sum_rows, x_scale, w_scale, w_corr,
                                              o_hat, accumulate, bias, *g, d, per_sample, acc_out,
                                              x_zp, w_csum);
  MODIFF_LAUNCH_CHECK("igemm_simt_kernel");
  return MODIFF_OK;
}

}  // namespace modiff
