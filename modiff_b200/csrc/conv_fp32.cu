// fp32 implicit-GEMM conv / linear on CUDA cores: the first sampling step, where the
// reference feeds UNQUANTISED activations through fake-quantised weights plus bias
// (qdiff/quant_layer.py:326-327, 358-359), and the weight-only / unquantised paths
// (:309-311, :364-365).  Plain IEEE fp32 multiply-add, no TF32.
#include "common.cuh"

namespace modiff {

namespace {

constexpr int BM = 128, BN = 64, BK = 8;
constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
conv_fp32_kernel(const float* __restrict__ x, const float* __restrict__ w_kn,
                 const float* __restrict__ bias, float* __restrict__ out, modiff_conv_geom g,
                 Derived d) {
  __shared__ float As[BK][BM];
  __shared__ float Bs[BK][BN];

  const int howo = d.ho * d.wo;
  const int M = g.batch * howo;
  const int K = g.cin * d.taps;
  const int m0 = blockIdx.x * BM;
  const int n0 = blockIdx.y * BN;
  const int tx = threadIdx.x & 15;   // along M
  const int ty = threadIdx.x >> 4;   // along N

  // A loader: column am (fixed per thread), rows ak0 + 2*i
  const int am = threadIdx.x & (BM - 1);
  const int ak0 = threadIdx.x >> 7;  // 0..1
  const int gm = m0 + am;
  const bool m_valid = gm < M;
  int a_n = 0, a_y = 0, a_x = 0;
  if (m_valid) {
    a_n = gm / howo;
    const int r = gm % howo;
    a_y = (r / d.wo) * g.stride - g.pad_t;
    a_x = (r % d.wo) * g.stride - g.pad_l;
  }
  const float* xn = x + (size_t)a_n * g.cin * g.h * g.w;
  // B loader: column bn, rows bk0 + 4*i
  const int bn = threadIdx.x & (BN - 1);
  const int bk0 = threadIdx.x >> 6;  // 0..3
  const bool n_valid = (n0 + bn) < g.cout;

  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < BK / 2; ++i) {
      const int kk = ak0 + 2 * i;
      const int k = k0 + kk;
      float v = 0.0f;
      if (m_valid && k < K) {
        const int c = k / d.taps;
        const int t = k % d.taps;
        const int yy = a_y + t / g.kw;
        const int xx = a_x + t % g.kw;
        if (yy >= 0 && yy < g.h && xx >= 0 && xx < g.w)
          v = __ldg(xn + ((size_t)c * g.h + yy) * g.w + xx);
      }
      As[kk][am] = v;
    }
#pragma unroll
    for (int i = 0; i < BK / 4; ++i) {
      const int kk = bk0 + 4 * i;
      const int k = k0 + kk;
      Bs[kk][bn] = (n_valid && k < K) ? __ldg(w_kn + (size_t)k * g.cout + n0 + bn) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[8], b[4];
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = As[kk][tx + 16 * i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][ty * 4 + j];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int co = n0 + ty * 4 + j;
    if (co >= g.cout) continue;
    const float bv = bias ? bias[co] : 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int m = m0 + tx + 16 * i;
      if (m >= M) continue;
      const int n = m / howo, r = m % howo;
      out[((size_t)n * g.cout + co) * howo + r] = acc[i][j] + bv;
    }
  }
}

}  // namespace
}  // namespace modiff

using namespace modiff;

extern "C" int modiff_conv_fp32(const float* x, const float* w_kn, const float* bias, float* out,
                                const modiff_conv_geom* g, void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(x && w_kn && out, "NULL pointer argument");
  Derived d = derive(*g);
  const int M = g->batch * d.ho * d.wo;
  dim3 grid(ceil_div(M, BM), ceil_div(g->cout, BN));
  conv_fp32_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(x, w_kn, bias, out, *g, d);
  MODIFF_LAUNCH_CHECK("conv_fp32_kernel");
  return MODIFF_OK;
}
