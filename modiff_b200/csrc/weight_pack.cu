// Per-output-channel asymmetric weight quantisation into the int8 weight-code layout.
//
// Arithmetic follows UniformAffineQuantizer with channel_wise=True, symmetric=False
// (qdiff/quant_layer.py:160-190 for delta / zero point, :94-102 for the codes): every
// operation is a single correctly-rounded fp32 operation in the same order, so the
// integer codes are identical to round(w / delta) + zp computed by PyTorch.
#include "common.cuh"

namespace modiff {

namespace {

__device__ inline float warp_min(float v) {
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ inline float warp_max(float v) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// One block per (output channel, segment).
__global__ void __launch_bounds__(256)
weight_pack_kernel(const float* __restrict__ w, const float* __restrict__ alpha,
                   const float* __restrict__ delta_in, const float* __restrict__ zp_in,
                   modiff_conv_geom g, Derived d, int n_bits,
                   int with_sum_rows, int8_t* __restrict__ wcodes, float* __restrict__ w_scale,
                   float* __restrict__ w_zp, int32_t* __restrict__ w_corr,
                   float* __restrict__ w_dq, int32_t* __restrict__ w_csum) {
  const int co = blockIdx.x;
  const int seg = blockIdx.y;
  const int cb = (seg == 0) ? 0 : g.split;
  const int ce = (d.nseg == 1 || seg == 1) ? g.cin : g.split;
  const int taps = d.taps;
  const int n = (ce - cb) * taps;
  const float* wrow = w + ((size_t)co * g.cin + cb) * taps;  // contiguous [ce-cb][taps]
  const float* arow = alpha ? alpha + ((size_t)co * g.cin + cb) * taps : nullptr;

  __shared__ float s_min[8], s_max[8];
  __shared__ float s_delta, s_zp;
  __shared__ int s_sum;
  if (threadIdx.x == 0) s_sum = 0;

  float mn = INFINITY, mx = -INFINITY;
  if (!delta_in) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      float v = wrow[i];
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
  }
  mn = warp_min(mn);
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) {
    s_min[threadIdx.x >> 5] = mn;
    s_max[threadIdx.x >> 5] = mx;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) {
      mn = fminf(mn, s_min[i]);
      mx = fmaxf(mx, s_max[i]);
    }
    const float n_levels = (float)(1 << n_bits);
    float delta = __fdiv_rn(__fsub_rn(mx, mn), __fsub_rn(n_levels, 1.0f));
    if (delta < 1e-8f) delta = 1e-8f;
    float zp = rintf(__fdiv_rn(-mn, delta));
    if (delta_in) {
      delta = delta_in[seg * g.cout + co];
      zp = zp_in[seg * g.cout + co];
    }
    s_delta = delta;
    s_zp = zp;
    int zpi = (int)zp;
    int zoff = (n_bits >= 8) ? 128 : min(max(zpi, 0), 127);
    w_scale[seg * g.cout + co] = delta;
    w_zp[seg * g.cout + co] = zp;
    w_corr[seg * g.cout + co] = zoff - zpi;
  }
  __syncthreads();
  const float delta = s_delta, zp = s_zp;
  const int zpi = (int)zp;
  const int zoff = (n_bits >= 8) ? 128 : min(max(zpi, 0), 127);
  const float qmax = (float)((1 << n_bits) - 1);
  const int row = with_sum_rows ? (co / 128) * 144 + (co % 128) : co;
  int8_t* crow = wcodes + (size_t)row * taps * d.kp;
  int centred_sum = 0;     // sum of q - zp over this (channel, segment): the factor of an
                           // activation-code offset in the layer's output
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int c = cb + i / taps;
    const int tap = i % taps;
    float v = wrow[i];
    float xi;
    if (arow) {   // learned rounding: floor plus the hard target
      xi = __fadd_rn(__fadd_rn(floorf(__fdiv_rn(v, delta)), arow[i] >= 0.0f ? 1.0f : 0.0f), zp);
    } else {
      xi = __fadd_rn(rintf(__fdiv_rn(v, delta)), zp);
    }
    float q = fminf(fmaxf(xi, 0.0f), qmax);
    crow[(size_t)tap * d.kp + c] = (int8_t)((int)q - zoff);
    centred_sum += (int)q - zpi;
    if (w_dq) {
      w_dq[((size_t)c * taps + tap) * g.cout + co] = __fmul_rn(__fsub_rn(q, zp), delta);
    }
  }
  if (w_csum) {
    for (int o = 16; o > 0; o >>= 1) centred_sum += __shfl_xor_sync(0xffffffffu, centred_sum, o);
    if ((threadIdx.x & 31) == 0) atomicAdd(&s_sum, centred_sum);
    __syncthreads();
    if (threadIdx.x == 0) w_csum[seg * g.cout + co] = s_sum;
  }
}

// Row 128 of every 144-row tile is all ones over the real input channels, so that the
// tensor-core kernel obtains the receptive-field sum of the activation codes as one
// more accumulator column.
__global__ void weight_sum_rows_kernel(int8_t* __restrict__ wcodes, modiff_conv_geom g, Derived d) {
  const int tile = blockIdx.x;
  int8_t* row = wcodes + ((size_t)tile * 144 + 128) * d.taps * d.kp;
  const int n = d.taps * d.kp;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int c = i % d.kp;
    row[i] = (c < g.cin) ? 1 : 0;
  }
}

}  // namespace
}  // namespace modiff

using namespace modiff;

extern "C" int modiff_weight_pack_rounded(const float* w, const float* alpha, const float* delta_in,
                                          const float* zp_in, const modiff_conv_geom* g, int n_bits,
                                          int with_sum_rows, int8_t* wcodes, float* w_scale,
                                          float* w_zp, int32_t* w_corr, float* w_dq,
                                          int32_t* w_csum, void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(w && wcodes && w_scale && w_zp && w_corr, "NULL pointer argument");
  MODIFF_CHECK_ARG((delta_in == nullptr) == (zp_in == nullptr),
                   "delta_in and zp_in must be given together");
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 8, "weight n_bits %d outside [2, 8]", n_bits);
  cudaStream_t s = (cudaStream_t)stream;
  Derived d = derive(*g);
  MODIFF_CUDA(cudaMemsetAsync(wcodes, 0, (size_t)modiff_wcodes_bytes(g, with_sum_rows), s));
  dim3 grid(g->cout, d.nseg);
  weight_pack_kernel<<<grid, 256, 0, s>>>(w, alpha, delta_in, zp_in, *g, d, n_bits, with_sum_rows,
                                          wcodes, w_scale, w_zp, w_corr, w_dq, w_csum);
  MODIFF_LAUNCH_CHECK("weight_pack_kernel");
  if (with_sum_rows) {
    weight_sum_rows_kernel<<<ceil_div(g->cout, 128), 256, 0, s>>>(wcodes, *g, d);
    MODIFF_LAUNCH_CHECK("weight_sum_rows_kernel");
  }
  return MODIFF_OK;
}

extern "C" int modiff_weight_pack(const float* w, const modiff_conv_geom* g, int n_bits,
                                  int with_sum_rows, int8_t* wcodes, float* w_scale, float* w_zp,
                                  int32_t* w_corr, float* w_dq, void* stream) {
  return modiff_weight_pack_rounded(w, nullptr, nullptr, nullptr, g, n_bits, with_sum_rows, wcodes,
                                    w_scale, w_zp, w_corr, w_dq, nullptr, stream);
}

// Stand-alone fake quantisation with learned (AdaRound) hard rounding, elementwise over a
// [rows][row_len] weight whose scale and zero point belong to the row:
//   out = (clamp(floor(w / delta[r]) + (alpha >= 0) + zp[r], 0, 2^b - 1) - zp[r]) * delta[r]
// (qdiff/adaptive_rounding.py:49-61 with soft_targets False; every step one rounded fp32
// operation, as the reference's tensor expression).
namespace modiff {
namespace {
__global__ void adaround_fake_quant_kernel(const float* __restrict__ w, const float* __restrict__ alpha,
                                           const float* __restrict__ delta, const float* __restrict__ zp,
                                           float* __restrict__ out, long long n, int row_len,
                                           int per_row, float top) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = per_row ? i / row_len : 0;
    const float d = delta[r], z = zp[r];
    const float up = alpha[i] >= 0.0f ? 1.0f : 0.0f;
    const float x_int = __fadd_rn(floorf(__fdiv_rn(w[i], d)), up);
    const float q = fminf(fmaxf(__fadd_rn(x_int, z), 0.0f), top);
    out[i] = __fmul_rn(__fsub_rn(q, z), d);
  }
}
}  // namespace
}  // namespace modiff

extern "C" int modiff_adaround_fake_quant(const float* w, const float* alpha, const float* delta,
                                          const float* zero_point, float* out, int64_t rows,
                                          int64_t row_len, int per_row, int n_bits, void* stream) {
  MODIFF_CHECK_ARG(w && alpha && delta && zero_point && out, "NULL pointer argument");
  MODIFF_CHECK_ARG(rows > 0 && row_len > 0 && row_len < (1ll << 31), "bad shape");
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 8, "weight n_bits %d outside [2, 8]", n_bits);
  const long long n = rows * row_len;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  modiff::adaround_fake_quant_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(
      w, alpha, delta, zero_point, out, n, (int)row_len, per_row, (float)((1 << n_bits) - 1));
  MODIFF_LAUNCH_CHECK("adaround_fake_quant_kernel");
  return MODIFF_OK;
}

// Packed 4-bit weights for modiff_igemm_conv_packed4: the packed-weight rows of
// modiff_weight_pack (int8 q - zero_point) become unsigned nibbles q, two per byte, element 2i in
// the low nibble of byte i (the nibble order of qdiff/quant_layer_int4.py:341-346).
namespace modiff {
namespace {
__global__ void pack_weights_int4_kernel(const int8_t* __restrict__ wcodes,
                                         const float* __restrict__ w_zp,
                                         uint8_t* __restrict__ packed, long long n_pairs,
                                         int row_pairs, int* __restrict__ bad) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_pairs;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / row_pairs;
    const int zp = (int)w_zp[r];
    const int a = (int)wcodes[2 * i] + zp, b = (int)wcodes[2 * i + 1] + zp;
    if ((a | b) & ~15) atomicExch(bad, 1);           // a code outside 0..15: not a 4-bit layer
    packed[i] = (uint8_t)((a & 15) | ((b & 15) << 4));
  }
}
}  // namespace
}  // namespace modiff

extern "C" int modiff_pack_weights_int4(const int8_t* wcodes, const float* w_zp, uint8_t* packed,
                                        int64_t rows, int64_t row_bytes, int* bad, void* stream) {
  MODIFF_CHECK_ARG(wcodes && w_zp && packed && bad, "NULL pointer argument");
  MODIFF_CHECK_ARG(rows > 0 && row_bytes > 0 && row_bytes % 2 == 0 && row_bytes < (1ll << 31),
                   "bad shape");
  const long long n = rows * row_bytes / 2;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  modiff::pack_weights_int4_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(
      wcodes, w_zp, packed, n, (int)(row_bytes / 2), bad);
  MODIFF_LAUNCH_CHECK("pack_weights_int4_kernel");
  return MODIFF_OK;
}
