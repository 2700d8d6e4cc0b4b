// Modulated activation quantiser (two kernels on one stream):
//   1. modq_absmax_kernel : max |x - a_hat| per scale slot; the last block to finish
//                           turns it into delta (double division, as the reference's
//                           Python float arithmetic does) and re-zeroes the scratch;
//   2. modq_encode_kernel : codes = clamp(rne((x - a_hat) / delta)), a_hat += codes*delta,
//                           NCHW fp32 -> NHWC int8 code planes through a shared-memory
//                           transpose.
//
// Reference arithmetic: qdiff/quant_layer.py:329-336 (residual, cache update),
// :191-214 (per-tensor 'max' scale), :160-190 (per-sample scale), :94-102 (codes).
// Every floating-point step is an explicitly rounded single operation (no FMA
// contraction, true division) so codes and the cache are bit-identical to PyTorch.
#include "common.cuh"

#include <cstdlib>
#include <mutex>

namespace modiff {

namespace {

constexpr int kTileC = 64;   // channels per block
constexpr int kTileP = 64;   // pixels per block
constexpr int kThreads = 256;

struct ModqScratch {
  unsigned int counter;
  unsigned int pad[3];
  unsigned int absmax_bits[1];  // [slots]
};

template <bool VEC4>
__device__ inline void load4(const float* __restrict__ base, int p, int hw, float (&v)[4]) {
  if (VEC4) {
    float4 t = __ldg(reinterpret_cast<const float4*>(base + p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = (p + j < hw) ? __ldg(base + p + j) : 0.0f;
  }
}

template <bool VEC4>
__device__ inline void store4(float* __restrict__ base, int p, int hw, const float (&v)[4]) {
  if (VEC4) {
    *reinterpret_cast<float4*>(base + p) = make_float4(v[0], v[1], v[2], v[3]);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (p + j < hw) base[p + j] = v[j];
  }
}

// clamp(rne(t), lo, hi) for integer lo, hi with |lo|, |hi| < 2^22, without the conversion pipe:
// clamping first gives the same result (rne is monotonic and keeps integers), and adding
// 1.5 * 2^23 rounds to nearest-even at unit spacing.  The low byte of the sum's bit pattern is
// the two's-complement code.
__device__ inline float round_clamp(float t, float lo, float hi, uint32_t& bits) {
  const float u = __fadd_rn(fminf(fmaxf(t, lo), hi), 12582912.0f);
  bits = __float_as_uint(u);
  return __fadd_rn(u, -12582912.0f);
}
// clamp(rne(fl(r / delta)), lo, hi) with the division done as a multiplication by
// inv = rn(1 / delta) wherever that provably cannot change the result.  t = fl(r * inv) differs
// from the correctly rounded quotient by at most 1.5 * 2^-23 * |quotient| (one rounding each for
// inv, the product and the quotient itself), i.e. by less than 2^-14 wherever the clamp does
// not decide (|quotient| <= 256).  So unless t lies within 2^-14 of a tie both round to the same
// integer; the few elements that do (about one in 4000) take the true division.  Beyond the
// clamp range both saturate.
__device__ inline float quantise_clamp(float r, float delta, float inv, float lo, float hi,
                                       uint32_t& bits) {
  const float tc = fminf(fmaxf(__fmul_rn(r, inv), lo), hi);
  float u = __fadd_rn(tc, 12582912.0f);
  float qf = __fadd_rn(u, -12582912.0f);
  if (fabsf(__fsub_rn(tc, qf)) > 0.5f - 6.103515625e-5f) {
    const float te = fminf(fmaxf(__fdiv_rn(r, delta), lo), hi);
    u = __fadd_rn(te, 12582912.0f);
    qf = __fadd_rn(u, -12582912.0f);
  }
  bits = __float_as_uint(u);
  return qf;
}
// 8-bit asymmetric codes q in [0, 255] do not fit an int8 plane centred (q - zp spans 9 bits), so
// the planes hold q - 128 = (q - zp) + (zp - 128): this is the integer added to the centred
// code's bit pattern before its low byte is stored.  The convolution's epilogue takes the
// constant (zp - 128) * sum(w) back out (modiff_asym_bias).  Narrower codes stay centred.
__device__ inline uint32_t plane_shift(const float* x_zp, int slot, int n_levels) {
  return (x_zp && n_levels == 127) ? (uint32_t)((int)x_zp[slot] - 128) : 0u;
}
// low bytes of four words -> one word
__device__ inline uint32_t pack_low_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

// Device-side view of a modiff_act_source.
struct SrcView {
  const float* x0;
  const float* x1;
  const float* bias;
  const float* affine;
  int c0, c1, silu;
};

// Four consecutive pixels of channel c of image n, after the source transform.
template <bool VEC4, bool XFORM>
__device__ inline void load_src(const SrcView& s, int n, int c, int cin, int p, int hw,
                                float (&v)[4]) {
  if (!XFORM) {
    load4<VEC4>(s.x0 + ((size_t)n * cin + c) * hw, p, hw, v);
    return;
  }
  const float* base = (c < s.c0) ? s.x0 + ((size_t)n * s.c0 + c) * hw
                                 : s.x1 + ((size_t)n * s.c1 + (c - s.c0)) * hw;
  load4<VEC4>(base, p, hw, v);
  if (s.affine) {
    const float2 ab = __ldg(reinterpret_cast<const float2*>(s.affine) + (size_t)n * cin + c);
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = fmaf(v[j], ab.x, ab.y);
  } else if (s.bias) {
    const float b = __ldg(s.bias + (size_t)n * cin + c);
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __fadd_rn(v[j], b);
  }
  if (s.silu) {
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = silu_f(v[j]);
  }
}

// slot of channel c of image n: per-sample -> n; split -> segment; else 0
__device__ inline int slot_of(int n, int c, int split, int per_sample) {
  if (per_sample) return n;
  return (split > 0 && c >= split) ? 1 : 0;
}

struct TileGrid {
  int pb, cb, total;   // pixel blocks, channel blocks, pb * cb * batch
  FastDiv per_image;   // / (pb * cb)
  FastDiv by_pb;       // / pb
  FastDiv by_w;        // / g.w
  FastDiv by_stride;   // / g.stride
  // tile -> image, first channel, first pixel
  __device__ inline void decode(int tile, int& n, int& c0, int& p0) const {
    int rem;
    n = per_image.divmod(tile, rem);
    int pbi;
    const int cbi = by_pb.divmod(rem, pbi);
    c0 = cbi * kTileC;
    p0 = pbi * kTileP;
  }
};

template <bool VEC4, bool XFORM>
__global__ void __launch_bounds__(kThreads)
modq_absmax_kernel(const SrcView src, const float* __restrict__ a_hat,
                   modiff_conv_geom g, TileGrid tg, int n_levels, int per_sample, int slots,
                   ModqScratch* __restrict__ scratch, float* __restrict__ x_scale) {
  const int hw = g.h * g.w;
  const int cg = threadIdx.x >> 4;
  const int pq = threadIdx.x & 15;
  __shared__ float s0[kThreads / 32], s1[kThreads / 32];
  __shared__ bool is_last;

  float m0 = 0.0f, m1 = 0.0f;
  int cur_n = -1;
  // Each block walks a strided list of tiles and publishes one maximum per scale slot, so the
  // number of same-address atomics is bounded by the grid size, not by the tensor size.
  for (int tile = blockIdx.x; tile < tg.total; tile += gridDim.x) {
    int n, c0, p0;
    tg.decode(tile, n, c0, p0);
    const int p = p0 + 4 * pq;
    if (per_sample && n != cur_n) {
      // flush the running maximum of the previous image
      if (cur_n >= 0) {
        float v = m0;
        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
        if ((threadIdx.x & 31) == 0 && v > 0.0f)
          atomicMax(&scratch->absmax_bits[cur_n], __float_as_uint(v));
      }
      m0 = 0.0f;
      cur_n = n;
    }
    if (p < hw) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = c0 + 4 * cg + i;
        if (c < g.cin) {
          const size_t off = ((size_t)n * g.cin + c) * hw;
          float xv[4], av[4] = {0.f, 0.f, 0.f, 0.f};
          load_src<VEC4, XFORM>(src, n, c, g.cin, p, hw, xv);
          if (a_hat) load4<VEC4>(a_hat + off, p, hw, av);
          float m = 0.0f;
#pragma unroll
          for (int j = 0; j < 4; ++j) m = fmaxf(m, fabsf(__fsub_rn(xv[j], av[j])));
          if (g.split > 0 && c >= g.split) m1 = fmaxf(m1, m); else m0 = fmaxf(m0, m);
        }
      }
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, o));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, o));
  }
  if ((threadIdx.x & 31) == 0) {
    s0[threadIdx.x >> 5] = m0;
    s1[threadIdx.x >> 5] = m1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < kThreads / 32; ++i) {
      m0 = fmaxf(m0, s0[i]);
      m1 = fmaxf(m1, s1[i]);
    }
    // Non-negative floats order like their bit patterns.
    const int slot0 = per_sample ? (cur_n < 0 ? 0 : cur_n) : 0;
    if (m0 > 0.0f) atomicMax(&scratch->absmax_bits[slot0], __float_as_uint(m0));
    if (g.split > 0 && m1 > 0.0f) atomicMax(&scratch->absmax_bits[1], __float_as_uint(m1));
    __threadfence();
    const unsigned int ticket = atomicAdd(&scratch->counter, 1u);
    is_last = (ticket == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    __threadfence();
    for (int s = threadIdx.x; s < slots; s += blockDim.x) {
      const unsigned int bits = atomicExch(&scratch->absmax_bits[s], 0u);
      // delta = x_absmax / n_levels in Python floats (doubles), floor 1e-8, then cast
      // to fp32 by torch.tensor(delta).type_as(x).
      double delta = (double)__uint_as_float(bits) / (double)n_levels;
      if (delta < 1e-8) delta = 1e-8;
      x_scale[s] = (float)delta;
    }
    if (threadIdx.x == 0) scratch->counter = 0u;
  }
}

// UP2: the layer's input is the nearest-neighbour 2x upsample of `src` (g is the convolution's
// geometry at the doubled size, stride 1).  Input, cache and residual then repeat every value in
// 2x2 blocks, so the quantiser works at the source resolution and writes each code four times.
template <bool VEC4, bool XFORM, bool UP2 = false>
__global__ void __launch_bounds__(kThreads)
modq_encode_kernel(const SrcView src, float* __restrict__ a_hat,
                   int8_t* __restrict__ codes, const float* __restrict__ x_scale,
                   const float* __restrict__ x_zp, modiff_conv_geom g, Derived d, TileGrid tg,
                   int n_levels, int per_sample) {
  __shared__ uint32_t tile_sh[kTileP][kTileC / 4 + 1];
  const int hw = UP2 ? (g.h >> 1) * (g.w >> 1) : g.h * g.w;
  const int cg = threadIdx.x >> 4;
  const int pq = threadIdx.x & 15;
  const float lo = (float)(-n_levels - 1), hi = (float)n_levels;

  // Tiles are visited in the REVERSE of the absmax kernel's order: what that pass touched
  // last is still in L2 and is consumed first.
  for (int it = blockIdx.x; it < tg.total; it += gridDim.x) {
    const int tile = tg.total - 1 - it;
    int n, c0, p0;
    tg.decode(tile, n, c0, p0);
    const int p = p0 + 4 * pq;

    uint32_t q[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) q[i][j] = 0;

    if (p < hw) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = c0 + 4 * cg + i;
        if (c < g.cin) {
          const int slot = slot_of(n, c, g.split, per_sample);
          const float delta = x_scale[slot];
          // asymmetric codes: centred range [-zp, 2^b - 1 - zp]
          const float lo_s = x_zp ? -x_zp[slot] : lo;
          const float hi_s = x_zp ? (float)(2 * n_levels + 1) - x_zp[slot] : hi;
          const uint32_t zshift = plane_shift(x_zp, slot, n_levels);
          const size_t off = ((size_t)n * g.cin + c) * hw;
          float xv[4], av[4] = {0.f, 0.f, 0.f, 0.f}, nv[4];
          load_src<VEC4, XFORM>(src, n, c, g.cin, p, hw, xv);
          if (a_hat) load4<VEC4>(a_hat + off, p, hw, av);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float r = __fsub_rn(xv[j], av[j]);
            const float qf = round_clamp(__fdiv_rn(r, delta), lo_s, hi_s, q[i][j]);
            q[i][j] += zshift;
            nv[j] = __fadd_rn(av[j], __fmul_rn(qf, delta));
          }
          if (a_hat) store4<VEC4>(a_hat + off, p, hw, nv);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      tile_sh[4 * pq + j][cg] = pack_low_bytes(q[0][j], q[1][j], q[2][j], q[3][j]);
    }
    __syncthreads();
    // 4 threads per pixel, 16 bytes each.
    const int px = threadIdx.x >> 2;
    const int piece = threadIdx.x & 3;
    const int pp = p0 + px;
    const int cbase = c0 + 16 * piece;
    if (pp < hw && cbase < d.cp) {
      int y, xq, ys, xs;
      y = tg.by_w.divmod(pp, xq);          // UP2: by_w divides by the source width
      int4 v = make_int4(tile_sh[px][4 * piece], tile_sh[px][4 * piece + 1],
                         tile_sh[px][4 * piece + 2], tile_sh[px][4 * piece + 3]);
      if (UP2) {
#pragma unroll
        for (int dy = 0; dy < 2; ++dy)
#pragma unroll
          for (int dx = 0; dx < 2; ++dx) {
            const size_t pix = ((size_t)n * d.hp + (2 * y + dy + g.pad_t)) * d.wp +
                               (2 * xq + dx + g.pad_l);
            *reinterpret_cast<int4*>(codes + pix * d.cp + cbase) = v;
          }
      } else {
        const int yq = tg.by_stride.divmod(y + g.pad_t, ys);
        const int xqq = tg.by_stride.divmod(xq + g.pad_l, xs);
        const int plane = ys * g.stride + xs;
        const size_t pix = (((size_t)n * d.nplanes + plane) * d.hp + yq) * d.wp + xqq;
        *reinterpret_cast<int4*>(codes + pix * d.cp + cbase) = v;
      }
    }
    __syncthreads();
  }
}

// Encode pass with its inputs staged through shared memory by cp.async: the x and a_hat tiles
// of the NEXT tile are in flight while the current one is quantised, so the bytes in flight do
// not depend on how many registers or warps the arithmetic needs.  Same arithmetic, tile order
// and outputs as modq_encode_kernel<true, XFORM>.
constexpr int kStages = 2;
constexpr int kStageFloats = 2 * kTileC * kTileP;              // x tile | a_hat tile
constexpr int kStagedSmem = kStages * kStageFloats * 4;        // bytes of dynamic shared memory

template <bool XFORM>
__global__ void __launch_bounds__(kThreads)
modq_encode_staged_kernel(const SrcView src, float* __restrict__ a_hat,
                          int8_t* __restrict__ codes, const float* __restrict__ x_scale,
                          const float* __restrict__ x_zp, modiff_conv_geom g, Derived d,
                          TileGrid tg, int n_levels, int per_sample) {
  extern __shared__ __align__(16) float stage_sh[];
  __shared__ uint32_t tile_sh[kTileP][kTileC / 4 + 1];
  const int hw = g.h * g.w;
  const int cg = threadIdx.x >> 4;
  const int pq = threadIdx.x & 15;
  const float lo = (float)(-n_levels - 1), hi = (float)n_levels;
  // One thread moves the same 16-byte column of four rows (16 rows apart) of both tensors:
  // per-image base pointers once per tile, 32-bit offsets inside the image.
  const int lrow = threadIdx.x >> 4, lcol = (threadIdx.x & 15) * 4;
  const uint32_t sdst0 =
      (uint32_t)__cvta_generic_to_shared(stage_sh) + (uint32_t)(lrow * kTileP + lcol) * 4u;
  auto issue = [&](int it, int stage) {
    const int tile = tg.total - 1 - it;
    int n, c0, p0;
    tg.decode(tile, n, c0, p0);
    const int p = p0 + lcol;
    const float* xb0 = XFORM ? src.x0 + (size_t)n * src.c0 * hw : src.x0 + (size_t)n * g.cin * hw;
    const float* xb1 = XFORM && src.x1 ? src.x1 + (size_t)n * src.c1 * hw : xb0;
    const float* ab = a_hat ? a_hat + (size_t)n * g.cin * hw : nullptr;
    const int split_c = XFORM ? src.c0 : g.cin;
    const uint32_t sdst = sdst0 + (uint32_t)(stage * kStageFloats) * 4u;
#pragma unroll
    for (int r = 0; r < (kTileC * kTileP / 4) / kThreads; ++r) {
      const int c = c0 + lrow + 16 * r;
      const bool valid = (c < g.cin) && (p < hw);
      const int bytes = valid ? 16 : 0;     // 0: the 16 bytes are zero-filled, nothing is read
      const float* xp = xb0;
      if (valid) xp = (c < split_c) ? xb0 + (c * hw + p) : xb1 + ((c - split_c) * hw + p);
      const uint32_t d = sdst + (uint32_t)(16 * r * kTileP) * 4u;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(xp), "r"(bytes)
                   : "memory");
      if (a_hat) {
        const float* ap = valid ? ab + (c * hw + p) : ab;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(
                         d + (uint32_t)(kTileC * kTileP) * 4u),
                     "l"(ap), "r"(bytes)
                     : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  int k = 0;
  if ((int)blockIdx.x < tg.total) issue(blockIdx.x, 0);
  for (int it = blockIdx.x; it < tg.total; it += gridDim.x, ++k) {
    const int stage = k % kStages;
    if (it + (int)gridDim.x < tg.total) {
      issue(it + gridDim.x, (k + 1) % kStages);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();

    const int tile = tg.total - 1 - it;
    int n, c0, p0;
    tg.decode(tile, n, c0, p0);
    const int p = p0 + 4 * pq;
    const float* sx = stage_sh + stage * kStageFloats;
    const float* sa = sx + kTileC * kTileP;
    const size_t img = (size_t)n * g.cin;          // first (image, channel) row of this image
    const bool one_scale = !per_sample && g.split == 0;
    const float delta0 = x_scale[per_sample ? n : 0];
    const float delta1 = one_scale || per_sample ? delta0 : x_scale[1];
    const float inv0 = __frcp_rn(delta0), inv1 = __frcp_rn(delta1);
    // asymmetric codes: centred range [-zp, 2^b - 1 - zp] per scale slot
    const float zp0 = x_zp ? x_zp[per_sample ? n : 0] : 0.0f;
    const float zp1 = (x_zp && !(one_scale || per_sample)) ? x_zp[1] : zp0;
    const float top = (float)(2 * n_levels + 1);
    const float lo0 = x_zp ? -zp0 : lo, hi0 = x_zp ? top - zp0 : hi;
    const float lo1 = x_zp ? -zp1 : lo, hi1 = x_zp ? top - zp1 : hi;
    const bool shifted = x_zp && n_levels == 127;       // 8-bit asymmetric: planes hold q - 128
    const uint32_t zs0 = shifted ? (uint32_t)((int)zp0 - 128) : 0u;
    const uint32_t zs1 = shifted ? (uint32_t)((int)zp1 - 128) : 0u;

    uint32_t q[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) q[i][j] = 0;

    if (p < hw) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = 4 * cg + i;
        const int c = c0 + row;
        if (c < g.cin) {
          const bool seg1 = !(one_scale || per_sample) && c >= g.split;
          const float delta = seg1 ? delta1 : delta0;
          const float inv = seg1 ? inv1 : inv0;
          const float4 xt = *reinterpret_cast<const float4*>(sx + row * kTileP + 4 * pq);
          float xv[4] = {xt.x, xt.y, xt.z, xt.w}, av[4] = {0.f, 0.f, 0.f, 0.f}, nv[4];
          if (a_hat) {
            const float4 at = *reinterpret_cast<const float4*>(sa + row * kTileP + 4 * pq);
            av[0] = at.x; av[1] = at.y; av[2] = at.z; av[3] = at.w;
          }
          if (XFORM) {
            if (src.affine) {
              const float2 ab =
                  __ldg(reinterpret_cast<const float2*>(src.affine) + img + c);
#pragma unroll
              for (int j = 0; j < 4; ++j) xv[j] = fmaf(xv[j], ab.x, ab.y);
            } else if (src.bias) {
              const float b = __ldg(src.bias + img + c);
#pragma unroll
              for (int j = 0; j < 4; ++j) xv[j] = __fadd_rn(xv[j], b);
            }
            if (src.silu) {
#pragma unroll
              for (int j = 0; j < 4; ++j) xv[j] = silu_f(xv[j]);
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float r = __fsub_rn(xv[j], av[j]);
            const float qf = quantise_clamp(r, delta, inv, seg1 ? lo1 : lo0, seg1 ? hi1 : hi0, q[i][j]);
            q[i][j] += seg1 ? zs1 : zs0;
            nv[j] = __fadd_rn(av[j], __fmul_rn(qf, delta));
          }
          if (a_hat)
            *reinterpret_cast<float4*>(a_hat + (img + c) * hw + p) =
                make_float4(nv[0], nv[1], nv[2], nv[3]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      tile_sh[4 * pq + j][cg] = pack_low_bytes(q[0][j], q[1][j], q[2][j], q[3][j]);
    }
    __syncthreads();
    const int px = threadIdx.x >> 2;
    const int piece = threadIdx.x & 3;
    const int pp = p0 + px;
    const int cbase = c0 + 16 * piece;
    if (pp < hw && cbase < d.cp) {
      int y, xq, ys, xs;
      y = tg.by_w.divmod(pp, xq);
      const int yq = tg.by_stride.divmod(y + g.pad_t, ys);
      const int xqq = tg.by_stride.divmod(xq + g.pad_l, xs);
      const int plane = ys * g.stride + xs;
      const size_t pix = (((size_t)n * d.nplanes + plane) * d.hp + yq) * d.wp + xqq;
      int4 v = make_int4(tile_sh[px][4 * piece], tile_sh[px][4 * piece + 1],
                         tile_sh[px][4 * piece + 2], tile_sh[px][4 * piece + 3]);
      *reinterpret_cast<int4*>(codes + pix * d.cp + cbase) = v;
    }
    __syncthreads();   // tile_sh and the stage just read are rewritten next
  }
}

// ---------------------------------------------------------------------------------------
// Asymmetric activation codes (the reference's default without --a_sym,
// qdiff/quant_layer.py:191-214 with sym=False): delta = (max - min) / (2^b - 1),
// zero_point = round(-min / delta), q = clamp(round(r / delta) + zp, 0, 2^b - 1).
// The planes hold the CENTRED code q - zp (what the convolution multiplies), so the GEMM
// kernels and the zero halo are those of the symmetric path; that needs the centred range
// [-zp, 2^b - 1 - zp] inside int8, which holds for b <= 7 whenever the residual straddles zero.
// A scale slot whose range does not fit sets the sticky status word (bit 2).
__device__ int g_modq_status = 0;

__device__ inline unsigned int f2ord(float f) {     // order-preserving float -> unsigned
  const unsigned int b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ inline float ord2f(unsigned int o) {
  return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
}

// scratch as {counter, pad[3], mm[2 * slots]}: mm[2s] = max key, mm[2s+1] = ~(min key), both
// accumulated with atomicMax from zero and left zeroed again.
__device__ inline void publish_range(ModqScratch* scratch, int slot, float mn, float mx) {
  atomicMax(&scratch->absmax_bits[2 * slot], f2ord(mx));
  atomicMax(&scratch->absmax_bits[2 * slot + 1], ~f2ord(mn));
}

// last block: ranges -> delta, zero point (per tensor in Python-float arithmetic, per sample in
// fp32 tensor arithmetic, as the reference does)
__device__ inline void finalise_ranges(ModqScratch* scratch, int slots, int n_bits, int per_sample,
                                       float* x_scale, float* x_zp, float* range_out = nullptr) {
  const int top = (1 << n_bits) - 1;
  for (int s = threadIdx.x; s < slots; s += blockDim.x) {
    const unsigned int kmax = atomicExch(&scratch->absmax_bits[2 * s], 0u);
    const unsigned int kmin = atomicExch(&scratch->absmax_bits[2 * s + 1], 0u);
    const float xmax = kmax ? ord2f(kmax) : 0.0f;
    const float xmin = kmin ? ord2f(~kmin) : 0.0f;
    if (range_out) {              // the raw range, for the moving-average update
      range_out[2 * s] = xmin;
      range_out[2 * s + 1] = xmax;
    }
    float delta, zp;
    if (!per_sample) {
      double d = ((double)xmax - (double)xmin) / (double)top;
      if (d < 1e-8) d = 1e-8;
      zp = (float)rint(-(double)xmin / d);
      delta = (float)d;
    } else {
      delta = __fdiv_rn(__fsub_rn(xmax, xmin), (float)top);
      if (delta < 1e-8f) delta = 1e-8f;
      zp = rintf(__fdiv_rn(-xmin, delta));
    }
    // (with range_out the caller derives its own scale and checks it)
    if (!range_out && n_bits < 8 && !(-zp >= -128.0f && (float)top - zp <= 127.0f))
      atomicOr(&g_modq_status, 4);
    x_scale[s] = delta;
    x_zp[s] = zp;
  }
}

template <bool VEC4, bool XFORM>
__global__ void __launch_bounds__(kThreads)
modq_minmax_kernel(const SrcView src, const float* __restrict__ a_hat, modiff_conv_geom g,
                   TileGrid tg, int n_bits, int per_sample, int slots,
                   ModqScratch* __restrict__ scratch, float* __restrict__ x_scale,
                   float* __restrict__ x_zp, float* __restrict__ range_out = nullptr) {
  const int hw = g.h * g.w;
  const int cg = threadIdx.x >> 4;
  const int pq = threadIdx.x & 15;
  __shared__ bool is_last;
  float mx0 = -INFINITY, mn0 = INFINITY, mx1 = -INFINITY, mn1 = INFINITY;
  bool any0 = false, any1 = false;
  int cur_n = -1;
  auto flush = [&](int slot, float mn, float mx, bool any) {
    for (int o = 16; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    any = __any_sync(0xffffffffu, any);
    if ((threadIdx.x & 31) == 0 && any) publish_range(scratch, slot, mn, mx);
  };
  for (int tile = blockIdx.x; tile < tg.total; tile += gridDim.x) {
    int n, c0, p0;
    tg.decode(tile, n, c0, p0);
    const int p = p0 + 4 * pq;
    if (per_sample && n != cur_n) {
      if (cur_n >= 0) flush(cur_n, mn0, mx0, any0);
      mx0 = -INFINITY; mn0 = INFINITY; any0 = false;
      cur_n = n;
    }
    if (p < hw) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = c0 + 4 * cg + i;
        if (c < g.cin) {
          const size_t off = ((size_t)n * g.cin + c) * hw;
          float xv[4], av[4] = {0.f, 0.f, 0.f, 0.f};
          load_src<VEC4, XFORM>(src, n, c, g.cin, p, hw, xv);
          if (a_hat) load4<VEC4>(a_hat + off, p, hw, av);
          float lo = INFINITY, hi = -INFINITY;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (VEC4 || p + j < hw) {
              const float r = __fsub_rn(xv[j], av[j]);
              lo = fminf(lo, r);
              hi = fmaxf(hi, r);
            }
          }
          if (g.split > 0 && c >= g.split) {
            mn1 = fminf(mn1, lo); mx1 = fmaxf(mx1, hi); any1 = true;
          } else {
            mn0 = fminf(mn0, lo); mx0 = fmaxf(mx0, hi); any0 = true;
          }
        }
      }
    }
  }
  flush(per_sample ? (cur_n < 0 ? 0 : cur_n) : 0, mn0, mx0, any0);
  if (g.split > 0) flush(1, mn1, mx1, any1);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int ticket = atomicAdd(&scratch->counter, 1u);
    is_last = (ticket == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    __threadfence();
    finalise_ranges(scratch, slots, n_bits, per_sample, x_scale, x_zp, range_out);
    if (threadIdx.x == 0) scratch->counter = 0u;
  }
}

__global__ void __launch_bounds__(kThreads)
modq_flat_minmax_kernel(const float4* __restrict__ x, const float4* __restrict__ a_hat, int64_t n4,
                        int cin, int split, int n_bits, int per_sample, int slots,
                        ModqScratch* __restrict__ scratch, float* __restrict__ x_scale,
                        float* __restrict__ x_zp, float* __restrict__ range_out = nullptr) {
  __shared__ bool is_last;
  float mx0 = -INFINITY, mn0 = INFINITY, mx1 = -INFINITY, mn1 = INFINITY;
  bool any0 = false, any1 = false;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 xv = __ldg(x + i);
    const float4 av = a_hat ? __ldg(a_hat + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float r0 = __fsub_rn(xv.x, av.x), r1 = __fsub_rn(xv.y, av.y), r2 = __fsub_rn(xv.z, av.z),
                r3 = __fsub_rn(xv.w, av.w);
    const float lo = fminf(fminf(r0, r1), fminf(r2, r3)), hi = fmaxf(fmaxf(r0, r1), fmaxf(r2, r3));
    const int c = (int)((i * 4) % cin);
    if (per_sample) {
      publish_range(scratch, (int)((i * 4) / cin), lo, hi);
    } else if (split > 0 && c >= split) {
      mn1 = fminf(mn1, lo); mx1 = fmaxf(mx1, hi); any1 = true;
    } else {
      mn0 = fminf(mn0, lo); mx0 = fmaxf(mx0, hi); any0 = true;
    }
  }
  if (!per_sample) {
    for (int o = 16; o > 0; o >>= 1) {
      mn0 = fminf(mn0, __shfl_xor_sync(0xffffffffu, mn0, o));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
      mn1 = fminf(mn1, __shfl_xor_sync(0xffffffffu, mn1, o));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
    }
    any0 = __any_sync(0xffffffffu, any0);
    any1 = __any_sync(0xffffffffu, any1);
    if ((threadIdx.x & 31) == 0) {
      if (any0) publish_range(scratch, 0, mn0, mx0);
      if (any1) publish_range(scratch, 1, mn1, mx1);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int ticket = atomicAdd(&scratch->counter, 1u);
    is_last = (ticket == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    __threadfence();
    finalise_ranges(scratch, slots, n_bits, per_sample, x_scale, x_zp, range_out);
    if (threadIdx.x == 0) scratch->counter = 0u;
  }
}

// Linear layers (h = w = 1, cin a multiple of 16): activations [rows][cin] and codes
// [rows][cin] share one flat index, so both passes are plain elementwise sweeps.
__global__ void __launch_bounds__(kThreads)
modq_flat_absmax_kernel(const float4* __restrict__ x, const float4* __restrict__ a_hat, int64_t n4,
                        int cin, int split, int n_levels, int per_sample, int slots,
                        ModqScratch* __restrict__ scratch, float* __restrict__ x_scale) {
  __shared__ float s0[kThreads / 32], s1[kThreads / 32];
  __shared__ bool is_last;
  float m0 = 0.0f, m1 = 0.0f;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 xv = __ldg(x + i);
    float4 av = a_hat ? __ldg(a_hat + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    float m = fmaxf(fmaxf(fabsf(__fsub_rn(xv.x, av.x)), fabsf(__fsub_rn(xv.y, av.y))),
                    fmaxf(fabsf(__fsub_rn(xv.z, av.z)), fabsf(__fsub_rn(xv.w, av.w))));
    const int c = (int)((i * 4) % cin);
    if (per_sample) {
      if (m > 0.0f) atomicMax(&scratch->absmax_bits[(i * 4) / cin], __float_as_uint(m));
    } else if (split > 0 && c >= split) {
      m1 = fmaxf(m1, m);
    } else {
      m0 = fmaxf(m0, m);
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, o));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, o));
  }
  if ((threadIdx.x & 31) == 0) {
    s0[threadIdx.x >> 5] = m0;
    s1[threadIdx.x >> 5] = m1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < kThreads / 32; ++i) {
      m0 = fmaxf(m0, s0[i]);
      m1 = fmaxf(m1, s1[i]);
    }
    if (m0 > 0.0f) atomicMax(&scratch->absmax_bits[0], __float_as_uint(m0));
    if (m1 > 0.0f) atomicMax(&scratch->absmax_bits[1], __float_as_uint(m1));
    __threadfence();
    const unsigned int ticket = atomicAdd(&scratch->counter, 1u);
    is_last = (ticket == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    __threadfence();
    for (int s = threadIdx.x; s < slots; s += blockDim.x) {
      const unsigned int bits = atomicExch(&scratch->absmax_bits[s], 0u);
      double delta = (double)__uint_as_float(bits) / (double)n_levels;
      if (delta < 1e-8) delta = 1e-8;
      x_scale[s] = (float)delta;
    }
    if (threadIdx.x == 0) scratch->counter = 0u;
  }
}

__global__ void __launch_bounds__(kThreads)
modq_flat_encode_kernel(const float4* __restrict__ x, float4* __restrict__ a_hat,
                        uint32_t* __restrict__ codes, const float* __restrict__ x_scale,
                        const float* __restrict__ x_zp, int64_t n4, int cin, int split, int n_levels,
                        int per_sample) {
  const float lo = (float)(-n_levels - 1), hi = (float)n_levels;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const int c = (int)((i * 4) % cin);
    const int slot = per_sample ? (int)((i * 4) / cin) : ((split > 0 && c >= split) ? 1 : 0);
    const float delta = x_scale[slot];
    const float lo_s = x_zp ? -x_zp[slot] : lo;
    const float hi_s = x_zp ? (float)(2 * n_levels + 1) - x_zp[slot] : hi;
    const uint32_t zshift = plane_shift(x_zp, slot, n_levels);
    float4 xv = __ldg(x + i);
    float4 av = a_hat ? a_hat[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    float xs[4] = {xv.x, xv.y, xv.z, xv.w}, as[4] = {av.x, av.y, av.z, av.w}, nv[4];
    uint32_t qb[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float qf = round_clamp(__fdiv_rn(__fsub_rn(xs[j], as[j]), delta), lo_s, hi_s, qb[j]);
      qb[j] += zshift;
      nv[j] = __fadd_rn(as[j], __fmul_rn(qf, delta));
    }
    if (a_hat) a_hat[i] = make_float4(nv[0], nv[1], nv[2], nv[3]);
    codes[i] = pack_low_bytes(qb[0], qb[1], qb[2], qb[3]);
  }
}


// Linear layers whose input is LayerNorm(x) over the last dimension (the transformer blocks'
// norm1 / norm2 / norm3 in front of to_q and the feed-forward projection,
// ldm/modules/attention.py:229-241): the normalised tensor is never written.  A warp owns a row,
// holds it in registers, takes its statistics exactly as layernorm_kernel<NV> does (same
// functions, same bits) and evaluates the residual against the cached input, in both passes.
// Symmetric per-tensor codes, one scale.
template <int NV>
__global__ void __launch_bounds__(kThreads)
modq_ln_absmax_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                      const float* __restrict__ beta, float eps, const float* __restrict__ a_hat,
                      int64_t rows, int c, int n_levels, ModqScratch* __restrict__ scratch,
                      float* __restrict__ x_scale) {
  __shared__ float s0[kThreads / 32];
  __shared__ bool is_last;
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  constexpr int kWarps = kThreads / 32;
  const int c4 = c >> 2;
  float m = 0.0f;
  for (int64_t row = (int64_t)blockIdx.x * kWarps + wib; row < rows; row += (int64_t)gridDim.x * kWarps) {
    float4 v[NV], av[NV];
    ln_row_load<NV>(x + row * c, c4, lane, v);
    ln_row_load<NV>(a_hat + row * c, c4, lane, av);
    float mean, rstd;
    ln_row_stats<NV>(v, c4, lane, eps, mean, rstd);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int idx = lane + 32 * k;
      if (idx < c4) {
        const float4 y = ln_value4(v[k], mean, rstd, __ldg(reinterpret_cast<const float4*>(gamma) + idx),
                                   __ldg(reinterpret_cast<const float4*>(beta) + idx));
        m = fmaxf(m, fmaxf(fmaxf(fabsf(__fsub_rn(y.x, av[k].x)), fabsf(__fsub_rn(y.y, av[k].y))),
                           fmaxf(fabsf(__fsub_rn(y.z, av[k].z)), fabsf(__fsub_rn(y.w, av[k].w)))));
      }
    }
  }
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) s0[wib] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < kWarps; ++i) m = fmaxf(m, s0[i]);
    if (m > 0.0f) atomicMax(&scratch->absmax_bits[0], __float_as_uint(m));
    __threadfence();
    const unsigned int ticket = atomicAdd(&scratch->counter, 1u);
    is_last = (ticket == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last && threadIdx.x == 0) {
    __threadfence();
    const unsigned int bits = atomicExch(&scratch->absmax_bits[0], 0u);
    double delta = (double)__uint_as_float(bits) / (double)n_levels;   // as modq_flat_absmax_kernel
    if (delta < 1e-8) delta = 1e-8;
    x_scale[0] = (float)delta;
    scratch->counter = 0u;
  }
}

template <int NV>
__global__ void __launch_bounds__(kThreads)
modq_ln_encode_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                      const float* __restrict__ beta, float eps, float* __restrict__ a_hat,
                      uint32_t* __restrict__ codes, const float* __restrict__ x_scale, int64_t rows,
                      int c, int n_levels) {
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  constexpr int kWarps = kThreads / 32;
  const int c4 = c >> 2;
  const float lo = (float)(-n_levels - 1), hi = (float)n_levels;
  const float delta = x_scale[0];
  const float inv = __frcp_rn(delta);
  for (int64_t row = (int64_t)blockIdx.x * kWarps + wib; row < rows; row += (int64_t)gridDim.x * kWarps) {
    float4 v[NV], av[NV];
    ln_row_load<NV>(x + row * c, c4, lane, v);
    float4* ar = reinterpret_cast<float4*>(a_hat + row * c);
#pragma unroll
    for (int k = 0; k < NV; ++k) {     // plain loads: this kernel writes the cache below
      const int idx = lane + 32 * k;
      av[k] = idx < c4 ? ar[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float mean, rstd;
    ln_row_stats<NV>(v, c4, lane, eps, mean, rstd);
    uint32_t* cr = codes + row * c4;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int idx = lane + 32 * k;
      if (idx < c4) {
        const float4 y = ln_value4(v[k], mean, rstd, __ldg(reinterpret_cast<const float4*>(gamma) + idx),
                                   __ldg(reinterpret_cast<const float4*>(beta) + idx));
        const float ys[4] = {y.x, y.y, y.z, y.w}, as[4] = {av[k].x, av[k].y, av[k].z, av[k].w};
        float nv[4];
        uint32_t qb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float qf = quantise_clamp(__fsub_rn(ys[j], as[j]), delta, inv, lo, hi, qb[j]);
          nv[j] = __fadd_rn(as[j], __fmul_rn(qf, delta));
        }
        ar[idx] = make_float4(nv[0], nv[1], nv[2], nv[3]);
        cr[idx] = pack_low_bytes(qb[0], qb[1], qb[2], qb[3]);
      }
    }
  }
}

// Linear layers whose input is GEGLU(h) = h[:, :n] * gelu(h[:, n:]) (the feed-forward's second
// linear layer, ldm/modules/attention.py:37-64): both passes evaluate the gate on the fly from the
// projection's output [rows][2n] with geglu_kernel's own function (same bits); the gated tensor is
// never written.  Symmetric per-tensor codes, one scale; n a multiple of 4.
__device__ inline float4 geglu_load4(const float* __restrict__ h, int64_t i, int n4) {
  const int64_t r = i / n4;
  const int j = (int)(i - r * n4);
  const float4* row = reinterpret_cast<const float4*>(h) + r * 2 * n4;
  const float4 a = __ldg(row + j), g = __ldg(row + n4 + j);
  return make_float4(geglu_value(a.x, g.x), geglu_value(a.y, g.y), geglu_value(a.z, g.z),
                     geglu_value(a.w, g.w));
}

__global__ void __launch_bounds__(kThreads)
modq_geglu_absmax_kernel(const float* __restrict__ h, const float4* __restrict__ a_hat, int64_t total4,
                         int n4, int n_levels, ModqScratch* __restrict__ scratch,
                         float* __restrict__ x_scale) {
  __shared__ float s0[kThreads / 32];
  __shared__ bool is_last;
  float m = 0.0f;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += stride) {
    const float4 y = geglu_load4(h, i, n4);
    const float4 av = __ldg(a_hat + i);
    m = fmaxf(m, fmaxf(fmaxf(fabsf(__fsub_rn(y.x, av.x)), fabsf(__fsub_rn(y.y, av.y))),
                       fmaxf(fabsf(__fsub_rn(y.z, av.z)), fabsf(__fsub_rn(y.w, av.w)))));
  }
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) s0[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < kThreads / 32; ++i) m = fmaxf(m, s0[i]);
    if (m > 0.0f) atomicMax(&scratch->absmax_bits[0], __float_as_uint(m));
    __threadfence();
    const unsigned int ticket = atomicAdd(&scratch->counter, 1u);
    is_last = (ticket == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last && threadIdx.x == 0) {
    __threadfence();
    const unsigned int bits = atomicExch(&scratch->absmax_bits[0], 0u);
    double delta = (double)__uint_as_float(bits) / (double)n_levels;   // as modq_flat_absmax_kernel
    if (delta < 1e-8) delta = 1e-8;
    x_scale[0] = (float)delta;
    scratch->counter = 0u;
  }
}

__global__ void __launch_bounds__(kThreads)
modq_geglu_encode_kernel(const float* __restrict__ h, float4* __restrict__ a_hat,
                         uint32_t* __restrict__ codes, const float* __restrict__ x_scale,
                         int64_t total4, int n4, int n_levels) {
  const float lo = (float)(-n_levels - 1), hi = (float)n_levels;
  const float delta = x_scale[0];
  const float inv = __frcp_rn(delta);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += stride) {
    const float4 y = geglu_load4(h, i, n4);
    const float4 av = a_hat[i];
    const float ys[4] = {y.x, y.y, y.z, y.w}, as[4] = {av.x, av.y, av.z, av.w};
    float nv[4];
    uint32_t qb[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float qf = quantise_clamp(__fsub_rn(ys[j], as[j]), delta, inv, lo, hi, qb[j]);
      nv[j] = __fadd_rn(as[j], __fmul_rn(qf, delta));
    }
    a_hat[i] = make_float4(nv[0], nv[1], nv[2], nv[3]);
    codes[i] = pack_low_bytes(qb[0], qb[1], qb[2], qb[3]);
  }
}

// GroupNorm statistics and the residual maximum in ONE sweep over the source.
//
// A block takes one (image, group) slab at a time and keeps it in registers (NV float4 per
// thread): it sums the slab exactly as groupnorm_silu_kernel does (same thread count, same
// per-thread order, so mean and variance have the same bits), writes the per-(image, channel)
// scale / shift table that the encode pass reads, and then evaluates
// max |silu(x * scale + shift) - a_hat| on the values it still holds.  The stand-alone
// statistics pass (4 bytes per element) disappears.
constexpr int kGnMaxCpg = 64;

// Second quantiser of the same tensor (DUAL): a layer that reads the RAW source next to the one
// that reads its GroupNorm (a residual block's shortcut convolution next to its first
// convolution).  Its residual maximum is taken in the same sweep from the values already held.
struct SecondQuantiser {
  const float* a_hat;       // cached input of the second layer
  int split;                // its scale segments: channels >= split use slot 1
  int n_levels;
  ModqScratch* scratch;
  float* x_scale;
};

// ASYM (never with DUAL or per_sample): the sweep tracks the residual's true minimum and maximum
// per scale segment instead of its largest magnitude (m0 / m1 hold the maxima, r0 / r1 the
// minima) and the last block derives delta and the zero point (finalise_ranges); `n_levels`
// then carries n_bits.
template <int NV, bool DUAL, bool ASYM = false>
__global__ void __launch_bounds__(512, NV <= 4 ? 2 : 1)
gn_absmax_kernel(const SrcView src, const float* __restrict__ film, float* __restrict__ affine,
                 const float* __restrict__ gamma, const float* __restrict__ beta,
                 const float* __restrict__ a_hat, int batch, int c, int hw, int groups, float eps,
                 int lg_hw4, int split, int n_levels, int per_sample, int slots,
                 ModqScratch* __restrict__ scratch, float* __restrict__ x_scale,
                 const SecondQuantiser second, float* __restrict__ x_zp = nullptr) {
  __shared__ float sh[64];
  __shared__ float2 tab[kGnMaxCpg];
  __shared__ float bias_sh[kGnMaxCpg];
  __shared__ float s0[16], s1[16];
  __shared__ bool is_last;
  const int cpg = c / groups;
  const int count = cpg * hw;
  const int total4 = cpg << lg_hw4;
  const int items = batch * groups;
  const bool has_bias = src.bias != nullptr;

  float m0 = ASYM ? -INFINITY : 0.0f, m1 = m0;
  float r0 = ASYM ? INFINITY : 0.0f, r1 = r0;   // second quantiser: raw residual maxima of its
                                                // two segments (ASYM: this quantiser's minima)
  int cur_n = -1;
  // (image, group) of the current item, advanced without divisions
  const int n_step = gridDim.x / groups, g_step = gridDim.x % groups;
  int n = blockIdx.x / groups, grp = blockIdx.x % groups;
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    if (item != (int)blockIdx.x) {
      n += n_step;
      grp += g_step;
      if (grp >= groups) {
        grp -= groups;
        ++n;
      }
    }
    const int cbeg = grp * cpg;
    if (per_sample && n != cur_n) {
      if (cur_n >= 0) {
        float v = m0;
        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
        if ((threadIdx.x & 31) == 0 && v > 0.0f)
          atomicMax(&scratch->absmax_bits[cur_n], __float_as_uint(v));
      }
      m0 = 0.0f;
      cur_n = n;
    }
    // The slab (cpg whole channels of one image) is one contiguous run of the NCHW tensor.
    const float4* xs = reinterpret_cast<const float4*>(
        (cbeg < src.c0) ? src.x0 + ((size_t)n * src.c0 + cbeg) * hw
                        : src.x1 + ((size_t)n * src.c1 + (cbeg - src.c0)) * hw);
    const float4* as = a_hat
        ? reinterpret_cast<const float4*>(a_hat + ((size_t)n * c + cbeg) * hw) : nullptr;

    float4 xv[NV], av[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      xv[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      av[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < total4) {
        xv[k] = __ldg(xs + i);
        if (a_hat) av[k] = __ldg(as + i);
      }
    }
    if (DUAL) {
      const float4* bs =
          reinterpret_cast<const float4*>(second.a_hat + ((size_t)n * c + cbeg) * hw);
      float ri = 0.0f;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < total4) {
          const float4 b = __ldg(bs + i);
          ri = fmaxf(fmaxf(ri, fabsf(__fsub_rn(xv[k].x, b.x))), fabsf(__fsub_rn(xv[k].y, b.y)));
          ri = fmaxf(fmaxf(ri, fabsf(__fsub_rn(xv[k].z, b.z))), fabsf(__fsub_rn(xv[k].w, b.w)));
        }
      }
      if (second.split > 0 && cbeg >= second.split) r1 = fmaxf(r1, ri); else r0 = fmaxf(r0, ri);
    }
    // normalisation parameters of this slab's channels (threads 0 .. cpg-1), fetched before the
    // reductions so that their latency is off the critical path
    float g_ch = 0.0f, b_ch = 0.0f, f_sc = 0.0f, f_sh = 0.0f, cb_ch = 0.0f;
    if ((int)threadIdx.x < cpg) {
      const int ch = cbeg + threadIdx.x;
      g_ch = __ldg(gamma + ch);
      b_ch = __ldg(beta + ch);
      if (has_bias) cb_ch = __ldg(src.bias + (size_t)n * c + ch);
      if (film) {
        f_sc = __ldg(film + (size_t)n * 2 * c + ch);
        f_sh = __ldg(film + (size_t)n * 2 * c + c + ch);
      }
      bias_sh[threadIdx.x] = cb_ch;
    }
    float shift = __ldg(reinterpret_cast<const float*>(xs));
    float s = 0.0f, q = 0.0f;
    if (has_bias) {
      __syncthreads();
      shift = __fadd_rn(shift, bias_sh[0]);
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < total4) {
          const float b = bias_sh[i >> lg_hw4];
          const float a = __fadd_rn(xv[k].x, b) - shift, bb = __fadd_rn(xv[k].y, b) - shift,
                      cc = __fadd_rn(xv[k].z, b) - shift, dd = __fadd_rn(xv[k].w, b) - shift;
          s += (a + bb) + (cc + dd);
          q += (a * a + bb * bb) + (cc * cc + dd * dd);
        }
      }
    } else {
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < total4) {
          // x + 0 == x, so this is the arithmetic of the biased branch
          const float a = xv[k].x - shift, bb = xv[k].y - shift, cc = xv[k].z - shift,
                      dd = xv[k].w - shift;
          s += (a + bb) + (cc + dd);
          q += (a * a + bb * bb) + (cc * cc + dd * dd);
        }
      }
    }
    block_sum2(s, q, sh);
    const float ms = s / (float)count;                   // the same operations, in the same order,
    const float mean = shift + ms;                       // as groupnorm_silu_kernel
    const float var = fmaxf(q / (float)count - ms * ms, 0.0f);
    const float rstd = 1.0f / sqrtf(var + eps);
    if ((int)threadIdx.x < cpg) {      // cpg <= kGnMaxCpg <= blockDim.x
      const int ch = cbeg + threadIdx.x;
      float ga = g_ch * rstd;
      float sf = fmaf(cb_ch - mean, ga, b_ch);
      if (film) {
        const float f = 1.0f + f_sc;
        ga *= f;
        sf = fmaf(sf, f, f_sh);
      }
      tab[threadIdx.x] = make_float2(ga, sf);
      reinterpret_cast<float2*>(affine)[(size_t)n * c + ch] = make_float2(ga, sf);
    }
    __syncthreads();
    float mi = ASYM ? -INFINITY : 0.0f, mlo = INFINITY;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < total4) {
        const float2 ab = tab[i >> lg_hw4];
        float v0 = fmaf(xv[k].x, ab.x, ab.y), v1 = fmaf(xv[k].y, ab.x, ab.y),
              v2 = fmaf(xv[k].z, ab.x, ab.y), v3 = fmaf(xv[k].w, ab.x, ab.y);
        if (src.silu) {
          v0 = silu_f(v0); v1 = silu_f(v1); v2 = silu_f(v2); v3 = silu_f(v3);
        }
        if (ASYM) {
          const float d0 = __fsub_rn(v0, av[k].x), d1 = __fsub_rn(v1, av[k].y),
                      d2 = __fsub_rn(v2, av[k].z), d3 = __fsub_rn(v3, av[k].w);
          mi = fmaxf(fmaxf(fmaxf(mi, d0), d1), fmaxf(d2, d3));
          mlo = fminf(fminf(fminf(mlo, d0), d1), fminf(d2, d3));
        } else {
          mi = fmaxf(fmaxf(mi, fabsf(__fsub_rn(v0, av[k].x))), fabsf(__fsub_rn(v1, av[k].y)));
          mi = fmaxf(fmaxf(mi, fabsf(__fsub_rn(v2, av[k].z))), fabsf(__fsub_rn(v3, av[k].w)));
        }
      }
    }
    if (split > 0 && cbeg >= split) {
      m1 = fmaxf(m1, mi);
      if (ASYM) r1 = fminf(r1, mlo);
    } else {
      m0 = fmaxf(m0, mi);
      if (ASYM) r0 = fminf(r0, mlo);
    }
    __syncthreads();   // tab and bias_sh are rewritten by the next slab
  }
  for (int o = 16; o > 0; o >>= 1) {
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, o));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, o));
  }
  __shared__ float s2[16], s3[16];
  if (DUAL) {
    for (int o = 16; o > 0; o >>= 1) {
      r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, o));
      r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, o));
    }
  }
  if (ASYM) {
    for (int o = 16; o > 0; o >>= 1) {
      r0 = fminf(r0, __shfl_xor_sync(0xffffffffu, r0, o));
      r1 = fminf(r1, __shfl_xor_sync(0xffffffffu, r1, o));
    }
  }
  if ((threadIdx.x & 31) == 0) {
    s0[threadIdx.x >> 5] = m0;
    s1[threadIdx.x >> 5] = m1;
    if (DUAL || ASYM) {
      s2[threadIdx.x >> 5] = r0;
      s3[threadIdx.x >> 5] = r1;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) {
      m0 = fmaxf(m0, s0[i]);
      m1 = fmaxf(m1, s1[i]);
      if (DUAL) {
        r0 = fmaxf(r0, s2[i]);
        r1 = fmaxf(r1, s3[i]);
      }
      if (ASYM) {
        r0 = fminf(r0, s2[i]);
        r1 = fminf(r1, s3[i]);
      }
    }
    const int slot0 = per_sample ? (cur_n < 0 ? 0 : cur_n) : 0;
    if (ASYM) {
      // a block that saw no element of a segment still holds the initial (+inf, -inf) pair
      if (m0 >= r0) publish_range(scratch, 0, r0, m0);
      if (split > 0 && m1 >= r1) publish_range(scratch, 1, r1, m1);
    } else {
      if (m0 > 0.0f) atomicMax(&scratch->absmax_bits[slot0], __float_as_uint(m0));
      if (split > 0 && m1 > 0.0f) atomicMax(&scratch->absmax_bits[1], __float_as_uint(m1));
    }
    if (DUAL) {
      if (r0 > 0.0f) atomicMax(&second.scratch->absmax_bits[0], __float_as_uint(r0));
      if (second.split > 0 && r1 > 0.0f)
        atomicMax(&second.scratch->absmax_bits[1], __float_as_uint(r1));
    }
    __threadfence();
    const unsigned int ticket = atomicAdd(&scratch->counter, 1u);
    is_last = (ticket == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    __threadfence();
    if (ASYM) {
      finalise_ranges(scratch, slots, n_levels, 0, x_scale, x_zp);   // n_levels carries n_bits
    } else {
      for (int sl = threadIdx.x; sl < slots; sl += blockDim.x) {
        const unsigned int bits = atomicExch(&scratch->absmax_bits[sl], 0u);
        double delta = (double)__uint_as_float(bits) / (double)n_levels;
        if (delta < 1e-8) delta = 1e-8;
        x_scale[sl] = (float)delta;
      }
    }
    if (DUAL) {
      const int slots2 = second.split > 0 ? 2 : 1;
      for (int sl = threadIdx.x; sl < slots2; sl += blockDim.x) {
        const unsigned int bits = atomicExch(&second.scratch->absmax_bits[sl], 0u);
        double delta = (double)__uint_as_float(bits) / (double)second.n_levels;
        if (delta < 1e-8) delta = 1e-8;
        second.x_scale[sl] = (float)delta;
      }
    }
    if (threadIdx.x == 0) scratch->counter = 0u;
  }
}

// The same sweep for slabs under 1024 elements (the 4x4 and 8x8 levels of the UNet): one WARP
// per slab, eight independent slabs per block, warp shuffles instead of block barriers.  The
// per-lane order and the butterfly are those of a 32-thread groupnorm_silu_kernel block.
template <int NV>
__global__ void __launch_bounds__(256)
gn_absmax_warp_kernel(const SrcView src, const float* __restrict__ film, float* __restrict__ affine,
                      const float* __restrict__ gamma, const float* __restrict__ beta,
                      const float* __restrict__ a_hat, int batch, int c, int hw, int groups,
                      float eps, int lg_hw4, int split, int n_levels, int per_sample, int slots,
                      ModqScratch* __restrict__ scratch, float* __restrict__ x_scale) {
  __shared__ float s0[8], s1[8];
  __shared__ bool is_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  const int cpg = c / groups;            // <= 32: lane k keeps the parameters of channel k
  const int count = cpg * hw;
  const int total4 = cpg << lg_hw4;
  const int items = batch * groups;
  const bool has_bias = src.bias != nullptr;

  float m0 = 0.0f, m1 = 0.0f;
  int cur_n = -1;
  for (int item = blockIdx.x * wpb + warp; item < items; item += gridDim.x * wpb) {
    const int n = item / groups;
    const int cbeg = (item - n * groups) * cpg;
    if (per_sample && n != cur_n) {
      if (cur_n >= 0) {
        float v = m0;
        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
        if (lane == 0 && v > 0.0f) atomicMax(&scratch->absmax_bits[cur_n], __float_as_uint(v));
      }
      m0 = 0.0f;
      cur_n = n;
    }
    const float4* xs = reinterpret_cast<const float4*>(
        (cbeg < src.c0) ? src.x0 + ((size_t)n * src.c0 + cbeg) * hw
                        : src.x1 + ((size_t)n * src.c1 + (cbeg - src.c0)) * hw);
    const float4* as = a_hat
        ? reinterpret_cast<const float4*>(a_hat + ((size_t)n * c + cbeg) * hw) : nullptr;
    float4 xv[NV], av[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = lane + 32 * k;
      xv[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      av[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < total4) {
        xv[k] = __ldg(xs + i);
        if (a_hat) av[k] = __ldg(as + i);
      }
    }
    float g_ch = 0.0f, b_ch = 0.0f, f_sc = 0.0f, f_sh = 0.0f, cb_ch = 0.0f;
    if (lane < cpg) {
      const int ch = cbeg + lane;
      g_ch = __ldg(gamma + ch);
      b_ch = __ldg(beta + ch);
      if (has_bias) cb_ch = __ldg(src.bias + (size_t)n * c + ch);
      if (film) {
        f_sc = __ldg(film + (size_t)n * 2 * c + ch);
        f_sh = __ldg(film + (size_t)n * 2 * c + c + ch);
      }
    }
    const float shift =
        __fadd_rn(__ldg(reinterpret_cast<const float*>(xs)), __shfl_sync(0xffffffffu, cb_ch, 0));
    float s = 0.0f, q = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = lane + 32 * k;
      const float b = __shfl_sync(0xffffffffu, cb_ch, min(i >> lg_hw4, cpg - 1));
      if (i < total4) {
        const float a = __fadd_rn(xv[k].x, b) - shift, bb = __fadd_rn(xv[k].y, b) - shift,
                    cc = __fadd_rn(xv[k].z, b) - shift, dd = __fadd_rn(xv[k].w, b) - shift;
        s += (a + bb) + (cc + dd);
        q += (a * a + bb * bb) + (cc * cc + dd * dd);
      }
    }
    for (int o = 16; o > 0; o >>= 1) {
      s += __shfl_xor_sync(0xffffffffu, s, o);
      q += __shfl_xor_sync(0xffffffffu, q, o);
    }
    const float ms = s / (float)count;
    const float mean = shift + ms;
    const float var = fmaxf(q / (float)count - ms * ms, 0.0f);
    const float rstd = 1.0f / sqrtf(var + eps);
    float ga = g_ch * rstd;
    float sf = fmaf(cb_ch - mean, ga, b_ch);
    if (film) {
      const float f = 1.0f + f_sc;
      ga *= f;
      sf = fmaf(sf, f, f_sh);
    }
    if (lane < cpg)
      reinterpret_cast<float2*>(affine)[(size_t)n * c + cbeg + lane] = make_float2(ga, sf);
    float mi = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = lane + 32 * k;
      const int kc = min(i >> lg_hw4, cpg - 1);
      const float ax = __shfl_sync(0xffffffffu, ga, kc), ay = __shfl_sync(0xffffffffu, sf, kc);
      if (i < total4) {
        float v0 = fmaf(xv[k].x, ax, ay), v1 = fmaf(xv[k].y, ax, ay), v2 = fmaf(xv[k].z, ax, ay),
              v3 = fmaf(xv[k].w, ax, ay);
        if (src.silu) {
          v0 = silu_f(v0); v1 = silu_f(v1); v2 = silu_f(v2); v3 = silu_f(v3);
        }
        mi = fmaxf(fmaxf(mi, fabsf(__fsub_rn(v0, av[k].x))), fabsf(__fsub_rn(v1, av[k].y)));
        mi = fmaxf(fmaxf(mi, fabsf(__fsub_rn(v2, av[k].z))), fabsf(__fsub_rn(v3, av[k].w)));
      }
    }
    if (split > 0 && cbeg >= split) m1 = fmaxf(m1, mi); else m0 = fmaxf(m0, mi);
  }
  for (int o = 16; o > 0; o >>= 1) {
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, o));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, o));
  }
  if (per_sample) {
    // images differ between the warps of a block: every warp publishes its own maximum
    if (lane == 0 && cur_n >= 0 && m0 > 0.0f)
      atomicMax(&scratch->absmax_bits[cur_n], __float_as_uint(m0));
    m0 = 0.0f;
  }
  if (lane == 0) {
    s0[warp] = m0;
    s1[warp] = m1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < wpb; ++i) {
      m0 = fmaxf(m0, s0[i]);
      m1 = fmaxf(m1, s1[i]);
    }
    if (m0 > 0.0f) atomicMax(&scratch->absmax_bits[0], __float_as_uint(m0));
    if (split > 0 && m1 > 0.0f) atomicMax(&scratch->absmax_bits[1], __float_as_uint(m1));
    __threadfence();
    const unsigned int ticket = atomicAdd(&scratch->counter, 1u);
    is_last = (ticket == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    __threadfence();
    for (int sl = threadIdx.x; sl < slots; sl += blockDim.x) {
      const unsigned int bits = atomicExch(&scratch->absmax_bits[sl], 0u);
      double delta = (double)__uint_as_float(bits) / (double)n_levels;
      if (delta < 1e-8) delta = 1e-8;
      x_scale[sl] = (float)delta;
    }
    if (threadIdx.x == 0) scratch->counter = 0u;
  }
}

// Encode pass for TWO layers that read the same tensor: layer A through GroupNorm (+ SiLU), from
// the scale / shift table, layer B raw (a residual block's first convolution and its shortcut
// convolution).  One read of x serves both; each layer keeps its own cache, scale slots and
// code planes.  Tile walk, staging and arithmetic are those of modq_encode_staged_kernel.
struct EncodeTarget {
  float* a_hat;
  int8_t* codes;
  const float* x_scale;
  modiff_conv_geom g;
  Derived d;
  int n_levels;
};
constexpr int kPairStageFloats = 2 * kTileC * kTileP;          // x | a_hat A (B comes by registers)
constexpr int kPairSmem = kStages * kPairStageFloats * 4;

__global__ void __launch_bounds__(kThreads, 3)
modq_encode_pair_kernel(const SrcView src, const EncodeTarget ta, const EncodeTarget tb,
                        TileGrid tg) {
  extern __shared__ __align__(16) float stage_sh[];
  __shared__ uint32_t tile_a[kTileP][kTileC / 4 + 1];
  __shared__ uint32_t tile_b[kTileP][kTileC / 4 + 1];
  const modiff_conv_geom& g = ta.g;
  const int hw = g.h * g.w;
  const int cg = threadIdx.x >> 4;
  const int pq = threadIdx.x & 15;
  const float lo_a = (float)(-ta.n_levels - 1), hi_a = (float)ta.n_levels;
  const float lo_b = (float)(-tb.n_levels - 1), hi_b = (float)tb.n_levels;
  const int lrow = threadIdx.x >> 4, lcol = (threadIdx.x & 15) * 4;
  const uint32_t sdst0 =
      (uint32_t)__cvta_generic_to_shared(stage_sh) + (uint32_t)(lrow * kTileP + lcol) * 4u;
  auto issue = [&](int it, int stage) {
    const int tile = tg.total - 1 - it;
    int n, c0, p0;
    tg.decode(tile, n, c0, p0);
    const int p = p0 + lcol;
    const float* xb0 = src.x0 + (size_t)n * src.c0 * hw;
    const float* xb1 = src.x1 ? src.x1 + (size_t)n * src.c1 * hw : xb0;
    const float* aa = ta.a_hat + (size_t)n * g.cin * hw;
    const uint32_t sdst = sdst0 + (uint32_t)(stage * kPairStageFloats) * 4u;
#pragma unroll
    for (int r = 0; r < (kTileC * kTileP / 4) / kThreads; ++r) {
      const int c = c0 + lrow + 16 * r;
      const bool valid = (c < g.cin) && (p < hw);
      const int bytes = valid ? 16 : 0;
      const float* xp = xb0;
      const float* pa = aa;
      if (valid) {
        xp = (c < src.c0) ? xb0 + (c * hw + p) : xb1 + ((c - src.c0) * hw + p);
        pa = aa + (c * hw + p);
      }
      const uint32_t d = sdst + (uint32_t)(16 * r * kTileP) * 4u;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(xp), "r"(bytes)
                   : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(
                       d + (uint32_t)(kTileC * kTileP) * 4u),
                   "l"(pa), "r"(bytes)
                   : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // code -> plane address of layer t for pixel pp of image n
  auto plane_pixel = [&](const EncodeTarget& t, int n, int pp) -> size_t {
    int y, xq, ys, xs;
    y = tg.by_w.divmod(pp, xq);
    const int yq = tg.by_stride.divmod(y + t.g.pad_t, ys);
    const int xqq = tg.by_stride.divmod(xq + t.g.pad_l, xs);
    const int plane = ys * t.g.stride + xs;
    return (((size_t)n * t.d.nplanes + plane) * t.d.hp + yq) * t.d.wp + xqq;
  };

  int k = 0;
  if ((int)blockIdx.x < tg.total) issue(blockIdx.x, 0);
  for (int it = blockIdx.x; it < tg.total; it += gridDim.x, ++k) {
    const int stage = k % kStages;
    const bool more = it + (int)gridDim.x < tg.total;
    if (more) issue(it + gridDim.x, (k + 1) % kStages);
    const int tile = tg.total - 1 - it;
    int n, c0, p0;
    tg.decode(tile, n, c0, p0);
    const int p = p0 + 4 * pq;
    const size_t img = (size_t)n * g.cin;
    // layer B's cached rows travel through registers, in flight while the staged tile lands
    float4 brow[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = c0 + 4 * cg + i;
      brow[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (p < hw && c < g.cin)
        brow[i] = __ldg(reinterpret_cast<const float4*>(tb.a_hat + (img + c) * hw + p));
    }
    if (more) {
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* sx = stage_sh + stage * kPairStageFloats;
    const float* sa = sx + kTileC * kTileP;
    const float da = ta.x_scale[0], ia = __frcp_rn(da);
    const float db0 = tb.x_scale[0], db1 = tb.g.split > 0 ? tb.x_scale[1] : db0;
    const float ib0 = __frcp_rn(db0), ib1 = __frcp_rn(db1);

    uint32_t qa[4][4], qb[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        qa[i][j] = 0;
        qb[i][j] = 0;
      }
    if (p < hw) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = 4 * cg + i;
        const int c = c0 + row;
        if (c < g.cin) {
          const float4 xt = *reinterpret_cast<const float4*>(sx + row * kTileP + 4 * pq);
          const float4 at = *reinterpret_cast<const float4*>(sa + row * kTileP + 4 * pq);
          const float4 bt = brow[i];
          const float xr[4] = {xt.x, xt.y, xt.z, xt.w};
          const float av[4] = {at.x, at.y, at.z, at.w};
          const float bv[4] = {bt.x, bt.y, bt.z, bt.w};
          const float2 aff = __ldg(reinterpret_cast<const float2*>(src.affine) + img + c);
          const bool seg1 = tb.g.split > 0 && c >= tb.g.split;
          const float db = seg1 ? db1 : db0, ib = seg1 ? ib1 : ib0;
          float na[4], nb[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float va = fmaf(xr[j], aff.x, aff.y);
            if (src.silu) va = silu_f(va);
            const float fa = quantise_clamp(__fsub_rn(va, av[j]), da, ia, lo_a, hi_a, qa[i][j]);
            na[j] = __fadd_rn(av[j], __fmul_rn(fa, da));
            const float fb = quantise_clamp(__fsub_rn(xr[j], bv[j]), db, ib, lo_b, hi_b, qb[i][j]);
            nb[j] = __fadd_rn(bv[j], __fmul_rn(fb, db));
          }
          *reinterpret_cast<float4*>(ta.a_hat + (img + c) * hw + p) =
              make_float4(na[0], na[1], na[2], na[3]);
          *reinterpret_cast<float4*>(tb.a_hat + (img + c) * hw + p) =
              make_float4(nb[0], nb[1], nb[2], nb[3]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      tile_a[4 * pq + j][cg] = pack_low_bytes(qa[0][j], qa[1][j], qa[2][j], qa[3][j]);
      tile_b[4 * pq + j][cg] = pack_low_bytes(qb[0][j], qb[1][j], qb[2][j], qb[3][j]);
    }
    __syncthreads();
    const int px = threadIdx.x >> 2;
    const int piece = threadIdx.x & 3;
    const int pp = p0 + px;
    const int cbase = c0 + 16 * piece;
    if (pp < hw && cbase < ta.d.cp) {
      const size_t pix_a = plane_pixel(ta, n, pp), pix_b = plane_pixel(tb, n, pp);
      *reinterpret_cast<int4*>(ta.codes + pix_a * ta.d.cp + cbase) =
          make_int4(tile_a[px][4 * piece], tile_a[px][4 * piece + 1], tile_a[px][4 * piece + 2],
                    tile_a[px][4 * piece + 3]);
      *reinterpret_cast<int4*>(tb.codes + pix_b * tb.d.cp + cbase) =
          make_int4(tile_b[px][4 * piece], tile_b[px][4 * piece + 1], tile_b[px][4 * piece + 2],
                    tile_b[px][4 * piece + 3]);
    }
    __syncthreads();
  }
}
}  // namespace

// MODIFF_MODQ_STAGED=0 selects the register-path encode kernel (debug aid, same outputs)
static bool staged_encode_enabled() {
  static const bool on = [] {
    const char* e = getenv("MODIFF_MODQ_STAGED");
    return !(e && e[0] == '0');
  }();
  return on;
}

// x_zp != nullptr selects asymmetric codes (range pass instead of the maximum pass).
int launch_modq_src(const SrcView& src, bool xform, float* a_hat, int8_t* codes, float* x_scale,
                    const modiff_conv_geom* g, int n_bits, int per_sample, void* scratch,
                    bool compute_scale, cudaStream_t s, float* x_zp = nullptr,
                    float* range_out = nullptr, bool do_encode = true) {
  Derived d = derive(*g);
  const int hw = g->h * g->w;
  const int n_levels = sym_levels(n_bits);
  const int slots = per_sample ? g->batch : d.nseg;
  const float* x = src.x0;
  const bool aligned = (((uintptr_t)x & 15) == 0) && (((uintptr_t)src.x1 & 15) == 0) &&
                       (a_hat == nullptr || ((uintptr_t)a_hat & 15) == 0);
  constexpr int kMaxBlocks = 148 * 8;

  if (!xform && hw == 1 && g->cin % 16 == 0 && aligned && g->split % 4 == 0 && g->stride == 1 &&
      g->pad_t + g->pad_b + g->pad_l + g->pad_r == 0) {
    const int64_t n4 = (int64_t)g->batch * g->cin / 4;
    int blocks = (int)ceil_div64(n4, kThreads);
    if (blocks > kMaxBlocks) blocks = kMaxBlocks;
    if (compute_scale && x_zp) {
      modq_flat_minmax_kernel<<<blocks, kThreads, 0, s>>>(
          (const float4*)x, (const float4*)a_hat, n4, g->cin, g->split, n_bits, per_sample, slots,
          (ModqScratch*)scratch, x_scale, x_zp, range_out);
      MODIFF_LAUNCH_CHECK("modq_flat_minmax_kernel");
    } else if (compute_scale) {
      modq_flat_absmax_kernel<<<blocks, kThreads, 0, s>>>(
          (const float4*)x, (const float4*)a_hat, n4, g->cin, g->split, n_levels, per_sample, slots,
          (ModqScratch*)scratch, x_scale);
      MODIFF_LAUNCH_CHECK("modq_flat_absmax_kernel");
    }
    if (!do_encode) return MODIFF_OK;
    modq_flat_encode_kernel<<<blocks, kThreads, 0, s>>>((const float4*)x, (float4*)a_hat,
                                                        (uint32_t*)codes, x_scale, x_zp, n4, g->cin,
                                                        g->split, n_levels, per_sample);
    MODIFF_LAUNCH_CHECK("modq_flat_encode_kernel");
    return MODIFF_OK;
  }

  TileGrid tg;
  tg.pb = ceil_div(hw, kTileP);
  tg.cb = ceil_div(g->cin, kTileC);
  tg.per_image = FastDiv(tg.pb * tg.cb);
  tg.by_pb = FastDiv(tg.pb);
  tg.by_w = FastDiv(g->w);
  tg.by_stride = FastDiv(g->stride);
  const int64_t total = (int64_t)tg.pb * tg.cb * g->batch;
  if (total >= (1ll << 31)) return set_error(MODIFF_ERR_INVALID, "activation tensor too large");
  tg.total = (int)total;
  const int blocks = tg.total < kMaxBlocks ? tg.total : kMaxBlocks;
  const bool vec = (hw % 4 == 0) && aligned;
#define MODIFF_MODQ_SCALE(V, X)                                                                    \
  if (compute_scale && x_zp) {                                                                   \
    modq_minmax_kernel<V, X><<<blocks, kThreads, 0, s>>>(src, a_hat, *g, tg, n_bits, per_sample,   \
                                                        slots, (ModqScratch*)scratch, x_scale,   \
                                                        x_zp, range_out);                        \
    MODIFF_LAUNCH_CHECK("modq_minmax_kernel");                                                   \
  } else if (compute_scale) {                                                                    \
    modq_absmax_kernel<V, X><<<blocks, kThreads, 0, s>>>(src, a_hat, *g, tg, n_levels, per_sample, \
                                                        slots, (ModqScratch*)scratch, x_scale);  \
    MODIFF_LAUNCH_CHECK("modq_absmax_kernel");                                                   \
  }
#define MODIFF_MODQ_LAUNCH(V, X)                                                                   \
  {                                                                                              \
    MODIFF_MODQ_SCALE(V, X)                                                                      \
    if (!do_encode) return MODIFF_OK;                                                            \
    modq_encode_kernel<V, X><<<blocks, kThreads, 0, s>>>(src, a_hat, codes, x_scale, x_zp, *g, d,  \
                                                        tg, n_levels, per_sample);               \
    MODIFF_LAUNCH_CHECK("modq_encode_kernel");                                                   \
  }
  if (vec && staged_encode_enabled()) {
    // three 68 KB blocks per SM keep three tiles of input in flight
    const int sblocks = tg.total < 148 * 3 ? tg.total : 148 * 3;
    if (xform) {
      MODIFF_MODQ_SCALE(true, true)
    } else {
      MODIFF_MODQ_SCALE(true, false)
    }
    if (!do_encode) return MODIFF_OK;
    static SmemLimit smem_limit[2];
    if (xform) {
      MODIFF_CUDA(raise_smem_limit(modq_encode_staged_kernel<true>, kStagedSmem, smem_limit[1]));
      modq_encode_staged_kernel<true><<<sblocks, kThreads, kStagedSmem, s>>>(
          src, a_hat, codes, x_scale, x_zp, *g, d, tg, n_levels, per_sample);
    } else {
      MODIFF_CUDA(raise_smem_limit(modq_encode_staged_kernel<false>, kStagedSmem, smem_limit[0]));
      modq_encode_staged_kernel<false><<<sblocks, kThreads, kStagedSmem, s>>>(
          src, a_hat, codes, x_scale, x_zp, *g, d, tg, n_levels, per_sample);
    }
    MODIFF_LAUNCH_CHECK("modq_encode_staged_kernel");
    return MODIFF_OK;
  }
  if (vec && xform) MODIFF_MODQ_LAUNCH(true, true)
  else if (vec) MODIFF_MODQ_LAUNCH(true, false)
  else if (xform) MODIFF_MODQ_LAUNCH(false, true)
  else MODIFF_MODQ_LAUNCH(false, false)
#undef MODIFF_MODQ_LAUNCH
#undef MODIFF_MODQ_SCALE
  return MODIFF_OK;
}

int launch_modq(const float* x, float* a_hat, int8_t* codes, float* x_scale,
                const modiff_conv_geom* g, int n_bits, int per_sample, void* scratch,
                bool compute_scale, cudaStream_t s) {
  SrcView v = {};
  v.x0 = x;
  v.c0 = g->cin;
  return launch_modq_src(v, false, a_hat, codes, x_scale, g, n_bits, per_sample, scratch,
                         compute_scale, s);
}

}  // namespace modiff

using namespace modiff;

extern "C" int modiff_modq(const float* x, float* a_hat, int8_t* codes, float* x_scale,
                           const modiff_conv_geom* g, int n_bits, int per_sample, void* scratch,
                           void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(x && codes && x_scale && scratch, "NULL pointer argument");
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 8, "activation n_bits %d outside [2, 8]", n_bits);
  MODIFF_CHECK_ARG(!(per_sample && g->split > 0), "per-sample scales cannot be combined with split");
  MODIFF_CHECK_ARG(((uintptr_t)codes & 15) == 0, "codes must be 16-byte aligned");
  return launch_modq(x, a_hat, codes, x_scale, g, n_bits, per_sample, scratch, true,
                     (cudaStream_t)stream);
}

extern "C" int modiff_modq_geglu(const float* h, int64_t rows, int n, float* a_hat, int8_t* codes,
                                 float* x_scale, int n_bits, void* scratch, void* stream) {
  MODIFF_CHECK_ARG(h && a_hat && codes && x_scale && scratch, "NULL pointer argument");
  MODIFF_CHECK_ARG(rows > 0 && n > 0 && n % 16 == 0, "rows %lld x channels %d: channels must be a "
                   "positive multiple of 16", (long long)rows, n);
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 8, "activation n_bits %d outside [2, 8]", n_bits);
  MODIFF_CHECK_ARG(((((uintptr_t)h | (uintptr_t)a_hat | (uintptr_t)codes) & 15) == 0),
                   "buffers must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  const int n_levels = sym_levels(n_bits);
  const int64_t total4 = rows * (n / 4);
  int64_t blocks = ceil_div64(total4, kThreads);
  if (blocks > 148 * 8) blocks = 148 * 8;
  modq_geglu_absmax_kernel<<<(int)blocks, kThreads, 0, s>>>(h, (const float4*)a_hat, total4, n / 4,
                                                           n_levels, (ModqScratch*)scratch, x_scale);
  MODIFF_LAUNCH_CHECK("modq_geglu_absmax_kernel");
  modq_geglu_encode_kernel<<<(int)blocks, kThreads, 0, s>>>(h, (float4*)a_hat, (uint32_t*)codes, x_scale,
                                                           total4, n / 4, n_levels);
  MODIFF_LAUNCH_CHECK("modq_geglu_encode_kernel");
  return MODIFF_OK;
}

extern "C" int modiff_modq_ln(const float* x, const float* gamma, const float* beta, float eps,
                              int64_t rows, int c, float* a_hat, int8_t* codes, float* x_scale,
                              int n_bits, void* scratch, void* stream) {
  MODIFF_CHECK_ARG(x && gamma && beta && a_hat && codes && x_scale && scratch, "NULL pointer argument");
  MODIFF_CHECK_ARG(rows > 0 && c > 0 && c % 16 == 0 && c <= kLnMaxChannels,
                   "rows %lld x channels %d: channels must be a positive multiple of 16, at most %d",
                   (long long)rows, c, kLnMaxChannels);
  MODIFF_CHECK_ARG(((((uintptr_t)x | (uintptr_t)gamma | (uintptr_t)beta | (uintptr_t)a_hat |
                      (uintptr_t)codes) & 15) == 0), "buffers must be 16-byte aligned");
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 8, "activation n_bits %d outside [2, 8]", n_bits);
  cudaStream_t s = (cudaStream_t)stream;
  const int n_levels = sym_levels(n_bits);
  int64_t blocks = ceil_div64(rows, kThreads / 32);
  if (blocks > 148 * 8) blocks = 148 * 8;
#define MODIFF_LN_LAUNCH(NV)                                                                      \
  modq_ln_absmax_kernel<NV><<<(int)blocks, kThreads, 0, s>>>(x, gamma, beta, eps, a_hat, rows, c,   \
                                                            n_levels, (ModqScratch*)scratch, x_scale); \
  MODIFF_LAUNCH_CHECK("modq_ln_absmax_kernel");                                                    \
  modq_ln_encode_kernel<NV><<<(int)blocks, kThreads, 0, s>>>(x, gamma, beta, eps, a_hat,            \
                                                            (uint32_t*)codes, x_scale, rows, c, n_levels)
  switch (ln_chunks_per_lane(c)) {
    case 3: { MODIFF_LN_LAUNCH(3); break; }
    case 5: { MODIFF_LN_LAUNCH(5); break; }
    default: { MODIFF_LN_LAUNCH(10); break; }
  }
#undef MODIFF_LN_LAUNCH
  MODIFF_LAUNCH_CHECK("modq_ln_encode_kernel");
  return MODIFF_OK;
}

extern "C" int modiff_modq_src(const modiff_act_source* src, float* a_hat, int8_t* codes,
                               float* x_scale, const modiff_conv_geom* g, int n_bits, int per_sample,
                               void* scratch, void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(src && src->x0 && codes && x_scale && scratch, "NULL pointer argument");
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 8, "activation n_bits %d outside [2, 8]", n_bits);
  MODIFF_CHECK_ARG(!(per_sample && g->split > 0), "per-sample scales cannot be combined with split");
  MODIFF_CHECK_ARG(((uintptr_t)codes & 15) == 0, "codes must be 16-byte aligned");
  MODIFF_CHECK_ARG(src->c0 > 0 && src->c0 <= g->cin && (src->c0 == g->cin || src->x1),
                   "bad concat split c0=%d for cin=%d", src->c0, g->cin);
  SrcView v;
  v.x0 = src->x0;
  v.x1 = src->x1;
  v.bias = src->chan_bias;
  v.affine = src->affine;
  v.c0 = src->c0;
  v.c1 = g->cin - src->c0;
  v.silu = src->silu;
  const bool xform = src->x1 || src->chan_bias || src->affine || src->silu;
  return launch_modq_src(v, xform, a_hat, codes, x_scale, g, n_bits, per_sample, scratch, true,
                         (cudaStream_t)stream);
}

extern "C" int modiff_modq_up2(const float* x, float* a_hat, int8_t* codes, float* x_scale,
                               const modiff_conv_geom* g, int n_bits, int fixed_scale, void* scratch,
                               void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(x && a_hat && codes && x_scale && (scratch || fixed_scale),
                   "NULL pointer argument");
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 8, "activation n_bits %d outside [2, 8]", n_bits);
  MODIFF_CHECK_ARG(((uintptr_t)codes & 15) == 0, "codes must be 16-byte aligned");
  MODIFF_CHECK_ARG(g->stride == 1 && g->split == 0 && g->h % 2 == 0 && g->w % 2 == 0,
                   "upsampled input needs stride 1, no split and even h, w (got %d x %d)", g->h, g->w);
  cudaStream_t s = (cudaStream_t)stream;
  Derived d = derive(*g);
  modiff_conv_geom gs = *g;          // the source tensor as a layer input of its own
  gs.h = g->h / 2;
  gs.w = g->w / 2;
  const int hw = gs.h * gs.w;
  const int n_levels = sym_levels(n_bits);
  SrcView v = {};
  v.x0 = x;
  v.c0 = g->cin;
  TileGrid tg;
  tg.pb = ceil_div(hw, kTileP);
  tg.cb = ceil_div(g->cin, kTileC);
  tg.per_image = FastDiv(tg.pb * tg.cb);
  tg.by_pb = FastDiv(tg.pb);
  tg.by_w = FastDiv(gs.w);
  tg.by_stride = FastDiv(1);
  const int64_t total = (int64_t)tg.pb * tg.cb * g->batch;
  if (total >= (1ll << 31)) return set_error(MODIFF_ERR_INVALID, "activation tensor too large");
  tg.total = (int)total;
  const int blocks = tg.total < 148 * 8 ? tg.total : 148 * 8;
  const bool vec = (hw % 4 == 0) && ((((uintptr_t)x | (uintptr_t)a_hat) & 15) == 0);
  if (vec) {
    if (!fixed_scale) {
      modq_absmax_kernel<true, false><<<blocks, kThreads, 0, s>>>(v, a_hat, gs, tg, n_levels, 0, 1,
                                                                 (ModqScratch*)scratch, x_scale);
      MODIFF_LAUNCH_CHECK("modq_absmax_kernel");
    }
    modq_encode_kernel<true, false, true><<<blocks, kThreads, 0, s>>>(v, a_hat, codes, x_scale,
                                                                     nullptr, *g, d, tg, n_levels, 0);
  } else {
    if (!fixed_scale) {
      modq_absmax_kernel<false, false><<<blocks, kThreads, 0, s>>>(v, a_hat, gs, tg, n_levels, 0, 1,
                                                                  (ModqScratch*)scratch, x_scale);
      MODIFF_LAUNCH_CHECK("modq_absmax_kernel");
    }
    modq_encode_kernel<false, false, true><<<blocks, kThreads, 0, s>>>(v, a_hat, codes, x_scale,
                                                                      nullptr, *g, d, tg, n_levels, 0);
  }
  MODIFF_LAUNCH_CHECK("modq_encode_kernel (upsampled input)");
  return MODIFF_OK;
}

extern "C" int modiff_modq_gn(const modiff_act_source* src, const float* film, const float* gamma,
                              const float* beta, int groups, float eps, float* affine,
                              float* a_hat, int8_t* codes, float* x_scale,
                              const modiff_conv_geom* g, int n_bits, int per_sample, void* scratch,
                              void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(src && src->x0 && gamma && beta && affine && codes && x_scale && scratch,
                   "NULL pointer argument");
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 8, "activation n_bits %d outside [2, 8]", n_bits);
  MODIFF_CHECK_ARG(!(per_sample && g->split > 0), "per-sample scales cannot be combined with split");
  MODIFF_CHECK_ARG(((uintptr_t)codes & 15) == 0, "codes must be 16-byte aligned");
  MODIFF_CHECK_ARG(src->c0 > 0 && src->c0 <= g->cin && (src->c0 == g->cin || src->x1),
                   "bad concat split c0=%d for cin=%d", src->c0, g->cin);
  MODIFF_CHECK_ARG(groups > 0 && g->cin % groups == 0, "bad GroupNorm shape: c=%d groups=%d",
                   g->cin, groups);
  MODIFF_CHECK_ARG(((uintptr_t)affine & 7) == 0, "affine table must be 8-byte aligned");
  MODIFF_CHECK_ARG(src->affine == nullptr || src->affine == affine,
                   "src->affine must be NULL or the table this call writes");
  cudaStream_t s = (cudaStream_t)stream;
  const int hw = g->h * g->w;
  const int cpg = g->cin / groups;
  const int count = cpg * hw;
  const int threads = groupnorm_threads(count);
  const int lg_hw4 = groupnorm_lg_hw4(hw);
  const int nv = lg_hw4 >= 0 ? ceil_div(count / 4, threads) : 0;
  const bool aligned = ((((uintptr_t)src->x0 | (uintptr_t)src->x1 | (uintptr_t)a_hat) & 15) == 0);

  SrcView v;
  v.x0 = src->x0;
  v.x1 = src->x1;
  v.c0 = src->c0;
  v.c1 = g->cin - src->c0;
  v.silu = src->silu;
  const int n_levels = sym_levels(n_bits);
  const int slots = per_sample ? g->batch : derive(*g).nseg;

  // a slab must be whole channels of ONE source tensor and of ONE scale segment
  const bool whole = (src->c0 % cpg == 0) && (g->split % cpg == 0);
  if (lg_hw4 >= 0 && threads == 32 && cpg <= 32 && aligned && whole) {
    // small slabs: one warp each
    v.bias = src->chan_bias;
    v.affine = nullptr;
    const int items = g->batch * groups;
    const int nvw = ceil_div(count / 4, 32);
    const int blocks = ceil_div(items, 8) < 148 * 8 ? ceil_div(items, 8) : 148 * 8;
#define MODIFF_GN_ABSMAX_WARP(NV)                                                                \
  gn_absmax_warp_kernel<NV><<<blocks, 256, 0, s>>>(v, film, affine, gamma, beta, a_hat, g->batch,  \
                                                   g->cin, hw, groups, eps, lg_hw4, g->split,     \
                                                   n_levels, per_sample, slots,                   \
                                                   (ModqScratch*)scratch, x_scale)
    if (nvw <= 1) MODIFF_GN_ABSMAX_WARP(1);
    else if (nvw <= 2) MODIFF_GN_ABSMAX_WARP(2);
    else if (nvw <= 4) MODIFF_GN_ABSMAX_WARP(4);
    else MODIFF_GN_ABSMAX_WARP(8);
#undef MODIFF_GN_ABSMAX_WARP
    MODIFF_LAUNCH_CHECK("gn_absmax_warp_kernel");
    v.bias = nullptr;
    v.affine = affine;
    return launch_modq_src(v, true, a_hat, codes, x_scale, g, n_bits, per_sample, scratch, false, s);
  }
  if (lg_hw4 >= 0 && threads >= 256 && nv <= 8 && cpg <= kGnMaxCpg && aligned && whole) {
    v.bias = src->chan_bias;
    v.affine = nullptr;
    const int items = g->batch * groups;
    const int per_sm = threads >= 512 ? 2 : (threads >= 256 ? 4 : 8);
    const int blocks = items < 148 * per_sm ? items : 148 * per_sm;
#define MODIFF_GN_ABSMAX(NV)                                                                     \
  gn_absmax_kernel<NV, false><<<blocks, threads, 0, s>>>(                                         \
      v, film, affine, gamma, beta, a_hat, g->batch, g->cin, hw, groups, eps, lg_hw4, g->split,    \
      n_levels, per_sample, slots, (ModqScratch*)scratch, x_scale, SecondQuantiser{})
    if (nv <= 1) MODIFF_GN_ABSMAX(1);
    else if (nv <= 2) MODIFF_GN_ABSMAX(2);
    else if (nv <= 4) MODIFF_GN_ABSMAX(4);
    else MODIFF_GN_ABSMAX(8);
#undef MODIFF_GN_ABSMAX
    MODIFF_LAUNCH_CHECK("gn_absmax_kernel");
    v.bias = nullptr;
    v.affine = affine;
    return launch_modq_src(v, true, a_hat, codes, x_scale, g, n_bits, per_sample, scratch, false, s);
  }
  // slabs too large for registers (or odd sizes): statistics pass, then the two quantiser passes
  rc = modiff_groupnorm_silu(src->x0, src->x1, src->c0, src->chan_bias, film, nullptr, affine, gamma,
                             beta, g->batch, g->cin, hw, groups, eps, 0, stream);
  if (rc) return rc;
  v.bias = nullptr;
  v.affine = affine;
  return launch_modq_src(v, true, a_hat, codes, x_scale, g, n_bits, per_sample, scratch, true, s);
}

extern "C" int modiff_modq_gn_asym(const modiff_act_source* src, const float* film,
                                   const float* gamma, const float* beta, int groups, float eps,
                                   float* affine, float* a_hat, int8_t* codes, float* x_scale,
                                   float* x_zp, const modiff_conv_geom* g, int n_bits, void* scratch,
                                   void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(src && src->x0 && gamma && beta && affine && codes && x_scale && x_zp && scratch,
                   "NULL pointer argument");
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 8, "activation n_bits %d outside [2, 8]", n_bits);
  MODIFF_CHECK_ARG(((uintptr_t)codes & 15) == 0, "codes must be 16-byte aligned");
  MODIFF_CHECK_ARG(src->c0 > 0 && src->c0 <= g->cin && (src->c0 == g->cin || src->x1),
                   "bad concat split c0=%d for cin=%d", src->c0, g->cin);
  MODIFF_CHECK_ARG(groups > 0 && g->cin % groups == 0, "bad GroupNorm shape: c=%d groups=%d",
                   g->cin, groups);
  MODIFF_CHECK_ARG(((uintptr_t)affine & 7) == 0, "affine table must be 8-byte aligned");
  MODIFF_CHECK_ARG(src->affine == nullptr || src->affine == affine,
                   "src->affine must be NULL or the table this call writes");
  cudaStream_t s = (cudaStream_t)stream;
  const int hw = g->h * g->w;
  const int cpg = g->cin / groups;
  const int count = cpg * hw;
  const int threads = groupnorm_threads(count);
  const int lg_hw4 = groupnorm_lg_hw4(hw);
  const int nv = lg_hw4 >= 0 ? ceil_div(count / 4, threads) : 0;
  const bool aligned = ((((uintptr_t)src->x0 | (uintptr_t)src->x1 | (uintptr_t)a_hat) & 15) == 0);
  SrcView v;
  v.x0 = src->x0;
  v.x1 = src->x1;
  v.c0 = src->c0;
  v.c1 = g->cin - src->c0;
  v.silu = src->silu;
  const int slots = derive(*g).nseg;
  const bool whole = (src->c0 % cpg == 0) && (g->split % cpg == 0);
  if (lg_hw4 >= 0 && threads >= 256 && nv <= 8 && cpg <= kGnMaxCpg && aligned && whole) {
    v.bias = src->chan_bias;
    v.affine = nullptr;
    const int items = g->batch * groups;
    const int per_sm = threads >= 512 ? 2 : 4;
    const int blocks = items < 148 * per_sm ? items : 148 * per_sm;
#define MODIFF_GN_RANGE(NV)                                                                       \
  gn_absmax_kernel<NV, false, true><<<blocks, threads, 0, s>>>(                                    \
      v, film, affine, gamma, beta, a_hat, g->batch, g->cin, hw, groups, eps, lg_hw4, g->split,    \
      n_bits, 0, slots, (ModqScratch*)scratch, x_scale, SecondQuantiser{}, x_zp)
    if (nv <= 1) MODIFF_GN_RANGE(1);
    else if (nv <= 2) MODIFF_GN_RANGE(2);
    else if (nv <= 4) MODIFF_GN_RANGE(4);
    else MODIFF_GN_RANGE(8);
#undef MODIFF_GN_RANGE
    MODIFF_LAUNCH_CHECK("gn_absmax_kernel (range)");
    v.bias = nullptr;
    v.affine = affine;
    return launch_modq_src(v, true, a_hat, codes, x_scale, g, n_bits, 0, scratch, false, s, x_zp);
  }
  // small or odd slabs: statistics pass, then the range and encode passes
  rc = modiff_groupnorm_silu(src->x0, src->x1, src->c0, src->chan_bias, film, nullptr, affine, gamma,
                             beta, g->batch, g->cin, hw, groups, eps, 0, stream);
  if (rc) return rc;
  v.bias = nullptr;
  v.affine = affine;
  return launch_modq_src(v, true, a_hat, codes, x_scale, g, n_bits, 0, scratch, true, s, x_zp);
}

extern "C" int modiff_modq_pair(const modiff_act_source* src, const float* gamma, const float* beta,
                                int groups, float eps, float* affine, float* a_hat_a,
                                int8_t* codes_a, float* x_scale_a, const modiff_conv_geom* g_a,
                                int n_bits_a, void* scratch_a, float* a_hat_b, int8_t* codes_b,
                                float* x_scale_b, const modiff_conv_geom* g_b, int n_bits_b,
                                void* scratch_b, void* stream) {
  int rc = validate_geom(g_a);
  if (rc) return rc;
  rc = validate_geom(g_b);
  if (rc) return rc;
  MODIFF_CHECK_ARG(src && src->x0 && gamma && beta && affine && a_hat_a && codes_a && x_scale_a &&
                       scratch_a && a_hat_b && codes_b && x_scale_b && scratch_b,
                   "NULL pointer argument");
  MODIFF_CHECK_ARG(g_a->batch == g_b->batch && g_a->cin == g_b->cin && g_a->h == g_b->h &&
                       g_a->w == g_b->w,
                   "the two layers must read the same tensor");
  MODIFF_CHECK_ARG(g_a->split == 0 && g_a->stride == 1 && g_b->stride == 1,
                   "layer A must have one scale; both layers stride 1");
  MODIFF_CHECK_ARG(n_bits_a >= 2 && n_bits_a <= 8 && n_bits_b >= 2 && n_bits_b <= 8,
                   "activation n_bits outside [2, 8]");
  MODIFF_CHECK_ARG(src->chan_bias == nullptr && (src->affine == nullptr || src->affine == affine),
                   "the paired quantiser takes no channel bias");
  MODIFF_CHECK_ARG(src->c0 > 0 && src->c0 <= g_a->cin && (src->c0 == g_a->cin || src->x1),
                   "bad concat split c0=%d for cin=%d", src->c0, g_a->cin);
  MODIFF_CHECK_ARG(groups > 0 && g_a->cin % groups == 0, "bad GroupNorm shape");
  MODIFF_CHECK_ARG(((((uintptr_t)codes_a | (uintptr_t)codes_b) & 15) == 0) &&
                       (((uintptr_t)affine & 7) == 0),
                   "buffers must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  const modiff_conv_geom* g = g_a;
  const int hw = g->h * g->w;
  const int cpg = g->cin / groups;
  const int count = cpg * hw;
  const int threads = groupnorm_threads(count);
  const int lg_hw4 = groupnorm_lg_hw4(hw);
  const int nv = lg_hw4 >= 0 ? ceil_div(count / 4, threads) : 0;
  const bool aligned = ((((uintptr_t)src->x0 | (uintptr_t)src->x1 | (uintptr_t)a_hat_a |
                          (uintptr_t)a_hat_b) & 15) == 0);
  const bool whole = (src->c0 % cpg == 0) && (g_b->split % cpg == 0);
  if (!(lg_hw4 >= 0 && threads >= 256 && nv <= 8 && cpg <= kGnMaxCpg && aligned && whole)) {
    // shapes outside the paired kernels: the two quantisers one after the other
    modiff_act_source raw = *src;
    raw.affine = nullptr;
    rc = modiff_modq_gn(&raw, nullptr, gamma, beta, groups, eps, affine, a_hat_a, codes_a, x_scale_a,
                        g_a, n_bits_a, 0, scratch_a, stream);
    if (rc) return rc;
    raw.silu = 0;
    return modiff_modq_src(&raw, a_hat_b, codes_b, x_scale_b, g_b, n_bits_b, 0, scratch_b, stream);
  }
  SrcView v = {};
  v.x0 = src->x0;
  v.x1 = src->x1;
  v.c0 = src->c0;
  v.c1 = g->cin - src->c0;
  v.silu = src->silu;
  SecondQuantiser second;
  second.a_hat = a_hat_b;
  second.split = g_b->split;
  second.n_levels = sym_levels(n_bits_b);
  second.scratch = (ModqScratch*)scratch_b;
  second.x_scale = x_scale_b;
  const int items = g->batch * groups;
  const int per_sm = threads >= 512 ? 2 : 4;
  const int blocks = items < 148 * per_sm ? items : 148 * per_sm;
#define MODIFF_GN_ABSMAX2(NV)                                                                    \
  gn_absmax_kernel<NV, true><<<blocks, threads, 0, s>>>(                                          \
      v, nullptr, affine, gamma, beta, a_hat_a, g->batch, g->cin, hw, groups, eps, lg_hw4, 0,      \
      sym_levels(n_bits_a), 0, 1, (ModqScratch*)scratch_a, x_scale_a, second)
  if (nv <= 1) MODIFF_GN_ABSMAX2(1);
  else if (nv <= 2) MODIFF_GN_ABSMAX2(2);
  else if (nv <= 4) MODIFF_GN_ABSMAX2(4);
  else MODIFF_GN_ABSMAX2(8);
#undef MODIFF_GN_ABSMAX2
  MODIFF_LAUNCH_CHECK("gn_absmax_kernel (paired)");

  v.affine = affine;
  EncodeTarget ta, tb;
  ta.a_hat = a_hat_a; ta.codes = codes_a; ta.x_scale = x_scale_a; ta.g = *g_a; ta.d = derive(*g_a);
  ta.n_levels = sym_levels(n_bits_a);
  tb.a_hat = a_hat_b; tb.codes = codes_b; tb.x_scale = x_scale_b; tb.g = *g_b; tb.d = derive(*g_b);
  tb.n_levels = sym_levels(n_bits_b);
  TileGrid tg;
  tg.pb = ceil_div(hw, kTileP);
  tg.cb = ceil_div(g->cin, kTileC);
  tg.per_image = FastDiv(tg.pb * tg.cb);
  tg.by_pb = FastDiv(tg.pb);
  tg.by_w = FastDiv(g->w);
  tg.by_stride = FastDiv(1);
  const int64_t total = (int64_t)tg.pb * tg.cb * g->batch;
  if (total >= (1ll << 31)) return set_error(MODIFF_ERR_INVALID, "activation tensor too large");
  tg.total = (int)total;
  static SmemLimit smem_limit;
  MODIFF_CUDA(raise_smem_limit(modq_encode_pair_kernel, kPairSmem, smem_limit));
  const int eblocks = tg.total < 148 * 3 ? tg.total : 148 * 3;
  modq_encode_pair_kernel<<<eblocks, kThreads, kPairSmem, s>>>(v, ta, tb, tg);
  MODIFF_LAUNCH_CHECK("modq_encode_pair_kernel");
  return MODIFF_OK;
}

extern "C" int modiff_modq_asym(const modiff_act_source* src, float* a_hat, int8_t* codes,
                                float* x_scale, float* x_zp, const modiff_conv_geom* g, int n_bits,
                                int per_sample, void* scratch, void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(src && src->x0 && codes && x_scale && x_zp && scratch, "NULL pointer argument");
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 8, "activation n_bits %d outside [2, 8]", n_bits);
  MODIFF_CHECK_ARG(!(n_bits == 8 && per_sample),
                   "8-bit asymmetric codes need one zero point per scale segment, not per image");
  MODIFF_CHECK_ARG(!(per_sample && g->split > 0), "per-sample scales cannot be combined with split");
  MODIFF_CHECK_ARG(((uintptr_t)codes & 15) == 0, "codes must be 16-byte aligned");
  MODIFF_CHECK_ARG(src->c0 > 0 && src->c0 <= g->cin && (src->c0 == g->cin || src->x1),
                   "bad concat split c0=%d for cin=%d", src->c0, g->cin);
  SrcView v;
  v.x0 = src->x0;
  v.x1 = src->x1;
  v.bias = src->chan_bias;
  v.affine = src->affine;
  v.c0 = src->c0;
  v.c1 = g->cin - src->c0;
  v.silu = src->silu;
  const bool xform = src->x1 || src->chan_bias || src->affine || src->silu;
  return launch_modq_src(v, xform, a_hat, codes, x_scale, g, n_bits, per_sample, scratch, true,
                         (cudaStream_t)stream, x_zp);
}

namespace modiff {
namespace {
// act_momentum_update (qdiff/quant_layer.py:113-132) on device state: range[0..3] holds the
// moving (min, max) of segment 0 / 1, range[4..7] the range of the current call.  `init`: the
// first call of the quantiser, which records the range and takes its scale from it with the
// per-tensor 'max' rule in Python-float arithmetic (:191-214); otherwise fp32 tensor arithmetic
// exactly as the reference's EMA lines.
__global__ void running_scale_kernel(float* __restrict__ range, float* __restrict__ x_scale,
                                     float* __restrict__ x_zp, int slots, int n_bits, int sym,
                                     int init, float momentum, float one_minus) {
  const int s = threadIdx.x;
  if (s >= slots) return;
  const float cmin = range[4 + 2 * s], cmax = range[4 + 2 * s + 1];
  const int n_levels = sym ? (1 << (n_bits - 1)) - 1 : (1 << n_bits);
  float delta, zp = 0.0f;
  if (init) {
    range[2 * s] = cmin;
    range[2 * s + 1] = cmax;
    double d;
    if (sym) {
      const double lo = cmin < 0.0f ? (double)cmin : 0.0, hi = cmax > 0.0f ? (double)cmax : 0.0;
      d = fmax(fabs(lo), hi) / (double)n_levels;
    } else {
      d = ((double)cmax - (double)cmin) / (double)(n_levels - 1);
    }
    if (d < 1e-8) d = 1e-8;
    if (!sym) zp = (float)rint(-(double)cmin / d);
    delta = (float)d;
  } else {
    const float emin = __fadd_rn(__fmul_rn(range[2 * s], momentum), __fmul_rn(cmin, one_minus));
    const float emax = __fadd_rn(__fmul_rn(range[2 * s + 1], momentum), __fmul_rn(cmax, one_minus));
    range[2 * s] = emin;
    range[2 * s + 1] = emax;
    if (sym) {
      delta = __fdiv_rn(fmaxf(fabsf(emin), fabsf(emax)), (float)n_levels);
    } else {
      delta = __fdiv_rn(__fsub_rn(emax, emin), (float)(n_levels - 1));
    }
    if (delta < 1e-8f) delta = 1e-8f;
    if (!sym) zp = rintf(__fdiv_rn(-emin, delta));
  }
  if (!sym && n_bits < 8 && !(-zp >= -128.0f && (float)(n_levels - 1) - zp <= 127.0f))
    atomicOr(&g_modq_status, 4);
  x_scale[s] = delta;
  x_zp[s] = zp;
}
}  // namespace
}  // namespace modiff

extern "C" int modiff_modq_running(const modiff_act_source* src, float* a_hat, int8_t* codes,
                                   float* x_scale, float* x_zp, float* x_range,
                                   const modiff_conv_geom* g, int n_bits, int symmetric, int init,
                                   double momentum, void* scratch, void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(src && src->x0 && codes && x_scale && x_zp && x_range && scratch,
                   "NULL pointer argument");
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 8, "activation n_bits %d outside [2, 8]", n_bits);
  MODIFF_CHECK_ARG(((uintptr_t)codes & 15) == 0, "codes must be 16-byte aligned");
  MODIFF_CHECK_ARG(src->c0 > 0 && src->c0 <= g->cin && (src->c0 == g->cin || src->x1),
                   "bad concat split c0=%d for cin=%d", src->c0, g->cin);
  MODIFF_CHECK_ARG(momentum >= 0.0 && momentum <= 1.0, "momentum %f outside [0, 1]", momentum);
  SrcView v;
  v.x0 = src->x0;
  v.x1 = src->x1;
  v.bias = src->chan_bias;
  v.affine = src->affine;
  v.c0 = src->c0;
  v.c1 = g->cin - src->c0;
  v.silu = src->silu;
  const bool xform = src->x1 || src->chan_bias || src->affine || src->silu;
  cudaStream_t s = (cudaStream_t)stream;
  const int slots = derive(*g).nseg;
  // range pass only (its own delta / zero point are overwritten below)
  rc = launch_modq_src(v, xform, a_hat, codes, x_scale, g, n_bits, 0, scratch, true, s, x_zp,
                       x_range + 4, false);
  if (rc) return rc;
  // the reference's momentum and 1 - momentum are Python floats (doubles), each rounded to
  // fp32 when it meets the fp32 tensor
  const float one_minus = (float)(1.0 - momentum);
  running_scale_kernel<<<1, 32, 0, s>>>(x_range, x_scale, x_zp, slots, n_bits, symmetric, init,
                                        (float)momentum, one_minus);
  MODIFF_LAUNCH_CHECK("running_scale_kernel");
  return launch_modq_src(v, xform, a_hat, codes, x_scale, g, n_bits, 0, nullptr, false, s,
                         symmetric ? nullptr : x_zp);
}

extern "C" int modiff_modq_fixed(const modiff_act_source* src, float* a_hat, int8_t* codes,
                                 const float* x_scale, const float* x_zp,
                                 const modiff_conv_geom* g, int n_bits, int per_sample,
                                 void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(src && src->x0 && codes && x_scale, "NULL pointer argument");
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 8, "activation n_bits %d outside [2, 8]", n_bits);
  MODIFF_CHECK_ARG(!(per_sample && g->split > 0), "per-sample scales cannot be combined with split");
  MODIFF_CHECK_ARG(((uintptr_t)codes & 15) == 0, "codes must be 16-byte aligned");
  MODIFF_CHECK_ARG(src->c0 > 0 && src->c0 <= g->cin && (src->c0 == g->cin || src->x1),
                   "bad concat split c0=%d for cin=%d", src->c0, g->cin);
  SrcView v;
  v.x0 = src->x0;
  v.x1 = src->x1;
  v.bias = src->chan_bias;
  v.affine = src->affine;
  v.c0 = src->c0;
  v.c1 = g->cin - src->c0;
  v.silu = src->silu;
  const bool xform = src->x1 || src->chan_bias || src->affine || src->silu;
  // the scale pass is skipped: the encode pass only reads x_scale / x_zp
  return launch_modq_src(v, xform, a_hat, codes, const_cast<float*>(x_scale), g, n_bits, per_sample,
                         nullptr, false, (cudaStream_t)stream, const_cast<float*>(x_zp));
}

namespace modiff {
int read_device_status_modq(int* status, int reset) {
  MODIFF_CUDA(cudaMemcpyFromSymbol(status, g_modq_status, sizeof(int)));
  if (reset) {
    int zero = 0;
    MODIFF_CUDA(cudaMemcpyToSymbol(g_modq_status, &zero, sizeof(int)));
  }
  return MODIFF_OK;
}
}  // namespace modiff

// ---------------------------------------------------------------------------------------
// Built-in scratch for callers that cannot allocate.
//
// The array below lives in every GPU that loads the library until the process exits.  Its
// name is only a host-side handle: the device address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and that address is what the kernels get.
constexpr int kStaticSlots = MODIFF_MODQ_STATIC_MAX_BATCH;
constexpr size_t kStaticScratchBytes = 64 + 4 * (size_t)kStaticSlots;
static __device__ __align__(256) unsigned char g_modq_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
void* g_static_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_static_scratch_mutex;

// Device address of the built-in scratch on the CURRENT device (looked up on first use).
int static_scratch_address(void** out) {
  int dev = 0;
  MODIFF_CUDA(cudaGetDevice(&dev));
  MODIFF_CHECK_ARG(dev >= 0 && dev < kMaxDevices, "device index %d beyond %d", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    MODIFF_CUDA(cudaGetSymbolAddress(&ptr, g_modq_static_scratch));
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return MODIFF_OK;
}
}  // namespace

extern "C" int modiff_modq_static(const float* x, float* a_hat, int8_t* codes, float* x_scale,
                                  const modiff_conv_geom* g, int n_bits, int per_sample,
                                  void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(x && codes && x_scale, "NULL pointer argument");
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 8, "activation n_bits %d outside [2, 8]", n_bits);
  MODIFF_CHECK_ARG(!(per_sample && g->split > 0), "per-sample scales cannot be combined with split");
  MODIFF_CHECK_ARG(((uintptr_t)codes & 15) == 0, "codes must be 16-byte aligned");
  const int slots = per_sample ? g->batch : 2;
  MODIFF_CHECK_ARG(slots <= kStaticSlots,
                   "per-sample batch %d needs more scratch than the built-in %d slots; use "
                   "modiff_modq with caller-owned scratch",
                   g->batch, kStaticSlots);
  void* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  // The array keeps whatever the previous call left (an interrupted call may leave partial
  // maxima), so the part this call uses is cleared first, in stream order.
  MODIFF_CUDA(cudaMemsetAsync(scratch, 0, 64 + 4 * (size_t)slots, s));
  return launch_modq(x, a_hat, codes, x_scale, g, n_bits, per_sample, scratch, true, s);
}

namespace modiff {
namespace {
// Gathers the receptive field of every output pixel from the code planes into one row:
// out[m][c * taps + tap] = code of input channel c at filter tap `tap` of output pixel m.
// Turns a convolution with very few input channels (the 3-channel input conv) into a dense
// K = cin*kh*kw GEMM that the tensor-core kernel can run as a 1x1 layer.
__global__ void im2col_codes_kernel(const int8_t* __restrict__ codes, int8_t* __restrict__ out,
                                    modiff_conv_geom g, Derived d, int out_stride) {
  const int howo = d.ho * d.wo;
  const int64_t total = (int64_t)g.batch * howo;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t m = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; m < total; m += stride) {
    const int n = (int)(m / howo), r = (int)(m % howo);
    const int oy = r / d.wo, ox = r % d.wo;
    int8_t* row = out + m * out_stride;
    for (int tap = 0; tap < d.taps; ++tap) {
      const int ry = tap / g.kw, rx = tap % g.kw;
      const int plane = (ry % g.stride) * g.stride + (rx % g.stride);
      const size_t pix = (((size_t)n * d.nplanes + plane) * d.hp + oy + ry / g.stride) * d.wp + ox +
                         rx / g.stride;
      const int8_t* src = codes + pix * d.cp;
      for (int c = 0; c < g.cin; ++c) row[c * d.taps + tap] = src[c];
    }
  }
}
}  // namespace
}  // namespace modiff

extern "C" int modiff_im2col_codes(const int8_t* codes, int8_t* out, const modiff_conv_geom* g,
                                   int out_stride, void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(codes && out, "NULL pointer argument");
  Derived d = derive(*g);
  MODIFF_CHECK_ARG(out_stride >= g->cin * d.taps, "out_stride %d < cin*kh*kw", out_stride);
  const int64_t total = (int64_t)g->batch * d.ho * d.wo;
  int64_t blocks = ceil_div64(total, 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  im2col_codes_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(codes, out, *g, d, out_stride);
  MODIFF_LAUNCH_CHECK("im2col_codes_kernel");
  return MODIFF_OK;
}

namespace modiff {
namespace {
// 16 channels of one plane cell per thread; cells that hold an input pixel are skipped.
__global__ void codes_fill_halo_kernel(int8_t* __restrict__ codes, const float* __restrict__ x_zp,
                                       modiff_conv_geom g, Derived d) {
  const int pieces = d.cp / 16;
  const int64_t total = (int64_t)g.batch * d.nplanes * d.hp * d.wp * pieces;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int z0 = (int)x_zp[0] - 128;
  const int z1 = g.split > 0 ? (int)x_zp[1] - 128 : z0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int piece = (int)(i % pieces);
    int64_t cell = i / pieces;
    const int xq = (int)(cell % d.wp);
    int64_t t = cell / d.wp;
    const int yq = (int)(t % d.hp);
    const int plane = (int)((t / d.hp) % d.nplanes);
    const int y = yq * g.stride + plane / g.stride - g.pad_t;
    const int x = xq * g.stride + plane % g.stride - g.pad_l;
    if (y >= 0 && y < g.h && x >= 0 && x < g.w) continue;
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      uint32_t word = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int c = piece * 16 + 4 * k + b;
        const int v = c < g.cin ? ((g.split > 0 && c >= g.split) ? z1 : z0) : 0;
        word |= (uint32_t)(v & 0xff) << (8 * b);
      }
      w[k] = word;
    }
    *reinterpret_cast<int4*>(codes + cell * d.cp + piece * 16) =
        make_int4((int)w[0], (int)w[1], (int)w[2], (int)w[3]);
  }
}

// stride 1: the padding cells are pad_t + pad_b full rows and pad_l + pad_r cells of every other
// row, enumerated directly (one thread per 16 channels of a padding cell)
__global__ void codes_fill_border_kernel(int8_t* __restrict__ codes, const float* __restrict__ x_zp,
                                         modiff_conv_geom g, Derived d, int cells_per_image) {
  const int pieces = d.cp / 16;
  const int per_image = cells_per_image * pieces;
  const int total = g.batch * per_image;
  const int z0 = (int)x_zp[0] - 128;
  const int z1 = g.split > 0 ? (int)x_zp[1] - 128 : z0;
  const int rows_full = (g.pad_t + g.pad_b) * d.wp;
  const int side = g.pad_l + g.pad_r;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int n = i / per_image;
    int k = i - n * per_image;
    const int piece = k % pieces;
    k /= pieces;
    int y, x;
    if (k < rows_full) {
      y = k / d.wp;
      x = k - y * d.wp;
      if (y >= g.pad_t) y += g.h;                 // bottom rows
    } else {
      k -= rows_full;
      y = g.pad_t + k / side;
      x = k % side;
      if (x >= g.pad_l) x += g.w;                 // right columns
    }
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t word = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int c = piece * 16 + 4 * q + b;
        const int v = c < g.cin ? ((g.split > 0 && c >= g.split) ? z1 : z0) : 0;
        word |= (uint32_t)(v & 0xff) << (8 * b);
      }
      w[q] = word;
    }
    const size_t cell = ((size_t)n * d.hp + y) * d.wp + x;
    *reinterpret_cast<int4*>(codes + cell * d.cp + piece * 16) =
        make_int4((int)w[0], (int)w[1], (int)w[2], (int)w[3]);
  }
}

__global__ void asym_bias_kernel(const float* __restrict__ x_scale, const float* __restrict__ x_zp,
                                 const float* __restrict__ w_scale,
                                 const int32_t* __restrict__ w_csum,
                                 const float* __restrict__ bias_in, float* __restrict__ bias_out,
                                 int cout, int nseg) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cout) return;
  float acc = bias_in ? bias_in[c] : 0.0f;
  for (int seg = 0; seg < nseg; ++seg) {
    const long long k = -(long long)((int)x_zp[seg] - 128) * (long long)w_csum[seg * cout + c];
    acc = __fadd_rn(acc, __fmul_rn((float)k, __fmul_rn(x_scale[seg], w_scale[seg * cout + c])));
  }
  bias_out[c] = acc;
}
}  // namespace
}  // namespace modiff

extern "C" int modiff_codes_fill_halo(int8_t* codes, const float* x_zp, const modiff_conv_geom* g,
                                      void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(codes && x_zp, "NULL pointer argument");
  MODIFF_CHECK_ARG(((uintptr_t)codes & 15) == 0, "codes must be 16-byte aligned");
  Derived d = derive(*g);
  if ((int64_t)d.nplanes * d.hp * d.wp == (int64_t)g->h * g->w) return MODIFF_OK;   // no padding cell
  if (g->stride == 1) {
    const int cells = d.hp * d.wp - g->h * g->w;
    const int64_t n = (int64_t)g->batch * cells * (d.cp / 16);
    if (n < (1ll << 31)) {
      int nb = (int)ceil_div64(n, 256);
      if (nb > 148 * 8) nb = 148 * 8;
      codes_fill_border_kernel<<<nb, 256, 0, (cudaStream_t)stream>>>(codes, x_zp, *g, d, cells);
      MODIFF_LAUNCH_CHECK("codes_fill_border_kernel");
      return MODIFF_OK;
    }
  }
  const int64_t total = (int64_t)g->batch * d.nplanes * d.hp * d.wp * (d.cp / 16);
  int64_t blocks = ceil_div64(total, 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  codes_fill_halo_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(codes, x_zp, *g, d);
  MODIFF_LAUNCH_CHECK("codes_fill_halo_kernel");
  return MODIFF_OK;
}

extern "C" int modiff_asym_bias(const float* x_scale, const float* x_zp, const float* w_scale,
                                const int32_t* w_csum, const float* bias_in, float* bias_out,
                                int cout, int nseg, void* stream) {
  MODIFF_CHECK_ARG(x_scale && x_zp && w_scale && w_csum && bias_out, "NULL pointer argument");
  MODIFF_CHECK_ARG(cout > 0 && (nseg == 1 || nseg == 2), "bad cout %d / nseg %d", cout, nseg);
  asym_bias_kernel<<<ceil_div(cout, 128), 128, 0, (cudaStream_t)stream>>>(
      x_scale, x_zp, w_scale, w_csum, bias_in, bias_out, cout, nseg);
  MODIFF_LAUNCH_CHECK("asym_bias_kernel");
  return MODIFF_OK;
}

extern "C" int modiff_quantize_static(const float* x, const float* delta, int8_t* codes,
                                      const modiff_conv_geom* g, int n_bits, void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(x && codes && delta, "NULL pointer argument");
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 8, "activation n_bits %d outside [2, 8]", n_bits);
  MODIFF_CHECK_ARG(((uintptr_t)codes & 15) == 0, "codes must be 16-byte aligned");
  return launch_modq(x, nullptr, codes, const_cast<float*>(delta), g, n_bits, 0, nullptr, false,
                     (cudaStream_t)stream);
}
