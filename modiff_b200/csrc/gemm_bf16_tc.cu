// Split-bf16 implicit GEMM on the 5th-generation tensor cores (sm_100a), fp32 accumulation.
//
// fp32 operands are carried as two bf16 planes (hi = bf16(x), lo = bf16(x - hi)); the products
// hi*hi, hi*lo, lo*hi are accumulated in fp32 in tensor memory, which keeps ~16 mantissa bits of
// each operand (relative error ~1e-5, far inside the 1e-3 per-layer bound).  Used for
//   - the first sampling step, where the reference multiplies UNQUANTISED activations with
//     fake-quantised weights (qdiff/quant_layer.py:326-327, 358-359): the weights' integer part
//     (q - zp, |.| <= 255) is exact in bf16 and delta_w[c] is applied in the epilogue;
//   - the attention matmuls, which the reference keeps in floating point
//     (qdiff/quant_block.py:344-360): here both operands are split and B differs per image.
// Same structure as the int8 kernel: TMA-fed 128-byte-swizzled shared-memory ring,
// tcgen05.mma.cta_group::1.kind::f16 (M=128, K=16 per instruction), double-buffered fp32
// accumulators in tensor memory, persistent warp-specialised CTAs, bounded mbarrier waits.
#include "common.cuh"
#include "tc_common.cuh"

namespace modiff {

namespace {

constexpr int kTileM = 128;
constexpr int kChunkBytes = 128;        // bytes of K per pipeline stage (64 bf16 elements)
constexpr int kChunkElems = 64;
constexpr int kATileBytes = kTileM * kChunkBytes;
constexpr int kBTileBytes = 128 * kChunkBytes;
constexpr int kStageBytes = kATileBytes + kBTileBytes;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + 32 * kEpiWarps;   // TMA warp, MMA warp, epilogue warps
constexpr int kStages = 6;

struct BfParams {
  modiff_conv_geom g;
  Derived d;
  int bw, bh, bn;                 // box of output pixels forming one M tile
  int tiles_w, tiles_h, tiles_n;
  int n_tiles, total_tiles;
  int umma_n;                     // accumulator columns per segment (multiple of 16, <= 128)
  int nseg;
  int nbuf, buf_cols, tmem_cols;
  int a_parts, b_parts, b_batched;
  int planes_per_part;            // stride*stride
  int kb;                         // B: K stride per tap in elements
  int a_bytes, b_bytes;           // bytes one tile copy delivers
  int chunks[2];                  // 64-element K chunks per tap of segment 0 / 1
  int cbeg[2];                    // first channel of segment 0 / 1
  int valid_rows;                 // rows of a tile that hold real pixels (batched mode)
  float scale;
  const float* col_scale;         // [nseg][cout] or NULL
  const float* bias;              // [cout] or NULL
  float* out;                     // fp32 [batch][cout][ho*wo]
};

struct TileCoord {
  int tn, th, tw, nt;
};
__device__ inline TileCoord decode_tile(int tile, const BfParams& p) {
  TileCoord t;
  t.nt = tile % p.n_tiles;
  int m = tile / p.n_tiles;
  t.tw = m % p.tiles_w;
  m /= p.tiles_w;
  t.th = m % p.tiles_h;
  t.tn = m / p.tiles_h;
  return t;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const BfParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];
  __shared__ __align__(8) uint64_t bar_tmem_full[2];
  __shared__ __align__(8) uint64_t bar_tmem_empty[2];
  __shared__ uint32_t tmem_base_sh;
  __shared__ int abort_sh;
  __shared__ float ep_scale[2][128];
  __shared__ float ep_bias[128];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &abort_sh;
  const uint32_t ring = smem_u32(smem_raw);

  if (threadIdx.x == 0) {
    abort_sh = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_tmem_full[b]), 1);
      mbar_init(smem_u32(&bar_tmem_empty[b]), kEpiWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_base_sh)),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_sh;
  const int products = p.a_parts * p.b_parts - ((p.a_parts == 2 && p.b_parts == 2) ? 1 : 0);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
        const TileCoord t = decode_tile(tile, p);
        const int img = t.tn * p.bn;
        for (int seg = 0; seg < p.nseg && ok; ++seg) {
          for (int pr = 0; pr < products && ok; ++pr) {
            // product order: (hi,hi), (hi,lo) or (lo,hi), (lo,hi); lo*lo is dropped
            const int pa = (p.b_parts == 2) ? (pr == 2 ? 1 : 0) : pr;
            const int pb = (p.b_parts == 2) ? (pr == 1 ? 1 : 0) : 0;
            for (int tap = 0; tap < p.d.taps && ok; ++tap) {
              const int r = tap / p.g.kw, sx = tap % p.g.kw;
              const int plane = (r % p.g.stride) * p.g.stride + (sx % p.g.stride);
              const int dh = r / p.g.stride, dw = sx / p.g.stride;
              for (int ch = 0; ch < p.chunks[seg]; ++ch) {
                ok = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_flag);
                if (!ok) break;
                const uint32_t full = smem_u32(&bar_full[stage]);
                const uint32_t a_dst = ring + stage * kStageBytes;
                const uint32_t b_dst = a_dst + kATileBytes;
                const int c0 = p.cbeg[seg] + ch * kChunkElems;
                mbar_arrive_expect_tx(full, (uint32_t)(p.a_bytes + p.b_bytes));
                tma_load_5d(a_dst, &map_a, full, c0, t.tw * p.bw + dw, t.th * p.bh + dh,
                            pa * p.planes_per_part + plane, img);
                tma_load_3d(b_dst, &map_b, full, tap * p.kb + c0, t.nt * 128,
                            (p.b_batched ? img * p.b_parts : 0) + pb);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
              }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // All lanes walk the loop (descriptors and addresses stay warp-uniform values); one
    // elected lane issues the MMAs and commits.
    {
      const uint32_t idesc = make_idesc_bf16(kTileM, p.umma_n);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t bphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
        ok = mbar_wait(smem_u32(&bar_tmem_empty[buf]), bphase ^ 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
        for (int seg = 0; seg < p.nseg; ++seg) {
          const uint32_t d_tmem = tmem_base + (uint32_t)(buf * p.buf_cols + seg * p.umma_n);
          const int iters = products * p.d.taps * p.chunks[seg];
          for (int it = 0; it < iters; ++it) {
            ok = mbar_wait(smem_u32(&bar_full[stage]), phase, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t a_src = ring + stage * kStageBytes;
            const uint64_t adesc = make_smem_desc(a_src);
            const uint64_t bdesc = make_smem_desc(a_src + kATileBytes);
            if (elect_one()) {
#pragma unroll
              for (int k = 0; k < kChunkBytes / 32; ++k)
                tc_mma_bf16(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                            (it > 0 || k > 0) ? 1u : 0u);
              tc_commit(smem_u32(&bar_empty[stage]));
            }
            __syncwarp();
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
        }
        if (!ok) break;
        if (elect_one()) tc_commit(smem_u32(&bar_tmem_full[buf]));
        __syncwarp();
        if (++buf == p.nbuf) { buf = 0; bphase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int ep_tid = threadIdx.x - 64;
    const int row = quarter * 32 + lane;
    const int howo = p.d.ho * p.d.wo;
    const int tile_px = p.bh * p.bw;
    const int ni = row / tile_px;
    const int pl = row % tile_px;
    const int hi = pl / p.bw, wi = pl % p.bw;
    int buf = 0;
    uint32_t bphase = 0;
    int last_nt = -1;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
      const TileCoord t = decode_tile(tile, p);
      if (t.nt != last_nt) {
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (ep_tid < 128) {
          const int co = t.nt * 128 + ep_tid;
          const bool cv = co < p.g.cout;
          for (int seg = 0; seg < p.nseg; ++seg)
            ep_scale[seg][ep_tid] =
                cv ? p.scale * (p.col_scale ? p.col_scale[seg * p.g.cout + co] : 1.0f) : 0.0f;
          ep_bias[ep_tid] = (cv && p.bias) ? p.bias[co] : 0.0f;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        last_nt = t.nt;
      }
      if (ok) ok = mbar_wait(smem_u32(&bar_tmem_full[buf]), bphase, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * p.buf_cols);
      const int n = t.tn * p.bn + ni;
      const int hw = (t.th * p.bh + hi) * p.d.wo + (t.tw * p.bw + wi);
      const bool valid = (n < p.g.batch) && (row < p.valid_rows);
#pragma unroll 1
      for (int c2 = 0; c2 < 2; ++c2) {
        const int col0 = half * 64 + c2 * 32;
        if (col0 >= p.umma_n) break;                 // narrow accumulators (few output columns)
        const int co0 = t.nt * 128 + col0;
        const int ncols = min(32, p.g.cout - co0);
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = ep_bias[col0 + j];
        for (int seg = 0; seg < p.nseg; ++seg) {
          int a[32];
          tc_ld32(t_row + seg * p.umma_n + col0, a);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fmaf(__int_as_float(a[j]), ep_scale[seg][col0 + j], v[j]);
        }
        if (valid) {
          float* obase = p.out + ((size_t)n * p.g.cout + co0) * howo + hw;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < ncols) obase[(size_t)j * howo] = v[j];
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_tmem_empty[buf]));
      if (++buf == p.nbuf) { buf = 0; bphase ^= 1u; }
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  if (abort_sh) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);   // let copies in flight land
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
  }
}

}  // namespace
}  // namespace modiff

// =====================================================================================
// Operand preparation: fp32 -> (hi, lo) bf16 planes
// =====================================================================================
namespace modiff {
namespace {

__device__ inline uint16_t bf16_rn(float x) {   // round to nearest even, NaN/Inf passed through
  uint32_t u = __float_as_uint(x);
  if ((u & 0x7f800000u) == 0x7f800000u) return (uint16_t)(u >> 16);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
__device__ inline float bf16_to_f(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }

constexpr int kSplitTileC = 64, kSplitTileP = 64;

// NCHW fp32 -> two NHWC bf16 planes in the code-plane geometry of `g` (halo, parity planes):
// out[image][part][plane][hp][wp][cp].  Same tile transpose as the int8 quantiser.
__global__ void __launch_bounds__(256)
split_bf16_planes_kernel(const float* __restrict__ x, uint16_t* __restrict__ out,
                         modiff_conv_geom g, Derived d, int cp, int pb, int cb, int total) {
  __shared__ uint32_t tile_sh[2][kSplitTileP][kSplitTileC / 2 + 1];   // [part][pixel][channel pair]
  const int hw = g.h * g.w;
  const int cg = threadIdx.x >> 4;   // channel group: 4 channels
  const int pq = threadIdx.x & 15;   // pixel quad
  const size_t part_stride = (size_t)d.nplanes * d.hp * d.wp * cp;
  const bool vec4 = (hw % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
    const int n = tile / (pb * cb);
    const int rem = tile % (pb * cb);
    const int c0 = (rem / pb) * kSplitTileC;
    const int p0 = (rem % pb) * kSplitTileP;
    const int p = p0 + 4 * pq;
    uint16_t hi[4][4], lo[4][4];
    float xv[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {      // all loads first: sixteen values, four 16-byte loads
      const int c = c0 + 4 * cg + i;
      const float* src = x + ((size_t)n * g.cin + c) * hw + p;
      if (vec4 && c < g.cin && p < hw) {
        const float4 f = __ldg(reinterpret_cast<const float4*>(src));
        xv[i][0] = f.x; xv[i][1] = f.y; xv[i][2] = f.z; xv[i][3] = f.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) xv[i][j] = (c < g.cin && p + j < hw) ? __ldg(src + j) : 0.0f;
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        hi[i][j] = bf16_rn(xv[i][j]);
        lo[i][j] = bf16_rn(xv[i][j] - bf16_to_f(hi[i][j]));
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      tile_sh[0][4 * pq + j][2 * cg] = (uint32_t)hi[0][j] | ((uint32_t)hi[1][j] << 16);
      tile_sh[0][4 * pq + j][2 * cg + 1] = (uint32_t)hi[2][j] | ((uint32_t)hi[3][j] << 16);
      tile_sh[1][4 * pq + j][2 * cg] = (uint32_t)lo[0][j] | ((uint32_t)lo[1][j] << 16);
      tile_sh[1][4 * pq + j][2 * cg + 1] = (uint32_t)lo[2][j] | ((uint32_t)lo[3][j] << 16);
    }
    __syncthreads();
    // 4 threads per pixel; each writes 16 channels (32 bytes) of both parts
    const int px = threadIdx.x >> 2;
    const int piece = threadIdx.x & 3;
    const int pp = p0 + px;
    const int cbase = c0 + 16 * piece;
    if (pp < hw && cbase < cp) {
      const int y = pp / g.w + g.pad_t;
      const int xq = pp % g.w + g.pad_l;
      const int plane = (y % g.stride) * g.stride + (xq % g.stride);
      const size_t pix = ((size_t)plane * d.hp + y / g.stride) * d.wp + xq / g.stride;
      for (int part = 0; part < 2; ++part) {
        uint16_t* dst = out + ((size_t)n * 2 + part) * part_stride + pix * cp + cbase;
        const int nvalid = min(16, cp - cbase);     // cp is a multiple of 8
        for (int k = 0; k < nvalid; k += 8) {
          int4 v = make_int4(tile_sh[part][px][8 * piece + k / 2], tile_sh[part][px][8 * piece + k / 2 + 1],
                             tile_sh[part][px][8 * piece + k / 2 + 2], tile_sh[part][px][8 * piece + k / 2 + 3]);
          *reinterpret_cast<int4*>(dst + k) = v;
        }
      }
    }
    __syncthreads();
  }
}

// x[nb][rows][len] fp32 -> out[nb][2][rows_pad][len_pad] bf16 (zero padding, no transposition).
// One thread converts eight consecutive elements of a row (two 16-byte loads, two 16-byte
// stores); VEC8 needs len and len_pad to be multiples of 8 and 16-byte aligned buffers.
template <bool VEC8>
__global__ void __launch_bounds__(256)
split_bf16_rows_kernel(const float* __restrict__ x, uint16_t* __restrict__ out, int64_t nb,
                       int rows, int len, int rows_pad, int len_pad) {
  const int groups = (len_pad + 7) / 8;                 // 8-element groups per padded row
  const int64_t total = nb * rows_pad * groups;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t plane = (int64_t)rows_pad * len_pad;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t row = i / groups;                     // b * rows_pad + r
    const int c0 = (int)(i - row * groups) * 8;
    const int64_t b = row / rows_pad;
    const int r = (int)(row - b * rows_pad);
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = 0.0f;
    if (r < rows) {
      const float* src = x + (b * rows + r) * (int64_t)len + c0;
      if (VEC8) {
        if (c0 < len) {
          const float4 a = __ldg(reinterpret_cast<const float4*>(src));
          const float4 c = __ldg(reinterpret_cast<const float4*>(src) + 1);
          v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
          v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
        }
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (c0 + k < len) v[k] = __ldg(src + k);
      }
    }
    uint16_t h[8], l[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      h[k] = bf16_rn(v[k]);
      l[k] = bf16_rn(v[k] - bf16_to_f(h[k]));
    }
    uint16_t* dst = out + (b * 2 * rows_pad + r) * (int64_t)len_pad + c0;
    if (VEC8) {
      uint4 hv, lv;
      hv.x = h[0] | ((uint32_t)h[1] << 16); hv.y = h[2] | ((uint32_t)h[3] << 16);
      hv.z = h[4] | ((uint32_t)h[5] << 16); hv.w = h[6] | ((uint32_t)h[7] << 16);
      lv.x = l[0] | ((uint32_t)l[1] << 16); lv.y = l[2] | ((uint32_t)l[3] << 16);
      lv.z = l[4] | ((uint32_t)l[5] << 16); lv.w = l[6] | ((uint32_t)l[7] << 16);
      *reinterpret_cast<uint4*>(dst) = hv;
      *reinterpret_cast<uint4*>(dst + plane) = lv;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (c0 + k < len_pad) {
          dst[k] = h[k];
          dst[k + plane] = l[k];
        }
    }
  }
}

// Softmax over keys of S[image][key][query] (the layout the GEMM epilogue writes: keys are the
// output "channels") -> probabilities as split bf16 planes P[image][2][query][key], the A
// operand of the second attention GEMM (qdiff/quant_block.py:353-358).
// A block owns 32 queries; a thread owns one query and every eighth key.  With at most
// kSmRegKeys keys the scores are read ONCE into registers (exp evaluated once per score).
constexpr int kSmQ = 32, kSmKeys = 256, kSmRegKeys = 256;
template <bool IN_REGS>
__global__ void __launch_bounds__(256)
softmax_split_kernel(const float* __restrict__ s, uint16_t* __restrict__ p, int tk, int tq,
                     int tk_pad) {
  __shared__ float red[8][kSmQ];
  __shared__ uint16_t stage[2][kSmQ][kSmKeys + 2];   // odd word pitch: conflict-free columns
  const int b = blockIdx.y;
  const int q0 = blockIdx.x * kSmQ;
  const int q = threadIdx.x & 31, kg = threadIdx.x >> 5;
  const bool qv = (q0 + q) < tq;
  const float* sb = s + (size_t)b * tk * tq + q0 + q;
  float e[IN_REGS ? kSmRegKeys / 8 : 1];
  float mx = -INFINITY;
  if (IN_REGS) {
#pragma unroll
    for (int i = 0; i < kSmRegKeys / 8; ++i) {
      const int k = kg + 8 * i;
      e[i] = (qv && k < tk) ? __ldg(sb + (size_t)k * tq) : -INFINITY;
      mx = fmaxf(mx, e[i]);
    }
  } else if (qv) {
    for (int k = kg; k < tk; k += 8) mx = fmaxf(mx, __ldg(sb + (size_t)k * tq));
  }
  red[kg][q] = mx;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 8; ++i) mx = fmaxf(mx, red[i][q]);
  __syncthreads();
  float sum = 0.0f;
  if (IN_REGS) {
#pragma unroll
    for (int i = 0; i < kSmRegKeys / 8; ++i) {
      e[i] = (qv && kg + 8 * i < tk) ? expf(e[i] - mx) : 0.0f;
      sum += e[i];
    }
  } else if (qv) {
    for (int k = kg; k < tk; k += 8) sum += expf(__ldg(sb + (size_t)k * tq) - mx);
  }
  red[kg][q] = sum;
  __syncthreads();
  sum = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) sum += red[i][q];
  const float inv = 1.0f / sum;
  for (int k0 = 0; k0 < tk_pad; k0 += kSmKeys) {
    __syncthreads();
    if (IN_REGS) {
#pragma unroll
      for (int i = 0; i < kSmRegKeys / 8; ++i) {
        const int k = kg + 8 * i;
        if (k < tk_pad) {
          const float pv = e[i] * inv;
          const uint16_t h = bf16_rn(pv);
          stage[0][q][k] = h;
          stage[1][q][k] = bf16_rn(pv - bf16_to_f(h));
        }
      }
    } else {
      for (int k = kg; k < kSmKeys && k0 + k < tk_pad; k += 8) {
        const float pv =
            (qv && k0 + k < tk) ? expf(__ldg(sb + (size_t)(k0 + k) * tq) - mx) * inv : 0.0f;
        const uint16_t h = bf16_rn(pv);
        stage[0][q][k] = h;
        stage[1][q][k] = bf16_rn(pv - bf16_to_f(h));
      }
    }
    __syncthreads();
    // each warp writes whole query rows: contiguous keys, 4 bytes per lane when aligned
    const int nk = min(kSmKeys, tk_pad - k0);
    for (int r = kg; r < kSmQ; r += 8) {
      if (q0 + r >= tq) continue;
      for (int part = 0; part < 2; ++part) {
        uint16_t* dst = p + (((size_t)b * 2 + part) * tq + q0 + r) * tk_pad + k0;
        if ((nk & 1) == 0 && (tk_pad & 1) == 0) {
          for (int k = 2 * q; k < nk; k += 64)
            *reinterpret_cast<uint32_t*>(dst + k) =
                *reinterpret_cast<const uint32_t*>(&stage[part][r][k]);
        } else {
          for (int k = q; k < nk; k += 32) dst[k] = stage[part][r][k];
        }
      }
    }
  }
}

// Integer weight values (q - zp, exact in bf16) as the B operand: out[cout][taps][kb].
__global__ void weights_bf16_kernel(const float* __restrict__ w, const float* __restrict__ alpha,
                                    const float* __restrict__ w_scale,
                                    const float* __restrict__ w_zp, uint16_t* __restrict__ out,
                                    modiff_conv_geom g, int taps, int kb, int n_bits) {
  const int co = blockIdx.x;
  const float qmax = (float)((1 << n_bits) - 1);
  for (int i = threadIdx.x; i < g.cin * taps; i += blockDim.x) {
    const int c = i / taps, tap = i % taps;
    const int seg = (g.split > 0 && c >= g.split) ? 1 : 0;
    const float delta = w_scale[seg * g.cout + co], zp = w_zp[seg * g.cout + co];
    const float v = w[((size_t)co * g.cin + c) * taps + tap];
    float xi = rintf(__fdiv_rn(v, delta));
    if (alpha)   // learned rounding: floor plus the hard target
      xi = __fadd_rn(floorf(__fdiv_rn(v, delta)),
                     alpha[((size_t)co * g.cin + c) * taps + tap] >= 0.0f ? 1.0f : 0.0f);
    const float q = fminf(fmaxf(__fadd_rn(xi, zp), 0.0f), qmax);
    out[((size_t)co * taps + tap) * kb + c] = bf16_rn(__fsub_rn(q, zp));
  }
}

}  // namespace
}  // namespace modiff

// =====================================================================================
// Host side
// =====================================================================================
namespace modiff {

int read_device_status_bf16(int* status, int reset) { return read_status_this_unit(status, reset); }

namespace {
inline bool pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }
inline int bf16_cp(int cin) { return cin < 64 ? 64 : round_up(cin, 8); }   // >= one K chunk
}  // namespace

}  // namespace modiff

using namespace modiff;

extern "C" int64_t modiff_bf16_planes_bytes(const modiff_conv_geom* g) {
  if (!g) return 0;
  Derived d = derive(*g);
  return (int64_t)g->batch * 2 * d.nplanes * d.hp * d.wp * bf16_cp(g->cin) * 2;
}

extern "C" int64_t modiff_weights_bf16_bytes(const modiff_conv_geom* g) {
  if (!g) return 0;
  Derived d = derive(*g);
  return (int64_t)g->cout * d.taps * bf16_cp(g->cin) * 2;
}

extern "C" int modiff_split_bf16(const float* x, uint16_t* planes, const modiff_conv_geom* g,
                                 void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(x && planes, "NULL pointer argument");
  MODIFF_CHECK_ARG(((uintptr_t)planes & 15) == 0, "planes must be 16-byte aligned");
  Derived d = derive(*g);
  const int hw = g->h * g->w;
  if (hw == 1 && d.nplanes * d.hp * d.wp == 1)
    // token-major linear layer: the planes are [token][2][cp], i.e. one padded row per token
    return modiff_split_bf16_rows(x, planes, g->batch, 1, g->cin, 1, bf16_cp(g->cin), stream);
  const int pb = ceil_div(hw, kSplitTileP), cb = ceil_div(g->cin, kSplitTileC);
  const int64_t total = (int64_t)pb * cb * g->batch;
  MODIFF_CHECK_ARG(total < (1ll << 31), "activation tensor too large");
  const int blocks = total < 148 * 8 ? (int)total : 148 * 8;
  split_bf16_planes_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(x, planes, *g, d, bf16_cp(g->cin),
                                                                   pb, cb, (int)total);
  MODIFF_LAUNCH_CHECK("split_bf16_planes_kernel");
  return MODIFF_OK;
}

extern "C" int modiff_split_bf16_rows(const float* x, uint16_t* out, int64_t nb, int rows, int len,
                                      int rows_pad, int len_pad, void* stream) {
  MODIFF_CHECK_ARG(x && out && nb > 0 && rows > 0 && len > 0 && rows_pad >= rows && len_pad >= len,
                   "bad argument");
  int64_t blocks = ceil_div64(nb * rows_pad * ((len_pad + 7) / 8), 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  const bool vec = (len % 8 == 0) && (len_pad % 8 == 0) &&
                   ((((uintptr_t)x | (uintptr_t)out) & 15) == 0);
  if (vec)
    split_bf16_rows_kernel<true><<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
        x, out, nb, rows, len, rows_pad, len_pad);
  else
    split_bf16_rows_kernel<false><<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
        x, out, nb, rows, len, rows_pad, len_pad);
  MODIFF_LAUNCH_CHECK("split_bf16_rows_kernel");
  return MODIFF_OK;
}

extern "C" int modiff_weights_bf16(const float* w, const float* w_scale, const float* w_zp,
                                   uint16_t* out, const modiff_conv_geom* g, int n_bits,
                                   void* stream) {
  return modiff_weights_bf16_rounded(w, nullptr, w_scale, w_zp, out, g, n_bits, stream);
}

extern "C" int modiff_weights_bf16_rounded(const float* w, const float* alpha, const float* w_scale,
                                           const float* w_zp, uint16_t* out,
                                           const modiff_conv_geom* g, int n_bits, void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(w && w_scale && w_zp && out, "NULL pointer argument");
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 8, "weight n_bits %d outside [2, 8]", n_bits);
  Derived d = derive(*g);
  cudaStream_t s = (cudaStream_t)stream;
  MODIFF_CUDA(cudaMemsetAsync(out, 0, (size_t)modiff_weights_bf16_bytes(g), s));
  weights_bf16_kernel<<<g->cout, 256, 0, s>>>(w, alpha, w_scale, w_zp, out, *g, d.taps,
                                             bf16_cp(g->cin), n_bits);
  MODIFF_LAUNCH_CHECK("weights_bf16_kernel");
  return MODIFF_OK;
}

extern "C" int modiff_softmax_split(const float* s, uint16_t* p, int batch, int tk, int tq,
                                    int tk_pad, void* stream) {
  MODIFF_CHECK_ARG(s && p && batch > 0 && tk > 0 && tq > 0 && tk_pad >= tk, "bad argument");
  MODIFF_CHECK_ARG(batch <= 65535, "batch*heads %d exceeds the grid limit 65535", batch);
  dim3 grid(ceil_div(tq, kSmQ), batch);
  if (tk_pad <= kSmRegKeys)
    softmax_split_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(s, p, tk, tq, tk_pad);
  else
    softmax_split_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(s, p, tk, tq, tk_pad);
  MODIFF_LAUNCH_CHECK("softmax_split_kernel");
  return MODIFF_OK;
}

extern "C" int modiff_gemm_bf16(const modiff_gemm_bf16_desc* desc, const modiff_conv_geom* g,
                                void* stream) {
  int rc = validate_geom(g);
  if (rc) return rc;
  MODIFF_CHECK_ARG(desc && desc->a && desc->b && desc->out, "NULL pointer argument");
  MODIFF_CHECK_ARG((desc->a_parts == 1 || desc->a_parts == 2) &&
                       (desc->b_parts == 1 || desc->b_parts == 2),
                   "operand parts must be 1 or 2");
  Derived d = derive(*g);
  const int cp = bf16_cp(g->cin);
  const int b_rows = desc->b_rows > 0 ? desc->b_rows : g->cout;
  if (g->cin < 8 || g->cin % 8 || g->cout < 16 || b_rows < (g->cout >= 128 ? g->cout : round_up(g->cout, 16)) || !pow2(d.wo) || !pow2(d.ho) || d.wo > 128 ||
      g->split % 64 || g->kh > 7 || g->kw > 7 || desc->kb % 8 || desc->kb < g->cin)
    return set_error(MODIFF_ERR_UNSUPPORTED,
                     "bf16 tensor-core path needs cin a multiple of 8, cout >= 16 (B rows padded to a "
                     "multiple of 16), power-of-two output sizes <= 128, split %% 64 == 0");
  EncodeTiledFn encode = get_encode_fn();
  if (!encode) return set_error(MODIFF_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is not available");

  BfParams p;
  p.g = *g;
  p.d = d;
  p.bw = d.wo < 128 ? d.wo : 128;
  p.bh = (d.ho < 128 / p.bw) ? d.ho : 128 / p.bw;
  p.bn = desc->b_batched ? 1 : 128 / (p.bw * p.bh);
  p.valid_rows = desc->b_batched ? p.bw * p.bh : 128;
  p.tiles_w = d.wo / p.bw;
  p.tiles_h = d.ho / p.bh;
  p.tiles_n = ceil_div(g->batch, p.bn);
  p.n_tiles = ceil_div(g->cout, 128);
  p.total_tiles = p.tiles_w * p.tiles_h * p.tiles_n * p.n_tiles;
  p.umma_n = g->cout >= 128 ? 128 : round_up(g->cout, 16);
  p.nseg = d.nseg;
  p.buf_cols = round_up(p.nseg * p.umma_n, 32);
  const int slack = (p.umma_n % 32) ? 32 : 0;
  p.nbuf = (2 * p.buf_cols + slack <= 512) ? 2 : 1;
  p.tmem_cols = 32;
  while (p.tmem_cols < p.nbuf * p.buf_cols + slack) p.tmem_cols *= 2;
  p.a_parts = desc->a_parts;
  p.b_parts = desc->b_parts;
  p.b_batched = desc->b_batched ? 1 : 0;
  p.planes_per_part = d.nplanes;
  p.kb = desc->kb;
  p.cbeg[0] = 0;
  p.cbeg[1] = g->split;
  p.chunks[0] = ceil_div(p.nseg == 2 ? g->split : g->cin, kChunkElems);
  p.chunks[1] = p.nseg == 2 ? ceil_div(g->cin - g->split, kChunkElems) : 0;
  p.scale = desc->scale;
  p.col_scale = desc->col_scale;
  p.bias = desc->bias;
  p.out = desc->out;

  CUtensorMap map_a, map_b;
  {
    const int bn_box = p.bn < g->batch ? p.bn : g->batch;
    p.a_bytes = kChunkBytes * p.bw * p.bh * bn_box;
    const cuuint64_t plane_b = (cuuint64_t)d.hp * d.wp * cp * 2;
    cuuint64_t dims[5] = {(cuuint64_t)cp, (cuuint64_t)d.wp, (cuuint64_t)d.hp,
                          (cuuint64_t)(p.a_parts * d.nplanes), (cuuint64_t)g->batch};
    cuuint64_t strides[4] = {(cuuint64_t)cp * 2, (cuuint64_t)d.wp * cp * 2, plane_b,
                             plane_b * p.a_parts * d.nplanes};
    cuuint32_t box[5] = {(cuuint32_t)kChunkElems, (cuuint32_t)p.bw, (cuuint32_t)p.bh, 1u,
                         (cuuint32_t)bn_box};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = encode(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, (void*)desc->a, dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return set_error(MODIFF_ERR_CUDA, "cuTensorMapEncodeTiled(bf16 A planes) failed: %d", (int)r);
  }
  {
    const cuuint64_t row_b = (cuuint64_t)d.taps * p.kb * 2;
    const int zcount = (p.b_batched ? g->batch : 1) * p.b_parts;
    cuuint64_t dims[3] = {(cuuint64_t)d.taps * p.kb, (cuuint64_t)b_rows, (cuuint64_t)zcount};
    cuuint64_t strides[2] = {row_b, row_b * b_rows};
    cuuint32_t box[3] = {(cuuint32_t)kChunkElems, (cuuint32_t)p.umma_n, 1u};
    cuuint32_t estr[3] = {1, 1, 1};
    p.b_bytes = p.umma_n * kChunkBytes;
    CUresult r = encode(&map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, (void*)desc->b, dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return set_error(MODIFF_ERR_CUDA, "cuTensorMapEncodeTiled(bf16 B operand) failed: %d", (int)r);
  }

  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    MODIFF_CUDA(cudaGetDevice(&dev));
    MODIFF_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  const size_t smem = (size_t)kStages * kStageBytes;
  static SmemLimit smem_limit;
  MODIFF_CUDA(raise_smem_limit(gemm_bf16_kernel, smem, smem_limit));
  const int grid = p.total_tiles < sm_count ? p.total_tiles : sm_count;
  gemm_bf16_kernel<<<grid, kThreads, smem, (cudaStream_t)stream>>>(map_a, map_b, p);
  MODIFF_LAUNCH_CHECK("gemm_bf16_kernel");
  return MODIFF_OK;
}
