// Integer attention on the tensor cores (tcgen05.mma kind::i8), opt-in.
//
// The reference constructs 8-bit quantisers for q, k, v and for the softmax output on every
// attention block (qdiff/quant_block.py:120-121, 139-144, 223-235, 331-335) but its forward
// passes keep both products in floating point (:123-128, 146-148, 181-203, 338-366).  This
// file applies them: q, k, v through per-tensor symmetric dynamic quantisers, the softmax
// output through an unsigned 8-bit quantiser with zero point 0, both products as int8 MMAs
// with int32 accumulation, the softmax itself in fp32.  The floating-point kernel
// (attention_tc.cu) stays the default; the exact definition is restated on the CPU in
// oracle/attention_i8.py.
//
//   modiff_attn_quantize   absmax of q, k, v (one launch), then codes in the layouts the MMAs
//                          read: q / k token-major [head][token][dp] (dp = channels padded to
//                          32, 64, 128 or 256 bytes), v channel-major [head][d_rows][keys padded
//                          to 128]
//   modiff_attention_i8    per 128-query tile and head, keys in blocks of 128:
//        pass A  S = q_int k_int^T (M = 128, N = 128) into tensor memory, double buffered;
//                the softmax warps keep the exact integer row maximum m;
//        pass B  S again; w = rne(255 * exp2((S - m) * c2)) written as the u8 A operand of the
//                second product straight into shared memory (128-byte-swizzled K-major rows);
//                O += w v_int^T (u8 x s8) in tensor memory; l = sum w (integer);
//        end     out = O * (dv / l).
// Knowing the exact maximum before any probability is formed makes every weight, and hence the
// result, independent of the order of the key blocks; the price is the first product computed
// twice, which is small next to the exponentials.  Scores and weights never leave the SM.
// Every mbarrier wait is bounded.
#include "common.cuh"
#include "tc_common.cuh"

#include <limits.h>

namespace modiff {
namespace {

// Bytes of a q / k code row: the head's channels padded to 32, 64, 128 or 256.  Rows of up to 128
// bytes are one tile row in shared memory (32-, 64- or 128-byte swizzle); 256 bytes are two chunks.
inline int attn_row_bytes(int c) { return c <= 32 ? 32 : c <= 64 ? 64 : c <= 128 ? 128 : 256; }

// ---------------------------------------------------------------------------------- quantise
struct TensorView {
  const float* x;
  long long sb, sh, sc, st;      // element strides of (image, head, channel, token)
  int t;                         // tokens
};

struct QuantParams {
  TensorView tv[3];              // q, k, v
  int batch, heads, c;
  int n_levels;
  float* scales;                 // [3] out: delta of q, k, v
  unsigned int* scratch;         // [4]: absmax bits of q, k, v and a block counter; left zeroed
  int8_t* codes[3];
  int dp, d_rows, tkp;
  long long dense[3];            // element count when the tensor is one dense block, else 0
};

__device__ inline const float* elem(const TensorView& v, int b, int h, int c, int t) {
  return v.x + (long long)b * v.sb + (long long)h * v.sh + (long long)c * v.sc + (long long)t * v.st;
}

// grid (blocks, 3): tensor blockIdx.y; every block sweeps rows of the unit-stride dimension
__global__ void __launch_bounds__(256) attn_absmax_kernel(const QuantParams p) {
  const TensorView tv = p.tv[blockIdx.y];
  const bool cmajor = tv.st == 1;            // tokens contiguous, else channels contiguous
  const int inner = cmajor ? tv.t : p.c;
  const int outer = cmajor ? p.c : tv.t;
  const long long rows = (long long)p.batch * p.heads * outer;
  float mx = 0.0f;
  if (p.dense[blockIdx.y] > 0) {
    // every element of a dense block belongs to the tensor: one flat vectorised sweep
    const long long n4 = p.dense[blockIdx.y] >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(tv.x);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
      const float4 v = __ldg(x4 + i);
      mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
    }
  } else if (inner % 4 == 0 && ((tv.sb | tv.sh | (cmajor ? tv.sc : tv.st)) & 3) == 0 &&
             (reinterpret_cast<uintptr_t>(tv.x) & 15) == 0) {
    // rows of the contiguous dimension, 16 bytes per load; short rows share a block
    const int inner4 = inner >> 2;
    const int rpb = inner4 >= 256 ? 1 : 256 / inner4;
    const int sub = inner4 >= 256 ? 0 : (int)threadIdx.x / inner4;
    const int col0 = inner4 >= 256 ? (int)threadIdx.x : (int)threadIdx.x % inner4;
    const int step = inner4 >= 256 ? 256 : inner4;
    if (sub < rpb) {
      for (long long r = (long long)blockIdx.x * rpb + sub; r < rows; r += (long long)gridDim.x * rpb) {
        const int o = (int)(r % outer);
        const int bh = (int)(r / outer);
        const int b = bh / p.heads, h = bh % p.heads;
        const float4* base =
            reinterpret_cast<const float4*>(cmajor ? elem(tv, b, h, o, 0) : elem(tv, b, h, 0, o));
        for (int i = col0; i < inner4; i += step) {
          const float4 v = __ldg(base + i);
          mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
        }
      }
    }
  } else {
    // rows of the contiguous dimension; short rows share a block (256 / inner rows at a time)
    const int rpb = inner >= 256 ? 1 : 256 / inner;
    const int sub = inner >= 256 ? 0 : (int)threadIdx.x / inner;
    const int col0 = inner >= 256 ? (int)threadIdx.x : (int)threadIdx.x % inner;
    const int step = inner >= 256 ? 256 : inner;
    if (sub < rpb) {
      for (long long r = (long long)blockIdx.x * rpb + sub; r < rows; r += (long long)gridDim.x * rpb) {
        const int o = (int)(r % outer);
        const int bh = (int)(r / outer);
        const int b = bh / p.heads, h = bh % p.heads;
        const float* base = cmajor ? elem(tv, b, h, o, 0) : elem(tv, b, h, 0, o);
        for (int i = col0; i < inner; i += step) mx = fmaxf(mx, fabsf(__ldg(base + i)));
      }
    }
  }
  __shared__ float red[8];
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
    atomicMax(&p.scratch[blockIdx.y], __float_as_uint(mx));     // non-negative floats order as uints
    __threadfence();
    const unsigned int done = atomicAdd(&p.scratch[3], 1u) + 1u;
    if (done == gridDim.x * gridDim.y) {
      // last block: delta = absmax / n_levels in double, floor 1e-8, rounded to fp32
      // (qdiff/quant_layer.py:197-213, Python-float arithmetic)
      for (int k = 0; k < 3; ++k) {
        const float am = __uint_as_float(atomicExch(&p.scratch[k], 0u));
        double d = (double)am / (double)p.n_levels;
        if (d < 1e-8) d = 1e-8;
        p.scales[k] = (float)d;
      }
      p.scratch[3] = 0u;
    }
  }
}

// clamp(rne(fl(x / delta)), lo, hi): multiplication by rn(1 / delta) wherever that provably gives
// the same integer as the division, the division itself within 2^-14 of a tie (the argument of
// modq.cu's quantise_clamp)
__device__ inline int quantise_code(float x, float delta, float inv, float lo, float hi) {
  const float tc = fminf(fmaxf(__fmul_rn(x, inv), lo), hi);
  float u = __fadd_rn(tc, 12582912.0f);
  float qf = __fadd_rn(u, -12582912.0f);
  if (fabsf(__fsub_rn(tc, qf)) > 0.5f - 6.103515625e-5f) {
    const float te = fminf(fmaxf(__fdiv_rn(x, delta), lo), hi);
    u = __fadd_rn(te, 12582912.0f);
    qf = __fadd_rn(u, -12582912.0f);
  }
  return (int)qf;
}

// grid (token tiles of 64, channel tiles of 64, heads * 3): one 64 x 64 tile of one tensor,
// quantised on the way in (four values of the contiguous dimension per load where alignment
// allows), transposed in shared memory where the output layout differs, written 16 bytes per
// thread
__global__ void __launch_bounds__(256) attn_encode_kernel(const QuantParams p) {
  __shared__ __align__(16) int8_t tile[64][80];            // [channel][token], rows 16-byte aligned
  const int which = blockIdx.z % 3;
  const int bh = blockIdx.z / 3;
  const TensorView tv = p.tv[which];
  const int b = bh / p.heads, h = bh % p.heads;
  const int t0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
  const bool is_v = which == 2;
  // extent of the output in this tile's coordinates
  const int t_out = is_v ? p.tkp : tv.t;
  const int c_out = is_v ? p.d_rows : p.dp;
  if (t0 >= t_out || c0 >= c_out) return;
  const float delta = p.scales[which];
  const float inv = __frcp_rn(delta);
  const float lo = (float)(-p.n_levels - 1), hi = (float)p.n_levels;
  const bool cmajor = tv.st == 1;
  const int a4 = (threadIdx.x & 15) * 4, g = threadIdx.x >> 4;    // 16 x 4 along the contiguous dim
  // four consecutive elements of the contiguous dimension are one aligned 16-byte load when the
  // other strides and the base keep that alignment
  const bool vec = (((tv.sb | tv.sh | (cmajor ? tv.sc : tv.st)) & 3) == 0) &&
                   (((uintptr_t)tv.x & 15) == 0) && ((cmajor ? tv.t : p.c) % 4 == 0);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int o = g + 16 * i;                       // index along the strided dimension
    const int c = cmajor ? c0 + o : c0 + a4;
    const int t = cmajor ? t0 + a4 : t0 + o;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    const int inner_left = cmajor ? tv.t - t : p.c - c;
    const bool row_ok = cmajor ? c < p.c : t < tv.t;
    if (row_ok && inner_left > 0) {
      const float* src = elem(tv, b, h, c, t);
      if (vec && inner_left >= 4) {
        const float4 f = __ldg(reinterpret_cast<const float4*>(src));
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (e < inner_left) v[e] = __ldg(src + e);
      }
    }
    int q[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) q[e] = quantise_code(v[e], delta, inv, lo, hi);   // 0 -> 0
    if (cmajor) {
      *reinterpret_cast<uint32_t*>(&tile[o][a4]) =
          (uint32_t)(uint8_t)q[0] | ((uint32_t)(uint8_t)q[1] << 8) |
          ((uint32_t)(uint8_t)q[2] << 16) | ((uint32_t)(uint8_t)q[3] << 24);
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) tile[a4 + e][o] = (int8_t)q[e];
    }
  }
  __syncthreads();
  const int part = threadIdx.x & 3, row = threadIdx.x >> 2;    // 4 x 16 bytes per row, 64 rows
  if (is_v) {
    // [head][channel row][key]: rows are channels, sixteen consecutive keys per thread
    const int c = c0 + row, t = t0 + 16 * part;
    if (c < p.d_rows && t < p.tkp)
      *reinterpret_cast<uint4*>(p.codes[2] + ((size_t)bh * p.d_rows + c) * p.tkp + t) =
          *reinterpret_cast<const uint4*>(&tile[row][16 * part]);
  } else {
    // [head][token][dp]: rows are tokens, sixteen consecutive channels per thread
    const int t = t0 + row, c = c0 + 16 * part;
    if (t < tv.t && c < p.dp) {
      uint32_t w[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        w[k] = (uint32_t)(uint8_t)tile[16 * part + 4 * k][row] |
               ((uint32_t)(uint8_t)tile[16 * part + 4 * k + 1][row] << 8) |
               ((uint32_t)(uint8_t)tile[16 * part + 4 * k + 2][row] << 16) |
               ((uint32_t)(uint8_t)tile[16 * part + 4 * k + 3][row] << 24);
      *reinterpret_cast<uint4*>(p.codes[which] + ((size_t)bh * tv.t + t) * p.dp + c) =
          make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// ---------------------------------------------------------------------------------- attention
constexpr int kRowBytes = 128;
constexpr int kTile = 128 * kRowBytes;           // 16 KB: 128 rows x 128 bytes
constexpr int kStageBytes = 256 * kRowBytes;     // 32 KB: a key tile (16 KB) or a v tile (<= 32 KB)
constexpr int kStages = 4;
constexpr int kEpiWarps = 16;               // softmax warps: kParts per tensor-memory lane quarter
constexpr int kParts = kEpiWarps / 4;       // each takes 128 / kParts keys of a block
constexpr int kPartCols = 128 / kParts;     // 32
constexpr int kCtlWarps = 4;                // copy producer, score MMAs, weighted-sum MMAs, (idle)
constexpr int kThreads = 32 * (kCtlWarps + kEpiWarps);
static_assert(kPartCols == 32, "a softmax warp handles one 32-column tensor-memory load per key block");

struct AttnI8Params {
  int bh, heads, c, t, tk;
  int cch;                  // chunks of a q / k row: 1, or 2 for 256-byte rows
  int rb;                   // bytes of a chunk row in shared memory: 32, 64 or 128
  int ksteps;               // rb / 32: MMAs (K = 32 bytes) per chunk
  int d_rows;               // rows of a v tile (multiple of 16, <= 256)
  int nkb;                  // key blocks of 128
  int q_tiles, total_tiles;
  float scale;
  const float* scales;      // delta of q, k, v
  float* out;
  long long ob, oh, oc, ot; // element strides of the output (image, head, channel, token)
};

// Instruction descriptor of kind::i8 with an unsigned A operand: u8 x s8 -> s32, K-major.
__device__ inline uint32_t make_idesc_u8s8(int m, int n) {
  uint32_t d = 0;
  d |= 2u << 4;                 // D format: s32
  d |= 0u << 7;                 // A format: unsigned 8 bit
  d |= 1u << 10;                // B format: signed 8 bit
  d |= (uint32_t)(n >> 3) << 17;
  d |= (uint32_t)(m >> 4) << 24;
  return d;
}
// Shared-memory descriptor of a K-major tile whose rows are `rb` bytes (32, 64 or 128) stored with
// the swizzle of that width: groups of eight rows are 8 * rb bytes apart.
__device__ inline uint64_t make_smem_desc_rows(uint32_t saddr, int rb) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3ffffu) >> 4);            // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                              // leading byte offset (unused: one atom wide)
  d |= (uint64_t)((8 * rb) >> 4) << 32;                // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                              // descriptor version of sm_100
  d |= (uint64_t)(rb == 128 ? 2 : rb == 64 ? 4 : 6) << 61;   // swizzle: 128 / 64 / 32 bytes
  return d;
}
__device__ inline float exp2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// Softmax weights of 32 scores of one query row: u8 codes rne(255 * exp2((S - m) * c2)), (S - m) <= 0
// exactly, one fp32 product, hardware exp2.  The codes go to the row's 128-byte line of the weight
// tile (16-byte chunks XORed with row % 8, the tile's swizzle); their sum is added to l_part.
// MAGIC: (float)(S - m) without the conversion unit (the caller guarantees |S - m| < 2^22).
// MASK: only the first `nvalid` scores are keys, the others get weight 0.
template <bool MAGIC, bool MASK>
__device__ inline void weights32(const int (&a)[32], int m_row, float c2, int nvalid, uint8_t* prow,
                                 int chunk0, int row, int& l_part) {
  const int bias_i = 0x4B400000 - m_row;       // bits of 12582912.0f = 1.5 * 2^23
#pragma unroll
  for (int g8 = 0; g8 < 2; ++g8) {
    uint32_t wds[4];
#pragma unroll
    for (int wd = 0; wd < 4; ++wd) {
      uint32_t u[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int idx = g8 * 16 + wd * 4 + e;
        const float x = MAGIC ? __fadd_rn(__int_as_float(a[idx] + bias_i), -12582912.0f)
                              : (float)(a[idx] - m_row);
        const float pr = exp2_approx(__fmul_rn(x, c2));
        // adding 1.5 * 2^23 rounds half to even and leaves the code in the low mantissa byte
        u[e] = __float_as_uint(__fadd_rn(__fmul_rn(pr, 255.0f), 12582912.0f));
        if (MASK && idx >= nvalid) u[e] = 0u;
      }
      wds[wd] = __byte_perm(__byte_perm(u[0], u[1], 0x0040), __byte_perm(u[2], u[3], 0x0040), 0x5410);
      l_part = (int)__dp4a(wds[wd], 0x01010101u, (unsigned)l_part);   // sum of four u8 codes
    }
    const int chunk = (chunk0 + g8) ^ (row & 7);
    *reinterpret_cast<uint4*>(prow + chunk * 16) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
  }
}

__global__ void __launch_bounds__(kThreads, 1)
attention_i8_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const AttnI8Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages], bar_empty[kStages];
  __shared__ __align__(8) uint64_t bar_q_full, bar_q_empty;
  __shared__ __align__(8) uint64_t bar_s_full[2], bar_s_empty[2], bar_p_ready[2], bar_p_free[2];
  __shared__ __align__(8) uint64_t bar_o_full, bar_o_empty;
  __shared__ uint32_t tmem_base_sh;
  __shared__ int abort_sh;
  __shared__ int red_max[kParts][128];
  __shared__ int red_sum[kParts][128];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &abort_sh;
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t q_smem = raw;                               // cch tiles of 16 KB
  const uint32_t p_smem = raw + 2 * kTile;                   // two weight tiles of 16 KB
  const uint32_t ring = raw + 4 * kTile;                     // operand stages

  if (threadIdx.x == 0) {
    abort_sh = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_q_full), 1);
    mbar_init(smem_u32(&bar_q_empty), 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_s_full[b]), 1);
      mbar_init(smem_u32(&bar_s_empty[b]), kEpiWarps);
      mbar_init(smem_u32(&bar_p_ready[b]), kEpiWarps);
      mbar_init(smem_u32(&bar_p_free[b]), 1);
    }
    mbar_init(smem_u32(&bar_o_full), 1);
    mbar_init(smem_u32(&bar_o_empty), kEpiWarps);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_base_sh)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_sh;
  const uint32_t v_tile_bytes = (uint32_t)p.d_rows * kRowBytes;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // Ring order = the order in which the MMA warps consume: pass A k(0..n-1); pass B k(0),
    // then k(j), v(j-1) for j = 1..n-1, then v(n-1).
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, qphase = 0;
      bool ok = true;
      auto load_k = [&](int img, int j) {
        for (int ch = 0; ch < p.cch && ok; ++ch) {
          ok = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_flag);
          if (!ok) break;
          const uint32_t full = smem_u32(&bar_full[stage]);
          mbar_arrive_expect_tx(full, (uint32_t)(128 * p.rb));
          // key rows beyond tk are filled with zeros by the copy and masked in the softmax
          tma_load_3d(ring + stage * kStageBytes, &map_k, full, ch * kRowBytes, j * 128, img);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      };
      auto load_v = [&](int img, int j) {
        ok = ok && mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_flag);
        if (!ok) return;
        const uint32_t full = smem_u32(&bar_full[stage]);
        mbar_arrive_expect_tx(full, v_tile_bytes);
        tma_load_3d(ring + stage * kStageBytes, &map_v, full, j * 128, 0, img);
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      };
      for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
        const int img = tile / p.q_tiles, qt = tile % p.q_tiles;
        ok = mbar_wait(smem_u32(&bar_q_empty), qphase ^ 1u, abort_flag);
        if (!ok) break;
        const uint32_t qfull = smem_u32(&bar_q_full);
        mbar_arrive_expect_tx(qfull, (uint32_t)(p.cch * 128 * p.rb));
        for (int ch = 0; ch < p.cch; ++ch)
          tma_load_3d(q_smem + ch * kTile, &map_q, qfull, ch * kRowBytes, qt * 128, img);
        qphase ^= 1u;
        for (int j = 0; j < p.nkb && ok; ++j) load_k(img, j);
        for (int j = 0; j < p.nkb && ok; ++j) {
          load_k(img, j);
          if (j > 0) load_v(img, j - 1);
        }
        load_v(img, p.nkb - 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer 1: scores
    // The two MMA roles sit on different schedulers: each is one serial instruction stream that
    // shares its scheduler with four busy softmax warps, and together they set the pace.  Both
    // walk the SAME ring sequence (pass A: k(0..n-1); pass B: k(0), then k(j), v(j-1), then
    // v(n-1)); each consumes its own entries and steps over the other's.  All lanes walk the
    // loop; one elected lane issues the MMAs and commits.
    {
      const uint32_t idesc_s = make_idesc_i8(128, 128);
      int stage = 0;
      uint32_t phase = 0, qphase = 0;
      uint32_t s_count = 0;
      bool ok = true;
      auto skip = [&](int n) {
        for (int i = 0; i < n; ++i)
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
      };
      // scores of key block: S[s_count & 1] = q k^T
      auto scores = [&]() {
        const uint32_t b = s_count & 1u, par = (s_count >> 1) & 1u;
        ok = ok && mbar_wait(smem_u32(&bar_s_empty[b]), par ^ 1u, abort_flag);
        if (!ok) return;
        tc_fence_after();
        for (int ch = 0; ch < p.cch; ++ch) {
          ok = mbar_wait(smem_u32(&bar_full[stage]), phase, abort_flag);
          if (!ok) return;
          tc_fence_after();
          const uint64_t adesc = make_smem_desc_rows(q_smem + ch * kTile, p.rb);
          const uint64_t bdesc = make_smem_desc_rows(ring + stage * kStageBytes, p.rb);
          if (elect_one()) {
            for (int k = 0; k < p.ksteps; ++k)
              tc_mma_i8(tmem_base + b * 128u, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k),
                        idesc_s, (ch > 0 || k > 0) ? 1u : 0u);
            tc_commit(smem_u32(&bar_empty[stage]));
            if (ch == p.cch - 1) tc_commit(smem_u32(&bar_s_full[b]));
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        ++s_count;
      };
      for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
        ok = mbar_wait(smem_u32(&bar_q_full), qphase, abort_flag);
        if (!ok) break;
        qphase ^= 1u;
        for (int j = 0; j < p.nkb; ++j) scores();                       // pass A
        for (int j = 0; j < p.nkb; ++j) {                               // pass B
          scores();
          if (j > 0) skip(1);                                           // v(j-1)
        }
        skip(1);                                                        // v(n-1)
        if (!ok) break;
        if (elect_one()) tc_commit(smem_u32(&bar_q_empty));             // every product read q
        __syncwarp();
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------ MMA issuer 2: weighted sums
    {
      const uint32_t idesc_o = make_idesc_u8s8(128, p.d_rows);
      int stage = 0;
      uint32_t phase = 0, ophase = 0;
      uint32_t p_count = 0;
      bool ok = true;
      auto skip = [&](int n) {
        for (int i = 0; i < n; ++i)
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
      };
      // O += w v^T for the weight tile p_count & 1
      auto weighted = [&](bool first) {
        const uint32_t b = p_count & 1u, par = (p_count >> 1) & 1u;
        ok = ok && mbar_wait(smem_u32(&bar_p_ready[b]), par, abort_flag);
        if (ok && first) ok = mbar_wait(smem_u32(&bar_o_empty), ophase ^ 1u, abort_flag);
        if (ok) ok = mbar_wait(smem_u32(&bar_full[stage]), phase, abort_flag);
        if (!ok) return;
        tc_fence_after();
        const uint64_t adesc = make_smem_desc(p_smem + b * kTile);
        const uint64_t bdesc = make_smem_desc(ring + stage * kStageBytes);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_i8(tmem_base + 256u, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc_o,
                      (first && k == 0) ? 0u : 1u);
          tc_commit(smem_u32(&bar_empty[stage]));
          tc_commit(smem_u32(&bar_p_free[b]));
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
        ++p_count;
      };
      for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
        skip(p.nkb * p.cch);                                            // pass A: k(0..n-1)
        for (int j = 0; j < p.nkb; ++j) {                               // pass B
          skip(p.cch);                                                  // k(j)
          if (j > 0) weighted(j == 1);
        }
        weighted(p.nkb == 1);
        if (!ok) break;
        if (elect_one()) tc_commit(smem_u32(&bar_o_full));
        __syncwarp();
        ophase ^= 1u;
      }
    }
  } else if (warp == 3) {
    // idle: keeps the softmax warps' indices aligned with their tensor-memory lane quarters
  } else {
    // ------------------------------------------------------------ softmax + epilogue (warps 4..19)
    // kParts warps share a tensor-memory lane quarter; a lane is one query row, each warp of the
    // group takes 32 of the 128 keys of a block and every kParts-th 32-channel slice of the
    // output.  Four warps per scheduler hide the tensor-memory loads and the exp2 latency.
    const int quarter = warp & 3;
    const int part = (warp - kCtlWarps) >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    uint8_t* p_ptr = smem_raw + 2 * kTile;
    const float dq = p.scales[0], dk = p.scales[1], dv = p.scales[2];
    const float c2 = __fmul_rn(__fmul_rn(dq, dk), __fmul_rn(p.scale, 1.4426950408889634f));
    // |S - m| <= 2 * 128 * 128 * channels: below 2^22 the integer-to-float conversion is an integer
    // add into the mantissa of 1.5 * 2^23 and one exact subtraction (no conversion-unit cycles)
    const bool magic_ok = p.c * 32768 < (1 << 22);
    uint32_t s_count = 0, p_count = 0, ophase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
      const int img = tile / p.q_tiles, qt = tile % p.q_tiles;
      const int q = qt * 128 + row;
      // ---- pass A: exact integer row maximum
      int mx = INT_MIN;
      for (int j = 0; j < p.nkb && ok; ++j) {
        const uint32_t b = s_count & 1u, par = (s_count >> 1) & 1u;
        ok = mbar_wait(smem_u32(&bar_s_full[b]), par, abort_flag);
        if (!ok) break;
        tc_fence_after();
        {
          int a[32];
          tc_ld32(t_lane + b * 128u + (uint32_t)(part * kPartCols), a);
          tc_wait_ld();
          const int key0 = j * 128 + part * kPartCols;
          if (key0 + 32 <= p.tk) {
#pragma unroll
            for (int e = 0; e < 32; ++e) mx = max(mx, a[e]);
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (key0 + e < p.tk) mx = max(mx, a[e]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_s_empty[b]));
        ++s_count;
      }
      if (!ok) break;
      red_max[part][row] = mx;
      asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps) : "memory");
      int m_row = red_max[0][row];
#pragma unroll
      for (int i = 1; i < kParts; ++i) m_row = max(m_row, red_max[i][row]);
      // ---- pass B: weights, integer row sum
      int l_part = 0;
      for (int j = 0; j < p.nkb && ok; ++j) {
        const uint32_t b = s_count & 1u, par = (s_count >> 1) & 1u;
        const uint32_t pb = p_count & 1u, ppar = (p_count >> 1) & 1u;
        ok = mbar_wait(smem_u32(&bar_s_full[b]), par, abort_flag);
        // the MMAs that read the previous contents of this weight tile have completed
        if (ok) ok = mbar_wait(smem_u32(&bar_p_free[pb]), ppar ^ 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
        uint8_t* prow = p_ptr + (size_t)pb * kTile + (size_t)row * kRowBytes;
        {
          int a[32];
          tc_ld32(t_lane + b * 128u + (uint32_t)(part * kPartCols), a);
          tc_wait_ld();
          const int key0 = j * 128 + part * kPartCols;
          const int chunk0 = part * (kPartCols / 16);
          const bool ragged = key0 + 32 > p.tk;      // only the last key block can be
          if (magic_ok) {
            if (ragged) weights32<true, true>(a, m_row, c2, p.tk - key0, prow, chunk0, row, l_part);
            else weights32<true, false>(a, m_row, c2, 32, prow, chunk0, row, l_part);
          } else {
            if (ragged) weights32<false, true>(a, m_row, c2, p.tk - key0, prow, chunk0, row, l_part);
            else weights32<false, false>(a, m_row, c2, 32, prow, chunk0, row, l_part);
          }
        }
        tc_fence_before();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&bar_p_ready[pb]));
          mbar_arrive(smem_u32(&bar_s_empty[b]));
        }
        ++s_count;
        ++p_count;
      }
      if (!ok) break;
      red_sum[part][row] = l_part;
      asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps) : "memory");
      int l_row = red_sum[0][row];
#pragma unroll
      for (int i = 1; i < kParts; ++i) l_row += red_sum[i][row];
      const float inv = __fdiv_rn(dv, (float)l_row);
      // ---- output
      ok = mbar_wait(smem_u32(&bar_o_full), ophase, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const int bimg = img / p.heads, head = img % p.heads;
      float* obase = p.out + (long long)bimg * p.ob + (long long)head * p.oh + (long long)q * p.ot;
      for (int c0 = part * 32; c0 < p.d_rows; c0 += 32 * kParts) {
        int a[32];
        tc_ld32(t_lane + 256u + (uint32_t)c0, a);
        tc_wait_ld();
        if (q < p.t) {
          if (p.oc == 1 && c0 + 32 <= p.c && ((p.ob | p.oh | p.ot) & 3) == 0) {
#pragma unroll
            for (int e = 0; e < 32; e += 4)
              *reinterpret_cast<float4*>(obase + c0 + e) =
                  make_float4(__fmul_rn((float)a[e], inv), __fmul_rn((float)a[e + 1], inv),
                              __fmul_rn((float)a[e + 2], inv), __fmul_rn((float)a[e + 3], inv));
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (c0 + e < p.c) obase[(long long)(c0 + e) * p.oc] = __fmul_rn((float)a[e], inv);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_o_empty));
      ophase ^= 1u;
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  if (abort_sh) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u)
                 : "memory");
  }
}

}  // namespace

int read_device_status_attention_i8(int* status, int reset) {
  return read_status_this_unit(status, reset);
}

}  // namespace modiff

using namespace modiff;

extern "C" int64_t modiff_attn_codes_bytes(int heads_total, int c, int tq, int tk, int which) {
  const int dp = attn_row_bytes(c);
  const int d_rows = round_up(c, 16);
  const int tkp = round_up(tk, 128);
  if (which == 0) return (int64_t)heads_total * tq * dp;
  if (which == 1) return (int64_t)heads_total * tk * dp;
  return (int64_t)heads_total * d_rows * tkp;
}

extern "C" int modiff_attn_quantize(const float* q, const float* k, const float* v, int batch,
                                    int heads, int c, int tq, int tk, const int64_t* strides_q,
                                    const int64_t* strides_kv, int n_bits, int8_t* q_codes,
                                    int8_t* k_codes, int8_t* v_codes, float* scales, void* scratch,
                                    void* stream) {
  MODIFF_CHECK_ARG(q && k && v && q_codes && k_codes && v_codes && scales && scratch,
                   "NULL pointer argument");
  MODIFF_CHECK_ARG(strides_q && strides_kv, "NULL stride argument");
  MODIFF_CHECK_ARG(batch > 0 && heads > 0 && c > 0 && tq > 0 && tk > 0, "bad shape");
  MODIFF_CHECK_ARG(c <= 256, "heads wider than 256 channels are not covered");
  MODIFF_CHECK_ARG(n_bits >= 2 && n_bits <= 8, "n_bits must lie in [2, 8]");
  MODIFF_CHECK_ARG((((uintptr_t)q_codes | (uintptr_t)k_codes | (uintptr_t)v_codes) & 15) == 0,
                   "code buffers must be 16-byte aligned");
  QuantParams p;
  const float* xs[3] = {q, k, v};
  for (int i = 0; i < 3; ++i) {
    const int64_t* st = i == 0 ? strides_q : strides_kv;
    MODIFF_CHECK_ARG(st[2] == 1 || st[3] == 1, "channels or tokens must be contiguous");
    p.tv[i].x = xs[i];
    p.tv[i].sb = st[0];
    p.tv[i].sh = st[1];
    p.tv[i].sc = st[2];
    p.tv[i].st = st[3];
    p.tv[i].t = i == 0 ? tq : tk;
    // one dense block (either canonical order), 16-byte aligned, a multiple of four elements
    const long long t = p.tv[i].t, n = (long long)batch * heads * c * t;
    // (a stride that is multiplied by an index that is always 0 does not matter)
    const bool h_ok_cm = heads == 1 || st[1] == (long long)c * t;
    const bool b_ok = batch == 1 || st[0] == (long long)heads * c * t;
    const bool cm = st[3] == 1 && st[2] == t && h_ok_cm && b_ok;
    const bool tm = st[2] == 1 && (heads == 1 || st[1] == c) && st[3] == (long long)heads * c && b_ok;
    p.dense[i] = ((cm || tm) && n % 4 == 0 && ((uintptr_t)xs[i] & 15) == 0) ? n : 0;
  }
  p.batch = batch;
  p.heads = heads;
  p.c = c;
  p.n_levels = sym_levels(n_bits);
  p.scales = scales;
  p.scratch = reinterpret_cast<unsigned int*>(scratch);
  p.codes[0] = q_codes;
  p.codes[1] = k_codes;
  p.codes[2] = v_codes;
  p.dp = attn_row_bytes(c);
  p.d_rows = round_up(c, 16);
  p.tkp = round_up(tk, 128);
  cudaStream_t s = (cudaStream_t)stream;
  // about 4096 elements per block of the largest tensor: small levels get small grids (fewer
  // same-address atomics and no waves of idle blocks), large ones every SM eight times
  const long long elems = (long long)batch * heads * c * (tq > tk ? tq : tk);
  const long long want = (elems + 4095) / 4096;
  const int blocks = (int)(want < 1 ? 1 : (want < 1184 ? want : 1184));
  attn_absmax_kernel<<<dim3(blocks, 3), 256, 0, s>>>(p);
  MODIFF_LAUNCH_CHECK("attn_absmax_kernel");
  const int tmax = tq > p.tkp ? tq : p.tkp;
  const dim3 grid(ceil_div(tmax, 64), ceil_div(p.dp, 64), batch * heads * 3);
  attn_encode_kernel<<<grid, 256, 0, s>>>(p);
  MODIFF_LAUNCH_CHECK("attn_encode_kernel");
  return MODIFF_OK;
}

extern "C" int modiff_attention_i8(const int8_t* q_codes, const int8_t* k_codes,
                                   const int8_t* v_codes, const float* scales, float* out,
                                   int batch, int heads, int c, int tq, int tk,
                                   const int64_t* strides_out, float scale, void* stream) {
  MODIFF_CHECK_ARG(q_codes && k_codes && v_codes && scales && out && strides_out,
                   "NULL pointer argument");
  MODIFF_CHECK_ARG(batch > 0 && heads > 0 && c > 0 && tq > 0 && tk > 0, "bad shape");
  MODIFF_CHECK_ARG(c <= 256, "heads wider than 256 channels are not covered");
  MODIFF_CHECK_ARG((((uintptr_t)q_codes | (uintptr_t)k_codes | (uintptr_t)v_codes) & 15) == 0,
                   "code buffers must be 16-byte aligned");
  EncodeTiledFn encode = get_encode_fn();
  if (!encode) return set_error(MODIFF_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is not available");
  const int dp = attn_row_bytes(c);
  const int d_rows = round_up(c, 16);
  const int tkp = round_up(tk, 128);
  const int bh = batch * heads;

  AttnI8Params p;
  p.bh = bh;
  p.heads = heads;
  p.c = c;
  p.t = tq;
  p.tk = tk;
  p.cch = dp > 128 ? 2 : 1;
  p.rb = dp < 128 ? dp : 128;
  p.ksteps = p.rb / 32;
  p.d_rows = d_rows;
  p.nkb = tkp / 128;
  p.q_tiles = ceil_div(tq, 128);
  p.total_tiles = bh * p.q_tiles;
  p.scale = scale;
  p.scales = scales;
  p.out = out;
  p.ob = strides_out[0];
  p.oh = strides_out[1];
  p.oc = strides_out[2];
  p.ot = strides_out[3];

  CUtensorMap map_q, map_k, map_v;
  // a box is `box_rows` rows of `row_bytes` (32, 64 or 128), stored with the swizzle of that width
  auto make = [&](CUtensorMap* m, const void* base, int inner, int rows, int box_rows,
                  int row_bytes) -> CUresult {
    cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)bh};
    cuuint64_t strides[2] = {(cuuint64_t)inner, (cuuint64_t)inner * rows};
    cuuint32_t box[3] = {(cuuint32_t)row_bytes, (cuuint32_t)box_rows, 1u};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapSwizzle sw = row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                    : CU_TENSOR_MAP_SWIZZLE_32B;
    return encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r = make(&map_q, q_codes, dp, tq, 128, p.rb);                 // [head][query][dp]
  if (r == CUDA_SUCCESS) r = make(&map_k, k_codes, dp, tk, 128, p.rb);   // [head][key][dp]
  if (r == CUDA_SUCCESS) r = make(&map_v, v_codes, tkp, d_rows, d_rows, 128);   // [head][channel][key]
  if (r != CUDA_SUCCESS)
    return set_error(MODIFF_ERR_CUDA, "cuTensorMapEncodeTiled(attention codes) failed: %d", (int)r);

  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    MODIFF_CUDA(cudaGetDevice(&dev));
    MODIFF_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  const size_t smem = (size_t)4 * kTile + (size_t)kStages * kStageBytes;
  static SmemLimit smem_limit;
  MODIFF_CUDA(raise_smem_limit(attention_i8_kernel, smem, smem_limit));
  const int grid = p.total_tiles < sm_count ? p.total_tiles : sm_count;
  attention_i8_kernel<<<grid, kThreads, smem, (cudaStream_t)stream>>>(map_q, map_k, map_v, p);
  MODIFF_LAUNCH_CHECK("attention_i8_kernel");
  return MODIFF_OK;
}
