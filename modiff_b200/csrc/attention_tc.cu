// Attention in ONE kernel on the 5th-generation tensor cores (sm_100a):
//   S = scale * q^T k  ->  softmax over keys  ->  out = P v            (per image / head)
// (qdiff/quant_block.py:344-360 and 191-203, ldm/modules/diffusionmodules/openaimodel.py:384-406:
// the reference keeps both matmuls and the softmax in floating point).  fp32 accuracy comes from
// split-bf16 operands as in gemm_bf16_tc.cu (hi*hi + hi*lo + lo*hi, fp32 accumulation in tensor
// memory).  Scores and probabilities never touch global memory.
//
// A CTA owns 128 queries of one image at a time and walks the keys in blocks of 256:
//   phase 1  tcgen05.mma (M=128, N=256) accumulates the block's scores in tensor-memory columns
//            [0, 256) from TMA-fed q / k plane tiles;
//   phase 2  the epilogue warps take the block's row maximum, fold it into the running maximum
//            (online softmax: the output accumulator is rescaled in tensor memory when the
//            maximum grows), and write the UNNORMALISED probabilities exp(s - max), 128 keys at a
//            time, as two bf16 planes straight into shared memory in the 128-byte-swizzled
//            K-major layout an MMA A operand needs;
//   phase 3  tcgen05.mma (N=channels<=256) accumulates P v in columns [256, 512), A operand
//            = those shared-memory planes, B operand = TMA-fed v plane tiles;
//   phase 4  after the last key block the epilogue divides by the row sum and writes
//            out[image][channel][query].
// Phase 1 of the next tile overlaps phase 4 of this one.  Every mbarrier wait is bounded.
#include "common.cuh"
#include "tc_common.cuh"

namespace modiff {
namespace {

constexpr int kChunkBytes = 128;                 // 64 bf16 of K per tile row
constexpr int kATile = 128 * kChunkBytes;        // 16 KB: 128 queries
constexpr int kBTileMax = 256 * kChunkBytes;     // 32 KB: up to 256 keys / channels
constexpr int kStage = kATile + kBTileMax;       // 48 KB
constexpr int kStages = 3;
constexpr int kPBytes = 2 * 2 * kATile;          // two planes x two 64-key chunks (128 keys) x 16 KB
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + 32 * kEpiWarps;

struct AttnParams {
  int batch, c, t, tk;          // images*heads, channels per head, queries, keys
  int tkp;                      // keys padded to a multiple of 64
  int crow;                     // channel rows of the v planes (multiple of 64, <= 256)
  int cch;                      // 64-element K chunks of phase 1: ceil(cp / 64)
  int n_s;                      // score columns per key block: min(256, tkp)
  int nsb;                      // key blocks: ceil(tkp / 256)
  int q_tiles;                  // ceil(t / 128)
  int total_tiles;
  float scale;
  float* out;                   // [batch][c][t]
};

// the three products of a split-bf16 multiplication, (a part, b part): hi*hi, hi*lo, lo*hi
__device__ inline int prod_a(int pr) { return pr == 2 ? 1 : 0; }
__device__ inline int prod_b(int pr) { return pr == 1 ? 1 : 0; }

// two floats -> packed bf16 pair (round to nearest even), first argument in the low half
__device__ inline uint32_t bf16_pair(float lo_half, float hi_half) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi_half), "f"(lo_half));
  return r;
}
// exp(x) for x <= 0 through the hardware exp2 (relative error ~2^-22, far below the 2^-16 the
// split probabilities keep)
__device__ inline float exp_neg(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x * 1.4426950408889634f));
  return r;
}

__global__ void __launch_bounds__(kThreads, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages], bar_empty[kStages];
  __shared__ __align__(8) uint64_t bar_s_full, bar_p_ready, bar_p_free, bar_o_full, bar_o_empty;
  __shared__ uint32_t tmem_base_sh;
  __shared__ int abort_sh;
  __shared__ float red_max[2][128], red_sum[2][128];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &abort_sh;
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t p_smem = raw;                       // probability planes
  const uint32_t ring = raw + kPBytes;               // operand stages

  if (threadIdx.x == 0) {
    abort_sh = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_s_full), 1);
    mbar_init(smem_u32(&bar_p_ready), kEpiWarps);
    mbar_init(smem_u32(&bar_p_free), 1);
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
  const uint32_t k_tile_bytes = (uint32_t)p.n_s * kChunkBytes;
  const uint32_t v_tile_bytes = (uint32_t)p.crow * kChunkBytes;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
        const int img = tile / p.q_tiles, qt = tile % p.q_tiles;
        for (int sb = 0; sb < p.nsb && ok; ++sb) {
          for (int ch = 0; ch < p.cch && ok; ++ch) {
            for (int pr = 0; pr < 3; ++pr) {
              ok = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_flag);
              if (!ok) break;
              const uint32_t full = smem_u32(&bar_full[stage]);
              const uint32_t dst = ring + stage * kStage;
              mbar_arrive_expect_tx(full, (uint32_t)kATile + k_tile_bytes);
              tma_load_3d(dst, &map_q, full, ch * 64, qt * 128, img * 2 + prod_a(pr));
              // key rows beyond tkp are filled with zeros by the copy and masked in the softmax
              tma_load_3d(dst + kATile, &map_k, full, ch * 64, sb * 256, img * 2 + prod_b(pr));
              if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
          }
          const int kch = min(4, (p.tkp - sb * 256) >> 6);
          for (int kc = 0; kc < kch && ok; ++kc) {
            for (int pr = 0; pr < 3; ++pr) {
              ok = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_flag);
              if (!ok) break;
              const uint32_t full = smem_u32(&bar_full[stage]);
              mbar_arrive_expect_tx(full, v_tile_bytes);
              tma_load_3d(ring + stage * kStage + kATile, &map_v, full, sb * 256 + kc * 64, 0,
                          img * 2 + prod_b(pr));
              if (++stage == kStages) { stage = 0; phase ^= 1u; }
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
      const uint32_t idesc_s = make_idesc_bf16(128, p.n_s);
      const uint32_t idesc_o = make_idesc_bf16(128, p.crow);
      int stage = 0;
      uint32_t phase = 0, tphase = 0, pphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
        uint32_t fresh_pv = 1u;
        for (int sb = 0; sb < p.nsb; ++sb) {
          // phase 1: scores of this key block.  The softmax has finished reading the previous
          // block's scores (its last p_ready preceded the MMAs issued just before this point).
          for (int it = 0; it < 3 * p.cch; ++it) {
            ok = mbar_wait(smem_u32(&bar_full[stage]), phase, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t a_src = ring + stage * kStage;
            const uint64_t adesc = make_smem_desc(a_src);
            const uint64_t bdesc = make_smem_desc(a_src + kATile);
            if (elect_one()) {
#pragma unroll
              for (int k = 0; k < 4; ++k)
                tc_mma_bf16(tmem_base, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc_s,
                            (it > 0 || k > 0) ? 1u : 0u);
              tc_commit(smem_u32(&bar_empty[stage]));
            }
            __syncwarp();
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
          if (elect_one()) tc_commit(smem_u32(&bar_s_full));
          __syncwarp();
          // phase 3, 128 keys at a time: the probability planes of one half sit in shared memory
          // while the epilogue warps wait to write the next half; the tile's first product also
          // needs the previous tile's output drained
          const int kch = min(4, (p.tkp - sb * 256) >> 6);
          const int halves = (kch + 1) >> 1;
          for (int kh = 0; kh < halves; ++kh) {
            ok = mbar_wait(smem_u32(&bar_p_ready), pphase, abort_flag);
            pphase ^= 1u;
            if (ok && fresh_pv) ok = mbar_wait(smem_u32(&bar_o_empty), tphase ^ 1u, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const int kc_end = min(kch, 2 * kh + 2);
            for (int kc = 2 * kh; kc < kc_end; ++kc) {
              for (int pr = 0; pr < 3; ++pr) {
                ok = mbar_wait(smem_u32(&bar_full[stage]), phase, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint64_t adesc =
                    make_smem_desc(p_smem + (uint32_t)((prod_a(pr) * 2 + (kc & 1)) * kATile));
                const uint64_t bdesc = make_smem_desc(ring + stage * kStage + kATile);
                if (elect_one()) {
#pragma unroll
                  for (int k = 0; k < 4; ++k)
                    tc_mma_bf16(tmem_base + 256u, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k),
                                idesc_o, (fresh_pv && k == 0) ? 0u : 1u);
                  tc_commit(smem_u32(&bar_empty[stage]));
                }
                __syncwarp();
                fresh_pv = 0u;
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
              }
              if (!ok) break;
            }
            if (!ok) break;
            if (elect_one()) tc_commit(smem_u32(&bar_p_free));
            __syncwarp();
          }
          if (!ok) break;
        }
        if (!ok) break;
        if (elect_one()) tc_commit(smem_u32(&bar_o_full));
        __syncwarp();
        tphase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue (warps 2..9)
    // Two warps share a tensor-memory lane quarter; a lane is one query row, each warp of the
    // pair takes half of the columns.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int ccols = p.crow >> 1;           // channel columns of this warp (multiple of 32)
    uint8_t* p_ptr = smem_raw;
    uint32_t tphase = 0, sphase = 0, fphase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
      const int img = tile / p.q_tiles, qt = tile % p.q_tiles;
      const int q = qt * 128 + row;
      float m_run = -INFINITY;      // running row maximum (the same in both warps of a pair)
      float l_part = 0.0f;          // running sum of this warp's columns, in units of exp(-m_run)
      for (int sb = 0; sb < p.nsb && ok; ++sb) {
        const int keys_sb = min(256, p.tkp - sb * 256);
        const int halves = (keys_sb + 127) >> 7;
        ok = mbar_wait(smem_u32(&bar_s_full), sphase, abort_flag);
        sphase ^= 1u;
        if (!ok) break;
        tc_fence_after();
        // Keys are handled 128 at a time (kh); inside a half the two warps of a lane quarter
        // take half of its keys each (32 or 64 columns).
        // ---- row maximum of this key block, folded into the running maximum
        float mx = -INFINITY;
        for (int kh = 0; kh < halves; ++kh) {
          const int nk = min(128, keys_sb - 128 * kh) >> 1;
          for (int c0 = 0; c0 < nk; c0 += 32) {
            const int col0 = 128 * kh + half * nk + c0;
            int a[32];
            tc_ld32(t_lane + (uint32_t)col0, a);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (sb * 256 + col0 + j < p.tk) mx = fmaxf(mx, __int_as_float(a[j]) * p.scale);
          }
        }
        red_max[half][row] = mx;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const float m_new = fmaxf(m_run, fmaxf(red_max[0][row], red_max[1][row]));
        // exp(m_run - m_new): 0 for the first block (m_run = -inf), 1 while the maximum stands
        const float alpha = exp_neg(m_run - m_new);
        l_part *= alpha;
        m_run = m_new;
        // ---- exp, row sum, probabilities -> shared memory (K-major rows of 128 bytes, the
        //      16-byte chunk index XORed with row % 8: the layout TMA writes with 128-byte swizzle)
        for (int kh = 0; kh < halves && ok; ++kh) {
          // the MMAs that read the previous contents of the planes (and accumulated into the
          // output columns) have completed
          ok = mbar_wait(smem_u32(&bar_p_free), fphase ^ 1u, abort_flag);
          fphase ^= 1u;
          if (!ok) break;
          if (kh == 0 && sb > 0) {
            // online softmax: bring the accumulated output to the new maximum
            tc_fence_after();
            for (int c0 = 0; c0 < ccols; c0 += 32) {
              int a[32];
              tc_ld32(t_lane + 256u + (uint32_t)(half * ccols + c0), a);
              tc_wait_ld();
#pragma unroll
              for (int j = 0; j < 32; ++j) a[j] = __float_as_int(__int_as_float(a[j]) * alpha);
              tc_st32(t_lane + 256u + (uint32_t)(half * ccols + c0), a);
            }
            tc_wait_st();
          }
          const int nk = min(128, keys_sb - 128 * kh) >> 1;
          for (int c0 = 0; c0 < nk; c0 += 32) {
            const int col0 = 128 * kh + half * nk + c0;       // multiple of 32
            const int key0 = sb * 256 + col0;
            int a[32];
            tc_ld32(t_lane + (uint32_t)col0, a);
            tc_wait_ld();
            const int kc = (col0 >> 6) & 1;                   // 64-key chunk inside the half
            const int chunk0 = (col0 & 63) >> 3;              // first 16-byte chunk of the row: 0 or 4
            uint8_t* hi_row = p_ptr + (size_t)(0 * 2 + kc) * kATile + (size_t)row * 128;
            uint8_t* lo_row = p_ptr + (size_t)(1 * 2 + kc) * kATile + (size_t)row * 128;
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {
              uint32_t hw[4], lw[4];
#pragma unroll
              for (int e = 0; e < 8; e += 2) {
                float pv[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                  const int j = g8 * 8 + e + u;
                  const float sv = __int_as_float(a[j]) * p.scale;
                  pv[u] = (key0 + j < p.tk) ? exp_neg(sv - m_run) : 0.0f;
                  l_part += pv[u];
                }
                const uint32_t h = bf16_pair(pv[0], pv[1]);
                hw[e >> 1] = h;
                lw[e >> 1] = bf16_pair(pv[0] - __uint_as_float(h << 16),
                                       pv[1] - __uint_as_float(h & 0xffff0000u));
              }
              const int chunk = (chunk0 + g8) ^ (row & 7);
              *reinterpret_cast<uint4*>(hi_row + chunk * 16) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
              *reinterpret_cast<uint4*>(lo_row + chunk * 16) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
            }
          }
          // a half with 64 keys fills one chunk; the MMA of this half then reads one chunk only
          tc_fence_before();
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("bar.sync 1, 256;" ::: "memory");
          if (lane == 0) mbar_arrive(smem_u32(&bar_p_ready));
        }
      }
      if (!ok) break;
      red_sum[half][row] = l_part;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      const float inv = 1.0f / (red_sum[0][row] + red_sum[1][row]);
      // ---- output
      ok = mbar_wait(smem_u32(&bar_o_full), tphase, abort_flag);
      if (!ok) break;
      tc_fence_after();
      for (int c0 = 0; c0 < ccols; c0 += 32) {
        int a[32];
        tc_ld32(t_lane + 256u + (uint32_t)(half * ccols + c0), a);
        tc_wait_ld();
        if (q < p.t) {
          float* dst = p.out + ((size_t)img * p.c + half * ccols + c0) * p.t + q;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (half * ccols + c0 + j < p.c) dst[(size_t)j * p.t] = __int_as_float(a[j]) * inv;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_o_empty));
      tphase ^= 1u;
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

int read_device_status_attention(int* status, int reset) {
  return read_status_this_unit(status, reset);
}

}  // namespace modiff

using namespace modiff;

extern "C" int modiff_attention_tc(const uint16_t* q_planes, const uint16_t* k_planes,
                                   const uint16_t* v_planes, float* out, int batch, int c, int t,
                                   int tk, int cp, int tkp, int crow, float scale, void* stream) {
  MODIFF_CHECK_ARG(q_planes && k_planes && v_planes && out, "NULL pointer argument");
  MODIFF_CHECK_ARG(batch > 0 && c > 0 && t > 0 && tk > 0, "bad shape");
  if (tkp < tk || tkp % 64 || crow < c || crow > 256 || crow % 64 || cp < c || cp % 8 || cp < 64 ||
      cp > 256)
    return set_error(MODIFF_ERR_UNSUPPORTED,
                     "single-kernel attention needs keys padded to a multiple of 64, channel rows a "
                     "multiple of 64 <= 256 and 64 <= cp <= 256 (got tkp=%d crow=%d cp=%d)", tkp, crow,
                     cp);
  MODIFF_CHECK_ARG((((uintptr_t)q_planes | (uintptr_t)k_planes | (uintptr_t)v_planes) & 15) == 0,
                   "plane buffers must be 16-byte aligned");
  EncodeTiledFn encode = get_encode_fn();
  if (!encode) return set_error(MODIFF_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is not available");

  AttnParams p;
  p.batch = batch;
  p.c = c;
  p.t = t;
  p.tk = tk;
  p.tkp = tkp;
  p.crow = crow;
  p.cch = ceil_div(cp, 64);
  p.n_s = tkp < 256 ? tkp : 256;
  p.nsb = ceil_div(tkp, 256);
  p.q_tiles = ceil_div(t, 128);
  p.total_tiles = batch * p.q_tiles;
  p.scale = scale;
  p.out = out;

  CUtensorMap map_q, map_k, map_v;
  auto make = [&](CUtensorMap* m, const void* base, int inner, int rows, int box_rows) -> CUresult {
    cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)batch * 2};
    cuuint64_t strides[2] = {(cuuint64_t)inner * 2, (cuuint64_t)inner * rows * 2};
    cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, 1u};
    cuuint32_t estr[3] = {1, 1, 1};
    return encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r = make(&map_q, q_planes, cp, t, 128);            // [image*2+part][query][cp]
  if (r == CUDA_SUCCESS) r = make(&map_k, k_planes, cp, tkp, p.n_s);   // [image*2+part][key][cp]
  if (r == CUDA_SUCCESS) r = make(&map_v, v_planes, tkp, crow, crow);  // [image*2+part][channel][key]
  if (r != CUDA_SUCCESS)
    return set_error(MODIFF_ERR_CUDA, "cuTensorMapEncodeTiled(attention operands) failed: %d", (int)r);

  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    MODIFF_CUDA(cudaGetDevice(&dev));
    MODIFF_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  const size_t smem = (size_t)kPBytes + (size_t)kStages * kStage;
  static SmemLimit smem_limit;
  MODIFF_CUDA(raise_smem_limit(attention_tc_kernel, smem, smem_limit));
  const int grid = p.total_tiles < sm_count ? p.total_tiles : sm_count;
  attention_tc_kernel<<<grid, kThreads, smem, (cudaStream_t)stream>>>(map_q, map_k, map_v, p);
  MODIFF_LAUNCH_CHECK("attention_tc_kernel");
  return MODIFF_OK;
}
