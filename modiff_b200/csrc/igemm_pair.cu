// Int8 implicit-GEMM for 3x3, stride-1, pad-1 convolutions on a PAIR of SMs
// (tcgen05.mma.cta_group::2): a cluster of two CTAs computes one output tile of
// 2 x (mh x 128) pixels x umma_n channels.
//
// Why a pair.  With one CTA per tile (igemm_halo_kernel, M = 128, N = 128) every MMA reads a
// 4 KB A tile and a 4 KB B tile from shared memory for 64 tensor-pipe cycles, which is the
// whole shared-memory bandwidth of the SM, and every CTA pulls the full weight tile through
// its L2 port.  In a pair each CTA holds its own 128 pixel rows of A and only HALF of the
// weight rows (B is split along N between the two CTAs' shared memories), so per CTA the
// weight fill and the operand reads per MMA cycle are halved; with umma_n = 256 one activation
// copy serves 256 output channels.
//
// Roles per CTA: warp 0 operand TMA (each CTA loads its own activation copies and its half of
// the weight tile with plain, non-multicast copies), warp 1 MMA issue in the leader CTA (rank
// 0) / forwarding of "operands landed" signals in the peer CTA, warps 2-9 epilogue for the
// CTA's own pixels, warp 10 cached-output loads.
// Signals: the leader's MMA thread waits for its own copies (local mbarriers) and for the
// peer's (the peer's warp 1 observes its local mbarrier and arrives on a mirror barrier in the
// leader's shared memory); tcgen05.commit with a two-CTA mask releases operand stages and
// publishes finished accumulators in both CTAs; the peer's epilogue warps release an
// accumulator buffer by arriving remotely on the leader's barrier.  Every wait is bounded.
//
// Activation copies follow igemm_halo_kernel: per K chunk three copies (one per horizontal
// tap) of rows+2 input rows; the vertical taps are the same copy read a whole number of
// swizzle periods later.  Epilogue: cached-output half tiles (64 channels x 128 pixels) arrive
// by bulk tensor copies through a small ring; out = o_hat + acc * (delta_x * delta_w[c]) is
// stored straight from registers (a lane is a pixel).
//
// Reference arithmetic: qdiff/quant_layer.py:345-365.
#include "common.cuh"
#include "tc_common.cuh"

#include <cstdlib>

namespace modiff {
namespace {

constexpr int kChunkK = 128;                     // bytes of K per weight tile row
constexpr int kEpiWarps = 8;
constexpr int kMaxASlots = 3;
constexpr int kMaxOSlots = 3;
constexpr int kOHalfBytes = 64 * 128 * 4;        // 64 channels x 128 pixels fp32
constexpr int kMaxBStages = 8;
constexpr int kLoadWarp = 2 + kEpiWarps;
constexpr int kThreads = 32 * (3 + kEpiWarps);
constexpr int kMaxN = 256;

struct PairParams {
  int w, h, batch, cout;
  int rows;             // output rows per CTA tile (mh * 128 / w)
  int mh;               // 128-pixel halves per CTA tile: 1 or 2
  int half_rows;        // rows / mh
  int blocks_per_image; // h / rows
  int n_tiles;          // cout / n_real
  int n_real;           // output channels per tile (128 or 256)
  int total_tiles;      // pair tiles
  int chunks;           // 128-byte K chunks per tap
  int kp;               // weight K stride per tap
  int b_stages;
  int a_bytes;          // bytes of one activation copy: (rows + 2) * w * 128
  int a_slot_bytes;
  int a_slots;
  int tmem_cols;
  int o_slots;          // cached-output half tiles in flight (2 or 3)
  float* o_out;         // the cached output itself: new values are stored straight from registers
  int nbuf;             // accumulator buffers: 1 or 2
  int accumulate;
  int umma_n;           // 128, 256, or 144 (128 channels + receptive-field-sum rows)
  int b_half_rows;      // umma_n / 2: weight rows held by one CTA
  int b_tile_bytes;     // b_half_rows * 128
  int b_tile_rows;      // rows of one tile in the packed weights (umma_n)
  const float* x_scale;
  const float* w_scale;
  const int32_t* w_corr;
  const float* x_zp;          // offset (8-bit asymmetric) activation codes, else NULL
  const int32_t* w_csum;
  const float* residual;      // optional [batch][cout][h*w]: sum_out = new output + residual
  float* sum_out;
};

__device__ inline void tc_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(bar), "h"(mask)
      : "memory");
}
__device__ inline void tc_mma_i8_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                      uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

struct PairTile {
  int n, rb, nt;      // image, row block inside the image, channel tile (of THIS CTA)
};
__device__ inline PairTile decode(int tile, uint32_t rank, const PairParams& p) {
  PairTile t;
  t.nt = tile % p.n_tiles;
  const int mblock = (tile / p.n_tiles) * 2 + (int)rank;   // CTA-level pixel block
  t.rb = mblock % p.blocks_per_image;
  t.n = mblock / p.blocks_per_image;
  return t;
}

__global__ void __launch_bounds__(kThreads, 1)
igemm_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                  const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_o, const PairParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_a_full[kMaxASlots], bar_a_empty[kMaxASlots];
  __shared__ __align__(8) uint64_t bar_b_full[kMaxBStages], bar_b_empty[kMaxBStages];
  // mirrors of the peer CTA's "landed" barriers; used in the leader's shared memory only
  __shared__ __align__(8) uint64_t bar_a_peer[kMaxASlots], bar_b_peer[kMaxBStages];
  __shared__ __align__(8) uint64_t bar_tmem_full[2], bar_tmem_empty[2];
  __shared__ __align__(8) uint64_t bar_o_full[kMaxOSlots], bar_o_empty[kMaxOSlots];
  __shared__ uint32_t tmem_base_sh;
  __shared__ int abort_sh;
  __shared__ float ep_scale[kMaxN];
  __shared__ int ep_corr[kMaxN];
  __shared__ int ep_off[kMaxN];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &abort_sh;
  const uint32_t rank = cluster_ctarank();
  const int pair_id = (int)(blockIdx.x >> 1);
  const int num_pairs = (int)(gridDim.x >> 1);

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t a_ring = raw;
  const uint32_t b_ring = a_ring + (uint32_t)p.a_slots * (uint32_t)p.a_slot_bytes;
  const uint32_t b_tile = (uint32_t)p.b_tile_bytes;
  const uint32_t obuf = b_ring + (uint32_t)p.b_stages * b_tile;
  float* obuf_ptr = reinterpret_cast<float*>(smem_raw + (obuf - raw));

  if (threadIdx.x == 0) {
    abort_sh = 0;
    for (int s = 0; s < p.a_slots; ++s) {
      mbar_init(smem_u32(&bar_a_full[s]), 1);
      mbar_init(smem_u32(&bar_a_empty[s]), 1);
      mbar_init(smem_u32(&bar_a_peer[s]), 1);
    }
    for (int s = 0; s < p.b_stages; ++s) {
      mbar_init(smem_u32(&bar_b_full[s]), 1);
      mbar_init(smem_u32(&bar_b_empty[s]), 1);
      mbar_init(smem_u32(&bar_b_peer[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_tmem_full[b]), 1);
      mbar_init(smem_u32(&bar_tmem_empty[b]), 2 * kEpiWarps);   // both CTAs' epilogue warps
    }
    for (int b = 0; b < p.o_slots; ++b) {
      mbar_init(smem_u32(&bar_o_full[b]), 1);
      mbar_init(smem_u32(&bar_o_empty[b]), kEpiWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_base_sh)),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();        // both CTAs' barriers and tensor memory exist before any signal
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_sh;
  const int buf_cols = p.mh * p.umma_n;

  if (warp == 0) {
    // ------------------------------------------------------------ operand TMA producer
    if (lane == 0) {
      int aslot = 0, bst = 0;
      uint32_t aphase = 0, bphase = 0;
      bool ok = true;
      for (int tile = pair_id; tile < p.total_tiles && ok; tile += num_pairs) {
        const PairTile t = decode(tile, rank, p);
        for (int ch = 0; ch < p.chunks && ok; ++ch) {
          for (int dx = 0; dx < 3 && ok; ++dx) {
            ok = mbar_wait(smem_u32(&bar_a_empty[aslot]), aphase ^ 1u, abort_flag);
            if (!ok) break;
            const uint32_t afull = smem_u32(&bar_a_full[aslot]);
            mbar_arrive_expect_tx(afull, (uint32_t)p.a_bytes);
            // padded input rows rb*rows .. rb*rows+rows+1, padded columns dx .. dx+w-1
            tma_load_5d(a_ring + aslot * (uint32_t)p.a_slot_bytes, &map_a, afull, ch * kChunkK, dx,
                        t.rb * p.rows, 0, t.n);
            if (++aslot == p.a_slots) { aslot = 0; aphase ^= 1u; }
            for (int dy = 0; dy < 3; ++dy) {
              ok = mbar_wait(smem_u32(&bar_b_empty[bst]), bphase ^ 1u, abort_flag);
              if (!ok) break;
              const uint32_t bfull = smem_u32(&bar_b_full[bst]);
              mbar_arrive_expect_tx(bfull, b_tile);
              // this CTA's half of the weight rows of the tile
              tma_load_2d(b_ring + bst * b_tile, &map_b, bfull,
                          (dy * 3 + dx) * p.kp + ch * kChunkK,
                          t.nt * p.b_tile_rows + (int)rank * p.b_half_rows);
              if (++bst == p.b_stages) { bst = 0; bphase ^= 1u; }
            }
          }
        }
      }
    }
  } else if (warp == 1 && rank != 0) {
    // ------------------------------------------------------------ peer: forward "landed"
    // The leader's MMA reads this CTA's shared memory; it learns that a copy has landed here
    // through a mirror barrier in its own shared memory.
    if (lane == 0) {
      int aslot = 0, bst = 0;
      uint32_t aphase = 0, bphase = 0;
      bool ok = true;
      for (int tile = pair_id; tile < p.total_tiles && ok; tile += num_pairs) {
        for (int ch = 0; ch < p.chunks && ok; ++ch) {
          for (int dx = 0; dx < 3 && ok; ++dx) {
            ok = mbar_wait(smem_u32(&bar_a_full[aslot]), aphase, abort_flag);
            if (!ok) break;
            mbar_arrive_remote(map_to_cta(smem_u32(&bar_a_peer[aslot]), 0));
            if (++aslot == p.a_slots) { aslot = 0; aphase ^= 1u; }
            for (int dy = 0; dy < 3; ++dy) {
              ok = mbar_wait(smem_u32(&bar_b_full[bst]), bphase, abort_flag);
              if (!ok) break;
              mbar_arrive_remote(map_to_cta(smem_u32(&bar_b_peer[bst]), 0));
              if (++bst == p.b_stages) { bst = 0; bphase ^= 1u; }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ leader: MMA issuer
    // The whole warp walks the loop and one elected lane issues, so that descriptors and
    // addresses are warp-uniform values (a single lane running the loop spent about twice the
    // tensor-pipe time of an MMA on issuing it).
    {
      const uint32_t idesc = make_idesc_i8(256, p.umma_n);
      int aslot = 0, bst = 0, buf = 0;
      uint32_t aphase = 0, bphase = 0, tphase = 0;
      bool ok = true;
      for (int tile = pair_id; tile < p.total_tiles; tile += num_pairs) {
        ok = mbar_wait_cluster(smem_u32(&bar_tmem_empty[buf]), tphase ^ 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
        uint32_t fresh = 1u;        // the tile's first MMA overwrites the accumulator
        for (int ch = 0; ch < p.chunks; ++ch) {
          for (int dx = 0; dx < 3; ++dx) {
            ok = mbar_wait(smem_u32(&bar_a_full[aslot]), aphase, abort_flag) &&
                 mbar_wait_cluster(smem_u32(&bar_a_peer[aslot]), aphase, abort_flag);
            if (!ok) break;
            const uint32_t a_base = a_ring + aslot * (uint32_t)p.a_slot_bytes;
            for (int dy = 0; dy < 3; ++dy) {
              ok = mbar_wait(smem_u32(&bar_b_full[bst]), bphase, abort_flag) &&
                   mbar_wait_cluster(smem_u32(&bar_b_peer[bst]), bphase, abort_flag);
              if (!ok) break;
              tc_fence_after();
              const uint64_t bdesc = make_smem_desc(b_ring + bst * b_tile);
              // rows dy .. of the copy: a whole number of 1024-byte swizzle periods
              const uint64_t adesc0 = make_smem_desc(a_base + (uint32_t)(dy * p.w) * (uint32_t)kChunkK);
              const uint64_t adesc1 =
                  make_smem_desc(a_base + (uint32_t)((p.half_rows + dy) * p.w) * (uint32_t)kChunkK);
              const uint32_t d_tmem = tmem_base + (uint32_t)(buf * buf_cols);
              if (elect_one()) {
#pragma unroll
                for (int k = 0; k < kChunkK / 32; ++k)
                  tc_mma_i8_pair(d_tmem, adesc0 + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                                 (fresh && k == 0) ? 0u : 1u);
                if (p.mh == 2) {
#pragma unroll
                  for (int k = 0; k < kChunkK / 32; ++k)
                    tc_mma_i8_pair(d_tmem + (uint32_t)p.umma_n, adesc1 + (uint64_t)(2 * k),
                                   bdesc + (uint64_t)(2 * k), idesc, (fresh && k == 0) ? 0u : 1u);
                }
                tc_commit_pair(smem_u32(&bar_b_empty[bst]));
                if (dy == 2) tc_commit_pair(smem_u32(&bar_a_empty[aslot]));
              }
              __syncwarp();
              fresh = 0u;
              if (++bst == p.b_stages) { bst = 0; bphase ^= 1u; }
            }
            if (!ok) break;
            if (++aslot == p.a_slots) { aslot = 0; aphase ^= 1u; }
          }
          if (!ok) break;
        }
        if (!ok) break;
        if (elect_one()) tc_commit_pair(smem_u32(&bar_tmem_full[buf]));
        __syncwarp();
        if (++buf == p.nbuf) { buf = 0; tphase ^= 1u; }
      }
    }
  } else if (warp == kLoadWarp) {
    // ------------------------------------------------------------ cached-output loads
    if (lane == 0) {
      int oslot = 0;
      uint32_t ophase = 0;
      bool ok = true;
      const int quarters = p.n_real / 64;
      for (int tile = pair_id; tile < p.total_tiles && ok; tile += num_pairs) {
        const PairTile t = decode(tile, rank, p);
        for (int m = 0; m < p.mh && ok; ++m) {
          for (int hh = 0; hh < quarters; ++hh) {
            ok = mbar_wait(smem_u32(&bar_o_empty[oslot]), ophase ^ 1u, abort_flag);
            if (!ok) break;
            const uint32_t ofull = smem_u32(&bar_o_full[oslot]);
            if (p.accumulate) {
              mbar_arrive_expect_tx(ofull, (uint32_t)kOHalfBytes);
              tma_load_3d(obuf + oslot * kOHalfBytes, &map_o, ofull,
                          (t.rb * p.rows + m * p.half_rows) * p.w, t.nt * p.n_real + hh * 64, t.n);
            } else {
              mbar_arrive(ofull);
            }
            if (++oslot == p.o_slots) { oslot = 0; ophase ^= 1u; }
          }
        }
      }
    }
  } else if (warp >= 2 && warp < 2 + kEpiWarps) {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    // Two warps share each tensor-memory lane quarter; each takes 32 of the 64 channels of a
    // cached-output half tile.  A lane is one output pixel of this CTA.
    const int quarter = warp & 3;
    const int sub = (warp - 2) >> 2;
    const int ep_tid = threadIdx.x - 64;
    const int row = quarter * 32 + lane;
    const int quarters = p.n_real / 64;
    const uint32_t empty_remote = map_to_cta(smem_u32(&bar_tmem_empty[0]), 0);
    int buf = 0, oslot = 0, last_nt = -1;
    uint32_t tphase = 0, ophase = 0;
    bool ok = true;
    for (int tile = pair_id; tile < p.total_tiles; tile += num_pairs) {
      const PairTile t = decode(tile, rank, p);
      if (t.nt != last_nt) {
        asm volatile("bar.sync 1, 256;" ::: "memory");
        for (int c = ep_tid; c < p.n_real; c += 256) {
          ep_scale[c] = __fmul_rn(p.x_scale[0], p.w_scale[t.nt * p.n_real + c]);
          ep_corr[c] = p.w_corr ? p.w_corr[t.nt * p.n_real + c] : 0;
          ep_off[c] = p.x_zp ? -((int)p.x_zp[0] - 128) * p.w_csum[t.nt * p.n_real + c] : 0;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        last_nt = t.nt;
      }
      if (ok) ok = mbar_wait(smem_u32(&bar_tmem_full[buf]), tphase, abort_flag);
      if (!ok) break;
      tc_fence_after();
      for (int m = 0; m < p.mh && ok; ++m) {
        const uint32_t t_row =
            tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * buf_cols + m * p.umma_n);
        int rsum = 0;
        if (p.w_corr) {      // column n_real: sum of the receptive field's activation codes
          tc_ld1(t_row + (uint32_t)p.n_real, rsum);
          tc_wait_ld();
        }
        for (int hh = 0; hh < quarters; ++hh) {
          const int colbase = hh * 64 + sub * 32;
          const size_t out_off = ((size_t)t.n * p.cout + t.nt * p.n_real + colbase) * (size_t)(p.h * p.w) +
                                 (size_t)(t.rb * p.rows + m * p.half_rows) * p.w + row;
          float res[32];
          if (p.residual) {
#pragma unroll
            for (int j = 0; j < 32; ++j) res[j] = __ldg(p.residual + out_off + (size_t)j * (p.h * p.w));
          }
          ok = mbar_wait(smem_u32(&bar_o_full[oslot]), ophase, abort_flag);
          if (!ok) break;
          const float* orow = obuf_ptr + (size_t)oslot * (kOHalfBytes / 4) + (size_t)(sub * 32) * 128 + row;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = p.accumulate ? orow[j * 128] : 0.0f;
          // the slot is free as soon as it has been read: new values leave from registers
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_o_empty[oslot]));
          int a[32];
          tc_ld32(t_row + colbase, a);
          tc_wait_ld();
          const bool last = (m == p.mh - 1) && (hh == quarters - 1);
          if (last) {
            // the accumulator buffer of BOTH CTAs is released on the leader's barrier
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if (rank == 0) mbar_arrive(smem_u32(&bar_tmem_empty[buf]));
              else mbar_arrive_remote(empty_remote + (uint32_t)(buf * 8));
            }
          }
          if (p.w_corr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) a[j] += ep_corr[colbase + j] * rsum;
          }
          if (p.x_zp) {
#pragma unroll
            for (int j = 0; j < 32; ++j) a[j] += ep_off[colbase + j];
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fmaf((float)a[j], ep_scale[colbase + j], v[j]);
#pragma unroll
          for (int j = 0; j < 32; ++j) p.o_out[out_off + (size_t)j * (p.h * p.w)] = v[j];
          if (p.residual) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              p.sum_out[out_off + (size_t)j * (p.h * p.w)] = __fadd_rn(res[j], v[j]);
          }
          if (++oslot == p.o_slots) { oslot = 0; ophase ^= 1u; }
        }
      }
      if (!ok) break;
      if (++buf == p.nbuf) { buf = 0; tphase ^= 1u; }
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  if (abort_sh) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);   // let copies in flight land
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();        // the peer may still be read by / signalling this CTA
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
  }
}

bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

double wave_efficiency(int tiles, int units) {
  const int waves = (tiles + units - 1) / units;
  return (double)tiles / ((double)waves * units);
}

}  // namespace

// Whether the pair kernel covers this call.
bool pair_supported(const modiff_conv_geom* g, int with_sum_rows, int per_sample, const float* bias,
                    const int32_t* acc_out, const float* o_hat) {
  if (g->kh != 3 || g->kw != 3 || g->stride != 1) return false;
  if (g->pad_t != 1 || g->pad_b != 1 || g->pad_l != 1 || g->pad_r != 1) return false;
  if (per_sample || bias || acc_out || g->split != 0) return false;
  if (g->cout % 128 != 0 || g->cin < 128 || g->cin % 16 != 0) return false;
  if (!is_pow2(g->w) || !is_pow2(g->h) || g->w < 16 || g->w > 64) return false;
  if (g->h * g->w < 128 || (128 / g->w) > g->h) return false;
  // a pair covers two consecutive 128-pixel (or 256-pixel) blocks
  if (((int64_t)g->batch * (g->h / (128 / g->w))) % 2 != 0) return false;
  if (((uintptr_t)o_hat & 15) != 0) return false;
  return true;
}

int launch_igemm_pair(const int8_t* codes, const int8_t* wcodes, int with_sum_rows,
                      const float* x_scale, const float* w_scale, const int32_t* w_corr,
                      float* o_hat, int accumulate, const modiff_conv_geom* g, cudaStream_t s,
                      const float* residual, float* sum_out, const float* x_zp,
                      const int32_t* w_csum) {
  EncodeTiledFn encode = get_encode_fn();
  if (!encode) return set_error(MODIFF_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is not available");
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    MODIFF_CUDA(cudaGetDevice(&dev));
    MODIFF_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  const int pairs = sm_count / 2;
  Derived d = derive(*g);
  PairParams p;
  p.w = g->w;
  p.h = g->h;
  p.batch = g->batch;
  p.cout = g->cout;
  // 256 output channels per tile where the packed weights are plain 128-row tiles (no
  // receptive-field-sum rows) and the layer has them; else one 128-channel tile (144 rows with
  // the sum rows)
  if (with_sum_rows) {
    p.umma_n = 144;
    p.n_real = 128;
  } else if (g->cout % 256 == 0) {
    p.umma_n = 256;
    p.n_real = 256;
  } else {
    p.umma_n = 128;
    p.n_real = 128;
  }
  p.b_tile_rows = p.umma_n;
  p.b_half_rows = p.umma_n / 2;
  p.b_tile_bytes = p.b_half_rows * kChunkK;
  p.n_tiles = g->cout / p.n_real;
  const int rows1 = 128 / g->w, rows2 = 256 / g->w;
  const int chunks = ceil_div(g->cin, kChunkK);
  // 256 pixels per CTA halve the weight fill per output but need mh * umma_n accumulator
  // columns per buffer: compare shared-memory fill bytes per 128 output pixels divided by the
  // wave efficiency; a single accumulator buffer (512 columns in use) costs the overlap of the
  // epilogue with the next tile's MMAs, charged as one eighth
  auto cost = [&](int mh) {
    const int rows = mh * rows1;
    const double fill = (3.0 * chunks * (rows + 2) * g->w * kChunkK + 9.0 * chunks * p.b_tile_bytes) / mh +
                        (p.n_real / 64) * (double)kOHalfBytes;
    const int nbuf = (2 * mh * p.umma_n <= 512) ? 2 : 1;
    const int64_t mblocks = (int64_t)g->batch * (g->h / rows);
    const double eff = wave_efficiency((int)(mblocks / 2) * p.n_tiles, pairs);
    return fill / eff * (nbuf == 1 ? 1.125 : 1.0);
  };
  p.mh = 1;
  const bool mh2_ok = rows2 <= g->h && g->h % rows2 == 0 && 2 * p.umma_n <= 512 &&
                      ((int64_t)g->batch * (g->h / rows2)) % 2 == 0;
  if (mh2_ok && cost(2) < cost(1)) p.mh = 2;
  if (const char* e = getenv("MODIFF_PAIR_MH")) {      // measurement aid: force the tile height
    if (e[0] == '1') p.mh = 1;
    if (e[0] == '2' && mh2_ok) p.mh = 2;
  }
  p.rows = p.mh * rows1;
  p.half_rows = rows1;
  p.blocks_per_image = g->h / p.rows;
  p.total_tiles = (int)(((int64_t)g->batch * p.blocks_per_image) / 2) * p.n_tiles;
  p.chunks = chunks;
  p.kp = d.kp;
  p.a_bytes = (p.rows + 2) * g->w * kChunkK;
  p.a_slot_bytes = round_up(p.a_bytes, 1024);
  p.nbuf = (2 * p.mh * p.umma_n <= 512) ? 2 : 1;
  const int cols_needed = p.nbuf * p.mh * p.umma_n;
  p.tmem_cols = cols_needed <= 128 ? 128 : (cols_needed <= 256 ? 256 : 512);
  const int budget = 222 * 1024;
  p.a_slots = 2;
  p.o_slots = 2;
  auto left = [&]() { return budget - p.a_slots * p.a_slot_bytes - p.o_slots * kOHalfBytes; };
  if (left() - kOHalfBytes >= 3 * p.b_tile_bytes) p.o_slots = 3;
  if (left() - p.a_slot_bytes >= 4 * p.b_tile_bytes) p.a_slots = 3;
  const int fixed = p.a_slots * p.a_slot_bytes + p.o_slots * kOHalfBytes;
  p.b_stages = (budget - fixed) / p.b_tile_bytes;
  if (p.b_stages > kMaxBStages) p.b_stages = kMaxBStages;
  if (p.b_stages < 2) return set_error(MODIFF_ERR_UNSUPPORTED, "tile does not fit shared memory");
  p.accumulate = accumulate;
  p.x_scale = x_scale;
  p.w_scale = w_scale;
  p.w_corr = w_corr;
  p.x_zp = x_zp;
  p.w_csum = w_csum;
  p.residual = residual;
  p.sum_out = sum_out;
  p.o_out = o_hat;
  const size_t smem = (size_t)fixed + (size_t)p.b_stages * p.b_tile_bytes;

  CUtensorMap map_a, map_b, map_o;
  {
    cuuint64_t dims[5] = {(cuuint64_t)d.cp, (cuuint64_t)d.wp, (cuuint64_t)d.hp, 1u,
                          (cuuint64_t)g->batch};
    cuuint64_t strides[4] = {(cuuint64_t)d.cp, (cuuint64_t)d.wp * d.cp,
                             (cuuint64_t)d.hp * d.wp * d.cp, (cuuint64_t)d.hp * d.wp * d.cp};
    cuuint32_t box[5] = {(cuuint32_t)kChunkK, (cuuint32_t)g->w, (cuuint32_t)(p.rows + 2), 1u, 1u};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = encode(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, (void*)codes, dims, strides, box,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return set_error(MODIFF_ERR_CUDA, "cuTensorMapEncodeTiled(activation codes) failed: %d", (int)r);
  }
  {
    const int tiles128 = with_sum_rows ? ceil_div(g->cout, 128) * 144 : round_up(g->cout, 128);
    cuuint64_t dims[2] = {(cuuint64_t)d.taps * d.kp, (cuuint64_t)tiles128};
    cuuint64_t strides[1] = {(cuuint64_t)d.taps * d.kp};
    cuuint32_t box[2] = {(cuuint32_t)kChunkK, (cuuint32_t)p.b_half_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)wcodes, dims, strides, box,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return set_error(MODIFF_ERR_CUDA, "cuTensorMapEncodeTiled(weight codes) failed: %d", (int)r);
  }
  {
    const int hw = g->h * g->w;
    cuuint64_t dims[3] = {(cuuint64_t)hw, (cuuint64_t)g->cout, (cuuint64_t)g->batch};
    cuuint64_t strides[2] = {(cuuint64_t)hw * 4, (cuuint64_t)g->cout * hw * 4};
    cuuint32_t box[3] = {128u, 64u, 1u};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode(&map_o, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)o_hat, dims, strides, box,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return set_error(MODIFF_ERR_CUDA, "cuTensorMapEncodeTiled(cached output) failed: %d", (int)r);
  }

  static SmemLimit smem_limit;
  MODIFF_CUDA(raise_smem_limit(igemm_pair_kernel, smem, smem_limit));
  const int use_pairs = p.total_tiles < pairs ? p.total_tiles : pairs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * use_pairs);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MODIFF_CUDA(cudaLaunchKernelEx(&cfg, igemm_pair_kernel, map_a, map_b, map_o, p));
  MODIFF_LAUNCH_CHECK("igemm_pair_kernel");
  return MODIFF_OK;
}

int read_device_status_pair(int* status, int reset) { return read_status_this_unit(status, reset); }

}  // namespace modiff
