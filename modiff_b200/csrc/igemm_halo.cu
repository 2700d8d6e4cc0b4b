// Int8 implicit-GEMM for 3x3, stride-1, pad-1 convolutions with activation-tile reuse.
//
// igemm_tc_kernel fetches one activation tile per filter tap (nine copies of almost the same
// pixels) and one weight tile per tap for every 128 output pixels; at these layer sizes the
// kernel is bound by that shared-memory fill traffic, not by the tensor cores or by HBM.
// This variant cuts the fill traffic per output pixel by about 40 %:
//   - an output tile is `rows` full image rows (128 or 256 pixels of ONE image).  For each of
//     the three horizontal taps dx one copy of rows+2 input rows (shifted by dx) arrives by
//     TMA; the three vertical taps are the same copy read at a row offset of dy*w*128 bytes,
//     which is a multiple of the 1024-byte swizzle period, so the UMMA descriptor just starts
//     later.  3 activation copies per K chunk instead of 9.
//   - with 256 pixels per tile two M=128 MMAs share every weight tile.
// Accumulators: int32 in tensor memory, [buffer][m-half][128 columns], double buffered.
// Epilogue: the cached output o_hat arrives in half tiles (64 channels x 128 pixels) by bulk
// tensor copies through a ring of two or three shared-memory slots; a slot is released as soon
// as the epilogue warps have read it into registers, and out = o_hat + acc * (delta_x *
// delta_w[c]) is stored straight from registers (a lane is a pixel: 128 consecutive bytes per
// channel and warp).  An earlier version sent the new values back through the same slot with a
// bulk store; the slot then stayed busy for load latency + epilogue + store drain, and that round
// trip, not the operand feed or the tensor pipe, set the kernel's pace (the L2-to-SM port was
// 17 % busy, the tensor pipe 31 %).
// Roles: warp 0 operand TMA, warp 1 MMA issue, warps 2-9 epilogue, warp 10 cached-output loads.
// Every mbarrier wait is bounded.
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
constexpr int kMaxBStages = 6;
constexpr int kLoadWarp = 2 + kEpiWarps;
constexpr int kThreads = 32 * (3 + kEpiWarps);
// packed 4-bit operands: four more warps expand nibbles into the int8 operand tiles
constexpr int kUnpackWarps = 4;
constexpr int kFirstUnpackWarp = kLoadWarp + 1;
constexpr int kThreadsPacked = kThreads + 32 * kUnpackWarps;
constexpr int kPkSlots = 2;

struct HaloParams {
  int w, h, batch, cout;
  int rows;             // output rows per tile
  int mh;               // 128-pixel halves per tile: 1 or 2
  int half_rows;        // rows / mh
  int tiles_h;          // h / rows
  int n_tiles;          // cout / n_real
  int n_real;           // output channels per tile: 128, or 256 (plain 128-row weight tiles only)
  int nbuf;             // accumulator buffers in tensor memory: 2, or 1 when mh * umma_n = 512
  int total_tiles;
  int chunks;           // 128-byte K chunks per tap
  int kp;               // weight K stride per tap
  int b_stages;
  int a_bytes;          // bytes of one activation copy: (rows + 2) * w * 128
  int a_slot_bytes;
  int a_slots;          // activation copies in flight (2..4)
  int tmem_cols;
  int o_slots;          // cached-output half tiles in flight (2 or 3)
  float* o_out;         // the cached output itself: new values are stored straight from registers
  int accumulate;
  int umma_n;           // 128 or 256, or 144 with the receptive-field-sum rows (zero-point correction)
  int b_tile_bytes;     // umma_n * 128
  const float* x_scale;
  const float* w_scale;
  const int32_t* w_corr;
  const float* x_zp;          // offset (8-bit asymmetric) activation codes, else NULL
  const int32_t* w_csum;
  const float* residual;   // optional [batch][cout][h*w]: sum_out = new output + residual
  float* sum_out;
  // packed 4-bit operands (igemm_halo_kernel<true>): staging slots hold what TMA delivers, two
  // codes per byte; the unpack warps write the int8 tiles the MMAs read
  int pk_a_bytes;          // one packed activation copy: a_bytes / 2
  int pk_a_slot_bytes;
  int pk_b_bytes;          // one packed weight tile: b_tile_bytes / 2
  const float* w_zp;       // weight zero point per output channel (packed weights hold q, not q - zp)
};

struct HaloTile {
  int n, th, nt;
};
__device__ inline HaloTile decode(int tile, const HaloParams& p) {
  HaloTile t;
  t.nt = tile % p.n_tiles;
  const int m = tile / p.n_tiles;
  t.th = m % p.tiles_h;
  t.n = m / p.tiles_h;
  return t;
}

// 16 int8 codes from 16 nibbles (8 bytes, element 2i in the low nibble of byte i, 2i+1 in the
// high nibble: the order of qdiff/quant_layer_int4.py:341-346).  SIGNED: two's-complement
// nibbles are sign-extended; else unsigned nibbles minus `sub4` (a byte replicated four times).
template <bool SIGNED>
__device__ inline uint4 unpack16(uint2 pk, uint32_t sub4) {
  uint32_t o[4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t w = h == 0 ? pk.x : pk.y;
    uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
    if (SIGNED) {
      lo |= (lo & 0x08080808u) * 0x1Eu;      // bit 3 set -> bits 4..7 set, no carry between bytes
      hi |= (hi & 0x08080808u) * 0x1Eu;
    } else {
      lo = __vsub4(lo, sub4);
      hi = __vsub4(hi, sub4);
    }
    o[2 * h] = __byte_perm(lo, hi, 0x5140);      // lo0 hi0 lo1 hi1
    o[2 * h + 1] = __byte_perm(lo, hi, 0x7362);  // lo2 hi2 lo3 hi3
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

template <bool PACKED>
__global__ void __launch_bounds__(PACKED ? kThreadsPacked : kThreads, 1)
igemm_halo_kernel(const __grid_constant__ CUtensorMap map_a,
                  const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_o, const HaloParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_a_full[kMaxASlots], bar_a_empty[kMaxASlots];
  __shared__ __align__(8) uint64_t bar_b_full[kMaxBStages], bar_b_empty[kMaxBStages];
  __shared__ __align__(8) uint64_t bar_tmem_full[2], bar_tmem_empty[2];
  __shared__ __align__(8) uint64_t bar_o_full[kMaxOSlots], bar_o_empty[kMaxOSlots];
  __shared__ __align__(8) uint64_t bar_pa_full[kPkSlots], bar_pa_empty[kPkSlots];
  __shared__ __align__(8) uint64_t bar_pb_full[kPkSlots], bar_pb_empty[kPkSlots];
  __shared__ uint32_t zp4_sh[128];
  __shared__ uint32_t tmem_base_sh;
  __shared__ int abort_sh;
  __shared__ float ep_scale[256];
  __shared__ int ep_corr[256];
  __shared__ int ep_off[256];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &abort_sh;

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t a_ring = raw;
  const uint32_t b_ring = a_ring + (uint32_t)p.a_slots * (uint32_t)p.a_slot_bytes;
  const uint32_t b_tile = (uint32_t)p.b_tile_bytes;
  const uint32_t obuf = b_ring + (uint32_t)p.b_stages * b_tile;
  float* obuf_ptr = reinterpret_cast<float*>(smem_raw + (obuf - raw));
  // staging of packed operands behind the cached-output ring
  const uint32_t pk_a = obuf + (uint32_t)p.o_slots * kOHalfBytes;
  const uint32_t pk_b = pk_a + kPkSlots * (uint32_t)p.pk_a_slot_bytes;

  if (threadIdx.x == 0) {
    abort_sh = 0;
    // operand tiles are complete when the copy has landed, or, with packed operands, when the
    // four unpack warps have written them
    const uint32_t fillers = PACKED ? kUnpackWarps : 1;
    for (int s = 0; s < p.a_slots; ++s) {
      mbar_init(smem_u32(&bar_a_full[s]), fillers);
      mbar_init(smem_u32(&bar_a_empty[s]), 1);
    }
    for (int s = 0; s < p.b_stages; ++s) {
      mbar_init(smem_u32(&bar_b_full[s]), fillers);
      mbar_init(smem_u32(&bar_b_empty[s]), 1);
    }
    for (int s = 0; s < kPkSlots; ++s) {
      mbar_init(smem_u32(&bar_pa_full[s]), 1);
      mbar_init(smem_u32(&bar_pa_empty[s]), kUnpackWarps);
      mbar_init(smem_u32(&bar_pb_full[s]), 1);
      mbar_init(smem_u32(&bar_pb_empty[s]), kUnpackWarps);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_tmem_full[b]), 1);
      mbar_init(smem_u32(&bar_tmem_empty[b]), kEpiWarps);
    }
    for (int b = 0; b < p.o_slots; ++b) {
      mbar_init(smem_u32(&bar_o_full[b]), 1);
      mbar_init(smem_u32(&bar_o_empty[b]), kEpiWarps);
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
  const int buf_cols = p.mh * p.umma_n;

  if (warp == 0 && PACKED) {
    // ------------------------------------------------------------ packed operand TMA producer
    // Same order of copies as below, two codes per byte, into the staging slots.
    if (lane == 0) {
      int as = 0, bs = 0;
      uint32_t aphase = 0, bphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
        const HaloTile t = decode(tile, p);
        for (int ch = 0; ch < p.chunks && ok; ++ch) {
          for (int dx = 0; dx < 3 && ok; ++dx) {
            ok = mbar_wait(smem_u32(&bar_pa_empty[as]), aphase ^ 1u, abort_flag);
            if (!ok) break;
            const uint32_t afull = smem_u32(&bar_pa_full[as]);
            mbar_arrive_expect_tx(afull, (uint32_t)p.pk_a_bytes);
            tma_load_5d(pk_a + as * (uint32_t)p.pk_a_slot_bytes, &map_a, afull, ch * (kChunkK / 2), dx,
                        t.th * p.rows, 0, t.n);
            if (++as == kPkSlots) { as = 0; aphase ^= 1u; }
            for (int dy = 0; dy < 3; ++dy) {
              ok = mbar_wait(smem_u32(&bar_pb_empty[bs]), bphase ^ 1u, abort_flag);
              if (!ok) break;
              const uint32_t bfull = smem_u32(&bar_pb_full[bs]);
              mbar_arrive_expect_tx(bfull, (uint32_t)p.pk_b_bytes);
              tma_load_2d(pk_b + bs * (uint32_t)p.pk_b_bytes, &map_b, bfull,
                          ((dy * 3 + dx) * p.kp + ch * kChunkK) / 2, t.nt * p.umma_n);
              if (++bs == kPkSlots) { bs = 0; bphase ^= 1u; }
            }
          }
        }
      }
    }
  } else if (PACKED && warp >= kFirstUnpackWarp) {
    // ------------------------------------------------------------ unpack warps (packed operands)
    // nibbles -> int8 in the 128-byte-swizzled K-major layout a tensor copy would have written:
    // row r, 16-byte chunk j of the tile lives at r * 128 + ((j ^ (r & 7)) << 4).  Activation
    // codes are two's-complement nibbles; weight nibbles hold the unsigned code q and become
    // q - zero_point[channel], the value the convolution multiplies.
    const int ut = threadIdx.x - 32 * kFirstUnpackWarp;          // 0 .. 127
    uint8_t* const a_ring_ptr = smem_raw;
    uint8_t* const b_ring_ptr = smem_raw + (b_ring - raw);
    const uint8_t* const pk_a_ptr = smem_raw + (pk_a - raw);
    const uint8_t* const pk_b_ptr = smem_raw + (pk_b - raw);
    const int a_items = (p.a_bytes / kChunkK) * 8;               // 16-byte output chunks per copy
    const int b_items = p.umma_n * 8;
    int as = 0, bs = 0, aslot = 0, bst = 0, last_nt = -1;
    uint32_t pa_phase = 0, pb_phase = 0, aphase = 0, bphase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
      const HaloTile t = decode(tile, p);
      if (t.nt != last_nt) {
        asm volatile("bar.sync 2, 128;" ::: "memory");           // the table's readers are done
        const uint32_t z = (uint32_t)(int)p.w_zp[t.nt * p.umma_n + ut] & 0xffu;
        zp4_sh[ut] = z * 0x01010101u;
        asm volatile("bar.sync 2, 128;" ::: "memory");
        last_nt = t.nt;
      }
      for (int ch = 0; ch < p.chunks && ok; ++ch) {
        for (int dx = 0; dx < 3 && ok; ++dx) {
          ok = mbar_wait(smem_u32(&bar_pa_full[as]), pa_phase, abort_flag) &&
               mbar_wait(smem_u32(&bar_a_empty[aslot]), aphase ^ 1u, abort_flag);
          if (!ok) break;
          {
            const uint8_t* src = pk_a_ptr + (size_t)as * p.pk_a_slot_bytes;
            uint8_t* dst = a_ring_ptr + (size_t)aslot * p.a_slot_bytes;
            for (int i = ut; i < a_items; i += 32 * kUnpackWarps) {
              const int r = i >> 3, j = i & 7;
              const uint2 pk = *reinterpret_cast<const uint2*>(src + r * 64 + j * 8);
              *reinterpret_cast<uint4*>(dst + r * 128 + ((j ^ (r & 7)) << 4)) = unpack16<true>(pk, 0u);
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(smem_u32(&bar_a_full[aslot]));
            mbar_arrive(smem_u32(&bar_pa_empty[as]));
          }
          if (++as == kPkSlots) { as = 0; pa_phase ^= 1u; }
          if (++aslot == p.a_slots) { aslot = 0; aphase ^= 1u; }
          for (int dy = 0; dy < 3; ++dy) {
            ok = mbar_wait(smem_u32(&bar_pb_full[bs]), pb_phase, abort_flag) &&
                 mbar_wait(smem_u32(&bar_b_empty[bst]), bphase ^ 1u, abort_flag);
            if (!ok) break;
            {
              const uint8_t* src = pk_b_ptr + (size_t)bs * p.pk_b_bytes;
              uint8_t* dst = b_ring_ptr + (size_t)bst * p.b_tile_bytes;
              for (int i = ut; i < b_items; i += 32 * kUnpackWarps) {
                const int r = i >> 3, j = i & 7;
                const uint2 pk = *reinterpret_cast<const uint2*>(src + r * 64 + j * 8);
                *reinterpret_cast<uint4*>(dst + r * 128 + ((j ^ (r & 7)) << 4)) =
                    unpack16<false>(pk, zp4_sh[r]);
              }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(smem_u32(&bar_b_full[bst]));
              mbar_arrive(smem_u32(&bar_pb_empty[bs]));
            }
            if (++bs == kPkSlots) { bs = 0; pb_phase ^= 1u; }
            if (++bst == p.b_stages) { bst = 0; bphase ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------ operand TMA producer
    if (lane == 0) {
      int aslot = 0, bst = 0;
      uint32_t aphase = 0, bphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
        const HaloTile t = decode(tile, p);
        for (int ch = 0; ch < p.chunks && ok; ++ch) {
          for (int dx = 0; dx < 3 && ok; ++dx) {
            ok = mbar_wait(smem_u32(&bar_a_empty[aslot]), aphase ^ 1u, abort_flag);
            if (!ok) break;
            const uint32_t afull = smem_u32(&bar_a_full[aslot]);
            mbar_arrive_expect_tx(afull, (uint32_t)p.a_bytes);
            // padded input rows th*rows .. th*rows+rows+1, padded columns dx .. dx+w-1
            tma_load_5d(a_ring + aslot * (uint32_t)p.a_slot_bytes, &map_a, afull, ch * kChunkK, dx,
                        t.th * p.rows, 0, t.n);
            if (++aslot == p.a_slots) { aslot = 0; aphase ^= 1u; }
            for (int dy = 0; dy < 3; ++dy) {
              ok = mbar_wait(smem_u32(&bar_b_empty[bst]), bphase ^ 1u, abort_flag);
              if (!ok) break;
              const uint32_t bfull = smem_u32(&bar_b_full[bst]);
              mbar_arrive_expect_tx(bfull, b_tile);
              tma_load_2d(b_ring + bst * b_tile, &map_b, bfull,
                          (dy * 3 + dx) * p.kp + ch * kChunkK, t.nt * p.umma_n);
              if (++bst == p.b_stages) { bst = 0; bphase ^= 1u; }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp walks the loop (waits included) and one elected lane issues: descriptors
    // and addresses are then warp-uniform values.  With a single lane running the loop the
    // issue of one MMA took about 130 cycles, twice the 64 cycles the MMA occupies the tensor
    // pipe, and the issuing thread - not the operand feed, the epilogue or the tensor pipe -
    // set the pace of the kernel.
    {
      const uint32_t idesc = make_idesc_i8(128, p.umma_n);
      int aslot = 0, bst = 0, buf = 0;
      uint32_t aphase = 0, bphase = 0, tphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
        ok = mbar_wait(smem_u32(&bar_tmem_empty[buf]), tphase ^ 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
        uint32_t fresh = 1u;        // the tile's first MMA overwrites the accumulator
        for (int ch = 0; ch < p.chunks; ++ch) {
          for (int dx = 0; dx < 3; ++dx) {
            ok = mbar_wait(smem_u32(&bar_a_full[aslot]), aphase, abort_flag);
            if (!ok) break;
            const uint32_t a_base = a_ring + aslot * (uint32_t)p.a_slot_bytes;
            for (int dy = 0; dy < 3; ++dy) {
              ok = mbar_wait(smem_u32(&bar_b_full[bst]), bphase, abort_flag);
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
                  tc_mma_i8(d_tmem, adesc0 + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                            (fresh && k == 0) ? 0u : 1u);
                if (p.mh == 2) {
#pragma unroll
                  for (int k = 0; k < kChunkK / 32; ++k)
                    tc_mma_i8(d_tmem + (uint32_t)p.umma_n, adesc1 + (uint64_t)(2 * k),
                              bdesc + (uint64_t)(2 * k), idesc, (fresh && k == 0) ? 0u : 1u);
                }
                tc_commit(smem_u32(&bar_b_empty[bst]));
                if (dy == 2) tc_commit(smem_u32(&bar_a_empty[aslot]));
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
        if (elect_one()) tc_commit(smem_u32(&bar_tmem_full[buf]));
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
      for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
        const HaloTile t = decode(tile, p);
        for (int m = 0; m < p.mh && ok; ++m) {
          for (int hh = 0; hh < p.n_real / 64; ++hh) {
            ok = mbar_wait(smem_u32(&bar_o_empty[oslot]), ophase ^ 1u, abort_flag);
            if (!ok) break;
            const uint32_t ofull = smem_u32(&bar_o_full[oslot]);
            if (p.accumulate) {
              mbar_arrive_expect_tx(ofull, (uint32_t)kOHalfBytes);
              tma_load_3d(obuf + oslot * kOHalfBytes, &map_o, ofull,
                          (t.th * p.rows + m * p.half_rows) * p.w, t.nt * p.n_real + hh * 64, t.n);
            } else {
              mbar_arrive(ofull);
            }
            if (++oslot == p.o_slots) { oslot = 0; ophase ^= 1u; }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    // Two warps share each tensor-memory lane quarter; each takes 32 of the 64 channels of a
    // half tile.  A lane is one output pixel, so shared-memory accesses of a warp are 32
    // consecutive floats of one channel row.
    const int quarter = warp & 3;
    const int sub = (warp - 2) >> 2;
    const int ep_tid = threadIdx.x - 64;
    const int row = quarter * 32 + lane;
    int buf = 0, oslot = 0, last_nt = -1;
    uint32_t tphase = 0, ophase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
      const HaloTile t = decode(tile, p);
      if (t.nt != last_nt) {
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (ep_tid < p.n_real) {
          const int co = t.nt * p.n_real + ep_tid;
          const bool cv = co < p.cout;          // the last channel tile may be partly empty
          ep_scale[ep_tid] = cv ? __fmul_rn(p.x_scale[0], p.w_scale[co]) : 0.0f;
          ep_corr[ep_tid] = (cv && p.w_corr) ? p.w_corr[co] : 0;
          ep_off[ep_tid] = (cv && p.x_zp) ? -((int)p.x_zp[0] - 128) * p.w_csum[co] : 0;
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
        if (p.w_corr) {      // column 128: sum of the receptive field's activation codes
          tc_ld1(t_row + 128, rsum);
          tc_wait_ld();
        }
        for (int hh = 0; hh < p.n_real / 64; ++hh) {
          const int colbase = hh * 64 + sub * 32;
          // a lane is a pixel: for every channel the 32 lanes of a warp touch 128 consecutive
          // bytes of the NCHW tensors
          const size_t out_off = ((size_t)t.n * p.cout + t.nt * p.n_real + colbase) * (size_t)(p.h * p.w) +
                                 (size_t)(t.th * p.rows + m * p.half_rows) * p.w + row;
          // residual of the block (x + h, qdiff/quant_block.py:313): issued before the wait below
          // so that the loads are in flight while the cached-output tile arrives
          // channels of this warp's 32 that exist (all of them except in a ragged last tile)
          const int cvalid = min(32, p.cout - (t.nt * p.n_real + colbase));
          float res[32];
          if (p.residual) {
            if (cvalid >= 32) {          // warp-uniform: full tiles keep unpredicated accesses
#pragma unroll
              for (int j = 0; j < 32; ++j) res[j] = __ldg(p.residual + out_off + (size_t)j * (p.h * p.w));
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                res[j] = j < cvalid ? __ldg(p.residual + out_off + (size_t)j * (p.h * p.w)) : 0.0f;
            }
          }
          ok = mbar_wait(smem_u32(&bar_o_full[oslot]), ophase, abort_flag);
          if (!ok) break;
          const float* orow = obuf_ptr + (size_t)oslot * (kOHalfBytes / 4) + (size_t)(sub * 32) * 128 + row;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = p.accumulate ? orow[j * 128] : 0.0f;
          // the slot is free for the next cached-output tile as soon as it has been read: the new
          // values leave straight from registers, so no store has to drain from shared memory
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_o_empty[oslot]));
          int a[32];
          tc_ld32(t_row + colbase, a);
          tc_wait_ld();
          const bool last = (m == p.mh - 1) && (hh == p.n_real / 64 - 1);
          if (last) {
            // the accumulator buffer can be overwritten once every warp has read its last columns
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_tmem_empty[buf]));
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
          if (cvalid >= 32) {
#pragma unroll
            for (int j = 0; j < 32; ++j) p.o_out[out_off + (size_t)j * (p.h * p.w)] = v[j];
            if (p.residual) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                p.sum_out[out_off + (size_t)j * (p.h * p.w)] = __fadd_rn(res[j], v[j]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < cvalid) p.o_out[out_off + (size_t)j * (p.h * p.w)] = v[j];
            if (p.residual) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < cvalid) p.sum_out[out_off + (size_t)j * (p.h * p.w)] = __fadd_rn(res[j], v[j]);
            }
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
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
  }
}

bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

// share of the last wave that does work when `tiles` tiles run on `sms` persistent CTAs
double wave_efficiency(int tiles, int sms) {
  const int waves = (tiles + sms - 1) / sms;
  return (double)tiles / ((double)waves * sms);
}

}  // namespace

// Whether the activation-reuse kernel covers this call.
bool halo_supported(const modiff_conv_geom* g, int with_sum_rows, int per_sample, const float* bias,
                    const int32_t* acc_out, const float* o_hat) {
  // with correction rows only 128-pixel tiles fit tensor memory; at 16 pixels per row they were
  // measured no faster than one copy per tap
  if (with_sum_rows && g->w < 32) return false;
  if (g->kh != 3 || g->kw != 3 || g->stride != 1) return false;
  if (g->pad_t != 1 || g->pad_b != 1 || g->pad_l != 1 || g->pad_r != 1) return false;
  if (per_sample || bias || acc_out || g->split != 0) return false;
  // channel counts that are not a multiple of 128 (192, 320, ...) leave the last channel tile
  // partly empty: the cached-output copies clip at the tensor's edge, the stores are masked
  if (g->cout < 128 || g->cout % 32 != 0 || g->cin < 128 || g->cin % 16 != 0) return false;
  if (!is_pow2(g->w) || !is_pow2(g->h) || g->w < 16 || g->w > 64) return false;
  if (g->h * g->w < 128 || (128 / g->w) > g->h) return false;
  if (((uintptr_t)o_hat & 15) != 0) return false;
  return true;
}

int launch_igemm_halo(const int8_t* codes, const int8_t* wcodes, int with_sum_rows,
                      const float* x_scale, const float* w_scale, const int32_t* w_corr,
                      float* o_hat, int accumulate, const modiff_conv_geom* g, cudaStream_t s,
                      const float* residual, float* sum_out, const float* x_zp,
                      const int32_t* w_csum, const float* packed_w_zp) {
  // packed_w_zp != NULL: `codes` and `wcodes` hold two 4-bit codes per byte (activations
  // two's complement, weights the unsigned code q) and are expanded in shared memory
  const bool packed = packed_w_zp != nullptr;
  EncodeTiledFn encode = get_encode_fn();
  if (!encode) return set_error(MODIFF_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is not available");
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    MODIFF_CUDA(cudaGetDevice(&dev));
    MODIFF_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  Derived d = derive(*g);
  HaloParams p;
  p.w = g->w;
  p.h = g->h;
  p.batch = g->batch;
  p.cout = g->cout;
  // Tile shape.  The pace of this kernel is set by how fast one thread can issue MMAs, so the
  // fewer and larger they are the better: 256 output channels per MMA (UMMA N = 256, 128 cycles
  // of the tensor pipe each) wherever the packed weights are plain 128-row tiles and the layer
  // has a multiple of 256 channels, with 128-pixel tiles so that two accumulator buffers fit
  // tensor memory (2 x 256 columns) and the epilogue overlaps the next tile's MMAs.  Otherwise
  // 128 channels (144 rows with the receptive-field-sum rows) and 128 or 256 pixels.
  const int rows1 = 128 / g->w, rows2 = 256 / g->w;
  const int chunks = ceil_div(g->cin, kChunkK);
  const char* force_n = getenv("MODIFF_HALO_N");      // measurement aid: "128" keeps N = 128
  const bool wide = !with_sum_rows && !packed && g->cout % 256 == 0 &&
                    !(force_n && force_n[0] == '1');
  p.umma_n = with_sum_rows ? 144 : (wide ? 256 : 128);
  p.n_real = wide ? 256 : 128;
  p.n_tiles = ceil_div(g->cout, p.n_real);
  p.b_tile_bytes = p.umma_n * kChunkK;
  // 256-pixel tiles halve the weight traffic but can leave the last wave emptier: compare
  // shared-memory fill bytes per 128 output pixels divided by the wave efficiency
  auto cost = [&](int mh) {
    const int rows = mh * rows1;
    const double fill = (3.0 * chunks * (rows + 2) * g->w * kChunkK + 9.0 * chunks * p.b_tile_bytes) / mh +
                        4.0 * kOHalfBytes;
    return fill / wave_efficiency(g->batch * (g->h / rows) * p.n_tiles, sm_count);
  };
  p.mh = 1;
  // two m-halves of 144 columns, double buffered, would need 576 of the 512 tensor-memory columns
  if (!with_sum_rows && !wide && !packed && rows2 <= g->h && g->h % rows2 == 0 && cost(2) < cost(1))
    p.mh = 2;
  if (const char* e = getenv("MODIFF_HALO_MH")) {      // measurement aid: force the tile height
    if (e[0] == '1') p.mh = 1;
    if (e[0] == '2' && !with_sum_rows && !wide && !packed && rows2 <= g->h && g->h % rows2 == 0) p.mh = 2;
  }
  p.nbuf = 2;
  p.rows = p.mh * rows1;
  p.half_rows = rows1;
  p.tiles_h = g->h / p.rows;
  p.total_tiles = g->batch * p.tiles_h * p.n_tiles;
  p.chunks = chunks;
  p.kp = d.kp;
  p.a_bytes = (p.rows + 2) * g->w * kChunkK;
  p.a_slot_bytes = round_up(p.a_bytes, 1024);
  // shared memory: at least two activation copies, two cached-output half tiles and four weight
  // stages; what is left goes first to a third cached-output tile (its load latency from HBM is
  // the longest in the kernel), then to a third activation copy, then to weight stages
  p.pk_a_bytes = packed ? p.a_bytes / 2 : 0;
  p.pk_a_slot_bytes = round_up(p.pk_a_bytes, 128);
  p.pk_b_bytes = packed ? p.b_tile_bytes / 2 : 0;
  p.w_zp = packed_w_zp;
  const int staging = kPkSlots * (p.pk_a_slot_bytes + p.pk_b_bytes);
  const int budget = 222 * 1024 - staging;
  p.a_slots = 2;
  p.o_slots = 2;
  auto left = [&]() { return budget - p.a_slots * p.a_slot_bytes - p.o_slots * kOHalfBytes; };
  if (left() - kOHalfBytes >= 3 * p.b_tile_bytes) p.o_slots = 3;
  if (left() - p.a_slot_bytes >= 4 * p.b_tile_bytes) p.a_slots = 3;
  const int fixed = p.a_slots * p.a_slot_bytes + p.o_slots * kOHalfBytes;
  p.b_stages = (budget - fixed) / p.b_tile_bytes;
  if (p.b_stages > kMaxBStages) p.b_stages = kMaxBStages;
  if (p.b_stages < 2) return set_error(MODIFF_ERR_UNSUPPORTED, "tile does not fit shared memory");
  p.tmem_cols = (p.nbuf * p.mh * p.umma_n) > 256 ? 512 : 256;
  p.accumulate = accumulate;
  p.x_scale = x_scale;
  p.w_scale = w_scale;
  p.w_corr = w_corr;
  p.x_zp = x_zp;
  p.w_csum = w_csum;
  p.residual = residual;
  p.sum_out = sum_out;
  p.o_out = o_hat;
  const size_t smem = (size_t)fixed + (size_t)p.b_stages * p.b_tile_bytes + (size_t)staging;

  // packed operands: every byte extent along the channel / K dimension halves, and the staging
  // slots are plain rows (the unpack warps apply the swizzle)
  const int pk = packed ? 2 : 1;
  const CUtensorMapSwizzle swz = packed ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap map_a, map_b, map_o;
  {
    cuuint64_t dims[5] = {(cuuint64_t)d.cp / pk, (cuuint64_t)d.wp, (cuuint64_t)d.hp, 1u,
                          (cuuint64_t)g->batch};
    cuuint64_t strides[4] = {(cuuint64_t)d.cp / pk, (cuuint64_t)d.wp * d.cp / pk,
                             (cuuint64_t)d.hp * d.wp * d.cp / pk, (cuuint64_t)d.hp * d.wp * d.cp / pk};
    cuuint32_t box[5] = {(cuuint32_t)kChunkK / pk, (cuuint32_t)g->w, (cuuint32_t)(p.rows + 2), 1u, 1u};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = encode(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, (void*)codes, dims, strides, box,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return set_error(MODIFF_ERR_CUDA, "cuTensorMapEncodeTiled(activation codes) failed: %d", (int)r);
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)d.taps * d.kp / pk, (cuuint64_t)p.n_tiles * p.umma_n};
    cuuint64_t strides[1] = {(cuuint64_t)d.taps * d.kp / pk};
    cuuint32_t box[2] = {(cuuint32_t)kChunkK / pk, (cuuint32_t)p.umma_n};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)wcodes, dims, strides, box,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
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

  const int grid = p.total_tiles < sm_count ? p.total_tiles : sm_count;
  if (packed) {
    static SmemLimit smem_limit_packed;
    MODIFF_CUDA(raise_smem_limit(igemm_halo_kernel<true>, smem, smem_limit_packed));
    igemm_halo_kernel<true><<<grid, kThreadsPacked, smem, s>>>(map_a, map_b, map_o, p);
  } else {
    static SmemLimit smem_limit;
    MODIFF_CUDA(raise_smem_limit(igemm_halo_kernel<false>, smem, smem_limit));
    igemm_halo_kernel<false><<<grid, kThreads, smem, s>>>(map_a, map_b, map_o, p);
  }
  MODIFF_LAUNCH_CHECK("igemm_halo_kernel");
  return MODIFF_OK;
}

int read_device_status_halo(int* status, int reset) { return read_status_this_unit(status, reset); }


}  // namespace modiff
