// Tensor-pipe probe for tcgen05.mma kind::i8: one small kernel that (a) measures the int8
// ceiling of this device with the operands resident in shared memory (MMA loop only, every SM
// busy), the denominator the GEMM kernels' achieved TOPS are reported against, and (b) checks
// the operand / accumulator layout of both issue modes against a host product:
//   mode 1: cta_group::1, one CTA per SM, M = 128, N = umma_n;
//   mode 2: cta_group::2, a cluster of two CTAs on two SMs, M = 256 (128 rows per CTA),
//           N = umma_n split in halves between the two CTAs' shared memory.
// No counterpart in the reference (its arithmetic is PyTorch fp32, qdiff/quant_layer.py:345-365).
//
// Operand tiles: K = 128 bytes per row, 128-byte swizzle (the layout TMA writes), written here
// by ordinary stores.  Every wait is bounded; tensor memory is freed on every path.
#include "common.cuh"
#include "tc_common.cuh"

namespace modiff {
namespace {

constexpr int kProbeThreads = 128;
constexpr int kProbeK = 128;

struct ProbeParams {
  const int8_t* a;      // [pairs or ctas][M_total][128]
  const int8_t* b;      // [umma_n][128]
  int32_t* acc_out;     // [M_total][umma_n] of tile 0, or NULL
  int* debug;           // [4]: tensor-memory base of CTA 0 / CTA 1, their cluster ranks
  int umma_n;
  int iters;            // repetitions of the four K = 32 steps
  int m_rows;           // rows per CTA (128)
};


// rows x 128 bytes from global memory into the 128-byte-swizzled tile at `dst`
__device__ inline void fill_swizzled(uint8_t* dst, const int8_t* src, int rows) {
  for (int i = threadIdx.x; i < rows * 8; i += blockDim.x) {
    const int r = i >> 3, c = i & 7;
    const uint4 v = *reinterpret_cast<const uint4*>(src + (size_t)r * kProbeK + c * 16);
    *reinterpret_cast<uint4*>(dst + (size_t)r * kProbeK + ((c ^ (r & 7)) << 4)) = v;
  }
}

template <int GROUP>
__global__ void __launch_bounds__(kProbeThreads, 1) i8_probe_kernel(const ProbeParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_done;
  __shared__ uint32_t tmem_base_sh;
  __shared__ int abort_sh;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = (GROUP == 2) ? cluster_ctarank() : 0u;
  const int unit = (GROUP == 2) ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int b_rows = p.umma_n / GROUP;          // rows of B held by this CTA
  uint8_t* a_tile = smem_raw;
  uint8_t* b_tile = smem_raw + p.m_rows * kProbeK;
  const uint32_t tmem_cols = p.umma_n <= 128 ? 128u : (p.umma_n <= 256 ? 256u : 512u);

  if (threadIdx.x == 0) {
    abort_sh = 0;
    mbar_init(smem_u32(&bar_done), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  fill_swizzled(a_tile, p.a + ((size_t)unit * GROUP + rank) * p.m_rows * kProbeK, p.m_rows);
  fill_swizzled(b_tile, p.b + (size_t)rank * b_rows * kProbeK, b_rows);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 0) {
    if (GROUP == 2) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(&tmem_base_sh)), "r"(tmem_cols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(&tmem_base_sh)), "r"(tmem_cols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (GROUP == 2) cluster_sync_all();     // both CTAs' tiles and allocations are in place
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_sh;
  if (threadIdx.x == 0 && p.debug && unit == 0) {
    p.debug[rank] = (int)tmem_base;
    p.debug[2 + rank] = (int)rank;
  }

  if (warp == 0 && lane == 0 && rank == 0) {
    const uint32_t idesc = make_idesc_i8(128 * GROUP, p.umma_n);
    const uint64_t adesc = make_smem_desc(smem_u32(a_tile));
    const uint64_t bdesc = make_smem_desc(smem_u32(b_tile));
    for (int it = 0; it < p.iters; ++it) {
#pragma unroll
      for (int k = 0; k < kProbeK / 32; ++k) {
        const uint32_t acc = (it == 0 && k == 0) ? 0u : 1u;
        if (GROUP == 2) {
          asm volatile(
              "{\n\t.reg .pred q;\n\t"
              "setp.ne.b32 q, %4, 0;\n\t"
              "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, q;\n\t}" ::"r"(tmem_base),
              "l"(adesc + (uint64_t)(2 * k)), "l"(bdesc + (uint64_t)(2 * k)), "r"(idesc), "r"(acc)
              : "memory");
        } else {
          tc_mma_i8(tmem_base, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, acc);
        }
      }
    }
    if (GROUP == 2) {
      const uint16_t mask = 3;
      asm volatile(
          "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
          "[%0], %1;" ::"r"(smem_u32(&bar_done)), "h"(mask)
          : "memory");
    } else {
      tc_commit(smem_u32(&bar_done));
    }
  }
  __syncwarp();
  // every warp waits for the accumulators (bounded), then dumps its lane quarter of tile 0
  const bool ok = mbar_wait(smem_u32(&bar_done), 0u, &abort_sh);
  tc_fence_after();
  if (ok && p.acc_out && unit == 0) {
    const int row = warp * 32 + lane;
    for (int c0 = 0; c0 < p.umma_n; c0 += 32) {
      int v[32];
      tc_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
      tc_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (c0 + j < p.umma_n)
          p.acc_out[((size_t)rank * p.m_rows + row) * p.umma_n + c0 + j] = v[j];
    }
  }
  tc_fence_before();
  __syncthreads();
  if (GROUP == 2) cluster_sync_all();     // the peer may still read operands / accumulators
  if (warp == 0) {
    tc_fence_after();
    if (GROUP == 2)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"(tmem_cols) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"(tmem_cols) : "memory");
  }
}

// A wait that nothing satisfies: the barrier expects one arrival and no thread arrives.  The
// waiting thread gives up after `limit_ns`, records it in the status word and the kernel
// returns normally: the path every tensor-core kernel takes when a copy or a peer never
// signals, exercised here without any copy or tensor-memory allocation in flight.
__global__ void wait_probe_kernel(unsigned long long limit_ns, int* gave_up) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_sh;
  if (threadIdx.x == 0) {
    abort_sh = 0;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait_limit(smem_u32(&bar), 0u, &abort_sh, limit_ns);
    if (gave_up) *gave_up = ok ? 0 : 1;
  }
  __syncthreads();
}

}  // namespace

int read_device_status_probe(int* status, int reset) { return read_status_this_unit(status, reset); }

}  // namespace modiff

using namespace modiff;

extern "C" int modiff_i8_mma_probe(int mode, int umma_n, int iters, int units, const int8_t* a,
                                   const int8_t* b, int32_t* acc_out, int* debug, void* stream) {
  MODIFF_CHECK_ARG(mode == 1 || mode == 2, "mode must be 1 (cta_group::1) or 2 (cta_group::2)");
  MODIFF_CHECK_ARG(umma_n >= 32 && umma_n <= 256 && umma_n % 32 == 0,
                   "umma_n must be a multiple of 32 in [32, 256]");
  MODIFF_CHECK_ARG(iters >= 1 && units >= 1, "iters and units must be positive");
  MODIFF_CHECK_ARG(a && b, "NULL operand pointer");
  MODIFF_CHECK_ARG((((uintptr_t)a | (uintptr_t)b) & 15) == 0, "operands must be 16-byte aligned");
  ProbeParams p;
  p.a = a;
  p.b = b;
  p.acc_out = acc_out;
  p.debug = debug;
  p.umma_n = umma_n;
  p.iters = iters;
  p.m_rows = 128;
  const size_t smem = (size_t)(128 + umma_n / mode) * kProbeK + 1024;
  cudaStream_t s = (cudaStream_t)stream;
  if (mode == 1) {
    static SmemLimit lim;
    MODIFF_CUDA(raise_smem_limit(i8_probe_kernel<1>, smem, lim));
    i8_probe_kernel<1><<<units, kProbeThreads, smem, s>>>(p);
  } else {
    static SmemLimit lim;
    MODIFF_CUDA(raise_smem_limit(i8_probe_kernel<2>, smem, lim));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * units);
    cfg.blockDim = dim3(kProbeThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MODIFF_CUDA(cudaLaunchKernelEx(&cfg, i8_probe_kernel<2>, p));
  }
  MODIFF_LAUNCH_CHECK("i8_probe_kernel");
  return MODIFF_OK;
}

extern "C" int modiff_wait_probe(int64_t limit_ns, int* gave_up, void* stream) {
  MODIFF_CHECK_ARG(limit_ns > 0 && limit_ns <= 1000000000ll,
                   "limit_ns must lie in (0, 1e9]: the probe is meant to give up quickly");
  wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((unsigned long long)limit_ns, gave_up);
  MODIFF_LAUNCH_CHECK("wait_probe_kernel");
  return MODIFF_OK;
}
