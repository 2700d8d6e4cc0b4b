// Several small quantised linear layers that read the SAME activation codes, in one launch.
//
// Every residual block projects the same swish(temb) (ddim/models/diffusion.py:121-123, 297-301;
// ldm/modules/diffusionmodules/openaimodel.py:236-262): ~20 GEMMs of batch x 512 x 256 per
// step, each far too small to fill the GPU and dominated by launch and prologue time.  The
// residual codes are shared already (one quantisation per step); this kernel also shares the
// launch: a block owns 16 output channels of one layer (its weight rows sit in shared memory)
// and one thread owns one batch row, accumulating with dp4a.
//
// Arithmetic per layer: out = o_hat + (sum codes * (q - zp)) * delta_x * delta_w[c]
// (qdiff/quant_layer.py:345-365), integer part exact.
#include "common.cuh"

namespace modiff {
namespace {

constexpr int kGroupChannels = 16;
constexpr int kGroupThreads = 256;

__global__ void __launch_bounds__(kGroupThreads)
linear_group_kernel(const int8_t* __restrict__ codes, const float* __restrict__ x_scale, int rows,
                    int cin, int kp, const modiff_linear_item* __restrict__ items,
                    const int32_t* __restrict__ block_map) {
  extern __shared__ __align__(16) int8_t w_sh[];   // [16][kp]
  const int layer = block_map[2 * blockIdx.x];
  const int c0 = block_map[2 * blockIdx.x + 1];
  const modiff_linear_item it = items[layer];
  const int pieces = kp / 16;
  for (int idx = threadIdx.x; idx < kGroupChannels * pieces; idx += blockDim.x) {
    const int r = idx / pieces, piece = idx - r * pieces;
    const int co = c0 + r;
    int4 v = make_int4(0, 0, 0, 0);
    if (co < it.cout) {
      const size_t slot = it.with_sum_rows ? (size_t)(co / 128) * 144 + (co % 128) : (size_t)co;
      v = __ldg(reinterpret_cast<const int4*>(it.wcodes + slot * kp) + piece);
    }
    reinterpret_cast<int4*>(w_sh)[idx] = v;
  }
  __syncthreads();
  const int n = blockIdx.y * blockDim.x + threadIdx.x;
  if (n >= rows) return;
  int acc[kGroupChannels];
#pragma unroll
  for (int c = 0; c < kGroupChannels; ++c) acc[c] = 0;
  int rsum = 0;
  const int4* arow = reinterpret_cast<const int4*>(codes + (size_t)n * cin);
  for (int k = 0; k < cin / 16; ++k) {
    const int4 a = __ldg(arow + k);
    rsum = __dp4a(a.x, 0x01010101, rsum);
    rsum = __dp4a(a.y, 0x01010101, rsum);
    rsum = __dp4a(a.z, 0x01010101, rsum);
    rsum = __dp4a(a.w, 0x01010101, rsum);
#pragma unroll
    for (int c = 0; c < kGroupChannels; ++c) {
      const int4 w = reinterpret_cast<const int4*>(w_sh + (size_t)c * kp)[k];   // broadcast read
      int s = acc[c];
      s = __dp4a(a.x, w.x, s);
      s = __dp4a(a.y, w.y, s);
      s = __dp4a(a.z, w.z, s);
      s = __dp4a(a.w, w.w, s);
      acc[c] = s;
    }
  }
  const float xs = x_scale[0];
  float* orow = it.o_hat + (size_t)n * it.cout + c0;
#pragma unroll
  for (int c = 0; c < kGroupChannels; ++c) {
    const int co = c0 + c;
    if (co < it.cout) {
      int iv = acc[c];
      if (it.w_corr) iv += it.w_corr[co] * rsum;
      orow[c] = fmaf((float)iv, __fmul_rn(xs, it.w_scale[co]), orow[c]);
    }
  }
}

}  // namespace
}  // namespace modiff

using namespace modiff;

extern "C" int modiff_linear_group(const int8_t* codes, const float* x_scale, int rows, int cin,
                                   const modiff_linear_item* items, const int32_t* block_map,
                                   int n_blocks, void* stream) {
  MODIFF_CHECK_ARG(codes && x_scale && items && block_map, "NULL pointer argument");
  MODIFF_CHECK_ARG(rows > 0 && n_blocks > 0, "empty group");
  MODIFF_CHECK_ARG(cin > 0 && cin % 16 == 0 && cin <= 4096, "cin %d must be a multiple of 16 <= 4096",
                   cin);
  MODIFF_CHECK_ARG((((uintptr_t)codes | (uintptr_t)items) & 15) == 0, "buffers must be 16-byte aligned");
  const int kp = round_up(cin, 128);
  const size_t smem = (size_t)kGroupChannels * kp;
  if (smem > 48 * 1024) {
    static SmemLimit smem_limit;
    MODIFF_CUDA(raise_smem_limit(linear_group_kernel, smem, smem_limit));
  }
  dim3 grid(n_blocks, ceil_div(rows, kGroupThreads));
  linear_group_kernel<<<grid, kGroupThreads, smem, (cudaStream_t)stream>>>(codes, x_scale, rows, cin,
                                                                           kp, items, block_map);
  MODIFF_LAUNCH_CHECK("linear_group_kernel");
  return MODIFF_OK;
}
