/*
 * modiff_b200.h -- C ABI of libmodiff_b200.so
 *
 * Hand-written sm_100a CUDA for the modulated-quantization UNet sampling path of
 * MoDiff (qdiff.QuantModel / QuantModule / UniformAffineQuantizer).  The reference
 * has no native boundary: its arithmetic lives in Python/PyTorch, so every entry
 * point below cites the reference Python it stands in for (path:line inside the
 * reference project).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the comment says "host";
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it and
 *     nothing synchronises the device;
 *   - no entry point allocates device memory: callers own every buffer;
 *   - every function returns MODIFF_OK (0) or a negative/positive error code and
 *     leaves a human-readable message for modiff_last_error() (thread local);
 *   - fp32 activation tensors are NCHW (linear layers: rows x features, i.e.
 *     N = rows, H = W = 1); integer code tensors use the private layout below.
 *
 * Activation-code layout ("code planes")
 *   int8 [batch * nplanes][hp][wp][cp], nplanes = stride*stride,
 *   cp = round_up(cin, 16), hp = ceil((h + pad_t + pad_b) / stride),
 *   wp = ceil((w + pad_l + pad_r) / stride).
 *   Input pixel (y, x) of image n lives at padded coordinate (y + pad_t, x + pad_l),
 *   plane ((y + pad_t) % stride) * stride + (x + pad_l) % stride, row
 *   (y + pad_t) / stride, column (x + pad_l) / stride.  Halo positions and padded
 *   channels are never written: the caller zero-fills the buffer once.
 *
 * Weight-code layout
 *   int8 [cout_rows][kh*kw][kp], kp = round_up(cin, 128); value = q - zoff with
 *   zoff chosen per output channel so the value fits int8; w_corr = zoff - zp is
 *   the integer to multiply with the receptive-field sum of activation codes.
 */
#ifndef MODIFF_B200_H_
#define MODIFF_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MODIFF_OK 0
#define MODIFF_ERR_INVALID 1     /* bad argument / unsupported geometry */
#define MODIFF_ERR_CUDA 2        /* a CUDA runtime / driver call failed */
#define MODIFF_ERR_UNSUPPORTED 3 /* this build or device cannot run the request */
#define MODIFF_ERR_DEVICE 4      /* a kernel reported a bounded wait that ran out */

#define MODIFF_IMPL_AUTO 0
#define MODIFF_IMPL_SIMT 1     /* dp4a CUDA-core implicit GEMM (any geometry) */
#define MODIFF_IMPL_TCGEN05 2  /* tcgen05 kind::i8 tensor-core implicit GEMM */

/* Geometry of one conv2d / conv1d(k=1) / linear layer.
 * Mirrors the kwargs captured by QuantModule.__init__ (qdiff/quant_layer.py:268-278). */
typedef struct modiff_conv_geom {
  int32_t batch;  /* images, or rows for a linear layer */
  int32_t cin;
  int32_t cout;
  int32_t h, w;   /* input spatial size; 1,1 for linear */
  int32_t kh, kw;
  int32_t stride; /* 1 or 2 */
  int32_t pad_t, pad_l, pad_b, pad_r;
  int32_t split;  /* 0, or the channel count of the first activation/weight segment
                     (qdiff/quant_layer.py:313-319, 330-333, 346-349) */
} modiff_conv_geom;

/* Library / device information. */
int modiff_version(void);
const char* modiff_last_error(void);
/* Fills sm_count, cc_major, cc_minor of the current device (host pointers). */
int modiff_device_info(int* sm_count, int* cc_major, int* cc_minor);

/* Reads (and optionally clears) the sticky device status word: non-zero after a kernel
 * gave up on a bounded wait.  Synchronises the device.  `status` is a host pointer. */
int modiff_device_status(int* status, int reset);

/* Sizes (host side helpers, no device work). */
int64_t modiff_codes_bytes(const modiff_conv_geom* g);      /* activation-code buffer */
int64_t modiff_wcodes_bytes(const modiff_conv_geom* g, int with_sum_rows);
int32_t modiff_out_h(const modiff_conv_geom* g);
int32_t modiff_out_w(const modiff_conv_geom* g);
/* cout rows stored per 128-channel tile when the tcgen05 kernel needs the
 * receptive-field sum (one all-ones row + 15 zero rows are appended per tile). */
int32_t modiff_wcodes_rows(const modiff_conv_geom* g, int with_sum_rows);

/* Per-output-channel asymmetric weight quantisation, done once per weight tensor.
 * Replaces UniformAffineQuantizer.init_quantization_scale(channel_wise=True)
 * + forward on weights (qdiff/quant_layer.py:160-190, 94-102, 345-351).
 *   w        fp32 [cout][cin][kh*kw] (PyTorch conv/linear layout)
 *   wcodes   int8 weight-code layout (see top); with_sum_rows != 0 selects the
 *            tiled layout [cout/128 tiles][144 rows] used by the tcgen05 kernel
 *            when any w_corr is non-zero
 *   w_scale  fp32 [2][cout]  delta per segment (row 1 unused without split)
 *   w_zp     fp32 [2][cout]  zero point per segment (as the reference stores it)
 *   w_corr   int32 [2][cout] zoff - zp
 *   w_dq     fp32 [cin*kh*kw][cout]  dequantised weights (q - zp) * delta, K order
 *            (cin, ky, kx), for the first (unquantised-activation) step; may be NULL
 */
int modiff_weight_pack(const float* w, const modiff_conv_geom* g, int n_bits,
                       int with_sum_rows, int8_t* wcodes, float* w_scale, float* w_zp,
                       int32_t* w_corr, float* w_dq, void* stream);

/* modiff_weight_pack for a weight tensor with LEARNED rounding (AdaRound, hard targets) and
 * given scales, as a calibrated checkpoint stores them:
 *   q = clamp(floor(w / delta[c]) + (alpha >= 0) + zero_point[c], 0, 2^b - 1)
 * (qdiff/adaptive_rounding.py:49-58 with soft_targets False; the quantisers that
 * qdiff/utils.py:511-539 installs and :567 fills from the checkpoint).
 *   alpha     fp32, same layout as w; NULL = round to nearest (quant_layer.py:94)
 *   delta_in, zp_in  fp32 [2][cout] per segment like w_scale / w_zp; NULL = min/max rule
 * Outputs exactly as modiff_weight_pack (w_scale / w_zp receive the scales used), plus
 *   w_csum    int32 [2][cout] out, or NULL: sum over the segment's inputs of (q - zero_point),
 *             the factor modiff_asym_bias needs */
int modiff_weight_pack_rounded(const float* w, const float* alpha, const float* delta_in,
                               const float* zp_in, const modiff_conv_geom* g, int n_bits,
                               int with_sum_rows, int8_t* wcodes, float* w_scale, float* w_zp,
                               int32_t* w_corr, float* w_dq, int32_t* w_csum, void* stream);

/* Modulated activation quantiser: r = x - a_hat, dynamic symmetric per-tensor (or
 * per-segment with split) scale, round-half-even codes, a_hat += code * delta.
 * Replaces QuantModule.forward lines qdiff/quant_layer.py:325-336 together with
 * UniformAffineQuantizer.forward (:81-102) and init_quantization_scale (:191-214).
 *   x        fp32 NCHW [batch][cin][h][w]
 *   a_hat    fp32 NCHW, updated in place; NULL = plain (non-modulated) quantisation
 *   codes    int8 code planes (see top)
 *   x_scale  fp32 [2] out: delta of segment 0 / 1
 *   scratch  at least MODIFF_MODQ_SCRATCH_BYTES, zero-filled once by the caller;
 *            the kernels leave it zeroed again
 *   per_sample != 0: one scale per image (channel_wise activations, dim 0 = batch,
 *            qdiff/quant_layer.py:160-190); x_scale then has [batch] entries and
 *            split must be 0
 */
#define MODIFF_MODQ_SCRATCH_BYTES 64
int modiff_modq(const float* x, float* a_hat, int8_t* codes, float* x_scale,
                const modiff_conv_geom* g, int n_bits, int per_sample, void* scratch,
                void* stream);

/* Where a quantised layer's input comes from when it is not a materialised tensor: the channel
 * concat [x0 | x1], then either a per-(image, channel) scale / shift (GroupNorm with its
 * statistics and any bias folded in) or a plain per-(image, channel) bias, then optionally SiLU.  Lets the quantiser read the producer's output
 * directly instead of a normalised copy (ddim/models/diffusion.py:121-128, 345-349). */
typedef struct modiff_act_source {
  const float* x0;        /* NCHW [batch][c0][h*w] */
  const float* x1;        /* NCHW [batch][cin - c0][h*w], or NULL */
  int32_t c0;             /* channels of x0 (== cin when x1 is NULL) */
  int32_t silu;           /* apply x * sigmoid(x) last */
  const float* affine;    /* [batch][cin][2] scale, shift (modiff_groupnorm_silu), or NULL */
  const float* chan_bias; /* [batch][cin] added when affine is NULL, or NULL */
} modiff_act_source;

/* modiff_modq with the input described by a modiff_act_source (same arithmetic on the
 * transformed value; qdiff/quant_layer.py:325-336). */
int modiff_modq_src(const modiff_act_source* src, float* a_hat, int8_t* codes, float* x_scale,
                    const modiff_conv_geom* g, int n_bits, int per_sample, void* scratch,
                    void* stream);

/* modiff_modq for a linear layer whose input is GEGLU(h) = h[:, :n] * gelu(h[:, n:]) with the exact
 * (erf) gelu (the feed-forward's second linear layer, ldm/modules/attention.py:37-64) over
 * qdiff/quant_layer.py:325-336: both passes evaluate the gate on the fly with the arithmetic of
 * modiff_geglu (same bits), so the gated tensor is never written.  Symmetric per-tensor dynamic codes.
 *   h        fp32 [rows][2n], n a multiple of 16
 *   a_hat    fp32 [rows][n] in/out;  codes int8 [rows][n];  x_scale fp32 [1] out;  scratch as modiff_modq */
int modiff_modq_geglu(const float* h, int64_t rows, int n, float* a_hat, int8_t* codes, float* x_scale,
                      int n_bits, void* scratch, void* stream);

/* modiff_modq for a linear layer whose input is nn.LayerNorm(x) over the last dimension (the
 * transformer blocks' norm1 / norm2 / norm3 in front of to_q and the feed-forward projection,
 * ldm/modules/attention.py:229-241, qdiff/quant_block.py:249-256) over qdiff/quant_layer.py:325-336:
 * both passes normalise the row on the fly with the arithmetic of modiff_layernorm (same bits), so
 * the normalised tensor is never written.  Symmetric per-tensor dynamic codes, one scale.
 *   x        fp32 [rows][c], c a multiple of 16;  gamma, beta fp32 [c]
 *   a_hat    fp32 [rows][c] in/out;  codes int8 [rows][c];  x_scale fp32 [1] out
 *   scratch  as for modiff_modq (zero-filled once by the caller, left zeroed) */
int modiff_modq_ln(const float* x, const float* gamma, const float* beta, float eps, int64_t rows,
                   int c, float* a_hat, int8_t* codes, float* x_scale, int n_bits, void* scratch,
                   void* stream);

/* Two quantisers of ONE tensor in two sweeps instead of four: layer A reads
 * nonlinearity(norm(x)) (modiff_modq_gn), layer B reads x itself (modiff_modq_src) - a residual
 * block's first convolution and its shortcut convolution (qdiff/quant_block.py:279-283 and
 * 306-311 over qdiff/quant_layer.py:325-336).  x = [x0 | x1] as in modiff_act_source (no channel
 * bias).  Each layer keeps its own cache, scales (B may be split), scratch and code planes; the
 * results equal the two separate calls bit for bit.  Layer A must have split == 0; shapes the
 * paired kernels do not cover run the two calls one after the other. */
int modiff_modq_pair(const modiff_act_source* src, const float* gamma, const float* beta, int groups,
                     float eps, float* affine, float* a_hat_a, int8_t* codes_a, float* x_scale_a,
                     const modiff_conv_geom* g_a, int n_bits_a, void* scratch_a, float* a_hat_b,
                     int8_t* codes_b, float* x_scale_b, const modiff_conv_geom* g_b, int n_bits_b,
                     void* scratch_b, void* stream);

/* modiff_modq_src with ASYMMETRIC activation codes (the reference's quantiser without --a_sym:
 * sym=False in qdiff/quant_layer.py:191-214, 160-190, 94-102):
 *   delta = (max - min) / (2^b - 1), zero_point = round(-min / delta),
 *   q = clamp(round(r / delta) + zero_point, 0, 2^b - 1), dequantised (q - zero_point) * delta.
 * The code planes receive the CENTRED code q - zero_point, which is what the convolution
 * multiplies, so modiff_igemm_conv and the zero halo are used unchanged.  That range must fit
 * int8: n_bits <= 7, and a scale slot whose [-zero_point, 2^b - 1 - zero_point] leaves
 * [-128, 127] (a residual that does not straddle zero by far) sets bit 2 of
 * modiff_device_status.
 *   x_zp     fp32 out, same slots as x_scale: the zero points
 *   scratch  at least 16 + 8 * slots bytes (slots = 2, or batch with per_sample), zero-filled
 *            once by the caller
 * n_bits == 8 (the latent-diffusion drivers' default, W8A8 without --a_sym): q - zero_point spans
 * nine bits, so the planes receive q - 128 instead, i.e. every code is offset by
 * z' = zero_point - 128.  The caller then (1) writes z' into the planes' padding cells
 * (modiff_codes_fill_halo), so that padded positions still stand for the value 0, and (2) passes
 * modiff_igemm_conv the per-channel constant -z' * sum(q_w - zp_w) * delta_x * delta_w[c] as its
 * bias (modiff_asym_bias).  Not available with per_sample. */
int modiff_modq_asym(const modiff_act_source* src, float* a_hat, int8_t* codes, float* x_scale,
                     float* x_zp, const modiff_conv_geom* g, int n_bits, int per_sample,
                     void* scratch, void* stream);

/* Quantiser with MOVING-AVERAGE ranges (`--running_stat`: act_momentum_update,
 * qdiff/quant_layer.py:113-132, switched on by qdiff/quant_model.py:104-117 while activations are
 * calibrated): the range of this call's residual updates x_min / x_max,
 *   x_min = x_min * momentum + min(r) * (1 - momentum)   (same for x_max, fp32),
 * delta = max(|x_min|, |x_max|) / n_levels (symmetric) or (x_max - x_min) / (n_levels - 1) with
 * zero_point = round(-x_min / delta), floor 1e-8, and the call quantises with that scale.
 *   x_range    fp32 [8], caller-owned state: [0..3] moving (min, max) of segment 0 / 1,
 *              [4..7] work area
 *   init       non-zero on the quantiser's FIRST call: records min(r) / max(r) as the state and
 *              takes delta / zero_point from them by the per-tensor 'max' rule (:191-214)
 *   x_zp       fp32 [2] out (zero for symmetric); codes, a_hat, scratch as for modiff_modq_asym;
 *              8-bit asymmetric codes are stored as q - 128 (see modiff_modq_asym) */
int modiff_modq_running(const modiff_act_source* src, float* a_hat, int8_t* codes, float* x_scale,
                        float* x_zp, float* x_range, const modiff_conv_geom* g, int n_bits,
                        int symmetric, int init, double momentum, void* scratch, void* stream);

/* Companions of 8-bit asymmetric codes (planes hold q - 128, see modiff_modq_asym).
 * modiff_codes_fill_halo: every code-plane cell that is not an input pixel (the zero padding of
 * F.conv2d, qdiff/quant_layer.py:271) receives zero_point - 128 of its channel's segment, the
 * code of the value 0; call it after each quantiser run of a padded layer (the zero point moves
 * every step).  modiff_asym_bias:
 *   bias_out[c] = (bias_in ? bias_in[c] : 0)
 *                 - sum_seg (zero_point[seg] - 128) * w_csum[seg][c] * x_scale[seg] * w_scale[seg][c],
 * the constant that the offset codes add to channel c of the layer's output, with the sign that
 * removes it; pass it as `bias` to modiff_igemm_conv (honoured with accumulate too). */
int modiff_codes_fill_halo(int8_t* codes, const float* x_zp, const modiff_conv_geom* g,
                           void* stream);
int modiff_asym_bias(const float* x_scale, const float* x_zp, const float* w_scale,
                     const int32_t* w_csum, const float* bias_in, float* bias_out, int cout,
                     int nseg, void* stream);

/* modiff_igemm_conv (and, with residual / sum_out not NULL, modiff_igemm_conv_add) for OFFSET
 * activation codes, i.e. 8-bit asymmetric ones stored as q - 128 by modiff_modq_asym /
 * modiff_modq_fixed with the padding cells set by modiff_codes_fill_halo:
 *   out[c] = o_hat[c] + (acc[c] + w_corr[c] * rowsum - (zp[seg] - 128) * w_csum[seg][c])
 *            * x_scale[seg] * w_scale[seg][c]  (+ bias[c]),
 * the same value as qdiff/quant_layer.py:359-365 computes from (q - zp) * delta, with the offset
 * taken out of the integer accumulator (no separate bias vector, every kernel variant available).
 *   x_zp    fp32 [2]: zero point per scale segment;  w_csum int32 [2][cout] from
 *           modiff_weight_pack_rounded */
int modiff_igemm_conv_offset(const int8_t* codes, const int8_t* wcodes, int with_sum_rows,
                             const float* x_scale, const float* x_zp, const float* w_scale,
                             const int32_t* w_corr, const int32_t* w_csum, float* o_hat,
                             int accumulate, const float* bias, const modiff_conv_geom* g, int impl,
                             const float* residual, float* sum_out, void* stream);

/* modiff_modq_src / modiff_modq_asym with scales that are GIVEN instead of measured: the
 * reference's quantiser with dynamic=False (quant_mode 'qdiff'), whose delta / zero_point were
 * set by its first call or loaded from a calibrated checkpoint and are then only read
 * (qdiff/quant_layer.py:72-79 skipped, :94-102 applied; loaded by qdiff/utils.py:606-611).
 * One pass over the tensor: no maximum / range sweep, no scratch.
 *   x_scale  fp32 in, delta of segment 0 / 1 (or one per image with per_sample)
 *   x_zp     fp32 in, zero points in the same slots: asymmetric codes, stored centred
 *            (q - zero_point) for n_bits <= 7 (0 <= zero_point <= 128 is the caller's to
 *            check) and as q - 128 for n_bits == 8 (see modiff_modq_asym);
 *            NULL = symmetric codes clamp(round(r / delta), -2^(b-1), 2^(b-1) - 1) */
int modiff_modq_fixed(const modiff_act_source* src, float* a_hat, int8_t* codes,
                      const float* x_scale, const float* x_zp, const modiff_conv_geom* g,
                      int n_bits, int per_sample, void* stream);

/* modiff_modq_src for an input that is GroupNorm (+ FiLM) (+ SiLU) of [x0 | x1] (+ chan_bias):
 * the normalisation statistics and the residual maximum come from ONE sweep over the source.
 * Replaces `h = self.norm1(h); h = nonlinearity(h); h = self.conv1(h)` and its siblings
 * (qdiff/quant_block.py:279-306, 91-109, 331-335 with ddim/models/diffusion.py:32-33 and
 * ldm/modules/diffusionmodules/util.py:214-216) followed by qdiff/quant_layer.py:325-336.
 *   src     x0 / x1 / c0 / silu / chan_bias as in modiff_act_source; src->affine is ignored
 *   film    [batch][2*cin] FiLM scale | shift applied after the normalisation, or NULL
 *   gamma, beta  GroupNorm weight / bias [cin];  groups, eps as in nn.GroupNorm
 *   affine  OUT [batch][cin][2]: the per-(image, channel) scale / shift the encode pass used;
 *           a later modiff_modq_src on the same input may pass it as src->affine
 * Slabs of (cin / groups) * h * w <= 16384 floats (h * w / 4 a power of two) are kept in
 * registers; anything else runs the statistics pass of modiff_groupnorm_silu first. */
int modiff_modq_gn(const modiff_act_source* src, const float* film, const float* gamma,
                   const float* beta, int groups, float eps, float* affine, float* a_hat,
                   int8_t* codes, float* x_scale, const modiff_conv_geom* g, int n_bits,
                   int per_sample, void* scratch, void* stream);

/* modiff_modq_gn with asymmetric codes (modiff_modq_asym's arithmetic, per-tensor scales): the
 * GroupNorm statistics and the residual's minimum / maximum come from one sweep.  x_zp as in
 * modiff_modq_asym; n_bits == 8 stores q - 128 (see there). */
int modiff_modq_gn_asym(const modiff_act_source* src, const float* film, const float* gamma,
                        const float* beta, int groups, float eps, float* affine, float* a_hat,
                        int8_t* codes, float* x_scale, float* x_zp, const modiff_conv_geom* g,
                        int n_bits, void* scratch, void* stream);

/* modiff_modq for a layer whose input is the nearest-neighbour 2x upsample of x (the conv of
 * `Upsample`: ddim/models/diffusion.py:45-51, ldm/modules/diffusionmodules/openaimodel.py:105-115,
 * followed by qdiff/quant_layer.py:325-336).  The upsampled input, the cached input and so the
 * residual repeat every value in 2x2 blocks; the quantiser therefore runs on the SOURCE tensor and
 * writes each code to its four cells.  Same scale, codes and cache values as upsampling first.
 *   x, a_hat  fp32 [batch][cin][h/2][w/2]; a_hat is the cache AT SOURCE RESOLUTION, updated in place
 *   g         the convolution's geometry (h, w the upsampled size; stride 1, no split)
 *   codes, x_scale, scratch  as for modiff_modq (symmetric per-tensor scale)
 *   fixed_scale  non-zero: x_scale[0] is read, not measured (a non-dynamic quantiser, see
 *                modiff_modq_fixed); scratch may then be NULL */
int modiff_modq_up2(const float* x, float* a_hat, int8_t* codes, float* x_scale,
                    const modiff_conv_geom* g, int n_bits, int fixed_scale, void* scratch,
                    void* stream);

/* One launch for several modulated linear layers that read the same activation codes (every
 * residual block's projection of swish(temb): ddim/models/diffusion.py:121-123, 297-301;
 * ldm/modules/diffusionmodules/openaimodel.py:236-262): for each item
 *   o_hat[row][c] += (sum_k codes[row][k] * wcode[c][k] + w_corr[c] * sum_k codes[row][k])
 *                    * x_scale[0] * w_scale[c]                  (qdiff/quant_layer.py:345-365).
 *   codes     [rows][cin] int8, from modiff_modq of a linear geometry (cin a multiple of 16)
 *   items     DEVICE array, one per layer; wcodes / w_scale / w_corr as modiff_weight_pack
 *             wrote them for a (cin -> cout, 1x1) geometry, o_hat [rows][cout] fp32
 *   block_map DEVICE int32 [n_blocks][2]: (item index, first output channel) of each block;
 *             a block covers 16 output channels, so an item needs ceil(cout / 16) entries */
typedef struct modiff_linear_item {
  const int8_t* wcodes;
  const float* w_scale;
  const int32_t* w_corr;      /* NULL when the layer needs no correction */
  float* o_hat;
  int32_t cout;
  int32_t with_sum_rows;      /* layout flag given to modiff_weight_pack */
} modiff_linear_item;
int modiff_linear_group(const int8_t* codes, const float* x_scale, int rows, int cin,
                        const modiff_linear_item* items, const int32_t* block_map, int n_blocks,
                        void* stream);

/* Same quantiser as modiff_modq for callers that cannot hand over scratch memory.
 * This entry point has no counterpart in the reference; it exists for hosts that must not
 * allocate once they are running - for example a serving process whose device memory is
 * carved up at start-up and frozen, where a later cudaMalloc may fail against the fixed budget
 * and stalls every stream of the device while it runs - and that own no spare buffer to pass
 * as `scratch`.  The two reduction words and the per-image maxima live instead in an array
 * compiled into the library (file-scope __device__, 64 + 4 * MODIFF_MODQ_STATIC_MAX_BATCH
 * bytes, resident on every GPU that loads the library until the process exits).
 *   - x, a_hat, codes, x_scale, g, n_bits, per_sample: exactly as for modiff_modq; inputs and
 *     outputs are still the caller's.
 *   - nothing is allocated or freed, here or in any routine it calls.
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress
 *     with that device current) and caches it; make that first call before any stream capture.
 *     The cached address belongs to the device's primary context: after cudaDeviceReset (or any
 *     other teardown of that context) it is stale and this entry point must not be used again
 *     in the process.
 *   - per_sample != 0 needs one slot per image: batch > MODIFF_MODQ_STATIC_MAX_BATCH is
 *     rejected with MODIFF_ERR_INVALID (use modiff_modq with your own scratch instead).
 *   - all calls on a device share the one array and it keeps the previous call's contents; the
 *     part a call uses is cleared in stream order before its kernels run.  Calls that may
 *     overlap on the GPU (different streams) race on it: serialise them.
 */
#define MODIFF_MODQ_STATIC_MAX_BATCH 4096
int modiff_modq_static(const float* x, float* a_hat, int8_t* codes, float* x_scale,
                       const modiff_conv_geom* g, int n_bits, int per_sample, void* stream);

/* Int8 implicit-GEMM conv / linear with the modulation epilogue
 *   out = acc0 * (x_scale[0] * w_scale[0][c]) (+ acc1 * (x_scale[1] * w_scale[1][c]))
 *         (+ o_hat) (+ bias[c]);   acc = sum codes * (wcodes + w_corr)
 * Replaces F.conv2d / F.linear on fake-quantised operands plus "out = o_hat + out;
 * o_hat = out" (qdiff/quant_layer.py:357-365).
 *   o_hat    fp32 NCHW [batch][cout][ho][wo]; read when accumulate != 0, always written
 *   bias     fp32 [cout] or NULL
 *   w_corr   may be NULL when all corrections are zero
 *   impl     MODIFF_IMPL_*; AUTO picks tcgen05 when the geometry allows it
 *   acc_out  optional int32 [batch*ho*wo][cout] raw corrected accumulators of
 *            segment 0 (+ segment 1 at offset batch*ho*wo*cout) for parity tests
 */
int modiff_igemm_conv(const int8_t* codes, const int8_t* wcodes, int with_sum_rows,
                      const float* x_scale, const float* w_scale, const int32_t* w_corr,
                      float* o_hat, int accumulate, const float* bias,
                      const modiff_conv_geom* g, int per_sample, int impl,
                      int32_t* acc_out, void* stream);

/* modiff_igemm_conv (per-tensor scales, no bias) that also writes sum_out = residual + new output,
 * the `x + h` that ends a residual block (qdiff/quant_block.py:313; ddim/models/diffusion.py:128):
 * on the activation-reuse 3x3 kernel the sum is formed in the epilogue from the values it holds,
 * elsewhere modiff_add runs after the GEMM.  residual and sum_out are fp32 [batch][cout][ho*wo]. */
int modiff_igemm_conv_add(const int8_t* codes, const int8_t* wcodes, int with_sum_rows,
                          const float* x_scale, const float* w_scale, const int32_t* w_corr,
                          float* o_hat, int accumulate, const modiff_conv_geom* g, int impl,
                          const float* residual, float* sum_out, void* stream);

/* Receptive-field gather of activation codes for layers with very few input channels (the
 * 3-channel input conv, ddim/models/diffusion.py:321): out[m][c*kh*kw + tap], one row of
 * out_stride bytes per output pixel m (bytes past cin*kh*kw are left untouched: zero-fill the
 * buffer once).  The layer then runs as a 1x1 layer over out with the weights packed as
 * [cout][cin*kh*kw] (PyTorch's own weight order). */
int modiff_im2col_codes(const int8_t* codes, int8_t* out, const modiff_conv_geom* g, int out_stride,
                        void* stream);

/* First-step conv / linear: fp32 activations x dequantised weights + bias
 * (qdiff/quant_layer.py:326-327, 358-359; also the weight-only-quant and
 * unquantised paths :309-311, :364-365).
 *   x fp32 NCHW, w_kn fp32 [cin*kh*kw][cout] (K order cin,ky,kx), out fp32 NCHW. */
int modiff_conv_fp32(const float* x, const float* w_kn, const float* bias, float* out,
                     const modiff_conv_geom* g, void* stream);

/* ---- split-bf16 tensor-core GEMM (first sampling step and attention matmuls) -------------
 * fp32 values travel as two bf16 planes, hi = bf16(x) and lo = bf16(x - hi); the GEMM adds the
 * products hi*hi + hi*lo + lo*hi in fp32 (relative error ~1e-5). */

/* fp32 NCHW [batch][cin][h][w] -> bf16 [batch][2][stride^2][hp][wp][max(64, round_up(cin,8))] in the
 * code-plane geometry of g (zero halo: the caller zero-fills the buffer once). */
int64_t modiff_bf16_planes_bytes(const modiff_conv_geom* g);
int modiff_split_bf16(const float* x, uint16_t* planes, const modiff_conv_geom* g, void* stream);
/* x fp32 [nb][rows][len] -> bf16 [nb][2][rows_pad][len_pad], zero padded, no layout change. */
int modiff_split_bf16_rows(const float* x, uint16_t* out, int64_t nb, int rows, int len,
                           int rows_pad, int len_pad, void* stream);
/* Integer part (q - zp) of the fake-quantised weights, exact in bf16, as
 * [cout][kh*kw][max(64, round_up(cin,8))]; w_scale / w_zp come from modiff_weight_pack
 * (qdiff/quant_layer.py:345-351). */
int64_t modiff_weights_bf16_bytes(const modiff_conv_geom* g);
int modiff_weights_bf16(const float* w, const float* w_scale, const float* w_zp, uint16_t* out,
                        const modiff_conv_geom* g, int n_bits, void* stream);
/* The same with AdaRound hard rounding floor(w / delta) + (alpha >= 0) when alpha (layout of w)
 * is not NULL (qdiff/adaptive_rounding.py:49-58); scales as modiff_weight_pack_rounded left them. */
int modiff_weights_bf16_rounded(const float* w, const float* alpha, const float* w_scale,
                                const float* w_zp, uint16_t* out, const modiff_conv_geom* g,
                                int n_bits, void* stream);

typedef struct modiff_gemm_bf16_desc {
  const uint16_t* a;      /* activation planes (modiff_split_bf16 layout) */
  const uint16_t* b;      /* [images or 1][b_parts][cout][kh*kw][kb] bf16, K-major */
  const float* col_scale; /* [2][cout] per-column factor per segment, or NULL */
  const float* bias;      /* [cout] or NULL */
  float* out;             /* fp32 NCHW [batch][cout][ho*wo] */
  int32_t a_parts;        /* 2 = hi and lo planes are used, 1 = hi only */
  int32_t b_parts;        /* 1 (exact bf16 weights) or 2 */
  int32_t b_batched;      /* != 0: one B per image (attention), tiles never mix images */
  int32_t kb;             /* K stride per filter tap of B, elements (multiple of 8, >= cin) */
  float scale;            /* uniform factor */
  int32_t b_rows;         /* physical rows of B per part (>= cout rounded up to 16); 0 = cout */
} modiff_gemm_bf16_desc;

/* out = scale * col_scale[c] * (A conv B) + bias[c]  on tcgen05 kind::f16, fp32 accumulation.
 * First step: F.conv2d(input, weight_q, bias) with unquantised input
 * (qdiff/quant_layer.py:358-359).  Attention: the bmm's of qdiff/quant_block.py:351, 360.
 * MODIFF_ERR_UNSUPPORTED when the geometry is outside the tensor-core path. */
int modiff_gemm_bf16(const modiff_gemm_bf16_desc* desc, const modiff_conv_geom* g, void* stream);

/* Whole attention for small token counts (t, tk <= 64) on CUDA cores, fp32:
 * out[b,:,i] = sum_j softmax_j(q[b,:,i].k[b,:,j] * scale) v[b,:,j]; q, out [batch][c][t],
 * k, v [batch][c][tk] (qdiff/quant_block.py:344-360; the 4x4 middle block of the pixel UNet). */
int modiff_attention_small(const float* q, const float* k, const float* v, float* out, int batch,
                           int c, int t, int tk, float scale, void* stream);

/* Attention in one kernel: scores, online softmax and the weighted sum of v on the tensor cores,
 * scores and probabilities kept on chip (qdiff/quant_block.py:344-360, 191-203;
 * ldm/modules/diffusionmodules/openaimodel.py:384-406).  Operands are split-bf16 planes:
 *   q_planes [batch][2][t][cp]      from modiff_split_bf16 of q (tokens as pixels)
 *   k_planes [batch][2][tkp][cp]    from modiff_split_bf16 of k, keys padded with zero rows
 *   v_planes [batch][2][crow][tkp]  from modiff_split_bf16_rows of v (channel rows padded to crow)
 *   out      [batch][c][t] fp32:  out[b][:, i] = sum_j softmax_j(scale * q[b][:, i] . k[b][:, j]) v[b][:, j]
 * `batch` counts images x heads.  Needs tkp % 64 == 0, crow % 64 == 0, c <= crow <= 256,
 * 64 <= cp <= 256; otherwise MODIFF_ERR_UNSUPPORTED (use modiff_gemm_bf16 / modiff_softmax_split). */
int modiff_attention_tc(const uint16_t* q_planes, const uint16_t* k_planes, const uint16_t* v_planes,
                        float* out, int batch, int c, int t, int tk, int cp, int tkp, int crow,
                        float scale, void* stream);

/* Softmax over keys of s fp32 [batch][tk][tq] (the layout modiff_gemm_bf16 writes when the keys
 * are its output columns) -> probabilities as split bf16 planes p [batch][2][tq][tk_pad], zero
 * beyond tk (softmax of qdiff/quant_block.py:197, 353, ddim/models/diffusion.py:185). */
int modiff_softmax_split(const float* s, uint16_t* p, int batch, int tk, int tq, int tk_pad,
                         void* stream);

/* Stand-alone fake quantiser returning the dequantised tensor
 * (UniformAffineQuantizer.forward, qdiff/quant_layer.py:70-111; scale rules
 * :160-214).  Supports symmetric / asymmetric, per-tensor ('max') and per-dim-0
 * slice scales, always_zero.
 *   x, y     fp32, `slices` x `slice_len` elements (slices = 1 for per-tensor)
 *   delta,zp fp32 [slices] out (in when dynamic == 0 and inited != 0)
 *   scratch  at least 16 * slices + 64 bytes, zero-filled once by the caller
 */
int modiff_fake_quant(const float* x, float* y, int64_t slices, int64_t slice_len,
                      int n_bits, int symmetric, int always_zero, int channel_wise,
                      int recompute, float* delta, float* zp, void* scratch, void* stream);

/* GroupNorm (+ optional SiLU) over NCHW fp32: y = act(gn(x) * gamma + beta).
 * Replaces Normalize + nonlinearity (ddim/models/diffusion.py:27-33, 121-128, 356-357).
 *   x = [x0 | x1] channel concat (x0: c0 channels, x1: c - c0 channels; x1 NULL when c0 == c),
 *       which fuses the torch.cat of the up path (ddim/models/diffusion.py:345-349);
 *   chan_bias fp32 [batch][c] or NULL: added to x first (the "+ temb_proj(...)[:, :, None, None]"
 *       of ddim/models/diffusion.py:124);
 *   film fp32 [batch][2c] or NULL: the norm output becomes gn * (1 + film[:, :c]) + film[:, c:]
 *       (scale-shift norm, ldm/modules/diffusionmodules/openaimodel.py:267-271);
 *   y may be NULL and affine non-NULL to obtain only the normalisation as a per-(image,
 *   channel) scale / shift with the bias folded in:
 *   affine fp32 [batch][c][2] out (or NULL): gn(x + bias) = x * affine[..][0] + affine[..][1]. */
int modiff_groupnorm_silu(const float* x0, const float* x1, int c0, const float* chan_bias,
                          const float* film, float* y, float* affine, const float* gamma,
                          const float* beta, int batch, int c, int hw, int groups, float eps,
                          int silu, void* stream);

/* LayerNorm over the last dimension of x [rows][c] (nn.LayerNorm of
 * ldm/modules/attention.py:229-231). */
int modiff_layernorm(const float* x, float* y, const float* gamma, const float* beta, int64_t rows,
                     int c, float eps, void* stream);
/* GEGLU gate: y[rows][n] = x[:, :n] * gelu(x[:, n:]), x [rows][2n] (ldm/modules/attention.py:37-44). */
int modiff_geglu(const float* x, float* y, int64_t rows, int n, void* stream);
/* Batched transpose x [batch][r][c] -> y [batch][c][r] (the b c (h w) <-> b (h w) c rearranges of
 * ldm/modules/attention.py:276-280 and the head split of :176). */
int modiff_transpose(const float* x, float* y, int batch, int r, int c, void* stream);

/* y = x * sigmoid(x)  (ddim/models/diffusion.py:27-29). */
int modiff_silu(const float* x, float* y, int64_t n, void* stream);

/* out = a + b, where b is either a full tensor (b_per_channel == 0) or a
 * [batch][c] tensor broadcast over hw (the "+ temb_proj(...)[:, :, None, None]" of
 * ddim/models/diffusion.py:124). */
int modiff_add(const float* a, const float* b, float* out, int batch, int c, int hw,
               int b_per_channel, void* stream);

/* Nearest-neighbour 2x upsample NCHW (ddim/models/diffusion.py:47-48). */
int modiff_upsample2x(const float* x, float* y, int batch, int c, int h, int w, void* stream);

/* 2x2 average pooling NCHW (the down-sampling ResBlocks of the latent UNets,
 * ldm/modules/diffusionmodules/openaimodel.py:134-160 with use_conv=False). */
int modiff_avgpool2x(const float* x, float* y, int batch, int c, int h, int w, void* stream);

/* Channel concat of two NCHW tensors (ddim/models/diffusion.py:345-349). */
int modiff_concat_c(const float* a, int ca, const float* b, int cb, float* y, int batch,
                    int hw, void* stream);

/* Sinusoidal timestep embedding [batch][dim]: sin(t*freq) | cos(t*freq)
 * (ddim/models/diffusion.py:6-24).  freq[dim/2] = exp(-i*log(10000)/(dim/2-1)) is supplied by
 * the caller so that it carries the same bits as the host library's exp.  cos_first != 0 gives
 * cos | sin, the order of ldm/modules/diffusionmodules/util.py:151-171. */
int modiff_timestep_embedding(const float* t, const float* freq, float* emb, int batch, int dim,
                              int cos_first, void* stream);

/* One DDIM (generalised) update (ddim/functions/denoising.py:30-48):
 *   x0 = (x - e*s1) / s2;  x' = s3*x0 + c1*noise + c2*e
 * with the host scalars s1 = sqrt(1-at), s2 = sqrt(at), s3 = sqrt(at_next) and c1, c2
 * as the reference computes them in fp32.  noise may be NULL (eta = 0); x0 may be NULL. */
int modiff_ddim_step(const float* x, const float* e, const float* noise, float* x_next,
                     float* x0, int64_t n, float s1, float s2, float s3, float c1, float c2,
                     void* stream);

/* Classifier-free guidance: out = e_uncond + scale * (e_cond - e_uncond)
 * (ldm/models/diffusion/ddim.py:207-208). */
int modiff_cfg_combine(const float* e_uncond, const float* e_cond, float* out, int64_t n,
                       float scale, void* stream);

/* int4 nibble pack / unpack of int8 codes: element 2i -> low nibble, 2i+1 -> high
 * nibble, two's complement (qdiff/quant_layer_int4.py:341-346, 354-366). */
int modiff_pack_int4(const int8_t* codes, uint8_t* packed, int64_t n, void* stream);
int modiff_unpack_int4(const uint8_t* packed, int8_t* codes, int64_t n, int is_signed,
                       void* stream);

/* NCHW fp32 -> code planes without modulation state: codes = clamp(rne(x / delta))
 * with a given scale (layout transform used by tests and by static-scale callers). */
int modiff_quantize_static(const float* x, const float* delta, int8_t* codes,
                           const modiff_conv_geom* g, int n_bits, void* stream);

/* Packed 4-bit operands: W4 weight codes and A4 / A3 activation codes travel two per byte
 * through HBM and L2 and are expanded to int8 in shared memory, because the tensor cores have
 * no 4-bit integer MMA (the storage convention of qdiff/quant_layer_int4.py:341-366: element 2i
 * in the low nibble of byte i; the arithmetic is that of modiff_igemm_conv,
 * qdiff/quant_layer.py:345-365, and the results are bit-identical to it).
 *   modiff_pack_weights_int4  rows of modiff_weight_pack's wcodes (int8 q - zero_point, no
 *                             receptive-field-sum rows) -> unsigned nibbles q; `bad` (device
 *                             int, zero on entry) is set when a code does not fit 4 bits
 *   modiff_igemm_conv_packed4 codes4 = modiff_pack_int4 of the activation code planes
 *                             (two's-complement nibbles), wcodes4 from above, w_zp fp32 [cout];
 *                             3x3 stride-1 pad-1 layers, cin and cout multiples of 128, per-tensor
 *                             scales, no split; residual / sum_out optional as in
 *                             modiff_igemm_conv_add */
int modiff_pack_weights_int4(const int8_t* wcodes, const float* w_zp, uint8_t* packed,
                             int64_t rows, int64_t row_bytes, int* bad, void* stream);
int modiff_igemm_conv_packed4(const uint8_t* codes4, const uint8_t* wcodes4, const float* w_zp,
                              const float* x_scale, const float* w_scale, float* o_hat,
                              int accumulate, const modiff_conv_geom* g, const float* residual,
                              float* sum_out, void* stream);

/* Stand-alone fake quantisation of a weight tensor with learned (AdaRound) hard rounding
 * (qdiff/adaptive_rounding.py:49-61, soft_targets False), what AdaRoundQuantizer.forward returns:
 *   out = (clamp(floor(w / delta) + (alpha >= 0) + zero_point, 0, 2^b - 1) - zero_point) * delta
 *   w, alpha, out  fp32 [rows][row_len];  delta, zero_point fp32 [rows] (per_row != 0) or [1] */
int modiff_adaround_fake_quant(const float* w, const float* alpha, const float* delta,
                               const float* zero_point, float* out, int64_t rows, int64_t row_len,
                               int per_row, int n_bits, void* stream);

/* Integer attention (opt-in).  The reference constructs 8-bit quantisers for q, k, v and for the
 * softmax output on every attention block (qdiff/quant_block.py:120-121, 139-144, 223-235,
 * 331-335) but never applies them (:123-128, 146-148, 181-203, 338-366 stay in floating point);
 * these two entry points apply them.  Exact definition: oracle/attention_i8.py.
 *
 * modiff_attn_quantize: per-tensor symmetric dynamic codes of q, k, v (absmax over the whole
 * tensor, delta = absmax / (2^(n_bits-1) - 1), floor 1e-8) in the layouts the MMAs read.
 *   q, k, v       fp32, addressed as x[b*s0 + h*s1 + c*s2 + t*s3] with the four element strides
 *                 of strides_q (q) / strides_kv (k and v); channels or tokens contiguous
 *   q_codes       int8 [batch*heads][tq][dp], dp = c padded to 32, 64, 128 or 256, zero padded
 *   k_codes       int8 [batch*heads][tk][dp]
 *   v_codes       int8 [batch*heads][round_up(c,16)][round_up(tk,128)], zero padded
 *                 (sizes: modiff_attn_codes_bytes(batch*heads, c, tq, tk, which = 0 / 1 / 2))
 *   scales        fp32 [3] out: delta of q, k, v
 *   scratch       16 bytes, zero on entry, left zero
 * modiff_attention_i8: out = softmax(scale * q k^T) v from those codes: both products as int8
 * tensor-core MMAs with int32 accumulation, fp32 softmax with the exact row maximum, softmax
 * weights as unsigned 8-bit codes rne(255 * exp(s - max)), renormalised by their integer sum.
 *   out           fp32, addressed with the four element strides of strides_out like q */
int64_t modiff_attn_codes_bytes(int heads_total, int c, int tq, int tk, int which);
int modiff_attn_quantize(const float* q, const float* k, const float* v, int batch, int heads,
                         int c, int tq, int tk, const int64_t* strides_q,
                         const int64_t* strides_kv, int n_bits, int8_t* q_codes, int8_t* k_codes,
                         int8_t* v_codes, float* scales, void* scratch, void* stream);
int modiff_attention_i8(const int8_t* q_codes, const int8_t* k_codes, const int8_t* v_codes,
                        const float* scales, float* out, int batch, int heads, int c, int tq,
                        int tk, const int64_t* strides_out, float scale, void* stream);

/* Tensor-pipe probe of tcgen05.mma kind::i8 (measurement aid; no counterpart in the reference,
 * whose convolutions are PyTorch fp32, qdiff/quant_layer.py:345-365).  Every unit holds a
 * 128-row A tile per CTA and the B tile in shared memory (K = 128 bytes) and repeats the four
 * K = 32 steps `iters` times, accumulating in tensor memory; timing the call with CUDA events
 * over `units` = the SM count (mode 1) or half of it (mode 2) gives the int8 ceiling the GEMM
 * kernels' achieved TOPS are reported against: ops = units * iters * 4 * 2 * M * umma_n * 32.
 *   mode    1: cta_group::1 (M = 128 per unit); 2: cta_group::2, a two-CTA cluster (M = 256)
 *   a       int8 [units * M][128] row-major;  b  int8 [umma_n][128] row-major
 *   acc_out optional int32 [M][umma_n]: unit 0's accumulators = iters * a b^T (layout check)
 *   debug   optional int32 [4]: tensor-memory base address seen by each CTA of unit 0 */
int modiff_i8_mma_probe(int mode, int umma_n, int iters, int units, const int8_t* a,
                        const int8_t* b, int32_t* acc_out, int* debug, void* stream);

/* Failure-path probe (no counterpart in the reference): one thread waits, with the same bounded
 * wait the tensor-core kernels use, on a barrier that nothing ever signals.  After `limit_ns`
 * (at most 1e9) it gives up, sets bit 0 of the device status word and the kernel returns
 * normally; `gave_up` (device int, may be NULL) receives 1.  Lets a host check its handling of
 * modiff_device_status without a copy, a peer or tensor memory being involved. */
int modiff_wait_probe(int64_t limit_ns, int* gave_up, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MODIFF_B200_H_ */
