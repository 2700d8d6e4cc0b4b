"""QuantModule / UniformAffineQuantizer with the reference's Python surface, backed by the
sm_100a kernels of libmodiff_b200.so.

Mirrors qdiff/quant_layer.py of the reference: same constructor arguments, attributes, flag
setters (including the misspelt `set_modualtion`) and forward semantics
(qdiff/quant_layer.py:307-367).  What differs is where the arithmetic happens: activations
are quantised to real int8 codes by `modiff_modq`, multiplied on the tensor cores by
`modiff_igemm_conv`, and the cached output `o_hat` is updated in the GEMM epilogue.

There is no CPU path: CUDA float32 tensors only, anything else raises `ModiffError`.
"""
import ctypes as C
import logging
import os
from typing import Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib
from ._lib import ConvGeom, ModiffError

logger = logging.getLogger(__name__)


class StraightThrough(nn.Module):
    """Identity placeholder (qdiff/quant_layer.py:11-16)."""

    def __init__(self, channel_num: int = 1):
        super().__init__()

    def forward(self, input):
        return input


def round_ste(x: torch.Tensor):
    """Round half to even with a straight-through gradient (qdiff/quant_layer.py:19-23)."""
    return (x.round() - x).detach() + x


def _zeros(n, dtype, device):
    return torch.zeros(n, dtype=dtype, device=device)


def check_scale_method(scale_method, channel_wise):
    """Which `scale_method` strings mean the min / max rule this library implements.

    Channel-wise scales: the reference takes its per-channel search only for the literal string
    'mse:' (qdiff/quant_layer.py:137) and the min / max rule for every other value, so the
    `'mse'` the latent-diffusion drivers put into their weight parameters
    (scripts/sample_diffusion_ldm.py:549, scripts/txt2img.py:380) IS min / max there, and here.
    Per-tensor scales: any name containing 'max' (:192), except the '..scale' variants, which
    shrink the range by (n_bits + 2) / 8 (:199-201) and are not implemented; per-tensor 'mse' is
    a calibration-time search (:215-231) outside the sampling path."""
    if channel_wise:
        if scale_method == 'mse:':
            raise ModiffError("scale_method 'mse:' (the per-channel search) is a calibration-time "
                              "procedure and is not part of the accelerated sampling path")
        return
    if 'max' not in scale_method:
        raise ModiffError(f"per-tensor scale_method {scale_method!r} is a calibration-time search "
                          "and is not part of the accelerated sampling path")
    if 'scale' in scale_method:
        raise ModiffError(f"scale_method {scale_method!r} shrinks the range by (n_bits + 2) / 8 in "
                          "the reference; only the plain 'max' rule is implemented")


class UniformAffineQuantizer(nn.Module):
    """Uniform affine fake quantiser (qdiff/quant_layer.py:36-111, scale rules :134-235).

    `forward(x)` returns the dequantised tensor like the reference.  `delta` and `zero_point`
    are device tensors (no host synchronisation); inside a `QuantModule` the activation
    quantiser's `delta` is a view of the scale buffer the kernels update every step.
    """

    def __init__(self, n_bits: int = 8, symmetric: bool = False, channel_wise: bool = False,
                 scale_method: str = 'max', leaf_param: bool = False, always_zero: bool = False,
                 dynamic: bool = False):
        super().__init__()
        self.sym = symmetric
        self.n_bits = n_bits
        self.n_levels = 2 ** self.n_bits if not self.sym else 2 ** (self.n_bits - 1) - 1
        self.delta = None
        self.zero_point = None
        self.inited = False
        self.leaf_param = leaf_param
        self.channel_wise = channel_wise
        self.scale_method = scale_method
        self.running_stat = False
        self.always_zero = always_zero
        if self.leaf_param:
            self.x_min, self.x_max = None, None
        self.dynamic = dynamic
        self._scratch = None

    def forward(self, x: torch.Tensor):
        _lib.require_cuda(x, "quantiser input")
        check_scale_method(self.scale_method, self.channel_wise)
        if self.running_stat:
            raise ModiffError("running_stat (EMA ranges) is not part of the accelerated path")
        x = x.contiguous()
        slices = x.shape[0] if self.channel_wise else 1
        slice_len = x.numel() // slices
        recompute = (not self.inited) or self.dynamic
        dev = x.device
        if self.delta is None or not isinstance(self.delta, torch.Tensor) or \
                self.delta.numel() != slices or self.delta.device != dev:
            if not recompute:
                raise ModiffError("quantiser scale does not match the input")
            shape = [slices] + [1] * (x.dim() - 1) if self.channel_wise else []
            self.delta = torch.empty(shape, dtype=torch.float32, device=dev)
            self.zero_point = torch.empty(shape, dtype=torch.float32, device=dev)
        if self._scratch is None or self._scratch.device != dev or \
                self._scratch.numel() < 16 * slices + 64:
            self._scratch = _zeros(16 * slices + 64, torch.uint8, dev)
        y = torch.empty_like(x)
        _lib.call('modiff_fake_quant',
                  x.data_ptr(), y.data_ptr(), slices, slice_len, self.n_bits, int(self.sym),
                  int(self.always_zero), int(self.channel_wise), int(recompute),
                  self.delta.data_ptr(), self.zero_point.data_ptr(), self._scratch.data_ptr(),
                  _lib.stream_ptr())
        self.inited = True
        return y

    def bitwidth_refactor(self, refactored_bit: int):
        """qdiff/quant_layer.py:246-249 (note: resets n_levels to the asymmetric count)."""
        self.n_bits = refactored_bit
        self.n_levels = 2 ** self.n_bits

    def extra_repr(self):
        return (f'bit={self.n_bits}, scale_method={self.scale_method}, symmetric={self.sym}, '
                f'channel_wise={self.channel_wise}, leaf_param={self.leaf_param}')


class _Buffers:
    """Device buffers of one layer geometry."""

    def __init__(self, g: ConvGeom, device, per_sample):
        l = _lib.lib()
        self.g = g
        self.codes = _zeros(l.modiff_codes_bytes(C.byref(g)), torch.int8, device)
        self.x_scale = _zeros(max(2, g.batch if per_sample else 2), torch.float32, device)
        self.x_zp = _zeros(max(2, g.batch if per_sample else 2), torch.float32, device)
        self.scratch = _zeros(_lib.MODQ_SCRATCH_BYTES + 8 * g.batch, torch.uint8, device)
        self.ho, self.wo = _lib.out_hw(g)
        # non-dynamic quantisers: True once x_scale / x_zp hold the scale that stays
        # (set by the first quantised call or by QuantModule.load_act_scale)
        self.scale_set = False
        # moving (min, max) per segment of a quantiser with running statistics + work area
        self.x_range = _zeros(8, torch.float32, device)
        self.range_set = False


class QuantModule(nn.Module):
    """Quantised conv2d / conv1d(k=1) / linear with MoDiff modulation caches.

    Same contract as qdiff/quant_layer.py:257-392.  `forward(input, split=0)`:
      * first modulated call: `a_hat = input`, fp32 activations x fake-quantised weights + bias;
      * later calls: int8 codes of `input - a_hat` with a dynamic scale, int8 GEMM, `+ o_hat`.
    The returned tensor IS the cached `o_hat` buffer unless `alias_output` is False, so callers
    must not modify it in place.
    """

    alias_output = True
    # MODIFF_IGEMM_IMPL=1 forces the CUDA-core kernel, =2 the tensor-core kernel (debug aid)
    igemm_impl = int(os.environ.get("MODIFF_IGEMM_IMPL", _lib.IMPL_AUTO))
    # MODIFF_FUSE_NORM_STATS=0 runs the GroupNorm statistics as their own pass (debug aid; the
    # codes are the same either way)
    fuse_norm_stats = os.environ.get("MODIFF_FUSE_NORM_STATS", "1") != "0"

    def __init__(self, org_module: Union[nn.Conv2d, nn.Linear, nn.Conv1d],
                 weight_quant_params: dict = {}, act_quant_params: dict = {},
                 disable_act_quant: bool = False, act_quant_mode: str = 'qdiff',
                 modulate: bool = False):
        super().__init__()
        self.weight_quant_params = weight_quant_params
        self.act_quant_params = act_quant_params
        if isinstance(org_module, (nn.Conv2d, nn.Conv1d)):
            self.fwd_kwargs = dict(stride=org_module.stride, padding=org_module.padding,
                                   dilation=org_module.dilation, groups=org_module.groups)
            self.fwd_func = F.conv2d if isinstance(org_module, nn.Conv2d) else F.conv1d
        else:
            self.fwd_kwargs = dict()
            self.fwd_func = F.linear
        self.weight = org_module.weight
        self.org_weight = org_module.weight.data.clone()
        if org_module.bias is not None:
            self.bias = org_module.bias
            self.org_bias = org_module.bias.data.clone()
        else:
            self.bias = None
            self.org_bias = None
        self.use_weight_quant = False
        self.use_act_quant = False
        self.act_quant_mode = act_quant_mode
        self.disable_act_quant = disable_act_quant
        self.weight_quantizer = UniformAffineQuantizer(**self.weight_quant_params)
        self.act_quantizer = UniformAffineQuantizer(**self.act_quant_params)
        self.split = 0

        self.activation_function = StraightThrough()
        self.ignore_reconstruction = False
        self.extra_repr = org_module.extra_repr

        self.modulate = modulate
        self.a_hat = None
        self.o_hat = None

        # private device state
        self._a_store = None      # storage of a_hat / o_hat, kept across reset_cache() so that
        self._o_store = None      # device addresses stay valid for captured CUDA graphs
        # small linear layers that share this layer's residual codes (forward_shared) are
        # computed together with it in one launch; see _group_launch
        self._group_members = []
        self._group_table = None
        self._group_served = None   # (owner id, owner step) of the grouped launch that wrote o_hat
        self._group_step = 0
        self._geom_buffers = {}
        self._wpack = None
        self._org_kn = None
        self._loaded_act_scale = None   # (delta per segment, zero point per segment) to install
        self._a_hat_half = False        # a_hat held at the input resolution of an Upsample block
        self.implicit_pad = (0, 0, 0, 0)   # extra (left, right, top, bottom) zero padding

    # ------------------------------------------------------------------ geometry
    def _geom(self, input, split):
        k = self.fwd_kwargs
        w = self.weight
        if self.fwd_func is F.linear:
            if input.shape[-1] != w.shape[1]:
                raise ModiffError(f"linear expects {w.shape[1]} features, got {input.shape[-1]}")
            rows = input.numel() // w.shape[1]
            return ConvGeom(rows, w.shape[1], w.shape[0], 1, 1, 1, 1, 1, 0, 0, 0, 0, split)
        if any(d != 1 for d in k['dilation']) or k['groups'] != 1:
            raise ModiffError("dilated / grouped convolutions are not supported")
        if isinstance(k['padding'], str):
            raise ModiffError("string padding modes are not supported")
        if self.fwd_func is F.conv2d:
            if input.dim() != 4 or input.shape[1] != w.shape[1]:
                raise ModiffError(f"conv2d expects [B,{w.shape[1]},H,W], got {tuple(input.shape)}")
            sh, sw = k['stride']
            ph, pw = k['padding']
            b, _, h, ww = input.shape
            kh, kw = w.shape[2], w.shape[3]
        else:
            if input.dim() != 3 or input.shape[1] != w.shape[1]:
                raise ModiffError(f"conv1d expects [B,{w.shape[1]},T], got {tuple(input.shape)}")
            sh, sw = 1, k['stride'][0]
            ph, pw = 0, k['padding'][0]
            b, _, ww = input.shape
            h, kh, kw = 1, 1, w.shape[2]
            if kw == 1 and sw == 1 and pw == 0 and ww > 1 and (ww & (ww - 1)) == 0:
                # pointwise over T tokens: any (h, w) factorisation is the same computation;
                # a near-square one gives the tensor-core kernel its 128-pixel tiles
                fw = 1
                while fw * fw < ww:
                    fw *= 2
                h, ww = ww // fw, fw
        if sh != sw and not (self.fwd_func is F.conv1d and sw == 1):
            raise ModiffError("anisotropic strides are not supported")
        el, er, et, eb = self.implicit_pad
        return ConvGeom(b, w.shape[1], w.shape[0], h, ww, kh, kw, sw,
                        ph + et, pw + el, ph + eb, pw + er, split)

    def _get_buffers(self, g, device):
        key = g.key()
        buf = self._geom_buffers.get(key)
        if buf is None or buf.codes.device != device:
            per_sample = bool(self.act_quantizer.channel_wise)
            old = next(iter(self._geom_buffers.values()), None)
            buf = _Buffers(g, device, per_sample)
            _lib.bump_generation()
            if (old is not None and not per_sample and not self.act_quantizer.dynamic
                    and old.codes.device == device and bool(old.g.split) == bool(g.split)
                    and (old.scale_set or old.range_set)):
                # a non-dynamic quantiser's scale, zero point and moving range belong to the
                # quantiser, not to an input shape (qdiff/quant_layer.py:72-79): they carry over
                # when the layer meets another batch size or resolution
                buf.x_scale.copy_(old.x_scale[:buf.x_scale.numel()])
                buf.x_zp.copy_(old.x_zp[:buf.x_zp.numel()])
                buf.x_range.copy_(old.x_range)
                buf.scale_set, buf.range_set = old.scale_set, old.range_set
            carried = buf.scale_set
            self._geom_buffers = {key: buf}   # one live geometry per layer
            n = g.batch if per_sample else 1
            self.act_quantizer.delta = buf.x_scale[0:n].view([n] + [1] * 3) if per_sample \
                else buf.x_scale[0:1].view([])
            asym = not self.act_quantizer.sym
            self.act_quantizer.zero_point = 0 if not asym else (
                buf.x_zp[0:n].view([n] + [1] * 3) if per_sample else buf.x_zp[0:1].view([]))
            self.act_quantizer.inited = True
            if g.split:
                self.act_quantizer_0.delta = buf.x_scale[1:2].view([])
                self.act_quantizer_0.zero_point = 0 if not asym else buf.x_zp[1:2].view([])
                self.act_quantizer_0.inited = True
            if not self.act_quantizer.dynamic and not carried:
                self.act_quantizer.inited = False      # until the first quantised call
                if g.split:
                    self.act_quantizer_0.inited = False
            if carried and buf.range_set:
                aq = self.act_quantizer
                aq.x_min, aq.x_max = buf.x_range[0:1].view([]), buf.x_range[1:2].view([])
                if g.split:
                    q0 = self.act_quantizer_0
                    q0.x_min, q0.x_max = buf.x_range[2:3].view([]), buf.x_range[3:4].view([])
            self._install_act_scale(buf)
        return buf

    def load_act_scale(self, delta, zero_point=None):
        """Install calibrated activation scales for a non-dynamic quantiser (what loading a
        checkpoint does to `act_quantizer.delta` / `.zero_point` in qdiff/utils.py:606-611).
        `delta` / `zero_point`: one value, or two with split (segment 0, segment 1)."""
        d = [float(v) for v in (delta if isinstance(delta, (list, tuple)) else [delta])]
        z = zero_point if zero_point is not None else [0.0] * len(d)
        z = [float(v) for v in (z if isinstance(z, (list, tuple)) else [z])]
        if len(d) != len(z) or len(d) not in (1, 2):
            raise ModiffError("load_act_scale expects one scale, or two for a split layer")
        aq = self.act_quantizer
        if aq.channel_wise:
            raise ModiffError("calibrated scales are per tensor; per-sample quantisers are dynamic")
        for v in z:
            if v != int(v):
                raise ModiffError(f"zero point {v} is not an integer")
            if aq.sym and v != 0:
                raise ModiffError("a symmetric quantiser has zero point 0")
            if not aq.sym and not 0 <= v <= (255 if aq.n_bits == 8 else 128):
                raise ModiffError(f"zero point {v} of a {aq.n_bits}-bit quantiser cannot be stored "
                                  "in the int8 code planes")
        if any(not v > 0 for v in d):
            raise ModiffError("activation scales must be positive")
        self._loaded_act_scale = (d, z)
        for buf in self._geom_buffers.values():
            self._install_act_scale(buf)

    def _install_act_scale(self, buf):
        if self._loaded_act_scale is None:
            return
        d, z = self._loaded_act_scale
        segs = 2 if buf.g.split else 1
        if len(d) != segs:
            raise ModiffError(f"{len(d)} calibrated scale(s) for a layer with {segs} segment(s)")
        buf.x_scale[:segs].copy_(torch.tensor(d, dtype=torch.float32), non_blocking=False)
        buf.x_zp[:segs].copy_(torch.tensor(z, dtype=torch.float32), non_blocking=False)
        buf.scale_set = True
        self.act_quantizer.inited = True
        if segs == 2:
            self.act_quantizer_0.inited = True

    # ------------------------------------------------------------------ weights
    def _pack_weights(self, g):
        """Quantise + pack the weights once per (weight version, bits, split)."""
        w = self.weight
        n_bits = self.weight_quantizer.n_bits
        wq = self.weight_quantizer
        learned = hasattr(wq, 'alpha')        # AdaRound quantiser from a calibrated checkpoint
        key = (w.data_ptr(), w._version, n_bits, g.split, str(w.device),
               (wq.alpha.data_ptr(), wq.alpha._version) if learned else None)
        if self._wpack is not None and self._wpack['key'] == key:
            return self._wpack
        if wq.sym or not wq.channel_wise:
            raise ModiffError("the accelerated path expects per-output-channel asymmetric "
                              "weight quantisation (the reference's wq_params)")
        check_scale_method(wq.scale_method, True)
        _lib.require_cuda(w, "weight")
        l = _lib.lib()
        dev = w.device
        wc = w.detach().contiguous()
        gp = g.copy(batch=1)
        taps = g.kh * g.kw
        pack = None
        alpha = delta_in = zp_in = None
        if learned:
            if wq.round_mode != 'learned_hard_sigmoid' or wq.soft_targets:
                raise ModiffError("only hard AdaRound targets are packed (inference)")
            qs = [wq] + ([self.weight_quantizer_0] if g.split else [])
            if any(not hasattr(q, 'alpha') for q in qs):
                raise ModiffError("split layer with one AdaRound and one uniform weight quantiser")
            alpha = torch.cat([q.alpha.detach().to(dev) for q in qs], dim=1).contiguous() \
                if g.split else wq.alpha.detach().to(dev).contiguous()
            if tuple(alpha.shape) != tuple(w.shape):
                raise ModiffError(f"AdaRound alpha {tuple(alpha.shape)} does not match the weight "
                                  f"{tuple(w.shape)}")
            delta_in = _zeros(2 * g.cout, torch.float32, dev)
            zp_in = _zeros(2 * g.cout, torch.float32, dev)
            for i, q in enumerate(qs):
                delta_in[i * g.cout:(i + 1) * g.cout] = q.delta.to(dev).reshape(-1)
                zp_in[i * g.cout:(i + 1) * g.cout] = torch.as_tensor(
                    q.zero_point, dtype=torch.float32, device=dev).reshape(-1)
        for with_sum in ((1,) if n_bits >= 8 else (0, 1)):
            wcodes = torch.empty(l.modiff_wcodes_bytes(C.byref(gp), with_sum), dtype=torch.int8,
                                 device=dev)
            w_scale = _zeros(2 * g.cout, torch.float32, dev)
            w_zp = _zeros(2 * g.cout, torch.float32, dev)
            w_corr = _zeros(2 * g.cout, torch.int32, dev)
            w_dq = torch.empty(g.cin * taps * g.cout, dtype=torch.float32, device=dev)
            w_csum = _zeros(2 * g.cout, torch.int32, dev)
            _lib.call('modiff_weight_pack_rounded', wc.data_ptr(), _lib.ptr(alpha),
                      _lib.ptr(delta_in), _lib.ptr(zp_in), C.byref(gp), n_bits, with_sum,
                      wcodes.data_ptr(), w_scale.data_ptr(), w_zp.data_ptr(),
                      w_corr.data_ptr(), w_dq.data_ptr(), w_csum.data_ptr(), _lib.stream_ptr())
            need_corr = bool(w_corr.any().item())      # one-time host read at pack time
            pack = dict(key=key, wcodes=wcodes, w_scale=w_scale, w_zp=w_zp,
                        w_corr=w_corr if need_corr else None, w_dq=w_dq, with_sum=with_sum,
                        alpha=alpha, w_csum=w_csum)
            if not need_corr or with_sum:
                break
        self._wpack = pack
        _lib.bump_generation()
        if learned:
            return pack                     # the AdaRound quantisers keep their own tensors
        shape = [g.cout] + [1] * (w.dim() - 1)
        self.weight_quantizer.delta = pack['w_scale'][:g.cout].view(shape)
        self.weight_quantizer.zero_point = pack['w_zp'][:g.cout].view(shape)
        self.weight_quantizer.inited = True
        if g.split:
            self.weight_quantizer_0.delta = pack['w_scale'][g.cout:].view(shape)
            self.weight_quantizer_0.zero_point = pack['w_zp'][g.cout:].view(shape)
            self.weight_quantizer_0.inited = True
        self._wpack = pack
        return pack

    def _org_weights_kn(self):
        """Unquantised weights as [cin*kh*kw][cout] for the fp32 kernel."""
        if self.org_weight.device != self.weight.device:   # plain attribute: .to() skips it
            self.org_weight = self.org_weight.to(self.weight.device)
            if self.org_bias is not None:
                self.org_bias = self.org_bias.to(self.weight.device)
        w = self.org_weight
        key = (w.data_ptr(), w._version)
        if self._org_kn is None or self._org_kn[0] != key:
            self._org_kn = (key, w.reshape(w.shape[0], -1).t().contiguous())
        return self._org_kn[1]

    def packed_weights(self, split=0):
        """Weight codes / scales as the kernels consume them (test and tooling hook)."""
        kh, kw = (self.weight.shape[2:] if self.weight.dim() == 4 else
                  (1, self.weight.shape[2]) if self.weight.dim() == 3 else (1, 1))
        g = ConvGeom(1, self.weight.shape[1], self.weight.shape[0], kh, kw, kh, kw,
                     1, 0, 0, 0, 0, split)
        return self._pack_weights(g)

    # ------------------------------------------------------------------ kernels
    def _conv_fp32(self, x, w_kn, bias, g, out):
        _lib.call('modiff_conv_fp32', x.data_ptr(), w_kn.data_ptr(), _lib.ptr(bias),
                  out.data_ptr(), C.byref(g), _lib.stream_ptr(),
                  nbytes=4 * (x.numel() + out.numel() + w_kn.numel()))

    @staticmethod
    def _bf16_ok(g, ho_wo):
        """Geometries the split-bf16 tensor-core GEMM covers (mirrors modiff_gemm_bf16)."""
        def pow2(v):
            return v > 0 and (v & (v - 1)) == 0
        ho, wo = ho_wo
        return (g.cin >= 64 and g.cin % 8 == 0 and g.cout >= 16
                and (g.cout >= 128 or g.cout % 16 == 0) and pow2(ho) and pow2(wo)
                and wo <= 128 and g.split % 64 == 0 and g.kh <= 7 and g.kw <= 7)

    def _conv_first_step(self, x, pack, bias, g, out, ho_wo):
        """Unquantised activations x fake-quantised weights + bias (quant_layer.py:358-359) on
        the tensor cores: activations split into two bf16 planes, integer weights exact in bf16,
        delta_w[c] and the bias applied in the epilogue."""
        if os.environ.get("MODIFF_FIRST_STEP_FP32", "0") == "1" or not self._bf16_ok(g, ho_wo):
            return self._conv_fp32(x, pack['w_dq'], bias, g, out)
        l = _lib.lib()
        dev = x.device
        if pack.get('w_bf16') is None:
            gp = g.copy(batch=1)
            wb = torch.empty(l.modiff_weights_bf16_bytes(C.byref(gp)) // 2, dtype=torch.int16,
                             device=dev)
            wc = self.weight.detach().contiguous()
            _lib.call('modiff_weights_bf16_rounded', wc.data_ptr(), _lib.ptr(pack.get('alpha')),
                      pack['w_scale'].data_ptr(), pack['w_zp'].data_ptr(), wb.data_ptr(),
                      C.byref(gp), self.weight_quantizer.n_bits, _lib.stream_ptr())
            pack['w_bf16'] = wb
        planes = torch.zeros(l.modiff_bf16_planes_bytes(C.byref(g)) // 2, dtype=torch.int16,
                             device=dev)
        _lib.call('modiff_split_bf16', x.data_ptr(), planes.data_ptr(), C.byref(g),
                  _lib.stream_ptr())
        kb = max(64, -(-g.cin // 8) * 8)
        desc = _lib.GemmBf16Desc(planes.data_ptr(), pack['w_bf16'].data_ptr(),
                                 pack['w_scale'].data_ptr(), _lib.ptr(bias), out.data_ptr(),
                                 2, 1, 0, kb, 1.0, 0)
        _lib.call('modiff_gemm_bf16', C.byref(desc), C.byref(g), _lib.stream_ptr(),
                  nbytes=4 * (x.numel() + out.numel()), tag=g.key())

    def _modq(self, x, a_hat, buf, g, src=None):
        aq = self.act_quantizer
        if src is not None and src.layernorm is not None:
            # LayerNorm in front of a linear layer: normalised inside the quantiser's two passes
            ln = src.layernorm
            if (aq.dynamic and aq.sym and not aq.channel_wise and not aq.running_stat
                    and a_hat is not None and g.split == 0 and g.h * g.w == 1 and g.kh * g.kw == 1
                    and g.cin % 16 == 0 and g.cin <= 1280 and ln.elementwise_affine):
                _lib.call('modiff_modq_ln', src.x0.data_ptr(), ln.weight.data_ptr(),
                          ln.bias.data_ptr(), float(ln.eps), g.batch, g.cin, a_hat.data_ptr(),
                          buf.codes.data_ptr(), buf.x_scale.data_ptr(), aq.n_bits,
                          buf.scratch.data_ptr(), _lib.stream_ptr(), nbytes=13 * src.numel(),
                          tag=g.key())
                return
            x, src = src.materialize(), None
        if src is not None and src.geglu:
            # GEGLU in front of the feed-forward's second linear layer: gated inside both passes
            if (aq.dynamic and aq.sym and not aq.channel_wise and not aq.running_stat
                    and a_hat is not None and g.split == 0 and g.h * g.w == 1 and g.kh * g.kw == 1
                    and g.cin % 16 == 0):
                _lib.call('modiff_modq_geglu', src.x0.data_ptr(), g.batch, g.cin, a_hat.data_ptr(),
                          buf.codes.data_ptr(), buf.x_scale.data_ptr(), aq.n_bits,
                          buf.scratch.data_ptr(), _lib.stream_ptr(), nbytes=13 * src.numel(),
                          tag=g.key())
                return
            x, src = src.materialize(), None
        first_static = (not aq.dynamic) and not buf.scale_set
        if aq.running_stat or (first_static and aq.leaf_param and not aq.channel_wise):
            # moving-average ranges (act_momentum_update, quant_layer.py:113-132), and the first
            # call of a non-dynamic leaf quantiser, which records the range they start from
            if aq.running_stat and (aq.dynamic or aq.channel_wise or not aq.leaf_param):
                raise ModiffError("running_stat needs a non-dynamic per-tensor leaf_param quantiser "
                                  "(quant_mode 'qdiff'), as in the reference's calibration flow")
            if aq.running_stat and not (buf.scale_set and buf.range_set):
                raise ModiffError("running_stat before the quantiser's first call (or after loading "
                                  "scales without ranges): x_min / x_max are not initialised")
            if src is not None:
                st = src.struct()
            else:
                st = _lib.ActSourceStruct(x.data_ptr(), None, g.cin, 0, None, None)
            n = src.numel() if src is not None else x.numel()
            _lib.call('modiff_modq_running', C.byref(st), _lib.ptr(a_hat), buf.codes.data_ptr(),
                      buf.x_scale.data_ptr(), buf.x_zp.data_ptr(), buf.x_range.data_ptr(),
                      C.byref(g), aq.n_bits, int(aq.sym), int(first_static), 0.95,
                      buf.scratch.data_ptr(), _lib.stream_ptr(),
                      nbytes=(13 if a_hat is not None else 5) * n, tag=g.key())
            buf.scale_set = buf.range_set = True
            aq.inited = True
            aq.x_min, aq.x_max = buf.x_range[0:1].view([]), buf.x_range[1:2].view([])
            if g.split:
                q0 = self.act_quantizer_0
                q0.inited = True
                q0.x_min, q0.x_max = buf.x_range[2:3].view([]), buf.x_range[3:4].view([])
            self._offset_codes_halo(buf, g)
            return
        if not aq.dynamic and buf.scale_set:
            # scale fixed by the first quantised call or a checkpoint: one encode pass
            if aq.channel_wise:
                raise ModiffError("non-dynamic per-sample activation scales are not supported")
            if src is not None:
                st = src.struct()
            else:
                st = _lib.ActSourceStruct(x.data_ptr(), None, g.cin, 0, None, None)
            n = src.numel() if src is not None else x.numel()
            _lib.call('modiff_modq_fixed', C.byref(st), _lib.ptr(a_hat), buf.codes.data_ptr(),
                      buf.x_scale.data_ptr(), None if aq.sym else buf.x_zp.data_ptr(),
                      C.byref(g), aq.n_bits, 0, _lib.stream_ptr(),
                      nbytes=(13 if a_hat is not None else 5) * n, tag=g.key())
            self._offset_codes_halo(buf, g)
            return
        if not aq.dynamic:
            # first quantised call of a non-dynamic quantiser measures its scale like a dynamic
            # one and keeps it (quant_layer.py:72-79)
            buf.scale_set = True
            aq.inited = True
            if g.split:
                self.act_quantizer_0.inited = True
        if not aq.sym:
            # asymmetric codes (the reference's default without --a_sym): centred codes
            # q - zero_point in the same int8 planes up to 7 bits, q - 128 at 8 bits
            if aq.n_bits > 7 and aq.channel_wise:
                raise ModiffError("8-bit asymmetric activation codes are stored offset by one zero "
                                  "point per tensor; per-sample (--act_tensor) scales need --a_sym "
                                  "or at most 7 bits")
            if src is not None and src.pending_norm() and self.fuse_norm_stats and \
                    not aq.channel_wise:
                nrm = src.norm
                raw, table = src.raw_struct()
                _lib.call('modiff_modq_gn_asym', C.byref(raw), _lib.ptr(src.film),
                          nrm.weight.data_ptr(), nrm.bias.data_ptr(), nrm.num_groups,
                          float(nrm.eps), table.data_ptr(), _lib.ptr(a_hat), buf.codes.data_ptr(),
                          buf.x_scale.data_ptr(), buf.x_zp.data_ptr(), C.byref(g), aq.n_bits,
                          buf.scratch.data_ptr(), _lib.stream_ptr(), nbytes=13 * src.numel(),
                          tag=g.key())
                self._offset_codes_halo(buf, g)
                return
            if src is not None:
                st = src.struct()
            else:
                st = _lib.ActSourceStruct(x.data_ptr(), None, g.cin, 0, None, None)
            n = src.numel() if src is not None else x.numel()
            _lib.call('modiff_modq_asym', C.byref(st), _lib.ptr(a_hat), buf.codes.data_ptr(),
                      buf.x_scale.data_ptr(), buf.x_zp.data_ptr(), C.byref(g), aq.n_bits,
                      int(aq.channel_wise), buf.scratch.data_ptr(), _lib.stream_ptr(),
                      nbytes=(13 if a_hat is not None else 5) * n, tag=g.key())
            self._offset_codes_halo(buf, g)
            return
        if src is not None and src.pending_norm() and self.fuse_norm_stats:
            n = src.norm
            raw, table = src.raw_struct()
            _lib.call('modiff_modq_gn', C.byref(raw), _lib.ptr(src.film), n.weight.data_ptr(),
                      n.bias.data_ptr(), n.num_groups, float(n.eps), table.data_ptr(),
                      _lib.ptr(a_hat), buf.codes.data_ptr(), buf.x_scale.data_ptr(), C.byref(g),
                      aq.n_bits, int(aq.channel_wise), buf.scratch.data_ptr(), _lib.stream_ptr(),
                      nbytes=13 * src.numel(), tag=g.key())
            return
        if src is not None:
            _lib.call('modiff_modq_src', C.byref(src.struct()), _lib.ptr(a_hat),
                      buf.codes.data_ptr(), buf.x_scale.data_ptr(), C.byref(g), aq.n_bits,
                      int(aq.channel_wise), buf.scratch.data_ptr(), _lib.stream_ptr(),
                      nbytes=13 * src.numel(), tag=g.key())
            return
        # algorithmic bytes: x 4 + a_hat read/write 8 + code 1 per element
        _lib.call('modiff_modq', x.data_ptr(), _lib.ptr(a_hat), buf.codes.data_ptr(),
                  buf.x_scale.data_ptr(), C.byref(g), aq.n_bits, int(aq.channel_wise),
                  buf.scratch.data_ptr(), _lib.stream_ptr(),
                  nbytes=(13 if a_hat is not None else 5) * x.numel(), tag=g.key())

    def _offset_codes(self):
        """8-bit asymmetric activation codes: the planes hold q - 128 (see modiff_modq_asym)."""
        aq = self.act_quantizer
        return (not aq.sym) and aq.n_bits == 8

    def _offset_codes_halo(self, buf, g):
        if self._offset_codes() and (g.pad_t or g.pad_b or g.pad_l or g.pad_r):
            _lib.call('modiff_codes_fill_halo', buf.codes.data_ptr(), buf.x_zp.data_ptr(),
                      C.byref(g), _lib.stream_ptr())

    def _use_im2col(self, g, buf):
        """Layers with very few input channels (the 3-channel input conv) run on the tensor
        cores as a dense K = cin*kh*kw GEMM over gathered codes."""
        def pow2(v):
            return v > 0 and (v & (v - 1)) == 0
        return (g.cin < 16 and g.cin * g.kh * g.kw <= 128 and g.split == 0 and pow2(buf.ho)
                and pow2(buf.wo) and buf.wo <= 128 and self.igemm_impl != _lib.IMPL_SIMT)

    def _igemm_im2col(self, buf, pack, o_hat, accumulate, bias, g, acc_out):
        l = _lib.lib()
        aq = self.act_quantizer
        taps = g.kh * g.kw
        if getattr(buf, 'im2col', None) is None:
            buf.im2col = _zeros(g.batch * buf.ho * buf.wo * 128, torch.int8, buf.codes.device)
        if pack.get('wcodes_im2col') is None:
            # same weights read as [cout][cin*kh*kw] (PyTorch's own order): identical scales
            gp = ConvGeom(1, g.cin * taps, g.cout, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0)
            dev = buf.codes.device
            wcodes = torch.empty(l.modiff_wcodes_bytes(C.byref(gp), pack['with_sum']),
                                 dtype=torch.int8, device=dev)
            tmp = [_zeros(2 * g.cout, dt, dev) for dt in (torch.float32, torch.float32, torch.int32)]
            wc = self.weight.detach().contiguous()
            # the layer's own scales (and learned rounding, if any) so both layouts hold one set
            # of integer weights
            _lib.call('modiff_weight_pack_rounded', wc.data_ptr(), _lib.ptr(pack.get('alpha')),
                      pack['w_scale'].data_ptr(), pack['w_zp'].data_ptr(), C.byref(gp),
                      self.weight_quantizer.n_bits, pack['with_sum'], wcodes.data_ptr(),
                      tmp[0].data_ptr(), tmp[1].data_ptr(), tmp[2].data_ptr(), None, None,
                      _lib.stream_ptr())
            pack['wcodes_im2col'] = wcodes
        _lib.call('modiff_im2col_codes', buf.codes.data_ptr(), buf.im2col.data_ptr(), C.byref(g),
                  128, _lib.stream_ptr())
        g2 = ConvGeom(g.batch, 128, g.cout, buf.ho, buf.wo, 1, 1, 1, 0, 0, 0, 0, 0)
        if self._offset_codes():
            return self._igemm_offset(buf.im2col, pack['wcodes_im2col'], buf, pack, o_hat,
                                      accumulate, bias, g2, None, None)
        _lib.call('modiff_igemm_conv',
                  buf.im2col.data_ptr(), pack['wcodes_im2col'].data_ptr(), pack['with_sum'],
                  buf.x_scale.data_ptr(), pack['w_scale'].data_ptr(), _lib.ptr(pack['w_corr']),
                  o_hat.data_ptr(), int(accumulate), _lib.ptr(bias), C.byref(g2),
                  int(aq.channel_wise), self.igemm_impl, _lib.ptr(acc_out), _lib.stream_ptr(),
                  nbytes=(8 if accumulate else 4) * o_hat.numel(), tag=g.key())

    def _igemm_offset(self, codes, wcodes, buf, pack, o_hat, accumulate, bias, g, residual, out):
        """GEMM over offset (8-bit asymmetric, q - 128) codes; `buf` holds their scale and zero
        point, `residual` / `out` optionally the block's residual sum."""
        n_out = o_hat.numel()
        _lib.call('modiff_igemm_conv_offset', codes.data_ptr(), wcodes.data_ptr(), pack['with_sum'],
                  buf.x_scale.data_ptr(), buf.x_zp.data_ptr(), pack['w_scale'].data_ptr(),
                  _lib.ptr(pack['w_corr']), pack['w_csum'].data_ptr(), o_hat.data_ptr(),
                  int(accumulate), _lib.ptr(bias), C.byref(g), self.igemm_impl, _lib.ptr(residual),
                  _lib.ptr(out), _lib.stream_ptr(),
                  nbytes=((8 if accumulate else 4) + (8 if residual is not None else 0)) * n_out
                  + g.batch * g.cin * g.h * g.w + g.cout * g.cin * g.kh * g.kw, tag=g.key())

    # MODIFF_PACKED_INT4=1 (or QuantModule.packed_int4 = True): W4 weight codes and A4 / A3
    # activation codes of the layers the activation-reuse kernel covers travel two per byte and
    # are expanded in shared memory (modiff_igemm_conv_packed4).  Same bits as the byte-per-code
    # path; the activation planes are repacked by a separate kernel, so this path demonstrates
    # the operand format rather than a speed-up and is off by default.
    packed_int4 = os.environ.get("MODIFF_PACKED_INT4", "0") == "1"

    def _packed4_ok(self, g, bias, acc_out):
        aq = self.act_quantizer
        return (self.packed_int4 and self.weight_quantizer.n_bits <= 4 and aq.n_bits <= 4 and aq.sym
                and not aq.channel_wise and bias is None and acc_out is None and g.split == 0
                and g.kh == 3 and g.kw == 3 and g.stride == 1
                and (g.pad_t, g.pad_l, g.pad_b, g.pad_r) == (1, 1, 1, 1)
                and g.cin % 128 == 0 and g.cout % 128 == 0 and g.w in (16, 32, 64)
                and g.h & (g.h - 1) == 0 and g.h * g.w >= 128 and g.h >= 128 // g.w)

    def _igemm_packed4(self, buf, pack, o_hat, accumulate, g, residual=None, out=None):
        from .ops import pack_int4
        if pack.get('wcodes4') is None:
            rows, row_bytes = g.cout, pack['wcodes'].numel() // g.cout
            w4 = torch.empty(rows * row_bytes // 2, dtype=torch.uint8, device=o_hat.device)
            bad = _zeros(1, torch.int32, o_hat.device)
            _lib.call('modiff_pack_weights_int4', pack['wcodes'].data_ptr(), pack['w_zp'].data_ptr(),
                      w4.data_ptr(), rows, row_bytes, bad.data_ptr(), _lib.stream_ptr())
            if int(bad.item()):                       # one-time host read at pack time
                raise ModiffError("weight codes do not fit 4 bits")
            pack['wcodes4'] = w4
            _lib.bump_generation()
        codes4 = pack_int4(buf.codes)
        _lib.call('modiff_igemm_conv_packed4', codes4.data_ptr(), pack['wcodes4'].data_ptr(),
                  pack['w_zp'].data_ptr(), buf.x_scale.data_ptr(), pack['w_scale'].data_ptr(),
                  o_hat.data_ptr(), int(accumulate), C.byref(g), _lib.ptr(residual), _lib.ptr(out),
                  _lib.stream_ptr(),
                  nbytes=(8 if accumulate else 4) * o_hat.numel() + (g.batch * g.cin * g.h * g.w
                                                                     + g.cout * g.cin * 9) // 2,
                  tag=g.key())

    def _igemm(self, buf, pack, o_hat, accumulate, bias, g, acc_out=None):
        aq = self.act_quantizer
        if pack['with_sum'] == 0 and self._packed4_ok(g, bias, acc_out):
            return self._igemm_packed4(buf, pack, o_hat, accumulate, g)
        if self._use_im2col(g, buf):
            return self._igemm_im2col(buf, pack, o_hat, accumulate, bias, g, acc_out)
        if self._offset_codes():
            return self._igemm_offset(buf.codes, pack['wcodes'], buf, pack, o_hat, accumulate, bias,
                                      g, None, None)
        # algorithmic bytes: o_hat read + write 8 per output element, 1 per input code, weights
        _lib.call('modiff_igemm_conv',
                  buf.codes.data_ptr(), pack['wcodes'].data_ptr(), pack['with_sum'],
                  buf.x_scale.data_ptr(), pack['w_scale'].data_ptr(), _lib.ptr(pack['w_corr']),
                  o_hat.data_ptr(), int(accumulate), _lib.ptr(bias), C.byref(g),
                  int(aq.channel_wise), self.igemm_impl, _lib.ptr(acc_out), _lib.stream_ptr(),
                  nbytes=(8 if accumulate else 4) * o_hat.numel() + g.batch * g.cin * g.h * g.w
                  + g.cout * g.cin * g.kh * g.kw, tag=g.key())

    # ------------------------------------------------------------------ forward
    fuse_residual_add = os.environ.get("MODIFF_FUSE_RESIDUAL_ADD", "1") != "0"

    def forward_add(self, input, residual):
        """`residual + self(input)`: the sum that ends a residual block
        (qdiff/quant_block.py:313).  In the steady modulated state the GEMM's epilogue writes
        the sum next to the cached output; otherwise the layer runs the ordinary way and the
        sum is a separate kernel."""
        from .ops import ActSource, add
        steady = (self.fuse_residual_add and self.modulate and self.use_act_quant
                  and self.use_weight_quant and not self.disable_act_quant
                  and self.a_hat is not None and self.o_hat is not None and self.split == 0
                  and self.fwd_func is F.conv2d and not self.act_quantizer.channel_wise
                  and self.activation_function.__class__.__name__ == "StraightThrough"
                  and torch.is_tensor(residual) and residual.is_cuda
                  and residual.dtype == torch.float32)
        if steady:
            g = self._geom(input, 0)
            steady = (tuple(residual.shape) == tuple(self.o_hat.shape)
                      and tuple(self.a_hat.shape) == tuple(input.shape)
                      and not self._use_im2col(g, self._get_buffers(g, residual.device)))
        if not steady:
            return add(residual, self.forward(input))
        src = input if isinstance(input, ActSource) and not input.trivial else None
        x = None
        if src is None:
            x = (input.x0 if isinstance(input, ActSource) else input).contiguous()
        pack = self._pack_weights(g)
        buf = self._get_buffers(g, residual.device)
        self._modq(x, self.a_hat, buf, g, src)
        residual = residual.contiguous()
        out = torch.empty_like(residual)
        if self._offset_codes():
            self._igemm_offset(buf.codes, pack['wcodes'], buf, pack, self.o_hat, True, None, g,
                               residual, out)
            return out
        _lib.call('modiff_igemm_conv_add',
                  buf.codes.data_ptr(), pack['wcodes'].data_ptr(), pack['with_sum'],
                  buf.x_scale.data_ptr(), pack['w_scale'].data_ptr(), _lib.ptr(pack['w_corr']),
                  self.o_hat.data_ptr(), 1, C.byref(g), self.igemm_impl, residual.data_ptr(),
                  out.data_ptr(), _lib.stream_ptr(),
                  nbytes=16 * self.o_hat.numel() + g.batch * g.cin * g.h * g.w
                  + g.cout * g.cin * g.kh * g.kw, tag=g.key())
        return out

    # ------------------------------------------------------------------ upsampled input
    upsampled_input_fusion = os.environ.get("MODIFF_FUSE_UPSAMPLE", "1") != "0"

    def forward_upsampled(self, x):
        """`self(upsample2x(x))` for the convolution of an `Upsample` block
        (ddim/models/diffusion.py:45-51).  In the steady modulated state the upsampled tensor is
        never written: input, cached input and residual repeat every value in 2x2 blocks, so the
        quantiser runs on `x` itself and writes each code four times (`modiff_modq_up2`).  The
        cache `a_hat` of such a layer is kept at the resolution of `x` (each value stands for its
        2x2 block); scale, codes and output are those of the ordinary path."""
        from .ops import upsample2x
        aq = self.act_quantizer
        k = self.fwd_kwargs
        ok = (self.upsampled_input_fusion and self.modulate and self.use_act_quant
              and self.use_weight_quant and not self.disable_act_quant and self.split == 0
              and self.fwd_func is F.conv2d and aq.sym and not aq.channel_wise
              and not aq.running_stat and torch.is_tensor(x) and x.is_cuda
              and x.dtype == torch.float32 and x.dim() == 4 and tuple(k['stride']) == (1, 1)
              and self.weight.shape[1] >= 16)
        if not ok:
            if self._a_hat_half and self.a_hat is not None:
                raise ModiffError("this layer's cache is held at the resolution of its upsample "
                                  "block's input; call reset_cache() before changing its mode (for "
                                  "running statistics set QuantModule.upsampled_input_fusion = False "
                                  "or MODIFF_FUSE_UPSAMPLE=0 first)")
            return self.forward(upsample2x(x))
        if self.a_hat is not None and not self._a_hat_half:
            # this epoch's cache was created by the ordinary path: stay on it
            return self.forward(upsample2x(x))
        x = x.contiguous()
        b, c, h, w = x.shape
        g = self._geom(torch.empty((b, c, 2 * h, 2 * w), device='meta'), 0)
        ho_wo = _lib.out_hw(g)
        out_shape = (g.batch, g.cout, ho_wo[0], ho_wo[1])
        pack = self._pack_weights(g)
        buf = self._get_buffers(g, x.device)
        if self.a_hat is None:
            # first step: unquantised activations (quant_layer.py:326-327, 358-359)
            self._a_store = self._reuse(self._a_store, x.shape, x.device)
            self._a_store.copy_(x)
            self.a_hat = self._a_store
            self._a_hat_half = True
            self._o_store = self._reuse(self._o_store, out_shape, x.device)
            self._conv_first_step(upsample2x(x), pack, self.bias, g, self._o_store, ho_wo)
            self.o_hat = self._o_store
        else:
            if not self._a_hat_half or tuple(self.a_hat.shape) != tuple(x.shape):
                raise ModiffError(f"input shape {tuple(x.shape)} does not match the cached "
                                  f"{tuple(self.a_hat.shape)}; call reset_cache() first")
            n = x.numel()
            # algorithmic bytes per SOURCE element: x 4 + a_hat read/write 8 + four codes
            fixed = (not aq.dynamic) and buf.scale_set
            if not aq.dynamic:      # the first quantised call measures the scale that stays
                buf.scale_set = True
                aq.inited = True
            _lib.call('modiff_modq_up2', x.data_ptr(), self.a_hat.data_ptr(), buf.codes.data_ptr(),
                      buf.x_scale.data_ptr(), C.byref(g), aq.n_bits, int(fixed),
                      buf.scratch.data_ptr(), _lib.stream_ptr(), nbytes=16 * n, tag=g.key())
            self._igemm(buf, pack, self.o_hat, True, None, g)
        out = self.o_hat if self.alias_output else self.o_hat.clone()
        return self.activation_function(out)

    def forward_shared(self, owner, input):
        """Forward of a layer whose input equals `owner`'s input at every step (the k and v
        projections next to q in an attention block): the residual codes, their scale and the
        cached input are the owner's, so the quantiser runs once for all of them."""
        return self.forward(input, 0, _owner=owner)

    def forward(self, input, split: int = 0, _owner=None):
        """`input` is a CUDA fp32 tensor, or an `ops.ActSource` describing one lazily."""
        from .ops import ActSource
        src = None
        if isinstance(input, ActSource):
            # only the modulated int8 steps read a source directly; every other path gets the tensor
            fused = (self.modulate and self.use_act_quant and not self.disable_act_quant and
                     self.use_weight_quant and self.a_hat is not None and not input.trivial)
            if fused:
                src = input
            else:
                input = input.x0 if input.trivial else input.materialize()
        if src is None:
            _lib.require_cuda(input, "QuantModule input")
            input = input.contiguous()

        if not self.use_weight_quant and not self.use_act_quant and not self.modulate:
            g = self._geom(input, 0)
            buf_ho_wo = _lib.out_hw(g)
            out = torch.empty(self._shape_from(input, g, buf_ho_wo), dtype=torch.float32,
                              device=input.device)
            self._conv_fp32(input, self._org_weights_kn(), self.org_bias, g, out)
            return self.activation_function(out)

        if split != 0:
            if self.split != 0:
                assert split == self.split
            else:
                logger.info(f"split at {split}!")
                self.split = split
                self.set_split()

        act_q = (not self.disable_act_quant) and self.use_act_quant
        g = self._geom(input, self.split if (act_q or self.use_weight_quant) else 0)
        ho_wo = _lib.out_hw(g)
        out_shape = self._shape_from(input, g, ho_wo)

        if self.use_weight_quant:
            pack = self._pack_weights(g)
            w_kn, bias = pack['w_dq'], self.bias
        else:
            pack = None
            w_kn, bias = self._org_weights_kn(), self.org_bias

        if not act_q:
            # weight-only quantisation or fully unquantised weights with modulate flag set
            out = torch.empty(out_shape, dtype=torch.float32, device=input.device)
            if self.modulate and self.use_act_quant:
                # disable_act_quant with modulation on: the reference still runs its cached-output
                # branch on the UNMODIFIED input, i.e. from the second call on it adds the
                # bias-free convolution to the previous output (qdiff/quant_layer.py:357-363)
                if self.o_hat is None:
                    self._conv_fp32(input, w_kn, bias, g, out)
                else:
                    from .ops import add
                    self._conv_fp32(input, w_kn, None, g, out)
                    out = add(self.o_hat, out)
                self.o_hat = out
                return self.activation_function(out if self.alias_output else out.clone())
            self._conv_fp32(input, w_kn, bias, g, out)
            return self.activation_function(out)

        if pack is None:
            raise ModiffError("activation quantisation without weight quantisation is not "
                              "part of the accelerated path (call set_quant_state(True, True))")

        # layers with the same input share one quantiser run only while their scales are the
        # same by construction, i.e. measured from that input at every step
        shared = (_owner is not None and self.modulate and _owner.modulate and
                  _owner.a_hat is not None and _owner is not self and
                  self.act_quantizer.dynamic and _owner.act_quantizer.dynamic)
        buf = self._get_buffers(g, input.device)
        if shared:
            obuf = _owner._geom_buffers.get(g.copy(cout=_owner.weight.shape[0]).key())
            shared = obuf is not None and _owner.act_quantizer.n_bits == self.act_quantizer.n_bits
        if self.modulate:
            if self.a_hat is None:
                # first step: activations pass through unquantised (quant_layer.py:326-327, 358-359)
                if shared:
                    self.a_hat = _owner.a_hat
                    _owner._group_register(self, g)
                else:
                    self._a_store = self._reuse(self._a_store, input.shape, input.device)
                    self._a_store.copy_(input)
                    self.a_hat = self._a_store
                self._o_store = self._reuse(self._o_store, out_shape, input.device)
                out = self._o_store
                self._conv_first_step(input, pack, bias, g, out, ho_wo)
                self.o_hat = out
            else:
                if self.a_hat.shape != input.shape:
                    raise ModiffError(f"input shape {tuple(input.shape)} differs from the cached "
                                      f"{tuple(self.a_hat.shape)}; call reset_cache() first")
                if shared and self.a_hat is _owner.a_hat:
                    buf = obuf             # the owner's quantiser already ran on this input
                    if self._group_served != (id(_owner), _owner._group_step):
                        self._igemm(buf, pack, self.o_hat, True, None, g)
                else:
                    self._modq(input, self.a_hat, buf, g, src)
                    if not self._group_launch(buf, pack, g):
                        self._igemm(buf, pack, self.o_hat, True, None, g)
            out = self.o_hat if self.alias_output else self.o_hat.clone()
        else:
            out = torch.empty(out_shape, dtype=torch.float32, device=input.device)
            self._modq(input, None, buf, g)
            self._igemm(buf, pack, out, False, bias, g)
        return self.activation_function(out)

    # ------------------------------------------------------------------ 1x1 convolutions around tokens
    # SpatialTransformer.proj_in / proj_out (ldm/modules/attention.py:270-285) sit between NCHW
    # feature maps and token-major [B, H*W, C] tensors.  A 1x1 convolution without padding is the
    # same GEMM in either layout (its code planes [B][H][W][C] ARE token-major rows), so the layer
    # can quantise in one layout and multiply in the other, and both `rearrange`s disappear: the
    # private caches (a_hat of a token-major input, o_hat of a token-major output) simply live in
    # the layout of the tensor they mirror.
    relayout_fusion = os.environ.get("MODIFF_FUSE_RELAYOUT", "1") != "0"

    def _relayout_ok(self):
        aq = self.act_quantizer
        k = self.fwd_kwargs
        return (self.relayout_fusion and self.fwd_func is F.conv2d
                and tuple(self.weight.shape[2:]) == (1, 1) and tuple(k['stride']) == (1, 1)
                and not isinstance(k['padding'], str) and tuple(k['padding']) == (0, 0)
                and tuple(self.implicit_pad) == (0, 0, 0, 0) and self.weight.shape[1] % 16 == 0
                and self.modulate and self.use_act_quant and not self.disable_act_quant
                and self.use_weight_quant and self.split == 0 and aq.dynamic and aq.sym
                and not aq.channel_wise and not aq.running_stat)

    def forward_tokens_out(self, input):
        """1x1 convolution of an NCHW tensor (or `ops.ActSource`) returned token-major,
        [B, H*W, Cout]: `rearrange(proj_in(x), 'b c h w -> b (h w) c')`."""
        from .ops import ActSource, transpose_last2
        b, c, h, w = input.shape
        cout = self.weight.shape[0]
        if not self._relayout_ok():
            return transpose_last2(self.forward(input).reshape(b, cout, h * w))
        if self.a_hat is None:
            # first evaluation: the public path, then the cached output moves to token-major
            y = self.forward(input)
            self._o_tok = self._reuse(getattr(self, '_o_tok', None), (b, h * w, cout), y.device)
            _lib.call('modiff_transpose', y.data_ptr(), self._o_tok.data_ptr(), b, cout, h * w,
                      _lib.stream_ptr())
            self.o_hat = self._o_tok
            return self.o_hat if self.alias_output else self.o_hat.clone()
        src = input if isinstance(input, ActSource) and not input.trivial else None
        x = None
        if src is None:
            x = (input.x0 if isinstance(input, ActSource) else input).contiguous()
        if tuple(self.a_hat.shape) != tuple(input.shape) or tuple(self.o_hat.shape) != (b, h * w, cout):
            raise ModiffError(f"input shape {tuple(input.shape)} differs from the cached "
                              f"{tuple(self.a_hat.shape)}; call reset_cache() first")
        gc = self._geom(input, 0)
        gl = ConvGeom(b * h * w, c, cout, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0)
        pack = self._pack_weights(gc)
        buf = self._get_buffers(gc, self.a_hat.device)
        self._modq(x, self.a_hat, buf, gc, src)          # codes [B][H][W][C] = token-major rows
        self._igemm(buf, pack, self.o_hat, True, None, gl)
        return self.o_hat if self.alias_output else self.o_hat.clone()

    def forward_tokens_in(self, tokens, h, w):
        """1x1 convolution of a token-major tensor [B, H*W, Cin] returned as NCHW:
        `proj_out(rearrange(x, 'b (h w) c -> b c h w'))`."""
        from .ops import transpose_last2
        _lib.require_cuda(tokens, "QuantModule input")
        tokens = tokens.contiguous()
        b, n, c = tokens.shape
        cout = self.weight.shape[0]
        if n != h * w:
            raise ModiffError(f"{n} tokens do not make a {h} x {w} map")
        if not self._relayout_ok():
            return self.forward(transpose_last2(tokens).reshape(b, c, h, w))
        if self.a_hat is None:
            y = self.forward(transpose_last2(tokens).reshape(b, c, h, w))
            self._a_tok = self._reuse(getattr(self, '_a_tok', None), tokens.shape, tokens.device)
            self._a_tok.copy_(tokens)
            self.a_hat = self._a_tok                   # the cached input mirrors the token layout
            return y
        if tuple(self.a_hat.shape) != tuple(tokens.shape) or tuple(self.o_hat.shape) != (b, cout, h, w):
            raise ModiffError(f"input shape {tuple(tokens.shape)} differs from the cached "
                              f"{tuple(self.a_hat.shape)}; call reset_cache() first")
        gc = ConvGeom(b, c, cout, h, w, 1, 1, 1, 0, 0, 0, 0, 0)
        gl = ConvGeom(b * n, c, cout, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0)
        pack = self._pack_weights(gc)
        buf = self._get_buffers(gc, tokens.device)
        self._modq(tokens, self.a_hat, buf, gl, None)    # flat rows = the convolution's code planes
        self._igemm(buf, pack, self.o_hat, True, None, gc)
        return self.o_hat if self.alias_output else self.o_hat.clone()

    # ------------------------------------------------------------------ two layers, one tensor
    pair_quantisers = os.environ.get("MODIFF_PAIR_QUANTISERS", "1") != "0"

    def forward_pair(self, src, other, other_split=0):
        """This layer on nonlinearity(norm(x)) (`src`, an `ops.ActSource` with a pending norm)
        and `other` on the raw x of the same source, e.g. a residual block's conv1 and its
        shortcut convolution (qdiff/quant_block.py:279-283, 306-311): x is read once per
        quantiser pass for both.  Returns (out_self, out_other), or None when the pair is not in
        the steady modulated state the fused kernels cover (the caller then runs the two layers
        the ordinary way)."""
        def steady(m):
            return (isinstance(m, QuantModule) and m.modulate and m.use_act_quant and
                    m.use_weight_quant and not m.disable_act_quant and m.a_hat is not None and
                    m.o_hat is not None and m.act_quantizer.sym and m.act_quantizer.dynamic and
                    not m.act_quantizer.channel_wise and m.fwd_func is F.conv2d)
        if not (self.pair_quantisers and self.fuse_norm_stats and steady(self) and steady(other)
                and self.split == 0 and src.pending_norm() and src.chan_bias is None
                and src.film is None and (other_split == other.split or other.split == 0)):
            return None
        if other_split and other.split == 0:
            return None          # the ordinary path registers the split on its first use
        ga = self._geom(src, 0)
        gb = other._geom(src, other.split)
        if (ga.stride != 1 or gb.stride != 1 or tuple(self.a_hat.shape) != tuple(src.shape)
                or tuple(other.a_hat.shape) != tuple(src.shape)):
            return None
        packa, packb = self._pack_weights(ga), other._pack_weights(gb)
        bufa, bufb = self._get_buffers(ga, src.device), other._get_buffers(gb, src.device)
        n = src.norm
        raw, table = src.raw_struct()
        _lib.call('modiff_modq_pair', C.byref(raw), n.weight.data_ptr(), n.bias.data_ptr(),
                  n.num_groups, float(n.eps), table.data_ptr(),
                  self.a_hat.data_ptr(), bufa.codes.data_ptr(), bufa.x_scale.data_ptr(),
                  C.byref(ga), self.act_quantizer.n_bits, bufa.scratch.data_ptr(),
                  other.a_hat.data_ptr(), bufb.codes.data_ptr(), bufb.x_scale.data_ptr(),
                  C.byref(gb), other.act_quantizer.n_bits, bufb.scratch.data_ptr(),
                  _lib.stream_ptr(), nbytes=26 * src.numel(), tag=ga.key())
        self._igemm(bufa, packa, self.o_hat, True, None, ga)
        other._igemm(bufb, packb, other.o_hat, True, None, gb)
        outs = []
        for m in (self, other):
            o = m.o_hat if m.alias_output else m.o_hat.clone()
            outs.append(m.activation_function(o))
        return outs[0], outs[1]

    # ------------------------------------------------------------------ grouped small linears
    group_small_linears = os.environ.get("MODIFF_LINEAR_GROUP", "1") != "0"
    _GROUP_MAX_ROWS = 512

    def _group_register(self, member, g):
        """Called on the first step by a layer that shares this layer's codes.  Small linear
        layers (every residual block's projection of the same swish(temb)) are remembered; from
        the next step on they are evaluated together with this layer in one launch."""
        if not (self.group_small_linears and g.h == 1 and g.w == 1 and g.kh == 1 and g.kw == 1
                and g.split == 0 and g.batch <= self._GROUP_MAX_ROWS and g.cin % 16 == 0
                and not self.act_quantizer.channel_wise and self.fwd_func is F.linear
                and member.fwd_func is F.linear and not self._offset_codes()):
            return
        if all(m is not member for m in self._group_members):
            self._group_members.append(member)
            self._group_table = None

    def _group_launch(self, buf, pack, g):
        """One launch for this layer and the registered layers that share its codes
        (`modiff_linear_group`); False when there is nothing to group."""
        members = self._group_members
        if not members or self.fwd_func is not F.linear or g.split != 0:
            return False
        layers = [self] + members
        for m in members:
            if m.a_hat is not self.a_hat or m.o_hat is None or m._wpack is None:
                return False
        sig = tuple((m.o_hat.data_ptr(), m._wpack['wcodes'].data_ptr()) for m in layers)
        if self._group_table is None or self._group_table['sig'] != sig:
            items = (_lib.LinearItem * len(layers))()
            block_map = []
            for i, m in enumerate(layers):
                p = m._wpack
                cout = m.weight.shape[0]
                items[i] = _lib.LinearItem(p['wcodes'].data_ptr(), p['w_scale'].data_ptr(),
                                           _lib.ptr(p['w_corr']), m.o_hat.data_ptr(), cout,
                                           int(p['with_sum']))
                block_map += [(i, c0) for c0 in range(0, cout, 16)]
            raw = torch.frombuffer(bytearray(bytes(items)), dtype=torch.uint8).to(buf.codes.device)
            bm = torch.tensor(block_map, dtype=torch.int32, device=buf.codes.device)
            torch.cuda.current_stream().synchronize()
            self._group_table = dict(sig=sig, items=raw, block_map=bm, n_blocks=len(block_map),
                                     keep=[m._wpack for m in layers])
        tab = self._group_table
        rows = g.batch
        nbytes = sum(8 * rows * m.weight.shape[0] for m in layers) + rows * g.cin
        _lib.call('modiff_linear_group', buf.codes.data_ptr(), buf.x_scale.data_ptr(), rows, g.cin,
                  tab['items'].data_ptr(), tab['block_map'].data_ptr(), tab['n_blocks'],
                  _lib.stream_ptr(), nbytes=nbytes, tag=g.key())
        self._group_step += 1
        for m in members:
            m._group_served = (id(self), self._group_step)
        return True

    @staticmethod
    def _reuse(store, shape, device):
        if store is not None and tuple(store.shape) == tuple(shape) and store.device == device:
            return store
        _lib.bump_generation()
        return torch.empty(tuple(shape), dtype=torch.float32, device=device)

    def _shape_from(self, input, g, ho_wo):
        if self.fwd_func is F.linear:
            return tuple(input.shape[:-1]) + (g.cout,)
        if self.fwd_func is F.conv1d:
            return (g.batch, g.cout, ho_wo[0] * ho_wo[1])
        return (g.batch, g.cout, ho_wo[0], ho_wo[1])

    # ------------------------------------------------------------------ flag setters
    # A flag set on one layer changes which kernels its next call launches; captured CUDA graphs
    # are dropped through the generation counter (graph.py).
    def set_quant_state(self, weight_quant: bool = False, act_quant: bool = False):
        _lib.bump_generation()
        self.use_weight_quant = weight_quant
        self.use_act_quant = act_quant

    def set_dynamic_state(self, dynamic):
        _lib.bump_generation()
        self.act_quantizer.dynamic = dynamic
        if self.split != 0:
            self.act_quantizer_0.dynamic = dynamic

    def set_modualtion(self, modulation):
        _lib.bump_generation()
        self.modulate = modulation

    def reset_cache(self):
        self.a_hat = None
        self.o_hat = None
        self._a_hat_half = False

    def set_split(self):
        _lib.bump_generation()
        self.weight_quantizer_0 = UniformAffineQuantizer(**self.weight_quant_params)
        self.act_quantizer_0 = UniformAffineQuantizer(**self.act_quant_params)

    def set_running_stat(self, running_stat: bool):
        _lib.bump_generation()
        self.act_quantizer.running_stat = running_stat
        if self.split != 0:
            self.act_quantizer_0.running_stat = running_stat
