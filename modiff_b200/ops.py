"""Thin Python wrappers over the fp32 graph kernels of libmodiff_b200.so.

Each function allocates its output with torch (device memory plumbing) and launches one
hand-written kernel on the current CUDA stream.  CUDA float32 tensors only.
"""
import ctypes as C
import math

import os

import torch

from . import _lib
from ._lib import ModiffError


def _req(*ts):
    for t in ts:
        if t is not None:
            _lib.require_cuda(t)


def groupnorm(x, norm, silu=False, x1=None, chan_bias=None, film=None):
    """GroupNorm (+SiLU) of `x` (+ a per-(image, channel) bias), or of the channel concat
    [x, x1] without materialising it.  `norm` is a torch.nn.GroupNorm."""
    _req(x, x1, chan_bias, film)
    x = x.contiguous()
    b, c0 = x.shape[0], x.shape[1]
    hw = x.numel() // (b * c0)
    c = c0
    if x1 is not None:
        x1 = x1.contiguous()
        c = c0 + x1.shape[1]
    if c != norm.num_channels:
        raise ModiffError(f"GroupNorm expects {norm.num_channels} channels, got {c}")
    if chan_bias is not None:
        chan_bias = chan_bias.contiguous()
    y = torch.empty((b, c) + tuple(x.shape[2:]), dtype=torch.float32, device=x.device)
    if film is not None:
        film = film.contiguous()
        if tuple(film.shape) != (b, 2 * c):
            raise ModiffError(f"film shape {tuple(film.shape)} != {(b, 2 * c)}")
    _lib.call('modiff_groupnorm_silu', x.data_ptr(), _lib.ptr(x1), c0, _lib.ptr(chan_bias),
              _lib.ptr(film), y.data_ptr(), None, norm.weight.data_ptr(), norm.bias.data_ptr(),
              b, c, hw, norm.num_groups, float(norm.eps), int(silu), _lib.stream_ptr())
    return y


class ActSource:
    """A quantised layer's input that has not been materialised: the channel concat
    [x0 | x1], plus an optional [B, C] bias, optionally GroupNorm'ed (`norm`) and SiLU'ed.

    A modulated `QuantModule` reads such a source directly in its quantiser kernels (the
    normalised tensor is never written); everything else calls `materialize()`.
    """

    layernorm = None          # set by LayerNormSource
    geglu = False             # set by GegluSource

    def __init__(self, x0, x1=None, chan_bias=None, norm=None, silu=False, film=None):
        _req(x0, x1, chan_bias, film)
        self.film = None if film is None else film.contiguous()   # [B, 2C] scale | shift
        self.x0 = x0.contiguous()
        self.x1 = None if x1 is None else x1.contiguous()
        self.chan_bias = None if chan_bias is None else chan_bias.contiguous()
        self.norm = norm
        self.silu = bool(silu)
        c = self.x0.shape[1] + (0 if self.x1 is None else self.x1.shape[1])
        self.shape = torch.Size((self.x0.shape[0], c) + tuple(self.x0.shape[2:]))
        self.device = self.x0.device
        self.dtype = self.x0.dtype
        self.is_cuda = True
        self._stats = None
        self._tensor = None
        self._struct = None

    def dim(self):
        return len(self.shape)

    def size(self, d):
        return self.shape[d]

    def numel(self):
        return self.shape.numel()

    def contiguous(self):
        return self

    @property
    def trivial(self):
        return self.x1 is None and self.chan_bias is None and self.norm is None and not self.silu

    def affine(self):
        """[B, C, 2] scale / shift of the GroupNorm over this source (bias folded in), computed
        once per source object."""
        if self._stats is None and self.norm is not None:
            b, c = self.shape[0], self.shape[1]
            hw = self.numel() // (b * c)
            n = self.norm
            if c != n.num_channels:
                raise ModiffError(f"GroupNorm expects {n.num_channels} channels, got {c}")
            self._stats = torch.empty((b, c, 2), dtype=torch.float32, device=self.device)
            _lib.call('modiff_groupnorm_silu', self.x0.data_ptr(), _lib.ptr(self.x1),
                      self.x0.shape[1], _lib.ptr(self.chan_bias), _lib.ptr(self.film), None,
                      self._stats.data_ptr(),
                      n.weight.data_ptr(), n.bias.data_ptr(), b, c, hw, n.num_groups,
                      float(n.eps), 0, _lib.stream_ptr())
        return self._stats

    def materialize(self):
        """The transformed tensor, computed once with the stand-alone kernels."""
        if self._tensor is None:
            if self.norm is not None:
                self._tensor = groupnorm(self.x0, self.norm, self.silu, self.x1, self.chan_bias,
                                         self.film)
            else:
                t = self.x0 if self.x1 is None else concat_channels(self.x0, self.x1)
                if self.chan_bias is not None:
                    t = add_channel_bias(t, self.chan_bias)
                if self.silu:
                    t = silu(t)
                self._tensor = t
        return self._tensor

    def pending_norm(self):
        """True while the GroupNorm statistics of this source have not been computed: the first
        quantiser that reads it computes them in its own sweep (`modiff_modq_gn`)."""
        return self.norm is not None and self._stats is None

    def raw_struct(self):
        """(modiff_act_source without the normalisation, empty [B, C, 2] table) for
        `modiff_modq_gn`, which fills the table that `affine()` returns from then on."""
        b, c = self.shape[0], self.shape[1]
        if c != self.norm.num_channels:
            raise ModiffError(f"GroupNorm expects {self.norm.num_channels} channels, got {c}")
        self._stats = torch.empty((b, c, 2), dtype=torch.float32, device=self.device)
        raw = _lib.ActSourceStruct(self.x0.data_ptr(), _lib.ptr(self.x1), self.x0.shape[1],
                                   int(self.silu), None, _lib.ptr(self.chan_bias))
        return raw, self._stats

    def struct(self):
        """ctypes mirror of modiff_act_source (keeps this object's tensors alive)."""
        if self._struct is None:
            aff = self.affine()
            self._struct = _lib.ActSourceStruct(
                self.x0.data_ptr(), _lib.ptr(self.x1), self.x0.shape[1], int(self.silu),
                _lib.ptr(aff), None if aff is not None else _lib.ptr(self.chan_bias))
        return self._struct


def silu(x):
    _req(x)
    x = x.contiguous()
    y = torch.empty_like(x)
    _lib.call('modiff_silu', x.data_ptr(), y.data_ptr(), x.numel(), _lib.stream_ptr())
    return y


def layernorm(x, norm):
    """nn.LayerNorm over the last dimension."""
    _req(x)
    x = x.contiguous()
    c = x.shape[-1]
    y = torch.empty_like(x)
    _lib.call('modiff_layernorm', x.data_ptr(), y.data_ptr(), norm.weight.data_ptr(),
              norm.bias.data_ptr(), x.numel() // c, c, float(norm.eps), _lib.stream_ptr())
    return y


class LayerNormSource(ActSource):
    """A linear layer's input that is nn.LayerNorm(x) over the last dimension and has not been
    written: a modulated `QuantModule` normalises the rows inside its quantiser passes
    (`modiff_modq_ln`); every other consumer calls `materialize()`."""

    def __init__(self, x, norm):
        _req(x)
        self.x0 = x.contiguous()
        self.x1 = self.chan_bias = self.film = self.norm = None
        self.silu = False
        self.layernorm = norm
        if self.x0.shape[-1] != norm.normalized_shape[-1] or len(norm.normalized_shape) != 1:
            raise ModiffError(f"LayerNorm{tuple(norm.normalized_shape)} on a tensor of shape "
                              f"{tuple(self.x0.shape)}")
        self.shape = self.x0.shape
        self.device = self.x0.device
        self.dtype = self.x0.dtype
        self.is_cuda = True
        self._stats = self._tensor = self._struct = None

    @property
    def trivial(self):
        return False

    def pending_norm(self):
        return False

    def materialize(self):
        if self._tensor is None:
            self._tensor = layernorm(self.x0, self.layernorm)
        return self._tensor

    def affine(self):
        raise ModiffError("a LayerNorm source has no per-channel table; materialize() it")

    struct = raw_struct = affine


class GegluSource(ActSource):
    """A linear layer's input that is GEGLU(h) = h[..., :n] * gelu(h[..., n:]) and has not been
    written: a modulated `QuantModule` evaluates the gate inside its quantiser passes
    (`modiff_modq_geglu`); every other consumer calls `materialize()`."""

    def __init__(self, h):
        _req(h)
        self.x0 = h.contiguous()
        self.x1 = self.chan_bias = self.film = self.norm = None
        self.silu = False
        self.geglu = True
        if self.x0.shape[-1] % 2:
            raise ModiffError(f"GEGLU needs an even last dimension, got {tuple(self.x0.shape)}")
        self.shape = torch.Size(tuple(self.x0.shape[:-1]) + (self.x0.shape[-1] // 2,))
        self.device = self.x0.device
        self.dtype = self.x0.dtype
        self.is_cuda = True
        self._stats = self._tensor = self._struct = None

    @property
    def trivial(self):
        return False

    def pending_norm(self):
        return False

    def materialize(self):
        if self._tensor is None:
            self._tensor = geglu(self.x0)
        return self._tensor

    def affine(self):
        raise ModiffError("a GEGLU source has no per-channel table; materialize() it")

    struct = raw_struct = affine


def geglu_source(h, consumer):
    """GEGLU(h) for a quantised consumer that can read it lazily, else the gated tensor."""
    from .quant_layer import QuantModule
    if GegluSource.enabled and isinstance(consumer, QuantModule):
        return GegluSource(h)
    return geglu(h)


GegluSource.enabled = os.environ.get("MODIFF_FUSE_GEGLU", "1") != "0"


def layernorm_source(x, norm, *consumers):
    """LayerNorm(x) for layers that can read it lazily (every consumer a quantised layer of this
    package), else the normalised tensor."""
    from .quant_layer import QuantModule
    if LayerNormSource.enabled and consumers and all(isinstance(c, QuantModule) for c in consumers):
        return LayerNormSource(x, norm)
    return layernorm(x, norm)


LayerNormSource.enabled = os.environ.get("MODIFF_FUSE_LAYERNORM", "1") != "0"


def geglu(x):
    """x[..., :n] * gelu(x[..., n:])."""
    _req(x)
    x = x.contiguous()
    n = x.shape[-1] // 2
    y = torch.empty(tuple(x.shape[:-1]) + (n,), dtype=torch.float32, device=x.device)
    _lib.call('modiff_geglu', x.data_ptr(), y.data_ptr(), x.numel() // (2 * n), n,
              _lib.stream_ptr())
    return y


def transpose_last2(x):
    """[B, R, C] -> [B, C, R] (contiguous)."""
    _req(x)
    x = x.contiguous()
    b, r, c = x.shape
    y = torch.empty((b, c, r), dtype=torch.float32, device=x.device)
    _lib.call('modiff_transpose', x.data_ptr(), y.data_ptr(), b, r, c, _lib.stream_ptr())
    return y


def add(a, b):
    """a + b for equal shapes."""
    _req(a, b)
    if a.shape != b.shape:
        raise ModiffError(f"add: shapes differ {tuple(a.shape)} vs {tuple(b.shape)}")
    a, b = a.contiguous(), b.contiguous()
    out = torch.empty_like(a)
    _lib.call('modiff_add', a.data_ptr(), b.data_ptr(), out.data_ptr(), 1, 1, a.numel(), 0,
                                     _lib.stream_ptr())
    return out


def add_channel_bias(a, b):
    """a[B,C,H,W] + b[B,C][:, :, None, None]."""
    _req(a, b)
    a, b = a.contiguous(), b.contiguous()
    bsz, c = a.shape[0], a.shape[1]
    if tuple(b.shape) != (bsz, c):
        raise ModiffError(f"add_channel_bias: bias shape {tuple(b.shape)} != {(bsz, c)}")
    hw = a.numel() // (bsz * c)
    out = torch.empty_like(a)
    _lib.call('modiff_add', a.data_ptr(), b.data_ptr(), out.data_ptr(), bsz, c, hw, 1,
                                     _lib.stream_ptr())
    return out


def upsample2x(x):
    _req(x)
    x = x.contiguous()
    b, c, h, w = x.shape
    y = torch.empty((b, c, 2 * h, 2 * w), dtype=torch.float32, device=x.device)
    _lib.call('modiff_upsample2x', x.data_ptr(), y.data_ptr(), b, c, h, w, _lib.stream_ptr())
    return y


def avgpool2x(x):
    _req(x)
    x = x.contiguous()
    b, c, h, w = x.shape
    y = torch.empty((b, c, h // 2, w // 2), dtype=torch.float32, device=x.device)
    _lib.call('modiff_avgpool2x', x.data_ptr(), y.data_ptr(), b, c, h, w, _lib.stream_ptr())
    return y


def concat_channels(a, b):
    _req(a, b)
    a, b = a.contiguous(), b.contiguous()
    bsz, ca, cb = a.shape[0], a.shape[1], b.shape[1]
    hw = a.numel() // (bsz * ca)
    y = torch.empty((bsz, ca + cb) + tuple(a.shape[2:]), dtype=torch.float32, device=a.device)
    _lib.call('modiff_concat_c', a.data_ptr(), ca, b.data_ptr(), cb, y.data_ptr(), bsz, hw,
                                          _lib.stream_ptr())
    return y


_FREQ_CACHE = {}


def _embedding_freqs(dim, device, style):
    """Frequency table evaluated by torch on the host (same bits as the reference's own exp),
    cached per device.  style 'ddim': exp(arange(half) * -(log(10000) / (half - 1)))
    (ddim/models/diffusion.py:17-19); style 'ldm': exp(-log(10000) * arange(half) / half)
    (ldm/modules/diffusionmodules/util.py:160-163)."""
    key = (dim, str(device), style)
    if key not in _FREQ_CACHE:
        half = dim // 2
        if style == "ddim":
            emb = math.log(10000) / (half - 1)
            f = torch.exp(torch.arange(half, dtype=torch.float32) * -emb)
        else:
            f = torch.exp(-math.log(10000) * torch.arange(start=0, end=half, dtype=torch.float32)
                          / half)
        _FREQ_CACHE[key] = f.to(device)
    return _FREQ_CACHE[key]


def timestep_embedding(t, dim, style="ddim"):
    """Sinusoidal embedding: 'ddim' = sin | cos, 'ldm' = cos | sin with the latent UNets'
    frequencies."""
    _req(t)
    t = t.contiguous()
    freq = _embedding_freqs(dim, t.device, style)
    emb = torch.empty((t.shape[0], dim), dtype=torch.float32, device=t.device)
    _lib.call('modiff_timestep_embedding', t.data_ptr(), freq.data_ptr(), emb.data_ptr(),
              t.shape[0], dim, int(style == "ldm"), _lib.stream_ptr())
    return emb


def ddim_step(x, e, s1, s2, s3, c1, c2, noise=None, want_x0=False):
    _req(x, e, noise)
    x, e = x.contiguous(), e.contiguous()
    x_next = torch.empty_like(x)
    x0 = torch.empty_like(x) if want_x0 else None
    _lib.call('modiff_ddim_step', x.data_ptr(), e.data_ptr(), _lib.ptr(noise),
                                           x_next.data_ptr(), _lib.ptr(x0), x.numel(),
                                           s1, s2, s3, c1, c2, _lib.stream_ptr())
    return (x_next, x0) if want_x0 else x_next


def cfg_combine(e_uncond, e_cond, scale):
    """Classifier-free guidance: e_uncond + scale * (e_cond - e_uncond)
    (ldm/models/diffusion/ddim.py:207-208)."""
    _req(e_uncond, e_cond)
    a, b = e_uncond.contiguous(), e_cond.contiguous()
    out = torch.empty_like(a)
    _lib.call('modiff_cfg_combine', a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(),
              float(scale), _lib.stream_ptr())
    return out


def pack_int4(codes):
    if not codes.is_cuda or codes.dtype != torch.int8:
        raise ModiffError("pack_int4 expects a CUDA int8 tensor")
    codes = codes.contiguous()
    n = codes.numel()
    out = torch.empty((n + 1) // 2, dtype=torch.uint8, device=codes.device)
    _lib.call('modiff_pack_int4', codes.data_ptr(), out.data_ptr(), n, _lib.stream_ptr())
    return out


def unpack_int4(packed, n, signed=True):
    if not packed.is_cuda or packed.dtype != torch.uint8:
        raise ModiffError("unpack_int4 expects a CUDA uint8 tensor")
    out = torch.empty(n, dtype=torch.int8, device=packed.device)
    _lib.call('modiff_unpack_int4', packed.data_ptr(), out.data_ptr(), n, int(signed),
                                             _lib.stream_ptr())
    return out


def _attn_hw(t):
    """Factor the token count into the (h, w) grid the GEMM tiles walk (powers of two)."""
    if t & (t - 1):
        return None
    w = 1
    while w * w < t:
        w *= 2
    return t // w, w


def _up(v, m):
    return -(-v // m) * m


# MODIFF_FUSED_ATTENTION=0 keeps the three-kernel pipeline for every shape (debug aid)
FUSED_ATTENTION = os.environ.get("MODIFF_FUSED_ATTENTION", "1") != "0"


def attention(q, k, v, scale):
    """Attention over channel-major tensors, one head per batch entry, fp32-accurate
    (qdiff/quant_block.py:191-203, 344-360): q [B, C, Tq], k and v [B, C, Tk];
    out[b,:,i] = sum_j softmax_j(q[b,:,i] . k[b,:,j] * scale) v[b,:,j].

    Two split-bf16 tensor-core GEMMs with a softmax between them (keys padded to a multiple of
    64 with zero probability); small token counts use one CUDA-core kernel."""
    _req(q, k, v)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    b, c, t = q.shape
    tk = k.shape[2]
    out = torch.empty((b, c, t), dtype=torch.float32, device=q.device)
    hw = _attn_hw(t)
    big = hw is not None and t >= 64 and hw[1] <= 128 and c % 8 == 0 and c >= 8 and tk >= 16
    if not big:
        if t > 64 or tk > 64:
            raise ModiffError(f"attention with {t} x {tk} tokens, {c} channels is not covered")
        _lib.call('modiff_attention_small', q.data_ptr(), k.data_ptr(), v.data_ptr(),
                  out.data_ptr(), b, c, t, tk, float(scale), _lib.stream_ptr())
        return out
    l = _lib.lib()
    dev = q.device
    h, w = hw
    cp = max(64, _up(c, 8))                 # channels per token in the bf16 planes
    tkp = _up(tk, 64)                       # keys padded: rows of K, K-extent of P and V
    crow = c if c >= 128 else _up(c, 16)    # rows of V the second GEMM's tile reads
    # GEMM1: S[image][key][query] = scale * q . k
    gq = _lib.ConvGeom(b, c, tk, h, w, 1, 1, 1, 0, 0, 0, 0, 0)
    qp = torch.empty(l.modiff_bf16_planes_bytes(C.byref(gq)) // 2, dtype=torch.int16, device=dev)
    _lib.call('modiff_split_bf16', q.data_ptr(), qp.data_ptr(), C.byref(gq), _lib.stream_ptr())
    gk = _lib.ConvGeom(b, c, tk, 1, tkp, 1, 1, 1, 0, 0, 0, 0, 0)     # keys as a 1 x tkp row
    kp = torch.zeros(b * 2 * tkp * cp, dtype=torch.int16, device=dev) if tkp != tk else \
        torch.empty(b * 2 * tkp * cp, dtype=torch.int16, device=dev)
    gk_src = _lib.ConvGeom(b, c, tk, 1, tk, 1, 1, 1, 0, 0, 0, tkp - tk, 0)  # right pad -> tkp
    _lib.call('modiff_split_bf16', k.data_ptr(), kp.data_ptr(), C.byref(gk_src), _lib.stream_ptr())
    if FUSED_ATTENTION and c <= 256:
        # one kernel: scores and probabilities stay in tensor / shared memory
        cr = _up(c, 64)                     # channel rows of the v planes (zero rows beyond c)
        vp = torch.empty(b * 2 * cr * tkp, dtype=torch.int16, device=dev)
        _lib.call('modiff_split_bf16_rows', v.data_ptr(), vp.data_ptr(), b, c, tk, cr, tkp,
                  _lib.stream_ptr())
        # three bf16 products (hi*hi, hi*lo, lo*hi) for each of the two matrix products
        _lib.call('modiff_attention_tc', qp.data_ptr(), kp.data_ptr(), vp.data_ptr(), out.data_ptr(),
                  b, c, t, tk, cp, tkp, cr, float(scale), _lib.stream_ptr(),
                  nbytes=2 * (qp.numel() + kp.numel() + vp.numel()) + 4 * out.numel(),
                  nops=3 * 2 * 2 * b * t * tk * c)
        return out
    s = torch.empty((b, tk, t), dtype=torch.float32, device=dev)
    d1 = _lib.GemmBf16Desc(qp.data_ptr(), kp.data_ptr(), None, None, s.data_ptr(), 2, 2, 1, cp,
                           float(scale), tkp)
    _lib.call('modiff_gemm_bf16', C.byref(d1), C.byref(gq), _lib.stream_ptr())
    # softmax over keys -> P[image][2][query][tkp]
    pp = torch.empty(b * 2 * t * tkp, dtype=torch.int16, device=dev)
    _lib.call('modiff_softmax_split', s.data_ptr(), pp.data_ptr(), b, tk, t, tkp, _lib.stream_ptr())
    # GEMM2: out[image][c][query] = P . v
    vp = torch.empty(b * 2 * crow * tkp, dtype=torch.int16, device=dev)
    _lib.call('modiff_split_bf16_rows', v.data_ptr(), vp.data_ptr(), b, c, tk, crow, tkp,
              _lib.stream_ptr())
    gv = _lib.ConvGeom(b, tkp, c, h, w, 1, 1, 1, 0, 0, 0, 0, 0)
    d2 = _lib.GemmBf16Desc(pp.data_ptr(), vp.data_ptr(), None, None, out.data_ptr(), 2, 2, 1, tkp,
                           1.0, crow)
    _lib.call('modiff_gemm_bf16', C.byref(d2), C.byref(gv), _lib.stream_ptr())
    return out


_ATTN_SCRATCH = {}


def attention_i8(q, k, v, scale, batch, heads, c, tq, tk, strides_q, strides_kv, out, strides_out,
                 n_bits=8):
    """Integer attention (opt-in; see csrc/attention_i8.cu and oracle/attention_i8.py): q, k, v
    through per-tensor symmetric dynamic quantisers of `n_bits`, both products as int8
    tensor-core MMAs, fp32 softmax with unsigned 8-bit weights.

    q, k, v are fp32 CUDA tensors addressed as x[b*s0 + h*s1 + c*s2 + t*s3] from their data
    pointers with the element strides `strides_q` (q) and `strides_kv` (k and v); `out` likewise
    with `strides_out`.  Channels or tokens must be the contiguous dimension."""
    _req(q, k, v, out)
    l = _lib.lib()
    dev = q.device
    bh = batch * heads
    sizes = [l.modiff_attn_codes_bytes(bh, c, tq, tk, i) for i in range(3)]
    qc, kc, vc = (torch.empty(n, dtype=torch.int8, device=dev) for n in sizes)
    scales = torch.empty(4, dtype=torch.float32, device=dev)
    scratch = _ATTN_SCRATCH.get(dev)
    if scratch is None:
        scratch = _ATTN_SCRATCH[dev] = torch.zeros(16, dtype=torch.uint8, device=dev)
    sq = (C.c_int64 * 4)(*[int(x) for x in strides_q])
    skv = (C.c_int64 * 4)(*[int(x) for x in strides_kv])
    so = (C.c_int64 * 4)(*[int(x) for x in strides_out])
    n_in = batch * heads * c * (tq + 2 * tk)
    _lib.call('modiff_attn_quantize', q.data_ptr(), k.data_ptr(), v.data_ptr(), batch, heads, c, tq,
              tk, sq, skv, n_bits, qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), scales.data_ptr(),
              scratch.data_ptr(), _lib.stream_ptr(), nbytes=9 * n_in)
    _lib.call('modiff_attention_i8', qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), scales.data_ptr(),
              out.data_ptr(), batch, heads, c, tq, tk, so, float(scale), _lib.stream_ptr(),
              nbytes=sum(sizes) + 4 * batch * heads * c * tq,
              # q k^T twice (maximum pass, weight pass) and w v^T once
              nops=2 * batch * heads * tq * tk * (2 * c + c))
    return out


def attention_i8_channel_major(q, k, v, scale, n_bits=8):
    """`attention_i8` for contiguous [B, C, T] tensors, one head per batch entry (the layout of
    `attention`)."""
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    b, c, t = q.shape
    tk = k.shape[2]
    out = torch.empty((b, c, t), dtype=torch.float32, device=q.device)
    return attention_i8(q, k, v, scale, b, 1, c, t, tk, (c * t, 0, t, 1), (c * tk, 0, tk, 1), out,
                        (c * t, 0, t, 1), n_bits)


def int8_attention_bits(quantizer, what):
    """Bit width of an attention quantiser for the integer kernel; it covers symmetric
    per-tensor quantisers only."""
    if not quantizer.sym or quantizer.channel_wise:
        raise ModiffError(f"int8 attention needs symmetric per-tensor {what} quantisers "
                          "(build the model with symmetric activation parameters, --a_sym)")
    return int(quantizer.n_bits)
