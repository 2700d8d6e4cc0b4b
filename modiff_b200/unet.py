"""Pixel-space DDPM UNet graph (the model of configs 'DDIM pixel UNet 3x32x32').

Same architecture, parameter names and construction order as the reference's
ddim/models/diffusion.py:197-360, so `torch.manual_seed(s); Model(cfg)` yields the same
random-init weights and reference `state_dict`s load unchanged.  The graph between the
conv / linear layers (GroupNorm, SiLU, adds, concat, resampling, attention) runs on the
library's CUDA kernels through `modiff_b200.ops`; conv / linear children are plain
torch modules until `QuantModel` swaps them for `QuantModule`s.
"""
import math
from types import SimpleNamespace

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops

CIFAR10_CONFIG = dict(
    data=dict(image_size=32, channels=3),
    model=dict(type="simple", in_channels=3, out_ch=3, ch=128, ch_mult=[1, 2, 2, 2],
               num_res_blocks=2, attn_resolutions=[16], dropout=0.1, resamp_with_conv=True),
    diffusion=dict(beta_schedule="linear", beta_start=0.0001, beta_end=0.02,
                   num_diffusion_timesteps=1000),
)


def make_config(d=None, split_shortcut=False):
    """Nested-namespace config as the reference builds from configs/cifar10.yml
    (scripts/sample_diffusion_ddim.py:680-688); `split_shortcut` is the --split flag (:74)."""
    d = CIFAR10_CONFIG if d is None else d

    def conv(v):
        return SimpleNamespace(**{k: conv(x) for k, x in v.items()}) if isinstance(v, dict) else v

    cfg = conv(d)
    cfg.split_shortcut = split_shortcut
    return cfg


def get_timestep_embedding(timesteps, embedding_dim):
    """Sinusoidal embedding, sin half then cos half (ddim/models/diffusion.py:6-24)."""
    assert timesteps.dim() == 1
    return ops.timestep_embedding(timesteps.float(), embedding_dim)


def nonlinearity(x):
    """swish (ddim/models/diffusion.py:27-29)."""
    return ops.silu(x)


def Normalize(in_channels):
    return nn.GroupNorm(num_groups=32, num_channels=in_channels, eps=1e-6, affine=True)


def _conv3(cin, cout, stride=1, padding=1):
    return nn.Conv2d(cin, cout, kernel_size=3, stride=stride, padding=padding)


def _conv1(cin, cout):
    return nn.Conv2d(cin, cout, kernel_size=1, stride=1, padding=0)


def _supports_implicit_pad(m):
    return hasattr(m, "implicit_pad")


class Upsample(nn.Module):
    """Nearest 2x then optional 3x3 conv (ddim/models/diffusion.py:36-52)."""

    def __init__(self, in_channels, with_conv):
        super().__init__()
        self.with_conv = with_conv
        if with_conv:
            self.conv = _conv3(in_channels, in_channels)

    def forward(self, x):
        if self.with_conv and hasattr(self.conv, 'forward_upsampled'):
            return self.conv.forward_upsampled(x)      # a QuantModule reads x at its own size
        x = ops.upsample2x(x)
        return self.conv(x) if self.with_conv else x


class Downsample(nn.Module):
    """Zero pad right/bottom by one, 3x3 stride-2 conv (ddim/models/diffusion.py:55-74).

    A QuantModule child receives the pad as part of its geometry, so the padded tensor is never
    materialised; the padded zeros quantise to code 0 either way.
    """

    def __init__(self, in_channels, with_conv):
        super().__init__()
        self.with_conv = with_conv
        if with_conv:
            self.conv = _conv3(in_channels, in_channels, stride=2, padding=0)

    def forward(self, x):
        if not self.with_conv:
            return F.avg_pool2d(x, kernel_size=2, stride=2)
        if _supports_implicit_pad(self.conv):
            self.conv.implicit_pad = (0, 1, 0, 1)
            return self.conv(x)
        return self.conv(F.pad(x, (0, 1, 0, 1), mode="constant", value=0))


class ResnetBlock(nn.Module):
    """GN-swish-conv, + temb projection, GN-swish-dropout-conv, shortcut
    (ddim/models/diffusion.py:77-148)."""

    def __init__(self, *, in_channels, out_channels=None, conv_shortcut=False, dropout,
                 temb_channels=512):
        super().__init__()
        out_channels = in_channels if out_channels is None else out_channels
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.use_conv_shortcut = conv_shortcut
        self.norm1 = Normalize(in_channels)
        self.conv1 = _conv3(in_channels, out_channels)
        self.temb_proj = nn.Linear(temb_channels, out_channels)
        self.norm2 = Normalize(out_channels)
        self.dropout = nn.Dropout(dropout)
        self.conv2 = _conv3(out_channels, out_channels)
        if in_channels != out_channels:
            if conv_shortcut:
                self.conv_shortcut = _conv3(in_channels, out_channels)
            else:
                self.nin_shortcut = _conv1(in_channels, out_channels)

    def forward(self, x, temb=None, split=0):
        return resnet_forward(self, x, temb, split)


def _is_quant(m):
    """QuantModule children take lazily described inputs (ops.ActSource)."""
    return hasattr(m, "implicit_pad")


def resnet_forward(blk, x, temb, split=0):
    """Shared by ResnetBlock and QuantResnetBlock (qdiff/quant_block.py:293-313).

    `x` is a tensor, or an `ops.ActSource` holding the two halves of the up path's channel
    concat.  With QuantModule children the GroupNorm + swish (+ temb bias) are described to the
    layer instead of being materialised; plain torch children get materialised tensors.
    """
    if temb is None:
        assert len(x) == 2
        x, temb = x
    if isinstance(x, ops.ActSource):
        xa, xb = x.x0, x.x1
    else:
        xa, xb = x, None
    quant = _is_quant(blk.conv1)
    if blk.dropout.training and blk.dropout.p > 0:
        quant = False   # dropout needs the materialised tensor

    src1 = ops.ActSource(xa, xb, norm=blk.norm1, silu=True)
    xs_pair = None
    if (quant and blk.in_channels != blk.out_channels and not blk.use_conv_shortcut
            and _is_quant(blk.nin_shortcut)):
        # conv1 reads norm1(x), the shortcut reads x: both quantisers share their sweeps over x
        pair = blk.conv1.forward_pair(src1, blk.nin_shortcut, split)
        if pair is not None:
            h, xs_pair = pair
    if xs_pair is None:
        h = blk.conv1(src1 if quant else src1.materialize())
    # every block projects the same swish(temb): computed once per step by the model, and the
    # projections share one quantisation of it (the first one to run owns the codes)
    ta = getattr(temb, "_modiff_act", None)
    if ta is None:
        ta = ops.silu(temb)
    owner = getattr(temb, "_modiff_owner", None)
    if owner is not None and owner is not blk.temb_proj and _is_quant(blk.temb_proj):
        tb = blk.temb_proj.forward_shared(owner, ta)
    else:
        tb = blk.temb_proj(ta)
        if _is_quant(blk.temb_proj) and hasattr(temb, "_modiff_act"):
            temb._modiff_owner = blk.temb_proj
    if xs_pair is not None:
        xs = xs_pair
    elif blk.in_channels != blk.out_channels:
        xin = ops.ActSource(xa, xb)
        short = blk.conv_shortcut if blk.use_conv_shortcut else blk.nin_shortcut
        if not _is_quant(short):
            xin = xin.x0 if xin.trivial else xin.materialize()
        if blk.use_conv_shortcut or split == 0:
            xs = short(xin)
        else:
            xs = short(xin, split)
    else:
        xs = xa if xb is None else ops.concat_channels(xa, xb)

    src2 = ops.ActSource(h, chan_bias=tb, norm=blk.norm2, silu=True)
    if quant and _is_quant(blk.conv2):
        # x + conv2(...): the sum is written by conv2's GEMM epilogue where that kernel allows it
        return blk.conv2.forward_add(src2, xs)
    if quant:
        h = blk.conv2(src2)
    else:
        h2 = src2.materialize()
        if blk.dropout.training and blk.dropout.p > 0:
            h2 = blk.dropout(h2)
        h = blk.conv2(h2)
    return ops.add(xs, h)


class AttnBlock(nn.Module):
    """Single-head spatial self attention (ddim/models/diffusion.py:151-194)."""

    def __init__(self, in_channels):
        super().__init__()
        self.in_channels = in_channels
        self.norm = Normalize(in_channels)
        self.q = _conv1(in_channels, in_channels)
        self.k = _conv1(in_channels, in_channels)
        self.v = _conv1(in_channels, in_channels)
        self.proj_out = _conv1(in_channels, in_channels)

    def forward(self, x):
        return attn_forward(self, x)


def attn_forward(blk, x):
    """Shared by AttnBlock and QuantAttnBlock (qdiff/quant_block.py:338-366): the attention
    matmuls and softmax stay in fp32, as in the reference."""
    src = ops.ActSource(x, norm=blk.norm, silu=False)
    h_ = src if _is_quant(blk.q) else src.materialize()
    q = blk.q(h_)
    if _is_quant(blk.q) and _is_quant(blk.k) and _is_quant(blk.v):
        k = blk.k.forward_shared(blk.q, h_)     # same input: one quantisation for q, k, v
        v = blk.v.forward_shared(blk.q, h_)
    else:
        k = blk.k(h_)
        v = blk.v(h_)
    b, c, h, w = q.shape
    if getattr(blk, "int8_attention", False) and getattr(blk, "use_act_quant", False):
        # the block's own (otherwise unused) q / k / v quantisers give the bit width
        bits = ops.int8_attention_bits(blk.act_quantizer_q, "attention")
        h_ = ops.attention_i8_channel_major(q.reshape(b, c, h * w), k.reshape(b, c, h * w),
                                            v.reshape(b, c, h * w), float(int(c) ** (-0.5)), bits)
    else:
        h_ = ops.attention(q.reshape(b, c, h * w), k.reshape(b, c, h * w),
                           v.reshape(b, c, h * w), float(int(c) ** (-0.5)))
    h_ = blk.proj_out(h_.reshape(b, c, h, w))
    return ops.add(x, h_)


_LAZY_BLOCKS = (ResnetBlock,)   # quant_block extends this with QuantResnetBlock


class Model(nn.Module):
    """UNet driver (ddim/models/diffusion.py:197-360)."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        m = config.model
        ch, out_ch, ch_mult = m.ch, m.out_ch, tuple(m.ch_mult)
        resolution = config.data.image_size
        if m.type == 'bayesian':
            self.logvar = nn.Parameter(torch.zeros(config.diffusion.num_diffusion_timesteps))
        self.ch = ch
        self.temb_ch = ch * 4
        self.num_resolutions = len(ch_mult)
        self.num_res_blocks = m.num_res_blocks
        self.resolution = resolution
        self.in_channels = m.in_channels

        self.temb = nn.Module()
        self.temb.dense = nn.ModuleList([nn.Linear(ch, self.temb_ch),
                                         nn.Linear(self.temb_ch, self.temb_ch)])
        self.conv_in = _conv3(m.in_channels, ch)

        def res(cin, cout):
            return ResnetBlock(in_channels=cin, out_channels=cout, temb_channels=self.temb_ch,
                               dropout=m.dropout)

        curr_res = resolution
        in_ch_mult = (1,) + ch_mult
        self.down = nn.ModuleList()
        block_in = None
        for lvl in range(self.num_resolutions):
            stage = nn.Module()
            stage.block = nn.ModuleList()
            stage.attn = nn.ModuleList()
            block_in = ch * in_ch_mult[lvl]
            block_out = ch * ch_mult[lvl]
            for _ in range(self.num_res_blocks):
                stage.block.append(res(block_in, block_out))
                block_in = block_out
                if curr_res in m.attn_resolutions:
                    stage.attn.append(AttnBlock(block_in))
            if lvl != self.num_resolutions - 1:
                stage.downsample = Downsample(block_in, m.resamp_with_conv)
                curr_res //= 2
            self.down.append(stage)

        self.mid = nn.Module()
        self.mid.block_1 = res(block_in, block_in)
        self.mid.attn_1 = AttnBlock(block_in)
        self.mid.block_2 = res(block_in, block_in)

        self.up = nn.ModuleList()
        for lvl in reversed(range(self.num_resolutions)):
            stage = nn.Module()
            stage.block = nn.ModuleList()
            stage.attn = nn.ModuleList()
            block_out = ch * ch_mult[lvl]
            skip_in = ch * ch_mult[lvl]
            for i in range(self.num_res_blocks + 1):
                if i == self.num_res_blocks:
                    skip_in = ch * in_ch_mult[lvl]
                stage.block.append(res(block_in + skip_in, block_out))
                block_in = block_out
                if curr_res in m.attn_resolutions:
                    stage.attn.append(AttnBlock(block_in))
            if lvl != 0:
                stage.upsample = Upsample(block_in, m.resamp_with_conv)
                curr_res *= 2
            self.up.insert(0, stage)

        self.norm_out = Normalize(block_in)
        self.conv_out = _conv3(block_in, out_ch)

    def forward(self, x, t=None, context=None):
        if t is None:
            assert len(x) == 2
            x, t = x
        assert x.shape[2] == x.shape[3] == self.resolution

        temb = get_timestep_embedding(t, self.ch)
        temb = self.temb.dense[0](temb)
        temb = nonlinearity(temb)
        temb = self.temb.dense[1](temb)
        temb._modiff_act = ops.silu(temb)      # shared by all residual blocks of this step
        temb._modiff_owner = None

        hs = [self.conv_in(x)]
        for lvl in range(self.num_resolutions):
            stage = self.down[lvl]
            for i in range(self.num_res_blocks):
                h = stage.block[i](hs[-1], temb)
                if len(stage.attn) > 0:
                    h = stage.attn[i](h)
                hs.append(h)
            if lvl != self.num_resolutions - 1:
                hs.append(stage.downsample(hs[-1]))

        h = hs[-1]
        h = self.mid.block_1(h, temb)
        h = self.mid.attn_1(h)
        h = self.mid.block_2(h, temb)

        split_shortcut = bool(getattr(self.config, "split_shortcut", False))
        for lvl in reversed(range(self.num_resolutions)):
            stage = self.up[lvl]
            for i in range(self.num_res_blocks + 1):
                split_ = h.size(1) if split_shortcut else 0
                blk = stage.block[i]
                skip = hs.pop()
                # our own blocks read the two halves of the concat in place
                cat = ops.ActSource(h, skip) if isinstance(blk, _LAZY_BLOCKS) \
                    else ops.concat_channels(h, skip)
                h = blk(cat, temb, split=split_) if split_shortcut else blk(cat, temb)
                if len(stage.attn) > 0:
                    h = stage.attn[i](h)
            if lvl != 0:
                h = stage.upsample(h)

        src = ops.ActSource(h, norm=self.norm_out, silu=True)
        return self.conv_out(src if _is_quant(self.conv_out) else src.materialize())

    def reset_cache(self):
        pass
