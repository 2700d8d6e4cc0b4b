"""Latent-diffusion UNet graph (the model of the LSUN-churches kl-8 config).

Same architecture, parameter names and construction order as the reference's
ldm/modules/diffusionmodules/openaimodel.py:447-782 (UNetModel with ResBlock, AttentionBlock,
QKVAttentionLegacy), so `torch.manual_seed(s); UNetModel(**cfg)` yields the same random-init
weights and reference `state_dict`s load unchanged.  Covers what that config uses: 2-D
convolutions, GroupNorm32 (eps 1e-5), scale-shift norm, up/down-sampling ResBlocks, multi-head
legacy attention; and (for the SD-v1 config) the spatial transformer with cross-attention; no class conditioning,
no fp16.

The graph between the conv / linear layers runs on the library's CUDA kernels (`ops`); conv /
linear children are torch modules until `QuantModel` swaps them for `QuantModule`s.
"""
import math

import torch
import torch.nn as nn

from . import ops

SD_V1 = dict(
    image_size=32, in_channels=4, out_channels=4, model_channels=320,
    attention_resolutions=[4, 2, 1], num_res_blocks=2, channel_mult=[1, 2, 4, 4], num_heads=8,
    use_spatial_transformer=True, transformer_depth=1, context_dim=768, legacy=False)

LSUN_CHURCHES_KL8 = dict(
    image_size=32, in_channels=4, out_channels=4, model_channels=192,
    attention_resolutions=[1, 2, 4, 8], num_res_blocks=2, channel_mult=[1, 2, 2, 4, 4],
    num_heads=8, use_scale_shift_norm=True, resblock_updown=True)


def _is_quant(m):
    return hasattr(m, "implicit_pad")


def normalization(channels):
    """GroupNorm32(32, channels) (ldm/modules/diffusionmodules/util.py:199-216)."""
    return nn.GroupNorm(32, channels)


def zero_module(module):
    """ldm/modules/diffusionmodules/util.py:174-180."""
    for p in module.parameters():
        p.detach().zero_()
    return module


def rerandomize_zero_tensors(model, seed=1234, std=0.02):
    """Random-init latent UNets output exactly 0 because of `zero_module`; for synthetic
    benchmarks every all-zero parameter is redrawn ~ N(0, std) from one seeded generator, in
    `named_parameters()` order (the same rule is applied to the reference model when the
    fixtures are generated)."""
    g = torch.Generator().manual_seed(seed)
    n = 0
    for _, p in model.named_parameters():
        if p.numel() > 0 and not bool(p.detach().any()):
            with torch.no_grad():
                p.copy_(torch.randn(p.shape, generator=g) * std)
            n += 1
    return n


class TimestepBlock(nn.Module):
    pass


class TimestepEmbedSequential(nn.Sequential, TimestepBlock):
    """Passes emb / split to the children that take them (openaimodel.py:74-88)."""

    def forward(self, x, emb, context=None, split=0):
        for layer in self:
            if isinstance(layer, TimestepBlock) or getattr(layer, "takes_emb", False):
                x = layer(x, emb, split=split)
            elif isinstance(layer, SpatialTransformer):
                x = layer(x, context)
            else:
                if isinstance(x, ops.ActSource):
                    x = x.materialize()
                x = layer(x)
        return x


class Upsample(nn.Module):
    """Nearest 2x (+ optional 3x3 conv) (openaimodel.py:91-119)."""

    def __init__(self, channels, use_conv, dims=2, out_channels=None, padding=1):
        super().__init__()
        self.channels = channels
        self.out_channels = out_channels or channels
        self.use_conv = use_conv
        if use_conv:
            self.conv = nn.Conv2d(self.channels, self.out_channels, 3, padding=padding)

    def forward(self, x):
        if self.use_conv and hasattr(self.conv, 'forward_upsampled'):
            return self.conv.forward_upsampled(x)      # a QuantModule reads x at its own size
        x = ops.upsample2x(x)
        return self.conv(x) if self.use_conv else x


class Downsample(nn.Module):
    """Stride-2 3x3 conv or 2x2 average pool (openaimodel.py:134-160)."""

    def __init__(self, channels, use_conv, dims=2, out_channels=None, padding=1):
        super().__init__()
        self.channels = channels
        self.out_channels = out_channels or channels
        self.use_conv = use_conv
        if use_conv:
            self.op = nn.Conv2d(self.channels, self.out_channels, 3, stride=2, padding=padding)

    def forward(self, x):
        return self.op(x) if self.use_conv else ops.avgpool2x(x)


class ResBlock(TimestepBlock):
    """openaimodel.py:163-278."""

    def __init__(self, channels, emb_channels, dropout, out_channels=None, use_conv=False,
                 use_scale_shift_norm=False, dims=2, use_checkpoint=False, up=False, down=False):
        super().__init__()
        self.channels = channels
        self.emb_channels = emb_channels
        self.dropout = dropout
        self.out_channels = out_channels or channels
        self.use_conv = use_conv
        self.use_checkpoint = use_checkpoint
        self.use_scale_shift_norm = use_scale_shift_norm
        self.in_layers = nn.Sequential(normalization(channels), nn.SiLU(),
                                       nn.Conv2d(channels, self.out_channels, 3, padding=1))
        self.updown = up or down
        if up:
            self.h_upd = Upsample(channels, False)
            self.x_upd = Upsample(channels, False)
        elif down:
            self.h_upd = Downsample(channels, False)
            self.x_upd = Downsample(channels, False)
        else:
            self.h_upd = self.x_upd = nn.Identity()
        self.emb_layers = nn.Sequential(
            nn.SiLU(),
            nn.Linear(emb_channels,
                      2 * self.out_channels if use_scale_shift_norm else self.out_channels))
        self.out_layers = nn.Sequential(
            normalization(self.out_channels), nn.SiLU(), nn.Dropout(p=dropout),
            zero_module(nn.Conv2d(self.out_channels, self.out_channels, 3, padding=1)))
        if self.out_channels == channels:
            self.skip_connection = nn.Identity()
        elif use_conv:
            self.skip_connection = nn.Conv2d(channels, self.out_channels, 3, padding=1)
        else:
            self.skip_connection = nn.Conv2d(channels, self.out_channels, 1)

    def forward(self, x, emb, split=0):
        return resblock_forward(self, x, emb, split)


def resblock_forward(blk, x, emb, split=0):
    """Shared by ResBlock and QuantResBlock (qdiff/quant_block.py:83-111).  `x` is a tensor or an
    `ops.ActSource` holding the two halves of a channel concat."""
    if isinstance(x, ops.ActSource):
        xa, xb = x.x0, x.x1
    else:
        xa, xb = x, None
    in_norm, in_conv = blk.in_layers[0], blk.in_layers[-1]
    quant = _is_quant(in_conv)
    src = ops.ActSource(xa, xb, norm=in_norm, silu=True)
    xs_pair = None
    if blk.updown:
        xs_in = blk.x_upd(xa if xb is None else ops.concat_channels(xa, xb))
        if (quant and isinstance(blk.h_upd, Upsample) and not blk.h_upd.use_conv
                and hasattr(in_conv, 'forward_upsampled')):
            # in_conv(upsample(silu(norm(x)))): quantised at the resolution of x
            h = in_conv.forward_upsampled(src.materialize())
        else:
            h = in_conv(blk.h_upd(src.materialize()))
        xa, xb = xs_in, None
    else:
        skip0 = blk.skip_connection
        if (quant and _is_quant(skip0) and skip0.fwd_func is nn.functional.conv2d
                and skip0.weight.shape[-1] == 1):
            # in_conv reads norm(x), the 1x1 skip connection reads x: shared quantiser sweeps
            pair = in_conv.forward_pair(src, skip0, split)
            if pair is not None:
                h, xs_pair = pair
        if xs_pair is None:
            h = in_conv(src if quant else src.materialize())
    ta = getattr(emb, "_modiff_act", None)
    if ta is None:
        ta = ops.silu(emb)
    proj = blk.emb_layers[-1]
    owner = getattr(emb, "_modiff_owner", None)
    if owner is not None and owner is not proj and _is_quant(proj):
        emb_out = proj.forward_shared(owner, ta)     # one quantisation of SiLU(emb) per step
    else:
        emb_out = proj(ta)
        if _is_quant(proj) and hasattr(emb, "_modiff_act"):
            emb._modiff_owner = proj
    out_norm, out_conv = blk.out_layers[0], blk.out_layers[-1]
    if blk.use_scale_shift_norm:
        src2 = ops.ActSource(h, norm=out_norm, silu=True, film=emb_out)
    else:
        src2 = ops.ActSource(h, chan_bias=emb_out, norm=out_norm, silu=True)
    skip = blk.skip_connection
    if xs_pair is not None:
        xs = xs_pair
    elif isinstance(skip, nn.Identity):
        xs = xa if xb is None else ops.concat_channels(xa, xb)
    else:
        xin = ops.ActSource(xa, xb)
        if not _is_quant(skip):
            xin = xin.x0 if xin.trivial else xin.materialize()
        xs = skip(xin, split=split) if split != 0 else skip(xin)
    drop = blk.out_layers[2]
    if quant and not (drop.training and drop.p > 0):
        if _is_quant(out_conv):
            # x + out_conv(...): the sum is written by the GEMM epilogue where that kernel allows it
            return out_conv.forward_add(src2, xs)
        h = out_conv(src2)
    else:
        h2 = src2.materialize()
        if drop.training and drop.p > 0:
            h2 = drop(h2)
        h = out_conv(h2)
    return ops.add(xs, h)


class QKMatMul(nn.Module):
    """Holder of the logit scale (openaimodel.py:350-360); the product itself happens inside
    `ops.attention`."""

    def __init__(self):
        super().__init__()
        self.scale = None


class SMVMatMul(nn.Module):
    """openaimodel.py:363-370."""


class QKVAttentionLegacy(nn.Module):
    """Multi-head attention over a fused [N, H*3*C, T] qkv tensor (openaimodel.py:373-406):
    heads are split before q / k / v, logits are scaled by ch^-1/2 in total (the reference
    multiplies q and k by ch^-1/4 each), softmax in fp32."""

    def __init__(self, n_heads):
        super().__init__()
        self.n_heads = n_heads
        self.qkv_matmul = QKMatMul()
        self.smv_matmul = SMVMatMul()

    def forward(self, qkv):
        bs, width, length = qkv.shape
        assert width % (3 * self.n_heads) == 0
        ch = width // (3 * self.n_heads)
        scale = 1 / math.sqrt(math.sqrt(ch))
        if self.qkv_matmul.scale is not None:
            assert self.qkv_matmul.scale == scale
        else:
            self.qkv_matmul.scale = scale
        qm = self.qkv_matmul
        if getattr(self, "int8_attention", False) and getattr(qm, "use_act_quant", False) and \
                hasattr(qm, "act_quantizer_q"):
            # heads stay where they are in the fused tensor: [N][H][q | k | v][ch][T]
            bits = ops.int8_attention_bits(qm.act_quantizer_q, "attention")
            qkv = qkv.contiguous()
            h = self.n_heads
            base = qkv.reshape(-1)
            out = torch.empty((bs, h * ch, length), dtype=torch.float32, device=qkv.device)
            st = (h * 3 * ch * length, 3 * ch * length, length, 1)
            ops.attention_i8(base, base[ch * length:], base[2 * ch * length:], scale * scale, bs, h,
                             ch, length, length, st, st, out, (h * ch * length, ch * length, length, 1),
                             bits)
            return out
        q, k, v = qkv.reshape(bs * self.n_heads, ch * 3, length).split(ch, dim=1)
        a = ops.attention(q, k, v, scale * scale)
        return a.reshape(bs, -1, length)


class AttentionBlock(nn.Module):
    """openaimodel.py:281-327."""

    def __init__(self, channels, num_heads=1, num_head_channels=-1, use_checkpoint=False,
                 use_new_attention_order=False):
        super().__init__()
        self.channels = channels
        if num_head_channels == -1:
            self.num_heads = num_heads
        else:
            assert channels % num_head_channels == 0
            self.num_heads = channels // num_head_channels
        self.use_checkpoint = use_checkpoint
        self.norm = normalization(channels)
        self.qkv = nn.Conv1d(channels, channels * 3, 1)
        if use_new_attention_order:
            raise NotImplementedError("use_new_attention_order is not used by the covered configs")
        self.attention = QKVAttentionLegacy(self.num_heads)
        self.proj_out = zero_module(nn.Conv1d(channels, channels, 1))

    def forward(self, x):
        return attention_block_forward(self, x)


def attention_block_forward(blk, x):
    """Shared by AttentionBlock and QuantAttentionBlock (openaimodel.py:321-327)."""
    b, c = x.shape[0], x.shape[1]
    spatial = tuple(x.shape[2:])
    x3 = x.reshape(b, c, -1)
    src = ops.ActSource(x3, norm=blk.norm, silu=False)
    qkv = blk.qkv(src if _is_quant(blk.qkv) else src.materialize())
    h = blk.attention(qkv)
    h = blk.proj_out(h)
    return ops.add(x3, h).reshape((b, c) + spatial)


# ---------------------------------------------------------------- spatial transformer (SD)
class GEGLU(nn.Module):
    """ldm/modules/attention.py:37-44."""

    def __init__(self, dim_in, dim_out):
        super().__init__()
        self.proj = nn.Linear(dim_in, dim_out * 2)

    def forward(self, x):
        return ops.geglu(self.proj(x))


class FeedForward(nn.Module):
    """ldm/modules/attention.py:47-64 (gated variant only)."""

    def __init__(self, dim, dim_out=None, mult=4, glu=False, dropout=0.):
        super().__init__()
        if not glu:
            raise NotImplementedError("only the gated feed-forward of the covered configs")
        inner_dim = int(dim * mult)
        dim_out = dim if dim_out is None else dim_out
        self.net = nn.Sequential(GEGLU(dim, inner_dim), nn.Dropout(dropout),
                                 nn.Linear(inner_dim, dim_out))

    def forward(self, x):
        # a quantised second layer evaluates the gate inside its quantiser passes
        return self.net[2](ops.geglu_source(self.net[0].proj(x), self.net[2]))


class CrossQKMatMul(nn.Module):
    def __init__(self, scale):
        super().__init__()
        self.scale = scale


class CrossSMVMatMul(nn.Module):
    pass


class CrossAttention(nn.Module):
    """ldm/modules/attention.py:152-198; the quantised model runs the same arithmetic
    (qdiff/quant_block.py:181-204): projections are quantised layers, the two attention matmuls
    and the softmax stay in floating point."""

    def __init__(self, query_dim, context_dim=None, heads=8, dim_head=64, dropout=0.):
        super().__init__()
        inner_dim = dim_head * heads
        context_dim = query_dim if context_dim is None else context_dim
        self.scale = dim_head ** -0.5
        self.heads = heads
        self.to_q = nn.Linear(query_dim, inner_dim, bias=False)
        self.to_k = nn.Linear(context_dim, inner_dim, bias=False)
        self.to_v = nn.Linear(context_dim, inner_dim, bias=False)
        self.qk_matmul = CrossQKMatMul(self.scale)
        self.smv_matmul = CrossSMVMatMul()
        self.to_out = nn.Sequential(nn.Linear(inner_dim, query_dim), nn.Dropout(dropout))

    def forward(self, x, context=None, mask=None):
        return cross_attention_forward(self, x, context, mask)


def cross_attention_forward(blk, x, context=None, mask=None):
    if mask is not None:
        raise NotImplementedError("attention masks are not used on the sampling path")
    h = blk.heads
    q = blk.to_q(x)
    if context is None:
        if _is_quant(blk.to_k) and _is_quant(blk.to_q) and _is_quant(blk.to_v):
            k = blk.to_k.forward_shared(blk.to_q, x)      # self-attention: q, k, v read one tensor
            v = blk.to_v.forward_shared(blk.to_q, x)
        else:
            k, v = blk.to_k(x), blk.to_v(x)
    else:
        k = blk.to_k(context)
        v = blk.to_v(context) if not (_is_quant(blk.to_k) and _is_quant(blk.to_v)) \
            else blk.to_v.forward_shared(blk.to_k, context)
    b, n, inner = q.shape
    d = inner // h
    if getattr(blk, "int8_attention", False) and getattr(blk, "use_act_quant", False) and \
            hasattr(blk, "act_quantizer_q"):
        # token-major in and out: 'b n (h d)' is read and written in place, no transposes
        bits = ops.int8_attention_bits(blk.act_quantizer_q, "attention")
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        nk = k.shape[1]
        out = torch.empty((b, n, inner), dtype=torch.float32, device=q.device)
        ops.attention_i8(q, k, v, blk.scale, b, h, d, n, nk, (n * inner, d, 1, inner),
                         (nk * inner, d, 1, inner), out, (n * inner, d, 1, inner), bits)
        return blk.to_out[0](out)
    # 'b n (h d) -> (b h) d n': one transpose per tensor gives the channel-major heads
    qt = ops.transpose_last2(q).reshape(b * h, d, n)
    kt = ops.transpose_last2(k).reshape(b * h, d, k.shape[1])
    vt = ops.transpose_last2(v).reshape(b * h, d, v.shape[1])
    out = ops.attention(qt, kt, vt, blk.scale)                    # [(b h), d, n]
    out = ops.transpose_last2(out.reshape(b, inner, n))           # b n (h d)
    return blk.to_out[0](out)


class BasicTransformerBlock(nn.Module):
    """ldm/modules/attention.py:218-241."""

    def __init__(self, dim, n_heads, d_head, dropout=0., context_dim=None, gated_ff=True,
                 checkpoint=True):
        super().__init__()
        self.attn1 = CrossAttention(query_dim=dim, heads=n_heads, dim_head=d_head, dropout=dropout)
        self.ff = FeedForward(dim, dropout=dropout, glu=gated_ff)
        self.attn2 = CrossAttention(query_dim=dim, context_dim=context_dim, heads=n_heads,
                                    dim_head=d_head, dropout=dropout)
        self.norm1 = nn.LayerNorm(dim)
        self.norm2 = nn.LayerNorm(dim)
        self.norm3 = nn.LayerNorm(dim)
        self.checkpoint = checkpoint

    def forward(self, x, context=None):
        return transformer_block_forward(self, x, context)


def transformer_block_forward(blk, x, context=None):
    """qdiff/quant_block.py:249-256."""
    # quantised consumers normalise the rows inside their quantiser passes (no LayerNorm output)
    a1, a2 = blk.attn1, blk.attn2
    x = ops.add(cross_attention_forward(
        a1, ops.layernorm_source(x, blk.norm1, a1.to_q, a1.to_k, a1.to_v)), x)
    x = ops.add(cross_attention_forward(a2, ops.layernorm_source(x, blk.norm2, a2.to_q), context), x)
    x = ops.add(blk.ff(ops.layernorm_source(x, blk.norm3, blk.ff.net[0].proj)), x)
    return x


class SpatialTransformer(nn.Module):
    """ldm/modules/attention.py:244-287."""

    def __init__(self, in_channels, n_heads, d_head, depth=1, dropout=0., context_dim=None):
        super().__init__()
        self.in_channels = in_channels
        inner_dim = n_heads * d_head
        self.norm = nn.GroupNorm(num_groups=32, num_channels=in_channels, eps=1e-6, affine=True)
        self.proj_in = nn.Conv2d(in_channels, inner_dim, kernel_size=1, stride=1, padding=0)
        self.transformer_blocks = nn.ModuleList(
            [BasicTransformerBlock(inner_dim, n_heads, d_head, dropout=dropout,
                                   context_dim=context_dim) for _ in range(depth)])
        self.proj_out = zero_module(nn.Conv2d(inner_dim, in_channels, kernel_size=1, stride=1,
                                              padding=0))

    def forward(self, x, context=None):
        b, c, h, w = x.shape
        src = ops.ActSource(x, norm=self.norm, silu=False)
        if _is_quant(self.proj_in):
            t = self.proj_in.forward_tokens_out(src)                 # b (h w) c, no rearrange
        else:
            t = self.proj_in(src.materialize())
            t = ops.transpose_last2(t.reshape(b, t.shape[1], h * w))
        inner = t.shape[2]
        for block in self.transformer_blocks:
            t = block(t, context)
        if _is_quant(self.proj_out):
            return ops.add(self.proj_out.forward_tokens_in(t, h, w), x)
        t = ops.transpose_last2(t).reshape(b, inner, h, w)
        return ops.add(self.proj_out(t), x)


class UNetModel(nn.Module):
    """openaimodel.py:447-782 for the covered options."""

    def __init__(self, image_size, in_channels, model_channels, out_channels, num_res_blocks,
                 attention_resolutions, dropout=0, channel_mult=(1, 2, 4, 8), conv_resample=True,
                 dims=2, num_classes=None, use_checkpoint=False, use_fp16=False, num_heads=-1,
                 num_head_channels=-1, num_heads_upsample=-1, use_scale_shift_norm=False,
                 resblock_updown=False, use_new_attention_order=False,
                 use_spatial_transformer=False, transformer_depth=1, context_dim=None,
                 n_embed=None, legacy=True):
        super().__init__()
        if num_classes is not None or dims != 2 or use_fp16 or n_embed:
            raise NotImplementedError("option outside the covered latent-UNet configurations")
        if use_spatial_transformer:
            assert context_dim is not None
            if not isinstance(context_dim, int):
                context_dim = list(context_dim)[0] if len(context_dim) == 1 else list(context_dim)
        if num_heads_upsample == -1:
            num_heads_upsample = num_heads
        assert num_heads != -1 or num_head_channels != -1
        self.image_size = image_size
        self.in_channels = in_channels
        self.model_channels = model_channels
        self.out_channels = out_channels
        self.num_res_blocks = num_res_blocks
        self.attention_resolutions = attention_resolutions
        self.dropout = dropout
        self.channel_mult = channel_mult
        self.conv_resample = conv_resample
        self.num_classes = num_classes
        self.num_heads = num_heads
        self.num_head_channels = num_head_channels
        self.num_heads_upsample = num_heads_upsample
        self.split = False

        time_embed_dim = model_channels * 4
        self.time_embed = nn.Sequential(nn.Linear(model_channels, time_embed_dim), nn.SiLU(),
                                        nn.Linear(time_embed_dim, time_embed_dim))

        def res(cin, cout=None, **kw):
            return ResBlock(cin, time_embed_dim, dropout, out_channels=cout,
                            use_checkpoint=use_checkpoint,
                            use_scale_shift_norm=use_scale_shift_norm, **kw)

        def attn(ch, heads):
            if num_head_channels == -1:
                dim_head = ch // heads
            else:
                heads = ch // num_head_channels
                dim_head = num_head_channels
            if legacy:
                dim_head = ch // heads if use_spatial_transformer else num_head_channels
            if use_spatial_transformer:
                return SpatialTransformer(ch, heads, dim_head, depth=transformer_depth,
                                          context_dim=context_dim)
            return AttentionBlock(ch, use_checkpoint=use_checkpoint, num_heads=heads,
                                  num_head_channels=dim_head,
                                  use_new_attention_order=use_new_attention_order)

        self.input_blocks = nn.ModuleList(
            [TimestepEmbedSequential(nn.Conv2d(in_channels, model_channels, 3, padding=1))])
        input_block_chans = [model_channels]
        ch = model_channels
        ds = 1
        for level, mult in enumerate(channel_mult):
            for _ in range(num_res_blocks):
                layers = [res(ch, mult * model_channels)]
                ch = mult * model_channels
                if ds in attention_resolutions:
                    layers.append(attn(ch, num_heads))
                self.input_blocks.append(TimestepEmbedSequential(*layers))
                input_block_chans.append(ch)
            if level != len(channel_mult) - 1:
                out_ch = ch
                self.input_blocks.append(TimestepEmbedSequential(
                    res(ch, out_ch, down=True) if resblock_updown
                    else Downsample(ch, conv_resample, out_channels=out_ch)))
                ch = out_ch
                input_block_chans.append(ch)
                ds *= 2

        self.middle_block = TimestepEmbedSequential(res(ch), attn(ch, num_heads), res(ch))

        self.output_blocks = nn.ModuleList([])
        for level, mult in list(enumerate(channel_mult))[::-1]:
            for i in range(num_res_blocks + 1):
                ich = input_block_chans.pop()
                layers = [res(ch + ich, model_channels * mult)]
                ch = model_channels * mult
                if ds in attention_resolutions:
                    layers.append(attn(ch, num_heads_upsample))
                if level and i == num_res_blocks:
                    out_ch = ch
                    layers.append(res(ch, out_ch, up=True) if resblock_updown
                                  else Upsample(ch, conv_resample, out_channels=out_ch))
                    ds //= 2
                self.output_blocks.append(TimestepEmbedSequential(*layers))

        self.out = nn.Sequential(normalization(ch), nn.SiLU(),
                                 zero_module(nn.Conv2d(model_channels, out_channels, 3, padding=1)))

    def forward(self, x, timesteps=None, context=None, y=None, **kwargs):
        hs = []
        t_emb = ops.timestep_embedding(timesteps.float(), self.model_channels, style="ldm")
        emb = self.time_embed[0](t_emb)
        emb = ops.silu(emb)
        emb = self.time_embed[2](emb)
        emb._modiff_act = ops.silu(emb)        # every ResBlock projects the same SiLU(emb)
        emb._modiff_owner = None
        h = x
        for module in self.input_blocks:
            h = module(h, emb, context)
            hs.append(h)
        h = self.middle_block(h, emb, context)
        for module in self.output_blocks:
            split = h.shape[1] if self.split else 0
            first = module[0]
            skip = hs.pop()
            cat = ops.ActSource(h, skip) if isinstance(first, _LAZY_BLOCKS) \
                else ops.concat_channels(h, skip)
            h = module(cat, emb, context, split=split)
        src = ops.ActSource(h, norm=self.out[0], silu=True)
        conv = self.out[2]
        return conv(src if _is_quant(conv) else src.materialize())


_LAZY_BLOCKS = (ResBlock,)   # quant_block extends this with QuantResBlock
