"""First-stage decoder of the latent-diffusion models: latents -> pixels
(ldm/models/autoencoder.py:330-333 `AutoencoderKL.decode`; ldm/modules/diffusionmodules/model.py
:465-573 `Decoder`, :85-145 `ResnetBlock`, :153-205 `AttnBlock`, :45-60 `Upsample`).

The decoder is not quantised in the reference and is not part of the timed sampling loop; it is
here so that the latent configurations end in images.  Every layer runs on this package's own
kernels in plain fp32: GroupNorm + SiLU (`modiff_groupnorm_silu`), convolutions as unquantised
`QuantModule`s (`modiff_conv_fp32`, IEEE fp32, no TF32), nearest upsampling, the mid-block
attention through `ops.attention`.  Module names and creation order are the reference's, so
`torch.manual_seed` reproduces its random initialisation and its checkpoints' `state_dict`
keys (`decoder.*`, `post_quant_conv.*`) load unchanged.  CUDA tensors only.
"""
import torch
import torch.nn as nn

from . import ops
from ._lib import ModiffError
from .quant_layer import QuantModule


def _normalize(channels):
    return nn.GroupNorm(num_groups=32, num_channels=channels, eps=1e-6, affine=True)


def _run_conv(conv, x):
    """An fp32 convolution on the library's kernel: the layer is wrapped once in a QuantModule
    left in its unquantised state (qdiff/quant_layer.py:309-311, the plain-convolution branch)."""
    key = (conv.weight.data_ptr(), conv.weight._version,
           None if conv.bias is None else conv.bias._version)
    runner = conv.__dict__.get("_modiff_runner")
    if runner is None or conv.__dict__.get("_modiff_runner_key") != key:
        # (re)built when the weights were moved or overwritten, e.g. by load_state_dict
        runner = QuantModule(conv, {'n_bits': 8, 'channel_wise': True, 'scale_method': 'max'},
                             {'n_bits': 8, 'symmetric': True, 'channel_wise': False,
                              'scale_method': 'max', 'leaf_param': True, 'dynamic': True})
        conv.__dict__["_modiff_runner"] = runner      # not a submodule: state_dict keys stay
        conv.__dict__["_modiff_runner_key"] = key
    return runner(x)


class ResnetBlock(nn.Module):
    """model.py:85-145 with temb_channels = 0 (the autoencoder has no timestep embedding)."""

    def __init__(self, *, in_channels, out_channels=None, conv_shortcut=False, dropout=0.0,
                 temb_channels=0):
        super().__init__()
        if temb_channels:
            raise ModiffError("the first-stage decoder's blocks take no timestep embedding")
        out_channels = in_channels if out_channels is None else out_channels
        self.in_channels, self.out_channels = in_channels, out_channels
        self.use_conv_shortcut = conv_shortcut
        self.norm1 = _normalize(in_channels)
        self.conv1 = nn.Conv2d(in_channels, out_channels, 3, 1, 1)
        self.norm2 = _normalize(out_channels)
        self.dropout = nn.Dropout(dropout)
        self.conv2 = nn.Conv2d(out_channels, out_channels, 3, 1, 1)
        if in_channels != out_channels:
            if conv_shortcut:
                self.conv_shortcut = nn.Conv2d(in_channels, out_channels, 3, 1, 1)
            else:
                self.nin_shortcut = nn.Conv2d(in_channels, out_channels, 1, 1, 0)

    def forward(self, x, temb=None):
        h = _run_conv(self.conv1, ops.groupnorm(x, self.norm1, True))
        h = _run_conv(self.conv2, ops.groupnorm(h, self.norm2, True))
        if self.in_channels != self.out_channels:
            x = _run_conv(self.conv_shortcut if self.use_conv_shortcut else self.nin_shortcut, x)
        return ops.add(x, h)


class AttnBlock(nn.Module):
    """Single-head spatial self-attention (model.py:153-205)."""

    def __init__(self, in_channels):
        super().__init__()
        self.in_channels = in_channels
        self.norm = _normalize(in_channels)
        self.q = nn.Conv2d(in_channels, in_channels, 1)
        self.k = nn.Conv2d(in_channels, in_channels, 1)
        self.v = nn.Conv2d(in_channels, in_channels, 1)
        self.proj_out = nn.Conv2d(in_channels, in_channels, 1)

    def forward(self, x):
        h_ = ops.groupnorm(x, self.norm, False)
        q, k, v = _run_conv(self.q, h_), _run_conv(self.k, h_), _run_conv(self.v, h_)
        b, c, h, w = q.shape
        a = ops.attention(q.reshape(b, c, h * w), k.reshape(b, c, h * w),
                              v.reshape(b, c, h * w), float(int(c) ** (-0.5)))
        return ops.add(x, _run_conv(self.proj_out, a.reshape(b, c, h, w)))


class Upsample(nn.Module):
    """Nearest x2 then an optional 3x3 convolution (model.py:45-60)."""

    def __init__(self, in_channels, with_conv):
        super().__init__()
        self.with_conv = with_conv
        if with_conv:
            self.conv = nn.Conv2d(in_channels, in_channels, 3, 1, 1)

    def forward(self, x):
        x = ops.upsample2x(x)
        return _run_conv(self.conv, x) if self.with_conv else x


class Decoder(nn.Module):
    """model.py:465-573: conv_in, a middle block (ResnetBlock, attention, ResnetBlock), one level
    per entry of `ch_mult` from the coarsest up (num_res_blocks + 1 ResnetBlocks, attention where
    the resolution is listed, nearest x2 upsampling with a convolution between levels),
    GroupNorm + SiLU, conv_out."""

    def __init__(self, *, ch, out_ch, ch_mult=(1, 2, 4, 8), num_res_blocks, attn_resolutions,
                 dropout=0.0, resamp_with_conv=True, in_channels, resolution, z_channels,
                 give_pre_end=False, tanh_out=False, use_linear_attn=False, attn_type="vanilla",
                 **ignorekwargs):
        super().__init__()
        if use_linear_attn or attn_type not in ("vanilla", "none"):
            raise ModiffError("only 'vanilla' / 'none' decoder attention is covered")
        self.ch, self.temb_ch = ch, 0
        self.num_resolutions = len(ch_mult)
        self.num_res_blocks = num_res_blocks
        self.resolution, self.in_channels = resolution, in_channels
        self.give_pre_end, self.tanh_out = give_pre_end, tanh_out
        block_in = ch * ch_mult[-1]
        curr_res = resolution // 2 ** (self.num_resolutions - 1)
        self.z_shape = (1, z_channels, curr_res, curr_res)

        def attention(channels):
            return AttnBlock(channels) if attn_type == "vanilla" else nn.Identity()

        self.conv_in = nn.Conv2d(z_channels, block_in, 3, 1, 1)
        self.mid = nn.Module()
        self.mid.block_1 = ResnetBlock(in_channels=block_in, out_channels=block_in, dropout=dropout)
        self.mid.attn_1 = attention(block_in)
        self.mid.block_2 = ResnetBlock(in_channels=block_in, out_channels=block_in, dropout=dropout)
        self.up = nn.ModuleList()
        for i_level in reversed(range(self.num_resolutions)):
            block, attn = nn.ModuleList(), nn.ModuleList()
            block_out = ch * ch_mult[i_level]
            for _ in range(num_res_blocks + 1):
                block.append(ResnetBlock(in_channels=block_in, out_channels=block_out,
                                         dropout=dropout))
                block_in = block_out
                if curr_res in attn_resolutions:
                    attn.append(attention(block_in))
            up = nn.Module()
            up.block, up.attn = block, attn
            if i_level != 0:
                up.upsample = Upsample(block_in, resamp_with_conv)
                curr_res *= 2
            self.up.insert(0, up)          # index = level, as the reference's state_dict keys
        self.norm_out = _normalize(block_in)
        self.conv_out = nn.Conv2d(block_in, out_ch, 3, 1, 1)

    @torch.no_grad()
    def forward(self, z):
        if not (torch.is_tensor(z) and z.is_cuda and z.dtype == torch.float32):
            raise ModiffError("the decoder runs on CUDA float32 tensors only (no CPU fallback)")
        h = _run_conv(self.conv_in, z.contiguous())
        h = self.mid.block_1(h)
        h = self.mid.attn_1(h)
        h = self.mid.block_2(h)
        for i_level in reversed(range(self.num_resolutions)):
            level = self.up[i_level]
            for i_block in range(self.num_res_blocks + 1):
                h = level.block[i_block](h)
                if len(level.attn) > 0:
                    h = level.attn[i_block](h)
            if i_level != 0:
                h = level.upsample(h)
        if self.give_pre_end:
            return h
        h = _run_conv(self.conv_out, ops.groupnorm(h, self.norm_out, True))
        return torch.tanh(h) if self.tanh_out else h


# ddconfig of the kl-f8 autoencoder both latent configurations use
# (configs/latent-diffusion/lsun_churches-ldm-kl-8.yaml:47-56; v1-inference.yaml has the same)
KL_F8 = dict(double_z=True, z_channels=4, resolution=256, in_channels=3, out_ch=3, ch=128,
             ch_mult=(1, 2, 4, 4), num_res_blocks=2, attn_resolutions=[], dropout=0.0)


class FirstStageDecoder(nn.Module):
    """The decoding half of `AutoencoderKL` (ldm/models/autoencoder.py:285-333): the 1x1
    `post_quant_conv` from `embed_dim` to `z_channels`, then `decoder`.  `decode(z)` takes the
    sampler's latents; callers divide by the model's `scale_factor` first, as
    `decode_first_stage` does (ldm/models/diffusion/ddpm.py)."""

    def __init__(self, ddconfig=None, embed_dim=4):
        super().__init__()
        ddconfig = dict(KL_F8 if ddconfig is None else ddconfig)
        self.decoder = Decoder(**ddconfig)
        self.post_quant_conv = nn.Conv2d(embed_dim, ddconfig["z_channels"], 1)
        self.embed_dim = embed_dim

    @torch.no_grad()
    def decode(self, z):
        if not (torch.is_tensor(z) and z.is_cuda and z.dtype == torch.float32):
            raise ModiffError("the decoder runs on CUDA float32 tensors only (no CPU fallback)")
        return self.decoder(_run_conv(self.post_quant_conv, z.contiguous()))

    forward = decode
