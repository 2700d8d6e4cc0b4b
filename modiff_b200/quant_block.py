"""Quantised block wrappers with the reference's class names and setters
(qdiff/quant_block.py:20-41 BaseQuantBlock, :267-313 QuantResnetBlock, :316-369
QuantAttnBlock, :372-384 get_specials).

Blocks are matched by class NAME, so both this package's `unet.ResnetBlock` / `AttnBlock`
and the reference's own classes of the same names are re-hosted.
"""
import torch.nn as nn

from .quant_layer import QuantModule, UniformAffineQuantizer, StraightThrough
from . import unet
from . import ldm_unet


class BaseQuantBlock(nn.Module):
    """Base of all block structures (qdiff/quant_block.py:20-41)."""

    def __init__(self, act_quant_params: dict = {}):
        super().__init__()
        self.use_weight_quant = False
        self.use_act_quant = False
        self.act_quantizer = UniformAffineQuantizer(**act_quant_params)
        self.activation_function = StraightThrough()
        self.ignore_reconstruction = False

    def set_quant_state(self, weight_quant: bool = False, act_quant: bool = False):
        self.use_weight_quant = weight_quant
        self.use_act_quant = act_quant
        for m in self.modules():
            if isinstance(m, QuantModule):
                m.set_quant_state(weight_quant, act_quant)


class QuantResnetBlock(BaseQuantBlock):
    """Re-hosted pixel-UNet residual block (qdiff/quant_block.py:267-313)."""

    def __init__(self, res, act_quant_params: dict = {}):
        super().__init__(act_quant_params)
        self.in_channels = res.in_channels
        self.out_channels = res.out_channels
        self.use_conv_shortcut = res.use_conv_shortcut
        self.norm1 = res.norm1
        self.conv1 = res.conv1
        self.temb_proj = res.temb_proj
        self.norm2 = res.norm2
        self.dropout = res.dropout
        self.conv2 = res.conv2
        if self.in_channels != self.out_channels:
            if self.use_conv_shortcut:
                self.conv_shortcut = res.conv_shortcut
            else:
                self.nin_shortcut = res.nin_shortcut

    def forward(self, x, temb=None, split=0):
        return unet.resnet_forward(self, x, temb, split)


class QuantAttnBlock(BaseQuantBlock):
    """Re-hosted pixel-UNet attention block (qdiff/quant_block.py:316-369).  As in the
    reference, the q/k/v/w quantisers are constructed (with sm_abit bits) but the attention
    matmuls themselves run unquantised."""

    def __init__(self, attn, act_quant_params: dict = {}, sm_abit=8):
        super().__init__(act_quant_params)
        self.in_channels = attn.in_channels
        self.norm = attn.norm
        self.q = attn.q
        self.k = attn.k
        self.v = attn.v
        self.proj_out = attn.proj_out
        params_w = act_quant_params.copy()
        params_w['n_bits'] = sm_abit
        self.act_quantizer_w = UniformAffineQuantizer(**params_w)
        self.act_quantizer_q = UniformAffineQuantizer(**params_w)
        self.act_quantizer_k = UniformAffineQuantizer(**params_w)
        self.act_quantizer_v = UniformAffineQuantizer(**params_w)

    def forward(self, x):
        return unet.attn_forward(self, x)

    def set_dynamic_state(self, dynamic):
        self.act_quantizer_w.dynamic = dynamic


# ---------------------------------------------------------------- latent UNets (LDM / SD)
class QuantResBlock(BaseQuantBlock, ldm_unet.TimestepBlock):
    """Re-hosted latent-UNet residual block (qdiff/quant_block.py:44-111)."""

    def __init__(self, res, act_quant_params: dict = {}):
        super().__init__(act_quant_params)
        self.channels = res.channels
        self.emb_channels = res.emb_channels
        self.dropout = res.dropout
        self.out_channels = res.out_channels
        self.use_conv = res.use_conv
        self.use_checkpoint = res.use_checkpoint
        self.use_scale_shift_norm = res.use_scale_shift_norm
        self.in_layers = res.in_layers
        self.updown = res.updown
        self.h_upd = res.h_upd
        self.x_upd = res.x_upd
        self.emb_layers = res.emb_layers
        self.out_layers = res.out_layers
        self.skip_connection = res.skip_connection

    def forward(self, x, emb=None, split=0):
        if emb is None:
            assert len(x) == 2
            x, emb = x
        return ldm_unet.resblock_forward(self, x, emb, split)


class QuantQKMatMul(BaseQuantBlock):
    """Holder of the logit scale and of the (never applied) q / k quantisers
    (qdiff/quant_block.py:114-132): the reference keeps this product in floating point."""

    def __init__(self, act_quant_params: dict = {}):
        super().__init__(act_quant_params)
        self.scale = None
        self.use_act_quant = False
        self.act_quantizer_q = UniformAffineQuantizer(**act_quant_params)
        self.act_quantizer_k = UniformAffineQuantizer(**act_quant_params)

    def set_quant_state(self, weight_quant: bool = False, act_quant: bool = False):
        self.use_act_quant = act_quant


class QuantSMVMatMul(BaseQuantBlock):
    """qdiff/quant_block.py:135-151 (quantisers constructed, product in floating point)."""

    def __init__(self, act_quant_params: dict = {}, sm_abit=8):
        super().__init__(act_quant_params)
        self.use_act_quant = False
        self.act_quantizer_v = UniformAffineQuantizer(**act_quant_params)
        params_w = act_quant_params.copy()
        params_w['n_bits'] = sm_abit
        params_w['symmetric'] = False
        params_w['always_zero'] = True
        self.act_quantizer_w = UniformAffineQuantizer(**params_w)

    def set_quant_state(self, weight_quant: bool = False, act_quant: bool = False):
        self.use_act_quant = act_quant


class QuantAttentionBlock(BaseQuantBlock):
    """Re-hosted latent-UNet attention block, used when activations are not quantised
    (qdiff/quant_block.py:154-178)."""

    def __init__(self, attn, act_quant_params: dict = {}):
        super().__init__(act_quant_params)
        self.channels = attn.channels
        self.num_heads = attn.num_heads
        self.use_checkpoint = attn.use_checkpoint
        self.norm = attn.norm
        self.qkv = attn.qkv
        self.attention = attn.attention
        self.proj_out = attn.proj_out

    def forward(self, x):
        return ldm_unet.attention_block_forward(self, x)


class QuantBasicTransformerBlock(BaseQuantBlock):
    """Re-hosted SD transformer block (qdiff/quant_block.py:207-265).  As in the reference the
    q / k / v / softmax quantisers are constructed on the attention modules but the attention
    matmuls run in floating point; the projections and feed-forward layers are QuantModules."""

    def __init__(self, tran, act_quant_params: dict = {}, sm_abit: int = 8):
        super().__init__(act_quant_params)
        self.attn1 = tran.attn1
        self.ff = tran.ff
        self.attn2 = tran.attn2
        self.norm1 = tran.norm1
        self.norm2 = tran.norm2
        self.norm3 = tran.norm3
        self.checkpoint = tran.checkpoint
        params_w = act_quant_params.copy()
        params_w['n_bits'] = sm_abit
        params_w['always_zero'] = True
        for attn in (self.attn1, self.attn2):
            attn.act_quantizer_q = UniformAffineQuantizer(**act_quant_params)
            attn.act_quantizer_k = UniformAffineQuantizer(**act_quant_params)
            attn.act_quantizer_v = UniformAffineQuantizer(**act_quant_params)
            attn.act_quantizer_w = UniformAffineQuantizer(**params_w)
            attn.use_act_quant = False

    def forward(self, x, context=None):
        if context is None and isinstance(x, (tuple, list)):
            assert len(x) == 2
            x, context = x
        return ldm_unet.transformer_block_forward(self, x, context)

    def set_quant_state(self, weight_quant: bool = False, act_quant: bool = False):
        self.attn1.use_act_quant = act_quant
        self.attn2.use_act_quant = act_quant
        self.use_weight_quant = weight_quant
        self.use_act_quant = act_quant
        for m in self.modules():
            if isinstance(m, QuantModule):
                m.set_quant_state(weight_quant, act_quant)


unet._LAZY_BLOCKS = unet._LAZY_BLOCKS + (QuantResnetBlock,)
ldm_unet._LAZY_BLOCKS = ldm_unet._LAZY_BLOCKS + (QuantResBlock,)


def get_specials(quant_act=False):
    """Class-name -> quantised block map (qdiff/quant_block.py:372-384, pixel- and latent-UNet entries)."""
    specials = {
        'ResBlock': QuantResBlock,
        'BasicTransformerBlock': QuantBasicTransformerBlock,
        'ResnetBlock': QuantResnetBlock,
        'AttnBlock': QuantAttnBlock,
    }
    if quant_act:
        specials['QKMatMul'] = QuantQKMatMul
        specials['SMVMatMul'] = QuantSMVMatMul
    else:
        specials['AttentionBlock'] = QuantAttentionBlock
    return specials
