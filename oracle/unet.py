"""Restatement of the pixel UNet forward (ddim/models/diffusion.py:308-360) and of its
quantised blocks (qdiff/quant_block.py:293-313 QuantResnetBlock, :338-366 QuantAttnBlock)
as a functional graph over a state dict, with every conv / linear an OracleQuantModule."""
import math

import torch
import torch.nn.functional as F

from .quant_module import OracleQuantModule


def pixel_unet_config():
    """Shape parameters of configs/cifar10.yml (:11-22)."""
    return dict(ch=128, out_ch=3, ch_mult=(1, 2, 2, 2), num_res_blocks=2, attn_resolutions=(16,),
                in_channels=3, resolution=32)


def timestep_embedding(t, dim):
    """ddim/models/diffusion.py:6-24."""
    half = dim // 2
    emb = math.log(10000) / (half - 1)
    emb = torch.exp(torch.arange(half, dtype=torch.float32) * -emb)
    emb = t.float()[:, None] * emb[None, :]
    emb = torch.cat([torch.sin(emb), torch.cos(emb)], dim=1)
    if dim % 2 == 1:
        emb = F.pad(emb, (0, 1, 0, 0))
    return emb


def swish(x):
    """ddim/models/diffusion.py:27-29."""
    return x * torch.sigmoid(x)


class OracleUNet:
    """`state` maps the reference Model's parameter names to CPU fp32 tensors."""

    def __init__(self, state, cfg=None, w_bits=8, a_bits=8, a_sym=True, modulate=True,
                 split_shortcut=False, a_channel_wise=False, quant=True, a_dynamic=True):
        self.cfg = cfg or pixel_unet_config()
        self.state = state
        self.split_shortcut = split_shortcut
        self.layers = {}
        for name, w in state.items():
            if not name.endswith(".weight") or w.dim() < 2:
                continue
            base = name[:-len(".weight")]
            stride, padding = 1, 0
            if w.dim() == 4:
                padding = 1 if w.shape[-1] == 3 else 0
                if base.endswith("downsample.conv"):
                    stride, padding = 2, 0
            m = OracleQuantModule(w, state.get(base + ".bias"), stride, padding, w_bits, a_bits,
                                  a_sym, a_channel_wise, modulate, a_dynamic)
            m.use_weight_quant = m.use_act_quant = quant
            if not quant:
                m.modulate = False
            self.layers[base] = m

    def reset_cache(self):
        for m in self.layers.values():
            m.reset_cache()

    def load_calibrated(self, ckpt, split_of=None, load_act=True, prefix="model."):
        """Install the quantiser tensors of a calibrated checkpoint (the state dict that
        qdiff/utils.py:542-628 loads): per layer `weight_quantizer[_0].alpha / delta /
        zero_point` and, with `load_act`, `act_quantizer[_0].delta / zero_point`.  `split_of`
        maps a layer name to its concat split (layers whose checkpoint has `_0` quantisers)."""
        for base, m in self.layers.items():
            k = prefix + base
            if k + ".weight_quantizer.alpha" not in ckpt:
                continue
            slots = ["weight_quantizer"]
            if k + ".weight_quantizer_0.alpha" in ckpt:
                slots.append("weight_quantizer_0")
                m.split = (split_of or {}).get(base, ckpt[k + ".weight_quantizer.alpha"].shape[1])
            m.adaround = [(ckpt[f"{k}.{s}.alpha"], ckpt[f"{k}.{s}.delta"],
                           ckpt[f"{k}.{s}.zero_point"]) for s in slots]
            m._wq = {}
            if load_act and k + ".act_quantizer.delta" in ckpt:
                aslots = ["act_quantizer"] + (["act_quantizer_0"] if len(slots) == 2 else [])
                m.act_scale = [(ckpt[f"{k}.{s}.delta"].reshape(()).float(),
                                int(ckpt.get(f"{k}.{s}.zero_point", torch.zeros(())).item()))
                               for s in aslots]

    # -------------------------------------------------------------- blocks
    def _gn(self, x, base):
        """Normalize = GroupNorm(32, C, eps=1e-6) (ddim/models/diffusion.py:32-33)."""
        return F.group_norm(x, 32, self.state[base + ".weight"], self.state[base + ".bias"], 1e-6)

    def _resnet(self, base, x, temb, split=0):
        """qdiff/quant_block.py:293-313."""
        L = self.layers
        h = swish(self._gn(x, base + ".norm1"))
        h = L[base + ".conv1"].forward(h)
        h = h + L[base + ".temb_proj"].forward(swish(temb))[:, :, None, None]
        h = swish(self._gn(h, base + ".norm2"))
        h = L[base + ".conv2"].forward(h)
        if (base + ".nin_shortcut") in L:
            x = L[base + ".nin_shortcut"].forward(x, split=split)
        return x + h

    def _attn(self, base, x):
        """qdiff/quant_block.py:338-366: attention matmuls unquantised fp32."""
        L = self.layers
        h_ = self._gn(x, base + ".norm")
        q = L[base + ".q"].forward(h_)
        k = L[base + ".k"].forward(h_)
        v = L[base + ".v"].forward(h_)
        b, c, h, w = q.shape
        q = q.reshape(b, c, h * w).permute(0, 2, 1)
        k = k.reshape(b, c, h * w)
        w_ = torch.bmm(q, k) * (int(c) ** (-0.5))
        w_ = F.softmax(w_, dim=2)
        v = v.reshape(b, c, h * w)
        h_ = torch.bmm(v, w_.permute(0, 2, 1)).reshape(b, c, h, w)
        h_ = L[base + ".proj_out"].forward(h_)
        return x + h_

    # -------------------------------------------------------------- forward
    def forward(self, x, t):
        """ddim/models/diffusion.py:308-360."""
        c = self.cfg
        L = self.layers
        nres = len(c["ch_mult"])
        nblk = c["num_res_blocks"]
        temb = timestep_embedding(t, c["ch"])
        temb = L["temb.dense.0"].forward(temb)
        temb = swish(temb)
        temb = L["temb.dense.1"].forward(temb)

        hs = [L["conv_in"].forward(x)]
        for lvl in range(nres):
            for i in range(nblk):
                h = self._resnet(f"down.{lvl}.block.{i}", hs[-1], temb)
                if f"down.{lvl}.attn.{i}.q" in L:
                    h = self._attn(f"down.{lvl}.attn.{i}", h)
                hs.append(h)
            if lvl != nres - 1:
                hs.append(L[f"down.{lvl}.downsample.conv"].forward(F.pad(hs[-1], (0, 1, 0, 1))))

        h = hs[-1]
        h = self._resnet("mid.block_1", h, temb)
        h = self._attn("mid.attn_1", h)
        h = self._resnet("mid.block_2", h, temb)

        for lvl in reversed(range(nres)):
            for i in range(nblk + 1):
                split = h.size(1) if self.split_shortcut else 0
                h = self._resnet(f"up.{lvl}.block.{i}", torch.cat([h, hs.pop()], dim=1), temb,
                                 split=split)
                if f"up.{lvl}.attn.{i}.q" in L:
                    h = self._attn(f"up.{lvl}.attn.{i}", h)
            if lvl != 0:
                h = F.interpolate(h, scale_factor=2.0, mode="nearest")
                h = L[f"up.{lvl}.upsample.conv"].forward(h)

        h = swish(self._gn(h, "norm_out"))
        return L["conv_out"].forward(h)
