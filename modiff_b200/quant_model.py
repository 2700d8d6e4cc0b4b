"""QuantModel: in-place rewrite of a UNet into quantised modules / blocks plus the flag
fan-out, with the reference's surface (qdiff/quant_model.py:12-118)."""
import logging

import torch.nn as nn

from .quant_block import (get_specials, BaseQuantBlock, QuantAttnBlock, QuantQKMatMul,
                          QuantSMVMatMul, QuantBasicTransformerBlock)
from .quant_layer import QuantModule, StraightThrough

logger = logging.getLogger(__name__)


class QuantModel(nn.Module):

    def __init__(self, model: nn.Module, weight_quant_params: dict = {},
                 act_quant_params: dict = {}, **kwargs):
        super().__init__()
        self.model = model
        self.sm_abit = kwargs.get('sm_abit', 8)
        self.modulate = kwargs.get("modulate", False)
        self.in_channels = model.in_channels
        if hasattr(model, 'image_size'):
            self.image_size = model.image_size
        self.specials = get_specials(act_quant_params['leaf_param'])
        self.quant_module_refactor(self.model, weight_quant_params, act_quant_params)
        self.quant_block_refactor(self.model, weight_quant_params, act_quant_params)
        # int8_attention=True (default False): apply the q / k / v / softmax quantisers the
        # blocks construct (qdiff/quant_block.py:120-121, 139-144, 223-235, 331-335) in an integer
        # attention kernel; the reference itself leaves them unapplied, so off reproduces it
        self.set_int8_attention(bool(kwargs.get("int8_attention", False)))

    def quant_module_refactor(self, module: nn.Module, weight_quant_params: dict = {},
                              act_quant_params: dict = {}):
        """Replace every Conv2d / Conv1d / Linear child by a QuantModule, recursively
        (qdiff/quant_model.py:26-44)."""
        for name, child in module.named_children():
            if isinstance(child, (nn.Conv2d, nn.Conv1d, nn.Linear)):
                setattr(module, name, QuantModule(child, weight_quant_params, act_quant_params,
                                                  modulate=self.modulate))
            elif isinstance(child, StraightThrough):
                continue
            else:
                self.quant_module_refactor(child, weight_quant_params, act_quant_params)

    def quant_block_refactor(self, module: nn.Module, weight_quant_params: dict = {},
                             act_quant_params: dict = {}):
        """Re-host residual / attention blocks (qdiff/quant_model.py:46-62)."""
        for name, child in module.named_children():
            special = self.specials.get(type(child).__name__)
            if special is not None and not isinstance(child, BaseQuantBlock):
                if special in (QuantAttnBlock, QuantBasicTransformerBlock):
                    setattr(module, name, special(child, act_quant_params, sm_abit=self.sm_abit))
                elif special is QuantSMVMatMul:
                    setattr(module, name, special(act_quant_params, sm_abit=self.sm_abit))
                elif special is QuantQKMatMul:
                    setattr(module, name, special(act_quant_params))
                else:
                    setattr(module, name, special(child, act_quant_params))
            else:
                self.quant_block_refactor(child, weight_quant_params, act_quant_params)

    def _config_changed(self):
        # captured CUDA graphs replay the kernels of the configuration they were captured in
        self._config_epoch = getattr(self, "_config_epoch", 0) + 1

    def set_quant_state(self, weight_quant: bool = False, act_quant: bool = False):
        self._config_changed()
        for m in self.model.modules():
            if isinstance(m, (QuantModule, BaseQuantBlock)):
                m.set_quant_state(weight_quant, act_quant)

    def reset_cache(self):
        self._cache_epoch = getattr(self, "_cache_epoch", 0) + 1
        for m in self.model.modules():
            if isinstance(m, QuantModule):
                m.reset_cache()

    def graphed(self):
        """This model behind a CUDA-graph replay of its steady-state steps (see graph.py)."""
        from .graph import GraphedModel
        if getattr(self, "_graphed", None) is None:
            object.__setattr__(self, "_graphed", GraphedModel(self))
        return self._graphed

    def set_dynamic_state(self, dynamic):
        self._config_changed()
        for m in self.model.modules():
            if isinstance(m, (QuantModule, QuantAttnBlock)):
                m.set_dynamic_state(dynamic)

    def set_modulation(self, modulation):
        self._config_changed()
        for m in self.model.modules():
            if isinstance(m, QuantModule):
                m.set_modualtion(modulation)

    def set_int8_attention(self, enabled: bool):
        """Switch the integer attention kernel on or off for every attention block (no
        counterpart in the reference, whose attention products stay in floating point)."""
        self._config_changed()
        self.int8_attention = bool(enabled)
        for m in self.model.modules():
            if type(m).__name__ in ("QuantAttnBlock", "QKVAttentionLegacy", "CrossAttention"):
                m.int8_attention = bool(enabled)

    def forward(self, x, timesteps=None, context=None):
        return self.model(x, timesteps, context)

    def set_running_stat(self, running_stat: bool, sm_only=False):
        self._config_changed()
        for m in self.model.modules():
            if isinstance(m, QuantBasicTransformerBlock):
                for attn in (m.attn1, m.attn2):
                    attn.act_quantizer_w.running_stat = running_stat
                    if not sm_only:
                        attn.act_quantizer_q.running_stat = running_stat
                        attn.act_quantizer_k.running_stat = running_stat
                        attn.act_quantizer_v.running_stat = running_stat
            if isinstance(m, QuantModule) and not sm_only:
                m.set_running_stat(running_stat)

    def set_grad_ckpt(self, grad_ckpt: bool):
        for _, m in self.model.named_modules():
            if hasattr(m, 'checkpoint') and isinstance(m, BaseQuantBlock):
                m.checkpoint = grad_ckpt
