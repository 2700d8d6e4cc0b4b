"""AdaRound weight quantiser as calibrated Q-Diffusion / MoDiff checkpoints store it
(qdiff/adaptive_rounding.py:9-78).

Only inference is covered: the hard rounding `floor(w / delta) + (alpha >= 0)` that a loaded
checkpoint applies.  Inside a `QuantModule` the integer weight codes are produced once by
`modiff_weight_pack_rounded` from `alpha`, `delta` and `zero_point`; `forward` below is the
stand-alone fake-quantisation with the same arithmetic (device tensors, no host synchronisation).
"""
import torch
from torch import nn

from ._lib import ModiffError
from .quant_layer import UniformAffineQuantizer


class AdaRoundQuantizer(nn.Module):
    """Same attributes as the reference class: n_bits, sym, delta, zero_point, n_levels,
    round_mode, alpha, soft_targets, gamma, zeta, beta."""

    def __init__(self, uaq: UniformAffineQuantizer, weight_tensor: torch.Tensor,
                 round_mode='learned_hard_sigmoid'):
        super().__init__()
        if uaq.delta is None:
            raise ModiffError("the weight quantiser has no scale yet: run one forward pass with "
                              "set_quant_state(True, False) before converting to AdaRound")
        self.n_bits = uaq.n_bits
        self.sym = uaq.sym
        # own copies: the source quantiser's tensors are views of a packed-weight buffer
        self.delta = uaq.delta.detach().clone()
        self.zero_point = uaq.zero_point.detach().clone() if torch.is_tensor(uaq.zero_point) \
            else uaq.zero_point
        self.n_levels = uaq.n_levels
        self.channel_wise = uaq.channel_wise
        self.scale_method = uaq.scale_method
        self.inited = True
        self.round_mode = round_mode
        self.alpha = None
        self.soft_targets = False
        self.gamma, self.zeta = -0.1, 1.1
        self.beta = 2 / 3
        self.init_alpha(x=weight_tensor.detach().clone())

    def forward(self, x):
        if self.round_mode in ('nearest', 'nearest_ste'):
            x_int = torch.round(x / self.delta)
        elif self.round_mode == 'learned_hard_sigmoid':
            x_floor = torch.floor(x / self.delta)
            if self.soft_targets:
                x_int = x_floor + self.get_soft_targets()
            else:
                x_int = x_floor + (self.alpha >= 0).float()
        else:
            raise ValueError('Wrong rounding mode')
        x_quant = torch.clamp(x_int + self.zero_point, 0, self.n_levels - 1)
        return (x_quant - self.zero_point) * self.delta

    def get_soft_targets(self):
        return torch.clamp(torch.sigmoid(self.alpha) * (self.zeta - self.gamma) + self.gamma, 0, 1)

    def init_alpha(self, x: torch.Tensor):
        """sigmoid(alpha) = fractional part of w / delta, so the initial hard rounding is
        round-to-nearest (qdiff/adaptive_rounding.py:66-74)."""
        if self.round_mode != 'learned_hard_sigmoid':
            raise NotImplementedError
        delta = self.delta.to(x.device)
        x_floor = torch.floor(x / delta)
        rest = (x / delta) - x_floor
        alpha = -torch.log((self.zeta - self.gamma) / (rest - self.gamma) - 1)
        self.alpha = nn.Parameter(alpha)

    def extra_repr(self):
        return f'bit={self.n_bits}, symmetric={self.sym}, round_mode={self.round_mode}'
