"""AdaRound weight quantiser in the form calibrated Q-Diffusion / MoDiff checkpoints store it:
per weight a rounding logit `alpha`, per output channel `delta` and `zero_point`
(qdiff/adaptive_rounding.py:9-78; installed by qdiff/utils.py:511-539 and filled from the
checkpoint at :567).

Sampling only ever takes the HARD decision - a weight is rounded up exactly when its logit is
non-negative - so that is all this class implements, and it implements it on the device:
inside a `QuantModule` the integer weight codes come from `modiff_weight_pack_rounded`, and the
stand-alone `forward` is the kernel `modiff_adaround_fake_quant`.  The training-time variants of
the reference class (soft targets, straight-through nearest rounding) raise.

The attribute set (n_bits, sym, delta, zero_point, n_levels, round_mode, alpha, soft_targets,
gamma, zeta, beta) and the parameter name `alpha` are the checkpoint contract and are kept.
"""
import torch
from torch import nn

from . import _lib
from ._lib import ModiffError
from .quant_layer import UniformAffineQuantizer

# rectified-sigmoid stretch of the AdaRound paper; the logits are stored relative to it
GAMMA, ZETA = -0.1, 1.1


def logit_of_fraction(frac):
    """The logit whose stretched sigmoid equals `frac` in (0, 1), i.e. the initial `alpha` that
    makes the hard decision "round up iff frac >= 0.5" (round to nearest).  Evaluated in the
    operation order of the reference's initialiser (qdiff/adaptive_rounding.py:66-74) so that the
    SIGN at frac = 0.5 (a -0.0, which counts as non-negative) agrees with it."""
    return -torch.log((ZETA - GAMMA) / (frac - GAMMA) - 1)


class AdaRoundQuantizer(nn.Module):

    def __init__(self, uaq: UniformAffineQuantizer, weight_tensor: torch.Tensor,
                 round_mode='learned_hard_sigmoid'):
        super().__init__()
        if uaq.delta is None:
            raise ModiffError("the weight quantiser has no scale yet: run one forward pass with "
                              "set_quant_state(True, False) before converting to AdaRound")
        if round_mode != 'learned_hard_sigmoid':
            raise ModiffError(f"round_mode {round_mode!r}: only 'learned_hard_sigmoid' (what "
                              "checkpoints hold) is part of the sampling path")
        for name in ("n_bits", "sym", "n_levels", "channel_wise", "scale_method"):
            setattr(self, name, getattr(uaq, name))
        # own copies: the source quantiser's tensors are views of a packed-weight buffer
        self.delta = uaq.delta.detach().clone()
        zp = uaq.zero_point
        self.zero_point = zp.detach().clone() if torch.is_tensor(zp) else zp
        self.inited = True
        self.round_mode = round_mode
        self.soft_targets = False
        self.gamma, self.zeta, self.beta = GAMMA, ZETA, 2 / 3
        self.alpha = None
        self.init_alpha(weight_tensor.detach().clone())

    def init_alpha(self, x: torch.Tensor):
        """Logits that reproduce round-to-nearest until a checkpoint overwrites them."""
        steps = x / self.delta.to(x.device)
        self.alpha = nn.Parameter(logit_of_fraction(steps - torch.floor(steps)))

    def forward(self, x):
        """Dequantised weights under the hard rounding decision (device kernel)."""
        if self.soft_targets or self.round_mode != 'learned_hard_sigmoid':
            raise ModiffError("soft AdaRound targets and the nearest modes belong to calibration; "
                              "the sampling path rounds hard (soft_targets = False)")
        _lib.require_cuda(x, "AdaRound input")
        x = x.contiguous()
        alpha = self.alpha.detach().to(x.device).contiguous()
        if alpha.shape != x.shape:
            raise ModiffError(f"alpha {tuple(alpha.shape)} does not match the weight {tuple(x.shape)}")
        rows = x.shape[0] if self.channel_wise else 1
        delta = torch.as_tensor(self.delta, dtype=torch.float32, device=x.device).reshape(-1)
        zp = torch.as_tensor(self.zero_point, dtype=torch.float32, device=x.device).reshape(-1)
        if delta.numel() != rows or zp.numel() not in (1, rows):
            raise ModiffError("delta / zero_point do not match the weight's output channels")
        zp = zp.expand(rows).contiguous()
        out = torch.empty_like(x)
        _lib.call('modiff_adaround_fake_quant', x.data_ptr(), alpha.data_ptr(),
                  delta.contiguous().data_ptr(), zp.data_ptr(), out.data_ptr(), rows,
                  x.numel() // rows, int(self.channel_wise), self.n_bits, _lib.stream_ptr())
        return out

    def get_soft_targets(self):
        raise ModiffError("soft AdaRound targets are a calibration-time quantity")

    def extra_repr(self):
        return f'bit={self.n_bits}, symmetric={self.sym}, round_mode={self.round_mode}'
