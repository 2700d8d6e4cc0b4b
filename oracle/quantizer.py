"""Restatement of UniformAffineQuantizer (qdiff/quant_layer.py:36-235) with torch CPU ops."""
import torch


def n_levels_of(n_bits, sym):
    """qdiff/quant_layer.py:54."""
    return 2 ** n_bits if not sym else 2 ** (n_bits - 1) - 1


def per_tensor_scale(x, n_bits, sym, always_zero=False):
    """Per-tensor 'max' scale (qdiff/quant_layer.py:191-214): Python-float arithmetic,
    floor 1e-8, delta cast to x's dtype; zero point is a Python int."""
    n_levels = n_levels_of(n_bits, sym)
    x_min = min(x.min().item(), 0)
    x_max = max(x.max().item(), 0)
    x_absmax = max(abs(x_min), x_max)
    if sym:
        delta = x_absmax / n_levels
    else:
        delta = float(x.max().item() - x.min().item()) / (n_levels - 1)
    if delta < 1e-8:
        delta = 1e-8
    zero_point = round(-x.min().item() / delta) if not (sym or always_zero) else 0
    return torch.tensor(delta).type_as(x), zero_point


def channel_wise_scale(x, n_bits, sym, always_zero=False):
    """Per dim-0 slice min/max scale (qdiff/quant_layer.py:160-190), fp32 tensor arithmetic."""
    n_levels = n_levels_of(n_bits, sym)
    flat = x.reshape(x.shape[0], -1)
    x_max = flat.max(dim=-1)[0]
    x_min = flat.min(dim=-1)[0]
    x_absmax = torch.maximum(x_min.abs(), x_max)
    if sym:
        delta = x_absmax / n_levels
    else:
        delta = (x_max - x_min) / (n_levels - 1)
    delta[delta < 1e-8] = 1e-8
    zero_point = (-x_min / delta).round() if not (sym or always_zero) else torch.zeros_like(delta)
    shape = [-1] + [1] * (x.dim() - 1)
    return delta.view(shape), zero_point.view(shape)


def quantize_codes(x, delta, zero_point, n_bits, sym):
    """Integer grid values before dequantisation (qdiff/quant_layer.py:94-101)."""
    n_levels = n_levels_of(n_bits, sym)
    x_int = torch.round(x / delta) + zero_point
    if sym:
        return torch.clamp(x_int, -n_levels - 1, n_levels)
    return torch.clamp(x_int, 0, n_levels - 1)


def fake_quant(x, n_bits, sym, channel_wise=False, always_zero=False, scale=None):
    """Full forward of a dynamic quantiser: returns (dequantised, codes, delta, zero_point)
    (qdiff/quant_layer.py:70-102)."""
    if scale is None:
        if channel_wise:
            delta, zp = channel_wise_scale(x, n_bits, sym, always_zero)
        else:
            delta, zp = per_tensor_scale(x, n_bits, sym, always_zero)
    else:
        delta, zp = scale
    q = quantize_codes(x, delta, zp, n_bits, sym)
    return (q - zp) * delta, q, delta, zp


def weight_codes(w, n_bits):
    """Per-output-channel asymmetric weight quantisation as the reference's wq_params give it
    (scripts/sample_diffusion_ddim.py:143; qdiff/quant_layer.py:160-190, 94-102).
    Returns (dequantised weights, unsigned codes, delta[c], zero_point[c])."""
    return fake_quant(w, n_bits, sym=False, channel_wise=True)


def adaround_codes(w, alpha, delta, zero_point, n_bits):
    """AdaRound hard rounding of a loaded checkpoint (qdiff/adaptive_rounding.py:49-58 with
    soft_targets False): floor(w / delta) + (alpha >= 0), shifted by the zero point and clamped.
    Returns (dequantised weights, unsigned codes, delta, zero_point) like weight_codes."""
    x_int = torch.floor(w / delta) + (alpha >= 0).float()
    q = torch.clamp(x_int + zero_point, 0, 2 ** n_bits - 1)
    return (q - zero_point) * delta, q, delta, zero_point
