"""Integer attention: the q / k / v / softmax quantisers that the reference CONSTRUCTS on its
attention blocks but never applies (qdiff/quant_block.py:120-121 QuantQKMatMul, :139-144
QuantSMVMatMul, :223-235 QuantBasicTransformerBlock, :331-335 QuantAttnBlock; the forward passes
at :123-128, :146-148, :181-203, :338-366 keep both products in floating point), applied the way
the upstream Q-Diffusion blocks do when activation quantisation reaches the attention:
q, k and v through per-tensor dynamic quantisers, the softmax output through an unsigned 8-bit
quantiser with zero point 0.

PARITY UNPINNED: no run of the reference executes these quantisers, so there is no reference
output to pin this file against; it is the definition the CUDA kernel `modiff_attention_i8` is
tested against, and full-model results with it are reported next to the floating-point
attention's, not instead of them.

Definition (one head per batch entry; q [B, C, Tq], k and v [B, C, Tk]):
    q_int, k_int, v_int : symmetric per-tensor codes, delta = absmax / (2^(b-1) - 1) over the whole
                          tensor (`oracle.quantizer.per_tensor_scale`, quantize_codes)
    S      = q_int^T k_int                                   exact integers
    m_i    = max_j S_ij                                      exact row maximum
    p_ij   = exp2((S_ij - m_i) * c2),  c2 = fp32((dq * dk) * (scale * log2 e))
    w_ij   = rne(255 * p_ij)                                 unsigned 8-bit code, zero point 0:
                                                             the row's largest probability is 255
    out_ci = (sum_j w_ij v_int_cj) * (dv / sum_j w_ij)       exact integer sums, one fp32 scale
The row-wise scale (every row uses the full 8-bit range, and the weights are renormalised by
their own integer sum) is finer than one scale for the whole probability tensor, and it makes
the result independent of the order in which key blocks are visited, so a blocked kernel can
reproduce it exactly up to the rounding of exp2.
"""
import numpy as np
import torch

from .quantizer import per_tensor_scale, quantize_codes

LOG2E = np.float32(1.4426950408889634)


def attention_i8(q, k, v, scale, n_bits=8):
    """Returns (out [B, C, Tq] fp32, dict of the integer intermediates)."""
    dq, _ = per_tensor_scale(q, n_bits, True)
    dk, _ = per_tensor_scale(k, n_bits, True)
    dv, _ = per_tensor_scale(v, n_bits, True)
    qi = quantize_codes(q, dq, 0, n_bits, True).to(torch.int64)
    ki = quantize_codes(k, dk, 0, n_bits, True).to(torch.int64)
    vi = quantize_codes(v, dv, 0, n_bits, True).to(torch.int64)
    s_int = torch.einsum("bci,bcj->bij", qi, ki)
    m = s_int.max(dim=2, keepdim=True)[0]
    c2 = np.float32(np.float32(float(dq)) * np.float32(float(dk))) * \
        np.float32(np.float32(scale) * LOG2E)
    t = (s_int - m).to(torch.float32) * torch.tensor(c2, dtype=torch.float32)
    p = torch.exp2(t)
    w = torch.round(p * 255.0).to(torch.int64)
    l = w.sum(dim=2)                                        # [B, Tq]
    o_int = torch.einsum("bij,bcj->bci", w, vi)             # [B, C, Tq]
    inv = dv.to(torch.float32) / l.to(torch.float32)        # one fp32 division per row
    out = o_int.to(torch.float32) * inv[:, None, :]
    return out, dict(q_int=qi, k_int=ki, v_int=vi, dq=dq, dk=dk, dv=dv, w=w, l=l, o_int=o_int,
                     c2=c2)


def attention_fp(q, k, v, scale):
    """The floating-point attention the reference runs (qdiff/quant_block.py:344-360)."""
    s = torch.einsum("bci,bcj->bij", q, k) * scale
    p = torch.softmax(s, dim=2)
    return torch.einsum("bij,bcj->bci", p, v)
