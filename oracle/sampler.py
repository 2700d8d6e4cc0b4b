"""Restatement of the DDIM loop and its schedule (ddim/functions/denoising.py:4-55;
scripts/sample_diffusion_ddim.py:24-44, 377-384) without the reference's hard-coded
.to('cuda'), plus the PSNR formula of trt/benchmark_comparison.py:186-191."""
import numpy as np
import torch


def linear_betas(beta_start=0.0001, beta_end=0.02, n=1000):
    """scripts/sample_diffusion_ddim.py:37-40, :88 (float64 linspace cast to float32)."""
    return torch.from_numpy(np.linspace(beta_start, beta_end, n, dtype=np.float64)).float()


def quad_sequence(num_timesteps=1000, steps=100):
    """scripts/sample_diffusion_ddim.py:377-384."""
    seq = np.linspace(0, np.sqrt(num_timesteps * 0.8), steps) ** 2
    return [int(s) for s in list(seq)]


def compute_alpha(beta, t):
    """ddim/functions/denoising.py:4-7."""
    beta = torch.cat([torch.zeros(1), beta], dim=0)
    return (1 - beta).cumprod(dim=0).index_select(0, t + 1).view(-1, 1, 1, 1)


@torch.no_grad()
def ddim_sample(x, seq, model_fn, betas, eta=0.0, generator=None, on_step=None):
    """ddim/functions/denoising.py:10-55; returns the final x."""
    n = x.size(0)
    seq_next = [-1] + list(seq[:-1])
    xt = x
    for step, (i, j) in enumerate(zip(reversed(seq), reversed(seq_next))):
        t = torch.ones(n) * i
        next_t = torch.ones(n) * j
        at = compute_alpha(betas, t.long())
        at_next = compute_alpha(betas, next_t.long())
        et = model_fn(xt, t)
        x0_t = (xt - et * (1 - at).sqrt()) / at.sqrt()
        c1 = eta * ((1 - at / at_next) * (1 - at_next) / (1 - at)).sqrt()
        c2 = ((1 - at_next) - c1 ** 2).sqrt()
        if eta != 0:
            noise = torch.randn(x.shape, generator=generator, dtype=x.dtype)
        else:
            noise = torch.zeros_like(x)
        xt = at_next.sqrt() * x0_t + c1 * noise + c2 * et
        if on_step is not None:
            on_step(step, i, xt, et)
    return xt


def psnr(baseline, other):
    """trt/benchmark_comparison.py:186-191 (peak = larger absolute maximum of the two)."""
    a = np.asarray(baseline, dtype=np.float32).ravel()
    b = np.asarray(other, dtype=np.float32).ravel()
    mse = np.mean((a - b) ** 2)
    max_val = max(np.abs(a).max(), np.abs(b).max())
    if mse > 0 and max_val > 0:
        return float(20 * np.log10(max_val / np.sqrt(mse)))
    return float("inf")
