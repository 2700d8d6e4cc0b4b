"""DDIM (generalised) sampling loop and its schedule helpers for the pixel UNet
(ddim/functions/denoising.py:4-55; scripts/sample_diffusion_ddim.py:24-67 beta schedule,
:377-384 timestep sequences).  State stays on the device for the whole loop; the per-step
coefficients are host scalars computed in fp32 exactly as the reference's tensor ops do.
"""
import os

import numpy as np
import torch

from . import ops, _lib


def get_beta_schedule(beta_schedule="linear", *, beta_start=0.0001, beta_end=0.02,
                      num_diffusion_timesteps=1000):
    """float64 numpy schedule (scripts/sample_diffusion_ddim.py:24-67)."""
    if beta_schedule == "linear":
        betas = np.linspace(beta_start, beta_end, num_diffusion_timesteps, dtype=np.float64)
    elif beta_schedule == "quad":
        betas = np.linspace(beta_start ** 0.5, beta_end ** 0.5, num_diffusion_timesteps,
                            dtype=np.float64) ** 2
    elif beta_schedule == "const":
        betas = beta_end * np.ones(num_diffusion_timesteps, dtype=np.float64)
    elif beta_schedule == "jsd":
        betas = 1.0 / np.linspace(num_diffusion_timesteps, 1, num_diffusion_timesteps,
                                  dtype=np.float64)
    elif beta_schedule == "sigmoid":
        x = np.linspace(-6, 6, num_diffusion_timesteps)
        betas = 1.0 / (np.exp(-x) + 1) * (beta_end - beta_start) + beta_start
    else:
        raise NotImplementedError(beta_schedule)
    assert betas.shape == (num_diffusion_timesteps,)
    return betas


def make_timestep_sequence(num_timesteps=1000, timesteps=100, skip_type="quad"):
    """Sampling timesteps (scripts/sample_diffusion_ddim.py:374-386)."""
    if skip_type == "uniform":
        skip = num_timesteps // timesteps
        return list(range(0, num_timesteps, skip))
    if skip_type == "quad":
        seq = np.linspace(0, np.sqrt(num_timesteps * 0.8), timesteps) ** 2
        return [int(s) for s in list(seq)]
    raise NotImplementedError(skip_type)


def alpha_table(betas):
    """cumprod(1 - [0, betas]) in fp32, as compute_alpha builds it per call
    (ddim/functions/denoising.py:4-7); entry t+1 is alpha-bar of timestep t."""
    b = torch.as_tensor(betas, dtype=torch.float32, device="cpu")
    b = torch.cat([torch.zeros(1), b], dim=0)
    return (1 - b).cumprod(dim=0)


def compute_alpha(beta, t):
    """Reference-compatible helper (ddim/functions/denoising.py:4-7)."""
    beta = torch.cat([torch.zeros(1).to(beta.device), beta], dim=0)
    return (1 - beta).cumprod(dim=0).index_select(0, t + 1).view(-1, 1, 1, 1)


def step_coefficients(alphas, i, j, eta=0.0):
    """fp32 scalars of one update: sqrt(1-at), sqrt(at), sqrt(at_next), c1, c2
    (ddim/functions/denoising.py:30-37)."""
    at = alphas[i + 1]
    an = alphas[j + 1]
    s1 = (1 - at).sqrt()
    s2 = at.sqrt()
    s3 = an.sqrt()
    c1 = eta * ((1 - at / an) * (1 - an) / (1 - at)).sqrt()
    c2 = ((1 - an) - c1 ** 2).sqrt()
    return tuple(float(v) for v in (s1, s2, s3, c1, c2))


def raise_on_device_status():
    """Reads (and clears) the library's sticky device status word - one 4-byte device-to-host
    copy, which waits for the stream - and raises when a kernel reported a failure: bit 0 a
    bounded wait that ran out (the kernel returned early, its outputs are incomplete), bit 2 an
    asymmetric zero point that did not fit the int8 code planes."""
    status = _lib.device_status(reset=True)
    if status:
        raise _lib.ModiffError(
            f"device status {status:#x} after sampling: a kernel gave up on a bounded wait or an "
            "activation zero point did not fit its code plane; the samples are not valid")


@torch.no_grad()
def generalized_steps(x, seq, model, b, with_t=False, last_only=True, **kwargs):
    """DDIM sampling (ddim/functions/denoising.py:10-55).

    Returns ([x_T, ..., x_0], [x0 predictions]) like the reference when `last_only` is
    False; with `last_only` (default) only the final sample is kept: ([x_0], []).
    Noise for eta > 0 comes from `generator` (a CUDA torch.Generator) when given.
    `cuda_graph` (default on, or MODIFF_CUDA_GRAPH=0 to turn it off): a QuantModel's steady-state
    steps are replayed as a CUDA graph (graph.py).
    `check_status` (default on): after the loop the device status word is read once and a
    non-zero value raises (`raise_on_device_status`); callers that time the loop on the device
    pass False and check once afterwards.
    """
    n = x.size(0)
    seq = list(seq)
    seq_next = [-1] + seq[:-1]
    eta = float(kwargs.get("eta", 0))
    generator = kwargs.get("generator", None)
    alphas = alpha_table(b.detach().cpu() if isinstance(b, torch.Tensor) else b)
    use_graph = kwargs.get("cuda_graph", os.environ.get("MODIFF_CUDA_GRAPH", "1") != "0")
    if use_graph and hasattr(model, "graphed") and x.is_cuda:
        model = model.graphed()
    xs, x0_preds, ts = [x], [], []
    xt = x
    for i, j in zip(reversed(seq), reversed(seq_next)):
        t = torch.full((n,), float(i), dtype=torch.float32, device=x.device)
        et = model(xt, t)
        s1, s2, s3, c1, c2 = step_coefficients(alphas, i, j, eta)
        noise = None
        if eta != 0:
            noise = torch.randn(x.shape, generator=generator, device=x.device, dtype=x.dtype)
        if last_only:
            xt = ops.ddim_step(xt, et, s1, s2, s3, c1, c2, noise=noise)
        else:
            xt, x0 = ops.ddim_step(xt, et, s1, s2, s3, c1, c2, noise=noise, want_x0=True)
            x0_preds.append(x0)
            xs.append(xt)
            ts.append(t)
    if last_only:
        xs = [xt]
    if kwargs.get("check_status", True) and x.is_cuda:
        raise_on_device_status()
    if with_t:
        return xs, ts, x0_preds
    return xs, x0_preds
