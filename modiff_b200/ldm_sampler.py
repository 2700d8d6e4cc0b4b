"""Latent DDIM sampler and its schedule helpers (ldm/models/diffusion/ddim.py:25-54, 117-234;
ldm/modules/diffusionmodules/util.py:21-74; LatentDiffusion.register_schedule,
ldm/models/diffusion/ddpm.py:118-139).  The sampler drives a UNet callable `model(x, t, context)`
directly (the reference reaches it through LatentDiffusion.apply_model -> DiffusionWrapper).
State stays on the device; per-step coefficients are host scalars computed in fp32 as the
reference's buffers are.
"""
import os

import numpy as np
import torch

from . import ops
from .sampler import raise_on_device_status


def make_beta_schedule(schedule, n_timestep, linear_start=1e-4, linear_end=2e-2, cosine_s=8e-3):
    """util.py:21-44 (float64 numpy)."""
    if schedule == "linear":
        betas = torch.linspace(linear_start ** 0.5, linear_end ** 0.5, n_timestep,
                               dtype=torch.float64) ** 2
    elif schedule == "sqrt_linear":
        betas = torch.linspace(linear_start, linear_end, n_timestep, dtype=torch.float64)
    elif schedule == "sqrt":
        betas = torch.linspace(linear_start, linear_end, n_timestep, dtype=torch.float64) ** 0.5
    else:
        raise ValueError(f"schedule '{schedule}' unknown.")
    return betas.numpy()


def make_ddim_timesteps(ddim_discr_method, num_ddim_timesteps, num_ddpm_timesteps, verbose=False):
    """util.py:44-61: note the c = T // S rule (S = 400 gives 500 timesteps) and the +1 offset."""
    if ddim_discr_method == 'uniform':
        c = num_ddpm_timesteps // num_ddim_timesteps
        ddim_timesteps = np.asarray(list(range(0, num_ddpm_timesteps, c)))
    elif ddim_discr_method == 'quad':
        ddim_timesteps = ((np.linspace(0, np.sqrt(num_ddpm_timesteps * .8),
                                       num_ddim_timesteps)) ** 2).astype(int)
    else:
        raise NotImplementedError(ddim_discr_method)
    return ddim_timesteps + 1


def make_ddim_sampling_parameters(alphacums, ddim_timesteps, eta, verbose=False):
    """util.py:64-74; `alphacums` is the float32 alphas_cumprod tensor."""
    alphas = alphacums[ddim_timesteps]
    alphas_prev = np.asarray([alphacums[0]] + alphacums[ddim_timesteps[:-1]].tolist())
    sigmas = eta * np.sqrt((1 - alphas_prev) / (1 - alphas) * (1 - alphas / alphas_prev))
    return sigmas, alphas, alphas_prev


class DDIMSampler:
    """Latent DDIM (ddim.py:12-234) over a UNet callable.

    `model(x, t, context)` returns eps; `linear_start` / `linear_end` / `timesteps` are the
    LatentDiffusion schedule parameters of the YAML config.
    """

    def __init__(self, model, linear_start, linear_end, timesteps=1000, schedule="linear"):
        self.model = model
        self.ddpm_num_timesteps = timesteps
        betas = make_beta_schedule(schedule, timesteps, linear_start, linear_end)
        self.alphas_cumprod = torch.tensor(np.cumprod(1. - betas, axis=0), dtype=torch.float32)

    def make_schedule(self, ddim_num_steps, ddim_discretize="uniform", ddim_eta=0., verbose=False):
        self.ddim_timesteps = make_ddim_timesteps(ddim_discretize, ddim_num_steps,
                                                  self.ddpm_num_timesteps)
        sig, al, alp = make_ddim_sampling_parameters(self.alphas_cumprod, self.ddim_timesteps,
                                                     ddim_eta)
        self.ddim_sigmas, self.ddim_alphas, self.ddim_alphas_prev = sig, al, alp
        self.ddim_sqrt_one_minus_alphas = np.sqrt(1. - al)

    def _coefficients(self, index):
        """fp32 scalars of p_sample_ddim (ddim.py:217-231)."""
        a_t = torch.full((1,), float(self.ddim_alphas[index]))
        a_prev = torch.full((1,), float(self.ddim_alphas_prev[index]))
        sigma = torch.full((1,), float(self.ddim_sigmas[index]))
        s1 = torch.full((1,), float(self.ddim_sqrt_one_minus_alphas[index]))
        c2 = (1. - a_prev - sigma ** 2).sqrt()
        return float(s1), float(a_t.sqrt()), float(a_prev.sqrt()), float(sigma), float(c2)

    @torch.no_grad()
    def sample(self, S, batch_size, shape, conditioning=None, eta=0., x_T=None,
               unconditional_guidance_scale=1., unconditional_conditioning=None, generator=None,
               max_evals=None, img_callback=None, eps_callback=None, cuda_graph=None,
               check_status=True, **kwargs):
        """Returns (samples, intermediates) like the reference; `max_evals` stops early.
        `img_callback(pred_x0, i)` as in the reference (ddim.py:165); `eps_callback(e_t, i)` sees
        the model output of every evaluation.  After the loop the device status word is read once
        (`check_status`): a kernel that gave up on a bounded wait, or an activation zero point
        that did not fit its code plane, raises instead of returning wrong samples."""
        self.make_schedule(S, ddim_eta=eta)
        model = self.model
        if cuda_graph is None:
            cuda_graph = os.environ.get("MODIFF_CUDA_GRAPH", "1") != "0"
        img = x_T
        if img is None:
            raise ValueError("x_T is required (noise is drawn by the caller so shards can be "
                             "re-created)")
        guided = unconditional_conditioning is not None and unconditional_guidance_scale != 1.
        if cuda_graph and hasattr(model, "graphed") and img.is_cuda:
            model = model.graphed()
        b = img.shape[0]
        timesteps = self.ddim_timesteps
        total = timesteps.shape[0]
        for i, step in enumerate(np.flip(timesteps)):
            if max_evals is not None and i >= max_evals:
                break
            index = total - i - 1
            t = torch.full((b,), float(step), dtype=torch.float32, device=img.device)
            if not guided:
                e_t = model(img, t, conditioning) if conditioning is not None else model(img, t)
            else:
                x_in = torch.cat([img] * 2)
                t_in = torch.cat([t] * 2)
                c_in = torch.cat([unconditional_conditioning, conditioning])
                e_all = model(x_in, t_in, c_in)
                e_t = ops.cfg_combine(e_all[:b], e_all[b:], float(unconditional_guidance_scale))
            s1, s2, s3, sigma, c2 = self._coefficients(index)
            noise = None
            if sigma != 0.0:
                noise = torch.randn(img.shape, generator=generator, device=img.device)
            if eps_callback is not None:
                eps_callback(e_t, i)
            if img_callback is not None:
                img, pred_x0 = ops.ddim_step(img, e_t, s1, s2, s3, sigma, c2, noise=noise,
                                             want_x0=True)
                img_callback(pred_x0, i)
            else:
                img = ops.ddim_step(img, e_t, s1, s2, s3, sigma, c2, noise=noise)
        if check_status:
            raise_on_device_status()
        return img, {}


class PLMSSampler(DDIMSampler):
    """Pseudo linear multistep sampler (ldm/models/diffusion/plms.py:12-240), what the reference's
    Stable-Diffusion command runs (`txt2img.py --plms`).  Same schedule and update as DDIM with
    eta = 0, but the eps that enters the update is an Adams-Bashforth combination of the last up
    to four model outputs; the first step evaluates the model twice."""

    def make_schedule(self, ddim_num_steps, ddim_discretize="uniform", ddim_eta=0., verbose=False):
        if ddim_eta != 0:
            raise ValueError('ddim_eta must be 0 for PLMS')          # plms.py:27-28
        super().make_schedule(ddim_num_steps, ddim_discretize, ddim_eta, verbose)

    @torch.no_grad()
    def sample(self, S, batch_size, shape, conditioning=None, eta=0., x_T=None,
               unconditional_guidance_scale=1., unconditional_conditioning=None, max_steps=None,
               img_callback=None, eps_callback=None, cuda_graph=None, check_status=True,
               **kwargs):
        """Returns (samples, intermediates); `eps_callback(e, k)` sees every model output in
        evaluation order, `img_callback(pred_x0, i)` every step's x0 prediction (plms.py:165);
        `max_steps` stops early; `check_status` as in DDIMSampler.sample."""
        self.make_schedule(S, ddim_eta=eta)
        model = self.model
        if cuda_graph is None:
            cuda_graph = os.environ.get("MODIFF_CUDA_GRAPH", "1") != "0"
        img = x_T
        if img is None:
            raise ValueError("x_T is required (noise is drawn by the caller so shards can be "
                             "re-created)")
        guided = unconditional_conditioning is not None and unconditional_guidance_scale != 1.
        if cuda_graph and hasattr(model, "graphed") and img.is_cuda:
            model = model.graphed()
        b = img.shape[0]
        time_range = np.flip(self.ddim_timesteps)
        total = time_range.shape[0]
        n_eval = [0]

        def model_output(x, step):
            t = torch.full((b,), float(step), dtype=torch.float32, device=x.device)
            if not guided:
                e = model(x, t, conditioning) if conditioning is not None else model(x, t)
                e = e.clone()          # the graphed model and aliased caches reuse their output buffer
            else:
                e_all = model(torch.cat([x] * 2), torch.cat([t] * 2),
                              torch.cat([unconditional_conditioning, conditioning]))
                e = ops.cfg_combine(e_all[:b], e_all[b:], float(unconditional_guidance_scale))
            if eps_callback is not None:
                eps_callback(e, n_eval[0])
            n_eval[0] += 1
            return e

        old_eps = []
        for i, step in enumerate(time_range):
            if max_steps is not None and i >= max_steps:
                break
            index = total - i - 1
            step_next = time_range[min(i + 1, total - 1)]
            s1, s2, s3, sigma, c2 = self._coefficients(index)
            e_t = model_output(img, step)
            # the combinations below are the reference's own tensor expressions, one rounding
            # per operation (plms.py:221-234)
            if len(old_eps) == 0:
                x_prev = ops.ddim_step(img, e_t, s1, s2, s3, 0.0, c2)
                e_t_next = model_output(x_prev, step_next)
                e_prime = (e_t + e_t_next) / 2
            elif len(old_eps) == 1:
                e_prime = (3 * e_t - old_eps[-1]) / 2
            elif len(old_eps) == 2:
                e_prime = (23 * e_t - 16 * old_eps[-1] + 5 * old_eps[-2]) / 12
            else:
                e_prime = (55 * e_t - 59 * old_eps[-1] + 37 * old_eps[-2] - 9 * old_eps[-3]) / 24
            if img_callback is not None:
                img, pred_x0 = ops.ddim_step(img, e_prime, s1, s2, s3, 0.0, c2, want_x0=True)
                img_callback(pred_x0, i)
            else:
                img = ops.ddim_step(img, e_prime, s1, s2, s3, 0.0, c2)
            old_eps.append(e_t)
            if len(old_eps) >= 4:
                old_eps.pop(0)
        if check_status:
            raise_on_device_status()
        return img, {}

