"""Calibration-data generation: the (x_t, t) pairs that Q-Diffusion / MoDiff calibration draws
its samples from (scripts/sample_diffusion_ddim.py:463-536, `Diffusion.generate`), produced by
this package's device-resident sampler.

The reference samples `cali_n` images with the model under calibration, keeps the state and the
timestep that ENTER every `interval`-th sampling step (`interval = timesteps // cali_st`), and
stacks them as xs [cali_st, n, C, H, W] / ts [cali_st, n]; with `--generate residual` it keeps in
addition, for every kept step, the pair of the step before (the same pair for the first two
steps), which is what MoDiff-aware reconstruction needs to form input residuals.  The
reconstruction loops that consume these tensors (qdiff/layer_recon.py, block_recon.py) are
training code and are not part of this package.
"""
import math

import torch

from .sampler import generalized_steps, make_timestep_sequence


def select_calibration_points(xs, ts, interval, cali_st, residual=False):
    """From one sampling run - `xs` the states [x_T, ..., x_0] (one more than steps), `ts` the
    timestep tensors of the steps - the entries the reference keeps
    (scripts/sample_diffusion_ddim.py:492-504): step t is kept when t % interval == 0, in slot
    t // interval; `residual` adds the previous step's pair (steps 0 and 1 repeat themselves).
    Returns lists of length `cali_st`: (x, t) or (x, t, x_prev, t_prev) per slot."""
    keep = [[] for _ in range(cali_st)]
    for t in range(len(ts)):
        if t % interval:
            continue
        slot = t // interval
        if slot >= cali_st:
            raise ValueError(f"step {t} falls into slot {slot} of {cali_st}: timesteps must be "
                             "cali_st * interval")
        entry = [xs[t], ts[t]]
        if residual:
            p = t if t <= 1 else t - 1
            entry += [xs[p], ts[p]]
        keep[slot].append(tuple(entry))
    return keep


@torch.no_grad()
def generate_calibration_data(model, shape, betas, timesteps=100, cali_n=256, cali_st=20,
                              batch_size=64, seed=1234, skip_type="quad", num_timesteps=1000,
                              residual=False, device="cuda", eta=0.0):
    """`Diffusion.generate` (scripts/sample_diffusion_ddim.py:463-536).

    model   callable eps = model(x, t): the UNet whose activations will be calibrated
    shape   (C, H, W) of one sample
    Returns (xs, ts) on the host, xs [cali_st, n, C, H, W], ts [cali_st, n] with
    n = ceil(cali_n / batch_size) * batch_size, or (xs, ts, xs_prev, ts_prev) with `residual`.
    Noise comes from a host generator seeded with `seed` (the reference draws it on the device
    after torch.manual_seed(seed); device generators are not reproducible across machines)."""
    if timesteps % cali_st:
        raise ValueError("timesteps must be a multiple of cali_st")
    interval = timesteps // cali_st
    rounds = math.ceil(cali_n / batch_size)
    seq = make_timestep_sequence(num_timesteps, timesteps, skip_type)
    g = torch.Generator().manual_seed(int(seed))
    slots = [[] for _ in range(cali_st)]
    for _ in range(rounds):
        x = torch.randn((batch_size,) + tuple(shape), generator=g).to(device)
        if hasattr(model, "reset_cache"):
            model.reset_cache()
        xs, ts, _ = generalized_steps(x, seq, model, betas, with_t=True, last_only=False, eta=eta)
        for slot, entries in enumerate(select_calibration_points(xs, ts, interval, cali_st,
                                                                  residual)):
            slots[slot] += [tuple(v.cpu() for v in e) for e in entries]
    width = 4 if residual else 2
    out = []
    for k in range(width):
        out.append(torch.stack([torch.cat([e[k] for e in entries], dim=0) for entries in slots],
                               dim=0))
    return tuple(out)
