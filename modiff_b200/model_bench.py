"""Steady-state time of one UNet evaluation for the latent (LSUN-churches kl-8) and the SD-v1
graphs, random-init weights, W8A8 modulated with symmetric (or, with --asym, asymmetric) dynamic
activation quantisers.

    python -m modiff_b200.model_bench --model ldm --batch 32 --evals 12
    python -m modiff_b200.model_bench --model sd --batch 8 --evals 8     # guidance: 2x effective batch

Prints one JSON line: milliseconds per evaluation (CUDA events over the evaluations after the
first three, which include the unquantised first step and graph capture) and images per second
for a sampler of `--steps` evaluations.  The headline benchmark is `bench.py`; this module only
times the other two model families on the same kernels.
"""
import argparse
import json

import torch

from . import _lib
from .ldm_sampler import DDIMSampler
from .ldm_unet import LSUN_CHURCHES_KL8, SD_V1, UNetModel, rerandomize_zero_tensors
from .quant_model import QuantModel


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=["ldm", "sd"], default="ldm")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--evals", type=int, default=12)
    ap.add_argument("--w-bits", type=int, default=8)
    ap.add_argument("--a-bits", type=int, default=8)
    ap.add_argument("--asym", action="store_true",
                    help="asymmetric activation quantisers (the drivers' default without --a_sym)")
    ap.add_argument("--breakdown", action="store_true",
                    help="also time every entry point with CUDA events (eager; one more evaluation)")
    args = ap.parse_args()
    dev = torch.device("cuda")
    torch.manual_seed(0)
    sd = args.model == "sd"
    cfg = SD_V1 if sd else LSUN_CHURCHES_KL8
    batch = args.batch or (8 if sd else 32)
    latent = 64 if sd else 32
    steps = 50 if sd else 400
    net = UNetModel(**cfg).eval()
    rerandomize_zero_tensors(net)
    wq = {'n_bits': args.w_bits, 'channel_wise': True, 'scale_method': 'max'}
    aq = {'n_bits': args.a_bits, 'symmetric': not args.asym, 'channel_wise': False, 'scale_method': 'max',
          'leaf_param': True, 'dynamic': True}
    qnn = QuantModel(net, wq, aq, sm_abit=8, modulate=True).to(dev).eval()
    qnn.set_quant_state(True, True)
    qnn.set_grad_ckpt(False)
    qnn.reset_cache()
    sched = dict(linear_start=0.00085, linear_end=0.0120) if sd else \
        dict(linear_start=0.0015, linear_end=0.0155)
    sampler = DDIMSampler(qnn, **sched)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(batch, 4, latent, latent, generator=g).to(dev)
    kw = {}
    if sd:
        kw = dict(conditioning=torch.randn(batch, 77, 768, generator=g).to(dev),
                  unconditional_conditioning=torch.randn(batch, 77, 768, generator=g).to(dev),
                  unconditional_guidance_scale=7.5)
    marks = []

    def mark(e, i):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        marks.append(ev)

    sampler.sample(steps, batch, (4, latent, latent), eta=0.0, x_T=x, max_evals=args.evals,
                   eps_callback=mark, **kw)
    torch.cuda.synchronize()
    skip = 3
    ms = marks[skip].elapsed_time(marks[-1]) / (len(marks) - 1 - skip)
    n_evals = steps + 100 if not sd else steps      # `-c 400` walks 500 timesteps (c = 1000 // 400)
    per_entry = None
    if args.breakdown:
        # one more steady-state evaluation, eager, with events around every library call
        qnn_in = torch.cat([x] * 2) if sd else x
        t_in = torch.full((qnn_in.shape[0],), 500.0, device=dev)
        ctx = torch.cat([kw["unconditional_conditioning"], kw["conditioning"]]) if sd else None
        _lib.TIMER = _lib.KernelTimer()
        qnn(qnn_in, t_in, ctx)
        per_entry = {n: round(v["ms"], 2) for n, v in _lib.TIMER.summary().items()}
        _lib.TIMER = None
    print(json.dumps({"model": args.model, "per_entry_point_ms": per_entry, "batch": batch, "effective_batch": batch * (2 if sd else 1),
                      "w_bits": args.w_bits, "a_bits": args.a_bits, "a_sym": not args.asym, "ms_per_eval": ms,
                      "evals_per_sample": n_evals,
                      "images_per_s": batch / (ms * n_evals / 1000.0),
                      "device_status": _lib.device_status()}))


if __name__ == "__main__":
    main()
