"""Generates the golden fixtures in this directory by RUNNING THE REFERENCE (MoDiff's qdiff +
ddim packages, imported read-only from a checkout) on CPU.

    python tests/golden/make_golden.py /path/to/reference [--only layers|unet|weights|quantizer|ldm|plms|sd|cali|running|sens|full|decoder [--case NAME]]

Needs the reference checkout, so it runs where that exists; the fixtures it writes are
committed and are all the tests read.  Inputs and weights are NOT stored: they are re-created
from the seeds recorded in `cases.py` (torch CPU generators), only the reference's outputs are.
"""
import json
import os
import sys
import time
import warnings

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.dont_write_bytecode = True
import cases  # noqa: E402

REF = next((a for a in sys.argv[1:] if not a.startswith("--") and os.path.isdir(a)),
           os.environ.get("MODIFF_REFERENCE", "reference"))
ONLY = sys.argv[sys.argv.index("--only") + 1] if "--only" in sys.argv else None
sys.path.insert(0, REF)
warnings.filterwarnings("ignore", category=SyntaxWarning)

from qdiff.quant_layer import QuantModule as RefQuantModule  # noqa: E402
from qdiff.quant_layer import UniformAffineQuantizer as RefQuantizer  # noqa: E402
from qdiff.quant_model import QuantModel as RefQuantModel  # noqa: E402
from ddim.models.diffusion import Model as RefModel  # noqa: E402
from ddim.functions.denoising import compute_alpha as ref_compute_alpha  # noqa: E402


def ref_config(split_shortcut):
    import yaml
    import argparse

    def ns(d):
        n = argparse.Namespace()
        for k, v in d.items():
            setattr(n, k, ns(v) if isinstance(v, dict) else v)
        return n

    with open(os.path.join(REF, "configs", "cifar10.yml")) as fh:
        cfg = ns(yaml.safe_load(fh))
    cfg.split_shortcut = split_shortcut
    return cfg


def gen_quantizer():
    out = {}
    for c in cases.QUANTIZER_CASES:
        x = cases.quantizer_input(c)
        q = RefQuantizer(n_bits=c["n_bits"], symmetric=c["sym"], channel_wise=c["channel_wise"],
                         scale_method="max", leaf_param=False, always_zero=c.get("always_zero", False),
                         dynamic=True)
        y = q(x)
        out[c["name"] + "/y"] = y.detach().numpy()
        out[c["name"] + "/delta"] = np.asarray(q.delta.detach().numpy(), dtype=np.float32).reshape(-1)
        zp = q.zero_point
        zp = zp.detach().numpy() if isinstance(zp, torch.Tensor) else np.asarray([zp])
        out[c["name"] + "/zp"] = np.asarray(zp, dtype=np.float32).reshape(-1)
    np.savez_compressed(os.path.join(HERE, "quantizer.npz"), **out)
    print("quantizer.npz", len(out))


def gen_layers():
    out = {}
    for c in cases.LAYER_CASES:
        org = cases.layer_module(c)
        wq, aq = cases.quant_params(c)
        m = RefQuantModule(org, wq, aq, modulate=True)
        m.set_quant_state(True, True)
        xs = cases.layer_inputs(c)
        with torch.no_grad():
            for s, x in enumerate(xs):
                if c.get("pad_br"):
                    x = F.pad(x, (0, 1, 0, 1))
                y = m(x, split=c.get("split", 0)) if c.get("split", 0) else m(x)
                out[f"{c['name']}/out{s}"] = y.numpy().copy()
                if s > 0:
                    d = [float(m.act_quantizer.delta)]
                    if c.get("split", 0):
                        d.append(float(m.act_quantizer_0.delta))
                    out[f"{c['name']}/delta{s}"] = np.asarray(d, dtype=np.float32)
                    if not c.get("a_sym", True):
                        z = [float(m.act_quantizer.zero_point)]
                        if c.get("split", 0):
                            z.append(float(m.act_quantizer_0.zero_point))
                        out[f"{c['name']}/zp{s}"] = np.asarray(z, dtype=np.float32)
            if not c.get("skip_a_hat"):
                out[f"{c['name']}/a_hat"] = m.a_hat.numpy().copy()
        wd = m.weight_quantizer.delta.detach().reshape(-1).numpy()
        out[f"{c['name']}/w_delta"] = wd.copy()
        out[f"{c['name']}/w_zp"] = m.weight_quantizer.zero_point.detach().reshape(-1).numpy().copy()
    np.savez_compressed(os.path.join(HERE, "layers.npz"), **out)
    print("layers.npz", len(out))


def gen_weights():
    torch.manual_seed(0)
    model = RefModel(ref_config(False))
    summary = {}
    for k, v in model.state_dict().items():
        v = v.double()
        summary[k] = [list(v.shape), float(v.sum()), float(v.abs().sum()),
                      float((v * torch.arange(1, v.numel() + 1, dtype=torch.float64).reshape(v.shape)
                             ).sum() / v.numel())]
    with open(os.path.join(HERE, "weights_seed0.json"), "w") as fh:
        json.dump(summary, fh)
    print("weights_seed0.json", len(summary))


def ref_sample(qnn, x, seq, betas, on_step=None):
    """ddim/functions/denoising.py:10-55 without its .to('cuda')."""
    n = x.size(0)
    seq_next = [-1] + list(seq[:-1])
    xt = x
    with torch.no_grad():
        for step, (i, j) in enumerate(zip(reversed(seq), reversed(seq_next))):
            t = torch.ones(n) * i
            next_t = torch.ones(n) * j
            at = ref_compute_alpha(betas, t.long())
            at_next = ref_compute_alpha(betas, next_t.long())
            et = qnn(xt, t)
            x0_t = (xt - et * (1 - at).sqrt()) / at.sqrt()
            c2 = (1 - at_next).sqrt()
            xt = at_next.sqrt() * x0_t + c2 * et
            if on_step:
                on_step(step, et, xt)
    return xt


def gen_unet():
    out = {}
    betas = torch.from_numpy(np.linspace(1e-4, 2e-2, 1000, dtype=np.float64)).float()
    for c in cases.UNET_CASES:
        t0 = time.time()
        torch.manual_seed(0)
        model = RefModel(ref_config(c["split"])).eval()
        x = cases.unet_noise(c)
        seq = cases.unet_sequence(c)
        if c["quant"]:
            wq, aq = cases.quant_params(c)
            qnn = RefQuantModel(model=model, weight_quant_params=wq, act_quant_params=aq,
                                sm_abit=8, modulate=True).eval()
            qnn.set_quant_state(True, True)
            qnn.reset_cache()
            fn = qnn
        else:
            fn = lambda a, b: model(a, b)  # noqa: E731
        eps = []

        def grab(step, et, xt):
            if step < c.get("keep_eps", 0):
                eps.append(et.numpy().copy())

        final = ref_sample(fn, x, seq, betas, grab)
        out[c["name"] + "/final"] = final.numpy().copy()
        for s, e in enumerate(eps):
            out[f"{c['name']}/eps{s}"] = e
        print(c["name"], f"{time.time() - t0:.1f}s", float(final.std()))
    np.savez_compressed(os.path.join(HERE, "unet.npz"), **out)
    print("unet.npz", len(out))


def gen_ldm():
    """Latent UNet (LSUN-churches kl-8 shapes, random init seed 0, zero-initialised tensors redrawn
    by modiff_b200.ldm_unet.rerandomize_zero_tensors), reference QuantModel with --a_sym."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from modiff_b200.ldm_unet import rerandomize_zero_tensors
    from oracle.ldm import ldm_schedule, latent_ddim_sample
    from ldm.modules.diffusionmodules.openaimodel import UNetModel as RefUNet
    out = {}
    ac = ldm_schedule(**cases.LDM_SCHEDULE)
    for c in cases.LDM_CASES:
        t0 = time.time()
        torch.manual_seed(0)
        model = RefUNet(**cases.LDM_CONFIG).eval()
        rerandomize_zero_tensors(model, seed=c["zero_seed"])
        wq, aq = cases.quant_params(c)
        qnn = RefQuantModel(model=model, weight_quant_params=wq, act_quant_params=aq, sm_abit=8,
                            modulate=True).eval()
        qnn.set_quant_state(True, True)
        qnn.set_grad_ckpt(False)
        qnn.reset_cache()
        eps = []
        final = latent_ddim_sample(cases.ldm_noise(c), lambda a, t: qnn(a, t), ac, c["ddim_steps"],
                                   max_evals=c["evals"],
                                   on_step=lambda i, e, im: eps.append(e.numpy().copy()))
        out[c["name"] + "/final"] = final.numpy().copy()
        for i, e in enumerate(eps):
            out[f"{c['name']}/eps{i}"] = e
        print(c["name"], f"{time.time() - t0:.1f}s", float(final.std()))
    np.savez_compressed(os.path.join(HERE, "ldm.npz"), **out)
    print("ldm.npz", len(out))


def gen_plms():
    """The latent UNet of gen_ldm under the PLMS loop (ldm/models/diffusion/plms.py:114-240)."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from modiff_b200.ldm_unet import rerandomize_zero_tensors
    from oracle.ldm import ldm_schedule, latent_plms_sample
    from ldm.modules.diffusionmodules.openaimodel import UNetModel as RefUNet
    out = {}
    ac = ldm_schedule(**cases.LDM_SCHEDULE)
    for c in cases.PLMS_CASES:
        t0 = time.time()
        torch.manual_seed(0)
        model = RefUNet(**cases.LDM_CONFIG).eval()
        rerandomize_zero_tensors(model, seed=c["zero_seed"])
        wq, aq = cases.quant_params(c)
        qnn = RefQuantModel(model=model, weight_quant_params=wq, act_quant_params=aq, sm_abit=8,
                            modulate=True).eval()
        qnn.set_quant_state(True, True)
        qnn.set_grad_ckpt(False)
        qnn.reset_cache()
        eps = []
        final = latent_plms_sample(cases.ldm_noise(c), lambda a, t: qnn(a, t), ac, c["ddim_steps"],
                                   max_steps=c["steps"],
                                   on_eval=lambda k, e: eps.append(e.numpy().copy()))
        out[c["name"] + "/final"] = final.numpy().copy()
        for i, e in enumerate(eps):
            out[f"{c['name']}/eps{i}"] = e
        print(c["name"], f"{time.time() - t0:.1f}s", len(eps), float(final.std()))
    np.savez_compressed(os.path.join(HERE, "plms.npz"), **out)
    print("plms.npz", len(out))


def gen_cali():
    """Calibrated-checkpoint path: reference QuantModel with non-dynamic activation quantisers,
    weight quantisers converted to AdaRound, a synthetic checkpoint loaded by the steps of
    qdiff/utils.py:542-628 (its .cuda() calls left out), then modulated sampling."""
    from qdiff.utils import convert_adaround
    from qdiff.adaptive_rounding import AdaRoundQuantizer
    out = {}
    betas = torch.from_numpy(np.linspace(1e-4, 2e-2, 1000, dtype=np.float64)).float()

    def params_on(qnn, also_act):
        for m in qnn.model.modules():
            if isinstance(m, AdaRoundQuantizer):
                m.zero_point = nn.Parameter(m.zero_point)
                m.delta = nn.Parameter(m.delta)
            elif also_act and isinstance(m, RefQuantizer) and m.zero_point is not None:
                zp = m.zero_point
                m.zero_point = nn.Parameter(zp if torch.is_tensor(zp) else torch.tensor(float(zp)))

    def params_off(qnn, also_act):
        for m in qnn.model.modules():
            if isinstance(m, AdaRoundQuantizer):
                z, d = m.zero_point.data, m.delta.data
                delattr(m, "zero_point")
                delattr(m, "delta")
                m.zero_point, m.delta = z, d
            elif also_act and isinstance(m, RefQuantizer) and m.zero_point is not None:
                z = m.zero_point.item()
                delattr(m, "zero_point")
                assert int(z) == z
                m.zero_point = int(z)

    for c in cases.CALI_CASES:
        t0 = time.time()
        wq, aq = cases.quant_params(c)
        x = cases.unet_noise(c)
        seq = cases.cali_sequence(c)

        # plausible activation scales: those of a dynamic run at its third evaluation
        torch.manual_seed(0)
        qd = RefQuantModel(model=RefModel(ref_config(c["split"])).eval(), weight_quant_params=wq,
                           act_quant_params=dict(aq), sm_abit=8, modulate=True).eval()
        qd.set_quant_state(True, True)
        qd.reset_cache()
        ref_sample(qd, x, seq[-3:], betas)
        scales = {}
        for name, m in qd.named_modules():
            if isinstance(m, RefQuantModule):
                for slot in ("act_quantizer", "act_quantizer_0"):
                    q = getattr(m, slot, None)
                    if q is not None and q.delta is not None:
                        scales[f"{name}.{slot}"] = (float(q.delta) * c["scale_margin"],
                                                    float(q.zero_point))
        del qd

        torch.manual_seed(0)
        model = RefModel(ref_config(c["split"])).eval()
        qnn = RefQuantModel(model=model, weight_quant_params=wq,
                            act_quant_params=dict(aq, dynamic=False), sm_abit=8,
                            modulate=True).eval()
        cx, ct = cases.cali_data(c)
        with torch.no_grad():
            qnn.set_quant_state(True, False)
            qnn(cx, ct)
            convert_adaround(qnn)
            params_on(qnn, False)
            qnn.set_quant_state(True, True)
            qnn(cx, ct)
            qnn(cx, ct)
            params_on_act = True
            params_off(qnn, False)
            params_on(qnn, params_on_act)
        sd = qnn.state_dict()
        keys = [[k, list(v.shape)] for k, v in sd.items()]
        ckpt = {}
        for k, v in sd.items():
            if k.endswith(".alpha"):
                ckpt[k] = cases.cali_alpha(k, v.shape, c["alpha_seed"])
                continue
            ckpt[k] = v.detach().clone()
            parts = k.split(".")
            if parts[-2].startswith("act_quantizer"):
                d, z = scales[".".join(parts[:-1])]
                ckpt[k] = torch.tensor(d if parts[-1] == "delta" else z, dtype=torch.float32)
            if parts[-2].startswith(("act_quantizer", "weight_quantizer")):
                out[f"{c['name']}/ckpt/{k}"] = ckpt[k].numpy().copy()
        out[c["name"] + "/keys"] = np.asarray(json.dumps(keys))
        # weights-only load (strict), then the full load, as the reference does in two stages
        qnn.load_state_dict(ckpt, strict=True)
        params_off(qnn, True)
        qnn.set_quant_state(True, True)
        qnn.reset_cache()
        eps = []

        def grab(step, et, xt):
            eps.append(et.numpy().copy())

        final = ref_sample(qnn, x, seq, betas, grab)
        out[c["name"] + "/final"] = final.numpy().copy()
        for s, e in enumerate(eps):
            out[f"{c['name']}/eps{s}"] = e
        print(c["name"], f"{time.time() - t0:.1f}s", len(keys), "keys", float(final.std()))
    np.savez_compressed(os.path.join(HERE, "cali.npz"), **out)
    print("cali.npz", len(out))


def gen_running():
    """Single layers with moving-average activation ranges (`--running_stat`)."""
    out = {}
    for name in cases.RUNNING_CASES:
        c = next(x for x in cases.LAYER_CASES if x["name"] == name)
        org = cases.layer_module(c)
        wq, aq = cases.quant_params(c)
        m = RefQuantModule(org, wq, dict(aq, dynamic=False), modulate=True)
        m.set_quant_state(True, True)
        with torch.no_grad():
            for s, x in enumerate(cases.running_inputs(c)):
                if c.get("pad_br"):
                    x = F.pad(x, (0, 1, 0, 1))
                m.set_running_stat(s in (2, 3, 4))
                y = m(x, split=c.get("split", 0)) if c.get("split", 0) else m(x)
                if s >= 4:
                    out[f"{name}/out{s}"] = y.numpy().copy()
                if s > 0:
                    qs = [m.act_quantizer] + ([m.act_quantizer_0] if c.get("split", 0) else [])
                    out[f"{name}/delta{s}"] = np.asarray([float(q.delta) for q in qs], np.float32)
                    out[f"{name}/zp{s}"] = np.asarray([float(q.zero_point) for q in qs], np.float32)
                    out[f"{name}/range{s}"] = np.asarray(
                        [[float(q.x_min), float(q.x_max)] for q in qs], np.float32)
        out[f"{name}/a_hat"] = m.a_hat.numpy().copy()
    np.savez_compressed(os.path.join(HERE, "running.npz"), **out)
    print("running.npz", len(out))


def gen_sd():
    """SD-v1 UNet shapes (random init seed 0, zero tensors redrawn), reference QuantModel with
    --a_sym, classifier-free guidance as ldm/models/diffusion/ddim.py:192-208."""
    import types
    oc, lc = types.ModuleType('omegaconf'), types.ModuleType('omegaconf.listconfig')

    class ListConfig(list):
        pass

    lc.ListConfig = ListConfig
    oc.listconfig = lc
    sys.modules.setdefault('omegaconf', oc)
    sys.modules.setdefault('omegaconf.listconfig', lc)
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from modiff_b200.ldm_unet import rerandomize_zero_tensors
    from oracle.ldm import ldm_schedule, latent_ddim_sample
    from ldm.modules.diffusionmodules.openaimodel import UNetModel as RefUNet
    out = {}
    ac = ldm_schedule(**cases.SD_SCHEDULE)
    for c in cases.SD_CASES:
        t0 = time.time()
        torch.manual_seed(0)
        model = RefUNet(**cases.SD_CONFIG).eval()
        rerandomize_zero_tensors(model, seed=c["zero_seed"])
        wq, aq = cases.quant_params(c)
        qnn = RefQuantModel(model=model, weight_quant_params=wq, act_quant_params=aq, sm_abit=8,
                            modulate=True).eval()
        qnn.set_quant_state(True, True)
        qnn.set_grad_ckpt(False)
        qnn.reset_cache()
        x, cond, uncond = cases.sd_inputs(c)
        eps = []
        final = latent_ddim_sample(x, lambda a, t, ctx: qnn(a, t, ctx), ac, c["ddim_steps"],
                                   max_evals=c["evals"], cond=cond, uncond=uncond,
                                   guidance=c["guidance"],
                                   on_step=lambda i, e, im: eps.append(e.numpy().copy()))
        out[c["name"] + "/final"] = final.numpy().copy()
        for i, e in enumerate(eps):
            out[f"{c['name']}/eps{i}"] = e
        print(c["name"], f"{time.time() - t0:.1f}s", float(final.std()))
    np.savez_compressed(os.path.join(HERE, "sd.npz"), **out)
    print("sd.npz", len(out))


def _psnr(a, b):
    """trt/benchmark_comparison.py:186-191."""
    a = np.asarray(a, dtype=np.float32).ravel()
    b = np.asarray(b, dtype=np.float32).ravel()
    mse = np.mean((a - b) ** 2)
    peak = max(np.abs(a).max(), np.abs(b).max())
    return float(20 * np.log10(peak / np.sqrt(mse))) if mse > 0 and peak > 0 else float("inf")


def _sd_stub():
    import types
    oc, lc = types.ModuleType('omegaconf'), types.ModuleType('omegaconf.listconfig')

    class ListConfig(list):
        pass

    lc.ListConfig = ListConfig
    oc.listconfig = lc
    sys.modules.setdefault('omegaconf', oc)
    sys.modules.setdefault('omegaconf.listconfig', lc)


def _runner(c):
    """`run(perturbed, on_eval) -> final` for any case: builds the reference model once; every
    run starts from reset caches.  `on_eval(i, eps, x)` sees each evaluation."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    kind = c.get("kind", "pixel")
    wq, aq = cases.quant_params(c)
    if kind == "pixel":
        betas = torch.from_numpy(np.linspace(1e-4, 2e-2, 1000, dtype=np.float64)).float()
        torch.manual_seed(0)
        qnn = RefQuantModel(model=RefModel(ref_config(c["split"])).eval(), weight_quant_params=wq,
                            act_quant_params=aq, sm_abit=8, modulate=True).eval()
        qnn.set_quant_state(True, True)

        def run(perturbed, on_eval=None):
            qnn.reset_cache()
            fn = cases.perturb_first_call(qnn) if perturbed else qnn
            return ref_sample(fn, cases.unet_noise(c), cases.unet_sequence(c), betas, on_eval)
        return run
    from modiff_b200.ldm_unet import rerandomize_zero_tensors
    from oracle.ldm import ldm_schedule, latent_ddim_sample, latent_plms_sample
    if kind == "sd":
        _sd_stub()
    from ldm.modules.diffusionmodules.openaimodel import UNetModel as RefUNet
    torch.manual_seed(0)
    model = RefUNet(**(cases.SD_CONFIG if kind == "sd" else cases.LDM_CONFIG)).eval()
    rerandomize_zero_tensors(model, seed=c["zero_seed"])
    qnn = RefQuantModel(model=model, weight_quant_params=wq, act_quant_params=aq, sm_abit=8,
                        modulate=True).eval()
    qnn.set_quant_state(True, True)
    qnn.set_grad_ckpt(False)
    ac = ldm_schedule(**(cases.SD_SCHEDULE if kind == "sd" else cases.LDM_SCHEDULE))

    def run(perturbed, on_eval=None):
        qnn.reset_cache()
        if kind == "sd":
            x, cond, uncond = cases.sd_inputs(c)
            fn = lambda a, t, ctx: qnn(a, t, ctx)  # noqa: E731
            fn = cases.perturb_first_call(fn) if perturbed else fn
            return latent_ddim_sample(x, fn, ac, c["ddim_steps"], max_evals=c.get("evals"),
                                      cond=cond, uncond=uncond, guidance=c["guidance"],
                                      on_step=on_eval)
        fn = lambda a, t: qnn(a, t)  # noqa: E731
        fn = cases.perturb_first_call(fn) if perturbed else fn
        if kind == "plms":
            return latent_plms_sample(cases.ldm_noise(c), fn, ac, c["ddim_steps"],
                                      max_steps=c["steps"],
                                      on_eval=(lambda k, e: on_eval(k, e, None)) if on_eval else None)
        return latent_ddim_sample(cases.ldm_noise(c), fn, ac, c["ddim_steps"],
                                  max_evals=c.get("evals"), on_step=on_eval)
    return run


def _sens(run, keep):
    """Runs the reference twice (second time with the first evaluation perturbed, cases.SENS_REL)
    and returns (final, kept trajectory points, per-evaluation PSNR between the runs, PSNR of
    the finals)."""
    base, kept = [], {}

    def on_base(i, e, x):
        base.append(e.numpy().copy())
        if i in keep and x is not None:
            kept[i] = x.numpy().copy()

    final = run(False, on_base)
    db = []
    final_p = run(True, lambda i, e, x: db.append(_psnr(base[i], e.numpy())))
    return final, kept, np.asarray(db, dtype=np.float32), _psnr(final.numpy(), final_p.numpy())


def gen_sens():
    """Self-sensitivity of the reference on the short whole-model cases (sens.npz)."""
    out = {}
    todo = [dict(c, kind="pixel") for c in cases.UNET_CASES if c["quant"]]
    todo += [dict(c, kind="ldm") for c in cases.LDM_CASES]
    todo += [dict(c, kind="plms") for c in cases.PLMS_CASES]
    todo += [dict(c, kind="sd") for c in cases.SD_CASES]
    for c in todo:
        t0 = time.time()
        _, _, db, fin = _sens(_runner(c), ())
        out[c["name"] + "/sens_db"] = db
        out[c["name"] + "/final_sens_db"] = np.float32(fin)
        print(c["name"], f"{time.time() - t0:.1f}s", np.round(db[:12], 1), round(fin, 1), flush=True)
        np.savez_compressed(os.path.join(HERE, "sens.npz"), **out)
    print("sens.npz", len(out))


def gen_full():
    """Full-length sampler loops (cases.FULL_CASES), one file per case: the final tensor, the
    state after a few evaluations, and the reference's self-sensitivity along the whole run.
    `--case NAME` limits the run to one case."""
    pick = sys.argv[sys.argv.index("--case") + 1] if "--case" in sys.argv else None
    for c in cases.FULL_CASES:
        if pick not in (None, c["name"]):
            continue
        t0 = time.time()
        n = {"pixel": c.get("steps"), "ldm": 500, "sd": c.get("ddim_steps")}[c["kind"]]
        keep = sorted({n // 10, n // 4, n // 2, 3 * n // 4})
        final, kept, db, fin = _sens(_runner(c), keep)
        out = {"final": final.numpy().copy(), "sens_db": db, "final_sens_db": np.float32(fin)}
        if c.get("batch", 1) < 64:          # batch-256 cases keep the final tensor only (3 MB)
            for i, x in kept.items():
                out[f"x_after{i}"] = x
        np.savez_compressed(os.path.join(HERE, f"full_{c['name']}.npz"), **out)
        print(c["name"], f"{time.time() - t0:.1f}s", float(final.std()), "final sens", round(fin, 1),
              "min sens", float(db.min()), flush=True)


def gen_decoder():
    """First-stage decoder: the reference's own Decoder (ldm/modules/diffusionmodules/model.py)
    behind a 1x1 post_quant_conv as AutoencoderKL.decode composes them
    (ldm/models/autoencoder.py:299-333; that class itself needs pytorch_lightning)."""
    from ldm.modules.diffusionmodules.model import Decoder as RefDecoder
    c = cases.DECODER_CASE
    torch.manual_seed(c["init_seed"])
    dec = RefDecoder(**cases.DECODER_CONFIG).eval()
    pqc = nn.Conv2d(c["embed_dim"], cases.DECODER_CONFIG["z_channels"], 1)
    z = cases.decoder_latents(c)
    with torch.no_grad():
        y = dec(pqc(z))
    out = {c["name"] + "/image": y.numpy().copy(),
           c["name"] + "/param_sum": np.float64(sum(float(p.double().sum()) for p in
                                                    list(dec.parameters()) + list(pqc.parameters())))}
    np.savez_compressed(os.path.join(HERE, "decoder.npz"), **out)
    print("decoder.npz", tuple(y.shape), float(y.std()))


if __name__ == "__main__":
    torch.set_num_threads(int(os.environ.get("MODIFF_GOLDEN_THREADS", os.cpu_count())))
    todo = dict(quantizer=gen_quantizer, layers=gen_layers, weights=gen_weights, unet=gen_unet,
                ldm=gen_ldm, plms=gen_plms, sd=gen_sd, cali=gen_cali, running=gen_running,
                sens=gen_sens, full=gen_full, decoder=gen_decoder)
    for name, fn in todo.items():
        if ONLY in (None, name):
            fn()
