"""Full sampler loops on the GPU against the reference's stored final tensors, at the sizes the
throughput figures are quoted on: the pixel UNet at batch 256 (W4A4 and W4A3, 100 DDIM steps),
the latent UNet over all 500 evaluations of `-c 400`, and the SD-v1 UNet over all 50 guided
evaluations.  The criterion is the final tensor's PSNR against the reference run on the same
seed and random-init weights (formula of trt/benchmark_comparison.py:186-191): at least 40 dB.

Each fixture (tests/golden/full_<case>.npz, written by make_golden.py from the live reference)
also stores how well the reference agrees with ITSELF when its first evaluation is perturbed by
1e-4 of the range (`final_sens_db`).  Where that self-agreement is itself below 43 dB, no
implementation that differs in the last bit anywhere can be expected to reach 40 dB, and the
bound becomes the self-agreement minus 3 dB; the test prints both figures.
"""
import os

import numpy as np
import pytest
import torch

import cases
import oracle

pytestmark = pytest.mark.gpu
GOLDEN = os.path.dirname(os.path.abspath(cases.__file__))


def _fixture(name):
    path = os.path.join(GOLDEN, f"full_{name}.npz")
    if not os.path.exists(path):
        pytest.skip(f"{os.path.basename(path)} has not been generated")
    return np.load(path)


def _bound(fx):
    sens = float(fx["final_sens_db"])
    return (40.0 if sens >= 43.0 else sens - 3.0), sens


def _report(name, fx, final):
    ref = fx["final"]
    p = oracle.psnr(ref, final)
    bound, sens = _bound(fx)
    print(f"{name}: final PSNR vs reference {p:.1f} dB (bound {bound:.1f} dB; the reference against "
          f"a perturbed copy of itself: {sens:.1f} dB)")
    assert np.isfinite(final).all()
    assert p >= bound, (p, bound, sens)


@pytest.mark.parametrize("name", ["pixel_w4a4_split_b256_s100", "pixel_w4a3_split_b256_s100"])
def test_pixel_unet_at_the_benchmarked_batch(cuda, name):
    """Batch 256: per-tensor dynamic scales depend on the whole batch, and the 256-pixel-tile /
    many-wave paths of the GEMM and quantiser kernels only run at this size."""
    import modiff_b200 as m
    c = next(f for f in cases.FULL_CASES if f["name"] == name)
    fx = _fixture(name)
    torch.manual_seed(0)
    net = m.Model(m.make_config(split_shortcut=c["split"])).eval()
    wq, aq = cases.quant_params(c)
    qnn = m.QuantModel(net, wq, aq, sm_abit=8, modulate=True).to(cuda).eval()
    qnn.set_quant_state(True, True)
    qnn.reset_cache()
    betas = torch.from_numpy(m.get_beta_schedule()).float()
    xs, _ = m.generalized_steps(cases.unet_noise(c).to(cuda), cases.unet_sequence(c), qnn, betas,
                                eta=0.0)
    _report(name, fx, xs[-1].cpu().numpy())


def test_latent_unet_all_500_evaluations(cuda):
    import modiff_b200 as m
    c = next(f for f in cases.FULL_CASES if f["name"] == "ldm_w8a8_b2_full")
    fx = _fixture(c["name"])
    torch.manual_seed(0)
    net = m.UNetModel(**cases.LDM_CONFIG).eval()
    m.rerandomize_zero_tensors(net, seed=c["zero_seed"])
    wq, aq = cases.quant_params(c)
    qnn = m.QuantModel(net, wq, aq, sm_abit=8, modulate=True).to(cuda).eval()
    qnn.set_quant_state(True, True)
    qnn.set_grad_ckpt(False)
    qnn.reset_cache()
    sampler = m.DDIMSampler(qnn, **cases.LDM_SCHEDULE)
    final, _ = sampler.sample(c["ddim_steps"], c["batch"], (4, 32, 32), eta=0.0,
                              x_T=cases.ldm_noise(c).to(cuda))
    assert len(sampler.ddim_timesteps) == 500
    _report(c["name"], fx, final.cpu().numpy())


def test_sd_unet_all_50_guided_evaluations(cuda):
    import modiff_b200 as m
    c = next(f for f in cases.FULL_CASES if f["name"] == "sd_w8a8_b1_full")
    fx = _fixture(c["name"])
    torch.manual_seed(0)
    net = m.UNetModel(**cases.SD_CONFIG).eval()
    m.rerandomize_zero_tensors(net, seed=c["zero_seed"])
    wq, aq = cases.quant_params(c)
    qnn = m.QuantModel(net, wq, aq, sm_abit=8, modulate=True).to(cuda).eval()
    qnn.set_quant_state(True, True)
    qnn.set_grad_ckpt(False)
    qnn.reset_cache()
    x, cond, uncond = cases.sd_inputs(c)
    sampler = m.DDIMSampler(qnn, **cases.SD_SCHEDULE)
    final, _ = sampler.sample(c["ddim_steps"], c["batch"], tuple(x.shape[1:]), eta=0.0,
                              conditioning=cond.to(cuda), x_T=x.to(cuda),
                              unconditional_guidance_scale=c["guidance"],
                              unconditional_conditioning=uncond.to(cuda))
    assert len(sampler.ddim_timesteps) == 50
    _report(c["name"], fx, final.cpu().numpy())


@pytest.mark.parametrize("kind", ["pixel_w8a8_b8", "ldm_full", "sd_full"])
def test_int8_attention_full_runs(cuda, kind, golden_unet):
    """The same full loops with the integer attention kernel switched on (QuantModel kwarg
    int8_attention=True).  The reference's attention is floating point, so this is NOT a parity
    test of the reference path: it records what applying the q / k / v / softmax quantisers
    costs in PSNR against the reference's samples and requires a sane result."""
    import modiff_b200 as m
    if kind == "pixel_w8a8_b8":
        c = next(u for u in cases.UNET_CASES if u["name"] == "w8a8_b8_s100")
        torch.manual_seed(0)
        net = m.Model(m.make_config(split_shortcut=c["split"])).eval()
        wq, aq = cases.quant_params(c)
        qnn = m.QuantModel(net, wq, aq, sm_abit=8, modulate=True, int8_attention=True).to(cuda).eval()
        qnn.set_quant_state(True, True)
        qnn.reset_cache()
        betas = torch.from_numpy(m.get_beta_schedule()).float()
        xs, _ = m.generalized_steps(cases.unet_noise(c).to(cuda), cases.unet_sequence(c), qnn, betas,
                                    eta=0.0)
        final, ref = xs[-1].cpu().numpy(), golden_unet[c["name"] + "/final"]
    else:
        sd = kind == "sd_full"
        c = next(f for f in cases.FULL_CASES if f["name"] == ("sd_w8a8_b1_full" if sd else
                                                                "ldm_w8a8_b2_full"))
        fx = _fixture(c["name"])
        torch.manual_seed(0)
        net = m.UNetModel(**(cases.SD_CONFIG if sd else cases.LDM_CONFIG)).eval()
        m.rerandomize_zero_tensors(net, seed=c["zero_seed"])
        wq, aq = cases.quant_params(c)
        qnn = m.QuantModel(net, wq, aq, sm_abit=8, modulate=True, int8_attention=True).to(cuda).eval()
        qnn.set_quant_state(True, True)
        qnn.set_grad_ckpt(False)
        qnn.reset_cache()
        sampler = m.DDIMSampler(qnn, **(cases.SD_SCHEDULE if sd else cases.LDM_SCHEDULE))
        if sd:
            x, cond, uncond = cases.sd_inputs(c)
            final, _ = sampler.sample(c["ddim_steps"], c["batch"], tuple(x.shape[1:]), eta=0.0,
                                      conditioning=cond.to(cuda), x_T=x.to(cuda),
                                      unconditional_guidance_scale=c["guidance"],
                                      unconditional_conditioning=uncond.to(cuda))
        else:
            final, _ = sampler.sample(c["ddim_steps"], c["batch"], (4, 32, 32), eta=0.0,
                                      x_T=cases.ldm_noise(c).to(cuda))
        final, ref = final.cpu().numpy(), fx["final"]
    p = oracle.psnr(ref, final)
    print(f"{kind} with int8 attention: final PSNR vs the reference (fp attention) {p:.1f} dB")
    assert np.isfinite(final).all() and p >= 15.0, p
