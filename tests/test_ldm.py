"""Latent UNet (LSUN-churches kl-8 shapes): oracle vs the reference's fixtures (CPU) and the CUDA
path vs the same fixtures (GPU).  W8A8 modulated, symmetric dynamic activations, random init
seed 0 with the zero-initialised tensors redrawn by `rerandomize_zero_tensors`."""
import os

import numpy as np
import pytest
import torch

import cases
import oracle
from conftest import sens_floor
from oracle.ldm import OracleLDMUNet, ldm_schedule, latent_ddim_sample

GOLDEN = os.path.dirname(os.path.abspath(cases.__file__))


@pytest.fixture(scope="module")
def golden_ldm():
    return np.load(os.path.join(GOLDEN, "ldm.npz"))


def _build():
    import modiff_b200 as m
    torch.manual_seed(0)
    net = m.UNetModel(**cases.LDM_CONFIG).eval()
    m.rerandomize_zero_tensors(net, seed=cases.LDM_CASES[0]["zero_seed"])
    return net


def test_structure_matches_reference_counts():
    """295 M parameters, 168 quantised layers, 21 attention blocks, 206 zero-initialised tensors
    (the figures measured on the reference model)."""
    import modiff_b200 as m
    torch.manual_seed(0)
    net = m.UNetModel(**cases.LDM_CONFIG)
    assert sum(p.numel() for p in net.parameters()) == 294966916
    assert m.rerandomize_zero_tensors(net) == 206
    wq, aq = cases.quant_params(cases.LDM_CASES[0])
    q = m.QuantModel(net, wq, aq, sm_abit=8, modulate=True)
    assert sum(isinstance(x, m.QuantModule) for x in q.modules()) == 168
    assert sum(type(x).__name__ == "QuantQKMatMul" for x in q.modules()) == 21
    assert sum(type(x).__name__ == "QuantResBlock" for x in q.modules()) == 35


def test_ddim_schedule_rule():
    from modiff_b200.ldm_sampler import make_ddim_timesteps
    ts = make_ddim_timesteps("uniform", 400, 1000)
    assert len(ts) == 500 and ts[0] == 1 and ts[-1] == 999      # c = 1000 // 400 = 2
    assert len(make_ddim_timesteps("uniform", 50, 1000)) == 50


@pytest.mark.parametrize("c", cases.LDM_CASES, ids=lambda c: c["name"])
def test_oracle_matches_reference(c, golden_ldm):
    net = _build()
    state = {k: v.detach().clone() for k, v in net.state_dict().items()}
    o = OracleLDMUNet(state, cases.LDM_CONFIG, c["w_bits"], c["a_bits"], c.get("a_sym", True))
    eps = []
    final = latent_ddim_sample(cases.ldm_noise(c), o.forward, ldm_schedule(**cases.LDM_SCHEDULE),
                               c["ddim_steps"], max_evals=3,
                               on_step=lambda i, e, im: eps.append(e.numpy().copy()))
    ref0 = golden_ldm[c["name"] + "/eps0"]
    assert np.abs(eps[0] - ref0).max() < 1e-4 * np.abs(ref0).max()
    for i in (1, 2):
        assert oracle.psnr(golden_ldm[f"{c['name']}/eps{i}"], eps[i]) > 40.0


@pytest.mark.gpu
@pytest.mark.parametrize("c", cases.LDM_CASES, ids=lambda c: c["name"])
def test_cuda_path_matches_reference(c, cuda, golden_ldm, golden_sens):
    import modiff_b200 as m
    net = _build()
    wq, aq = cases.quant_params(c)
    qnn = m.QuantModel(net, wq, aq, sm_abit=8, modulate=True).to(cuda).eval()
    qnn.set_quant_state(True, True)
    qnn.set_grad_ckpt(False)
    qnn.reset_cache()
    sampler = m.DDIMSampler(qnn, **cases.LDM_SCHEDULE)
    eps = []
    final, _ = sampler.sample(c["ddim_steps"], c["batch"], (4, 32, 32), eta=0.0,
                              x_T=cases.ldm_noise(c).to(cuda), max_evals=c["evals"],
                              eps_callback=lambda e, i: eps.append(e.clone()))
    torch.cuda.synchronize()
    assert m.device_status() == 0
    for i, e in enumerate(eps):
        ref = golden_ldm[f"{c['name']}/eps{i}"]
        err = np.abs(e.cpu().numpy() - ref).max() / np.abs(ref).max()
        p = oracle.psnr(ref, e.cpu().numpy())
        print(f"ldm eval {i}: max|eps-ref|/max|ref| = {err:.2e}, PSNR {p:.1f} dB")
        if i == 0:
            assert err < 1e-4, err       # unquantised first evaluation
        else:
            # the reference's own self-agreement at this evaluation minus a margin
            floor_db = sens_floor(golden_sens, c["name"], i)
            assert p >= floor_db, (i, p, floor_db)
    ref = golden_ldm[c["name"] + "/final"]
    assert oracle.psnr(ref, final.cpu().numpy()) >= 40.0


# ---------------------------------------------------------------- PLMS (txt2img.py --plms)
@pytest.fixture(scope="module")
def golden_plms():
    return np.load(os.path.join(GOLDEN, "plms.npz"))


def test_plms_oracle_matches_reference(golden_plms):
    """Two PLMS steps (three evaluations: the first step evaluates twice) of the oracle UNet
    under the oracle's PLMS loop against the reference QuantModel under the same loop."""
    from oracle.ldm import latent_plms_sample
    c = cases.PLMS_CASES[0]
    net = _build()
    state = {k: v.detach().clone() for k, v in net.state_dict().items()}
    o = OracleLDMUNet(state, cases.LDM_CONFIG, c["w_bits"], c["a_bits"])
    eps = []
    latent_plms_sample(cases.ldm_noise(c), o.forward, ldm_schedule(**cases.LDM_SCHEDULE),
                       c["ddim_steps"], max_steps=2, on_eval=lambda k, e: eps.append(e.numpy().copy()))
    assert len(eps) == 3
    ref0 = golden_plms[c["name"] + "/eps0"]
    assert np.abs(eps[0] - ref0).max() < 1e-4 * np.abs(ref0).max()
    for i in (1, 2):
        assert oracle.psnr(golden_plms[f"{c['name']}/eps{i}"], eps[i]) > 40.0


def test_plms_update_is_ddim_with_combined_eps():
    """The PLMS loop on a model whose eps is a known function: every step's update equals the
    DDIM update applied to the Adams-Bashforth combination (plms.py:221-236)."""
    from oracle.ldm import latent_plms_sample, ddim_parameters
    ac = ldm_schedule(**cases.LDM_SCHEDULE)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 4, 8, 8, generator=g)
    calls = []

    def model(xx, t):
        calls.append(int(t[0]))
        return 0.1 * xx + float(t[0]) * 1e-4

    out = latent_plms_sample(x, model, ac, 50, max_steps=4)
    ts, alphas, alphas_prev = ddim_parameters(ac, 50)
    tr = np.flip(ts)
    assert calls == [int(tr[0]), int(tr[1]), int(tr[1]), int(tr[2]), int(tr[3])]
    # replay by hand
    img, old = x, []
    for i in range(4):
        idx = len(ts) - 1 - i
        a_t, a_p = float(alphas[idx]), float(alphas_prev[idx])

        def step(e, img=img, a_t=a_t, a_p=a_p):
            a_t_, a_p_ = torch.full((2, 1, 1, 1), a_t), torch.full((2, 1, 1, 1), a_p)
            s1 = torch.full((2, 1, 1, 1), float(np.sqrt(1. - alphas)[idx]))
            return a_p_.sqrt() * ((img - s1 * e) / a_t_.sqrt()) + (1. - a_p_).sqrt() * e
        e = model(img, torch.full((2,), int(tr[i])))
        if i == 0:
            e2 = model(step(e), torch.full((2,), int(tr[1])))
            ep = (e + e2) / 2
        elif i == 1:
            ep = (3 * e - old[-1]) / 2
        elif i == 2:
            ep = (23 * e - 16 * old[-1] + 5 * old[-2]) / 12
        else:
            ep = (55 * e - 59 * old[-1] + 37 * old[-2] - 9 * old[-3]) / 24
        img = step(ep)
        old.append(e)
    assert torch.equal(img, out)


@pytest.mark.gpu
def test_plms_cuda_path_matches_reference(cuda, golden_plms, golden_sens):
    import modiff_b200 as m
    c = cases.PLMS_CASES[0]
    net = _build()
    wq, aq = cases.quant_params(c)
    qnn = m.QuantModel(net, wq, aq, sm_abit=8, modulate=True).to(cuda).eval()
    qnn.set_quant_state(True, True)
    qnn.set_grad_ckpt(False)
    qnn.reset_cache()
    sampler = m.PLMSSampler(qnn, **cases.LDM_SCHEDULE)
    eps = []
    final, _ = sampler.sample(c["ddim_steps"], c["batch"], (4, 32, 32), eta=0.0,
                              x_T=cases.ldm_noise(c).to(cuda), max_steps=c["steps"],
                              eps_callback=lambda e, k: eps.append(e.clone()))
    torch.cuda.synchronize()
    assert m.device_status() == 0
    assert len(eps) == 5
    for i, e in enumerate(eps):
        ref = golden_plms[f"{c['name']}/eps{i}"]
        err = np.abs(e.cpu().numpy() - ref).max() / np.abs(ref).max()
        p = oracle.psnr(ref, e.cpu().numpy())
        print(f"plms eval {i}: max|eps-ref|/max|ref| = {err:.2e}, PSNR {p:.1f} dB")
        if i == 0:
            assert err < 1e-4, err       # unquantised first evaluation
        else:
            floor_db = sens_floor(golden_sens, c["name"], i)
            assert p >= floor_db, (i, p, floor_db)
    assert oracle.psnr(golden_plms[c["name"] + "/final"], final.cpu().numpy()) >= 40.0
    with pytest.raises(ValueError):
        sampler.sample(c["ddim_steps"], c["batch"], (4, 32, 32), eta=0.5,
                       x_T=cases.ldm_noise(c).to(cuda))
