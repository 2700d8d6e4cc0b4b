"""Calibrated-checkpoint path: AdaRound weight quantisers and static (quant_mode 'qdiff')
activation scales loaded from a checkpoint in the reference's format (qdiff/utils.py:542-628,
qdiff/adaptive_rounding.py:39-61).  The fixture `cali.npz` holds what the reference QuantModel
produced after loading the synthetic checkpoint that `cases.cali_checkpoint` rebuilds here."""
import os

import numpy as np
import pytest
import torch

import cases
import oracle
from oracle.quantizer import adaround_codes, weight_codes

GOLDEN = os.path.dirname(os.path.abspath(cases.__file__))


@pytest.fixture(scope="module")
def golden_cali():
    return np.load(os.path.join(GOLDEN, "cali.npz"))


def _float_state(split):
    import modiff_b200 as m
    torch.manual_seed(0)
    return {k: v.detach().clone()
            for k, v in m.Model(m.make_config(split_shortcut=split)).state_dict().items()}


def test_adaround_with_initial_logits_is_round_to_nearest():
    """sigmoid(alpha) = frac(w / delta) at initialisation (adaptive_rounding.py:66-74), so the
    hard target alpha >= 0 reproduces round-half-up of w / delta: equal to the uniform
    quantiser's codes except exactly at ties."""
    g = torch.Generator().manual_seed(5)
    w = torch.randn(16, 8, 3, 3, generator=g)
    _, q, delta, zp = weight_codes(w, 4)
    rest = w / delta - torch.floor(w / delta)
    alpha = -torch.log(1.2 / (rest + 0.1) - 1)
    _, qa, _, _ = adaround_codes(w, alpha, delta, zp, 4)
    assert torch.equal(q, qa)


@pytest.mark.parametrize("c", cases.CALI_CASES, ids=lambda c: c["name"])
def test_oracle_loads_checkpoint_like_reference(c, golden_cali):
    name = c["name"]
    ckpt = cases.cali_checkpoint(c, _float_state(c["split"]), golden_cali, name)
    state = {k[len("model."):]: v for k, v in ckpt.items()
             if ".weight_quantizer" not in k and ".act_quantizer" not in k}
    net = oracle.OracleUNet(state, w_bits=c["w_bits"], a_bits=c["a_bits"], a_sym=c["a_sym"],
                            split_shortcut=c["split"], a_dynamic=False)
    net.load_calibrated(ckpt)
    eps = []
    seq = cases.cali_sequence(c)
    final = oracle.ddim_sample(cases.unet_noise(c), seq, net.forward, oracle.linear_betas(),
                               on_step=lambda s, i, xt, et: eps.append(et.numpy().copy()))
    for s, e in enumerate(eps):
        ref = golden_cali[f"{name}/eps{s}"]
        np.testing.assert_allclose(e, ref, rtol=0, atol=2e-3 * np.abs(ref).max())
    assert oracle.psnr(golden_cali[name + "/final"], final.numpy()) > 60.0


# ------------------------------------------------------------------------------------ GPU
def _resumed(c, cuda, golden_cali, act_quant_mode="qdiff"):
    import modiff_b200 as m
    torch.manual_seed(0)
    net = m.Model(m.make_config(split_shortcut=c["split"])).eval()
    state = {k: v.detach().clone() for k, v in net.state_dict().items()}
    wq, aq = cases.quant_params(c)
    aq = dict(aq, dynamic=(act_quant_mode == "dynamic"))
    qnn = m.QuantModel(net, wq, aq, sm_abit=8, modulate=True).to(cuda).eval()
    ckpt = cases.cali_checkpoint(c, state, golden_cali, c["name"])
    m.resume_cali_model(qnn, ckpt, cases.cali_data(c), quant_act=True,
                        act_quant_mode=act_quant_mode, cond=False)
    return qnn, ckpt


def _run(qnn, c, cuda, graph):
    import modiff_b200 as m
    eps = []
    model = qnn.graphed() if graph else qnn

    def fn(x, t):
        e = model(x, t)
        eps.append(e.clone())
        return e

    qnn.reset_cache()
    betas = torch.from_numpy(m.get_beta_schedule()).float()
    seq = cases.cali_sequence(c)
    xs, _ = m.generalized_steps(cases.unet_noise(c).to(cuda), seq, fn, betas, eta=0.0)
    torch.cuda.synchronize()
    assert m.device_status() == 0
    return xs[-1].cpu(), [e.cpu() for e in eps]


@pytest.mark.gpu
@pytest.mark.parametrize("c", cases.CALI_CASES, ids=lambda c: c["name"])
def test_resume_cali_model_matches_reference(c, cuda, golden_cali):
    """Every checkpoint key finds its place; the loaded scales are the checkpoint's; the
    modulated evaluations agree with the reference's (first one to 1e-4 of the range - it has
    no activation quantiser -, later ones to the PSNR floor of a free-running residual
    quantiser, cf. test_gpu_unet.test_eps_per_step)."""
    import modiff_b200 as m
    name = c["name"]
    qnn, ckpt = _resumed(c, cuda, golden_cali)
    mods = dict(qnn.named_modules())
    n_act = 0
    for key, val in ckpt.items():
        path, _, field = key.rpartition(".")
        owner, _, slot = path.rpartition(".")
        if slot.startswith("act_quantizer"):
            q = getattr(mods[owner], slot)
            got = q.delta if field == "delta" else q.zero_point
            assert q.inited
            assert float(torch.as_tensor(got)) == pytest.approx(float(val), rel=0, abs=0), key
            n_act += 1
        elif slot.startswith("weight_quantizer"):
            q = getattr(mods[owner], slot)
            assert isinstance(q, m.AdaRoundQuantizer)
            got = getattr(q, field)
            assert torch.equal(got.detach().cpu().reshape(val.shape), val), key
    assert n_act >= 2 * 113
    final, eps = _run(qnn, c, cuda, graph=False)
    for s, e in enumerate(eps):
        ref = golden_cali[f"{name}/eps{s}"]
        err = np.abs(e.numpy() - ref).max() / np.abs(ref).max()
        p = oracle.psnr(ref, e.numpy())
        print(f"{name} evaluation {s}: max err {err:.2e} of range, PSNR {p:.1f} dB")
        if s == 0:
            assert err < 1e-4, err
        else:
            # the oracle run twice, its x_T moved by 1e-5, agrees with itself to 55 dB (8-bit
            # symmetric case) / 43 dB (6-bit asymmetric case) on these evaluations
            assert p >= (40.0 if c["a_bits"] == 8 else 30.0), (s, p)
    # replay through CUDA graphs launches the same kernels on the same buffers
    final_g, eps_g = _run(qnn, c, cuda, graph=True)
    for a, b in zip(eps, eps_g):
        assert torch.equal(a, b)
    assert torch.equal(final, final_g)


@pytest.mark.gpu
def test_adaround_weight_codes_bit_exact(cuda, golden_cali):
    """Integer weight codes of one loaded layer equal the oracle's floor + (alpha >= 0)."""
    c = cases.CALI_CASES[0]
    qnn, ckpt = _resumed(c, cuda, golden_cali)
    for base in ("model.down.1.block.0.conv1", "model.up.2.block.0.nin_shortcut",
                 "model.temb.dense.0"):
        mod = dict(qnn.named_modules())[base]
        pack = mod.packed_weights(split=mod.split)
        w = ckpt[base + ".weight"]
        slots = ["weight_quantizer"] + (["weight_quantizer_0"] if mod.split else [])
        segs = [w[:, :mod.split], w[:, mod.split:]] if mod.split else [w]
        dq = []
        for s, seg in zip(slots, segs):
            d, _, _, _ = adaround_codes(seg.contiguous(), ckpt[f"{base}.{s}.alpha"],
                                        ckpt[f"{base}.{s}.delta"], ckpt[f"{base}.{s}.zero_point"],
                                        c["w_bits"])
            dq.append(d)
        want = torch.cat(dq, dim=1)
        # w_dq is [cin * taps][cout], K order (cin, ky, kx)
        got = pack["w_dq"].cpu().reshape(want.shape[1:].numel(), want.shape[0]).t().reshape(want.shape)
        assert torch.equal(got, want), base


@pytest.mark.gpu
def test_adaround_quantizer_forward_on_the_device(cuda):
    """AdaRoundQuantizer.forward (the stand-alone fake quantisation with the hard rounding
    decision) runs as a device kernel and equals the oracle's restatement of
    qdiff/adaptive_rounding.py:49-61 bit for bit; the training-time modes raise."""
    import modiff_b200 as m
    g = torch.Generator().manual_seed(6)
    w = torch.randn(24, 16, 3, 3, generator=g)
    uaq = m.UniformAffineQuantizer(n_bits=4, symmetric=False, channel_wise=True, scale_method="max")
    uaq(w.to(cuda))                                   # sets delta / zero_point per channel
    ada = m.AdaRoundQuantizer(uaq, w.to(cuda))
    # initial logits: round to nearest, i.e. the uniform quantiser's own result
    _, q, delta, zp = weight_codes(w, 4)
    assert torch.equal(ada.delta.cpu().reshape(-1), delta.reshape(-1))
    assert torch.equal(ada(w.to(cuda)).cpu(), (q - zp) * delta)
    # arbitrary logits, as a checkpoint would hold
    alpha = torch.randn(w.shape, generator=g)
    ada.alpha.data = alpha.to(cuda)
    want, _, _, _ = adaround_codes(w, alpha, delta, zp, 4)
    assert torch.equal(ada(w.to(cuda)).cpu(), want)
    ada.soft_targets = True
    with pytest.raises(m.ModiffError):
        ada(w.to(cuda))
    with pytest.raises(m.ModiffError):
        m.AdaRoundQuantizer(uaq, w.to(cuda), round_mode="nearest")


@pytest.mark.gpu
def test_static_scale_set_by_first_quantised_call(cuda):
    """Without a checkpoint a non-dynamic quantiser keeps the scale of its first quantised call
    (qdiff/quant_layer.py:72-79): compare a layer with the oracle over four steps."""
    import modiff_b200 as m
    from oracle.quant_module import OracleQuantModule
    lc = dict(cases.LAYER_CASES[0])
    org = cases.layer_module(lc)
    w_cpu, b_cpu = org.weight.detach().clone(), org.bias.detach().clone()
    wq, aq = cases.quant_params(lc)
    aq = dict(aq, dynamic=False)
    mod = m.QuantModule(org, wq, aq, modulate=True).to(cuda)
    mod.set_quant_state(True, True)
    orc = OracleQuantModule(w_cpu, b_cpu, lc["stride"], lc["pad"],
                            lc["w_bits"], lc["a_bits"], True, modulate=True, a_dynamic=False)
    xs = cases.layer_inputs(lc)
    xs.append(xs[-1] + 0.2 * torch.randn(xs[-1].shape, generator=torch.Generator().manual_seed(3)))
    for s, x in enumerate(xs):
        want = orc.forward(x)
        got = mod(x.to(cuda)).cpu()
        if s >= 1:
            assert float(mod.act_quantizer.delta) == float(orc.act_scale[0][0])
        np.testing.assert_allclose(got.numpy(), want.numpy(), rtol=0,
                                   atol=1e-4 * float(want.abs().max()))
        assert torch.equal(mod.a_hat.cpu(), orc.a_hat)
    # the last input saturates the fixed scale: codes clamp instead of the scale growing
    assert int(orc.last["codes"][0].abs().max()) >= 127


@pytest.mark.gpu
def test_static_scale_survives_another_batch_size(cuda):
    """A non-dynamic quantiser's scale belongs to the quantiser, not to an input shape
    (qdiff/quant_layer.py:72-79): measured at batch 2, it is the scale that quantises a batch of
    1 after reset_cache(), exactly as the oracle (and the reference) carry it over."""
    import modiff_b200 as m
    from oracle.quant_module import OracleQuantModule
    lc = dict(cases.LAYER_CASES[0])
    org = cases.layer_module(lc)
    w_cpu, b_cpu = org.weight.detach().clone(), org.bias.detach().clone()
    wq, aq = cases.quant_params(lc)
    mod = m.QuantModule(org, wq, dict(aq, dynamic=False), modulate=True).to(cuda)
    mod.set_quant_state(True, True)
    orc = OracleQuantModule(w_cpu, b_cpu, lc["stride"], lc["pad"], lc["w_bits"], lc["a_bits"], True,
                            modulate=True, a_dynamic=False)
    xs = cases.layer_inputs(lc)
    for x in xs[:3]:                       # batch 2: the first quantised call sets the scale
        orc.forward(x)
        mod(x.to(cuda))
    delta = float(mod.act_quantizer.delta)
    assert delta == float(orc.act_scale[0][0])
    mod.reset_cache()
    orc.reset_cache()
    for s, x in enumerate(xs[:3]):         # batch 1, other values: the scale must not move
        x1 = 0.5 * x[:1].contiguous()
        want = orc.forward(x1)
        got = mod(x1.to(cuda)).cpu()
        assert float(mod.act_quantizer.delta) == delta == float(orc.act_scale[0][0])
        np.testing.assert_allclose(got.numpy(), want.numpy(), rtol=0,
                                   atol=1e-4 * float(want.abs().max()))
        assert torch.equal(mod.a_hat.cpu(), orc.a_hat)
    assert m.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("lname", ["c3_w4a4", "c1_split_w4a4", "c3_w4a4_asym",
                                   "c1_split_w8a4_asym", "lin_w8a6_asym", "down_w8a8",
                                   "c3_w8a8_asym", "c1_split_w4a8_asym", "down_w8a8_asym"])
def test_layer_with_loaded_scales_and_adaround(cuda, lname):
    """One layer, teacher-forced inputs: AdaRound logits and activation scales installed the
    way the checkpoint loader does.  Codes are integers, so the cached input a_hat must equal
    the oracle's bit for bit at every step; outputs to 1e-4 of their range (the first step runs
    on split-bf16 tensor cores and stays in the cached output)."""
    import torch.nn.functional as F
    import modiff_b200 as m
    from oracle.quant_module import OracleQuantModule
    lc = next(c for c in cases.LAYER_CASES if c["name"] == lname)
    org = cases.layer_module(lc)
    w, b_cpu = org.weight.detach().clone(), org.bias.detach().clone()
    wq, aq = cases.quant_params(lc)
    aq = dict(aq, dynamic=False)
    split = lc.get("split", 0)
    sym = lc.get("a_sym", True)
    mod = m.QuantModule(org, wq, aq, modulate=True).to(cuda)
    xs = cases.layer_inputs(lc)
    if lc.get("pad_br"):
        xs = [F.pad(x, (0, 1, 0, 1)) for x in xs]
    fwd = (lambda mm, x: mm(x, split=split)) if split else (lambda mm, x: mm(x))
    with torch.no_grad():
        mod.set_quant_state(True, False)
        fwd(mod, xs[0].to(cuda))                     # initialises the weight quantisers
        m.convert_adaround(torch.nn.Sequential(mod))
        gen = torch.Generator().manual_seed(lc["seed"] + 7)
        segs = [w[:, :split], w[:, split:]] if split else [w]
        slots = ["weight_quantizer", "weight_quantizer_0"][:len(segs)]
        ada = []
        for s, seg in zip(slots, segs):
            q = getattr(mod, s)
            assert isinstance(q, m.AdaRoundQuantizer) and q.alpha.shape == seg.shape
            alpha = torch.randn(seg.shape, generator=gen)
            q.alpha.data.copy_(alpha.to(cuda))
            ada.append((alpha, q.delta.cpu(), q.zero_point.cpu()))
        mod._wpack = None
        # scales: a little under the largest residual, so that some codes clamp
        r = (xs[1] - xs[0])
        rs = [r[:, :split], r[:, split:]] if split else [r]
        n_lv = 2 ** lc["a_bits"] - 1
        if sym:
            deltas = [float(v.abs().max()) / (2 ** (lc["a_bits"] - 1)) for v in rs]
            zps = [0.0] * len(rs)
        else:
            deltas = [float(v.max() - v.min()) * 0.9 / n_lv for v in rs]
            zps = [float(round(-float(v.min()) * 0.9 / d)) for v, d in zip(rs, deltas)]
        mod.load_act_scale(deltas, zps)
        mod.set_quant_state(True, True)
        orc = OracleQuantModule(w, b_cpu, lc.get("stride", 1), lc.get("pad", 0),
                                lc["w_bits"], lc["a_bits"], sym, modulate=True, a_dynamic=False)
        orc.adaround = ada
        orc.act_scale = [(torch.tensor(d), int(z)) for d, z in zip(deltas, zps)]
        clamped = False
        for step, x in enumerate(xs):
            want = orc.forward(x, split) if split else orc.forward(x)
            got = fwd(mod, x.to(cuda)).cpu()
            err = float((got - want).abs().max() / want.abs().max())
            assert err < 1e-4, (step, err)
            assert torch.equal(mod.a_hat.cpu(), orc.a_hat), step
            if step:
                for codes, z in zip(orc.last["codes"], zps):
                    clamped |= int(codes.max()) == (127 if sym and lc["a_bits"] == 8 else
                                                    (2 ** (lc["a_bits"] - 1) - 1 if sym else n_lv))
        assert clamped
    assert m.device_status() == 0


@pytest.mark.gpu
def test_resume_weights_with_dynamic_activation_scales(cuda, golden_cali):
    """`--resume --quant_mode dynamic`: AdaRound weights from the checkpoint, activation scales
    still measured every step (the checkpoint's activation entries are not used,
    qdiff/utils.py:606-611).  Checked against the oracle with the same checkpoint."""
    import modiff_b200 as m
    c = cases.CALI_CASES[0]
    qnn, ckpt = _resumed(c, cuda, golden_cali, act_quant_mode="dynamic")
    assert all(q.dynamic for q in qnn.modules() if isinstance(q, m.UniformAffineQuantizer)
               and q.n_bits == c["a_bits"] and q.leaf_param)
    final, eps = _run(qnn, c, cuda, graph=True)
    state = {k[len("model."):]: v for k, v in ckpt.items()
             if ".weight_quantizer" not in k and ".act_quantizer" not in k}
    net = oracle.OracleUNet(state, w_bits=c["w_bits"], a_bits=c["a_bits"], a_sym=c["a_sym"],
                            split_shortcut=c["split"])
    net.load_calibrated(ckpt, load_act=False)
    want = []
    oracle.ddim_sample(cases.unet_noise(c), cases.cali_sequence(c), net.forward,
                       oracle.linear_betas(),
                       on_step=lambda s, i, xt, et: want.append(et.numpy().copy()))
    for s, (e, w) in enumerate(zip(eps, want)):
        p = oracle.psnr(w, e.numpy())
        print(f"dynamic scales, evaluation {s}: PSNR {p:.1f} dB")
        assert p >= (100.0 if s == 0 else 40.0), (s, p)
