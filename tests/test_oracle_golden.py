"""The CPU oracle against the fixtures produced by the live reference (tests/golden/*.npz)."""
import json
import os

import numpy as np
import pytest
import torch

import cases
import oracle
from oracle.quantizer import fake_quant

GOLDEN = os.path.dirname(os.path.abspath(cases.__file__))


@pytest.mark.parametrize("c", cases.QUANTIZER_CASES, ids=lambda c: c["name"])
def test_quantizer_matches_reference(c, golden_quantizer):
    x = cases.quantizer_input(c)
    y, q, delta, zp = fake_quant(x, c["n_bits"], c["sym"], c["channel_wise"],
                                 c.get("always_zero", False))
    g = golden_quantizer
    np.testing.assert_array_equal(np.asarray(delta, dtype=np.float32).reshape(-1),
                                  g[c["name"] + "/delta"])
    zp = zp.numpy() if isinstance(zp, torch.Tensor) else np.asarray([zp])
    np.testing.assert_array_equal(np.asarray(zp, dtype=np.float32).reshape(-1), g[c["name"] + "/zp"])
    np.testing.assert_array_equal(y.numpy(), g[c["name"] + "/y"])


def _oracle_layer(c):
    org = cases.layer_module(c)
    w = org.weight.detach()
    b = org.bias.detach()
    if c["kind"] == "linear":
        return oracle.OracleQuantModule(w, b, w_bits=c["w_bits"], a_bits=c["a_bits"],
                                        a_sym=c.get("a_sym", True))
    return oracle.OracleQuantModule(w, b, c["stride"], c["pad"], c["w_bits"], c["a_bits"],
                                    c.get("a_sym", True))


@pytest.mark.parametrize("c", cases.LAYER_CASES, ids=lambda c: c["name"])
def test_layer_matches_reference(c, golden_layers):
    m = _oracle_layer(c)
    g = golden_layers
    with torch.no_grad():
        for s, x in enumerate(cases.layer_inputs(c)):
            if c.get("pad_br"):
                x = torch.nn.functional.pad(x, (0, 1, 0, 1))
            y = m.forward(x, split=c.get("split", 0))
            ref = g[f"{c['name']}/out{s}"]
            np.testing.assert_allclose(y.numpy(), ref, rtol=0, atol=1e-5 * max(1.0, np.abs(ref).max()))
            if s > 0:
                d = np.asarray([float(v) for v in m.last["x_scale"]], dtype=np.float32)
                np.testing.assert_array_equal(d, g[f"{c['name']}/delta{s}"])
                if not c.get("a_sym", True):
                    z = np.asarray([float(v) for v in m.last["x_zp"]], dtype=np.float32)
                    np.testing.assert_array_equal(z, g[f"{c['name']}/zp{s}"])
    if not c.get("skip_a_hat"):
        np.testing.assert_array_equal(m.a_hat.numpy(), g[f"{c['name']}/a_hat"])
    np.testing.assert_array_equal(m.last["w_scale"][0].numpy(), g[f"{c['name']}/w_delta"])
    np.testing.assert_array_equal(m.last["w_zp"][0].numpy(), g[f"{c['name']}/w_zp"])


def test_layer_integer_view_is_the_fp_result():
    """out - o_hat_prev == acc * dx * dw[c] up to fp32 rounding: the exact integer
    accumulators describe the same computation as the reference's fp32 conv."""
    c = cases.LAYER_CASES[0]
    m = _oracle_layer(c)
    xs = cases.layer_inputs(c)
    with torch.no_grad():
        m.forward(xs[0])
        o_prev = m.o_hat.clone()
        out = m.forward(xs[1])
    acc = m.last["acc"][0].double()
    scale = float(m.last["x_scale"][0]) * m.last["w_scale"][0].double().view(1, -1, 1, 1)
    np.testing.assert_allclose((out - o_prev).double().numpy(), (acc * scale).numpy(),
                               atol=2e-5, rtol=1e-4)
    assert int(m.last["codes"][0].abs().max()) <= 127


def test_model_init_matches_reference_weights():
    """`torch.manual_seed(0); Model(cfg)` reproduces the reference's random-init weights."""
    import modiff_b200 as m
    with open(os.path.join(GOLDEN, "weights_seed0.json")) as fh:
        ref = json.load(fh)
    torch.manual_seed(0)
    sd = m.Model(m.make_config()).state_dict()
    assert list(sd.keys()) == list(ref.keys())
    for k, v in sd.items():
        shape, s, sa, sw = ref[k]
        assert list(v.shape) == shape, k
        v = v.double()
        w = torch.arange(1, v.numel() + 1, dtype=torch.float64).reshape(v.shape)
        got = (float(v.sum()), float(v.abs().sum()), float((v * w).sum() / v.numel()))
        np.testing.assert_allclose(got, (s, sa, sw), rtol=1e-12, atol=1e-12, err_msg=k)


def _state_dict():
    import modiff_b200 as m
    torch.manual_seed(0)
    return {k: v.detach().clone() for k, v in m.Model(m.make_config()).state_dict().items()}


@pytest.mark.parametrize("name", ["w8a8_b2_s10", "w4a4_split_b2_s10"])
def test_unet_sampling_matches_reference(name, golden_unet):
    c = next(u for u in cases.UNET_CASES if u["name"] == name)
    net = oracle.OracleUNet(_state_dict(), w_bits=c["w_bits"], a_bits=c["a_bits"],
                            split_shortcut=c["split"])
    eps = []
    final = oracle.ddim_sample(cases.unet_noise(c), cases.unet_sequence(c), net.forward,
                               oracle.linear_betas(),
                               on_step=lambda s, i, xt, et: eps.append(et.numpy().copy()))
    for s in range(c["keep_eps"]):
        ref = golden_unet[f"{name}/eps{s}"]
        # same ops in the same order; only CPU-kernel summation order may differ between hosts
        np.testing.assert_allclose(eps[s], ref, rtol=0, atol=2e-3 * np.abs(ref).max())
    ref = golden_unet[name + "/final"]
    assert oracle.psnr(ref, final.numpy()) > 60.0


def test_quad_sequence_and_schedule():
    seq = oracle.quad_sequence(1000, 100)
    assert len(seq) == 100 and seq[0] == 0 and seq[-1] == 800 and len(set(seq)) == 96
    b = oracle.linear_betas()
    assert b.dtype == torch.float32 and abs(float(b[0]) - 1e-4) < 1e-10 and abs(float(b[-1]) - 2e-2) < 1e-8
