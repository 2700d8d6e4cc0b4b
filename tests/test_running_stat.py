"""Moving-average activation ranges (`--running_stat`, act_momentum_update in
qdiff/quant_layer.py:113-132) on single layers, against `running.npz`: what the reference
QuantModule produced with non-dynamic leaf quantisers - call 0 unquantised, call 1 sets scale and
range, calls 2..4 with set_running_stat(True), call 5 with it off again."""
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import cases
import oracle

GOLDEN = os.path.dirname(os.path.abspath(cases.__file__))


@pytest.fixture(scope="module")
def golden_running():
    return np.load(os.path.join(GOLDEN, "running.npz"))


def _case(name):
    return next(c for c in cases.LAYER_CASES if c["name"] == name)


def _inputs(c):
    xs = cases.running_inputs(c)
    return [F.pad(x, (0, 1, 0, 1)) for x in xs] if c.get("pad_br") else xs


@pytest.mark.parametrize("name", cases.RUNNING_CASES)
def test_oracle_follows_reference(name, golden_running):
    c = _case(name)
    org = cases.layer_module(c)
    split = c.get("split", 0)
    orc = oracle.OracleQuantModule(org.weight.detach(), org.bias.detach(), c.get("stride", 1),
                                   c.get("pad", 0), c["w_bits"], c["a_bits"], c.get("a_sym", True),
                                   modulate=True, a_dynamic=False)
    for s, x in enumerate(_inputs(c)):
        orc.running_stat = s in (2, 3, 4)
        y = orc.forward(x, split) if split else orc.forward(x)
        if s > 0:
            d = np.asarray([float(a[0]) for a in orc.act_scale], np.float32)
            z = np.asarray([float(a[1]) for a in orc.act_scale], np.float32)
            r = np.asarray([[float(a), float(b)] for a, b in orc.act_range], np.float32)
            np.testing.assert_array_equal(d, golden_running[f"{name}/delta{s}"])
            np.testing.assert_array_equal(z, golden_running[f"{name}/zp{s}"])
            np.testing.assert_array_equal(r, golden_running[f"{name}/range{s}"])
        if s >= 4:
            ref = golden_running[f"{name}/out{s}"]
            np.testing.assert_allclose(y.numpy(), ref, rtol=0, atol=1e-5 * np.abs(ref).max())
    np.testing.assert_array_equal(orc.a_hat.numpy(), golden_running[name + "/a_hat"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", cases.RUNNING_CASES)
def test_cuda_path_follows_reference(name, cuda, golden_running):
    """Scale, zero point and the moving range bit-exact at every call, the cache bit-exact at
    the end, outputs to 1e-4 of their range (the first call runs on split-bf16 tensor cores)."""
    import modiff_b200 as m
    c = _case(name)
    org = cases.layer_module(c)
    split = c.get("split", 0)
    wq, aq = cases.quant_params(c)
    mod = m.QuantModule(org, wq, dict(aq, dynamic=False), modulate=True).to(cuda)
    mod.set_quant_state(True, True)
    xs = cases.running_inputs(c)          # the module applies the right / bottom pad itself
    if c.get("pad_br"):
        mod.implicit_pad = (0, 1, 0, 1)
    for s, x in enumerate(xs):
        mod.set_running_stat(s in (2, 3, 4))
        with torch.no_grad():
            y = mod(x.to(cuda), split=split) if split else mod(x.to(cuda))
        if s > 0:
            qs = [mod.act_quantizer] + ([mod.act_quantizer_0] if split else [])
            d = np.asarray([float(q.delta) for q in qs], np.float32)
            z = np.asarray([float(torch.as_tensor(q.zero_point)) for q in qs], np.float32)
            r = np.asarray([[float(q.x_min), float(q.x_max)] for q in qs], np.float32)
            np.testing.assert_array_equal(d, golden_running[f"{name}/delta{s}"])
            np.testing.assert_array_equal(z, golden_running[f"{name}/zp{s}"])
            np.testing.assert_array_equal(r, golden_running[f"{name}/range{s}"])
        if s >= 4:
            ref = golden_running[f"{name}/out{s}"]
            err = np.abs(y.cpu().numpy() - ref).max() / np.abs(ref).max()
            assert err < 1e-4, (s, err)
    a_ref = golden_running[name + "/a_hat"]
    a = mod.a_hat.cpu().numpy()
    if c.get("pad_br"):
        a_ref = a_ref[:, :, :-1, :-1]      # the reference cached the padded tensor
    np.testing.assert_array_equal(a, a_ref)
    assert m.device_status() == 0


@pytest.mark.gpu
def test_running_stat_needs_an_initialised_leaf_quantiser(cuda):
    import modiff_b200 as m
    c = _case("c3_w8a8")
    wq, aq = cases.quant_params(c)
    mod = m.QuantModule(cases.layer_module(c), wq, aq, modulate=True).to(cuda)   # dynamic
    mod.set_quant_state(True, True)
    xs = cases.running_inputs(c)
    mod(xs[0].to(cuda))
    mod.set_running_stat(True)
    with pytest.raises(m.ModiffError):
        mod(xs[1].to(cuda))


@pytest.mark.gpu
def test_running_stat_on_an_upsample_convolution(cuda):
    """With the source-resolution quantiser switched off, `forward_upsampled` is the ordinary
    layer on the upsampled tensor and takes running statistics like any other layer."""
    import copy
    import modiff_b200 as m
    from modiff_b200 import ops
    torch.manual_seed(61)
    org = torch.nn.Conv2d(64, 64, 3, padding=1)
    wq = {'n_bits': 8, 'channel_wise': True, 'scale_method': 'max'}
    aq = {'n_bits': 8, 'symmetric': True, 'channel_wise': False, 'scale_method': 'max',
          'leaf_param': True, 'dynamic': False}
    a = m.QuantModule(copy.deepcopy(org), wq, aq, modulate=True).to(cuda)
    b = m.QuantModule(copy.deepcopy(org), wq, aq, modulate=True).to(cuda)
    a.upsampled_input_fusion = False
    for q in (a, b):
        q.set_quant_state(True, True)
        q.alias_output = False
    g = torch.Generator().manual_seed(62)
    x = torch.randn(2, 64, 8, 8, generator=g)
    with torch.no_grad():
        for s in range(5):
            xs = (x + 0.05 * s * torch.randn(x.shape, generator=g)).to(cuda)
            for q in (a, b):
                q.set_running_stat(s >= 2)
            ya = a.forward_upsampled(xs)
            yb = b(ops.upsample2x(xs))
            assert torch.equal(ya, yb), s
            if s >= 1:
                assert float(a.act_quantizer.x_min) == float(b.act_quantizer.x_min)
                assert float(a.act_quantizer.delta) == float(b.act_quantizer.delta)
    assert m.device_status() == 0
