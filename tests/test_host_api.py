"""Host-side logic that needs no GPU: the class surface of the reference API, module rewriting,
flag fan-out, the C ABI's exported symbols, size helpers and loud failure on CPU tensors."""
import ctypes as C
import os
import re

import pytest
import torch
import torch.nn as nn

import modiff_b200 as m
from modiff_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WQ = {'n_bits': 4, 'channel_wise': True, 'scale_method': 'max'}
AQ = {'n_bits': 4, 'symmetric': True, 'channel_wise': False, 'scale_method': 'max',
      'leaf_param': True, 'dynamic': True}


@pytest.fixture(scope="module")
def qnn():
    torch.manual_seed(0)
    net = m.Model(m.make_config(split_shortcut=True))
    return m.QuantModel(net, WQ, AQ, sm_abit=8, modulate=True)


def test_header_symbols_are_exported_and_bound():
    """Every function declared in include/modiff_b200.h is exported by the shared library and
    has a ctypes signature; no compute call is made."""
    hdr = open(os.path.join(ROOT, "include", "modiff_b200.h")).read()
    code = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)          # drop comments
    declared = set(re.findall(r"\b(modiff_[a-z0-9_]+)\s*\(", code))
    declared -= {"modiff_conv_geom", "modiff_act_source", "modiff_gemm_bf16_desc"}
    assert len(declared) >= 20
    lib = _lib.lib()
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_lib.SIGNATURES) == declared
    assert lib.modiff_version() == 100


def test_size_helpers():
    lib = _lib.lib()
    g = _lib.ConvGeom(4, 128, 256, 32, 32, 3, 3, 1, 1, 1, 1, 1, 0)
    assert _lib.out_hw(g) == (32, 32)
    assert lib.modiff_codes_bytes(C.byref(g)) == 4 * 34 * 34 * 128
    assert lib.modiff_wcodes_rows(C.byref(g), 0) == 256 and lib.modiff_wcodes_rows(C.byref(g), 1) == 288
    assert lib.modiff_wcodes_bytes(C.byref(g), 1) == 288 * 9 * 128
    g2 = _lib.ConvGeom(2, 3, 128, 32, 32, 3, 3, 2, 0, 0, 1, 1, 0)   # stride 2, pad right/bottom
    assert _lib.out_hw(g2) == (16, 16)
    assert lib.modiff_codes_bytes(C.byref(g2)) == 2 * 4 * 17 * 17 * 16
    # integer attention: q / k rows are the head's channels padded to 32, 64, 128 or 256 bytes,
    # v rows are channels (multiple of 16) by keys padded to 128
    for c, dp in ((24, 32), (32, 32), (40, 64), (64, 64), (96, 128), (160, 256), (256, 256)):
        assert lib.modiff_attn_codes_bytes(16, c, 300, 77, 0) == 16 * 300 * dp
        assert lib.modiff_attn_codes_bytes(16, c, 300, 77, 1) == 16 * 77 * dp
        assert lib.modiff_attn_codes_bytes(16, c, 300, 77, 2) == 16 * (-(-c // 16) * 16) * 128


def test_invalid_geometry_is_reported_not_crashed():
    lib = _lib.lib()
    g = _lib.ConvGeom(1, 8, 8, 4, 4, 3, 3, 3, 0, 0, 0, 0, 0)   # stride 3 unsupported
    rc = lib.modiff_modq(None, None, None, None, C.byref(g), 8, 0, None, None)
    assert rc == 1 and b"stride" in lib.modiff_last_error()
    with pytest.raises(m.ModiffError):
        _lib.check(rc)


def test_quant_model_rewrites_the_unet(qnn):
    mods = [x for x in qnn.modules() if isinstance(x, m.QuantModule)]
    assert len(mods) == 113
    assert sum(isinstance(x, m.QuantResnetBlock) for x in qnn.modules()) == 22
    assert sum(isinstance(x, m.QuantAttnBlock) for x in qnn.modules()) == 6
    assert not any(isinstance(x, (nn.Conv2d, nn.Linear)) for x in qnn.modules())
    assert qnn.in_channels == 3 and qnn.sm_abit == 8 and qnn.modulate is True
    # parameters are shared with the wrapped model, not copied
    assert sum(p.numel() for p in qnn.parameters()) == 35746307


def test_flag_fan_out(qnn):
    qnn.set_quant_state(True, True)
    assert all(x.use_weight_quant and x.use_act_quant for x in qnn.modules()
               if isinstance(x, (m.QuantModule, m.BaseQuantBlock)))
    qnn.set_quant_state(True, False)
    assert not any(x.use_act_quant for x in qnn.modules() if isinstance(x, m.QuantModule))
    qnn.set_modulation(False)
    assert not any(x.modulate for x in qnn.modules() if isinstance(x, m.QuantModule))
    qnn.set_modulation(True)
    qnn.set_dynamic_state(False)
    assert not any(x.act_quantizer.dynamic for x in qnn.modules() if isinstance(x, m.QuantModule))
    qnn.set_dynamic_state(True)
    qnn.set_running_stat(True)
    assert all(x.act_quantizer.running_stat for x in qnn.modules() if isinstance(x, m.QuantModule))
    qnn.set_running_stat(False)
    for x in qnn.modules():
        if isinstance(x, m.QuantModule):
            x.a_hat = x.o_hat = torch.zeros(1)
    qnn.reset_cache()
    assert all(x.a_hat is None and x.o_hat is None for x in qnn.modules()
               if isinstance(x, m.QuantModule))
    qnn.set_grad_ckpt(False)


def test_quantizer_surface():
    q = m.UniformAffineQuantizer(n_bits=4, symmetric=True)
    assert q.n_levels == 7 and q.sym and not q.inited and q.delta is None
    q = m.UniformAffineQuantizer(n_bits=8)
    assert q.n_levels == 256 and not q.channel_wise and q.scale_method == 'max'
    q.bitwidth_refactor(4)
    assert q.n_bits == 4 and q.n_levels == 16
    x = torch.tensor([0.4, 0.5, 1.5, 2.5, -0.5, -1.5])
    assert torch.equal(m.round_ste(x), torch.tensor([0., 0., 2., 2., -0., -2.]))


def test_quant_module_surface_and_split():
    conv = nn.Conv2d(8, 4, 1)
    qm = m.QuantModule(conv, WQ, AQ, modulate=True)
    for attr in ("fwd_func", "fwd_kwargs", "weight", "bias", "org_weight", "org_bias",
                 "use_weight_quant", "use_act_quant", "act_quant_mode", "disable_act_quant",
                 "weight_quantizer", "act_quantizer", "split", "activation_function",
                 "ignore_reconstruction", "modulate", "a_hat", "o_hat"):
        assert hasattr(qm, attr), attr
    assert qm.weight is conv.weight and qm.split == 0 and qm.a_hat is None
    qm.set_split()
    assert isinstance(qm.weight_quantizer_0, m.UniformAffineQuantizer)
    assert isinstance(qm.act_quantizer_0, m.UniformAffineQuantizer)
    qm.set_modualtion(False)
    assert qm.modulate is False


def test_cpu_tensors_are_refused(qnn):
    """No CPU fallback anywhere on the quantised path."""
    qnn.set_quant_state(True, True)
    with pytest.raises(m.ModiffError):
        qnn(torch.randn(1, 3, 32, 32), torch.zeros(1))
    qm = m.QuantModule(nn.Linear(8, 8), WQ, AQ, modulate=True)
    qm.set_quant_state(True, True)
    with pytest.raises(m.ModiffError):
        qm(torch.randn(2, 8))
    with pytest.raises(m.ModiffError):
        m.UniformAffineQuantizer(8)(torch.randn(4))


def test_reference_class_names_are_rehosted():
    """Blocks are matched by class name, so the reference's own ResnetBlock / AttnBlock
    classes (ddim/models/diffusion.py) are re-hosted as well."""
    class ResnetBlock(nn.Module):
        def __init__(self):
            super().__init__()
            self.in_channels, self.out_channels, self.use_conv_shortcut = 32, 64, False
            self.norm1 = nn.GroupNorm(32, 32)
            self.conv1 = nn.Conv2d(32, 64, 3, padding=1)
            self.temb_proj = nn.Linear(16, 64)
            self.norm2 = nn.GroupNorm(32, 64)
            self.dropout = nn.Dropout(0.1)
            self.conv2 = nn.Conv2d(64, 64, 3, padding=1)
            self.nin_shortcut = nn.Conv2d(32, 64, 1)

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.in_channels = 32
            self.blk = ResnetBlock()

    q = m.QuantModel(Net(), WQ, AQ, modulate=True)
    assert isinstance(q.model.blk, m.QuantResnetBlock)
    assert isinstance(q.model.blk.nin_shortcut, m.QuantModule)


def test_sampler_schedule_helpers():
    seq = m.make_timestep_sequence(1000, 100, "quad")
    assert seq[:8] == [0, 0, 0, 0, 1, 2, 2, 3] and seq[-3:] == [768, 783, 800]
    assert m.make_timestep_sequence(1000, 10, "uniform") == list(range(0, 1000, 100))
    betas = torch.from_numpy(m.get_beta_schedule()).float()
    from modiff_b200.sampler import alpha_table, step_coefficients
    al = alpha_table(betas)
    ref = m.compute_alpha(betas, torch.tensor([800]))
    assert float(al[801]) == float(ref)
    s1, s2, s3, c1, c2 = step_coefficients(al, 0, -1, 0.0)
    assert s3 == 1.0 and c1 == 0.0 and c2 == 0.0


def test_reciprocal_multiply_with_tie_guard_equals_division():
    """The quantiser's encode pass divides by multiplying with rn(1/delta) and falls back to the
    true division only within 2^-14 of a rounding tie (csrc/modq.cu: quantise_clamp).  The same
    steps in IEEE float32 (numpy) give clamp(rne(r / delta)) for every input, including residuals
    placed a few ulps around every tie (qdiff/quant_layer.py:94-99)."""
    import numpy as np
    rng = np.random.default_rng(0)
    f32 = np.float32

    def reference(r, d, lo, hi):
        return np.clip(np.rint(r / d), lo, hi)

    def fast(r, d, lo, hi):
        inv = f32(1.0) / d
        tc = np.clip(r * inv, lo, hi)
        magic = f32(12582912.0)
        q = (tc + magic) - magic
        near_tie = np.abs(tc - q) > f32(0.5) - f32(6.103515625e-5)
        te = np.clip(r / d, lo, hi)
        qe = (te + magic) - magic
        return np.where(near_tie, qe, q), near_tie.mean()

    for bits in (8, 4, 3):
        n = (1 << (bits - 1)) - 1
        lo, hi = f32(-n - 1), f32(n)
        d = np.exp(rng.uniform(np.log(1e-8), np.log(10.0), 4000)).astype(f32)
        # random residuals over +-1.5x the code range
        r = (rng.uniform(-1.5 * (n + 1), 1.5 * (n + 1), (4000, 512)).astype(f32) * d[:, None]).astype(f32)
        got, frac = fast(r, d[:, None], lo, hi)
        assert np.array_equal(got, reference(r, d[:, None], lo, hi))
        assert frac < 1e-3
        # residuals a few ulps around every tie k + 0.5
        k = np.arange(-n - 3, n + 3, dtype=np.float64) + 0.5
        r0 = (k[None, :] * d[:, None].astype(np.float64)).astype(f32)
        for step in range(-4, 5):
            r = r0.copy()
            for _ in range(abs(step)):
                r = np.nextafter(r, f32(np.inf) if step > 0 else f32(-np.inf)).astype(f32)
            got, _ = fast(r, d[:, None], lo, hi)
            assert np.array_equal(got, reference(r, d[:, None], lo, hi)), (bits, step)


def test_calibrated_scale_validation():
    """`load_act_scale` (what a checkpoint's act_quantizer.delta / zero_point become) checks what
    the int8 code planes can hold before anything reaches the GPU."""
    def layer(bits, sym, per_sample=False):
        aq = {'n_bits': bits, 'symmetric': sym, 'channel_wise': per_sample, 'scale_method': 'max',
              'leaf_param': True, 'dynamic': False}
        return m.QuantModule(nn.Conv2d(16, 16, 3, padding=1),
                             {'n_bits': 8, 'channel_wise': True, 'scale_method': 'max'}, aq,
                             modulate=True)
    layer(8, True).load_act_scale(0.01)                       # symmetric: zero point 0
    layer(8, False).load_act_scale(0.01, 255)                 # 8-bit asymmetric: planes hold q - 128
    layer(6, False).load_act_scale([0.01], [63])
    with pytest.raises(m.ModiffError):
        layer(8, True).load_act_scale(0.01, 3)                # symmetric with a zero point
    with pytest.raises(m.ModiffError):
        layer(6, False).load_act_scale(0.01, 129)             # centred 6-bit code leaves int8
    with pytest.raises(m.ModiffError):
        layer(8, False).load_act_scale(0.01, 256)
    with pytest.raises(m.ModiffError):
        layer(8, False).load_act_scale(0.01, 12.5)            # not an integer
    with pytest.raises(m.ModiffError):
        layer(8, True).load_act_scale(0.0)                    # scale must be positive
    with pytest.raises(m.ModiffError):
        layer(8, True).load_act_scale([0.1, 0.2, 0.3])
    with pytest.raises(m.ModiffError):
        layer(8, True, per_sample=True).load_act_scale(0.01)  # calibrated scales are per tensor


def test_checkpoint_key_routing(qnn):
    """Quantiser tensors are told from ordinary parameters by their last two name parts; a key
    that points at no quantised layer is an error, as with strict loading in the reference."""
    from modiff_b200.utils import _split_key, load_calibrated_state
    assert _split_key("model.down.0.block.0.conv1.weight_quantizer.alpha") == \
        ("model.down.0.block.0.conv1", "weight_quantizer", "alpha")
    assert _split_key("model.up.1.block.0.nin_shortcut.act_quantizer_0.zero_point") == \
        ("model.up.1.block.0.nin_shortcut", "act_quantizer_0", "zero_point")
    assert _split_key("model.down.0.block.0.conv1.weight") is None
    assert _split_key("model.mid.attn_1.act_quantizer_w.delta") is None
    with pytest.raises(m.ModiffError):
        load_calibrated_state(qnn, {"model.nowhere.weight_quantizer.alpha": torch.zeros(1)})
    with pytest.raises(m.ModiffError):      # layer exists, but was not converted to AdaRound
        load_calibrated_state(qnn, {"model.conv_in.weight_quantizer.alpha": torch.zeros(1)})


def test_flag_setters_invalidate_captured_graphs(qnn):
    e0 = getattr(qnn, "_config_epoch", 0)
    qnn.set_dynamic_state(False)
    qnn.set_quant_state(True, True)
    qnn.set_modulation(True)
    assert qnn._config_epoch == e0 + 3
    qnn.set_dynamic_state(True)
