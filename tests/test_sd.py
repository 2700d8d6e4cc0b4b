"""SD-v1 UNet shapes (spatial transformer, cross-attention with a 77x768 context, classifier-free
guidance): oracle vs the reference's fixtures (CPU) and the CUDA path vs the same fixtures (GPU).
W8A8 modulated, symmetric dynamic activations, random init seed 0 with zero tensors redrawn."""
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
def golden_sd():
    return np.load(os.path.join(GOLDEN, "sd.npz"))


def _build():
    import modiff_b200 as m
    torch.manual_seed(0)
    net = m.UNetModel(**cases.SD_CONFIG).eval()
    m.rerandomize_zero_tensors(net, seed=cases.SD_CASES[0]["zero_seed"])
    return net


def test_structure_matches_reference_counts():
    """860 M parameters, 282 quantised layers, 16 transformer blocks, 187 zero tensors."""
    import modiff_b200 as m
    torch.manual_seed(0)
    net = m.UNetModel(**cases.SD_CONFIG)
    assert sum(p.numel() for p in net.parameters()) == 859520964
    assert m.rerandomize_zero_tensors(net) == 187
    wq, aq = cases.quant_params(cases.SD_CASES[0])
    q = m.QuantModel(net, wq, aq, sm_abit=8, modulate=True)
    assert sum(isinstance(x, m.QuantModule) for x in q.modules()) == 282
    assert sum(isinstance(x, m.QuantBasicTransformerBlock) for x in q.modules()) == 16


def test_oracle_matches_reference_first_eval(golden_sd):
    """One guided evaluation of the oracle (unquantised first step) against the reference."""
    c = cases.SD_CASES[0]
    net = _build()
    state = {k: v.detach().clone() for k, v in net.state_dict().items()}
    o = OracleLDMUNet(state, cases.SD_CONFIG, c["w_bits"], c["a_bits"])
    x, cond, uncond = cases.sd_inputs(c)
    eps = []
    latent_ddim_sample(x, o.forward, ldm_schedule(**cases.SD_SCHEDULE), c["ddim_steps"],
                       max_evals=1, cond=cond, uncond=uncond, guidance=c["guidance"],
                       on_step=lambda i, e, im: eps.append(e.numpy().copy()))
    ref0 = golden_sd[c["name"] + "/eps0"]
    assert np.abs(eps[0] - ref0).max() < 1e-4 * np.abs(ref0).max()


@pytest.mark.gpu
@pytest.mark.parametrize("c", cases.SD_CASES, ids=lambda c: c["name"])
def test_cuda_path_matches_reference(c, cuda, golden_sd, golden_sens):
    import modiff_b200 as m
    net = _build()
    wq, aq = cases.quant_params(c)
    qnn = m.QuantModel(net, wq, aq, sm_abit=8, modulate=True).to(cuda).eval()
    qnn.set_quant_state(True, True)
    qnn.set_grad_ckpt(False)
    qnn.reset_cache()
    x, cond, uncond = cases.sd_inputs(c)
    sampler = m.DDIMSampler(qnn, **cases.SD_SCHEDULE)
    eps = []
    final, _ = sampler.sample(c["ddim_steps"], c["batch"], tuple(x.shape[1:]), eta=0.0,
                              conditioning=cond.to(cuda), x_T=x.to(cuda), max_evals=c["evals"],
                              unconditional_guidance_scale=c["guidance"],
                              unconditional_conditioning=uncond.to(cuda),
                              eps_callback=lambda e, i: eps.append(e.clone()))
    torch.cuda.synchronize()
    assert m.device_status() == 0
    for i, e in enumerate(eps):
        ref = golden_sd[f"{c['name']}/eps{i}"]
        err = np.abs(e.cpu().numpy() - ref).max() / np.abs(ref).max()
        p = oracle.psnr(ref, e.cpu().numpy())
        print(f"sd eval {i}: max|eps-ref|/max|ref| = {err:.2e}, PSNR {p:.1f} dB")
        if i == 0:
            # unquantised first evaluation through 282 split-bf16 layers and 32 attentions:
            # observed 1.1e-4 of the eps range; the per-layer bound is 1e-3
            assert err < 5e-4, err
        else:
            # Free-running modulated evaluations are not reproducible between two machines:
            # the residual step is ~1/127 of an already small residual, so a 1e-4 difference
            # left by evaluation 0 puts many codes on the other side of a rounding boundary,
            # 282 layers compound it and guidance 7.5 multiplies it.  The floor is what the
            # REFERENCE itself reaches against a copy of itself whose evaluation 0 was disturbed
            # by 1e-4 of its range (sens.npz, written by make_golden.py: about 30 dB on
            # evaluations 1 and 2, 51.5 dB on the final latent), minus a margin.  Layer
            # arithmetic at these shapes is checked with identical inputs in
            # test_sd_layer_shapes_teacher_forced.
            floor_db = sens_floor(golden_sens, c["name"], i)
            assert p >= floor_db, (i, p, floor_db)
    assert oracle.psnr(golden_sd[c["name"] + "/final"], final.cpu().numpy()) >= 40.0


@pytest.mark.gpu
@pytest.mark.parametrize("kind,shape,cout", [
    ("linear", (2, 4096, 320), 2560),     # GEGLU projection at 64x64 tokens
    ("linear", (2, 4096, 1280), 320),     # feed-forward output
    ("linear", (2, 77, 768), 320),        # cross-attention key / value of the text context
    ("conv1", (2, 320, 64, 64), 320),     # spatial transformer proj_in (1x1)
    ("conv3", (2, 320, 64, 64), 320),     # ResBlock conv, cin not a multiple of 128
    ("conv3", (2, 960, 32, 32), 640),     # up path after the skip concat
])
def test_sd_layer_shapes_teacher_forced(cuda, kind, shape, cout):
    """One quantised layer at an SD-v1 shape, fed the same inputs as the oracle for three
    steps (qdiff/quant_layer.py:307-367): scale and cache bit-exact, output within 1e-4."""
    import modiff_b200 as m
    torch.manual_seed(5)
    if kind == "linear":
        org = torch.nn.Linear(shape[-1], cout)
        orc = oracle.OracleQuantModule(org.weight.detach().clone(), org.bias.detach().clone(),
                                       w_bits=8, a_bits=8)
    else:
        k = 3 if kind == "conv3" else 1
        org = torch.nn.Conv2d(shape[1], cout, k, padding=k // 2)
        orc = oracle.OracleQuantModule(org.weight.detach().clone(), org.bias.detach().clone(),
                                       1, k // 2, 8, 8)
    wq, aq = cases.quant_params(cases.SD_CASES[0])
    ours = m.QuantModule(org, wq, aq, modulate=True).to(cuda)
    ours.set_quant_state(True, True)
    ours.alias_output = False
    g = torch.Generator().manual_seed(17)
    x = torch.randn(shape, generator=g)
    with torch.no_grad():
        for step in range(3):
            xs = x + 0.05 * step * torch.randn(shape, generator=g)
            ref = orc.forward(xs)
            got = ours(xs.to(cuda)).cpu()
            err = float((got - ref).abs().max() / ref.abs().max())
            # the first step's split-bf16 product (bound 1e-4) stays in the cached output, so
            # the same bound holds for the later, exact-integer steps
            assert err < 1e-4, (step, err)
            if step > 0:
                assert float(ours.act_quantizer.delta) == float(orc.last['x_scale'][0])
                assert torch.equal(ours.a_hat.cpu(), orc.a_hat)
    assert m.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("rows,c,cout,bits", [(2 * 4096, 320, 320, 8), (300, 640, 5120, 8),
                                             (77, 1280, 1280, 6)])
def test_layernorm_inside_the_quantiser_equals_the_separate_kernel(cuda, rows, c, cout, bits):
    """A transformer block's LayerNorm in front of a quantised linear layer is evaluated inside
    the quantiser's two passes (modiff_modq_ln): cached input, codes' effect (the output) and
    scale equal, bit for bit, what the stand-alone LayerNorm kernel followed by the plain
    quantiser gives, over several steps."""
    import modiff_b200 as m
    from modiff_b200 import ops
    torch.manual_seed(3)
    lin = torch.nn.Linear(c, cout, bias=False)
    norm = torch.nn.LayerNorm(c)
    with torch.no_grad():
        norm.weight.uniform_(0.5, 1.5)
        norm.bias.normal_(0, 0.3)
    norm = norm.to(cuda)
    wq = {'n_bits': 8, 'channel_wise': True, 'scale_method': 'max'}
    aq = {'n_bits': bits, 'symmetric': True, 'channel_wise': False, 'scale_method': 'max',
          'leaf_param': True, 'dynamic': True}
    mods = []
    for _ in range(2):
        q = m.QuantModule(lin, wq, aq, modulate=True).to(cuda)
        q.set_quant_state(True, True)
        mods.append(q)
    x = torch.randn(2, rows // 2 if rows % 2 == 0 else rows, c, device=cuda) if rows % 2 == 0 \
        else torch.randn(1, rows, c, device=cuda)
    for step in range(4):
        x = x + 0.05 * torch.randn_like(x)
        fused = mods[0](ops.LayerNormSource(x, norm))
        plain = mods[1](ops.layernorm(x, norm))
        assert torch.equal(fused, plain), step
        assert torch.equal(mods[0].a_hat, mods[1].a_hat), step
    bufs = [next(iter(q._geom_buffers.values())) for q in mods]
    assert torch.equal(bufs[0].x_scale, bufs[1].x_scale)
    assert torch.equal(bufs[0].codes, bufs[1].codes)


@pytest.mark.gpu
@pytest.mark.parametrize("b,cin,cout,hw", [(2, 320, 320, 32), (3, 640, 1280, 8)])
def test_pointwise_convolutions_around_tokens_need_no_rearrange(cuda, b, cin, cout, hw):
    """SpatialTransformer.proj_in / proj_out: the layer quantises in one layout and multiplies in
    the other (its caches follow the token-major tensor), and gives the bits of
    rearrange + convolution / convolution + rearrange, step after step."""
    import modiff_b200 as m
    from modiff_b200 import ops
    torch.manual_seed(5)
    conv = torch.nn.Conv2d(cin, cout, 1)
    wq = {'n_bits': 8, 'channel_wise': True, 'scale_method': 'max'}
    aq = {'n_bits': 8, 'symmetric': True, 'channel_wise': False, 'scale_method': 'max',
          'leaf_param': True, 'dynamic': True}

    def pair():
        mods = []
        for fused in (True, False):
            q = m.QuantModule(conv, wq, aq, modulate=True).to(cuda)
            q.set_quant_state(True, True)
            q.relayout_fusion = fused
            mods.append(q)
        return mods

    out_f, out_p = pair()          # NCHW in, tokens out
    in_f, in_p = pair()            # tokens in, NCHW out
    x = torch.randn(b, cin, hw, hw, device=cuda)
    for step in range(4):
        x = x + 0.05 * torch.randn_like(x)
        tok_f, tok_p = out_f.forward_tokens_out(x), out_p.forward_tokens_out(x)
        assert tuple(tok_f.shape) == (b, hw * hw, cout)
        assert torch.equal(tok_f, tok_p), step
        assert torch.equal(tok_f, ops.transpose_last2(out_p.o_hat.reshape(b, cout, hw * hw))), step
        t = ops.transpose_last2(x.reshape(b, cin, hw * hw))
        y_f, y_p = in_f.forward_tokens_in(t, hw, hw), in_p.forward_tokens_in(t, hw, hw)
        assert tuple(y_f.shape) == (b, cout, hw, hw)
        assert torch.equal(y_f, y_p), step
        if step:
            assert tuple(in_f.a_hat.shape) == (b, hw * hw, cin)          # cache in the token layout
            assert torch.equal(ops.transpose_last2(in_f.a_hat).reshape(b, cin, hw, hw), in_p.a_hat)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,n,cout,bits", [(2 * 1024, 1280, 320, 8), (154, 2560, 640, 8),
                                             (77, 5120, 1280, 6)])
def test_geglu_inside_the_quantiser_equals_the_separate_kernel(cuda, rows, n, cout, bits):
    """The feed-forward's gate in front of its quantised second linear layer is evaluated inside
    the quantiser's two passes (modiff_modq_geglu): same cached input, codes, scale and output,
    bit for bit, as the stand-alone GEGLU kernel followed by the plain quantiser."""
    import modiff_b200 as m
    from modiff_b200 import ops
    torch.manual_seed(4)
    lin = torch.nn.Linear(n, cout)
    wq = {'n_bits': 8, 'channel_wise': True, 'scale_method': 'max'}
    aq = {'n_bits': bits, 'symmetric': True, 'channel_wise': False, 'scale_method': 'max',
          'leaf_param': True, 'dynamic': True}
    mods = []
    for _ in range(2):
        q = m.QuantModule(lin, wq, aq, modulate=True).to(cuda)
        q.set_quant_state(True, True)
        mods.append(q)
    h = torch.randn(1, rows, 2 * n, device=cuda)
    for step in range(4):
        h = h + 0.05 * torch.randn_like(h)
        fused = mods[0](ops.GegluSource(h))
        plain = mods[1](ops.geglu(h))
        assert tuple(fused.shape) == (1, rows, cout)
        assert torch.equal(fused, plain), step
        assert torch.equal(mods[0].a_hat, mods[1].a_hat), step
    bufs = [next(iter(q._geom_buffers.values())) for q in mods]
    assert torch.equal(bufs[0].x_scale, bufs[1].x_scale)
    assert torch.equal(bufs[0].codes, bufs[1].codes)
