"""Kernel-level parity of the CUDA path (through the C ABI) against the CPU oracle:
bit-exact for codes, caches, scales and integer accumulators; fp tolerance stated per test."""
import ctypes as C

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import cases
import oracle
from oracle.quantizer import fake_quant, per_tensor_scale, quantize_codes

pytestmark = pytest.mark.gpu


def _lib():
    from modiff_b200 import _lib
    return _lib


def _geom(batch, cin, cout, h, w, k=1, stride=1, pad=(0, 0, 0, 0), split=0):
    L = _lib()
    pt, pl, pb, pr = pad
    return L.ConvGeom(batch, cin, cout, h, w, k, k, stride, pt, pl, pb, pr, split)


def _codes_to_nchw(codes, g, cin):
    """Undo the code-plane layout -> [B, C, H, W] int8 tensor (host)."""
    L = _lib()
    l = L.lib()
    s = g.stride
    hp = -(-(g.h + g.pad_t + g.pad_b) // s)
    wp = -(-(g.w + g.pad_l + g.pad_r) // s)
    cp = -(-cin // 16) * 16
    planes = codes.cpu().view(g.batch, s * s, hp, wp, cp)
    out = torch.zeros(g.batch, cin, g.h, g.w, dtype=torch.int8)
    for y in range(g.h):
        for x in range(g.w):
            yy, xx = y + g.pad_t, x + g.pad_l
            out[:, :, y, x] = planes[:, (yy % s) * s + xx % s, yy // s, xx // s, :cin]
    return out, planes


def run_modq(x, a_hat, g, n_bits, per_sample=False):
    L = _lib()
    l = L.lib()
    dev = x.device
    codes = torch.zeros(l.modiff_codes_bytes(C.byref(g)), dtype=torch.int8, device=dev)
    scale = torch.zeros(max(2, g.batch), dtype=torch.float32, device=dev)
    scratch = torch.zeros(64 + 4 * g.batch, dtype=torch.uint8, device=dev)
    L.check(l.modiff_modq(x.data_ptr(), L.ptr(a_hat), codes.data_ptr(), scale.data_ptr(),
                          C.byref(g), n_bits, int(per_sample), scratch.data_ptr(), L.stream_ptr()))
    torch.cuda.synchronize()
    assert int(scratch.to(torch.int32).abs().sum()) == 0, "scratch must be left zeroed"
    return codes, scale


@pytest.mark.parametrize("shape,bits,split,pad,stride", [
    ((2, 128, 8, 8), 8, 0, (1, 1, 1, 1), 1),
    ((2, 128, 8, 8), 4, 0, (1, 1, 1, 1), 1),
    ((3, 256, 4, 4), 3, 0, (1, 1, 1, 1), 1),
    ((2, 384, 8, 8), 4, 256, (0, 0, 0, 0), 1),
    ((2, 128, 8, 8), 8, 0, (0, 0, 1, 1), 2),
    ((2, 3, 8, 8), 8, 0, (1, 1, 1, 1), 1),
    ((2, 20, 5, 7), 8, 0, (1, 1, 1, 1), 1),       # ragged: hw % 4 != 0, cin % 16 != 0
    ((1, 128, 33, 33), 8, 0, (0, 0, 0, 0), 2),    # pre-padded downsample input
    ((4, 512, 1, 1), 8, 0, (0, 0, 0, 0), 1),      # linear
])
def test_modq_bit_exact(cuda, shape, bits, split, pad, stride):
    torch.manual_seed(5)
    b, c, h, w = shape
    x = torch.randn(shape)
    a = x + 0.1 * torch.randn(shape)
    g = _geom(b, c, 64, h, w, k=3 if pad[0] or stride == 2 else 1, stride=stride, pad=pad, split=split)
    a_dev = a.to(cuda)
    codes, scale = run_modq(x.to(cuda), a_dev, g, bits)
    r = x - a
    segs = [r[:, :split], r[:, split:]] if split else [r]
    exp_q, exp_d = [], []
    for sgm in segs:
        y, q, d, _ = fake_quant(sgm, bits, True)
        exp_q.append(q)
        exp_d.append(float(d))
    q = torch.cat(exp_q, dim=1)
    rq = torch.cat([qq * torch.tensor(d) for qq, d in zip(exp_q, exp_d)], dim=1)
    got, planes = _codes_to_nchw(codes, g, c)
    assert [float(v) for v in scale[:len(segs)].cpu()] == exp_d
    assert torch.equal(got.to(torch.float32), q)
    assert torch.equal(a_dev.cpu(), a + rq), "a_hat update must be bit-exact"
    # halo and padded channels stay zero
    assert int(planes.to(torch.int32).abs().sum()) == int(got.to(torch.int32).abs().sum())


def test_modq_zero_residual_and_plain_mode(cuda):
    """delta floor 1e-8 (qdiff/quant_layer.py:209-211) and a_hat == NULL (non-modulated)."""
    x = torch.randn(2, 128, 4, 4)
    g = _geom(2, 128, 64, 4, 4, k=3, pad=(1, 1, 1, 1))
    a = x.clone().to(cuda)
    codes, scale = run_modq(x.to(cuda), a, g, 8)
    assert float(scale[0]) == float(torch.tensor(1e-8))
    assert int(codes.to(torch.int32).abs().sum()) == 0
    assert torch.equal(a.cpu(), x)
    codes, scale = run_modq(x.to(cuda), None, g, 8)
    y, q, d, _ = fake_quant(x, 8, True)
    got, _ = _codes_to_nchw(codes, g, 128)
    assert float(scale[0]) == float(d) and torch.equal(got.float(), q)


def test_modq_per_sample(cuda):
    torch.manual_seed(6)
    x = torch.randn(3, 128, 4, 4) * torch.tensor([1.0, 5.0, 0.2]).view(3, 1, 1, 1)
    g = _geom(3, 128, 64, 4, 4)
    codes, scale = run_modq(x.to(cuda), None, g, 8, per_sample=True)
    y, q, d, _ = fake_quant(x, 8, True, channel_wise=True)
    got, _ = _codes_to_nchw(codes, g, 128)
    assert torch.equal(scale[:3].cpu(), d.reshape(-1))
    assert torch.equal(got.float(), q)


def _pack(w, g, bits, with_sum, dev):
    L = _lib()
    l = L.lib()
    gp = g.copy(batch=1)
    wcodes = torch.empty(l.modiff_wcodes_bytes(C.byref(gp), with_sum), dtype=torch.int8, device=dev)
    ws = torch.zeros(2 * g.cout, device=dev)
    wz = torch.zeros(2 * g.cout, device=dev)
    wc = torch.zeros(2 * g.cout, dtype=torch.int32, device=dev)
    taps = g.kh * g.kw
    wdq = torch.empty(g.cin * taps * g.cout, device=dev)
    w_d = w.to(dev).contiguous()
    L.check(l.modiff_weight_pack(w_d.data_ptr(), C.byref(gp), bits, with_sum,
                                 wcodes.data_ptr(), ws.data_ptr(), wz.data_ptr(), wc.data_ptr(),
                                 wdq.data_ptr(), L.stream_ptr()))
    torch.cuda.synchronize()
    return wcodes, ws, wz, wc, wdq


@pytest.mark.parametrize("bits,split,with_sum", [(8, 0, 1), (4, 0, 0), (4, 128, 0), (8, 128, 1), (8, 0, 0)])
def test_weight_pack_bit_exact(cuda, bits, split, with_sum):
    torch.manual_seed(7)
    cout, cin, k = 160, 256, 3
    w = torch.randn(cout, cin, k, k) * 0.05
    g = _geom(1, cin, cout, 8, 8, k=k, pad=(1, 1, 1, 1), split=split)
    wcodes, ws, wz, wc, wdq = _pack(w, g, bits, with_sum, cuda)
    segs = [(0, split), (split, cin)] if split else [(0, cin)]
    rows = (-(-cout // 128)) * 144 if with_sum else -(-cout // 128) * 128
    kp = -(-cin // 128) * 128
    codes = wcodes.cpu().view(rows, k * k, kp).to(torch.int32)
    for s, (cb, ce) in enumerate(segs):
        dq, q, d, zp = oracle.weight_codes(w[:, cb:ce].contiguous(), bits)
        assert torch.equal(ws[s * cout:(s + 1) * cout].cpu(), d.reshape(-1))
        assert torch.equal(wz[s * cout:(s + 1) * cout].cpu(), zp.reshape(-1))
        corr = wc[s * cout:(s + 1) * cout].cpu()
        for co in (0, 1, 127, 128, cout - 1):
            row = (co // 128) * 144 + co % 128 if with_sum else co
            got = codes[row, :, cb:ce] + corr[co] + zp.reshape(-1)[co].to(torch.int32)
            exp = q[co].reshape(ce - cb, k * k).t().to(torch.int32)
            assert torch.equal(got, exp)
        exp_dq = dq.reshape(cout, ce - cb, k * k)
        got_dq = wdq.cpu().view(cin, k * k, cout)[cb:ce].permute(2, 0, 1)
        assert torch.equal(got_dq, exp_dq)
    if with_sum:
        assert torch.equal(codes[128, :, :cin], torch.ones(k * k, cin, dtype=torch.int32))
        assert int(codes[129:144].abs().sum()) == 0


def _run_igemm(x_codes, w, g, bits_w, impl, dev, x_scale=(0.01, 0.02), accumulate=True, bias=None,
               want_acc=True):
    """x_codes: [B, C, H, W] int8 (host).  Returns (out, acc) from the device."""
    L = _lib()
    l = L.lib()
    with_sum = 1 if bits_w >= 8 else 0
    wcodes, ws, wz, wc, wdq = _pack(w, g, bits_w, with_sum, dev)
    if bool(wc.any()) and not with_sum:     # corrections need the receptive-field-sum rows
        with_sum = 1
        wcodes, ws, wz, wc, wdq = _pack(w, g, bits_w, with_sum, dev)
    # place the codes through the static quantiser (delta = 1 -> codes = rne(x))
    codes = torch.zeros(l.modiff_codes_bytes(C.byref(g)), dtype=torch.int8, device=dev)
    one = torch.ones(2, device=dev)
    xf = x_codes.to(torch.float32).to(dev).contiguous()
    L.check(l.modiff_quantize_static(xf.data_ptr(), one.data_ptr(), codes.data_ptr(), C.byref(g), 8,
                                     L.stream_ptr()))
    ho, wo = L.out_hw(g)
    torch.manual_seed(9)
    o_prev = torch.randn(g.batch, g.cout, ho, wo)
    o_hat = o_prev.clone().to(dev)
    xs = torch.tensor(list(x_scale), dtype=torch.float32, device=dev)
    nseg = 2 if g.split else 1
    acc = torch.zeros(nseg * g.batch * ho * wo * g.cout, dtype=torch.int32, device=dev)
    need_corr = bool(wc.any())
    L.check(l.modiff_igemm_conv(codes.data_ptr(), wcodes.data_ptr(), with_sum, xs.data_ptr(),
                                ws.data_ptr(), wc.data_ptr() if need_corr else None,
                                o_hat.data_ptr(), int(accumulate), L.ptr(bias), C.byref(g), 0, impl,
                                acc.data_ptr() if want_acc else None, L.stream_ptr()))
    torch.cuda.synchronize()
    assert L.device_status() == 0, "a bounded wait ran out inside the kernel"
    return o_hat.cpu(), acc.cpu().view(nseg, g.batch, ho, wo, g.cout), o_prev, ws.cpu()


IGEMM_CASES = [
    # batch, cin, cout, hw, k, stride, pad, split, w_bits
    (2, 128, 128, 8, 3, 1, (1, 1, 1, 1), 0, 4),
    (2, 128, 128, 8, 3, 1, (1, 1, 1, 1), 0, 8),
    (1, 256, 256, 32, 3, 1, (1, 1, 1, 1), 0, 4),
    (3, 384, 128, 16, 1, 1, (0, 0, 0, 0), 256, 4),
    (3, 256, 128, 4, 1, 1, (0, 0, 0, 0), 128, 8),
    (2, 128, 128, 16, 3, 2, (0, 0, 1, 1), 0, 8),
    (9, 256, 256, 4, 3, 1, (1, 1, 1, 1), 0, 4),     # 8 images per tile, ragged last tile
    (5, 512, 256, 1, 1, 1, (0, 0, 0, 0), 0, 8),     # linear
    (2, 128, 3, 8, 3, 1, (1, 1, 1, 1), 0, 4),       # conv_out: 3 channels
    (2, 640, 200, 8, 3, 1, (1, 1, 1, 1), 0, 8),     # cin/cout not multiples of 128
]


def _expected_acc(x_codes, w, g, bits):
    segs = [(0, g.split), (g.split, g.cin)] if g.split else [(0, g.cin)]
    accs, dws = [], []
    for cb, ce in segs:
        dq, q, d, zp = oracle.weight_codes(w[:, cb:ce].contiguous(), bits)
        wi = (q - zp).double()
        xi = x_codes[:, cb:ce].double()
        xi = F.pad(xi, (g.pad_l, g.pad_r, g.pad_t, g.pad_b))
        accs.append(F.conv2d(xi, wi, None, stride=g.stride).round().to(torch.int64))
        dws.append(d.reshape(-1))
    return accs, dws


@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
@pytest.mark.parametrize("case", IGEMM_CASES, ids=lambda c: "b%d_c%d_o%d_hw%d_k%d_s%d_sp%d_w%d" % (
    c[0], c[1], c[2], c[3], c[4], c[5], c[7], c[8]))
def test_igemm_accumulators_exact(cuda, case, impl):
    b, cin, cout, hw, k, stride, pad, split, bits = case
    L = _lib()
    g = _geom(b, cin, cout, hw, hw, k=k, stride=stride, pad=pad, split=split)
    torch.manual_seed(8)
    x_codes = torch.randint(-127, 128, (b, cin, hw, hw), dtype=torch.int8)
    w = torch.randn(cout, cin, k, k) * 0.05
    w[1] = w[1].abs() + 0.01   # an all-positive channel: zero point outside the code range
    out, acc, o_prev, ws = _run_igemm(x_codes, w, g, bits,
                                      L.IMPL_SIMT if impl == "simt" else L.IMPL_TCGEN05, cuda)
    exp_acc, dws = _expected_acc(x_codes, w, g, bits)
    xs = (0.01, 0.02)
    exp = o_prev.double()
    for s, (a, dw) in enumerate(zip(exp_acc, dws)):
        assert torch.equal(acc[s].permute(0, 3, 1, 2).to(torch.int64), a), f"segment {s} accumulators"
        exp = exp + a.double() * (float(np.float32(xs[s])) * dw.double().view(1, -1, 1, 1))
    err = (out.double() - exp).abs().max() / exp.abs().max()
    assert err < 1e-5, err    # fp32 epilogue vs float64 evaluation of the same integers


HALO_CASES = [
    # batch, cin, cout, hw: 3x3 stride-1 pad-1 layers that take the activation-reuse kernel
    (5, 128, 128, 32),      # 256-pixel tiles (8 rows), one K chunk
    (3, 256, 256, 16),      # whole image per tile or 8-row tiles, two K chunks, two channel tiles
    (1, 320, 128, 64),      # 4-row tiles, last K chunk partly beyond cin
    (2, 192, 384, 16),      # three channel tiles
    (150, 128, 128, 16),    # more tiles than SMs: every CTA walks several tiles
    (80, 512, 256, 16),     # four K chunks, 256 output channels per tile, several tiles per pair
    (6, 192, 192, 32),      # latent-UNet width: K chunk and last channel tile half empty
    (4, 320, 320, 16),      # SD width: 2.5 channel tiles
]


@pytest.mark.parametrize("w_bits", [4, 8])
@pytest.mark.parametrize("accumulate", [True, False])
@pytest.mark.parametrize("case", HALO_CASES, ids=lambda c: "b%d_c%d_o%d_hw%d" % c)
def test_igemm_activation_reuse_kernel(cuda, case, accumulate, w_bits, monkeypatch):
    """The 3x3 kernels that reuse one activation copy for three filter taps - the two-SM kernel
    (cta_group::2, both tile heights) and the single-CTA one - give the same bits as the
    one-copy-per-tap kernel and match the exact integer convolution."""
    b, cin, cout, hw = case
    L = _lib()
    g = _geom(b, cin, cout, hw, hw, k=3, stride=1, pad=(1, 1, 1, 1))
    torch.manual_seed(12)
    x_codes = torch.randint(-8, 8, (b, cin, hw, hw), dtype=torch.int8)
    w = torch.randn(cout, cin, 3, 3) * 0.05
    w[1] = w[1].abs() + 0.01   # an all-positive channel: zero point outside the code range
    outs = {}
    for name, pair, halo, mh in (("pair, 128-pixel tiles", "1", "1", "1"),
                                 ("pair, 256-pixel tiles", "1", "1", "2"),
                                 ("single CTA", "0", "1", ""), ("per tap", "0", "0", "")):
        monkeypatch.setenv("MODIFF_IGEMM_PAIR", pair)
        monkeypatch.setenv("MODIFF_IGEMM_HALO", halo)
        monkeypatch.setenv("MODIFF_PAIR_MH", mh)
        out, _, o_prev, ws = _run_igemm(x_codes, w, g, w_bits, L.IMPL_TCGEN05, cuda,
                                        accumulate=accumulate, want_acc=False)
        outs[name] = out
    for name, out in outs.items():
        assert torch.equal(out, outs["per tap"]), name
    exp_acc, dws = _expected_acc(x_codes, w, g, w_bits)
    exp = o_prev.double() if accumulate else torch.zeros_like(o_prev).double()
    exp = exp + exp_acc[0].double() * (float(np.float32(0.01)) * dws[0].double().view(1, -1, 1, 1))
    err = (outs["per tap"].double() - exp).abs().max() / exp.abs().max()
    assert err < 1e-5, err


KSPLIT_CASES = [
    # batch, cin, cout, hw, k, w_bits: few output tiles and a long K range
    (32, 768, 768, 2, 3, 8),      # latent UNet's deepest level: 6 tiles, clusters of 8
    (32, 768, 768, 4, 3, 8),      # 24 tiles, clusters of 4
    (8, 512, 384, 4, 3, 4),       # 3 tiles, clusters of 4 (36 K iterations), no sum rows
    (7, 768, 200, 2, 3, 8),       # ragged rows and channels
    (3, 4096, 320, 1, 1, 8),      # linear layer with three rows, 32 K iterations, clusters of 4
]


@pytest.mark.parametrize("accumulate", [True, False])
@pytest.mark.parametrize("case", KSPLIT_CASES, ids=lambda c: "b%d_c%d_o%d_hw%d_k%d_w%d" % c)
def test_igemm_k_range_split_across_a_cluster(cuda, case, accumulate, monkeypatch):
    """Layers with fewer tiles than SMs: clusters of CTAs share each tile's K range and add their
    int32 partial sums through distributed shared memory.  Outputs and accumulators equal the
    unsplit kernel's bit for bit, and the accumulators equal the exact integer convolution."""
    b, cin, cout, hw, k, w_bits = case
    L = _lib()
    pad = (1, 1, 1, 1) if k == 3 else (0, 0, 0, 0)
    g = _geom(b, cin, cout, hw, hw, k=k, stride=1, pad=pad)
    torch.manual_seed(14)
    x_codes = torch.randint(-127, 128, (b, cin, hw, hw), dtype=torch.int8)
    w = torch.randn(cout, cin, k, k) * 0.05
    w[1] = w[1].abs() + 0.01
    bias = torch.randn(cout).to(cuda) if not accumulate else None
    for want_acc in (True, False):      # False: the unsplit kernel takes its bulk-copy epilogue
        res = {}
        for name, allow in (("split", "8"), ("unsplit", "1")):
            monkeypatch.setenv("MODIFF_TC_KSPLIT", allow)
            monkeypatch.setenv("MODIFF_IGEMM_HALO", "0")
            monkeypatch.setenv("MODIFF_IGEMM_PAIR", "0")
            res[name] = _run_igemm(x_codes, w, g, w_bits, L.IMPL_TCGEN05, cuda,
                                   accumulate=accumulate, bias=bias, want_acc=want_acc)
        assert torch.equal(res["split"][0], res["unsplit"][0]), want_acc
        if want_acc:
            assert torch.equal(res["split"][1], res["unsplit"][1])
            exp_acc, _ = _expected_acc(x_codes, w, g, w_bits)
            assert torch.equal(res["split"][1][0].permute(0, 3, 1, 2).to(torch.int64), exp_acc[0])


def test_conv_fp32_matches_torch(cuda):
    """First-step path: fp32 activations x dequantised weights + bias, tolerance 1e-4 relative
    to the output range (north-star bound for per-layer outputs is 1e-3)."""
    L = _lib()
    l = L.lib()
    torch.manual_seed(10)
    for (b, cin, cout, hw, k, stride, pad) in [(2, 128, 96, 8, 3, 1, (1, 1, 1, 1)),
                                               (2, 3, 128, 8, 3, 1, (1, 1, 1, 1)),
                                               (3, 64, 64, 9, 3, 2, (0, 0, 0, 0)),
                                               (5, 512, 300, 1, 1, 1, (0, 0, 0, 0))]:
        x = torch.randn(b, cin, hw, hw)
        w = torch.randn(cout, cin, k, k) * 0.05
        bias = torch.randn(cout)
        g = _geom(b, cin, cout, hw, hw, k=k, stride=stride, pad=pad)
        w_kn = w.reshape(cout, -1).t().contiguous().to(cuda)
        x_d, bias_d = x.to(cuda), bias.to(cuda)     # keep the device copies alive
        ho, wo = L.out_hw(g)
        out = torch.empty(b, cout, ho, wo, device=cuda)
        L.check(l.modiff_conv_fp32(x_d.data_ptr(), w_kn.data_ptr(), bias_d.data_ptr(),
                                   out.data_ptr(), C.byref(g), L.stream_ptr()))
        exp = F.conv2d(x.double(), w.double(), bias.double(), stride=stride,
                       padding=(pad[0], pad[1]))
        err = (out.cpu().double() - exp).abs().max() / exp.abs().max()
        assert err < 1e-5, err


@pytest.mark.parametrize("c", cases.QUANTIZER_CASES, ids=lambda c: c["name"])
def test_fake_quant_matches_reference_fixture(cuda, c, golden_quantizer):
    """UniformAffineQuantizer.forward on the device against the reference's own outputs."""
    from modiff_b200 import UniformAffineQuantizer
    x = cases.quantizer_input(c)
    q = UniformAffineQuantizer(n_bits=c["n_bits"], symmetric=c["sym"], channel_wise=c["channel_wise"],
                               scale_method="max", always_zero=c.get("always_zero", False),
                               dynamic=True)
    y = q(x.to(cuda))
    g = golden_quantizer
    np.testing.assert_array_equal(q.delta.cpu().numpy().reshape(-1), g[c["name"] + "/delta"])
    np.testing.assert_array_equal(q.zero_point.cpu().numpy().reshape(-1), g[c["name"] + "/zp"])
    np.testing.assert_array_equal(y.cpu().numpy(), g[c["name"] + "/y"])


def test_graph_kernels_match_torch(cuda):
    from modiff_b200 import ops
    torch.manual_seed(11)
    x = torch.randn(3, 64, 8, 8)
    x1 = torch.randn(3, 32, 8, 8)
    gn = torch.nn.GroupNorm(32, 96, eps=1e-6)
    with torch.no_grad():
        gn.weight.normal_()
        gn.bias.normal_()
    exp = F.group_norm(torch.cat([x, x1], 1), 32, gn.weight, gn.bias, 1e-6)
    gn_d = gn.to(cuda)
    got = ops.groupnorm(x.to(cuda), gn_d, silu=False, x1=x1.to(cuda)).cpu()
    assert (got - exp).abs().max() < 2e-5
    got = ops.groupnorm(torch.cat([x, x1], 1).to(cuda), gn_d, silu=True).cpu()
    assert (got - exp * torch.sigmoid(exp)).abs().max() < 2e-5
    # odd spatial size: scalar path
    xo = torch.randn(2, 64, 5, 3)
    gn2 = torch.nn.GroupNorm(32, 64, eps=1e-6).to(cuda)
    exp = F.group_norm(xo, 32, gn2.weight.cpu(), gn2.bias.cpu(), 1e-6)
    assert (ops.groupnorm(xo.to(cuda), gn2).cpu() - exp).abs().max() < 2e-5
    xd = x.to(cuda)
    assert (ops.silu(xd).cpu() - x * torch.sigmoid(x)).abs().max() < 1e-6
    assert torch.equal(ops.add(xd, xd).cpu(), x + x)
    bc = torch.randn(3, 64)
    assert torch.equal(ops.add_channel_bias(xd, bc.to(cuda)).cpu(), x + bc[:, :, None, None])
    assert torch.equal(ops.upsample2x(xd).cpu(), F.interpolate(x, scale_factor=2.0, mode="nearest"))
    assert torch.equal(ops.concat_channels(xd, x1.to(cuda)).cpu(), torch.cat([x, x1], 1))
    t = torch.tensor([0.0, 1.0, 37.0, 999.0])
    exp = oracle.unet.timestep_embedding(t, 128)
    assert (ops.timestep_embedding(t.to(cuda), 128).cpu() - exp).abs().max() < 2e-6
    q = torch.randn(2, 64, 48)
    k = torch.randn(2, 64, 48)
    v = torch.randn(2, 64, 48)
    w_ = torch.softmax(torch.bmm(q.permute(0, 2, 1), k) * 0.125, dim=2)
    exp = torch.bmm(v, w_.permute(0, 2, 1))
    assert (ops.attention(q.to(cuda), k.to(cuda), v.to(cuda), 0.125).cpu() - exp).abs().max() < 1e-4


def test_ddim_step_bit_exact(cuda):
    from modiff_b200 import ops
    from modiff_b200.sampler import alpha_table, step_coefficients, get_beta_schedule
    torch.manual_seed(12)
    x, e, nz = torch.randn(2, 3, 32, 32), torch.randn(2, 3, 32, 32), torch.randn(2, 3, 32, 32)
    betas = torch.from_numpy(get_beta_schedule()).float()
    alphas = alpha_table(betas)
    for (i, j, eta) in [(800, 783, 0.0), (0, -1, 0.0), (500, 400, 0.5)]:
        t = torch.full((2,), i, dtype=torch.long)
        tn = torch.full((2,), j, dtype=torch.long)
        at = oracle.sampler.compute_alpha(betas, t)
        an = oracle.sampler.compute_alpha(betas, tn)
        x0 = (x - e * (1 - at).sqrt()) / at.sqrt()
        c1 = eta * ((1 - at / an) * (1 - an) / (1 - at)).sqrt()
        c2 = ((1 - an) - c1 ** 2).sqrt()
        exp = an.sqrt() * x0 + c1 * nz + c2 * e
        co = step_coefficients(alphas, i, j, eta)
        got, got0 = ops.ddim_step(x.to(cuda), e.to(cuda), *co, noise=nz.to(cuda) if eta else None,
                                  want_x0=True)
        assert torch.equal(got0.cpu(), x0)
        assert torch.equal(got.cpu(), exp)


def test_int4_pack_roundtrip(cuda):
    from modiff_b200 import ops
    codes = torch.randint(-8, 8, (1001,), dtype=torch.int8)
    packed = ops.pack_int4(codes.to(cuda))
    exp = ((codes[0::2].to(torch.int32) & 0xf) |
           (torch.cat([codes[1::2], torch.zeros(1, dtype=torch.int8)]).to(torch.int32) & 0xf) << 4)
    assert torch.equal(packed.cpu().to(torch.int32), exp)   # element 2i low nibble, 2i+1 high
    assert torch.equal(ops.unpack_int4(packed, 1001).cpu(), codes)
    u = torch.randint(0, 16, (64,), dtype=torch.int8)
    assert torch.equal(ops.unpack_int4(ops.pack_int4(u.to(cuda)), 64, signed=False).cpu(), u)


@pytest.mark.parametrize("mode,n", [(1, 128), (1, 256), (2, 128), (2, 256)])
def test_i8_mma_probe_layout(cuda, mode, n):
    """The tensor-pipe probe's accumulators equal iters * A B^T exactly, for a single CTA
    (cta_group::1, M = 128) and for a CTA pair (cta_group::2, M = 256 with A's rows and B's
    rows split between the two CTAs' shared memory): pins the operand and accumulator layout
    both GEMM issue modes rely on."""
    L = _lib()
    units, iters = 2, 3
    m = 128 * mode
    g = torch.Generator().manual_seed(40 + n + mode)
    a = torch.randint(-127, 128, (units * m, 128), generator=g, dtype=torch.int8)
    b = torch.randint(-127, 128, (n, 128), generator=g, dtype=torch.int8)
    acc = torch.zeros(m, n, dtype=torch.int32, device=cuda)
    dbg = torch.full((4,), -1, dtype=torch.int32, device=cuda)
    a_d, b_d = a.to(cuda), b.to(cuda)
    L.call('modiff_i8_mma_probe', mode, n, iters, units, a_d.data_ptr(), b_d.data_ptr(),
           acc.data_ptr(), dbg.data_ptr(), L.stream_ptr())
    torch.cuda.synchronize()
    assert L.device_status() == 0, "the probe gave up on a bounded wait"
    print("tensor-memory bases / ranks of unit 0:", dbg.cpu().tolist())
    want = iters * (a[:m].to(torch.int64) @ b.to(torch.int64).t())
    assert torch.equal(acc.cpu().to(torch.int64), want)


def test_i8_peak_is_plausible(cuda):
    """The measured kind::i8 ceiling lies between a quarter of and a little above the nominal
    4.5 POPS (a sanity check of the probe's operation count, not a performance assertion)."""
    L = _lib()
    tops = L.measure_i8_peak(mode=1, umma_n=256, iters=2048, repeats=3)
    print(f"kind::i8 ceiling, cta_group::1 N=256: {tops:.0f} TOPS")
    assert 1100 < tops < 5500, tops


def test_bounded_wait_gives_up_and_the_library_recovers(cuda):
    """Failure detection on the device, without a fault: a wait that nothing satisfies runs out
    after its limit (1 ms here), the kernel RETURNS, the sticky status word reports it, a reset
    clears it, and the next ordinary call is bit-exact (the context stays usable)."""
    L = _lib()
    assert L.device_status() == 0
    gave_up = torch.zeros(1, dtype=torch.int32, device=cuda)
    L.call('modiff_wait_probe', 1_000_000, gave_up.data_ptr(), L.stream_ptr())
    torch.cuda.synchronize()
    assert int(gave_up) == 1
    assert L.device_status(reset=False) & 1, "the status word must record the timed-out wait"
    assert L.device_status(reset=True) & 1
    assert L.device_status() == 0, "reset must clear it"
    # samplers turn the flag into an exception
    from modiff_b200.sampler import raise_on_device_status
    L.call('modiff_wait_probe', 1_000_000, None, L.stream_ptr())
    with pytest.raises(L.ModiffError):
        raise_on_device_status()
    assert L.device_status() == 0
    # and the library still computes correctly afterwards
    torch.manual_seed(9)
    x = torch.randn(2, 128, 8, 8)
    a = x + 0.1 * torch.randn(2, 128, 8, 8)
    g = _geom(2, 128, 64, 8, 8, k=3, pad=(1, 1, 1, 1))
    a_dev = a.to(cuda)
    codes, scale = run_modq(x.to(cuda), a_dev, g, 8)
    y, q, d, _ = fake_quant(x - a, 8, True)
    got, _ = _codes_to_nchw(codes, g, 128)
    assert float(scale[0]) == float(d) and torch.equal(got.float(), q)
    with pytest.raises(L.ModiffError):
        L.call('modiff_wait_probe', 2_000_000_000, None, L.stream_ptr())   # limit above the cap


PACKED4_CASES = [
    # batch, cin, cout, hw
    (3, 256, 256, 16),      # two K chunks, two channel tiles
    (5, 128, 128, 32),      # 4-row tiles
    (150, 128, 128, 16),    # more tiles than SMs
    (1, 384, 128, 64),      # 2-row tiles, three K chunks
]


@pytest.mark.parametrize("accumulate", [True, False])
@pytest.mark.parametrize("case", PACKED4_CASES, ids=lambda c: "b%d_c%d_o%d_hw%d" % c)
def test_packed_int4_operands_give_the_same_bits(cuda, case, accumulate):
    """W4 weight codes and 4-bit activation codes stored two per byte (the nibble order of
    qdiff/quant_layer_int4.py:341-346) and expanded to int8 in shared memory: the output equals
    the byte-per-code kernel's bit for bit, and the packed buffers are half the size."""
    b, cin, cout, hw = case
    L = _lib()
    l = L.lib()
    g = _geom(b, cin, cout, hw, hw, k=3, stride=1, pad=(1, 1, 1, 1))
    torch.manual_seed(14)
    x_codes = torch.randint(-8, 8, (b, cin, hw, hw), dtype=torch.int8)
    w = torch.randn(cout, cin, 3, 3) * 0.05
    ref, _, o_prev, ws = _run_igemm(x_codes, w, g, 4, L.IMPL_TCGEN05, cuda, accumulate=accumulate,
                                    want_acc=False)
    wcodes, ws, wz, wc, wdq = _pack(w, g, 4, 0, cuda)
    assert not bool(wc.any())
    codes = torch.zeros(l.modiff_codes_bytes(C.byref(g)), dtype=torch.int8, device=cuda)
    one = torch.ones(2, device=cuda)
    xf = x_codes.to(torch.float32).to(cuda).contiguous()
    L.check(l.modiff_quantize_static(xf.data_ptr(), one.data_ptr(), codes.data_ptr(), C.byref(g), 8,
                                     L.stream_ptr()))
    codes4 = torch.empty(codes.numel() // 2, dtype=torch.uint8, device=cuda)
    L.check(l.modiff_pack_int4(codes.data_ptr(), codes4.data_ptr(), codes.numel(), L.stream_ptr()))
    w4 = torch.empty(wcodes.numel() // 2, dtype=torch.uint8, device=cuda)
    bad = torch.zeros(1, dtype=torch.int32, device=cuda)
    L.check(l.modiff_pack_weights_int4(wcodes.data_ptr(), wz.data_ptr(), w4.data_ptr(), cout,
                                       wcodes.numel() // cout, bad.data_ptr(), L.stream_ptr()))
    assert int(bad) == 0
    o_hat = o_prev.clone().to(cuda)
    xs = torch.tensor([0.01, 0.02], dtype=torch.float32, device=cuda)
    L.check(l.modiff_igemm_conv_packed4(codes4.data_ptr(), w4.data_ptr(), wz.data_ptr(),
                                        xs.data_ptr(), ws.data_ptr(), o_hat.data_ptr(),
                                        int(accumulate), C.byref(g), None, None, L.stream_ptr()))
    torch.cuda.synchronize()
    assert L.device_status() == 0, "a bounded wait ran out inside the kernel"
    assert torch.equal(o_hat.cpu(), ref)
    # the nibble convention: element 2i in the low nibble, 2i + 1 in the high nibble
    c8, c4 = codes.cpu().view(-1)[:64].to(torch.int32), codes4.cpu().view(-1)[:32].to(torch.int32)
    assert torch.equal(c4 & 15, c8[0::2] & 15) and torch.equal(c4 >> 4, c8[1::2] & 15)


def test_packed_int4_layer_switch(cuda, monkeypatch):
    """QuantModule.packed_int4 routes an eligible W4A4 layer through the packed kernel: same
    outputs and caches as the default path over three modulated steps."""
    import modiff_b200 as m
    torch.manual_seed(3)
    org = torch.nn.Conv2d(128, 128, 3, padding=1)
    wq = {'n_bits': 4, 'channel_wise': True, 'scale_method': 'max'}
    aq = {'n_bits': 4, 'symmetric': True, 'channel_wise': False, 'scale_method': 'max',
          'leaf_param': True, 'dynamic': True}
    outs = []
    for packed in (False, True):
        mod = m.QuantModule(org, wq, aq, modulate=True).to(cuda)
        mod.set_quant_state(True, True)
        mod.packed_int4 = packed
        mod.alias_output = False
        g = torch.Generator().manual_seed(4)
        x0 = torch.randn(4, 128, 32, 32, generator=g)
        ys = []
        with torch.no_grad():
            for step in range(3):
                ys.append(mod((x0 + 0.05 * step * torch.randn(x0.shape, generator=g)).to(cuda)))
        outs.append((ys, mod.a_hat.clone(), mod._wpack.get('wcodes4') is not None))
    assert outs[1][2] and not outs[0][2]
    for a, b in zip(outs[0][0], outs[1][0]):
        assert torch.equal(a, b)
    assert torch.equal(outs[0][1], outs[1][1])
    assert m.device_status() == 0


@pytest.mark.parametrize("rows,cin,cout,w_bits", [(300, 512, 320, 8), (4096, 320, 2560, 8),
                                                  (128, 128, 200, 4), (1000, 640, 640, 4)])
@pytest.mark.parametrize("accumulate", [True, False])
def test_linear_layers_bulk_copy_epilogue(cuda, rows, cin, cout, w_bits, accumulate):
    """Token-major outputs [rows][cout] of linear layers with at least 128 rows travel through the
    cached-output ring as swizzled 128 x 32 boxes: equal to the exact integer product (1e-5) and to
    the CUDA-core kernel, ragged row and channel counts included."""
    L = _lib()
    g = _geom(rows, cin, cout, 1, 1, k=1)
    torch.manual_seed(15)
    x_codes = torch.randint(-127, 128, (rows, cin, 1, 1), dtype=torch.int8)
    w = torch.randn(cout, cin, 1, 1) * 0.05
    w[1] = w[1].abs() + 0.01
    out_tc, _, o_prev, _ = _run_igemm(x_codes, w, g, w_bits, L.IMPL_TCGEN05, cuda,
                                      accumulate=accumulate, want_acc=False)
    out_simt, _, _, _ = _run_igemm(x_codes, w, g, w_bits, L.IMPL_SIMT, cuda, accumulate=accumulate,
                                   want_acc=False)
    exp_acc, dws = _expected_acc(x_codes, w, g, w_bits)
    exp = o_prev.double() if accumulate else torch.zeros_like(o_prev).double()
    exp = exp + exp_acc[0].double() * (float(np.float32(0.01)) * dws[0].double().view(1, -1, 1, 1))
    err = (out_tc.double() - exp).abs().max() / exp.abs().max()
    assert err < 1e-5, err
    assert (out_tc - out_simt).abs().max() <= 1e-6 * exp.abs().max()
