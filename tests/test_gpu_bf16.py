"""Split-bf16 tensor-core GEMM (first sampling step, attention) against float64 evaluations of
the same operands.  Tolerance 1e-4 of the output range: the split keeps ~16 mantissa bits per
operand, the stated per-layer bound is 1e-3."""
import ctypes as C

import pytest
import torch
import torch.nn.functional as F

import cases
import oracle

pytestmark = pytest.mark.gpu

CASES = [
    # batch, cin, cout, hw, k, stride, pad(t,l,b,r), split
    (2, 128, 128, 8, 3, 1, (1, 1, 1, 1), 0),
    (1, 256, 128, 32, 3, 1, (1, 1, 1, 1), 0),
    (3, 384, 128, 16, 1, 1, (0, 0, 0, 0), 256),
    (2, 128, 128, 16, 3, 2, (0, 0, 1, 1), 0),
    (9, 256, 256, 4, 3, 1, (1, 1, 1, 1), 0),
    (5, 512, 200, 1, 1, 1, (0, 0, 0, 0), 0),
    (2, 64, 16, 8, 1, 1, (0, 0, 0, 0), 0),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "b%d_c%d_o%d_hw%d_k%d_s%d_sp%d" % (
    c[0], c[1], c[2], c[3], c[4], c[5], c[7]))
@pytest.mark.parametrize("bits", [4, 8])
def test_first_step_conv_on_tensor_cores(cuda, case, bits):
    from modiff_b200 import _lib as L
    b, cin, cout, hw, k, stride, pad, split = case
    l = L.lib()
    g = L.ConvGeom(b, cin, cout, hw, hw, k, k, stride, pad[0], pad[1], pad[2], pad[3], split)
    torch.manual_seed(21)
    x = torch.randn(b, cin, hw, hw)
    w = torch.randn(cout, cin, k, k) * 0.05
    bias = torch.randn(cout)
    gp = g.copy(batch=1)
    x_d, w_d, bias_d = x.to(cuda), w.to(cuda).contiguous(), bias.to(cuda)
    wcodes = torch.empty(l.modiff_wcodes_bytes(C.byref(gp), 1), dtype=torch.int8, device=cuda)
    ws = torch.zeros(2 * cout, device=cuda)
    wz = torch.zeros(2 * cout, device=cuda)
    wc = torch.zeros(2 * cout, dtype=torch.int32, device=cuda)
    L.check(l.modiff_weight_pack(w_d.data_ptr(), C.byref(gp), bits, 1, wcodes.data_ptr(),
                                 ws.data_ptr(), wz.data_ptr(), wc.data_ptr(), None, L.stream_ptr()))
    wb = torch.empty(l.modiff_weights_bf16_bytes(C.byref(gp)) // 2, dtype=torch.int16, device=cuda)
    L.check(l.modiff_weights_bf16(w_d.data_ptr(), ws.data_ptr(), wz.data_ptr(), wb.data_ptr(),
                                  C.byref(gp), bits, L.stream_ptr()))
    planes = torch.zeros(l.modiff_bf16_planes_bytes(C.byref(g)) // 2, dtype=torch.int16, device=cuda)
    L.check(l.modiff_split_bf16(x_d.data_ptr(), planes.data_ptr(), C.byref(g), L.stream_ptr()))
    ho, wo = L.out_hw(g)
    out = torch.full((b, cout, ho, wo), float("nan"), device=cuda)
    kb = max(64, -(-cin // 8) * 8)
    desc = L.GemmBf16Desc(planes.data_ptr(), wb.data_ptr(), ws.data_ptr(), bias_d.data_ptr(),
                          out.data_ptr(), 2, 1, 0, kb, 1.0, 0)
    L.check(l.modiff_gemm_bf16(C.byref(desc), C.byref(g), L.stream_ptr()))
    torch.cuda.synchronize()
    assert L.device_status() == 0
    segs = [(0, split), (split, cin)] if split else [(0, cin)]
    dq = torch.cat([oracle.weight_codes(w[:, a:e].contiguous(), bits)[0] for a, e in segs], dim=1)
    xp = F.pad(x.double(), (pad[1], pad[3], pad[0], pad[2]))
    exp = F.conv2d(xp, dq.double(), bias.double(), stride=stride)
    err = (out.cpu().double() - exp).abs().max() / exp.abs().max()
    assert err < 1e-4, err


@pytest.mark.parametrize("b,c,t,tk", [(3, 256, 256, 256), (2, 64, 64, 64), (5, 256, 16, 16),
                                      (2, 128, 1024, 1024), (16, 24, 1024, 1024), (8, 40, 256, 77),
                                      (4, 160, 64, 77), (8, 96, 4, 4),
                                      # single-kernel path: many tiles per CTA, masked padded keys,
                                      # 192 channels, ragged query tile
                                      (300, 256, 256, 256), (4, 128, 256, 200), (3, 192, 128, 128),
                                      (2, 64, 128, 150)])
def test_attention_matches_float64(cuda, b, c, t, tk):
    from modiff_b200 import ops
    import modiff_b200 as m
    torch.manual_seed(22)
    q, k, v = torch.randn(b, c, t), torch.randn(b, c, tk), torch.randn(b, c, tk)
    scale = float(c) ** -0.5
    w_ = torch.softmax(torch.bmm(q.double().permute(0, 2, 1), k.double()) * scale, dim=2)
    exp = torch.bmm(v.double(), w_.permute(0, 2, 1))
    got = ops.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale)
    torch.cuda.synchronize()
    assert m.device_status() == 0
    err = (got.cpu().double() - exp).abs().max() / exp.abs().max()
    assert err < 1e-4, err
