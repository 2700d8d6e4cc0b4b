"""modiff_modq_static: the quantiser entry point that brings its own scratch memory.

Some hosts of this library may not allocate device memory while they run (their memory is
partitioned once at start-up, and a cudaMalloc in the hot loop both stalls the device and can
fail against that fixed budget), and they have no spare buffer to lend as scratch.  For them the
library carries a small built-in scratch array.  This test drives that entry point through the
C ABI and requires bit-identical codes, cache and scales to modiff_modq (caller-owned scratch),
and the same scales and cache as the CPU restatement of the reference quantiser, on two
consecutive calls, because the built-in array is shared and keeps the previous call's
contents.  The file name sorts last so every other test has already run when this one does.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(entry, x, a_hat, g, bits, per_sample, dev):
    from modiff_b200 import _lib as L
    l = L.lib()
    codes = torch.zeros(l.modiff_codes_bytes(C.byref(g)), dtype=torch.int8, device=dev)
    scale = torch.zeros(max(2, g.batch), dtype=torch.float32, device=dev)
    if entry == "modiff_modq":
        scratch = torch.zeros(64 + 4 * g.batch, dtype=torch.uint8, device=dev)
        L.check(l.modiff_modq(x.data_ptr(), a_hat.data_ptr(), codes.data_ptr(), scale.data_ptr(),
                              C.byref(g), bits, per_sample, scratch.data_ptr(), L.stream_ptr()))
    else:
        L.check(l.modiff_modq_static(x.data_ptr(), a_hat.data_ptr(), codes.data_ptr(),
                                     scale.data_ptr(), C.byref(g), bits, per_sample,
                                     L.stream_ptr()))
    torch.cuda.synchronize()
    return codes, scale


@pytest.mark.parametrize("shape,bits,split,per_sample", [
    ((4, 128, 16, 16), 8, 0, 0),
    ((3, 384, 8, 8), 4, 256, 0),
    ((5, 128, 8, 8), 4, 0, 1),
    ((6, 512, 1, 1), 8, 0, 0),
])
def test_static_scratch_matches_caller_scratch_twice(cuda, shape, bits, split, per_sample):
    from modiff_b200 import _lib as L
    b, c, h, w = shape
    pad = 1 if h > 1 else 0
    g = L.ConvGeom(b, c, 64, h, w, 3 if pad else 1, 3 if pad else 1, 1, pad, pad, pad, pad, split)
    torch.manual_seed(31)
    a0 = torch.randn(shape, device=cuda)
    a_ref, a_new = a0.clone(), a0.clone()
    for call in range(2):          # two calls in a row: the second sees the first one's leftovers
        x = a0 + 0.1 * (call + 1) * torch.randn(shape, device=cuda)
        a_before = a_new.clone()
        codes_ref, scale_ref = _run("modiff_modq", x, a_ref, g, bits, per_sample, cuda)
        codes_new, scale_new = _run("modiff_modq_static", x, a_new, g, bits, per_sample, cuda)
        assert torch.equal(codes_new, codes_ref), f"codes differ on call {call}"
        assert torch.equal(scale_new, scale_ref), f"scales differ on call {call}"
        assert torch.equal(a_new, a_ref), f"a_hat differs on call {call}"
        assert int(codes_ref.to(torch.int32).abs().sum()) > 0
        if not per_sample:
            # and directly against the CPU restatement of the reference quantiser: the scale of
            # every segment and the updated cache (cache + codes * scale) must be the same bits
            from oracle.quantizer import fake_quant
            r = (x - a_before).cpu()
            segs = [r[:, :split], r[:, split:]] if split else [r]
            outs = [fake_quant(sg, bits, True) for sg in segs]
            assert [float(v) for v in scale_new[:len(segs)].cpu()] == [float(o[2]) for o in outs]
            upd = torch.cat([o[1] * o[2] for o in outs], dim=1)
            assert torch.equal(a_new.cpu(), a_before.cpu() + upd), f"a_hat vs oracle, call {call}"


def test_static_scratch_rejects_oversized_batch(cuda):
    from modiff_b200 import _lib as L
    l = L.lib()
    g = L.ConvGeom(4097, 16, 16, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0)
    x = torch.zeros(4097 * 16, device=cuda)
    codes = torch.zeros(4097 * 16, dtype=torch.int8, device=cuda)
    scale = torch.zeros(4097, device=cuda)
    rc = l.modiff_modq_static(x.data_ptr(), None, codes.data_ptr(), scale.data_ptr(), C.byref(g), 8,
                              1, L.stream_ptr())
    assert rc == 1 and b"built-in" in l.modiff_last_error()
    # the same batch is fine when scales are per tensor (two slots)
    L.check(l.modiff_modq_static(x.data_ptr(), None, codes.data_ptr(), scale.data_ptr(), C.byref(g),
                                 8, 0, L.stream_ptr()))
    torch.cuda.synchronize()
