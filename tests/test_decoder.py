"""First-stage decoder (ldm/models/autoencoder.py:330-333, ldm/modules/diffusionmodules/model.py
:465-573): structure and initialisation against the reference on the CPU, the CUDA forward
against the reference's stored image."""
import os

import numpy as np
import pytest
import torch

import cases

GOLDEN = os.path.dirname(os.path.abspath(cases.__file__))


def _build():
    import modiff_b200 as m
    c = cases.DECODER_CASE
    torch.manual_seed(c["init_seed"])
    dec = m.Decoder(**cases.DECODER_CONFIG).eval()
    fs = m.FirstStageDecoder.__new__(m.FirstStageDecoder)
    torch.nn.Module.__init__(fs)
    fs.decoder = dec                       # same creation order as the fixture: decoder first,
    fs.post_quant_conv = torch.nn.Conv2d(c["embed_dim"], cases.DECODER_CONFIG["z_channels"], 1)
    fs.embed_dim = c["embed_dim"]          # then the 1x1 convolution
    return fs


def test_structure_and_seeded_weights_match_the_reference():
    """49 490 179 decoder parameters, the reference's state_dict key names, and (seed 0) the
    reference's random initialisation: the sum over all parameters equals the fixture's."""
    fx = np.load(os.path.join(GOLDEN, "decoder.npz"))
    fs = _build()
    assert sum(p.numel() for p in fs.decoder.parameters()) == 49490179
    keys = list(fs.state_dict().keys())
    assert "decoder.up.3.upsample.conv.weight" in keys and "decoder.mid.attn_1.q.weight" in keys
    assert "post_quant_conv.weight" in keys and "decoder.up.0.block.2.conv2.bias" in keys
    assert not any("_modiff" in k for k in keys)
    total = sum(float(p.double().sum()) for p in list(fs.decoder.parameters()) +
                list(fs.post_quant_conv.parameters()))
    assert abs(total - float(fx[cases.DECODER_CASE["name"] + "/param_sum"])) < 1e-6
    with pytest.raises(Exception):
        fs.decode(torch.zeros(1, 4, 8, 8))          # CPU tensors are refused


@pytest.mark.gpu
def test_decode_matches_the_reference(cuda):
    """Latents -> pixels on the device against the reference decoder's output for the same
    seeded weights and latents: 1e-4 of the image range (plain fp32 everywhere; the 512-channel
    mid-block attention runs as split-bf16 tensor-core products, relative error about 1e-5)."""
    import modiff_b200 as m
    fx = np.load(os.path.join(GOLDEN, "decoder.npz"))
    c = cases.DECODER_CASE
    fs = _build().to(cuda)
    y = fs.decode(cases.decoder_latents(c).to(cuda))
    torch.cuda.synchronize()
    assert m.device_status() == 0
    ref = fx[c["name"] + "/image"]
    assert tuple(y.shape) == ref.shape
    err = np.abs(y.cpu().numpy() - ref).max() / np.abs(ref).max()
    print(f"decoder: max |image - reference| / max |reference| = {err:.2e}")
    assert err < 1e-4, err
    # overwritten weights are picked up (the kernels hold no stale copy)
    with torch.no_grad():
        fs.decoder.conv_out.bias.add_(1.0)
    y2 = fs.decode(cases.decoder_latents(c).to(cuda))
    assert float((y2 - y - 1.0).abs().max()) < 1e-5
