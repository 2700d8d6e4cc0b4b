"""CPU restatement of the reference algorithm for the modulated-quantisation sampling path.

TEST INFRASTRUCTURE ONLY.  Nothing under modiff_b200/ imports this package; it is used by
tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline / reference arm as the
checker and the timed CPU baseline, never as the product.

The reference's arithmetic lives in PyTorch (third-party, unpinned in the reference's
environment.yml; 2.11.0 here), so the restatement is written with torch CPU ops in the same
order as the reference's Python, each function citing the reference lines it follows.  It is
pinned against the live reference by tests/golden/make_golden.py, which imports the reference,
runs both on the same seeds and commits the reference's outputs as fixtures; the reference
itself ships no tests or golden vectors.
"""
from .quantizer import (per_tensor_scale, channel_wise_scale, quantize_codes, fake_quant,
                        weight_codes)
from .quant_module import OracleQuantModule
from .unet import OracleUNet, pixel_unet_config
from .sampler import ddim_sample, quad_sequence, linear_betas, psnr

__all__ = ["per_tensor_scale", "channel_wise_scale", "quantize_codes", "fake_quant",
           "weight_codes", "OracleQuantModule", "OracleUNet", "pixel_unet_config",
           "ddim_sample", "quad_sequence", "linear_betas", "psnr"]
