"""B200-native (sm_100a) implementation of MoDiff's modulated-quantisation UNet sampling path
behind qdiff's Python API.  See include/modiff_b200.h for the C ABI the modules call into."""
from ._lib import ModiffError, lib, device_status
from .quant_layer import QuantModule, UniformAffineQuantizer, StraightThrough, round_ste
from .quant_block import (BaseQuantBlock, QuantResnetBlock, QuantAttnBlock, QuantResBlock,
                          QuantBasicTransformerBlock, QuantQKMatMul, QuantSMVMatMul,
                          QuantAttentionBlock, get_specials)
from .quant_model import QuantModel
from .adaptive_rounding import AdaRoundQuantizer
from .utils import convert_adaround, resume_cali_model, load_calibrated_state
from .unet import Model, make_config
from .ldm_unet import UNetModel, rerandomize_zero_tensors
from .ldm_sampler import DDIMSampler, PLMSSampler
from .sampler import (generalized_steps, compute_alpha, get_beta_schedule,
                      make_timestep_sequence)
from .autoencoder import Decoder, FirstStageDecoder, KL_F8
from .calibration import generate_calibration_data, select_calibration_points

__all__ = [
    "ModiffError", "lib", "device_status", "QuantModule", "UniformAffineQuantizer",
    "StraightThrough", "round_ste", "BaseQuantBlock", "QuantResnetBlock", "QuantAttnBlock",
    "QuantResBlock", "QuantBasicTransformerBlock", "QuantQKMatMul", "QuantSMVMatMul",
    "QuantAttentionBlock", "AdaRoundQuantizer", "convert_adaround", "resume_cali_model",
    "load_calibrated_state",
    "get_specials", "QuantModel", "Model", "UNetModel", "DDIMSampler", "PLMSSampler", "rerandomize_zero_tensors", "make_config", "generalized_steps", "compute_alpha",
    "get_beta_schedule", "make_timestep_sequence", "generate_calibration_data",
    "select_calibration_points", "Decoder", "FirstStageDecoder", "KL_F8",
]
