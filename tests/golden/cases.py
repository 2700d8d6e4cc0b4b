"""Case definitions shared by make_golden.py (which runs the reference on them) and by the
tests (which re-create the same inputs / weights from the recorded seeds)."""
import numpy as np
import torch
import torch.nn as nn

# ---------------------------------------------------------------- stand-alone quantiser
QUANTIZER_CASES = [
    dict(name="pt_sym8", shape=(2, 16, 8, 8), n_bits=8, sym=True, channel_wise=False, seed=11),
    dict(name="pt_sym4", shape=(2, 16, 8, 8), n_bits=4, sym=True, channel_wise=False, seed=12),
    dict(name="pt_sym3", shape=(3, 8, 5, 7), n_bits=3, sym=True, channel_wise=False, seed=13),
    dict(name="pt_asym8", shape=(2, 16, 8, 8), n_bits=8, sym=False, channel_wise=False, seed=14),
    dict(name="pt_asym4_pos", shape=(2, 16, 8, 8), n_bits=4, sym=False, channel_wise=False,
         seed=15, offset=3.0),
    dict(name="pt_asym8_az", shape=(4, 33), n_bits=8, sym=False, channel_wise=False, seed=16,
         always_zero=True, relu=True),
    dict(name="cw_asym8", shape=(32, 16, 3, 3), n_bits=8, sym=False, channel_wise=True, seed=17),
    dict(name="cw_asym4", shape=(32, 16, 3, 3), n_bits=4, sym=False, channel_wise=True, seed=18),
    dict(name="cw_sym8", shape=(6, 4, 9, 9), n_bits=8, sym=True, channel_wise=True, seed=19),
    dict(name="cw_asym8_2d", shape=(24, 40), n_bits=8, sym=False, channel_wise=True, seed=20),
    dict(name="pt_sym8_zero", shape=(2, 4, 4, 4), n_bits=8, sym=True, channel_wise=False, seed=21,
         scale=0.0),
    dict(name="pt_sym8_ties", shape=(1, 1, 1, 255), n_bits=8, sym=True, channel_wise=False,
         seed=22, ties=True),
]


def quantizer_input(c):
    g = torch.Generator().manual_seed(c["seed"])
    if c.get("ties"):
        # multiples of half a quantisation step: exercises round-half-to-even
        n = int(np.prod(c["shape"]))
        x = (torch.arange(n, dtype=torch.float32) - n // 2) * 0.5
        return x.reshape(c["shape"])
    x = torch.randn(c["shape"], generator=g) * c.get("scale", 1.0) + c.get("offset", 0.0)
    if c.get("relu"):
        x = torch.relu(x)
    return x


# ---------------------------------------------------------------- single modulated layers
LAYER_CASES = [
    dict(name="c3_w8a8", kind="conv", cin=128, cout=128, k=3, stride=1, pad=1, hw=8, batch=2,
         w_bits=8, a_bits=8, seed=101),
    dict(name="c3_w4a4", kind="conv", cin=256, cout=128, k=3, stride=1, pad=1, hw=8, batch=2,
         w_bits=4, a_bits=4, seed=102),
    dict(name="c3_w4a3", kind="conv", cin=128, cout=256, k=3, stride=1, pad=1, hw=4, batch=3,
         w_bits=4, a_bits=3, seed=103),
    dict(name="c1_split_w4a4", kind="conv", cin=384, cout=128, k=1, stride=1, pad=0, hw=8,
         batch=2, w_bits=4, a_bits=4, split=256, seed=104),
    dict(name="c1_split_w8a8", kind="conv", cin=256, cout=128, k=1, stride=1, pad=0, hw=4,
         batch=2, w_bits=8, a_bits=8, split=128, seed=105),
    dict(name="down_w8a8", kind="conv", cin=128, cout=128, k=3, stride=2, pad=0, hw=8, batch=2,
         w_bits=8, a_bits=8, pad_br=True, seed=106),
    dict(name="lin_w8a8", kind="linear", cin=512, cout=256, batch=4, w_bits=8, a_bits=8, seed=107),
    dict(name="lin_w4a4", kind="linear", cin=128, cout=512, batch=4, w_bits=4, a_bits=4, seed=108),
    dict(name="cin3_w8a8", kind="conv", cin=3, cout=128, k=3, stride=1, pad=1, hw=8, batch=2,
         w_bits=8, a_bits=8, seed=109),
    dict(name="cout3_w4a4", kind="conv", cin=128, cout=3, k=3, stride=1, pad=1, hw=8, batch=2,
         w_bits=4, a_bits=4, seed=110),
    dict(name="c3_32_w8a8", kind="conv", cin=128, cout=16, k=3, stride=1, pad=1, hw=32, batch=1,
         w_bits=8, a_bits=8, seed=111, skip_a_hat=True),
    # asymmetric activation codes: the LDM / SD drivers' default (no --a_sym)
    dict(name="c3_w4a4_asym", kind="conv", cin=128, cout=128, k=3, stride=1, pad=1, hw=8, batch=2,
         w_bits=4, a_bits=4, a_sym=False, seed=112),
    dict(name="c1_split_w8a4_asym", kind="conv", cin=256, cout=128, k=1, stride=1, pad=0, hw=8,
         batch=2, w_bits=8, a_bits=4, a_sym=False, split=128, seed=113),
    dict(name="lin_w8a6_asym", kind="linear", cin=256, cout=128, batch=6, w_bits=8, a_bits=6,
         a_sym=False, seed=114),
    # 8-bit asymmetric activations: what the latent-diffusion drivers run without --a_sym
    dict(name="c3_w8a8_asym", kind="conv", cin=128, cout=128, k=3, stride=1, pad=1, hw=8, batch=2,
         w_bits=8, a_bits=8, a_sym=False, seed=115),
    dict(name="c1_split_w4a8_asym", kind="conv", cin=256, cout=128, k=1, stride=1, pad=0, hw=8,
         batch=2, w_bits=4, a_bits=8, a_sym=False, split=128, seed=116),
    dict(name="down_w8a8_asym", kind="conv", cin=128, cout=128, k=3, stride=2, pad=0, hw=8, batch=2,
         w_bits=8, a_bits=8, a_sym=False, pad_br=True, seed=117),
    dict(name="lin_w8a8_asym", kind="linear", cin=256, cout=128, batch=6, w_bits=8, a_bits=8,
         a_sym=False, seed=118),
]


def layer_module(c):
    """The fp32 torch layer whose default init (seeded) supplies the weights."""
    torch.manual_seed(c["seed"])
    if c["kind"] == "linear":
        return nn.Linear(c["cin"], c["cout"])
    return nn.Conv2d(c["cin"], c["cout"], kernel_size=c["k"], stride=c["stride"], padding=c["pad"])


def layer_inputs(c):
    """Four drifting inputs: step 0 (unquantised), two residual steps, one zero-residual step."""
    g = torch.Generator().manual_seed(c["seed"] + 1000)
    shape = (c["batch"], c["cin"]) if c["kind"] == "linear" else \
        (c["batch"], c["cin"], c["hw"], c["hw"])
    x0 = torch.randn(shape, generator=g)
    x1 = x0 + 0.1 * torch.randn(shape, generator=g)
    x2 = x1 + 0.03 * torch.randn(shape, generator=g)
    return [x0, x1, x2, x2.clone()]


def quant_params(c):
    """The dicts scripts/sample_diffusion_ddim.py:143-146 builds for
    --ptq --quant_act --quant_mode dynamic --a_sym."""
    wq = {'n_bits': c["w_bits"], 'channel_wise': True, 'scale_method': 'max'}
    aq = {'n_bits': c["a_bits"], 'symmetric': c.get("a_sym", True), 'channel_wise': False,
          'scale_method': 'max',
          'leaf_param': True, 'dynamic': True}
    return wq, aq


# ---------------------------------------------------------------- whole-UNet sampling runs
UNET_CASES = [
    dict(name="fp32_b8_s100", quant=False, split=False, batch=8, steps=100, noise_seed=0),
    dict(name="w8a8_b8_s100", quant=True, split=False, w_bits=8, a_bits=8, batch=8, steps=100,
         noise_seed=0, keep_eps=3),
    dict(name="w4a4_split_b8_s100", quant=True, split=True, w_bits=4, a_bits=4, batch=8, steps=100,
         noise_seed=1, keep_eps=3),
    dict(name="w4a3_split_b4_s100", quant=True, split=True, w_bits=4, a_bits=3, batch=4, steps=100,
         noise_seed=2),
    dict(name="w8a8_b2_s10", quant=True, split=False, w_bits=8, a_bits=8, batch=2, steps=10,
         noise_seed=3, keep_eps=10),
    dict(name="w4a4_split_b2_s10", quant=True, split=True, w_bits=4, a_bits=4, batch=2, steps=10,
         noise_seed=4, keep_eps=10),
]


def unet_noise(c):
    g = torch.Generator().manual_seed(c["noise_seed"])
    return torch.randn(c["batch"], 3, 32, 32, generator=g)


def unet_sequence(c):
    """Quad skip over 1000 timesteps (scripts/sample_diffusion_ddim.py:377-384)."""
    seq = np.linspace(0, np.sqrt(1000 * 0.8), c["steps"]) ** 2
    return [int(s) for s in list(seq)]


# ---------------------------------------------------------------- latent UNet (LSUN-churches kl-8)
LDM_CONFIG = dict(
    image_size=32, in_channels=4, out_channels=4, model_channels=192,
    attention_resolutions=[1, 2, 4, 8], num_res_blocks=2, channel_mult=[1, 2, 2, 4, 4],
    num_heads=8, use_scale_shift_norm=True, resblock_updown=True)
LDM_SCHEDULE = dict(linear_start=0.0015, linear_end=0.0155)   # lsun_churches-ldm-kl-8.yaml:5-6

LDM_CASES = [
    # first `evals` UNet evaluations of the 500 that `-c 400` gives (uniform, c = 1000 // 400)
    dict(name="ldm_w8a8_b2", w_bits=8, a_bits=8, batch=2, ddim_steps=400, evals=6, noise_seed=11,
         zero_seed=1234),
    # the driver's default quantiser (no --a_sym): asymmetric per-tensor 8-bit activations
    dict(name="ldm_w8a8_asym_b2", w_bits=8, a_bits=8, a_sym=False, batch=2, ddim_steps=400, evals=5,
         noise_seed=13, zero_seed=1234),
]


PLMS_CASES = [
    # pseudo linear multistep over 50 DDIM timesteps: 4 steps = 5 UNet evaluations (the first step
    # evaluates twice), Adams-Bashforth orders 2, 3 and 4 all taken
    dict(name="ldm_plms_w8a8_b2", w_bits=8, a_bits=8, batch=2, ddim_steps=50, steps=4, noise_seed=12,
         zero_seed=1234),
]


def ldm_noise(c):
    g = torch.Generator().manual_seed(c["noise_seed"])
    return torch.randn(c["batch"], 4, 32, 32, generator=g)


# ---------------------------------------------------------------- SD-v1 UNet (v1-inference.yaml)
SD_CONFIG = dict(
    image_size=32, in_channels=4, out_channels=4, model_channels=320,
    attention_resolutions=[4, 2, 1], num_res_blocks=2, channel_mult=[1, 2, 4, 4], num_heads=8,
    use_spatial_transformer=True, transformer_depth=1, context_dim=768, legacy=False)
SD_SCHEDULE = dict(linear_start=0.00085, linear_end=0.0120)    # v1-inference.yaml:5-6

SD_CASES = [
    # latent 4x64x64, context 77x768 ~ N(0,1), classifier-free guidance 7.5 (2x effective batch),
    # first `evals` of the 50 DDIM evaluations
    dict(name="sd_w8a8_b1", w_bits=8, a_bits=8, batch=1, latent=64, ddim_steps=50, evals=3,
         guidance=7.5, noise_seed=21, zero_seed=1234),
    # the txt2img driver's default quantiser (no --a_sym): asymmetric 8-bit activations
    dict(name="sd_w8a8_asym_b1", w_bits=8, a_bits=8, a_sym=False, batch=1, latent=64, ddim_steps=50,
         evals=2, guidance=7.5, noise_seed=22, zero_seed=1234),
]


def sd_inputs(c):
    g = torch.Generator().manual_seed(c["noise_seed"])
    x = torch.randn(c["batch"], 4, c["latent"], c["latent"], generator=g)
    cond = torch.randn(c["batch"], 77, 768, generator=g)
    uncond = torch.randn(c["batch"], 77, 768, generator=g)
    return x, cond, uncond


# ---------------------------------------------------------------- calibrated checkpoints
CALI_CASES = [
    # pixel UNet, static (quant_mode 'qdiff') activation scales and AdaRound weights loaded from
    # a synthetic checkpoint in the reference's format; first `evals` of a 10-step quad run
    dict(name="cali_w4a8_split_b2", w_bits=4, a_bits=8, a_sym=True, split=True, batch=2, steps=100,
         first=30, evals=5, noise_seed=31, cali_seed=32, alpha_seed=33, scale_margin=1.5),
    dict(name="cali_w8a6_asym_b2", w_bits=8, a_bits=6, a_sym=False, split=False, batch=2, steps=100,
         first=30, evals=4, noise_seed=34, cali_seed=35, alpha_seed=36, scale_margin=1.25),
]


def cali_sequence(c):
    """`evals` consecutive timesteps from the middle of the 100-step quad sequence (t about
    70..90): step-to-step changes there are small against the activations, as in a real run,
    whereas a random-init UNet makes the first steps from pure noise jump."""
    return unet_sequence(c)[c["first"]:c["first"] + c["evals"]]


def cali_data(c):
    """The (x, t) pair scripts/sample_diffusion_ddim.py:160-162 hands to resume_cali_model."""
    g = torch.Generator().manual_seed(c["cali_seed"])
    return torch.randn(1, 3, 32, 32, generator=g), torch.randint(0, 1000, (1,), generator=g)


def cali_alpha(key, shape, seed):
    """AdaRound logits of the synthetic checkpoint: seeded noise, i.e. every weight is rounded up
    or down at random - a harder case than a trained checkpoint, whose logits mostly keep
    round-to-nearest."""
    import zlib
    g = torch.Generator().manual_seed(seed + zlib.crc32(key.encode()) % 100000)
    return torch.randn(tuple(shape), generator=g)


def cali_checkpoint(c, model_state, fixture, prefix):
    """The synthetic calibrated checkpoint of a case: UNet parameters from `model_state` (keys as
    the float model names them), AdaRound logits from seeds, quantiser scales from the fixture
    (entries `<prefix>/ckpt/<key>`), under the reference QuantModel's key names."""
    import json
    ckpt = {}
    for key, shape in json.loads(str(fixture[prefix + "/keys"])):
        stored = f"{prefix}/ckpt/{key}"
        if key.endswith(".alpha"):
            ckpt[key] = cali_alpha(key, shape, c["alpha_seed"])
        elif stored in fixture:
            ckpt[key] = torch.from_numpy(np.asarray(fixture[stored])).reshape(shape).clone()
        else:
            name = key[len("model."):]
            ckpt[key] = model_state[name].detach().cpu().clone()
        assert list(ckpt[key].shape) == list(shape), key
    return ckpt


# ---------------------------------------------------------------- moving-average ranges
# Layers of LAYER_CASES run with non-dynamic leaf quantisers: call 0 unquantised, call 1 sets the
# scale and the range, calls 2..4 with set_running_stat(True), call 5 with it off again.
RUNNING_CASES = ["c3_w8a8", "c1_split_w4a4", "c3_w4a4_asym", "lin_w8a8_asym", "down_w8a8_asym"]


def running_inputs(c):
    g = torch.Generator().manual_seed(c["seed"] + 2000)
    shape = (c["batch"], c["cin"]) if c["kind"] == "linear" else \
        (c["batch"], c["cin"], c["hw"], c["hw"])
    xs = [torch.randn(shape, generator=g)]
    for k in range(5):
        xs.append(xs[-1] + (0.08 - 0.01 * k) * (torch.randn(shape, generator=g) + 0.2 * (k % 2)))
    return xs


# ---------------------------------------------------------------- full-length runs and sensitivity
# Full sampler loops at the sizes the throughput figures are quoted on (pixel UNet: batch 256,
# the benchmarked batch; latent UNet: all 500 evaluations of `-c 400`; SD-v1: all 50 guided
# evaluations).  Only the final tensor and a few trajectory points are stored.
FULL_CASES = [
    dict(name="pixel_w4a4_split_b256_s100", kind="pixel", quant=True, split=True, w_bits=4, a_bits=4,
         batch=256, steps=100, noise_seed=1),
    dict(name="ldm_w8a8_b2_full", kind="ldm", w_bits=8, a_bits=8, batch=2, ddim_steps=400,
         noise_seed=11, zero_seed=1234),
    dict(name="sd_w8a8_b1_full", kind="sd", w_bits=8, a_bits=8, batch=1, latent=64, ddim_steps=50,
         guidance=7.5, noise_seed=21, zero_seed=1234),
    dict(name="pixel_w4a3_split_b256_s100", kind="pixel", quant=True, split=True, w_bits=4, a_bits=3,
         batch=256, steps=100, noise_seed=2),
]

# Self-sensitivity of the reference: the same run repeated with the FIRST evaluation's output
# perturbed by Gaussian noise of standard deviation SENS_REL x (max - min of that output).  The
# PSNR between the two runs, per evaluation, is what a last-bit-different but otherwise exact
# implementation can be expected to reach; tests derive their per-evaluation floors from it.
SENS_REL = 1e-4
SENS_SEED = 777


def perturb_first_call(fn, rel=SENS_REL, seed=SENS_SEED):
    """`fn` with the output of its first call perturbed (see SENS_REL)."""
    state = {"n": 0}

    def wrapped(*args):
        out = fn(*args)
        if state["n"] == 0:
            g = torch.Generator().manual_seed(seed)
            span = float(out.max() - out.min())
            out = out + rel * span * torch.randn(out.shape, generator=g)
        state["n"] += 1
        return out
    return wrapped


# ---------------------------------------------------------------- first-stage decoder (kl-f8)
# ddconfig of configs/latent-diffusion/lsun_churches-ldm-kl-8.yaml:47-56; random init seed 0; the
# decoder is fully convolutional, so a 16x16 latent (128x128 pixels) exercises every layer.
DECODER_CONFIG = dict(double_z=True, z_channels=4, resolution=256, in_channels=3, out_ch=3, ch=128,
                      ch_mult=(1, 2, 4, 4), num_res_blocks=2, attn_resolutions=[], dropout=0.0)
DECODER_CASE = dict(name="kl_f8_decode", embed_dim=4, batch=2, latent=16, init_seed=0, z_seed=41)


def decoder_latents(c):
    g = torch.Generator().manual_seed(c["z_seed"])
    return torch.randn(c["batch"], c["embed_dim"], c["latent"], c["latent"], generator=g)
