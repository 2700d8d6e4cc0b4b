"""Restatement of the latent-diffusion UNet forward with quantised blocks and of the latent DDIM
sampler, as functional torch-CPU code over a state dict (test infrastructure only).

Follows ldm/modules/diffusionmodules/openaimodel.py:447-782 (UNetModel), :163-278 (ResBlock),
:281-327 (AttentionBlock), :373-406 (QKVAttentionLegacy); qdiff/quant_block.py:83-111
(QuantResBlock._forward), :114-151 (the attention matmuls stay in floating point);
ldm/modules/diffusionmodules/util.py:21-74, 151-171; ldm/models/diffusion/ddim.py:25-54, 184-234.
"""
import math

import numpy as np
import torch
import torch.nn.functional as F

from .quant_module import OracleQuantModule


def ldm_timestep_embedding(t, dim):
    """util.py:151-171: cos | sin."""
    half = dim // 2
    freqs = torch.exp(-math.log(10000) * torch.arange(start=0, end=half, dtype=torch.float32) / half)
    args = t[:, None].float() * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


def unet_plan(cfg):
    """Block structure of UNetModel.__init__ (openaimodel.py:549-720) as lists of
    ('res', kind) / ('attn',) entries per TimestepEmbedSequential."""
    mc, mult_list = cfg["model_channels"], cfg["channel_mult"]
    nrb, ar = cfg["num_res_blocks"], cfg["attention_resolutions"]
    attn_kind = "st" if cfg.get("use_spatial_transformer", False) else "attn"
    updown = cfg.get("resblock_updown", False)
    inputs = [[("conv",)]]
    ds = 1
    for level, _ in enumerate(mult_list):
        for _ in range(nrb):
            layers = [("res", "plain")]
            if ds in ar:
                layers.append((attn_kind,))
            inputs.append(layers)
        if level != len(mult_list) - 1:
            inputs.append([("res", "down")] if updown else [("downsample",)])
            ds *= 2
    middle = [("res", "plain"), (attn_kind,), ("res", "plain")]
    outputs = []
    for level, _ in list(enumerate(mult_list))[::-1]:
        for i in range(nrb + 1):
            layers = [("res", "plain")]
            if ds in ar:
                layers.append((attn_kind,))
            if level and i == nrb:
                layers.append(("res", "up") if updown else ("upsample",))
                ds //= 2
            outputs.append(layers)
    return inputs, middle, outputs


class OracleLDMUNet:
    def __init__(self, state, cfg, w_bits=8, a_bits=8, a_sym=True, modulate=True, split=False,
                 quant=True):
        self.state, self.cfg, self.split = state, cfg, split
        self.layers = {}
        for name, w in state.items():
            if not name.endswith(".weight") or w.dim() < 2:
                continue
            base = name[:-len(".weight")]
            pad = 1 if (w.dim() == 4 and w.shape[-1] == 3) else 0
            stride = 2 if base.endswith(".op") else 1          # Downsample.op (openaimodel.py:148-151)
            m = OracleQuantModule(w, state.get(base + ".bias"), stride, pad, w_bits, a_bits, a_sym,
                                  False, modulate)
            m.use_weight_quant = m.use_act_quant = quant
            if not quant:
                m.modulate = False
            self.layers[base] = m
        self.plan = unet_plan(cfg)

    def reset_cache(self):
        for m in self.layers.values():
            m.reset_cache()

    def _gn(self, x, base):
        """GroupNorm32(32, C), eps 1e-5 (util.py:199-216)."""
        return F.group_norm(x.float(), 32, self.state[base + ".weight"], self.state[base + ".bias"],
                            1e-5)

    def _res(self, base, kind, x, emb, split=0):
        """qdiff/quant_block.py:83-111."""
        L = self.layers
        h = F.silu(self._gn(x, base + ".in_layers.0"))
        if kind == "down":
            h = F.avg_pool2d(h, 2, 2)
            x = F.avg_pool2d(x, 2, 2)
        elif kind == "up":
            h = F.interpolate(h, scale_factor=2, mode="nearest")
            x = F.interpolate(x, scale_factor=2, mode="nearest")
        h = L[base + ".in_layers.2"].forward(h)
        emb_out = L[base + ".emb_layers.1"].forward(F.silu(emb))[..., None, None]
        if self.cfg.get("use_scale_shift_norm", False):
            scale, shift = torch.chunk(emb_out, 2, dim=1)
            h = self._gn(h, base + ".out_layers.0") * (1 + scale) + shift
            h = F.silu(h)
        else:
            h = h + emb_out
            h = F.silu(self._gn(h, base + ".out_layers.0"))
        h = L[base + ".out_layers.3"].forward(h)
        if (base + ".skip_connection") in L:
            x = L[base + ".skip_connection"].forward(x, split=split)
        return x + h

    def _attn(self, base, x):
        """openaimodel.py:321-327, 384-406."""
        L = self.layers
        b, c = x.shape[0], x.shape[1]
        spatial = x.shape[2:]
        x3 = x.reshape(b, c, -1)
        qkv = self._conv1d(base + ".qkv", self._gn(x3, base + ".norm"))
        heads = self.cfg["num_heads"]
        bs, width, length = qkv.shape
        ch = width // (3 * heads)
        q, k, v = qkv.reshape(bs * heads, ch * 3, length).split(ch, dim=1)
        scale = 1 / math.sqrt(math.sqrt(ch))
        weight = torch.einsum("bct,bcs->bts", q * scale, k * scale)
        weight = torch.softmax(weight.float(), dim=-1)
        a = torch.einsum("bts,bcs->bct", weight, v).reshape(bs, -1, length)
        h = self._conv1d(base + ".proj_out", a)
        return (x3 + h).reshape(b, c, *spatial)

    def _conv1d(self, base, x):
        """A k=1 Conv1d QuantModule: F.conv1d on [B, C, T]."""
        m = self.layers[base]
        w2 = m.weight
        if w2.dim() == 3:
            # run the same QuantModule arithmetic through conv2d on [B, C, T, 1]
            if not hasattr(m, "_as4d"):
                m.weight = w2.unsqueeze(-1)
                m._wq = {}
                m._as4d = True
        return m.forward(x.unsqueeze(-1)).squeeze(-1)

    def _ln(self, x, base):
        return F.layer_norm(x, (x.shape[-1],), self.state[base + ".weight"],
                            self.state[base + ".bias"], 1e-5)

    def _cross_attn(self, base, x, context=None):
        """qdiff/quant_block.py:181-204."""
        L = self.layers
        h = self.cfg["num_heads"]
        q = L[base + ".to_q"].forward(x)
        ctx = x if context is None else context
        k = L[base + ".to_k"].forward(ctx)
        v = L[base + ".to_v"].forward(ctx)
        b, n, inner = q.shape
        d = inner // h

        def heads(t):
            return t.reshape(b, t.shape[1], h, d).permute(0, 2, 1, 3).reshape(b * h, t.shape[1], d)

        q, k, v = heads(q), heads(k), heads(v)
        sim = torch.einsum('b i d, b j d -> b i j', q, k) * (d ** -0.5)
        attn = sim.softmax(dim=-1)
        out = torch.einsum('b i j, b j d -> b i d', attn, v)
        out = out.reshape(b, h, n, d).permute(0, 2, 1, 3).reshape(b, n, inner)
        return L[base + ".to_out.0"].forward(out)

    def _st(self, base, x, context):
        """ldm/modules/attention.py:270-287 with qdiff/quant_block.py:249-256 blocks."""
        L = self.layers
        b, c, hh, ww = x.shape
        x_in = x
        t = F.group_norm(x, 32, self.state[base + ".norm.weight"], self.state[base + ".norm.bias"], 1e-6)
        t = L[base + ".proj_in"].forward(t)
        inner = t.shape[1]
        t = t.reshape(b, inner, hh * ww).permute(0, 2, 1)
        j = 0
        while f"{base}.transformer_blocks.{j}.attn1.to_q" in L:
            tb = f"{base}.transformer_blocks.{j}"
            t = self._cross_attn(tb + ".attn1", self._ln(t, tb + ".norm1")) + t
            t = self._cross_attn(tb + ".attn2", self._ln(t, tb + ".norm2"), context) + t
            ff = L[tb + ".ff.net.0.proj"].forward(self._ln(t, tb + ".norm3"))
            a, gate = ff.chunk(2, dim=-1)
            t = L[tb + ".ff.net.2"].forward(a * F.gelu(gate)) + t
            j += 1
        t = t.permute(0, 2, 1).reshape(b, inner, hh, ww)
        return L[base + ".proj_out"].forward(t) + x_in

    def _seq(self, prefix, layers, h, emb, split=0, context=None):
        for j, layer in enumerate(layers):
            base = f"{prefix}.{j}"
            if layer[0] == "conv":
                h = self.layers[base].forward(h)
            elif layer[0] == "res":
                h = self._res(base, layer[1], h, emb, split if j == 0 else 0)
            elif layer[0] == "st":
                h = self._st(base, h, context)
            elif layer[0] == "downsample":
                h = self.layers[base + ".op"].forward(h)
            elif layer[0] == "upsample":
                h = self.layers[base + ".conv"].forward(F.interpolate(h, scale_factor=2, mode="nearest"))
            else:
                h = self._attn(base, h)
        return h

    def forward(self, x, t, context=None):
        """openaimodel.py:745-782."""
        L = self.layers
        inputs, middle, outputs = self.plan
        emb = ldm_timestep_embedding(t, self.cfg["model_channels"])
        emb = L["time_embed.0"].forward(emb)
        emb = F.silu(emb)
        emb = L["time_embed.2"].forward(emb)
        hs = []
        h = x
        for i, layers in enumerate(inputs):
            h = self._seq(f"input_blocks.{i}", layers, h, emb, context=context)
            hs.append(h)
        h = self._seq("middle_block", middle, h, emb, context=context)
        for i, layers in enumerate(outputs):
            split = h.shape[1] if self.split else 0
            h = torch.cat([h, hs.pop()], dim=1)
            h = self._seq(f"output_blocks.{i}", layers, h, emb, split, context=context)
        h = F.silu(self._gn(h, "out.0"))
        return L["out.2"].forward(h)


# ---------------------------------------------------------------- latent DDIM
def ldm_schedule(linear_start, linear_end, n_timestep=1000):
    """alphas_cumprod as LatentDiffusion.register_schedule keeps it (ddpm.py:118-139): float64
    numpy, cast to float32."""
    betas = (torch.linspace(linear_start ** 0.5, linear_end ** 0.5, n_timestep,
                            dtype=torch.float64) ** 2).numpy()
    return torch.tensor(np.cumprod(1.0 - betas, axis=0), dtype=torch.float32)


def ddim_parameters(alphas_cumprod, steps, n_timestep=1000):
    """util.py:44-74 with the 'uniform' discretisation (c = T // S, +1 offset), eta = 0."""
    c = n_timestep // steps
    ts = np.asarray(list(range(0, n_timestep, c))) + 1
    alphas = alphas_cumprod[ts]
    alphas_prev = np.asarray([alphas_cumprod[0]] + alphas_cumprod[ts[:-1]].tolist())
    return ts, alphas, alphas_prev


@torch.no_grad()
def latent_ddim_sample(x, model_fn, alphas_cumprod, steps, max_evals=None, on_step=None,
                       cond=None, uncond=None, guidance=1.0):
    """ldm/models/diffusion/ddim.py:117-234 with eta = 0.  With `uncond` and guidance != 1 the
    batch is doubled and e = e_uc + s * (e_c - e_uc) (:192-208).  `max_evals` stops early (for
    bounded tests)."""
    ts, alphas, alphas_prev = ddim_parameters(alphas_cumprod, steps)
    sqrt_one_minus = np.sqrt(1. - alphas)
    b = x.shape[0]
    img = x
    total = ts.shape[0]
    for i, step in enumerate(np.flip(ts)):
        if max_evals is not None and i >= max_evals:
            break
        index = total - i - 1
        t = torch.full((b,), int(step), dtype=torch.long)
        if uncond is None or guidance == 1.0:
            e_t = model_fn(img, t) if cond is None else model_fn(img, t, cond)
        else:
            e_all = model_fn(torch.cat([img] * 2), torch.cat([t] * 2), torch.cat([uncond, cond]))
            e_uc, e_c = e_all.chunk(2)
            e_t = e_uc + guidance * (e_c - e_uc)
        a_t = torch.full((b, 1, 1, 1), float(alphas[index]))
        a_prev = torch.full((b, 1, 1, 1), float(alphas_prev[index]))
        sqrt_one_minus_at = torch.full((b, 1, 1, 1), float(sqrt_one_minus[index]))
        pred_x0 = (img - sqrt_one_minus_at * e_t) / a_t.sqrt()
        dir_xt = (1. - a_prev).sqrt() * e_t
        img = a_prev.sqrt() * pred_x0 + dir_xt
        if on_step is not None:
            on_step(i, e_t, img)
    return img


@torch.no_grad()
def latent_plms_sample(x, model_fn, alphas_cumprod, steps, max_steps=None, on_eval=None,
                       cond=None, uncond=None, guidance=1.0):
    """ldm/models/diffusion/plms.py:114-240 (eta = 0): pseudo linear multistep over the DDIM
    schedule.  The first step evaluates the model twice (improved Euler, :221-225), later steps
    combine the last up to four eps with Adams-Bashforth weights (:226-234).  `on_eval(k, e)`
    sees every model output in evaluation order; `max_steps` stops early."""
    ts, alphas, alphas_prev = ddim_parameters(alphas_cumprod, steps)
    sqrt_one_minus = np.sqrt(1. - alphas)
    b = x.shape[0]
    img = x
    time_range = np.flip(ts)
    total = ts.shape[0]
    old_eps = []
    n_eval = [0]

    def model_output(xx, step):
        t = torch.full((b,), int(step), dtype=torch.long)
        if uncond is None or guidance == 1.0:
            e = model_fn(xx, t) if cond is None else model_fn(xx, t, cond)
        else:
            e_all = model_fn(torch.cat([xx] * 2), torch.cat([t] * 2), torch.cat([uncond, cond]))
            e_uc, e_c = e_all.chunk(2)
            e = e_uc + guidance * (e_c - e_uc)
        if on_eval is not None:
            on_eval(n_eval[0], e)
        n_eval[0] += 1
        return e

    def x_prev_of(e, index):
        a_t = torch.full((b, 1, 1, 1), float(alphas[index]))
        a_prev = torch.full((b, 1, 1, 1), float(alphas_prev[index]))
        sqrt_one_minus_at = torch.full((b, 1, 1, 1), float(sqrt_one_minus[index]))
        pred_x0 = (img - sqrt_one_minus_at * e) / a_t.sqrt()
        dir_xt = (1. - a_prev).sqrt() * e
        return a_prev.sqrt() * pred_x0 + dir_xt

    for i, step in enumerate(time_range):
        if max_steps is not None and i >= max_steps:
            break
        index = total - i - 1
        step_next = time_range[min(i + 1, len(time_range) - 1)]
        e_t = model_output(img, step)
        if len(old_eps) == 0:
            e_t_next = model_output(x_prev_of(e_t, index), step_next)
            e_prime = (e_t + e_t_next) / 2
        elif len(old_eps) == 1:
            e_prime = (3 * e_t - old_eps[-1]) / 2
        elif len(old_eps) == 2:
            e_prime = (23 * e_t - 16 * old_eps[-1] + 5 * old_eps[-2]) / 12
        else:
            e_prime = (55 * e_t - 59 * old_eps[-1] + 37 * old_eps[-2] - 9 * old_eps[-3]) / 24
        img = x_prev_of(e_prime, index)
        old_eps.append(e_t)
        if len(old_eps) >= 4:
            old_eps.pop(0)
    return img

