"""Loading calibrated checkpoints into a QuantModel (qdiff/utils.py:511-628).

A Q-Diffusion / MoDiff `ckpt.pth` is the state dict of the reference QuantModel after
calibration: the UNet's own parameters, per weight quantiser `alpha` (AdaRound logits), `delta`
and `zero_point`, and - when activations were calibrated with quant_mode 'qdiff' - per
activation quantiser `delta` and `zero_point`.  Module paths are the reference's, which this
package's QuantModel reproduces.
"""
import logging

import torch
import torch.nn as nn

from ._lib import ModiffError
from .adaptive_rounding import AdaRoundQuantizer
from .quant_block import BaseQuantBlock
from .quant_layer import QuantModule

logger = logging.getLogger(__name__)

_W_SLOTS = ("weight_quantizer", "weight_quantizer_0")
_A_SLOTS = ("act_quantizer", "act_quantizer_0")


def _to_adaround(module: QuantModule):
    w = module.org_weight.data
    if module.org_weight.device != module.weight.device:
        w = w.to(module.weight.device)
    if module.split != 0:
        module.weight_quantizer = AdaRoundQuantizer(
            uaq=module.weight_quantizer, round_mode='learned_hard_sigmoid',
            weight_tensor=w[:, :module.split, ...])
        module.weight_quantizer_0 = AdaRoundQuantizer(
            uaq=module.weight_quantizer_0, round_mode='learned_hard_sigmoid',
            weight_tensor=w[:, module.split:, ...])
    else:
        module.weight_quantizer = AdaRoundQuantizer(
            uaq=module.weight_quantizer, round_mode='learned_hard_sigmoid', weight_tensor=w)


def convert_adaround(model):
    """Swap every weight quantiser for an AdaRoundQuantizer initialised to round-to-nearest
    (qdiff/utils.py:511-539).  Layers and blocks with `ignore_reconstruction` are left alone."""
    for _, module in model.named_children():
        if isinstance(module, QuantModule):
            if module.ignore_reconstruction is True:
                continue
            _to_adaround(module)
        elif isinstance(module, BaseQuantBlock):
            if module.ignore_reconstruction is True:
                continue
            for _, sub in module.named_modules():
                if isinstance(sub, QuantModule):
                    _to_adaround(sub)
        else:
            convert_adaround(module)


def _run(qnn, cali_data, cond):
    dev = next(qnn.parameters()).device
    if not cond:
        xs, ts = cali_data[0], cali_data[1]
        return qnn(xs[:1].to(dev), ts[:1].to(dev))
    xs, ts, cs = cali_data
    return qnn(xs[:1].to(dev), ts[:1].to(dev), cs[:1].to(dev))


def _split_key(key):
    """'a.b.weight_quantizer.alpha' -> ('a.b', 'weight_quantizer', 'alpha'), else None."""
    parts = key.split('.')
    if len(parts) >= 3 and parts[-2] in _W_SLOTS + _A_SLOTS and \
            parts[-1] in ('alpha', 'delta', 'zero_point'):
        return '.'.join(parts[:-2]), parts[-2], parts[-1]
    return None


def load_calibrated_state(qnn, ckpt, load_act=False):
    """Copy a reference checkpoint (a dict of CPU tensors) into `qnn`: ordinary parameters
    through `load_state_dict`, quantiser tensors into the AdaRound quantisers and, with
    `load_act`, the activation scales.  Every key must find its place, and every AdaRound
    quantiser must receive its `alpha`, as `strict=True` enforces in the reference
    (qdiff/utils.py:567)."""
    modules = dict(qnn.named_modules())
    plain, act = {}, {}
    got_alpha = set()
    for key, val in ckpt.items():
        sk = _split_key(key)
        if sk is None:
            plain[key] = val
            continue
        path, slot, field = sk
        m = modules.get(path)
        if not isinstance(m, QuantModule):
            raise ModiffError(f"checkpoint key {key!r}: no quantised layer at {path!r}")
        if slot in _A_SLOTS:
            act.setdefault(path, {})[(slot, field)] = val
            continue
        q = getattr(m, slot, None)
        if not isinstance(q, AdaRoundQuantizer):
            raise ModiffError(f"checkpoint key {key!r}: {path}.{slot} is not an AdaRound quantiser "
                              "(split not registered, or convert_adaround not run)")
        dev = m.weight.device
        if field == 'alpha':
            if tuple(val.shape) != tuple(q.alpha.shape):
                raise ModiffError(f"{key}: shape {tuple(val.shape)} != {tuple(q.alpha.shape)}")
            q.alpha.data.copy_(val.to(dev))
            got_alpha.add((path, slot))
        elif field == 'delta':
            q.delta = val.detach().to(dev, torch.float32).reshape(q.delta.shape).clone()
        else:
            q.zero_point = val.detach().to(dev, torch.float32).reshape(q.delta.shape).clone()
        m._wpack = None                       # repack with the loaded rounding / scales
    for path, m in modules.items():
        if isinstance(m, QuantModule):
            for slot in _W_SLOTS:
                if isinstance(getattr(m, slot, None), AdaRoundQuantizer) and \
                        (path, slot) not in got_alpha:
                    raise ModiffError(f"checkpoint has no {path}.{slot}.alpha")
    own = {k for k in qnn.state_dict().keys() if _split_key(k) is None}
    missing = sorted(own - set(plain))
    unexpected = sorted(set(plain) - own)
    if missing or unexpected:
        raise ModiffError(f"checkpoint does not match the model: missing {missing[:5]} "
                          f"({len(missing)}), unexpected {unexpected[:5]} ({len(unexpected)})")
    qnn.load_state_dict(plain, strict=False)
    for m in modules.values():
        if isinstance(m, QuantModule):
            m._wpack = None
            m._org_kn = None
    if load_act:
        for path, fields in act.items():
            m = modules[path]
            slots = ["act_quantizer"] + (["act_quantizer_0"] if m.split != 0 else [])
            try:
                delta = [float(fields[(s, 'delta')]) for s in slots]
            except KeyError as e:
                raise ModiffError(f"checkpoint lacks {path}.{e.args[0][0]}.delta") from None
            zp = [float(fields.get((s, 'zero_point'), 0.0)) for s in slots]
            m.load_act_scale(delta, zp)


def resume_cali_model(qnn, ckpt_path, cali_data, quant_act=False, act_quant_mode='qdiff',
                      cond=False):
    """Same steps as the reference (qdiff/utils.py:542-628): initialise the weight quantisers
    with one forward pass, convert them to AdaRound, load the checkpoint; with `quant_act`,
    initialise the activation quantisers with two passes and (mode 'qdiff') load their
    calibrated scales.  `ckpt_path` is a file for `torch.load`, or an already loaded dict."""
    logger.info("Loading quantized model checkpoint")
    ckpt = ckpt_path if isinstance(ckpt_path, dict) else \
        torch.load(ckpt_path, map_location='cpu', weights_only=True)
    with torch.no_grad():
        qnn.set_quant_state(True, False)
        _run(qnn, cali_data, cond)
        convert_adaround(qnn)
        load_calibrated_state(qnn, ckpt, load_act=False)
        qnn.set_quant_state(weight_quant=True, act_quant=False)
        if quant_act:
            qnn.set_quant_state(True, True)
            _run(qnn, cali_data, cond)
            _run(qnn, cali_data, cond)
            if act_quant_mode == 'qdiff':
                load_calibrated_state(qnn, ckpt, load_act=True)
            qnn.set_quant_state(weight_quant=True, act_quant=True)
    return qnn
