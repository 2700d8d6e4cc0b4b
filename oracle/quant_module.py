"""Restatement of QuantModule.forward with MoDiff modulation (qdiff/quant_layer.py:307-367),
plus the exact-integer view of the same computation used to check codes and accumulators."""
import torch
import torch.nn.functional as F

from .quantizer import fake_quant, weight_codes, adaround_codes


class OracleQuantModule:
    """One conv2d / linear layer.  `weight` [Cout, Cin, kh, kw] or [Cout, Cin], `bias` or None.

    Mirrors the reference state: a_hat / o_hat caches, split, use_weight_quant /
    use_act_quant / modulate flags.  After every quantised call `last` holds the integer
    codes, scales and exact integer accumulators of that call.
    """

    def __init__(self, weight, bias, stride=1, padding=0, w_bits=8, a_bits=8, a_sym=True,
                 a_channel_wise=False, modulate=True, a_dynamic=True):
        self.weight = weight
        self.bias = bias
        self.stride = stride
        self.padding = padding
        self.w_bits, self.a_bits, self.a_sym = w_bits, a_bits, a_sym
        self.a_channel_wise = a_channel_wise
        self.modulate = modulate
        self.use_weight_quant = True
        self.use_act_quant = True
        self.split = 0
        self.a_hat = None
        self.o_hat = None
        self.last = {}
        self._wq = {}
        # non-dynamic activation quantisers (quant_mode 'qdiff'): the scale of the first
        # quantised call, or a loaded one, stays (qdiff/quant_layer.py:72-79)
        self.a_dynamic = a_dynamic
        self.act_scale = None       # per segment (delta tensor, zero point)
        self.act_range = None       # per segment (x_min, x_max) of a leaf_param quantiser
        self.running_stat = False   # set_running_stat (:389-392): moving-average ranges
        # AdaRound weight quantisers of a calibrated checkpoint: per segment (alpha, delta, zp)
        self.adaround = None

    def reset_cache(self):
        """qdiff/quant_layer.py:381-383."""
        self.a_hat = None
        self.o_hat = None

    def _fwd(self, x, w, b):
        if w.dim() == 2:
            return F.linear(x, w, b)
        return F.conv2d(x, w, b, stride=self.stride, padding=self.padding)

    def _quant_weight(self):
        """qdiff/quant_layer.py:345-351: each segment has its own per-channel quantiser."""
        key = self.split
        if key not in self._wq and self.adaround is not None:
            segs = [self.weight[:, :self.split, ...], self.weight[:, self.split:, ...]] \
                if self.split else [self.weight]
            assert len(segs) == len(self.adaround)
            self._wq[key] = [adaround_codes(s.contiguous(), a, d, z, self.w_bits)
                             for s, (a, d, z) in zip(segs, self.adaround)]
        if key not in self._wq:
            if self.split:
                parts = [weight_codes(self.weight[:, :self.split, ...].contiguous(), self.w_bits),
                         weight_codes(self.weight[:, self.split:, ...].contiguous(), self.w_bits)]
            else:
                parts = [weight_codes(self.weight, self.w_bits)]
            self._wq[key] = parts
        return self._wq[key]

    def _quant_act(self, x):
        """qdiff/quant_layer.py:330-335: two independent dynamic quantisers with split."""
        if self.split:
            segs = [x[:, :self.split, ...], x[:, self.split:, ...]]
        else:
            segs = [x]
        if self.a_dynamic:
            return [fake_quant(s, self.a_bits, self.a_sym, channel_wise=self.a_channel_wise)
                    for s in segs]
        if self.act_scale is None:
            first = [fake_quant(s, self.a_bits, self.a_sym) for s in segs]
            self.act_scale = [(f[2], f[3]) for f in first]
            # leaf_param quantisers record the range of their first call (:192-194)
            self.act_range = [(s.min(), s.max()) for s in segs]
            return first
        assert len(self.act_scale) == len(segs)
        if self.running_stat:
            self._momentum_update(segs)
        return [fake_quant(s, self.a_bits, self.a_sym, scale=sc)
                for s, sc in zip(segs, self.act_scale)]

    def _momentum_update(self, segs, momentum=0.95):
        """act_momentum_update (qdiff/quant_layer.py:113-132), per segment quantiser."""
        from .quantizer import n_levels_of
        n_levels = n_levels_of(self.a_bits, self.a_sym)
        for i, s in enumerate(segs):
            x_min, x_max = self.act_range[i]
            x_min = x_min * momentum + s.min() * (1 - momentum)
            x_max = x_max * momentum + s.max() * (1 - momentum)
            self.act_range[i] = (x_min, x_max)
            if self.a_sym:
                delta = torch.max(x_min.abs(), x_max.abs()) / n_levels
            else:
                delta = (x_max - x_min) / (n_levels - 1)
            delta = torch.clamp(delta, min=1e-8)
            zp = self.act_scale[i][1]
            if not self.a_sym:
                zp = int((-x_min / delta).round().item())
            self.act_scale[i] = (delta, zp)

    def forward(self, x, split=0):
        if not self.use_weight_quant and not self.use_act_quant and not self.modulate:
            return self._fwd(x, self.weight, self.bias)                     # :309-311
        if split != 0:                                                       # :313-319
            assert self.split in (0, split)
            self.split = split
        acts = None
        if self.use_act_quant:                                               # :321-343
            if self.modulate:
                if self.a_hat is None:
                    self.a_hat = x.clone()
                else:
                    r = x - self.a_hat
                    acts = self._quant_act(r)
                    x = torch.cat([a[0] for a in acts], dim=1) if self.split else acts[0][0]
                    self.a_hat = (self.a_hat + x).clone()
            else:
                acts = self._quant_act(x)
                x = torch.cat([a[0] for a in acts], dim=1) if self.split else acts[0][0]
        if self.use_weight_quant:                                            # :345-355
            wparts = self._quant_weight()
            w = torch.cat([p[0] for p in wparts], dim=1) if self.split else wparts[0][0]
        else:
            wparts, w = None, self.weight
        bias = self.bias
        if self.modulate and self.use_act_quant:                             # :357-365
            if self.o_hat is None:
                out = self._fwd(x, w, bias)
            else:
                out = self._fwd(x, w, None)
                out = self.o_hat + out
            self.o_hat = out.clone()
        else:
            out = self._fwd(x, w, bias)
        self.last = {}
        if acts is not None and wparts is not None:
            self.last = self._integer_view(acts, wparts)
        return out

    def _integer_view(self, acts, wparts):
        """Exact integer accumulators sum codes * (q - zp) per segment, computed in float64
        (|acc| < 2^53), and the per-segment scales."""
        accs = []
        for (xd, xq, dx, zx), (wd, wq, dw, zw) in zip(acts, wparts):
            a = (xq - zx).double()
            w_int = (wq - zw).double()
            accs.append(self._fwd(a, w_int, None).round().to(torch.int64))
        return dict(codes=[a[1].to(torch.int32) for a in acts],
                    x_scale=[a[2] for a in acts],
                    x_zp=[a[3] for a in acts],
                    w_codes=[p[1].to(torch.int32) for p in wparts],
                    w_scale=[p[2].reshape(-1) for p in wparts],
                    w_zp=[p[3].reshape(-1) for p in wparts],
                    acc=accs)
