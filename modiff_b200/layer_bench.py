"""Micro-benchmark of one modulated QuantModule geometry (quantiser + int8 GEMM kernels).

    python -m modiff_b200.layer_bench --cin 128 --cout 128 --hw 32 --k 3 --batch 256 --iters 20

Prints one JSON line: device time per call and achieved algorithmic GB/s of `modiff_modq`
and `modiff_igemm_conv` (CUDA events on the launching stream; the tensors of one layer at
batch 256 exceed L2).  Small enough to sit under `ncu -k regex:... -c 1`.
`--attention` times `ops.attention` (plane splits + attention kernel) at [batch, cin, hw*hw].
"""
import argparse
import json

import torch
import torch.nn as nn

from . import _lib
from .quant_layer import QuantModule


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cin", type=int, default=128)
    ap.add_argument("--cout", type=int, default=128)
    ap.add_argument("--hw", type=int, default=32)
    ap.add_argument("--k", type=int, default=3)
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--split", type=int, default=0)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--w-bits", type=int, default=4)
    ap.add_argument("--a-bits", type=int, default=4)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", type=int, default=_lib.IMPL_AUTO)
    ap.add_argument("--linear", action="store_true")
    ap.add_argument("--layernorm", action="store_true",
                    help="with --linear: the input is LayerNorm(x), evaluated inside the quantiser")
    ap.add_argument("--geglu", action="store_true",
                    help="with --linear: the input is GEGLU(h), h of 2*cin features, evaluated "
                         "inside the quantiser")
    ap.add_argument("--static", action="store_true",
                    help="non-dynamic activation quantiser: the scale of the first quantised call "
                         "stays and later calls are the one-pass modiff_modq_fixed")
    ap.add_argument("--asym", action="store_true", help="asymmetric activation codes")
    ap.add_argument("--fused", action="store_true",
                    help="feed the layer GroupNorm(32)+SiLU of the input as a lazy source")
    ap.add_argument("--pair", action="store_true",
                    help="a residual block's conv1 (3x3 on GroupNorm+SiLU of x) and 1x1 shortcut on "
                         "the same x, quantised in shared sweeps (modiff_modq_pair)")
    ap.add_argument("--attention-i8", action="store_true",
                    help="time the integer attention (quantise + kernel) on [batch, cin, hw*hw]")
    ap.add_argument("--attention", action="store_true",
                    help="time ops.attention on [batch, cin, hw*hw] tensors instead of a layer")
    args = ap.parse_args()

    dev = torch.device("cuda")
    torch.manual_seed(0)
    if args.attention_i8:
        from . import ops
        t = args.hw * args.hw
        q, k, v = (torch.randn(args.batch, args.cin, t, device=dev) for _ in range(3))
        scale = float(args.cin) ** -0.5
        for _ in range(args.warmup):
            ops.attention_i8_channel_major(q, k, v, scale)
        _lib.TIMER = _lib.KernelTimer()
        for _ in range(args.iters):
            ops.attention_i8_channel_major(q, k, v, scale)
        summ = _lib.TIMER.summary()
        _lib.TIMER = None
        print(json.dumps({"geometry": vars(args), "device_status": _lib.device_status(),
                          "us_per_call": {n: 1000.0 * v_["ms"] / v_["launches"]
                                          for n, v_ in summ.items()}}))
        return
    if args.attention:
        from . import ops
        t = args.hw * args.hw
        q, k, v = (torch.randn(args.batch, args.cin, t, device=dev) for _ in range(3))
        scale = float(args.cin) ** -0.5
        for _ in range(args.warmup):
            ops.attention(q, k, v, scale)
        _lib.TIMER = _lib.KernelTimer()
        for _ in range(args.iters):
            ops.attention(q, k, v, scale)
        summ = _lib.TIMER.summary()
        _lib.TIMER = None
        print(json.dumps({"geometry": vars(args), "device_status": _lib.device_status(),
                          "us_per_call": {n: 1000.0 * v_["ms"] / v_["launches"]
                                          for n, v_ in summ.items()}}))
        return
    if args.pair:
        from .ops import ActSource
        wq = {'n_bits': args.w_bits, 'channel_wise': True, 'scale_method': 'max'}
        aq = {'n_bits': args.a_bits, 'symmetric': True, 'channel_wise': False, 'scale_method': 'max',
              'leaf_param': True, 'dynamic': True}
        conv1 = QuantModule(nn.Conv2d(args.cin, args.cout, 3, padding=1), wq, aq, modulate=True).to(dev)
        short = QuantModule(nn.Conv2d(args.cin, args.cout, 1), wq, aq, modulate=True).to(dev)
        for q in (conv1, short):
            q.set_quant_state(True, True)
        norm = nn.GroupNorm(32, args.cin, eps=1e-6).to(dev)
        shape = (args.batch, args.cin, args.hw, args.hw)
        x = torch.randn(shape, device=dev)
        drift = [0.05 * torch.randn(shape, device=dev) for _ in range(2)]
        kw = dict(split=args.split) if args.split else {}

        def step(t):
            src = ActSource(t, norm=norm, silu=True)
            pair = conv1.forward_pair(src, short, args.split)
            if pair is None:
                conv1(src)
                short(t, **kw)

        with torch.no_grad():
            step(x)
            for i in range(args.warmup):
                step(x + drift[i % 2])
            _lib.TIMER = _lib.KernelTimer()
            for i in range(args.iters):
                step(x + drift[i % 2])
            summ = _lib.TIMER.summary()
            _lib.TIMER = None
        print(json.dumps({"geometry": vars(args), "device_status": _lib.device_status(),
                          "us_per_call": {n: 1000.0 * v_["ms"] / v_["launches"]
                                          for n, v_ in summ.items()},
                          "algorithmic_bytes_per_call": {n: v_["bytes"] // v_["launches"]
                                                         for n, v_ in summ.items()}}))
        return
    if args.linear:
        org = nn.Linear(args.cin, args.cout)
        shape = (args.batch, 2 * args.cin if args.geglu else args.cin)
    else:
        pad = args.k // 2 if args.stride == 1 else 0
        org = nn.Conv2d(args.cin, args.cout, args.k, stride=args.stride, padding=pad)
        shape = (args.batch, args.cin, args.hw, args.hw)
    wq = {'n_bits': args.w_bits, 'channel_wise': True, 'scale_method': 'max'}
    aq = {'n_bits': args.a_bits, 'symmetric': not args.asym, 'channel_wise': False,
          'scale_method': 'max', 'leaf_param': True, 'dynamic': not args.static}
    mod = QuantModule(org, wq, aq, modulate=True).to(dev)
    mod.set_quant_state(True, True)
    mod.igemm_impl = args.impl
    if args.stride == 2:
        mod.implicit_pad = (0, 1, 0, 1)

    x = torch.randn(shape, device=dev)
    drift = [0.05 * torch.randn(shape, device=dev) for _ in range(2)]
    kw = dict(split=args.split) if args.split else {}
    norm = nn.GroupNorm(32, args.cin, eps=1e-6).to(dev) if args.fused else None
    lnorm = nn.LayerNorm(args.cin).to(dev) if args.layernorm else None

    def feed(t):
        if lnorm is not None:
            from .ops import LayerNormSource
            return LayerNormSource(t, lnorm)
        if args.geglu:
            from .ops import GegluSource
            return GegluSource(t)
        if norm is None:
            return t
        from .ops import ActSource
        return ActSource(t, norm=norm, silu=True)

    with torch.no_grad():
        mod(feed(x), **kw)                             # first step: fp32 path, creates caches
        for i in range(args.warmup):
            mod(feed(x + drift[i % 2]), **kw)
        _lib.TIMER = _lib.KernelTimer()
        for i in range(args.iters):
            mod(feed(x + drift[i % 2]), **kw)
        summ = _lib.TIMER.summary()
        _lib.TIMER = None
    status = _lib.device_status()
    out = {"geometry": vars(args), "device_status": status}
    for name in ("modiff_modq", "modiff_modq_src", "modiff_modq_gn", "modiff_modq_fixed",
                 "modiff_modq_ln", "modiff_modq_geglu", "modiff_layernorm", "modiff_geglu",
                 "modiff_modq_asym", "modiff_codes_fill_halo", "modiff_groupnorm_silu",
                 "modiff_igemm_conv", "modiff_igemm_conv_offset"):
        if name not in summ:
            continue
        v = summ[name]
        out[name] = {"us_per_call": 1000.0 * v["ms"] / v["launches"],
                     "algorithmic_GBps": v["bytes"] / (v["ms"] / 1000.0) / 1e9,
                     "algorithmic_bytes_per_call": v["bytes"] // v["launches"]}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
