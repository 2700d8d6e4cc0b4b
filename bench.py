"""Throughput of modulated-quantisation sampling on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config NAME] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one full sampling pass of the hot path over one batch per GPU.  `--config`:

    pixel_w4a4 (default)  pixel UNet 3x32x32, W4A4 modulated, split shortcut, 100 DDIM quad steps,
                          batch 256 per GPU, x_T seed 1
    pixel_w8a8            same UNet, W8A8 modulated (no split), batch 256 per GPU, x_T seed 0
    pixel_w4a3            same UNet, W4A3 modulated, split shortcut, batch 256 per GPU, x_T seed 2
    ldm_w8a8              latent UNet (LSUN-churches kl-8 shapes), W8A8 modulated, batch 32 per GPU,
                          `-c 400` = 500 evaluations, decoder excluded
    sd_w8a8               SD-v1 UNet, latent 4x64x64, context 77x768, W8A8 modulated, guidance 7.5
                          (2x effective batch), 50 evaluations, batch 8 per GPU

Synthetic inputs (x_T, context ~ N(0,1)) and random-init weights (seed 0) stand in for the
checkpoints and data sets, which are not available offline.  The metric is images per second
over all GPUs.  Rank 0 prints one JSON line.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "UNet sampling images/sec"

CONFIGS = {
    "pixel_w4a4": dict(kind="pixel", w_bits=4, a_bits=4, split=True, batch=256, evals=100, seed=1,
                       workload="pixel UNet 3x32x32 W4A4 modulated, split shortcut, 100 DDIM quad "
                                "steps, batch 256/GPU"),
    "pixel_w8a8": dict(kind="pixel", w_bits=8, a_bits=8, split=False, batch=256, evals=100, seed=0,
                       workload="pixel UNet 3x32x32 W8A8 modulated, 100 DDIM quad steps, "
                                "batch 256/GPU"),
    "pixel_w4a3": dict(kind="pixel", w_bits=4, a_bits=3, split=True, batch=256, evals=100, seed=2,
                       workload="pixel UNet 3x32x32 W4A3 modulated, split shortcut, 100 DDIM quad "
                                "steps, batch 256/GPU"),
    "ldm_w8a8": dict(kind="ldm", w_bits=8, a_bits=8, batch=32, evals=500, seed=11, int8_attention=True,
                     workload="latent UNet 4x32x32 (LSUN-churches kl-8 shapes) W8A8 modulated, "
                              "DDIM -c 400 (500 evaluations), batch 32/GPU, decoder excluded"),
    "sd_w8a8": dict(kind="sd", w_bits=8, a_bits=8, batch=8, evals=50, seed=21, int8_attention=True,
                    workload="SD-v1 UNet 4x64x64, context 77x768, W8A8 modulated, guidance 7.5 "
                             "(2x effective batch), 50 DDIM evaluations, batch 8/GPU"),
}

# measured DRAM bytes / algorithmic bytes of one launch (ncu captures summarised in profiles/):
# the quantiser reads x and a_hat twice (two passes), 21 B moved per 13 B algorithmic
DRAM_TRAFFIC_RATIO = {"modiff_modq_src": 1.52, "modiff_modq_gn": 1.52, "modiff_modq_pair": 1.28,
                      "modiff_modq": 1.52, "modiff_igemm_conv": 0.83}

INT8_NOMINAL_TOPS = 4500.0      # dense INT8 of one B200 (2x the dense bf16 datasheet figure)


def quant_params(cfg, a_sym=True, dynamic=True):
    """The dicts the reference drivers build (scripts/sample_diffusion_ddim.py:143-146)."""
    wq = {'n_bits': cfg["w_bits"], 'channel_wise': True, 'scale_method': 'max'}
    aq = {'n_bits': cfg["a_bits"], 'symmetric': a_sym, 'channel_wise': False,
          'scale_method': 'max', 'leaf_param': True, 'dynamic': dynamic}
    return wq, aq


class ClockSampler:
    """Polls nvidia-smi for SM clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                     "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(parts)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        mhz = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


# ------------------------------------------------------------------------------ CPU arm
def cpu_reference_sample(cfg, threads, a_sym=True, full=False):
    """Times the CPU restatement of the reference path (oracle/) on the host cores, on a bounded
    sample of the workload, and extrapolates to a full sampling pass.  Returns
    (images per second, seconds spent, description of the sample)."""
    import modiff_b200 as m
    import oracle
    torch.set_num_threads(threads)
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(cfg["seed"])
    if cfg["kind"] == "pixel":
        batch, steps_run = 8, (cfg["evals"] if full else 25)
        net = m.Model(m.make_config(split_shortcut=cfg["split"]))
        state = {k: v.detach().clone() for k, v in net.state_dict().items()}
        ref = oracle.OracleUNet(state, w_bits=cfg["w_bits"], a_bits=cfg["a_bits"],
                                split_shortcut=cfg["split"])
        x = torch.randn(batch, 3, 32, 32, generator=g)
        seq = oracle.quad_sequence(1000, cfg["evals"])[-steps_run:]
        t0 = time.perf_counter()
        oracle.ddim_sample(x, seq, ref.forward, oracle.linear_betas())
        dt = time.perf_counter() - t0
        what = (f"batch {batch}, all {steps_run} DDIM steps" if full else
                f"batch {batch}, first {steps_run} of {cfg['evals']} DDIM steps (unquantised "
                f"first step included), extrapolated x{cfg['evals'] // steps_run}")
        return batch / (dt * cfg["evals"] / steps_run), dt, what
    from oracle.ldm import OracleLDMUNet, ldm_schedule, latent_ddim_sample
    from modiff_b200.ldm_unet import LSUN_CHURCHES_KL8, SD_V1
    sd = cfg["kind"] == "sd"
    mcfg = SD_V1 if sd else LSUN_CHURCHES_KL8
    net = m.UNetModel(**mcfg).eval()
    m.rerandomize_zero_tensors(net)
    state = {k: v.detach().clone() for k, v in net.state_dict().items()}
    del net
    ref = OracleLDMUNet(state, mcfg, cfg["w_bits"], cfg["a_bits"], a_sym)
    batch, evals_run = (1, 3) if sd else (2, 10)
    latent = 64 if sd else 32
    x = torch.randn(batch, 4, latent, latent, generator=g)
    sched = ldm_schedule(0.00085, 0.0120) if sd else ldm_schedule(0.0015, 0.0155)
    kw = {}
    if sd:
        kw = dict(cond=torch.randn(batch, 77, 768, generator=g),
                  uncond=torch.randn(batch, 77, 768, generator=g), guidance=7.5)
    t0 = time.perf_counter()
    latent_ddim_sample(x, ref.forward, sched, 50 if sd else 400, max_evals=evals_run, **kw)
    dt = time.perf_counter() - t0
    what = (f"batch {batch}, first {evals_run} of {cfg['evals']} "
            f"{'guided ' if sd else ''}evaluations (unquantised first one included), time per "
            f"evaluation x {cfg['evals']}")
    return batch / (dt * cfg["evals"] / evals_run), dt, what


def run_reference(args, cfg):
    """`--impl reference`: the reference's own (fake-quant fp32, CPU) implementation of the
    path, restated in oracle/, on all host threads.  Rank 0 only."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    a_sym = not args.asym
    for _ in range(min(args.warmup, 1 if cfg["kind"] != "pixel" else args.warmup)):
        cpu_reference_sample(cfg, threads, a_sym)
    t0 = time.perf_counter()
    runs = [cpu_reference_sample(cfg, threads, a_sym) for _ in range(args.steps)]
    dt = time.perf_counter() - t0
    v = sum(r[0] for r in runs) / len(runs)
    sample = runs[0][2] + " (per bench step)"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1000.0 * dt / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg["workload"], "name": args.config,
                   "reference_arm": "CPU restatement of qdiff fake-quant path"},
        "cpu_baseline": {"value": v, "unit": "images/s", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": v, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------------------ GPU arm
def conv_ops(key):
    """2 x MACs of one int8 GEMM call from its geometry key (the fields of modiff_conv_geom)."""
    batch, cin, cout, h, w, kh, kw, stride, pt, pl, pb, pr, _ = key
    ho = (h + pt + pb - kh) // stride + 1
    wo = (w + pl + pr - kw) // stride + 1
    return 2.0 * batch * ho * wo * cout * cin * kh * kw


def int8_summary(timer, hbm_peak, i8_peak):
    """Achieved int8 TOPS of the GEMM entry points: all layers together and per layer class."""
    classes = {}
    for (name, key), (launches, ms, nbytes) in timer.by_tag().items():
        if not name.startswith("modiff_igemm_conv") or ms <= 0:
            continue
        batch, cin, cout, h, w, kh, kw = key[:7]
        label = f"{kh}x{kw} {cin}->{cout} {h}x{w}" + (" +sum" if name.endswith("_add") else "")
        c = classes.setdefault(label, dict(launches=0, ms=0.0, ops=0.0, bytes=0.0))
        c["launches"] += launches
        c["ms"] += ms
        c["ops"] += conv_ops(key) * launches
        c["bytes"] += nbytes
    if not classes:
        return None
    ops = sum(c["ops"] for c in classes.values())
    ms = sum(c["ms"] for c in classes.values())
    top = sorted(classes.items(), key=lambda kv: -kv[1]["ms"])[:10]
    tops = ops / (ms / 1000.0) / 1e12
    return {
        "int8_tops": tops, "int8_gemm_ms": ms, "int8_tera_ops": ops / 1e12,
        "int8_frac_of_nominal": tops / INT8_NOMINAL_TOPS, "int8_nominal_tops": INT8_NOMINAL_TOPS,
        "int8_peak_measured": i8_peak,
        "int8_frac_of_measured": None if not i8_peak else tops / i8_peak,
        "int8_layers": [{"layer": k, "launches": c["launches"], "ms": round(c["ms"], 2),
                         "tops": round(c["ops"] / (c["ms"] / 1000.0) / 1e12, 1),
                         "gbs": round(c["bytes"] / (c["ms"] / 1000.0) / 1e9, 1),
                         "hbm_frac": round(c["bytes"] / (c["ms"] / 1000.0) / 1e9 / hbm_peak, 3)}
                        for k, c in top],
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="modiff_b200")
    ap.add_argument("--config", choices=sorted(CONFIGS), default="pixel_w4a4")
    ap.add_argument("--batch", type=int, default=None, help="images per GPU (profiling aid)")
    ap.add_argument("--evals", "--ddim-steps", dest="evals", type=int, default=None,
                    help="profiling aid: only the last n timesteps (pixel) / first n evaluations")
    ap.add_argument("--asym", action="store_true",
                    help="asymmetric activation quantisers (the latent drivers' default without "
                         "--a_sym); the headline lines use symmetric ones")
    ap.add_argument("--int8-attention", action="store_true",
                    help="integer attention kernel (q / k / v / softmax quantisers applied).  The "
                         "latent and SD configurations are quoted WITH it and switch it on by "
                         "default; the pixel configurations are quoted without")
    ap.add_argument("--fp-attention", action="store_true",
                    help="floating-point attention as the reference's code runs it (its attention "
                         "quantisers are built but never applied), also for ldm_w8a8 / sd_w8a8")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-full", action="store_true",
                    help="time the CPU baseline on ALL steps of a batch-8 pass instead of the "
                         "bounded sample (pixel configurations; about a minute)")
    ap.add_argument("--quant-mode", choices=["dynamic", "qdiff"], default="dynamic",
                    help="'qdiff': non-dynamic activation scales (each layer keeps the scale of its "
                         "first quantised call), the mode of a calibrated checkpoint; not the "
                         "headline configuration")
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    # the integer attention takes symmetric q / k / v quantisers only: --asym keeps the
    # floating-point attention unless --int8-attention asks for the error message
    args.int8_attention = (args.int8_attention or
                           (cfg.get("int8_attention", False) and not args.fp_attention
                            and not args.asym))
    if args.impl == "reference":
        return run_reference(args, cfg)

    import modiff_b200 as m
    from modiff_b200 import _lib, distributed as D
    import torch.distributed as dist

    rank, local_rank, world = D.init()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    batch = args.batch or cfg["batch"]
    evals = args.evals or cfg["evals"]
    kind = cfg["kind"]

    wq, aq = quant_params(cfg, a_sym=not args.asym, dynamic=(args.quant_mode == "dynamic"))
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(D.rank_seed(cfg["seed"], rank))
    host_in = []
    if kind == "pixel":
        net = m.Model(m.make_config(split_shortcut=cfg["split"])).eval()
        qnn = m.QuantModel(net, wq, aq, sm_abit=8, modulate=True,
                           int8_attention=args.int8_attention).to(dev).eval()
        qnn.set_quant_state(True, True)
        betas = torch.from_numpy(m.get_beta_schedule()).float()
        seq = m.make_timestep_sequence(1000, cfg["evals"], "quad")[-evals:]
        shape = (batch, 3, 32, 32)
        host_in.append(torch.randn(shape, generator=g).pin_memory())

        def sample(inputs, check):
            xs, _ = m.generalized_steps(inputs[0], seq, qnn, betas, eta=0.0, check_status=check)
            return xs[-1]
    else:
        from modiff_b200.ldm_unet import LSUN_CHURCHES_KL8, SD_V1
        sd = kind == "sd"
        net = m.UNetModel(**(SD_V1 if sd else LSUN_CHURCHES_KL8)).eval()
        m.rerandomize_zero_tensors(net)
        qnn = m.QuantModel(net, wq, aq, sm_abit=8, modulate=True,
                           int8_attention=args.int8_attention).to(dev).eval()
        qnn.set_quant_state(True, True)
        qnn.set_grad_ckpt(False)
        sched = dict(linear_start=0.00085, linear_end=0.0120) if sd else \
            dict(linear_start=0.0015, linear_end=0.0155)
        sampler = m.DDIMSampler(qnn, **sched)
        latent = 64 if sd else 32
        shape = (batch, 4, latent, latent)
        host_in.append(torch.randn(shape, generator=g).pin_memory())
        if sd:
            host_in.append(torch.randn(batch, 77, 768, generator=g).pin_memory())
            host_in.append(torch.randn(batch, 77, 768, generator=g).pin_memory())
        ddim_s = 50 if sd else 400

        def sample(inputs, check):
            kw = {}
            if sd:
                kw = dict(conditioning=inputs[1], unconditional_conditioning=inputs[2],
                          unconditional_guidance_scale=7.5)
            out, _ = sampler.sample(ddim_s, batch, shape[1:], eta=0.0, x_T=inputs[0],
                                    max_evals=evals, check_status=check, **kw)
            return out

    workload = cfg["workload"]
    if evals != cfg["evals"] or batch != cfg["batch"]:
        workload = f"REDUCED (profiling) {evals} evaluations, batch {batch}/GPU: " + workload
    if args.quant_mode != "dynamic":
        workload = "STATIC activation scales (quant_mode qdiff): " + workload
    if args.asym:
        workload += ", asymmetric activation codes"
    if args.int8_attention:
        workload += ", INT8 attention (q / k / v / softmax quantisers applied)"
    elif cfg.get("int8_attention"):
        workload += ", floating-point attention (reference behaviour)"

    out_host = torch.empty((world * batch,) + tuple(shape[1:])).pin_memory()
    dev_in = [t.to(dev) for t in host_in]

    def one_pass(inputs, check=False):
        qnn.reset_cache()
        return D.gather_samples(sample(inputs, check))

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, k):
        sync_all()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(k):
            fn()
        end.record()
        sync_all()
        ms = torch.tensor([start.elapsed_time(end)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)

    for _ in range(max(args.warmup, 1)):
        one_pass(dev_in)

    n0 = _lib.LAUNCHES[0]
    with ClockSampler(local_rank) as clocks:
        ms = timed(lambda: one_pass(dev_in), args.steps)
    launches = _lib.LAUNCHES[0] - n0
    # one 4-byte read of the library's status word, outside the timed steps: a kernel that gave
    # up on a bounded wait (or a zero point that did not fit) makes the run fail, not report
    status = _lib.device_status(reset=True)
    if status:
        raise SystemExit(f"device status {status:#x} after the timed passes: results invalid")

    def e2e_pass():
        xd = [t.to(dev, non_blocking=True) for t in host_in]
        res = one_pass(xd, check=True)      # the call a user makes, status check included
        out_host.copy_(res, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_pass()
    ms_e2e = timed(e2e_pass, args.steps)

    images = world * batch * args.steps
    value = images / (ms / 1000.0)
    e2e_value = images / (ms_e2e / 1000.0)

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel: one more pass with per-call CUDA events
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = json.load(open(peaks_path))["hbm_gbs"], "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    # tensor-pipe ceiling of kind::i8, measured here: MMA loop only, operands resident in shared
    # memory, every SM busy (csrc/i8_peak.cu)
    i8_peak = None
    try:
        i8_peak = _lib.measure_i8_peak()
    except Exception as e:                       # reported, never fatal for the throughput line
        sys.stderr.write(f"int8 peak probe failed: {e}\n")
    _lib.TIMER = _lib.KernelTimer()
    qnn.reset_cache()
    sample(dev_in, False)
    timer = _lib.TIMER
    summ = timer.summary()
    _lib.TIMER = None
    total_ms = sum(v["ms"] for v in summ.values())
    dom = max(summ, key=lambda k: summ[k]["ms"])
    d = summ[dom]
    achieved = d["bytes"] / (d["ms"] / 1000.0) / 1e9
    # DRAM traffic per launch: ncu's dram__bytes_read + dram__bytes_write of one captured launch
    # (profiles/), expressed as a ratio to that launch's algorithmic bytes and scaled to this
    # run's average launch; null for entry points that were not captured.
    ratio = DRAM_TRAFFIC_RATIO.get(dom)
    traffic = None if ratio is None else ratio * d["bytes"] / d["launches"]
    bound, unit, rpeak = "hbm", "GB/s", peak
    if d.get("ops", 0) > 0:
        # an attention kernel leads: its roofline is the tensor pipe (bf16 products against the
        # measured sustained cuBLAS bf16 figure, int8 products against the measured kind::i8 one)
        bound, unit = "tensor", ("TOP/s" if dom == "modiff_attention_i8" else "TFLOP/s")
        achieved = d["ops"] / (d["ms"] / 1000.0) / 1e12
        if dom == "modiff_attention_i8":
            rpeak = i8_peak or INT8_NOMINAL_TOPS
        else:
            rpeak = json.load(open(peaks_path)).get("bf16_tflops_sustained", 1376.4) \
                if os.path.exists(peaks_path) else 1400.0
        traffic = None
    roofline = {"kernel": dom, "bound": bound, "achieved": achieved, "peak": rpeak, "unit": unit,
                "frac": achieved / rpeak, "traffic": traffic, "peak_source": peak_src,
                "algorithmic_bytes_per_launch": d["bytes"] / d["launches"],
                "launches": d["launches"], "share_of_kernel_time": d["ms"] / total_ms,
                "per_entry_point_ms": {k: round(v["ms"], 2) for k, v in summ.items()}}
    i8 = int8_summary(timer, peak, i8_peak)
    if i8:
        roofline.update(i8)
    # whole-pass floors: the algorithmic bytes every entry point declared (quantisers 13 B per
    # input element, GEMMs 8 B per output element + codes + weights, ...) at the HBM peak, and the
    # int8 operations at the tensor-pipe ceiling; the pass cannot be faster than the larger one
    declared = sum(v["bytes"] for v in summ.values())
    byte_floor_ms = declared / (peak * 1e9) * 1e3
    op_floor_ms = (i8["int8_tera_ops"] * 1e12 / ((i8_peak or INT8_NOMINAL_TOPS) * 1e12) * 1e3) if i8 else 0.0
    roofline.update({"pass_algorithmic_gbytes": declared / 1e9, "pass_byte_floor_ms": byte_floor_ms,
                     "pass_op_floor_ms": op_floor_ms,
                     "pass_frac_of_floor": max(byte_floor_ms, op_floor_ms) / (ms / args.steps)})

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        v, dt, what = cpu_reference_sample(cfg, threads, not args.asym, full=args.cpu_full)
        cpu_baseline = {"value": v, "unit": "images/s", "cores": threads, "kind": "port",
                        "sample": f"{what} ({dt:.1f} s)"}

    line = {
        "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": {"workload": workload, "name": args.config, "global_batch": world * batch,
                   "evaluations": evals, "parallelism": f"dp{world}",
                   "l2": "working set (activation and output caches of every layer, GBs) exceeds L2"},
        "e2e": {"value": e2e_value, "unit": "images/s",
                "h2d_bytes_per_step": sum(t.numel() * 4 for t in host_in),
                "d2h_bytes_per_step": out_host.numel() * 4},
        "gpu_launches": launches,
        "device_status": status,
        "clocks": clocks.summary(),
        "roofline": roofline,
        "cpu_baseline": cpu_baseline,
    }
    print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
