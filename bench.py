"""Throughput of modulated-quantisation DDIM sampling with the pixel UNet.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one full sampling pass of the hot path over one batch: 100 DDIM steps (quad
skip, eta 0) of the W4A4 modulated UNet (split shortcut quantisation) on a batch of 256
images per GPU, x_T ~ N(0,1) (synthetic noise; random-init weights seed 0).  The metric is
images per second over all GPUs.  Rank 0 prints one JSON line.
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

BATCH_PER_GPU = 256
DDIM_STEPS = 100
W_BITS, A_BITS = 4, 4
METRIC = "UNet sampling images/sec"
WORKLOAD = "pixel UNet 3x32x32 W4A4 modulated, split shortcut, 100 DDIM quad steps, batch 256/GPU"

# measured DRAM bytes / algorithmic bytes of one launch (ncu captures summarised in profiles/):
# the quantiser reads x and a_hat twice (two passes), 21 B moved per 13 B algorithmic
DRAM_TRAFFIC_RATIO = {"modiff_modq_src": 1.52, "modiff_modq_gn": 1.52, "modiff_modq_pair": 1.28, "modiff_modq": 1.52, "modiff_igemm_conv": 0.83}

WQ = {'n_bits': W_BITS, 'channel_wise': True, 'scale_method': 'max'}
AQ = {'n_bits': A_BITS, 'symmetric': True, 'channel_wise': False, 'scale_method': 'max',
      'leaf_param': True, 'dynamic': True}


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


def cpu_reference_sample(steps_run, threads, batch=8):
    """Times the CPU restatement of the reference path (oracle/) on the host cores: `batch`
    images, the first `steps_run` DDIM steps of the 100-step schedule (the unquantised first
    step included), extrapolated to a full run.  Returns images per second."""
    import modiff_b200 as m
    import oracle
    torch.set_num_threads(threads)
    torch.manual_seed(0)
    net = m.Model(m.make_config(split_shortcut=True))
    state = {k: v.detach().clone() for k, v in net.state_dict().items()}
    ref = oracle.OracleUNet(state, w_bits=W_BITS, a_bits=A_BITS, split_shortcut=True)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(batch, 3, 32, 32, generator=g)
    seq = oracle.quad_sequence(1000, DDIM_STEPS)[-steps_run:]
    t0 = time.perf_counter()
    oracle.ddim_sample(x, seq, ref.forward, oracle.linear_betas())
    dt = time.perf_counter() - t0
    return batch / (dt * DDIM_STEPS / steps_run), dt


def run_reference(args):
    """`--impl reference`: the reference's own (fake-quant fp32, CPU) implementation of the
    path, restated in oracle/, on all host threads.  Rank 0 only."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    steps_run = 10
    for _ in range(args.warmup):
        cpu_reference_sample(2, threads)
    t0 = time.perf_counter()
    vals = [cpu_reference_sample(steps_run, threads)[0] for _ in range(args.steps)]
    dt = time.perf_counter() - t0
    v = sum(vals) / len(vals)
    sample = f"batch 8, first {steps_run} of {DDIM_STEPS} DDIM steps per bench step, extrapolated x{DDIM_STEPS // steps_run}"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1000.0 * dt / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "reference_arm": "CPU restatement of qdiff fake-quant path"},
        "cpu_baseline": {"value": v, "unit": "images/s", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": v, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="modiff_b200")
    ap.add_argument("--batch", type=int, default=BATCH_PER_GPU, help="images per GPU")
    ap.add_argument("--ddim-steps", type=int, default=DDIM_STEPS,
                    help="profiling aid: keep only the last n timesteps of the 100-step schedule")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quant-mode", choices=["dynamic", "qdiff"], default="dynamic",
                    help="'qdiff': non-dynamic activation scales (each layer keeps the scale of its "
                         "first quantised call), the mode of a calibrated checkpoint; not the "
                         "headline configuration")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import modiff_b200 as m
    from modiff_b200 import _lib, distributed as D
    import torch.distributed as dist

    rank, local_rank, world = D.init()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    batch = args.batch

    torch.manual_seed(0)
    net = m.Model(m.make_config(split_shortcut=True)).eval()
    aq = dict(AQ, dynamic=(args.quant_mode == "dynamic"))
    qnn = m.QuantModel(net, WQ, aq, sm_abit=8, modulate=True).to(dev).eval()
    qnn.set_quant_state(True, True)
    betas = torch.from_numpy(m.get_beta_schedule()).float()
    seq = m.make_timestep_sequence(1000, DDIM_STEPS, "quad")[-args.ddim_steps:]
    workload = WORKLOAD if (args.ddim_steps == DDIM_STEPS and batch == BATCH_PER_GPU) else \
        f"REDUCED (profiling) {args.ddim_steps} DDIM steps, batch {batch}/GPU: " + WORKLOAD
    if args.quant_mode != "dynamic":
        workload = "STATIC activation scales (quant_mode qdiff): " + workload

    g = torch.Generator().manual_seed(D.rank_seed(1, rank))
    x_host = torch.randn(batch, 3, 32, 32, generator=g).pin_memory()
    out_host = torch.empty(world * batch, 3, 32, 32).pin_memory()
    x_dev = x_host.to(dev)

    def one_pass(x):
        qnn.reset_cache()
        xs, _ = m.generalized_steps(x, seq, qnn, betas, eta=0.0)
        return D.gather_samples(xs[-1])

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
        one_pass(x_dev)

    n0 = _lib.LAUNCHES[0]
    with ClockSampler(local_rank) as clocks:
        ms = timed(lambda: one_pass(x_dev), args.steps)
    launches = _lib.LAUNCHES[0] - n0

    def e2e_pass():
        xd = x_host.to(dev, non_blocking=True)
        res = one_pass(xd)
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
    _lib.TIMER = _lib.KernelTimer()
    qnn.reset_cache()
    m.generalized_steps(x_dev, seq, qnn, betas, eta=0.0)
    summ = _lib.TIMER.summary()
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
    roofline = {"kernel": dom, "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
                "algorithmic_bytes_per_launch": d["bytes"] / d["launches"],
                "launches": d["launches"], "share_of_kernel_time": d["ms"] / total_ms,
                "per_entry_point_ms": {k: round(v["ms"], 2) for k, v in summ.items()}}

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        steps_run = 10
        v, dt = cpu_reference_sample(steps_run, threads)
        cpu_baseline = {"value": v, "unit": "images/s", "cores": threads, "kind": "port",
                        "sample": f"batch 8, first {steps_run} of {DDIM_STEPS} DDIM steps "
                                  f"({dt:.1f} s), extrapolated x{DDIM_STEPS // steps_run}"}

    line = {
        "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": {"workload": workload, "global_batch": world * batch, "ddim_steps": args.ddim_steps,
                   "parallelism": f"dp{world}", "l2": "working set (>10 GB of caches) exceeds L2"},
        "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": x_host.numel() * 4,
                "d2h_bytes_per_step": out_host.numel() * 4},
        "gpu_launches": launches,
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
