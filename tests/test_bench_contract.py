"""bench.py's command-line contract, as far as it can be checked without a GPU: the five
workloads, the reference arm's JSON line (the CPU oracle timed on a bounded sample), and that
under a multi-rank launch only rank 0 runs and prints it."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402


def test_every_quoted_workload_has_a_configuration():
    assert sorted(bench.CONFIGS) == ["ldm_w8a8", "pixel_w4a3", "pixel_w4a4", "pixel_w8a8", "sd_w8a8"]
    for name, cfg in bench.CONFIGS.items():
        assert {"kind", "w_bits", "a_bits", "batch", "evals", "seed", "workload"} <= set(cfg), name
        assert str(cfg["batch"]) in cfg["workload"]
    # batches and evaluation counts the throughput figures are quoted on
    assert bench.CONFIGS["pixel_w4a4"]["batch"] == 256 and bench.CONFIGS["pixel_w4a4"]["evals"] == 100
    assert bench.CONFIGS["ldm_w8a8"]["batch"] == 32 and bench.CONFIGS["ldm_w8a8"]["evals"] == 500
    assert bench.CONFIGS["sd_w8a8"]["batch"] == 8 and bench.CONFIGS["sd_w8a8"]["evals"] == 50
    # the latent and SD workloads are quoted with the integer attention, the pixel ones without
    assert bench.CONFIGS["ldm_w8a8"].get("int8_attention") and bench.CONFIGS["sd_w8a8"].get("int8_attention")
    assert not bench.CONFIGS["pixel_w4a4"].get("int8_attention")


def _run(args, env_extra):
    env = dict(os.environ, **env_extra)
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + args, cwd=ROOT, env=env,
                          capture_output=True, text=True, timeout=600)


def test_reference_arm_prints_one_json_line_on_rank_0_only():
    quiet = _run(["--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
                 {"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert quiet.returncode == 0 and quiet.stdout.strip() == ""
    out = _run(["--impl", "reference", "--steps", "1", "--warmup", "0"], {"RANK": "0", "WORLD_SIZE": "1"})
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == bench.METRIC
    assert line["unit"] == "images/s" and line["higher_is_better"] is True and line["value"] > 0
    assert line["steps"] == 1 and line["warmup"] == 0 and line["gpu_launches"] == 0
    assert line["config"]["name"] == "pixel_w4a4" and "batch 256" in line["config"]["workload"]
    base = line["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and base["value"] == line["value"]
    assert "25 of 100" in base["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "images/s", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
