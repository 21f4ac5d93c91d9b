"""bench.py keeps its contract: one JSON line with the agreed keys at one GPU, a refusal for more, and the reference arm's
`unavailable` line.  The measured run uses one layer of the headline shape (named in ``config``) to stay short."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*args, timeout=600):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], cwd=ROOT, capture_output=True,
                          text=True, timeout=timeout)


def test_more_than_one_gpu_is_refused_with_one_line():
    p = run_bench("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert p.returncode == 2
    assert len(p.stdout.strip().splitlines()) == 1 and "one GPU" in p.stdout


def test_reference_arm_says_why_it_is_unavailable():
    p = run_bench("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert p.returncode == 0
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


@pytest.mark.gpu
def test_the_line_of_a_short_run_has_every_agreed_key():
    p = run_bench("--layers", "1", "--steps", "3", "--warmup", "3", "--repeats", "2")
    assert p.returncode == 0, p.stderr[-2000:]
    d = json.loads(p.stdout.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "prefill", "roofline", "points", "e2e", "gpu_launches", "clocks"):
        assert key in d, key
    assert d["n_gpus"] == 1 and d["steps"] == 3 and d["warmup"] == 3 and d["higher_is_better"] is True
    assert d["value"] > 0 and d["unit"] == "tokens/s" and d["dtype"] == "bf16" and "synthetic" in d["data"]
    assert abs(d["value"] - d["config"]["global_batch"] * 1000.0 / d["ms_per_step"]) < 1e-6 * d["value"]
    # config: flat, at most 20 keys, both layer counts named
    cfg = d["config"]
    assert len(cfg) <= 20 and all(not isinstance(v, (dict, list)) for v in cfg.values())
    assert cfg["layers"] == 1 and cfg["layers_full"] == 24 and cfg["global_batch"] == 8 and cfg["seq_len"] == 4096
    for key in ("hidden", "heads", "kv_heads", "head_dim", "experts", "top_k", "moe_intermediate", "shared_intermediate", "vocab"):
        assert key in cfg
    pre = d["prefill"]
    assert pre["tokens"] == 2048 and pre["value"] > 0 and pre["ms"] > 0 and 0 < pre["frac"] < 1.5
    roof = d["roofline"]
    assert roof["bound"] == "hbm" and roof["unit"] == "GB/s" and roof["peak"] > 0
    assert abs(roof["frac"] - roof["achieved"] / roof["peak"]) < 1e-9 and 0 < roof["frac"] < 1.5
    assert set(d["points"]) == {"decode_b1", "decode_b64"} and all(v > 0 for v in d["points"].values())
    e2e = d["e2e"]
    assert e2e["value"] > 0 and e2e["h2d_bytes_per_step"] > 0 and e2e["d2h_bytes_per_step"] > 0
    assert e2e["value"] != d["value"]                       # measured through the entry point, not copied
    assert d["gpu_launches"] > 0
    assert d["clocks"]["sm_max_mhz"] and "reasons" in d["clocks"]
