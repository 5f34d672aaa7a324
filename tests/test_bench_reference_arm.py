"""The reference arm of bench.py (`--impl reference`) runs on the host cores alone: the CPU path of
the MoE layer for the headline configuration, one bounded step. Checks the JSON line's contract."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_one_json_line():
    env = dict(os.environ)
    env["CUDA_VISIBLE_DEVICES"] = ""  # the arm must not need a GPU
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference"
    assert d["metric"] == "moe_layer_decode_tokens_per_s" and d["unit"] == "layer_tokens/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 1
    assert d["value"] > 0 and d["ms_per_step"] > 0
    assert d["config"]["workload"] == "moe_ffn_decode_q4_0_T1"
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["sample"]
    assert abs(cb["value"] - d["value"]) <= 1e-9 * max(1.0, d["value"])
    e2e = d["e2e"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0
    assert abs(e2e["value"] - d["value"]) <= 1e-9 * max(1.0, d["value"]) and e2e["unit"] == d["unit"]
