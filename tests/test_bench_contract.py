"""The benchmark's CPU arm (`bench.py --impl reference`) prints the contract's
JSON line, honours the step counts, and stays silent on ranks other than 0.
The GPU arm needs a device and is exercised by the GPU runs themselves."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(extra, env_extra=None):
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        env.pop(k, None)
    env.update(env_extra or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference"] + extra,
                          cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)


def test_reference_arm_prints_the_contract_line():
    p = _run(["--steps", "2", "--warmup", "1"])
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference"
    assert d["metric"] == "ep_dispatch_combine_tokens_per_s" and d["unit"] == "tokens/s"
    assert d["n_gpus"] == 1 and d["steps"] == 2 and d["warmup"] == 1
    assert d["higher_is_better"] is True and d["scaling"] == "weak" and d["vs_baseline"] is None
    assert d["data"] == "synthetic" and d["dtype"] == "fp8_e4m3+bf16"
    assert d["config"]["workload"].startswith("c2")
    assert d["value"] > 0 and d["ms_per_step"] > 0
    # tokens of one layer over the time of one layer
    assert abs(d["value"] - 128 / (d["ms_per_step"] / 1e3)) < 1e-6 * d["value"]
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    e2e = d["e2e"]
    assert e2e["value"] == d["value"] and e2e["unit"] == d["unit"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


def test_reference_arm_is_silent_on_other_ranks():
    p = _run(["--gpus", "2", "--steps", "2", "--warmup", "1"],
             {"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"})
    assert p.returncode == 0
    assert not [l for l in p.stdout.splitlines() if l.startswith("{")]


def test_reference_arm_covers_all_ranks_work_in_a_group():
    p = _run(["--gpus", "2", "--workload", "c5", "--tokens", "16", "--steps", "1", "--warmup", "1"])
    assert p.returncode == 0, p.stderr[-2000:]
    d = json.loads([l for l in p.stdout.splitlines() if l.startswith("{")][0])
    assert d["n_gpus"] == 2 and d["config"]["ranks"] == 2
    assert abs(d["value"] - 2 * 16 / (d["ms_per_step"] / 1e3)) < 1e-6 * d["value"]
