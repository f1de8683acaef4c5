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


def _bench_module():
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_nvlink_bytes_come_from_the_routing_of_all_ranks():
    """The NVLink roofline is the busiest GPU's ingress or egress, from what every
    rank actually routes: for a routing that sends everything to rank 0's experts
    it is rank 0's ingress, not the uniform expectation."""
    import torch
    b = _bench_module()
    w = dict(T=8, H=4096, E=8, K=2, fp8=False, routing="uniform", name="c5", desc="")
    R, L = 4, 2
    idx_all = [torch.tensor([[0, 1]] * 8) for _ in range(R)]          # everybody picks experts 0 and 1
    nv = b.nvlink_bytes(w, R, idx_all=idx_all)
    remote_in_rank0 = 3 * 8 * 2                                      # three other ranks, 8 tokens, 2 picks
    assert nv["selections_remote_max_gpu"] == remote_in_rank0
    assert nv["dispatch_bytes_max_gpu"] == remote_in_rank0 * 2 * 4096
    assert nv["combine_bytes_max_gpu"] == remote_in_rank0 * 2 * 4096
    assert abs(nv["roofline_us"] - 2 * remote_in_rank0 * 8192 / 900e9 * 1e6) < 1e-9
    # an inactive rank neither sends nor receives
    nv2 = b.nvlink_bytes(w, R, inactive=3, idx_all=idx_all)
    assert nv2["selections_remote_max_gpu"] == 2 * 8 * 2
    # fp8 dispatch payload follows the reference's accounting: H + 4*H/128 + 16
    w8 = dict(w, fp8=True)
    assert b.nvlink_bytes(w8, R, idx_all=idx_all)["dispatch_bytes_max_gpu"] == remote_in_rank0 * (4096 + 128 + 16)
    # masked entries move nothing
    idx_masked = [torch.tensor([[0, -1]] * 8) for _ in range(R)]
    assert b.nvlink_bytes(w, R, idx_all=idx_masked)["selections_remote_max_gpu"] == 3 * 8


def test_both_arms_spell_the_workload_the_same_way():
    b = _bench_module()

    class A:
        inactive_rank = -1
    w = dict(b.WORKLOADS["c2"], name="c2")
    cfg = b.config_of(w, 8, A())
    assert set(cfg) == {"workload", "tokens_per_rank", "hidden", "experts", "experts_per_rank", "topk",
                        "ranks", "routing", "dispatch_payload", "inactive_rank"}
    assert cfg["experts_per_rank"] == 32 and cfg["dispatch_payload"] == "fp8_e4m3"
    p = _run(["--steps", "1", "--warmup", "1"])
    d = json.loads([l for l in p.stdout.splitlines() if l.startswith("{")][0])
    assert set(d["config"]) == set(cfg)
