"""The benchmark's reference arm runs on CPU and prints the contract's JSON line."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "moe_block_tokens_per_s" and d["unit"] == "tokens/s"
    assert d["higher_is_better"] is True and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["config"]["workload"].startswith("DiT-XL/2-MoE")


def test_other_ranks_of_the_reference_arm_do_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                       capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_bench_helpers_are_deterministic():
    """Every parameter is drawn from its own (layer, name) seed, so a trimmed expert-parallel block and an unsharded
    block hold the same values; the Zipf routing option parses as documented."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert bench._param_seed(0, 3, "experts.5.fc1.weight") == bench._param_seed(0, 3, "experts.5.fc1.weight")
    assert bench._param_seed(0, 3, "experts.5.fc1.weight") != bench._param_seed(0, 4, "experts.5.fc1.weight")
    assert bench._param_seed(0, 3, "experts.5.fc1.weight") != bench._param_seed(0, 3, "experts.6.fc1.weight")
    assert bench.zipf_route("router") is None
    assert bench.zipf_route("zipf:1.2") == (1.2, 1.0) and bench.zipf_route("zipf:1.2:0.5") == (1.2, 0.5)
    # algorithmic FLOPs of one FFN call: 2 rows per token x 4 h F (GELU), plus the shared expert in the SwiGLU variant
    assert bench.ffn_flops(16384, "gelu_tanh") == 2 * 16384 * 4 * 1152 * 4608
    assert bench.ffn_flops(16384, "swiglu") == 2 * 16384 * 6 * 1152 * 4608 + 16384 * 6 * 1152 * 2304
