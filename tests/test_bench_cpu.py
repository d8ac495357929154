"""bench.py's host-side logic and its reference arm, without a GPU."""
import importlib.util
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_flops_count_visible_pairs(bench):
    assert bench.flops(4, 16, 8192, 8192) == 4.0 * 4 * 16 * 8192 * 8192 * 128
    # causal, bottom-right aligned: row i of Lq sees (Lk - Lq) + i + 1 keys
    lq, lk = 5, 9
    pairs = sum((lk - lq) + i + 1 for i in range(lq))
    assert bench.flops(1, 1, lq, lk, causal=True) == 4.0 * pairs * 128


def test_scaling_and_config_of_the_headline_workload(bench):
    assert bench.scaling_of("main", 8) == "strong"
    assert bench.scaling_of("l4k", 8) == "weak"
    one = bench.workload_config("main", 1)
    assert one["global_batch"] == 4 and one["heads"] == 16 and one["len_q"] == one["len_kv"] == 8192
    assert one["parallelism"] == "single GPU" and "no flush" in one["l2_policy"]
    # the one problem dealt to the ranks: the global batch stays, a rank's inputs shrink
    two, four, eight = (bench.workload_config("main", n) for n in (2, 4, 8))
    assert eight["global_batch"] == 4 and "dealt to 8 GPUs" in eight["workload"]
    assert "no flush" in two["l2_policy"]                                      # 201 MB per rank
    assert "rewritten before every timed launch" in four["l2_policy"]          # 101 MB
    assert "rewritten before every timed launch" in eight["l2_policy"]         # 50 MB
    # every other workload: a copy per rank
    assert bench.workload_config("l4k", 4)["global_batch"] == 16 * 4


def test_l2_policy_threshold_is_the_l2_size(bench):
    assert "no flush" in bench.l2_policy_text(bench.L2_BYTES + 1)
    assert "rewritten" in bench.l2_policy_text(bench.L2_BYTES)
    assert bench.FLUSH_BYTES >= 2 * bench.L2_BYTES


def test_regime_arithmetic(bench):
    r = bench.regime(total_ms=32.0, n=20, step_flops=2.199e12, mhz=1700.0)
    assert r["launches"] == 20 and abs(r["ms_per_launch"] - 1.6) < 1e-12
    assert abs(r["tflops"] - 2.199e12 / 1.6e-3 / 1e12) < 1e-9
    assert abs(r["sm_cycles_per_launch"] - 1.6e-3 * 1700e6) < 1e-3
    assert "sm_cycles_per_launch" not in bench.regime(1.0, 1, 1.0, None)


def test_every_config_of_the_sweep_is_a_known_workload(bench):
    for name, layouts in bench.CONFIG_SWEEP:
        assert name in bench.WORKLOADS and set(layouts) <= {"bhld", "bshd"}
    for name, (_, source) in bench.NCU_TRAFFIC.items():
        assert name in bench.WORKLOADS and (ROOT / source).exists()


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "smoke",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads([ln for ln in out.stdout.splitlines() if ln.startswith("{")][-1])
    assert line["impl"] == "reference" and line["unit"] == "TFLOPS" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["gpu_launches"] == 0
    assert line["cpu_baseline"]["kind"] == "reference" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOPS", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    assert line["config"]["workload"].startswith("smoke:")
