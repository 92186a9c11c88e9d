"""Host-side pieces of bench.py that need no GPU: the two arms print the same ``config`` object,
the FLOP accounting gives the expected totals, and the reference arm (the CPU restatement on a
bounded sample) emits a well-formed line."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_algorithmic_flops_totals():
    b = _bench()
    cap = 32 * sum(k * 2048 - 256 for k in range(1, 64))
    f1, f2, f3 = b.algorithmic_flops(131072, 32, cap)
    assert abs(f1 / 1e12 - 6.53) < 0.01 and abs(f3 / 1e12 - 138.0) < 0.05
    assert abs((f1 + f2 + f3) / 1e12 - 145.1) < 0.1          # F(density 1) at 131072 tokens, Llama heads
    cap32 = 32 * sum(k * 2048 - 256 for k in range(1, 16))
    assert abs(sum(b.algorithmic_flops(32768, 32, cap32)) / 1e12 - 9.73) < 0.05


def test_both_arms_describe_the_same_workload():
    b = _bench()
    for gpus, exchange in ((1, "push"), (8, "push"), (2, "all_gather")):
        ours = b.workload_config(131072, gpus, exchange, 12.0, "")
        ref = b.workload_config(131072, gpus, exchange)
        assert ours == ref and set(ours) == {"workload", "parallelism", "exchange_note", "l2"}
    assert "8 GPU" in b.workload_config(131072, 8, "push")["parallelism"]


def test_reference_arm_prints_a_complete_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--seq", "4096",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "ms" and line["higher_is_better"] is False
    assert line["value"] > 0 and line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["config"]["workload"].startswith("anchor_attn layer, seq 4096")


def test_triton_bar_leg_reports_unavailable_without_a_checkout():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--triton-bar", "--ref-root",
                          "/nonexistent/reference"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["leg"] == "triton_bar" and str(line["triton_bar"]).startswith("unavailable")
