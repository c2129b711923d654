"""The reference arm of bench.py runs on the CPU, so its output contract can be checked without a GPU: one JSON
line with the agreed keys, the CPU baseline described, zero device traffic."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    j = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "impl"):
        assert key in j, key
    assert j["impl"] == "reference" and j["unit"] == "tokens/s" and j["higher_is_better"] is True and j["value"] > 0
    assert j["cpu_baseline"]["kind"] == "port" and j["cpu_baseline"]["cores"] >= 1 and j["cpu_baseline"]["value"] == j["value"]
    assert j["e2e"]["h2d_bytes_per_step"] == 0 and j["e2e"]["d2h_bytes_per_step"] == 0 and j["e2e"]["value"] == j["value"]
    assert "workload" in j["config"] and "config 1" in j["config"]["workload"]


def test_reference_arm_other_ranks_do_no_work():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert res.returncode == 0 and res.stdout.strip() == ""


def test_roofline_sum_arithmetic():
    """`roofline_sum` of the bench line: GEMM flops over the tensor peak plus stage bytes over the HBM peak, with the
    NVLink term only for an expert-parallel group."""
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    peaks = dict(hbm=6000.0, tf=1500.0, tf_sustained=1400.0, source="test")
    T = 16384
    r = bench.roofline_sum(T, 3 * T, 0.5, peaks)
    gemm = 3 * T * 6 * 1536 * 1280 / 1500e12 * 1e3
    hbm = T * (3088 + 9232 + 12304) / 6000e9 * 1e3
    assert abs(r["gemm_ms"] - gemm) < 1e-9 and abs(r["hbm_ms"] - hbm) < 1e-9
    assert abs(r["ms"] - (gemm + hbm)) < 1e-9 and abs(r["frac"] - (gemm + hbm) / 0.5) < 1e-9
    assert "comm_ms" not in r
    r8 = bench.roofline_sum(T, 3 * T, 1.0, peaks, world=8)
    comm = 2 * T * 2 * 1536 * 2 * 7 / 8 / 900e9 * 1e3
    assert abs(r8["comm_ms"] - comm) < 1e-9
    assert abs(r8["ms_overlapped"] - max(gemm + hbm, comm)) < 1e-9
