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


def test_parity_check_of_the_bench_line_detects_a_wrong_result(oracle):
    """`parity` of the bench line is computed by bench.parity_check from the layer's own forward. With a stand-in layer
    that returns the oracle's result the check passes; with a wrong selection, a wrong count or a wrong output row it
    reports it (bench.py then exits non-zero). No GPU is involved."""
    import importlib.util
    import numpy as np
    import torch
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    from prichs_b200 import synth
    from prichs_b200.moe import MoEStash
    spec = importlib.util.spec_from_file_location("bench_mod2", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    D, F, E, K = bench.D, bench.F, bench.E, bench.K
    T = 48
    ws = synth.layer_weights(11, D, F, E, bf16=True)
    bias = synth.router_bias(11, E, -0.1, 0.1)
    x = synth.tokens(11, T, D, bf16=True)
    ref = oracle.moe_forward_train(ws, bias, K, x)

    class StandIn:
        def __init__(self, out, sel, counts):
            self.out, self.sel, self.counts = out, sel, counts

        def forward(self, _x):
            return torch.from_numpy(self.out)

        def sync_status(self):
            pass

        def last_stash(self):
            return MoEStash(ref["logits"], self.sel.reshape(-1), ref["gating"].reshape(-1), self.counts)

    def run(out, sel, counts):
        p = bench.parity_check(StandIn(out, sel, counts), ws, bias, x, None, 32, 5)
        p["ok"] = bool(p["routing_bit_exact"] and p["max_rel"] <= 2e-2 and p["logits_max_abs_err"] <= 1e-3)
        return p

    good = run(ref["out"], ref["selected"], ref["counts"])
    assert good["ok"] and good["routing_bit_exact"] and good["max_rel"] == 0.0 and good["tokens_checked"] == 32
    swapped = ref["selected"].copy()
    swapped[3] = swapped[3][::-1]
    assert not run(ref["out"], swapped, ref["counts"])["routing_bit_exact"]
    wrong_counts = ref["counts"].copy()
    wrong_counts[0] += 1
    assert not run(ref["out"], ref["selected"], wrong_counts)["routing_bit_exact"]
    bad = ref["out"] * np.float32(1.1)
    r = run(bad, ref["selected"], ref["counts"])
    assert r["routing_bit_exact"] and not r["ok"] and r["max_rel"] > 2e-2
