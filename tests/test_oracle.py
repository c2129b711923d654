"""Pins the CPU oracle (oracle/moe_oracle.cpp). The reference ships no numeric vectors for this path, so the
pins are: closed-form answers for the constants of the reference's own MoE fixture
(crates/prichs-cuda/src/engine.rs:3091-3118: all weights 0.1, x = 0.5, gates 0.5), hand-computed top-k cases,
an independent numpy restatement, the committed golden file, and the structural properties the reference's
tests assert (crates/prichs-model/src/model.rs:1952-1963)."""
import math
import os

import numpy as np
import pytest

from _util import assert_close, golden_small_inputs, np_moe_forward, np_top_k_unbiased, small_int_weights


def _const_layer(d, f, E, w=0.1):
    ws = [np.full((d, E), w, np.float32)]
    for _ in range(1 + E):
        ws += [np.full((d, f), w, np.float32), np.full((d, f), w, np.float32), np.full((f, d), w, np.float32)]
    return ws


def test_reference_fixture_closed_form(oracle):
    # engine.rs:3067-3118: hidden 4, intermediate 8, 2 experts, every weight 0.1, every input 0.5.
    # gate = up = 4 * 0.5 * 0.1 = 0.2; act = silu(0.2) * 0.2; expert row = 8 * act * 0.1.
    # Equal router logits: top-2 of 2 experts picks both (index order), gates 0.5 each (as the fixture passes),
    # so out = shared + 0.5 * e0 + 0.5 * e1 = 2 * expert row.
    d, f, E, k, T = 4, 8, 2, 2, 2
    ws = _const_layer(d, f, E)
    x = np.full((T, d), 0.5, np.float32)
    r = oracle.moe_forward_train(ws, np.zeros(E, np.float32), k, x)
    act = (0.2 / (1.0 + math.exp(-0.2))) * 0.2
    row = 8 * act * 0.1
    np.testing.assert_allclose(r["shared_out"], row, rtol=2e-6)
    np.testing.assert_allclose(r["out"], 2 * row, rtol=2e-6)
    np.testing.assert_allclose(r["logits"], 0.2, rtol=1e-6)
    assert r["selected"].tolist() == [[0, 1], [0, 1]]
    np.testing.assert_allclose(r["gating"], 0.5, rtol=1e-6)
    assert r["counts"].tolist() == [2, 2]


def test_top_k_known_answers(oracle):
    # ties go to the lower index; gates come from the RAW logits of the selected experts (ops.rs:233-245)
    idx, w = oracle.top_k_gating_unbiased([1, 2, 2, 0.5], [1, 2, 2, 0.5], 2)
    assert idx.tolist() == [1, 2] and np.allclose(w, [0.5, 0.5])
    raw = np.array([0.0, 1.0, 2.0, 3.0], np.float32)
    routed = raw + np.array([5.0, 0.0, 0.0, 0.0], np.float32)  # the bias moves expert 0 to the front
    idx, w = oracle.top_k_gating_unbiased(raw, routed, 2)
    assert idx.tolist() == [0, 3]
    e = np.exp(np.array([0.0 - 3.0, 0.0], np.float32))
    np.testing.assert_allclose(w, e / (e.sum() + 1e-9), rtol=1e-6)
    idx, w = oracle.top_k_gating_unbiased([0.3, -1.0], [0.3, -1.0], 1)
    assert idx.tolist() == [0] and np.allclose(w, [1.0])
    idx, _ = oracle.top_k_gating_unbiased(np.zeros(8), np.zeros(8), 2)
    assert idx.tolist() == [0, 1]
    # -inf selection logits are still ordered stably
    idx, _ = oracle.top_k_gating_unbiased(np.zeros(4), [-np.inf, -np.inf, 1.0, -np.inf], 2)
    assert idx.tolist() == [2, 0]
    with pytest.raises(AssertionError):
        oracle.top_k_gating_unbiased([1.0], [1.0], 2)


def test_top_k_matches_numpy_restatement(oracle):
    rng = np.random.default_rng(0)
    for _ in range(300):
        n = int(rng.integers(2, 9))
        raw = rng.standard_normal(n).astype(np.float32)
        if rng.random() < 0.3:
            raw[rng.integers(0, n)] = raw[rng.integers(0, n)]  # force ties
        bias = (rng.standard_normal(n) * 0.1).astype(np.float32)
        k = int(rng.integers(1, min(n, 3) + 1))
        i0, w0 = oracle.top_k_gating_unbiased(raw, raw + bias, k)
        i1, w1 = np_top_k_unbiased(raw, raw + bias, k)
        assert i0.tolist() == i1.tolist()
        np.testing.assert_allclose(w0, w1, rtol=1e-6)
        assert abs(float(w0.sum()) - 1.0) < 1e-6


def test_matmul_matches_naive_loop(oracle):
    # the reference's only numeric GEMM assertion: against a naive loop at 1e-4 (engine.rs:2877-2945)
    rng = np.random.default_rng(1)
    a = rng.standard_normal((2, 4)).astype(np.float32)
    b = rng.standard_normal((4, 3)).astype(np.float32)
    c = oracle.matmul_2d(a, b)
    ref = np.zeros((2, 3), np.float32)
    for i in range(2):
        for kk in range(4):
            for j in range(3):
                ref[i, j] = np.float32(ref[i, j] + np.float32(a[i, kk] * b[kk, j]))
    assert np.array_equal(c, ref)  # same order, separate multiply and add -> bit identical
    with pytest.raises(ValueError):
        oracle.matmul_2d(a, b.T)
    big_a = rng.standard_normal((37, 300)).astype(np.float32)
    big_b = rng.standard_normal((300, 41)).astype(np.float32)
    np.testing.assert_allclose(oracle.matmul_2d(big_a, big_b), big_a.astype(np.float64) @ big_b, atol=1e-4)


def test_swiglu_and_add(oracle):
    g = np.linspace(-30, 30, 101).astype(np.float32)
    u = np.linspace(2, -2, 101).astype(np.float32)
    ref = (g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64)))) * u
    np.testing.assert_allclose(oracle.swiglu(g, u), ref, rtol=1e-6, atol=1e-30)
    assert np.array_equal(oracle.add_tensors(g, u), g + u)


@pytest.mark.parametrize("d,f,E,k,T", [(64, 32, 8, 2, 64), (32, 48, 4, 2, 33), (16, 16, 3, 1, 9)])
def test_forward_matches_numpy_restatement(oracle, d, f, E, k, T):
    rng = np.random.default_rng(d + T)
    ws = [rng.standard_normal((d, E)).astype(np.float32) * 0.3]
    for _ in range(1 + E):
        ws += [rng.standard_normal((d, f)).astype(np.float32) * 0.1, rng.standard_normal((d, f)).astype(np.float32) * 0.1,
               rng.standard_normal((f, d)).astype(np.float32) * 0.1]
    x = rng.standard_normal((T, d)).astype(np.float32)
    bias = (rng.standard_normal(E) * 0.05).astype(np.float32)
    cb = np.array([0.1, -0.2], np.float32)
    r = oracle.moe_forward_train(ws, bias, k, x, concept_bias=cb)
    n = np_moe_forward(ws, bias, k, x, concept_bias=cb)
    assert np.array_equal(r["selected"], n["selected"])
    assert np.array_equal(r["counts"], n["counts"])
    np.testing.assert_allclose(r["gating"], n["gating"], rtol=2e-6)
    assert_close(r["logits"], n["logits"], 1e-5, "logits")
    assert_close(r["out"], n["out"], 1e-5, "out")
    assert int(r["counts"].sum()) == T * k
    # token mask: masked rows equal the full run bit for bit, routing is unchanged
    mask = np.zeros(T, bool)
    mask[::3] = True
    rm = oracle.moe_forward_train(ws, bias, k, x, concept_bias=cb, token_mask=mask)
    assert np.array_equal(rm["out"][mask], r["out"][mask])
    assert np.array_equal(rm["selected"], r["selected"])


def test_golden_file(oracle):
    g = golden_small_inputs()
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "moe_small.npz"))
    r = oracle.moe_forward_train(g["ws"], g["bias"], g["top_k"], g["x"], concept_bias=g["concept_bias"])
    assert np.array_equal(r["selected"], gold["selected"])
    assert np.array_equal(r["counts"], gold["counts"])
    # logits of grid inputs are exact sums of multiples of 2^-9: bit identical on any machine
    assert np.array_equal(r["logits"], gold["logits"])
    np.testing.assert_allclose(r["gating"], gold["gating"], rtol=1e-6)
    assert_close(r["out"], gold["out"], 1e-6, "golden out")


def test_structural_properties_of_reference_tests(oracle):
    # model.rs:1952-1963: with 64 random tokens at least 6 of 8 experts are active, and one bias step moves
    # the bias (towards the under-loaded experts).
    rng = np.random.default_rng(3)
    d, f, E, k, T = 64, 32, 8, 2, 64
    ws = [rng.standard_normal((d, E)).astype(np.float32) * np.float32(math.sqrt(2 / (d + E)))]
    for _ in range(1 + E):
        ws += [rng.standard_normal((d, f)).astype(np.float32) * 0.1] * 2 + [rng.standard_normal((f, d)).astype(np.float32) * 0.1]
    x = rng.standard_normal((T, d)).astype(np.float32)
    r = oracle.moe_forward_train(ws, np.zeros(E, np.float32), k, x)
    assert int((r["counts"] > 0).sum()) >= 6
    b = oracle.update_aux_free_bias(np.zeros(E, np.float32), r["counts"], T, 0.001, k)
    assert np.any(b != 0)
    lo, hi = int(np.argmin(r["counts"])), int(np.argmax(r["counts"]))
    assert b[lo] > b[hi]


def test_bias_update_known_answer(oracle):
    # b_i += gamma * (k/E - count_i/total)   (moe.rs:237-244), f32 arithmetic step by step
    counts = np.array([10, 0, 3, 3], np.int64)
    b0 = np.array([0.5, -0.25, 0.0, 1.0], np.float32)
    b = oracle.update_aux_free_bias(b0, counts, 8, 0.001, 2)
    exp = b0.copy()
    for i in range(4):
        target = np.float32(2) / np.float32(4)
        actual = np.float32(counts[i]) / np.float32(8)
        exp[i] = np.float32(exp[i] + np.float32(np.float32(0.001) * np.float32(target - actual)))
    assert np.array_equal(b, exp)
    assert np.array_equal(oracle.update_aux_free_bias(b0, counts, 0, 0.001, 2), b0)  # total_tokens == 0: no-op


def test_route_with_given_logits(oracle):
    rng = np.random.default_rng(5)
    lg = rng.standard_normal((50, 8)).astype(np.float32)
    bias = (rng.standard_normal(8) * 0.1).astype(np.float32)
    r = oracle.route(None, np.zeros((16, 8), np.float32), bias, 2, logits=lg)
    for t in range(50):
        i, w = np_top_k_unbiased(lg[t], lg[t] + bias, 2)
        assert r["selected"][t].tolist() == i.tolist()
    assert int(r["counts"].sum()) == 100


def test_rms_norm_known_answer(oracle):
    # the reference's own RMSNorm check uses x = [1, 2, 3, 4], weight 1, eps 1e-5 (crates/prichs-cli/src/main.rs:1210-1213,
    # crates/prichs-cuda/src/engine.rs:3032-3064): rms = sqrt(30/4 + 1e-5)
    x = np.array([[1.0, 2.0, 3.0, 4.0]], np.float32)
    out = oracle.rms_norm(x, np.ones(4, np.float32), 1e-5)
    np.testing.assert_allclose(out, x / np.sqrt(7.5 + 1e-5), rtol=1e-6)
    w = np.array([0.5, 2.0, -1.0, 0.0], np.float32)
    np.testing.assert_allclose(oracle.rms_norm(x, w, 1e-5), x / np.sqrt(7.5 + 1e-5) * w, rtol=1e-6)
    with pytest.raises(ValueError):
        oracle.rms_norm(x, np.ones(3, np.float32), 1e-5)


def test_route_properties_hypothesis(oracle):
    """Randomised properties of the routing restatement: gates of a token sum to 1, the selected experts are distinct,
    adding a constant to all selection logits changes nothing, and a bias only changes WHICH experts are picked, never
    the gate formula (gates depend on the raw logits of the picked experts, ops.rs:233-245)."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=60, deadline=None)
    @given(st.integers(1, 40), st.integers(2, 8), st.integers(1, 2), st.integers(0, 2**31 - 1))
    def prop(T, E, k, seed):
        rng = np.random.default_rng(seed)
        lg = rng.standard_normal((T, E)).astype(np.float32) * 3
        bias = rng.standard_normal(E).astype(np.float32)
        w = np.zeros((4, E), np.float32)
        r = oracle.route(None, w, bias, k, logits=lg)
        assert np.allclose(r["gating"].sum(axis=1), 1.0, atol=1e-6)
        assert all(len(set(row)) == k for row in r["selected"].tolist())
        assert int(r["counts"].sum()) == T * k
        r2 = oracle.route(None, w, bias + np.float32(8.0), k, logits=lg)  # exact shift: 8 is a power of two
        shifted_same = np.array_equal((lg + bias).astype(np.float32) + np.float32(8.0), lg + (bias + np.float32(8.0)))
        if shifted_same:
            assert np.array_equal(r["selected"], r2["selected"])
        for t in range(T):
            raw = lg[t, r["selected"][t]]
            e = np.exp(raw - raw.max(), dtype=np.float32)
            s = np.float32(0)
            for v in e:
                s = np.float32(s + v)
            assert np.allclose(r["gating"][t], e * (np.float32(1) / np.float32(s + np.float32(1e-9))), rtol=2e-6)

    prop()
