"""Training forward and the engine's call shape on the GPU.

`forward_train` keeps the activations the backward pass reads (the reference's MoEStash / ExpertForwardStash,
crates/prichs-model/src/moe.rs:32-53,186-208); the engine-shaped entry points are driven in the order of the
reference's training step (crates/prichs-model/src/model.rs:1327-1408: gpu_moe_forward_shared, router + top-k,
gpu_moe_forward_expert per expert, gpu_moe_finalize_forward) and must give what one prichs_moe_forward gives and
what the oracle gives."""
import ctypes as C

import numpy as np
import pytest

from _util import assert_close

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _case(seed, T, d, f, E):
    from prichs_b200 import synth
    ws = synth.layer_weights(seed, d, f, E, std=0.05, bf16=True)
    bias = synth.router_bias(seed, E, -0.1, 0.1)
    x = synth.round_bf16(synth.normal(seed + 1, 0, (T, d)))
    return ws, bias, x


def _oracle_stash(oracle, ws, x_rows, slot):
    """gate, up, act, out of one expert (slot 0 = shared) on the rows it saw, with the GPU's rounding points: bf16
    operands, act rounded to bf16 before the down projection."""
    from prichs_b200 import synth
    g = oracle.matmul_2d(x_rows, ws[1 + 3 * slot])
    u = oracle.matmul_2d(x_rows, ws[2 + 3 * slot])
    a = oracle.swiglu(g, u)
    return g, u, a, oracle.matmul_2d(synth.round_bf16(a), ws[3 + 3 * slot])


@pytest.mark.parametrize("T,route_kernel", [(300, 2), (1500, 1)])
def test_forward_train_stash_matches_oracle(oracle, T, route_kernel):
    import torch
    from prichs_b200 import MoELayer
    d, f, E, k = 512, 256, 8, 2
    ws, bias, x = _case(301, T, d, f, E)
    m = MoELayer.from_weights(ws, k, route_kernel=route_kernel)
    m.router_bias = bias
    xd = torch.from_numpy(x).cuda().bfloat16()
    y_plain = m.forward(xd).float().cpu().numpy()
    y, st = m.forward_train(xd)
    m.sync_status()
    assert np.array_equal(y.float().cpu().numpy(), y_plain), "the stash must not change the result"
    given = oracle.route(None, ws[0], bias, k, logits=st.router_logits)
    sel = st.selected_experts.reshape(T, k)
    assert np.array_equal(sel, given["selected"])
    for got, exp, name in zip((st.shared_gate, st.shared_up, st.shared_act, st.shared_out), _oracle_stash(oracle, ws, x, 0),
                              ("shared gate", "shared up", "shared act", "shared out")):
        assert_close(got, exp, TOL, name)
    rs = st.routed_stashes
    assert [r.expert_idx for r in rs] == [e for e in range(E) if st.expert_token_counts[e] > 0]
    for r in rs:
        tok, slot = np.nonzero(sel == r.expert_idx)  # ascending tokens: the reference's expert_assignments order
        assert np.array_equal(r.token_indices, tok)
        assert np.array_equal(r.weights, st.gating_weights.reshape(T, k)[tok, slot])
        assert np.array_equal(r.x, x[tok]), "stashed rows are exact copies of the tokens"
        for got, exp, name in zip((r.gate, r.up, r.act, r.out), _oracle_stash(oracle, ws, x[tok], 1 + r.expert_idx),
                                  ("gate", "up", "act", "out")):
            assert_close(got, exp, TOL, f"expert {r.expert_idx} {name}")


def test_backward_after_forward_train_equals_backward_with_recomputation(oracle):
    """The backward pass reads the stashed pre-activations after a training forward and recomputes them after a plain
    one: both must give the same gradients (the stash holds exactly what the recomputation produces)."""
    import torch
    from prichs_b200 import MoELayer, synth
    T, d, f, E, k = 300, 512, 256, 8, 2
    ws, bias, x = _case(311, T, d, f, E)
    R = synth.round_bf16(synth.normal(313, 0, (T, d)))
    res = []
    for train in (False, True):
        m = MoELayer.from_weights(ws, k)
        m.router_bias = bias
        xd = torch.from_numpy(x).cuda().bfloat16()
        m.forward_train(xd) if train else m.forward(xd)
        grads = [torch.zeros(w.shape, device="cuda") for w in ws]
        dx = m.backward(xd, torch.from_numpy(R).cuda(), grads)
        m.sync_status()
        res.append([dx.cpu().numpy()] + [g.cpu().numpy() for g in grads])
    for a, b in zip(*res):
        assert np.array_equal(a, b)
    ref = oracle.moe_backward(ws, bias, k, x, R)
    assert_close(res[1][0], ref["d_x"], 3e-2, "d_x after a training forward")


@pytest.mark.parametrize("on_device", [False, True])
def test_engine_call_sequence(capi, oracle, on_device):
    """gpu_moe_forward_shared -> routing -> gpu_moe_forward_expert per expert -> gpu_moe_finalize_forward, in the order
    of the reference's step (model.rs:1327-1408), through the C-ABI."""
    import torch
    from prichs_b200 import MoELayer
    L = capi.lib()
    T, d, f, E, k = 200, 256, 256, 8, 2
    ws, bias, x = _case(321, T, d, f, E)
    bias[6] = -50.0  # expert 6 receives nothing: the caller skips it (model.rs:1366)
    m = MoELayer.from_weights(ws, k, max_tokens=T)
    m.router_bias = bias
    m._ensure(T)
    h = m._h
    fp = lambda a: a.ctypes.data
    # 1. shared expert (and, here, the whole layer)
    sg, su, sa = (np.empty((T, f), np.float32) for _ in range(3))
    so = np.empty((T, d), np.float32)
    if on_device:
        xd = torch.from_numpy(x).cuda().bfloat16()
        rc = L.prichs_engine_moe_forward_shared(h, xd.data_ptr(), 1, capi.DTYPE_BF16, T, fp(sg), fp(su), fp(sa), fp(so))
    else:
        rc = L.prichs_engine_moe_forward_shared(h, fp(x), 0, capi.DTYPE_F32, T, fp(sg), fp(su), fp(sa), fp(so))
    assert rc == 0, capi.last_error()
    # 2. router logits and top-k (computed on the device by the call above)
    logits = np.empty((T, E), np.float32)
    selected = np.empty((T, k), np.uintp)
    gating = np.empty((T, k), np.float32)
    assert L.prichs_engine_moe_routing(h, fp(logits), fp(selected), fp(gating), T) == 0, capi.last_error()
    given = oracle.route(None, ws[0], bias, k, logits=logits)
    assert np.array_equal(selected.astype(np.int64), given["selected"])
    np.testing.assert_allclose(gating, given["gating"], rtol=2e-6, atol=1e-7)
    # 3. routed experts, ascending, empty ones skipped
    total = np.zeros((T, d), np.float32) + so  # the reference's accumulation: shared out, then w * expert rows
    for e in range(E):
        n = C.c_size_t(0)
        assert L.prichs_engine_moe_forward_expert(h, e, None, None, 0, C.byref(n), None, None, None, None, None) == 0
        exp_tok, exp_slot = np.nonzero(given["selected"] == e)
        assert n.value == len(exp_tok)
        if n.value == 0:
            assert e == 6
            continue
        idx = np.empty(n.value, np.int32)
        w = np.empty(n.value, np.float32)
        ex, eo = (np.empty((n.value, d), np.float32) for _ in range(2))
        eg, eu, ea = (np.empty((n.value, f), np.float32) for _ in range(3))
        rc = L.prichs_engine_moe_forward_expert(h, e, fp(idx), fp(w), n.value, C.byref(n), fp(ex), fp(eg), fp(eu), fp(ea), fp(eo))
        assert rc == 0, capi.last_error()
        assert np.array_equal(idx, exp_tok) and np.array_equal(w, gating[exp_tok, exp_slot])
        assert np.array_equal(ex, x[exp_tok])
        for got, exp, name in zip((eg, eu, ea, eo), _oracle_stash(oracle, ws, x[exp_tok], 1 + e), ("gate", "up", "act", "out")):
            assert_close(got, exp, TOL, f"expert {e} {name}")
        total[idx] += w[:, None] * eo
    for got, exp, name in zip((sg, su, sa, so), _oracle_stash(oracle, ws, x, 0), ("shared gate", "shared up", "shared act", "shared out")):
        assert_close(got, exp, TOL, name)
    # 4. the layer output
    out = np.empty((T, d), np.float32)
    assert L.prichs_engine_moe_finalize_forward(h, fp(out), out.size) == 0, capi.last_error()
    # ... equals what the pieces add up to (the reference's scatter-add), one prichs_moe_forward, and the oracle
    assert_close(out, total, 1e-2, "output against the sum of the stashed pieces")
    if on_device:  # same bf16 rows; the device forward rounds its output to bf16, the engine path returns fp32
        y = m.forward(torch.from_numpy(x).cuda().bfloat16()).float().cpu().numpy()
        assert_close(y, out, 1e-2, "prichs_moe_forward against the engine sequence")
    else:          # same fp32 rows, same kernels, fp32 output: identical
        y = m.forward(torch.from_numpy(x).cuda()).cpu().numpy()
        assert np.array_equal(y, out), "prichs_moe_forward against the engine sequence"
    ref = oracle.moe_forward_train(ws, bias, k, x)
    agree = np.all(ref["selected"] == given["selected"], axis=1)
    assert_close(out[agree], ref["out"][agree], TOL, "engine sequence against the oracle")
    assert L.prichs_engine_moe_finalize_forward(h, fp(out), 5) == capi.ERR_BAD_SHAPE
