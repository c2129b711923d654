"""GPU parity of prichs_moe_backward against the oracle's restatement of the reference's MoE backward pass
(crates/prichs-model/src/model.rs:566-766).

The file sorts after the forward suites so that a run which stops at the first failure has covered the forward first."""
import numpy as np
import pytest

from _util import assert_close

pytestmark = pytest.mark.gpu

TOL = 3e-2  # bf16 operands, fp32 accumulation, two chained products


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available(), "these tests need a GPU"
    return torch


def _run(torch, oracle, seed, T, d, f, E, k, bias=None, x_kind="bf16", dy_kind="f32"):
    from prichs_b200 import MoELayer, synth
    ws = synth.layer_weights(seed, d, f, E, std=0.05, bf16=True)
    bias = synth.router_bias(seed, E, -0.1, 0.1) if bias is None else bias
    x = synth.round_bf16(synth.normal(seed + 1, 0, (T, d)))
    R = synth.round_bf16(synth.normal(seed + 2, 0, (T, d)))
    m = MoELayer.from_weights(ws, k, mode="bf16")
    m.router_bias = bias
    to = {"bf16": torch.bfloat16, "f32": torch.float32}
    xd = torch.from_numpy(x).cuda().to(to[x_kind])
    m.forward(xd)
    st = m.last_stash()
    grads = [torch.zeros(w.shape, dtype=torch.float32, device="cuda") for w in ws]
    dx = m.backward(xd, torch.from_numpy(R).cuda().to(to[dy_kind]), grads).cpu().numpy()
    m.sync_status()
    ref_fwd = oracle.moe_forward_train(ws, bias, k, x)
    agree = np.all(ref_fwd["selected"] == st.selected_experts.reshape(T, k), axis=1)
    ref = oracle.moe_backward(ws, bias, k, x, R)
    return dx, [g.cpu().numpy() for g in grads], ref, agree, st


def _rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / (np.linalg.norm(b.astype(np.float64)) + 1e-30))


def test_backward_intermediates_stage_by_stage(torch_cuda, oracle):
    """Every intermediate of the backward pass against the numpy model of its decomposition, in execution order, so
    that a wrong kernel shows up at its own stage: recomputed [gate | up], dY rows, scalars, d_act, [d_gate | d_up],
    dX rows, d_logits."""
    import torch
    from prichs_b200 import MoELayer, synth
    from _util import np_backward_decomposed
    T, d, f, E, k = 200, 256, 256, 8, 2
    ws = synth.layer_weights(231, d, f, E, std=0.05, bf16=True)
    bias = synth.router_bias(231, E, -0.1, 0.1)
    x = synth.round_bf16(synth.normal(232, 0, (T, d)))
    R = synth.round_bf16(synth.normal(233, 0, (T, d)))
    m = MoELayer.from_weights(ws, k, mode="bf16")
    m.router_bias = bias
    xd = torch.from_numpy(x).cuda().bfloat16()
    m.forward(xd)
    st = m.last_stash()
    sel = st.selected_experts.reshape(T, k).astype(np.int64)
    gates = st.gating_weights.reshape(T, k).astype(np.float32)
    dx = m.backward(xd, torch.from_numpy(R).cuda(), [torch.zeros(w.shape, device="cuda") for w in ws]).cpu().numpy()
    m.sync_status()
    model = np_backward_decomposed(ws, x, R, sel, gates, st.expert_token_counts.astype(np.int64))
    pos = m.debug_buffer(4, T * 2 * 4).view(np.int32).reshape(T, 2)
    assert np.array_equal(pos, model["pos"]), "row map of the forward"
    live = model["live"]
    rows = int(live.max()) + 1

    def bf(which, width):
        return synth.from_bf16_bits(m.debug_buffer(which, rows * width * 2).view(np.uint16)).reshape(rows, width)

    for which, width, key in ((9, 2 * f, "gu"), (10, d, "dyall")):
        assert_close(bf(which, width)[live], model[key][live], TOL, key)
    scal = m.debug_buffer(14, T * 2 * 4).view(np.float32).reshape(T, 2)
    assert_close(scal, model["scal"], TOL, "scalars <expert row, d_out>")
    for which, width, key in ((11, f, "dh"), (12, 2 * f, "dgu"), (13, d, "dxall")):
        assert_close(bf(which, width)[live], model[key][live], TOL, key)
    dlog = m.debug_buffer(15, T * 8 * 4).view(np.float32).reshape(T, 8)[:, :E]
    assert_close(dlog, model["dlog"], TOL, "d_logits")
    assert_close(dx, model["dx"], TOL, "d_x")


def test_backward_matches_oracle(torch_cuda, oracle):
    import torch
    T, d, f, E, k = 300, 512, 256, 8, 2
    dx, grads, ref, agree, _ = _run(torch, oracle, 201, T, d, f, E, k)
    assert agree.all(), "pick another seed: the comparison of weight gradients needs identical routing"
    assert_close(dx, ref["d_x"], TOL, "d_x")
    for i, (g, r) in enumerate(zip(grads, ref["grads"])):
        assert _rel(g, r) <= TOL, (i, _rel(g, r))


def test_backward_empty_expert_and_accumulation(torch_cuda, oracle):
    import torch
    T, d, f, E, k = 130, 256, 256, 8, 2
    bias = np.zeros(E, np.float32)
    bias[5] = -50.0  # expert 5 receives nothing: its gradients must stay as they were (model.rs:641-643)
    dx, grads, ref, agree, st = _run(torch, oracle, 211, T, d, f, E, k, bias=bias, x_kind="f32", dy_kind="bf16")
    assert st.expert_token_counts[5] == 0
    assert agree.all()
    assert_close(dx, ref["d_x"], TOL, "d_x")
    for j in range(3):
        assert not grads[4 + 3 * 5 + j].any()
    for i, (g, r) in enumerate(zip(grads, ref["grads"])):
        if r.any():
            assert _rel(g, r) <= TOL, (i, _rel(g, r))


def test_backward_dx_only_and_errors(torch_cuda, oracle):
    import torch
    from prichs_b200 import MoELayer, PrichsError, synth
    T, d, f, E, k = 64, 256, 256, 4, 2
    ws = synth.layer_weights(221, d, f, E, std=0.05, bf16=True)
    x = synth.round_bf16(synth.normal(222, 0, (T, d)))
    R = synth.round_bf16(synth.normal(223, 0, (T, d)))
    m = MoELayer.from_weights(ws, k, mode="bf16")
    xd = torch.from_numpy(x).cuda().bfloat16()
    with pytest.raises(PrichsError):
        m.backward(xd, torch.from_numpy(R).cuda())  # no forward yet
    m.forward(xd)
    dx = m.backward(xd, torch.from_numpy(R).cuda()).cpu().numpy()
    ref = oracle.moe_backward(ws, np.zeros(E, np.float32), k, x, R)
    assert_close(dx, ref["d_x"], TOL, "d_x without weight gradients")
    with pytest.raises(PrichsError):
        m.backward(xd[:10], torch.from_numpy(R[:10]).cuda())  # not the batch of the last forward


@pytest.mark.parametrize("x_kind", ["bf16", "f32"])
def test_block_backward_matches_oracle(torch_cuda, oracle, x_kind):
    """x_res -> rms_norm -> MoE -> + x_res, backwards: oracle.moe_backward on the normalised rows, then
    oracle.rmsnorm_backward seeded with d_out (model.rs:566-789)."""
    import torch
    from prichs_b200 import MoELayer, synth
    T, d, f, E, k, eps = 150, 512, 256, 8, 2, 1e-5
    ws = synth.layer_weights(241, d, f, E, std=0.05, bf16=True)
    bias = synth.router_bias(241, E, -0.1, 0.1)
    x_res = synth.normal(242, 0, (T, d), 0.0, 2.0)
    if x_kind == "bf16":
        x_res = synth.round_bf16(x_res)
    R = synth.round_bf16(synth.normal(243, 0, (T, d)))
    w = (1.0 + 0.1 * synth.normal(244, 0, (d,))).astype(np.float32)
    m = MoELayer.from_weights(ws, k, mode="bf16")
    m.router_bias = bias
    xd = torch.from_numpy(x_res).cuda().to({"bf16": torch.bfloat16, "f32": torch.float32}[x_kind])
    wd = torch.from_numpy(w).cuda()
    m.block_forward(xd, wd, eps)
    st = m.last_stash()
    grads = [torch.zeros(wt.shape, dtype=torch.float32, device="cuda") for wt in ws]
    d_norm = torch.zeros(d, dtype=torch.float32, device="cuda")
    dx = m.block_backward(xd, wd, eps, torch.from_numpy(R).cuda(), grads, d_norm).cpu().numpy()
    m.sync_status()
    xn = synth.round_bf16(oracle.rms_norm(x_res, w, eps))  # the layer's input in bf16 mode
    ref_fwd = oracle.moe_forward_train(ws, bias, k, xn)
    assert np.all(ref_fwd["selected"] == st.selected_experts.reshape(T, k)), "pick another seed: routing must agree"
    ref = oracle.moe_backward(ws, bias, k, xn, R)
    ref_dx, ref_dg = oracle.rmsnorm_backward(ref["d_x"], x_res, w, eps, d_x=R)
    assert_close(dx, ref_dx, TOL, "d_x_residual")
    assert _rel(d_norm.cpu().numpy(), ref_dg) <= TOL
    for i, (g, r) in enumerate(zip(grads, ref["grads"])):
        assert _rel(g.cpu().numpy(), r) <= TOL, (i, _rel(g.cpu().numpy(), r))
    with pytest.raises(Exception):
        m.backward(xd, torch.from_numpy(R).cuda())  # the last forward was the block entry point
