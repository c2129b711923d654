"""Routing without allocation: prichs_moe_route_static against the handle-based path.

Who needs this: code that must get routing decisions at a point where it may not allocate device memory --
a plugin inside an application that owns the memory pool, a latency-critical loop that must stay out of the
allocator, a callback where cudaMalloc would stall the device. Such a caller cannot create a handle, so the
library keeps the router stage's scratch in a fixed 1 MiB device array of its own.

The test calls the entry point through the C-ABI twice in a row (a larger batch first, then a smaller one with
different data and a bias, so that leftovers of the first call would show) and compares logits, selected
experts, gates and counts with what prichs_moe_forward reports for the same inputs (both paths run the same
router kernel, so that comparison is exact) and with the CPU oracle (which shares no code with them). This file sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _bf16_dev(torch, a):
    from prichs_b200 import synth
    return torch.from_numpy(synth.to_bf16_bits(a).view(np.int16)).view(torch.bfloat16).cuda()


def _route_static(torch, capi, x, router, bias, k):
    T, d = x.shape
    E = router.shape[1]
    xd = _bf16_dev(torch, x)
    rd = torch.from_numpy(np.ascontiguousarray(router, np.float32)).cuda()
    bd = torch.from_numpy(np.ascontiguousarray(bias, np.float32)).cuda() if bias is not None else None
    logits = torch.full((T, E), float("nan"), device="cuda")
    sel = torch.full((T, k), -7, dtype=torch.int32, device="cuda")
    gat = torch.full((T, k), float("nan"), device="cuda")
    cnt = torch.full((E,), -7, dtype=torch.int32, device="cuda")
    rc = capi.lib().prichs_moe_route_static(xd.data_ptr(), rd.data_ptr(), bd.data_ptr() if bd is not None else None, T, d, E, k,
                                            logits.data_ptr(), sel.data_ptr(), gat.data_ptr(), cnt.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream)
    assert rc == 0, capi.last_error()
    torch.cuda.synchronize()
    return logits.cpu().numpy(), sel.cpu().numpy(), gat.cpu().numpy(), cnt.cpu().numpy()


def _route_handle(torch, ws, bias, k, x):
    from prichs_b200 import MoELayer
    m = MoELayer.from_weights(ws, k)
    if bias is not None:
        m.router_bias = bias
    m.forward(_bf16_dev(torch, x))
    m.sync_status()
    st = m.last_stash()
    T = x.shape[0]
    out = st.router_logits, st.selected_experts.reshape(T, k), st.gating_weights.reshape(T, k), st.expert_token_counts
    m.close()
    return out


def test_route_static_matches_handle_path_twice_in_a_row(capi, oracle):
    import torch
    from prichs_b200 import synth
    assert torch.cuda.is_available()
    d, f, E, k = 512, 384, 8, 2
    cases = [(300, 7, None, True), (100, 8, synth.router_bias(8, E, -0.2, 0.2), False)]
    for T, seed, bias, bf16_router in cases:
        ws = synth.layer_weights(seed, d, f, E, std=0.05, bf16=True)
        if not bf16_router:
            ws[0] = synth.normal(seed, 1, (d, E), 0.0, 0.05)  # fp32 router weights exercise the 3-way split
        x = synth.tokens(seed, T, d, bf16=True)
        lo, sel, gat, cnt = _route_static(torch, capi, x, ws[0], bias, k)
        lo_h, sel_h, gat_h, cnt_h = _route_handle(torch, ws, bias, k, x)
        assert np.array_equal(lo, lo_h), "logits differ from the handle path"
        assert np.array_equal(sel, sel_h), "selected experts differ from the handle path"
        assert np.array_equal(gat, gat_h), "gates differ from the handle path"
        assert np.array_equal(cnt, cnt_h.astype(np.int32)), "counts differ from the handle path"
        assert int(cnt.sum()) == T * k
        # ... and against the CPU oracle, which shares no code with either GPU path: selection, gates and counts are
        # bit-exact when its top-k is fed the GPU's own logits, and the logits agree with its own to 1e-4
        b = bias if bias is not None else np.zeros(E, np.float32)
        given = oracle.route(None, ws[0], b, k, logits=lo)
        assert np.array_equal(sel, given["selected"]), "selected experts differ from the oracle on the GPU's logits"
        assert np.array_equal(cnt, given["counts"].astype(np.int32)), "counts differ from the oracle"
        np.testing.assert_allclose(gat, given["gating"], rtol=2e-6, atol=1e-7)
        own = oracle.route(x, ws[0], b, k)
        assert np.abs(lo - own["logits"]).max() <= 1e-4


def test_route_static_rejects_sizes_beyond_its_scratch(capi):
    import torch
    L = capi.lib()
    one = torch.zeros(16, device="cuda")
    p = one.data_ptr()
    st = torch.cuda.current_stream().cuda_stream
    assert L.prichs_moe_route_static(p, p, None, 16385, 512, 8, 2, p, p, p, p, st) == capi.ERR_CAPACITY
    assert "exceed the static scratch limits" in capi.last_error()
    assert L.prichs_moe_route_static(p, p, None, 16, 4096, 8, 2, p, p, p, p, st) == capi.ERR_CAPACITY
    assert L.prichs_moe_route_static(p, p, None, 16, 300, 8, 2, p, p, p, p, st) == capi.ERR_BAD_SHAPE
    assert L.prichs_moe_route_static(p, p, None, 16, 512, 9, 2, p, p, p, p, st) == capi.ERR_BAD_SHAPE
    assert L.prichs_moe_route_static(None, p, None, 16, 512, 8, 2, p, p, p, p, st) == capi.ERR_BAD_ARG
