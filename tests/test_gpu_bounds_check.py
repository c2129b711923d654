"""The index-checking build (libprichs_moe_check.so, -DPRICHS_BOUNDS_CHECK) on the ragged and degenerate cases.

Every row index the routing-side kernels compute is compared with the extent of its buffer before the access; a
violation would be recorded in the status word and reported as PRICHS_ERR_BOUNDS by sync_status (which every case
below calls), never by a fault. The cases run in a child process whose Python binding loads the checking build."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import sys
import numpy as np, torch
sys.path.insert(0, %(root)r); sys.path.insert(0, %(root)r + "/tests")
from prichs_b200 import MoELayer, synth, _capi
from oracle import oracle as O
assert _capi.lib().prichs_bounds_checking() == 1, "not the checking build"
d, f, E, k = 256, 128, 8, 2
for route_kernel in (1, 2):
    for T in (1, 2, 15, 16, 17, 127, 128, 129, 1100):
        ws = synth.layer_weights(400 + T, d, f, E, std=0.05, bf16=True)
        x = synth.round_bf16(synth.normal(500 + T, 0, (T, d)))
        for bias in (synth.router_bias(T, E, -0.1, 0.1),
                     np.array([50, 40, 0, 0, 0, 0, 0, 0], np.float32)):   # second: every token picks experts 0 and 1
            m = MoELayer.from_weights(ws, k, route_kernel=route_kernel)
            m.router_bias = bias
            y = m.forward(torch.from_numpy(x).cuda().bfloat16()).float().cpu().numpy()
            m.sync_status()   # raises PrichsError(ERR_BOUNDS) if any index check failed
            st = m.last_stash()
            given = O.route(None, ws[0], bias, k, logits=st.router_logits)
            assert np.array_equal(st.selected_experts.reshape(T, k), given["selected"])
            assert np.array_equal(st.expert_token_counts, given["counts"])
            ref = O.moe_forward_train(ws, bias, k, x)
            same = np.all(ref["selected"] == given["selected"], axis=1)
            rms = float(np.sqrt(np.mean(ref["out"] ** 2)))
            assert (np.abs(y[same] - ref["out"][same]) / (np.abs(ref["out"][same]) + rms)).max() <= 2e-2
            m.close()
print("BOUNDS_OK")
"""


def test_ragged_cases_under_the_index_checking_build():
    from prichs_b200 import build
    lib = build.build(check=True)
    env = dict(os.environ, PRICHS_B200_LIB=lib)
    res = subprocess.run([sys.executable, "-c", CHILD % {"root": ROOT}], capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    sys.stdout.write(res.stdout[-2000:])
    sys.stderr.write(res.stderr[-4000:])
    assert res.returncode == 0 and "BOUNDS_OK" in res.stdout


@pytest.mark.parametrize("T,route_kernel", [(129, 2), (1100, 1), (5000, 1)])
def test_canaries_around_the_callers_buffers_stay_intact(T, route_kernel):
    """The caller's x, residual and y sit inside larger allocations whose guard zones carry a bit pattern: the forward
    must read nothing it depends on from them (the result is unchanged when the pattern changes) and write nothing
    into them (the pattern is intact afterwards). Product build."""
    import numpy as np
    import torch
    from prichs_b200 import MoELayer, synth
    d, f, E, k, G = 256, 128, 8, 2, 4096  # G guard elements on each side
    ws = synth.layer_weights(600 + T, d, f, E, std=0.05, bf16=True)
    x = synth.round_bf16(synth.normal(601 + T, 0, (T, d)))
    r = synth.round_bf16(synth.normal(602 + T, 0, (T, d)))
    m = MoELayer.from_weights(ws, k, route_kernel=route_kernel)
    outs = []
    for pattern in (0x7FC1, 0x4242):  # a NaN pattern, then an ordinary number
        bufs = []
        for src in (x, r, None):
            big = torch.full((T * d + 2 * G,), 0, dtype=torch.int16, device="cuda")
            big[:] = pattern if pattern < 0x8000 else pattern - 0x10000
            view = big[G:G + T * d].view(torch.bfloat16).view(T, d)
            if src is not None:
                view.copy_(torch.from_numpy(src).cuda().bfloat16())
            bufs.append((big, view))
        (bx, vx), (br, vr), (by, vy) = bufs
        m.forward_with_memory(vx, None, residual=vr, out=vy)
        m.sync_status()
        for big, _ in bufs:
            guard = torch.cat([big[:G], big[G + T * d:]]).cpu().numpy().astype(np.uint16)
            assert (guard == pattern).all(), "a guard zone was written"
        outs.append(vy.float().cpu().numpy())
    assert np.array_equal(outs[0], outs[1]), "the result depends on memory outside the caller's buffers"
    assert np.isfinite(outs[0]).all()
