"""CPU-side checks of the C-ABI library: it builds for sm_100a, loads, exports every symbol the header
declares, and refuses to run without a device (there is no CPU fallback)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "prichs_moe.h")).read()
    return sorted(set(re.findall(r"PRICHS_API\s+[\w\s\*]+?\b(prichs_\w+|launch_\w+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(capi):
    names = _declared_symbols()
    assert len(names) >= 20
    L = C.CDLL(capi.LIB_PATH)
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/prichs_moe.h but not exported"
    # the Python binding covers exactly the header
    assert sorted(capi.SYMBOLS) == names


def test_last_error_and_launch_counter(capi):
    L = capi.lib()
    assert isinstance(capi.last_error(), str)
    assert L.prichs_kernel_launches() >= 0


def test_bad_arguments_are_rejected_before_touching_a_device(capi):
    L = capi.lib()
    h = C.c_void_p()
    for bad in (dict(hidden_dim=100), dict(intermediate_dim=100), dict(num_experts=9), dict(top_k=3),
                dict(num_experts=1, top_k=2), dict(max_tokens=0), dict(mode=7), dict(ep_world=3)):
        base = dict(hidden_dim=256, intermediate_dim=128, num_experts=8, top_k=2, max_tokens=64, mode=0, device=-1,
                    ep_world=1, ep_rank=0, ep_max_recv_rows=0, ep_waves=0)
        base.update(bad)
        cfg = capi.Config(**base)
        rc = L.prichs_moe_create(C.byref(cfg), C.byref(h))
        assert rc in (capi.ERR_BAD_SHAPE, capi.ERR_BAD_ARG), (bad, rc, capi.last_error())
        assert not h.value
    assert L.prichs_moe_create(None, C.byref(h)) == capi.ERR_BAD_ARG
    assert L.prichs_moe_destroy(None) == capi.OK


def test_no_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the no-device behaviour is checked on CPU-only machines")
    from prichs_b200 import MoELayer, PrichsError
    m = MoELayer(256, 128, 8, 2, seed=0)
    with pytest.raises(PrichsError) as ei:
        m.forward(np.zeros((4, 256), np.float32))
    assert ei.value.code == -3


def test_python_layer_mirrors_reference_fields():
    from prichs_b200 import MoELayer
    m = MoELayer(256, 128, 8, 2, seed=0)
    assert m.router.shape == (256, 8) and m.router_bias.shape == (8,) and np.all(m.router_bias == 0)
    assert len(m.experts) == 8 and m.top_k == 2
    assert m.shared_expert.gate_proj.shape == (256, 128) and m.shared_expert.down_proj.shape == (128, 256)
    # MoELayer::new / Expert::new initialisation scale (moe.rs:13,73): std = sqrt(2 / (fan_in + fan_out))
    assert abs(m.experts[0].gate_proj.std() - (2 / (256 + 128)) ** 0.5) < 0.01
    assert len(m.parameter_list()) == 1 + 3 * 9
    for name in ("forward", "forward_with_memory", "forward_train", "update_aux_free_bias"):
        assert callable(getattr(m, name))
