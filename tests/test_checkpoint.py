"""PRICHS02 checkpoint reader (prichs_b200/checkpoint.py) against a file written in the reference's format
(crates/prichs-model/src/model.rs:1648-1670) with the reference's parameter order (model.rs:341-364)."""
import os
import struct

import numpy as np
import pytest


def _fake_model_tensors(rng, vocab, d, f, E, n_layers, heads_dim=32):
    """All parameter tensors of a small model in get_parameter_tensors order; returns (flat list, moe tensors per layer)."""
    ts = [rng.standard_normal(vocab * d).astype(np.float32), np.ones(d, np.float32)]
    moe = []
    for _ in range(n_layers):
        blk = [np.ones(d, np.float32)] + [rng.standard_normal(d * heads_dim).astype(np.float32) for _ in range(4)]
        norm = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
        router = (rng.standard_normal((d, E)) * 0.1).astype(np.float32)
        experts = []
        for _ in range(1 + E):
            experts += [(rng.standard_normal((d, f)) * 0.05).astype(np.float32), (rng.standard_normal((d, f)) * 0.05).astype(np.float32),
                        (rng.standard_normal((f, d)) * 0.05).astype(np.float32)]
        ts += blk + [norm, router] + experts
        moe.append((norm, [router] + experts))
    return ts, moe


def test_reader_follows_reference_format_and_order(tmp_path):
    from prichs_b200 import checkpoint as ck, PrichsError
    rng = np.random.default_rng(0)
    d, f, E, n_layers = 256, 128, 8, 3
    ts, moe = _fake_model_tensors(rng, 50, d, f, E, n_layers)
    path = str(tmp_path / "model.prichs")
    ck.write_tensors(path, 1234, 2.5, ts)
    # byte-level layout of the header, as the reference writes it
    raw = open(path, "rb").read(36)
    assert raw[:8] == b"PRICHS02" and struct.unpack("<Q", raw[8:16])[0] == 1234
    assert struct.unpack("<f", raw[16:20])[0] == 2.5 and struct.unpack("<Q", raw[20:28])[0] == len(ts)
    assert struct.unpack("<Q", raw[28:36])[0] == ts[0].size
    step, loss, flat = ck.read_tensors(path)
    assert (step, loss, len(flat)) == (1234, 2.5, 2 + n_layers * (10 + 3 * E))
    assert all(np.array_equal(a, b.reshape(-1)) for a, b in zip(flat, ts))
    # base = 2 + l * (10 + 3 E); router at base + 6, shared at base + 7..9, expert e at base + 10 + 3 e
    ix = ck.moe_tensor_indices(1, E)
    assert ix["router"] == 2 + 34 + 6 and ix["shared"] == (43, 44, 45) and ix["experts"][2] == (52, 53, 54)
    ck.save_router_bias(path, np.arange(n_layers * E, dtype=np.float32).reshape(n_layers, E) / 100)
    layers, norms, step, loss = ck.load_moe_layers(path, d, f, E, 2)
    assert len(layers) == n_layers and step == 1234
    for l, (m, norm) in enumerate(zip(layers, norms)):
        exp_norm, exp_ws = moe[l]
        assert np.array_equal(norm, exp_norm)
        for a, b in zip(m.parameter_list(), exp_ws):
            assert np.array_equal(a, b)
        assert np.allclose(m.router_bias, np.arange(E) / 100 + l * E / 100)
    # errors in the reference's words
    with pytest.raises(PrichsError, match="parameter count"):
        ck.load_moe_layers(path, d, f, 4, 2)
    with pytest.raises(PrichsError, match="expects"):
        ck.load_moe_layers(path, d, 2 * f, E, 2)
    bad = str(tmp_path / "bad.prichs")
    open(bad, "wb").write(b"PRICHS_X" + bytes(40))
    with pytest.raises(PrichsError, match="Invalid checkpoint magic"):
        ck.read_tensors(bad)
    open(bad, "wb").write(open(path, "rb").read()[:5000])
    with pytest.raises(PrichsError, match="truncated"):
        ck.read_tensors(bad)


@pytest.mark.gpu
def test_loaded_layers_run_the_block_sublayer(tmp_path, oracle):
    """Weights loaded from a checkpoint drive the block's MoE sub-layer on the GPU; parity against the oracle."""
    import torch
    from prichs_b200 import checkpoint as ck, synth
    from _util import assert_close
    rng = np.random.default_rng(1)
    d, f, E, k, T, n_layers = 256, 128, 8, 2, 150, 2
    ts, moe = _fake_model_tensors(rng, 20, d, f, E, n_layers)
    ts = [synth.round_bf16(t) for t in ts]
    path = str(tmp_path / "model.prichs")
    ck.write_tensors(path, 7, 0.0, ts)
    layers, norms, _, _ = ck.load_moe_layers(path, d, f, E, k)
    x = synth.round_bf16(synth.normal(5, 0, (T, d), 0.0, 2.0))
    xd = torch.from_numpy(synth.to_bf16_bits(x).view(np.int16)).view(torch.bfloat16).cuda()
    for m, norm in zip(layers, norms):
        y = m.block_forward(xd, torch.from_numpy(norm), 1e-5).float().cpu().numpy()
        m.sync_status()
        ws = m.parameter_list()
        xn = synth.round_bf16(oracle.rms_norm(x, norm, 1e-5))
        ref = oracle.moe_forward_train(ws, np.zeros(E, np.float32), k, xn)
        sel = m.last_stash().selected_experts.reshape(T, k)
        agree = np.all(ref["selected"] == sel, axis=1)
        assert (~agree).sum() <= 3
        assert_close(y[agree], (x + ref["out"])[agree], 2e-2, "block output from checkpoint weights")
        x = synth.round_bf16(y)  # feed the next block, as the model would
        xd = torch.from_numpy(synth.to_bf16_bits(x).view(np.int16)).view(torch.bfloat16).cuda()
