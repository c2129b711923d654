"""Helpers shared by the tests: an independent numpy restatement of the reference path (second opinion for
the C++ oracle), error metrics in the style of the reference's parity report
(crates/prichs-cli/src/bin/diagnostics_parity.rs:108-121), small-integer test tensors."""
import numpy as np


def np_silu(x):
    x = x.astype(np.float32)
    return x / (np.float32(1.0) + np.exp(-x, dtype=np.float32))


def np_top_k_unbiased(raw, routing, k):
    # stable descending order: ties keep the lower index (ops.rs:226-229)
    order = sorted(range(len(routing)), key=lambda i: -float(routing[i]))  # Python's sort is stable
    idx = order[:k]
    sel = np.array([raw[i] for i in idx], np.float32)
    m = sel.max()
    e = np.exp(sel - m, dtype=np.float32)
    s = np.float32(0)
    for v in e:
        s = np.float32(s + v)
    inv = np.float32(1.0) / np.float32(s + np.float32(1e-9))
    return np.array(idx), (e * inv).astype(np.float32)


def np_moe_forward(ws, bias, top_k, x, concept_bias=None):
    """float64-accumulated numpy version of moe.rs:93-211 (not bit-identical to the oracle's f32 loop order;
    agreement is checked to 1e-5 relative)."""
    router = ws[0]
    d, E = router.shape
    x = x.astype(np.float32)
    T = x.shape[0]

    def mlp(xx, wg, wu, wd):
        g = (xx.astype(np.float64) @ wg.astype(np.float64)).astype(np.float32)
        u = (xx.astype(np.float64) @ wu.astype(np.float64)).astype(np.float32)
        a = np_silu(g) * u
        return (a.astype(np.float64) @ wd.astype(np.float64)).astype(np.float32)

    out = mlp(x, ws[1], ws[2], ws[3]).astype(np.float64)
    logits = (x.astype(np.float64) @ router.astype(np.float64)).astype(np.float32)
    sel = np.zeros((T, top_k), np.int64)
    gat = np.zeros((T, top_k), np.float32)
    for t in range(T):
        s = logits[t] + bias.astype(np.float32)
        if concept_bias is not None:
            cb = np.asarray(concept_bias, np.float32)
            s[:min(E, cb.size)] += cb[:E]
        sel[t], gat[t] = np_top_k_unbiased(logits[t], s, top_k)
    counts = np.bincount(sel.reshape(-1), minlength=E)
    for e in range(E):
        tok, slot = np.nonzero(sel == e)
        if tok.size == 0:
            continue
        ye = mlp(x[tok], ws[4 + 3 * e], ws[5 + 3 * e], ws[6 + 3 * e])
        out[tok] += gat[tok, slot][:, None].astype(np.float64) * ye
    return dict(out=out.astype(np.float32), logits=logits, selected=sel, gating=gat, counts=counts)


def report(a, b):
    """max-abs, mean-abs, cosine and the worst |a-b| / (|b| + rms(b)) of `a` against the expectation `b`."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    diff = np.abs(a - b)
    rms = float(np.sqrt(np.mean(b * b))) if b.size else 0.0
    rel = diff / (np.abs(b) + rms + 1e-30)
    cos = float((a * b).sum() / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-30)) if b.size else 1.0
    return dict(max_abs=float(diff.max(initial=0.0)), mean_abs=float(diff.mean()) if b.size else 0.0, cos=cos,
                max_rel=float(rel.max(initial=0.0)), rms=rms)


def assert_close(a, b, tol, what=""):
    """|a - b| <= tol * (|b| + rms(b)) element-wise."""
    r = report(a, b)
    assert r["max_rel"] <= tol, f"{what}: {r}"
    return r


def grid_tensor(seed, tensor_id, shape, span, denom):
    """Values k/denom with integer |k| <= span from pure 64-bit integer hashing (no libm, identical on every
    machine); exactly representable in bf16 for the spans used here."""
    from prichs_b200.synth import _stream
    n = int(np.prod(shape))
    k = (_stream(seed, tensor_id, 0, n) >> np.uint64(33)) % np.uint64(2 * span + 1)
    return ((k.astype(np.int64) - span).astype(np.float32) / np.float32(denom)).reshape(shape)


def small_int_weights(seed, d, f, E):
    """Layer weights on the grid k/64, |k| <= 8, in the reference's parameter order."""
    ws = [grid_tensor(seed, 1, (d, E), 8, 64)]
    tid = 2
    for _ in range(1 + E):
        ws += [grid_tensor(seed, tid, (d, f), 8, 64), grid_tensor(seed, tid + 1, (d, f), 8, 64),
               grid_tensor(seed, tid + 2, (f, d), 8, 64)]
        tid += 3
    return ws


def golden_small_inputs():
    """Inputs of tests/golden/moe_small.npz (the fixture stores only the expected outputs)."""
    d, f, E, k, T = 256, 128, 8, 2, 48
    ws = small_int_weights(7, d, f, E)
    x = grid_tensor(11, 0, (T, d), 16, 8)
    bias = grid_tensor(11, 1000, (E,), 4, 32)
    cb = np.array([0.25, -0.125, 0.0], np.float32)
    return dict(ws=ws, x=x, bias=bias, concept_bias=cb, top_k=k)
