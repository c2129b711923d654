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


def np_backward_decomposed(ws, x, R, sel, gates, counts, pad=256):
    """fp32 numpy model of the steps prichs_moe_backward performs, in its row space: shared rows [0,T), permuted row
    Tcap + pos with pos = expert * Tcap + rank in the expert's bin; [gate | up] in blocks of 256 columns (128 gate then 128 up of the same hidden units). Returns the
    intermediates (gu, hall, yall, dyall, scal, dh, dgu, dxall, dlog), the row map (Tcap, seg_base, pos, live rows) and
    the results (dx, grads in the order of `ws`)."""
    T, d = x.shape
    E = ws[0].shape[1]
    f = ws[1].shape[1]
    k = sel.shape[1]
    Tcap = (T + pad - 1) // pad * pad
    seg_base = np.arange(E, dtype=np.int64) * Tcap  # fixed-capacity segments (the handle is created for T tokens)
    Rtot = Tcap + E * Tcap
    pos = np.full((T, k), -1, np.int64)
    fill = np.zeros(E, np.int64)
    row_expert = np.full(Rtot, -1, np.int64)
    for t in range(T):
        for j in range(k):
            e = sel[t, j]
            pos[t, j] = seg_base[e] + fill[e]
            row_expert[Tcap + pos[t, j]] = e
            fill[e] += 1
    row_expert[:T] = -2  # shared expert

    def blocked(wg, wu):
        out = np.zeros((d, 2 * f), np.float32)
        for b in range(f // 128):
            out[:, 256 * b:256 * b + 128] = wg[:, 128 * b:128 * b + 128]
            out[:, 256 * b + 128:256 * b + 256] = wu[:, 128 * b:128 * b + 128]
        return out

    wgu = [blocked(ws[1 + 3 * s], ws[2 + 3 * s]) for s in range(1 + E)]  # slot 0 = shared
    wdn = [ws[3 + 3 * s] for s in range(1 + E)]
    slot_of_row = np.where(row_expert == -2, 0, row_expert + 1)
    silu = lambda g: g / (1.0 + np.exp(-g))

    xall = np.zeros((Rtot, d), np.float32)
    xall[:T] = x
    for t in range(T):
        for j in range(k):
            xall[Tcap + pos[t, j]] = x[t]
    live = np.where(row_expert != -1)[0]
    gu = np.zeros((Rtot, 2 * f), np.float32)
    hall = np.zeros((Rtot, f), np.float32)
    yall = np.zeros((Rtot, d), np.float32)
    for r in live:
        s = slot_of_row[r]
        gu[r] = xall[r] @ wgu[s]
        gb = gu[r].reshape(-1, 256)
        hall[r] = (silu(gb[:, :128]) * gb[:, 128:]).reshape(-1)
        yall[r] = hall[r] @ wdn[s]
    # 1. d_out into the row space + the router's scalars
    dyall = np.zeros((Rtot, d), np.float32)
    dyall[:T] = R
    scal = np.zeros((T, k), np.float32)
    for t in range(T):
        for j in range(k):
            r = Tcap + pos[t, j]
            dyall[r] = gates[t, j] * R[t]
            scal[t, j] = yall[r] @ R[t]
    # 3. d_act, 4. SwiGLU backward in the blocked order, 5. dX over K = 2f
    dh = np.zeros((Rtot, f), np.float32)
    dgu = np.zeros_like(gu)
    dxall = np.zeros((Rtot, d), np.float32)
    for r in live:
        s = slot_of_row[r]
        dh[r] = dyall[r] @ wdn[s].T
        gb = gu[r].reshape(-1, 256)
        g, u = gb[:, :128], gb[:, 128:]
        dhb = dh[r].reshape(-1, 128)
        sig = 1.0 / (1.0 + np.exp(-g))
        dgu[r] = np.concatenate([dhb * u * (sig * (1.0 + g * (1.0 - sig))), dhb * (g * sig)], axis=1).reshape(-1)
        dxall[r] = dgu[r] @ wgu[s].T
    # 6. router VJP, 7. d_x: shared + experts ascending (gate weight once more, as the reference) + router
    dlog = np.zeros((T, E), np.float32)
    for t in range(T):
        weighted = float((gates[t] * scal[t]).sum())
        for j in range(k):
            dlog[t, sel[t, j]] = gates[t, j] * (scal[t, j] - weighted)
    dx = dxall[:T].copy()
    for t in range(T):
        for j in np.argsort(sel[t]):
            dx[t] += gates[t, j] * dxall[Tcap + pos[t, j]]
    dx += dlog @ ws[0].T
    # 8./10. weight gradients: router, then per slot a K window of the transposed copies
    grads = [np.zeros_like(w) for w in ws]
    grads[0] = x.T @ dlog
    xT, hT, dyT, dguT = xall.T, hall.T, dyall.T, dgu.T
    for s in range(1 + E):
        k0, n = (0, T) if s == 0 else (Tcap + int(seg_base[s - 1]), int(counts[s - 1]))
        if n == 0:
            continue
        grads[3 + 3 * s] = hT[:, k0:k0 + n] @ dyT[:, k0:k0 + n].T
        sb = (xT[:, k0:k0 + n] @ dguT[:, k0:k0 + n].T).reshape(d, -1, 256)  # [d, 2f], blocked columns
        grads[1 + 3 * s] = sb[:, :, :128].reshape(d, f)
        grads[2 + 3 * s] = sb[:, :, 128:].reshape(d, f)
    return dict(Tcap=Tcap, seg_base=seg_base, pos=pos, live=live, gu=gu, hall=hall, yall=yall, dyall=dyall, scal=scal, dh=dh,
                dgu=dgu, dxall=dxall, dlog=dlog, dx=dx, grads=grads)
