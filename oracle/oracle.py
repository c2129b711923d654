"""ctypes loader for the CPU oracle (oracle/moe_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline leg of the
benchmark; the shipped package never imports it. PARITY UNPINNED BY REFERENCE VECTORS (the reference holds
no golden vectors for this path and cannot be compiled without a Rust toolchain); see the header of
moe_oracle.cpp for what pins it instead.

The functions mirror the reference one to one:
  matmul_2d, swiglu, top_k_gating_unbiased, add_tensors      crates/prichs-core/src/ops.rs:8-61,142-159,219-248,250-267
  rms_norm                                                    crates/prichs-core/src/ops.rs:109-135
  moe_forward_train, update_aux_free_bias                     crates/prichs-model/src/moe.rs:93-211,228-245
  moe_backward, moe_router_unbiased_backward                  crates/prichs-model/src/model.rs:566-766,
                                                              crates/prichs-core/src/backward.rs:247-287
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmoe_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile; returns the path of the shared object."""
    src = os.path.join(_HERE, "moe_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-s", "-C", _HERE, "-B", "libmoe_oracle.so"], check=True)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        fp, zp, sz = C.POINTER(C.c_float), C.POINTER(C.c_size_t), C.c_size_t
        L.oracle_num_threads.restype = C.c_int
        L.oracle_set_num_threads.argtypes = [C.c_int]
        L.oracle_matmul_2d.argtypes = [fp, fp, fp, sz, sz, sz]
        L.oracle_swiglu.argtypes = [fp, fp, fp, sz]
        L.oracle_top_k_gating_unbiased.argtypes = [fp, fp, sz, sz, zp, fp]
        L.oracle_add_tensors.argtypes = [fp, fp, fp, sz]
        L.oracle_route.argtypes = [fp, fp, fp, fp, sz, sz, sz, sz, sz, fp, fp, zp, fp, zp]
        L.oracle_moe_forward_train.argtypes = [C.POINTER(fp), fp, sz, sz, sz, sz, fp, sz, fp, sz,
                                               C.POINTER(C.c_ubyte), fp, fp, zp, fp, zp, fp]
        L.oracle_moe_forward_train.restype = C.c_int
        L.oracle_update_aux_free_bias.argtypes = [fp, sz, sz, zp, sz, C.c_float]
        L.oracle_rms_norm.argtypes = [fp, fp, C.c_float, fp, sz, sz]
        L.oracle_moe_router_unbiased_backward.argtypes = [fp, fp, zp, sz, fp, sz]
        L.oracle_moe_backward.argtypes = [C.POINTER(fp), fp, sz, sz, sz, sz, fp, sz, fp, sz, fp, C.POINTER(fp), fp]
        L.oracle_moe_backward.restype = C.c_int
        L.oracle_rmsnorm_backward.argtypes = [fp, fp, fp, fp, fp, sz, sz, C.c_float]
        _lib = L
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(C.POINTER(C.c_float))


def _fnull():
    return C.POINTER(C.c_float)()


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(int(n))


def matmul_2d(a, b):
    a, pa = _f(a)
    b, pb = _f(b)
    m, k = a.shape
    k2, n = b.shape
    if k != k2:
        raise ValueError(f"Incompatible shapes for matmul: [{m}, {k}] x [{k2}, {n}]")
    out = np.empty((m, n), np.float32)
    lib().oracle_matmul_2d(pa, pb, out.ctypes.data_as(C.POINTER(C.c_float)), m, k, n)
    return out


def swiglu(gate, up):
    g, pg = _f(gate)
    u, pu = _f(up)
    if g.size != u.size:
        raise ValueError("Gate and Up tensors must have identical length")
    out = np.empty_like(g)
    lib().oracle_swiglu(pg, pu, out.ctypes.data_as(C.POINTER(C.c_float)), g.size)
    return out


def top_k_gating_unbiased(raw_logits, routing_logits, k):
    r, pr = _f(raw_logits)
    s, ps = _f(routing_logits)
    assert k <= r.size, "k must be <= logits length"
    assert r.size == s.size, "raw and routing logits must match"
    idx = np.empty(k, np.uintp)
    w = np.empty(k, np.float32)
    lib().oracle_top_k_gating_unbiased(pr, ps, r.size, k, idx.ctypes.data_as(C.POINTER(C.c_size_t)),
                                       w.ctypes.data_as(C.POINTER(C.c_float)))
    return idx.astype(np.int64), w


def add_tensors(a, b):
    a, pa = _f(a)
    b, pb = _f(b)
    if a.size != b.size:
        raise ValueError("Tensor length mismatch in addition")
    out = np.empty_like(a)
    lib().oracle_add_tensors(pa, pb, out.ctypes.data_as(C.POINTER(C.c_float)), a.size)
    return out


def rms_norm(x, weight, eps):
    """rms_norm of ops.rs:109-135 over the last dimension of a 2-D array."""
    x, px = _f(x)
    w, pw = _f(weight)
    if w.size != x.shape[-1]:
        raise ValueError(f"Weight length {w.size} != hidden_dim {x.shape[-1]}")
    out = np.empty_like(x)
    lib().oracle_rms_norm(px, pw, C.c_float(eps), out.ctypes.data_as(C.POINTER(C.c_float)), x.shape[0], x.shape[1])
    return out


def route(x, router, router_bias, top_k, concept_bias=None, logits=None):
    """Routing of moe.rs:114-142. With `logits` given, the x.W_r product is skipped and those fp32 logits
    are used. Returns dict(logits [T,E], selected [T,k] int64, gating [T,k], counts [E] int64)."""
    router, prt = _f(router)
    d, E = router.shape
    bias, pbias = _f(router_bias)
    if logits is not None:
        lg, plg = _f(logits)
        T = lg.shape[0]
        px = _fnull()
    else:
        x, px = _f(x)
        T = x.shape[0]
        plg = _fnull()
    if concept_bias is not None:
        cb, pcb = _f(concept_bias)
        ncb = cb.size
    else:
        pcb, ncb = _fnull(), 0
    lo = np.empty((T, E), np.float32)
    sel = np.empty((T, top_k), np.uintp)
    gat = np.empty((T, top_k), np.float32)
    cnt = np.empty(E, np.uintp)
    lib().oracle_route(px, prt, pbias, pcb, ncb, T, d, E, top_k, plg, lo.ctypes.data_as(C.POINTER(C.c_float)),
                       sel.ctypes.data_as(C.POINTER(C.c_size_t)), gat.ctypes.data_as(C.POINTER(C.c_float)),
                       cnt.ctypes.data_as(C.POINTER(C.c_size_t)))
    return dict(logits=lo, selected=sel.astype(np.int64), gating=gat, counts=cnt.astype(np.int64))


def moe_forward_train(weights, router_bias, top_k, x, concept_bias=None, token_mask=None):
    """MoELayer::forward_train. `weights` = [router, shared gate, up, down, e0 gate, up, down, ...] as f32
    arrays in the reference's x.W layout ([d,E], [d,f], [d,f], [f,d]). Returns dict(out, logits, selected,
    gating, counts, shared_out). With `token_mask` (bool [T]) only the masked rows of out/shared_out are
    computed (others are left zero); routing still covers every token."""
    ws = [np.ascontiguousarray(w, dtype=np.float32) for w in weights]
    d, E = ws[0].shape
    f = ws[1].shape[1]
    assert len(ws) == 1 + 3 * (1 + E)
    arr = (C.POINTER(C.c_float) * len(ws))(*[w.ctypes.data_as(C.POINTER(C.c_float)) for w in ws])
    bias, pbias = _f(router_bias)
    x, px = _f(x)
    T = x.shape[0]
    assert x.shape[1] == d
    if concept_bias is not None:
        cb, pcb = _f(concept_bias)
        ncb = cb.size
    else:
        pcb, ncb = _fnull(), 0
    if token_mask is not None:
        tm = np.ascontiguousarray(token_mask, dtype=np.uint8)
        ptm = tm.ctypes.data_as(C.POINTER(C.c_ubyte))
    else:
        ptm = C.POINTER(C.c_ubyte)()
    out = np.zeros((T, d), np.float32)
    sh = np.zeros((T, d), np.float32)
    lo = np.empty((T, E), np.float32)
    sel = np.empty((T, top_k), np.uintp)
    gat = np.empty((T, top_k), np.float32)
    cnt = np.empty(E, np.uintp)
    rc = lib().oracle_moe_forward_train(arr, pbias, d, f, E, top_k, px, T, pcb, ncb, ptm,
                                        out.ctypes.data_as(C.POINTER(C.c_float)),
                                        lo.ctypes.data_as(C.POINTER(C.c_float)),
                                        sel.ctypes.data_as(C.POINTER(C.c_size_t)),
                                        gat.ctypes.data_as(C.POINTER(C.c_float)),
                                        cnt.ctypes.data_as(C.POINTER(C.c_size_t)),
                                        sh.ctypes.data_as(C.POINTER(C.c_float)))
    if rc != 0:
        raise ValueError("k must be <= logits length")
    return dict(out=out, logits=lo, selected=sel.astype(np.int64), gating=gat, counts=cnt.astype(np.int64),
                shared_out=sh)


def update_aux_free_bias(router_bias, expert_token_counts, total_tokens, gamma, top_k):
    """MoELayer::update_aux_free_bias; returns the new bias (input left untouched)."""
    b = np.array(router_bias, dtype=np.float32, copy=True)
    c = np.ascontiguousarray(expert_token_counts, dtype=np.uintp)
    lib().oracle_update_aux_free_bias(b.ctypes.data_as(C.POINTER(C.c_float)), b.size, top_k,
                                      c.ctypes.data_as(C.POINTER(C.c_size_t)), int(total_tokens),
                                      C.c_float(gamma))
    return b


def moe_router_unbiased_backward(d_expert_weights, gating_weights, selected_indices, num_experts):
    """backward.rs:269-287: d logits [E] of one token from the k scalars <expert_i(x), d_out>."""
    dw, pdw = _f(d_expert_weights)
    gw, pgw = _f(gating_weights)
    idx = np.ascontiguousarray(selected_indices, dtype=np.uintp)
    out = np.empty(num_experts, np.float32)
    lib().oracle_moe_router_unbiased_backward(pdw, pgw, idx.ctypes.data_as(C.POINTER(C.c_size_t)), idx.size,
                                              out.ctypes.data_as(C.POINTER(C.c_float)), num_experts)
    return out


def moe_backward(weights, router_bias, top_k, x, d_out, concept_bias=None, grads=None):
    """MoE part of the block's backward pass (model.rs:566-766). Returns dict(d_x [T,d], grads = list of arrays in
    the order and shapes of `weights`). Gradients are accumulated into `grads` when given (the reference adds into
    its gradient buffers), else into zeros."""
    ws = [np.ascontiguousarray(w, dtype=np.float32) for w in weights]
    d, E = ws[0].shape
    f = ws[1].shape[1]
    assert len(ws) == 1 + 3 * (1 + E)
    fp = C.POINTER(C.c_float)
    arr = (fp * len(ws))(*[w.ctypes.data_as(fp) for w in ws])
    gs = [np.zeros_like(w) for w in ws] if grads is None else [np.ascontiguousarray(g, dtype=np.float32) for g in grads]
    assert all(g.shape == w.shape for g, w in zip(gs, ws))
    garr = (fp * len(gs))(*[g.ctypes.data_as(fp) for g in gs])
    bias, pbias = _f(router_bias)
    x, px = _f(x)
    dy, pdy = _f(d_out)
    T = x.shape[0]
    assert x.shape == (T, d) and dy.shape == (T, d)
    if concept_bias is not None:
        cb, pcb = _f(concept_bias)
        ncb = cb.size
    else:
        pcb, ncb = _fnull(), 0
    dx = np.empty((T, d), np.float32)
    rc = lib().oracle_moe_backward(arr, pbias, d, f, E, top_k, px, T, pcb, ncb, pdy, garr, dx.ctypes.data_as(fp))
    if rc != 0:
        raise ValueError("k must be <= logits length")
    return dict(d_x=dx, grads=gs)


def rmsnorm_backward(d_out, x, gamma, eps, d_x=None, d_gamma=None):
    """backward.rs:94-131. Returns (d_x, d_gamma); both ACCUMULATE into the arrays given (zeros otherwise): the
    reference seeds d_x with the gradient that flows through the residual connection (model.rs:777-789)."""
    dy, pdy = _f(d_out)
    x, px = _f(x)
    g, pg = _f(gamma)
    rows, d = x.shape
    assert dy.shape == x.shape and g.size == d
    dx = np.zeros((rows, d), np.float32) if d_x is None else np.array(d_x, dtype=np.float32, copy=True)
    dg = np.zeros(d, np.float32) if d_gamma is None else np.array(d_gamma, dtype=np.float32, copy=True)
    fp = C.POINTER(C.c_float)
    lib().oracle_rmsnorm_backward(pdy, px, pg, dx.ctypes.data_as(fp), dg.ctypes.data_as(fp), rows, d, C.c_float(eps))
    return dx, dg

