"""Host-side mirror of the reference's MoE layer API over the C-ABI library.

Same names, argument order and meaning as crates/prichs-model/src/moe.rs:
    Expert(hidden_dim, intermediate_dim)                 moe.rs:6-29   fields gate_proj, up_proj, down_proj
    MoELayer(hidden_dim, intermediate_dim, num_experts, top_k)         moe.rs:58-90
        .router [d,E], .router_bias [E], .shared_expert, .experts, .top_k   (public fields, moe.rs:59-63)
        .forward(x)                                      moe.rs:223-225
        .forward_with_memory(x, starkdb_concept_bias)    moe.rs:214-221
        .forward_train(x, starkdb_concept_bias) -> (out, MoEStash)    moe.rs:93-211
        .update_aux_free_bias(expert_token_counts, total_tokens, gamma)   moe.rs:228-245
`x` is a 2-D [T, d] array: a numpy float32 array (host buffers, like the reference's Tensor) or a CUDA torch
tensor (float32 or bfloat16; the result then stays on the device). Errors: shape mismatches raise
PrichsError like the reference's `bail!` (ops.rs:11-18); `top_k > num_experts` raises like its assert.

All arithmetic runs in libprichs_moe.so on the GPU. Nothing here computes the layer on the CPU.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

from . import _capi


class PrichsError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"[{code}] {msg}")
        self.code = code


def _check(rc: int):
    if rc != _capi.OK:
        raise PrichsError(rc, _capi.last_error())


def _randn(rng, shape, std):
    # Tensor::randn (crates/prichs-core/src/tensor.rs:49-63): N(0, std); the reference draws from an unseeded
    # thread_rng, here the generator is the caller's.
    return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)


class Expert:
    """SwiGLU expert weights in the reference's x.W layout (moe.rs:6-20)."""

    def __init__(self, hidden_dim: int, intermediate_dim: int, rng=None):
        rng = rng or np.random.default_rng()
        std = (2.0 / (hidden_dim + intermediate_dim)) ** 0.5
        self.gate_proj = _randn(rng, (hidden_dim, intermediate_dim), std)
        self.up_proj = _randn(rng, (hidden_dim, intermediate_dim), std)
        self.down_proj = _randn(rng, (intermediate_dim, hidden_dim), std)


@dataclass
class ExpertForwardStash:
    """One routed expert's part of the stash (moe.rs:32-42), host fp32 arrays in the reference's shapes."""
    expert_idx: int
    token_indices: np.ndarray  # [n] ascending
    weights: np.ndarray        # [n] gate weights
    x: np.ndarray              # [n, d]
    gate: np.ndarray           # [n, f]
    up: np.ndarray             # [n, f]
    act: np.ndarray            # [n, f]
    out: np.ndarray            # [n, d]


@dataclass
class MoEStash:
    """The reference's MoEStash (moe.rs:44-53). The routing fields are always filled. The activation fields
    (shared_gate / shared_up / shared_act / shared_out, routed_stashes) stay on the device after `forward_train` and
    are downloaded when first read; they are valid until the next forward on the layer."""
    router_logits: np.ndarray          # [T, E] fp32
    selected_experts: np.ndarray       # [T*k] int64, slot order = descending selection logit
    gating_weights: np.ndarray         # [T*k] fp32
    expert_token_counts: np.ndarray = field(default_factory=lambda: np.zeros(0, np.int64))  # [E]
    _layer: object = field(default=None, repr=False, compare=False)

    def _shared(self, which):
        if self._layer is None:
            raise PrichsError(_capi.ERR_BAD_ARG, "this stash carries no activations: use forward_train on device tensors")
        return self._layer.stash_field(0, which)

    shared_gate = property(lambda self: self._shared(1))
    shared_up = property(lambda self: self._shared(2))
    shared_act = property(lambda self: self._shared(3))
    shared_out = property(lambda self: self._shared(4))

    @property
    def routed_stashes(self) -> List[ExpertForwardStash]:
        """Experts that received tokens, ascending (the reference skips empty experts, moe.rs:151-153)."""
        if self._layer is None:
            raise PrichsError(_capi.ERR_BAD_ARG, "this stash carries no activations: use forward_train on device tensors")
        out = []
        for e in range(len(self.expert_token_counts)):
            if self.expert_token_counts[e] == 0:
                continue
            idx, w = self._layer.expert_assignments(e)
            out.append(ExpertForwardStash(e, idx, w, *[self._layer.stash_field(1 + e, i) for i in range(5)]))
        return out


class MoELayer:
    def __init__(self, hidden_dim: int, intermediate_dim: int, num_experts: int, top_k: int, *, seed=None,
                 mode: str = "bf16", max_tokens: int = 0, device: int = -1, ep_world: int = 1, ep_rank: int = 0,
                 ep_max_recv_rows: int = 0, ep_waves: int = 0, init: bool = True, **tuning):
        rng = np.random.default_rng(seed)
        self.hidden_dim, self.intermediate_dim = int(hidden_dim), int(intermediate_dim)
        self.top_k = int(top_k)
        self._num_experts = int(num_experts)
        if init:
            std = (2.0 / (hidden_dim + num_experts)) ** 0.5
            self.router = _randn(rng, (hidden_dim, num_experts), std)
            self.shared_expert = Expert(hidden_dim, intermediate_dim, rng)
            self.experts: List[Expert] = [Expert(hidden_dim, intermediate_dim, rng) for _ in range(num_experts)]
        else:
            self.router = None
            self.shared_expert = None
            self.experts = []
        self._bias_host = np.zeros(num_experts, np.float32)
        self.mode = {"bf16": _capi.MODE_BF16, "f32": _capi.MODE_F32}[mode]
        self._device, self._ep_world, self._ep_rank, self._ep_max_recv = device, ep_world, ep_rank, ep_max_recv_rows
        self._ep_waves = int(ep_waves)
        # tuning fields of prichs_moe_config_t (route_kernel, gemm_kernel, pdl, ...); absent = 0 = the default
        unknown = set(tuning) - set(_capi.TUNING_FIELDS)
        if unknown:
            raise TypeError(f"unknown MoELayer option(s): {sorted(unknown)}")
        self._tuning = {k: int(v) for k, v in tuning.items()}
        self._h = C.c_void_p()
        self._max_tokens = 0
        self._want_max_tokens = int(max_tokens)
        self._weights_dirty = True
        self._T_last = 0

    # ---- construction helpers -------------------------------------------------------------------
    @classmethod
    def from_weights(cls, weights: Sequence[np.ndarray], top_k: int, **kw) -> "MoELayer":
        """Build from the flat list [router, shared g/u/d, e0 g/u/d, ...] (model.rs:353-361 order)."""
        d, E = weights[0].shape
        f = weights[1].shape[1]
        if len(weights) != 1 + 3 * (1 + E):
            raise PrichsError(_capi.ERR_BAD_SHAPE, f"expected {1 + 3 * (1 + E)} weight arrays, got {len(weights)}")
        self = cls(d, f, E, top_k, init=False, **kw)
        self.router = np.ascontiguousarray(weights[0], np.float32)

        def mk(i):
            e = Expert.__new__(Expert)
            e.gate_proj, e.up_proj, e.down_proj = (np.ascontiguousarray(w, np.float32) for w in weights[i:i + 3])
            return e
        self.shared_expert = mk(1)
        self.experts = [mk(4 + 3 * i) for i in range(E)]
        return self

    def parameter_list(self) -> List[np.ndarray]:
        out = [self.router, self.shared_expert.gate_proj, self.shared_expert.up_proj, self.shared_expert.down_proj]
        for e in self.experts:
            out += [e.gate_proj, e.up_proj, e.down_proj]
        return out

    # ---- router_bias: public field of the reference, kept on the device between calls -------------
    @property
    def router_bias(self) -> np.ndarray:
        if self._h:
            b = np.empty(self._num_experts, np.float32)
            _check(_capi.lib().prichs_moe_get_bias(self._h, b.ctypes.data_as(C.POINTER(C.c_float)), b.size))
            self._bias_host = b
        return self._bias_host.copy()

    @router_bias.setter
    def router_bias(self, value):
        b = np.ascontiguousarray(value, np.float32).reshape(-1)
        if b.size != self._num_experts:
            raise PrichsError(_capi.ERR_BAD_SHAPE, f"router_bias has {b.size} entries, the layer has {self._num_experts} experts")
        self._bias_host = b.copy()
        if self._h:
            _check(_capi.lib().prichs_moe_set_bias(self._h, b.ctypes.data_as(C.POINTER(C.c_float)), b.size))

    # ---- device handle ----------------------------------------------------------------------------
    def mark_weights_changed(self):
        """Call after editing the public weight fields so the next forward uploads them again."""
        self._weights_dirty = True

    def _ensure(self, T: int):
        L = _capi.lib()
        if self._h and T > self._max_tokens and self._ep_world > 1:
            raise PrichsError(_capi.ERR_CAPACITY, "an expert-parallel layer cannot grow past the max_tokens it was connected with")
        if not self._h or T > self._max_tokens:
            bias = self.router_bias if self._h else self._bias_host
            self.close()
            cap = max(T, self._want_max_tokens, 1)
            cfg = _capi.Config(self.hidden_dim, self.intermediate_dim, self._num_experts, self.top_k, cap, self.mode,
                               self._device, self._ep_world, self._ep_rank, self._ep_max_recv, self._ep_waves)
            for name, value in self._tuning.items():
                setattr(cfg, name, value)
            h = C.c_void_p()
            _check(L.prichs_moe_create(C.byref(cfg), C.byref(h)))
            self._h, self._max_tokens, self._weights_dirty = h, cap, True
            _check(L.prichs_moe_set_bias(self._h, bias.ctypes.data_as(C.POINTER(C.c_float)), bias.size))
        if self._weights_dirty:
            ws = [None if w is None else np.ascontiguousarray(w, np.float32) for w in self.parameter_list()]
            shapes = [(self.hidden_dim, self._num_experts)] + [(self.hidden_dim, self.intermediate_dim)] * 2 + \
                     [(self.intermediate_dim, self.hidden_dim)]
            for i, w in enumerate(ws):
                want = shapes[0] if i == 0 else shapes[1 + (i - 1) % 3]
                if w is not None and w.shape != want:
                    raise PrichsError(_capi.ERR_BAD_SHAPE, f"weight {i} has shape {w.shape}, expected {want}")
            fp = C.POINTER(C.c_float)
            arr = (fp * len(ws))(*[fp() if w is None else w.ctypes.data_as(fp) for w in ws])
            _check(L.prichs_moe_upload_weights(self._h, arr, len(ws)))
            self._weights_dirty = False

    def close(self):
        if self._h:
            _capi.lib().prichs_moe_destroy(self._h)
            self._h = C.c_void_p()
            self._max_tokens = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- forward ----------------------------------------------------------------------------------
    @staticmethod
    def _cb(concept_bias):
        if concept_bias is None:
            return None, 0, None
        cb = np.ascontiguousarray(concept_bias, np.float32).reshape(-1)
        return cb.ctypes.data_as(C.POINTER(C.c_float)), cb.size, cb  # cb kept alive by the caller's tuple

    def forward_with_memory(self, x, starkdb_concept_bias: Optional[Sequence[float]] = None, residual=None, out=None,
                            stream=None, _train=False):
        """y = MoE(x) (+ residual when given: the caller's add of block.rs:67, fused)."""
        cbt = self._cb(starkdb_concept_bias)
        cb_ptr, cb_n = cbt[0], cbt[1]
        L = _capi.lib()
        if isinstance(x, np.ndarray):
            if x.ndim != 2 or x.shape[1] != self.hidden_dim:
                raise PrichsError(_capi.ERR_BAD_SHAPE, f"Incompatible shapes for matmul: {list(x.shape)} x [{self.hidden_dim}, ...]")
            xh = np.ascontiguousarray(x, np.float32)
            T = xh.shape[0]
            self._ensure(T)
            y = out if out is not None else np.empty((T, self.hidden_dim), np.float32)
            rp = None
            if residual is not None:
                rh = np.ascontiguousarray(residual, np.float32)
                if rh.shape != xh.shape:
                    raise PrichsError(_capi.ERR_BAD_SHAPE, "Tensor length mismatch in addition")
                rp = rh.ctypes.data
            _check(L.prichs_moe_forward_host(self._h, xh.ctypes.data, rp, cb_ptr, cb_n, y.ctypes.data, T))
            self._T_last = T
            return y
        import torch  # device path: torch is only the owner of the caller's device memory and stream
        if not (isinstance(x, torch.Tensor) and x.is_cuda):
            raise PrichsError(_capi.ERR_BAD_ARG, "x must be a numpy float32 array or a CUDA torch tensor")
        if x.dim() != 2 or x.shape[1] != self.hidden_dim:
            raise PrichsError(_capi.ERR_BAD_SHAPE, f"Incompatible shapes for matmul: {list(x.shape)} x [{self.hidden_dim}, ...]")
        dt = {torch.float32: _capi.DTYPE_F32, torch.bfloat16: _capi.DTYPE_BF16}.get(x.dtype)
        if dt is None:
            raise PrichsError(_capi.ERR_BAD_ARG, "x must be float32 or bfloat16")
        x = x.contiguous()
        T = x.shape[0]
        if self._device < 0:
            self._device = x.device.index
        self._ensure(T)
        y = out if out is not None else torch.empty_like(x)
        ydt = {torch.float32: _capi.DTYPE_F32, torch.bfloat16: _capi.DTYPE_BF16}[y.dtype]
        rp = None
        if residual is not None:
            if residual.shape != x.shape or residual.dtype != x.dtype:
                raise PrichsError(_capi.ERR_BAD_SHAPE, "Tensor length mismatch in addition")
            residual = residual.contiguous()
            rp = residual.data_ptr()
        st = stream if stream is not None else torch.cuda.current_stream(x.device).cuda_stream
        fwd = L.prichs_moe_forward_train if _train else L.prichs_moe_forward
        _check(fwd(self._h, x.data_ptr(), dt, rp, cb_ptr, cb_n, y.data_ptr(), ydt, T, st))
        self._T_last = T
        return y

    def forward(self, x, **kw):
        return self.forward_with_memory(x, None, **kw)

    def block_forward(self, x_residual, post_attn_norm, eps: float, starkdb_concept_bias=None, out=None, stream=None):
        """The MoE sub-layer of PrichsBlock::forward_with_rope (crates/prichs-model/src/block.rs:64-67) in one call:
        x_residual + MoE(rms_norm(x_residual, post_attn_norm, eps)). CUDA torch tensors; `post_attn_norm` is [d] fp32."""
        import torch
        x = x_residual
        if not (isinstance(x, torch.Tensor) and x.is_cuda) or x.dim() != 2 or x.shape[1] != self.hidden_dim:
            raise PrichsError(_capi.ERR_BAD_SHAPE, "x_residual must be a CUDA tensor of shape [T, hidden_dim]")
        if post_attn_norm.numel() != self.hidden_dim:
            raise PrichsError(_capi.ERR_BAD_SHAPE, f"Weight length {post_attn_norm.numel()} != hidden_dim {self.hidden_dim}")
        dt = {torch.float32: _capi.DTYPE_F32, torch.bfloat16: _capi.DTYPE_BF16}[x.dtype]
        x = x.contiguous()
        w = post_attn_norm.to(device=x.device, dtype=torch.float32).contiguous()
        T = x.shape[0]
        if self._device < 0:
            self._device = x.device.index
        self._ensure(T)
        y = out if out is not None else torch.empty_like(x)
        ydt = {torch.float32: _capi.DTYPE_F32, torch.bfloat16: _capi.DTYPE_BF16}[y.dtype]
        cb_ptr, cb_n, _keep = self._cb(starkdb_concept_bias)
        st = stream if stream is not None else torch.cuda.current_stream(x.device).cuda_stream
        _check(_capi.lib().prichs_moe_block_forward(self._h, x.data_ptr(), dt, w.data_ptr(), C.c_float(eps), cb_ptr, cb_n,
                                                    y.data_ptr(), ydt, T, st))
        self._T_last = T
        return y

    def backward(self, x, d_out, grads=None, stream=None):
        """MoE section of the reference's block backward pass (crates/prichs-model/src/model.rs:566-766) for the last
        forward of this layer. `x` is that forward's input and `d_out` the gradient of its output, CUDA torch tensors
        [T, hidden_dim] (fp32 or bf16). Returns d_x [T, hidden_dim] fp32. `grads`: list of 1 + 3 * (1 + E) CUDA fp32
        tensors (or None entries) in the order and layouts of the weights; the gradients are added to them."""
        import torch
        if not (isinstance(x, torch.Tensor) and x.is_cuda and isinstance(d_out, torch.Tensor) and d_out.is_cuda):
            raise PrichsError(_capi.ERR_BAD_ARG, "x and d_out must be CUDA tensors")
        if x.dim() != 2 or x.shape[1] != self.hidden_dim or tuple(d_out.shape) != tuple(x.shape):
            raise PrichsError(_capi.ERR_BAD_SHAPE, "x and d_out must both be [T, hidden_dim]")
        if not self._h or x.shape[0] != self._T_last:
            raise PrichsError(_capi.ERR_BAD_ARG, "backward needs the forward of the same batch to have run last")
        dts = {torch.float32: _capi.DTYPE_F32, torch.bfloat16: _capi.DTYPE_BF16}
        x, d_out = x.contiguous(), d_out.contiguous()
        dx = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        n = 1 + 3 * (1 + self._num_experts)
        if grads is not None:
            if len(grads) != n:
                raise PrichsError(_capi.ERR_BAD_SHAPE, f"expected {n} gradient buffers, got {len(grads)}")
            for g in grads:
                if g is not None and not (g.is_cuda and g.dtype == torch.float32 and g.is_contiguous()):
                    raise PrichsError(_capi.ERR_BAD_ARG, "gradient buffers must be contiguous CUDA fp32 tensors")
            arr = (C.c_void_p * n)(*[C.c_void_p(g.data_ptr()) if g is not None else C.c_void_p(0) for g in grads])
        else:
            arr = None
        st = stream if stream is not None else torch.cuda.current_stream(x.device).cuda_stream
        _check(_capi.lib().prichs_moe_backward(self._h, x.data_ptr(), dts[x.dtype], d_out.data_ptr(), dts[d_out.dtype], dx.data_ptr(),
                                               arr, n if grads is not None else 0, st))
        return dx

    def block_backward(self, x_residual, post_attn_norm, eps: float, d_out, grads=None, d_norm=None, stream=None):
        """Backward of the last `block_forward` (crates/prichs-model/src/model.rs:566-789): MoE backward on the
        normalised rows, then rmsnorm_backward with the residual gradient seeded in. Returns d_x_residual [T, d] fp32.
        `grads` as in `backward`; `d_norm` ([d] fp32 CUDA tensor or None) accumulates the norm weight's gradient."""
        import torch
        x = x_residual
        if not (isinstance(x, torch.Tensor) and x.is_cuda and isinstance(d_out, torch.Tensor) and d_out.is_cuda):
            raise PrichsError(_capi.ERR_BAD_ARG, "x_residual and d_out must be CUDA tensors")
        if x.dim() != 2 or x.shape[1] != self.hidden_dim or tuple(d_out.shape) != tuple(x.shape):
            raise PrichsError(_capi.ERR_BAD_SHAPE, "x_residual and d_out must both be [T, hidden_dim]")
        if not self._h or x.shape[0] != self._T_last:
            raise PrichsError(_capi.ERR_BAD_ARG, "block_backward needs block_forward of the same batch to have run last")
        dts = {torch.float32: _capi.DTYPE_F32, torch.bfloat16: _capi.DTYPE_BF16}
        x, d_out = x.contiguous(), d_out.contiguous()
        w = post_attn_norm.to(device=x.device, dtype=torch.float32).contiguous()
        dx = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        n = 1 + 3 * (1 + self._num_experts)
        arr = None
        if grads is not None:
            if len(grads) != n:
                raise PrichsError(_capi.ERR_BAD_SHAPE, f"expected {n} gradient buffers, got {len(grads)}")
            arr = (C.c_void_p * n)(*[C.c_void_p(g.data_ptr()) if g is not None else C.c_void_p(0) for g in grads])
        if d_norm is not None and not (d_norm.is_cuda and d_norm.dtype == torch.float32 and d_norm.numel() == self.hidden_dim):
            raise PrichsError(_capi.ERR_BAD_ARG, "d_norm must be a CUDA fp32 tensor of hidden_dim elements")
        st = stream if stream is not None else torch.cuda.current_stream(x.device).cuda_stream
        _check(_capi.lib().prichs_moe_block_backward(self._h, x.data_ptr(), dts[x.dtype], w.data_ptr(), C.c_float(eps), d_out.data_ptr(),
                                                     dts[d_out.dtype], dx.data_ptr(), d_norm.data_ptr() if d_norm is not None else None,
                                                     arr, n if grads is not None else 0, st))
        return dx

    def forward_train(self, x, starkdb_concept_bias: Optional[Sequence[float]] = None, **kw):
        """MoELayer::forward_train (moe.rs:93-211): (out, MoEStash). For CUDA tensors in bf16 mode with all experts local
        the forward keeps the backward pass's activations on the device (prichs_moe_forward_train); the stash's
        activation fields download them on demand. Otherwise only the routing fields are available."""
        import_ok = not isinstance(x, np.ndarray) and self.mode == _capi.MODE_BF16 and self._ep_world == 1
        out = self.forward_with_memory(x, starkdb_concept_bias, _train=import_ok, **kw)
        st = self.last_stash()
        if import_ok:
            st._layer = self
        return out, st

    def stash_field(self, slot: int, which: int) -> np.ndarray:
        """One stash vector of the last forward (prichs_moe_get_stash): slot 0 shared / 1 + e routed expert e;
        which 0 x, 1 gate, 2 up, 3 act, 4 out."""
        n = self._T_last if slot == 0 else int(self.last_counts()[slot - 1])
        width = self.hidden_dim if which in (0, 4) else self.intermediate_dim
        out = np.empty((n, width), np.float32)
        _check(_capi.lib().prichs_moe_get_stash(self._h, slot, which, out.ctypes.data, out.size))
        return out

    def expert_assignments(self, expert: int):
        """(token_indices, weights) of routed expert `expert` for the last forward, tokens ascending."""
        n = C.c_size_t(0)
        cap = int(self.last_counts()[expert])
        idx = np.empty(cap, np.int32)
        w = np.empty(cap, np.float32)
        _check(_capi.lib().prichs_moe_get_expert_assignments(self._h, expert, idx.ctypes.data, w.ctypes.data, cap, C.byref(n)))
        assert n.value == cap
        return idx.astype(np.int64), w

    def last_stash(self) -> MoEStash:
        """Routing results of the last forward (waits for its stream)."""
        L = _capi.lib()
        cnt = self.last_counts()
        T = self._T_last
        E, k = self._num_experts, self.top_k
        lo = np.empty((T, E), np.float32)
        sel = np.empty((T, k), np.int32)
        gw = np.empty((T, k), np.float32)
        if T:
            _check(L.prichs_moe_get_routing(self._h, lo.ctypes.data_as(C.POINTER(C.c_float)),
                                            sel.ctypes.data_as(C.POINTER(C.c_int32)),
                                            gw.ctypes.data_as(C.POINTER(C.c_float)), T))
        return MoEStash(lo, sel.astype(np.int64).reshape(-1), gw.reshape(-1), cnt)

    def last_counts(self) -> np.ndarray:
        c = np.zeros(self._num_experts, np.int64)
        if self._h:
            _check(_capi.lib().prichs_moe_get_counts(self._h, c.ctypes.data_as(C.POINTER(C.c_int64)), c.size))
        return c

    def debug_buffer(self, which: int, nbytes: int, offset: int = 0) -> np.ndarray:
        """Raw bytes of one internal buffer of the last forward (see prichs_moe_debug_copy in the header)."""
        out = np.empty(nbytes, np.uint8)
        _check(_capi.lib().prichs_moe_debug_copy(self._h, which, offset, out.ctypes.data, nbytes))
        return out

    @property
    def token_capacity(self) -> int:
        """max_tokens of the device handle (0 before the first forward)."""
        return self._max_tokens

    def debug_set(self, key: int, value: int):
        """Test knobs of the single-pass routing kernel (prichs_moe_debug_set)."""
        self._ensure(1)
        _check(_capi.lib().prichs_moe_debug_set(self._h, int(key), int(value)))

    def sync_status(self):
        if self._h:
            _check(_capi.lib().prichs_moe_sync_status(self._h))

    # ---- aux-loss-free load balancing ---------------------------------------------------------------
    def update_aux_free_bias(self, expert_token_counts: Sequence[int], total_tokens: int, gamma: float):
        counts = np.ascontiguousarray(expert_token_counts, np.uintp)
        if counts.size != self._num_experts:
            raise PrichsError(_capi.ERR_BAD_SHAPE, "expert_token_counts length differs from the number of experts")
        self._ensure(1)
        _check(_capi.lib().prichs_moe_update_aux_free_bias(self._h, counts.ctypes.data_as(C.POINTER(C.c_size_t)),
                                                           counts.size, int(total_tokens), C.c_float(gamma)))

    def update_bias_from_last(self, gamma: float, total_tokens: int = 0, stream=None):
        """Device-side variant: uses the counts of the last forward without a host round trip."""
        if not self._h:
            return
        _check(_capi.lib().prichs_moe_update_bias_from_last(self._h, C.c_float(gamma), int(total_tokens), stream))
