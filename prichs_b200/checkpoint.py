"""Reader for the reference's `PRICHS02` checkpoints: pulls the MoE-layer tensors of every block out of a
whole-model file and builds `MoELayer`s from them.

File format (crates/prichs-model/src/model.rs:1648-1670): b"PRICHS02", step u64 LE, loss f32 LE, n_params u64 LE,
then per tensor `len u64 LE` + len f32 LE values, in the order of `get_parameter_tensors` (model.rs:341-364):
    0 wte, 1 final_norm, then per block l with base = 2 + l * (10 + 3 E):
    +0 input_norm, +1 q_proj, +2 k_proj, +3 v_proj, +4 out_proj, +5 post_attn_norm, +6 moe.router,
    +7 shared gate, +8 shared up, +9 shared down, +10 + 3 e + {0, 1, 2} expert e gate / up / down.
Tensors carry no shape in the file; shapes come from the model configuration, as in the reference's loader
(model.rs:1697-1709). The reference never saves `router_bias` (it is not a parameter tensor), so a trained bias is
kept in a side file `<checkpoint>.router_bias.npy` of shape [n_layers, E] written by `save_router_bias`.
"""
from __future__ import annotations

import os
import struct
from typing import List, Optional, Tuple

import numpy as np

from .moe import MoELayer, PrichsError

MAGIC = b"PRICHS02"
_ERR_BAD_SHAPE = -1


def read_tensors(path: str) -> Tuple[int, float, List[np.ndarray]]:
    """(step, loss, flat f32 arrays in file order). Arrays are views into a memory map of the file."""
    size = os.path.getsize(path)
    with open(path, "rb") as fh:
        head = fh.read(28)
    if len(head) < 28 or head[:8] != MAGIC:
        raise PrichsError(_ERR_BAD_SHAPE, f"Invalid checkpoint magic in {path!r}: {head[:8]!r}")
    step, = struct.unpack_from("<Q", head, 8)
    loss, = struct.unpack_from("<f", head, 16)
    n_params, = struct.unpack_from("<Q", head, 20)
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    tensors, off = [], 28
    for _ in range(n_params):
        if off + 8 > size:
            raise PrichsError(_ERR_BAD_SHAPE, "checkpoint is truncated")
        n = int(mm[off:off + 8].view("<u8")[0])
        off += 8
        if off + 4 * n > size:
            raise PrichsError(_ERR_BAD_SHAPE, "checkpoint is truncated")
        tensors.append(mm[off:off + 4 * n].view("<f4"))
        off += 4 * n
    return int(step), float(loss), tensors


def write_tensors(path: str, step: int, loss: float, tensors) -> None:
    """Writes a file in the same format (used by the tests and to re-export weights)."""
    with open(path, "wb") as fh:
        fh.write(MAGIC + struct.pack("<Q", step) + struct.pack("<f", loss) + struct.pack("<Q", len(tensors)))
        for t in tensors:
            a = np.ascontiguousarray(t, dtype="<f4").reshape(-1)
            fh.write(struct.pack("<Q", a.size))
            fh.write(a.tobytes())


def bias_path(path: str) -> str:
    return path + ".router_bias.npy"


def save_router_bias(path: str, biases) -> None:
    np.save(bias_path(path), np.asarray(biases, np.float32))


def moe_tensor_indices(layer: int, num_experts: int) -> dict:
    base = 2 + layer * (10 + 3 * num_experts)
    return {"post_attn_norm": base + 5, "router": base + 6, "shared": (base + 7, base + 8, base + 9),
            "experts": [(base + 10 + 3 * e, base + 11 + 3 * e, base + 12 + 3 * e) for e in range(num_experts)]}


def load_moe_layers(path: str, hidden_dim: int, intermediate_dim: int, num_experts: int, top_k: int, **layer_kw):
    """Returns (layers, post_attn_norms, step, loss): one MoELayer per block of the checkpoint with the block's
    post-attention norm weight (the pre-norm of the MoE sub-layer, block.rs:64). `layer_kw` goes to MoELayer."""
    step, loss, ts = read_tensors(path)
    per_block = 10 + 3 * num_experts
    if len(ts) < 2 or (len(ts) - 2) % per_block != 0:
        raise PrichsError(_ERR_BAD_SHAPE, f"Checkpoint parameter count {len(ts)} != model parameter count 2 + n_layers * {per_block}")
    n_layers = (len(ts) - 2) // per_block
    d, f, E = hidden_dim, intermediate_dim, num_experts
    bias = None
    if os.path.exists(bias_path(path)):
        bias = np.load(bias_path(path)).astype(np.float32)
        if bias.shape != (n_layers, E):
            raise PrichsError(_ERR_BAD_SHAPE, f"router bias side file has shape {bias.shape}, expected {(n_layers, E)}")

    def take(i, shape):
        t = ts[i]
        if t.size != int(np.prod(shape)):
            raise PrichsError(_ERR_BAD_SHAPE, f"tensor {i} has {t.size} values, the configuration expects {shape}")
        return np.array(t, dtype=np.float32).reshape(shape)

    layers, norms = [], []
    for l in range(n_layers):
        ix = moe_tensor_indices(l, E)
        ws = [take(ix["router"], (d, E)), take(ix["shared"][0], (d, f)), take(ix["shared"][1], (d, f)), take(ix["shared"][2], (f, d))]
        for g, u, dn in ix["experts"]:
            ws += [take(g, (d, f)), take(u, (d, f)), take(dn, (f, d))]
        m = MoELayer.from_weights(ws, top_k, **layer_kw)
        if bias is not None:
            m.router_bias = bias[l]
        layers.append(m)
        norms.append(take(ix["post_attn_norm"], (d,)))
    return layers, norms, step, loss
