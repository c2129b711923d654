"""Expert-parallel helpers on the host side.

`plan` restates, in numpy, the placement plan the device computes from the all-gathered counts matrix
(route::plan_from_cmat): where each expert's segment starts in its owner's receive buffer and where a given
source rank's rows sit inside it. Tests use it to check the device plan; it is not on the data path.

`connect` wires a group of MoELayer handles together using torch.distributed only as the byte channel that
the C ABI asks for (broadcast of the 128-byte id, all-gather of the 128-byte buffer handles).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _capi


def owner_of(expert: int, num_experts: int, world: int) -> int:
    return expert // (num_experts // world)


SEG_PAD = 256  # rows; every expert's segment starts on a multiple of it (one CTA-pair GEMM tile)


def plan(cmat: np.ndarray, rank: int, pad: int = SEG_PAD):
    """cmat[s, e] = assignments rank s produced for expert e. Returns total[e], src_off[e] (rows of lower ranks
    ahead of `rank` inside expert e's segment), seg_base[e] (start of the segment in the owner's buffer, segments
    padded to `pad` rows), recv_rows and n_mtiles (128-row tiles) of `rank`."""
    cmat = np.asarray(cmat, np.int64)
    world, E = cmat.shape
    El = E // world
    total = cmat.sum(axis=0)
    src_off = cmat[:rank].sum(axis=0)
    seg_base = np.zeros(E, np.int64)
    padded = (total + pad - 1) // pad * pad
    for o in range(world):
        base = 0
        for le in range(El):
            e = o * El + le
            seg_base[e] = base
            base += padded[e]
    mine = slice(rank * El, (rank + 1) * El)
    return dict(total=total, src_off=src_off, seg_base=seg_base, recv_rows=int(total[mine].sum()),
                n_mtiles=int(padded[mine].sum() // 128))


def connect(layer, dist, max_tokens: int):
    """Create the layer's device handle (for `max_tokens`) and join the expert-parallel group over `dist`
    (an initialised torch.distributed module). Collective: every rank calls it."""
    L = _capi.lib()
    layer._want_max_tokens = max(layer._want_max_tokens, int(max_tokens))
    layer._ensure(int(max_tokens))
    rank, world = dist.get_rank(), dist.get_world_size()
    ident = (C.c_char * 1024)()
    if rank == 0:
        rc = L.prichs_moe_ep_unique_id(ident)
        if rc != 0:
            raise RuntimeError(_capi.last_error())
    box = [bytes(ident)]
    dist.broadcast_object_list(box, src=0)
    blob = (C.c_char * 128)()
    rc = L.prichs_moe_ep_export(layer._h, blob)
    if rc != 0:
        raise RuntimeError(_capi.last_error())
    blobs = [None] * world
    dist.all_gather_object(blobs, bytes(blob))
    all_blobs = b"".join(blobs)
    rc = L.prichs_moe_ep_init(layer._h, box[0], all_blobs)
    if rc != 0:
        raise RuntimeError(_capi.last_error())
    layer._ep_connected = True


class FlagBoard:
    """Host restatement of the readiness flags of the expert-parallel exchange (route::ep_signal_kernel /
    ep_wait_kernel) over any key-value store with `set` / `get`: slot [kind][wave][source] of rank `dst`'s flag array
    holds the sequence number of the last forward whose part `kind` of `wave` rank `source` has finished. Tests use it to
    exercise the protocol (ordering, growing sequence numbers, bounded wait) on CPU ranks; it is not on the data path."""
    OK, TIMEOUT = 0, -5

    def __init__(self, store, rank: int, world: int):
        self.store, self.rank, self.world = store, rank, world

    @staticmethod
    def _key(dst, kind, wave, src):
        return f"flag/{dst}/{kind}/{wave}/{src}"

    @staticmethod
    def reached(value: int, seq: int) -> bool:
        """`value - seq >= 0` in 32-bit wrap-around arithmetic, as the device compares sequence numbers."""
        diff = (value - seq) & 0xFFFFFFFF
        return diff < 0x80000000

    def signal(self, kind: int, wave: int, seq: int, dst: int):
        self.store.set(self._key(dst, kind, wave, self.rank), str(seq))

    def wait(self, kind: int, wave: int, seq: int, budget_s: float) -> int:
        import time
        deadline = time.time() + budget_s
        pending = set(range(self.world))
        while pending:
            for src in list(pending):
                key = self._key(self.rank, kind, wave, src)
                if self.store.check([key]) and self.reached(int(self.store.get(key).decode()), seq):
                    pending.discard(src)
            if pending and time.time() > deadline:
                return self.TIMEOUT
            if pending:
                time.sleep(0.002)
        return self.OK
