"""Expert-parallel protocol on CPU ranks (gloo, world_size 2): partition invariance.

Each rank routes its own tokens (oracle), the ranks all-gather their counts, build the placement plan with
prichs_b200.ep.plan (the host restatement of the device plan), place rows in the owners' receive buffers at
seg_base + src_off + local index exactly as the dispatch kernel does, run the owned experts, and the source
ranks gather the rows back and combine them in ascending expert order. The result must equal the single-rank
oracle bit for bit in fp32 (the layer is token-wise independent once routing is fixed)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    from oracle import oracle as O
    from prichs_b200 import ep
    from _util import small_int_weights, grid_tensor
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        O.set_num_threads(2)
        d, f, E, k = 64, 32, 8, 2
        El = E // world
        ws = small_int_weights(3, d, f, E)
        bias = grid_tensor(3, 1000, (E,), 4, 32)
        T = 50 + 13 * rank
        x = grid_tensor(3000 + rank, 0, (T, d), 16, 8)
        r = O.route(x, ws[0], bias, k)
        sel, gat, counts = r["selected"], r["gating"], r["counts"]
        allc = [None] * world
        dist.all_gather_object(allc, counts)
        cmat = np.stack(allc)
        p = ep.plan(cmat, rank)
        # dispatch: (owner, row, payload) for every assignment, rows in token order inside an expert
        seen = np.zeros(E, np.int64)
        pos = np.zeros((T, k), np.int64)
        outbox = [[] for _ in range(world)]
        for t in range(T):
            for j in range(k):
                e = int(sel[t, j])
                row = int(p["seg_base"][e] + p["src_off"][e] + seen[e])
                seen[e] += 1
                pos[t, j] = row
                outbox[e // El].append((row, x[t]))
        inboxes = [None] * world
        dist.all_gather_object(inboxes, outbox)
        mine = ep.plan(cmat, rank)
        cap = mine["n_mtiles"] * 128
        xp = np.zeros((cap, d), np.float32)
        filled = np.zeros(cap, bool)
        for src in range(world):
            for row, payload in inboxes[src][rank]:
                assert not filled[row], "two assignments landed on one row"
                xp[row], filled[row] = payload, True
        assert int(filled.sum()) == mine["recv_rows"]
        # owned experts over their 128-aligned segments
        yp = np.zeros((cap, d), np.float32)
        for le in range(El):
            e = rank * El + le
            lo, n = int(mine["seg_base"][e]), int(mine["total"][e])
            assert lo % 256 == 0 and filled[lo:lo + n].all() and not filled[lo + n:lo + (n + 255) // 256 * 256].any()
            if n:
                h = O.swiglu(O.matmul_2d(xp[lo:lo + n], ws[4 + 3 * e]), O.matmul_2d(xp[lo:lo + n], ws[5 + 3 * e]))
                yp[lo:lo + n] = O.matmul_2d(h, ws[6 + 3 * e])
        ybufs = [None] * world
        dist.all_gather_object(ybufs, yp)
        # combine on the source rank: shared row, then experts ascending, multiply and add rounded separately
        hs = O.swiglu(O.matmul_2d(x, ws[1]), O.matmul_2d(x, ws[2]))
        out = O.matmul_2d(hs, ws[3])
        for t in range(T):
            for j in np.argsort(sel[t], kind="stable"):
                e = int(sel[t, j])
                out[t] = out[t] + np.float32(gat[t, j]) * ybufs[e // El][pos[t, j]]
        ref = O.moe_forward_train(ws, bias, k, x)
        ok = np.array_equal(out, ref["out"]) and np.array_equal(ref["counts"], counts)
        # the bias update from global counts is the same on every rank
        b = O.update_aux_free_bias(bias, cmat.sum(axis=0), int(sum(50 + 13 * q for q in range(world))), 1e-3, k)
        allb = [None] * world
        dist.all_gather_object(allb, b)
        ok = ok and all(np.array_equal(b, o) for o in allb)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_expert_parallel_partition_invariance_gloo():
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29600 + os.getpid() % 200
    ctx = mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=False)
    import time
    deadline = time.time() + 240
    while not ctx.join(timeout=5):  # join() returns False while some rank is still running
        assert time.time() < deadline, "gloo ranks did not finish"
    assert dict(ret) == {0: True, 1: True}


def test_plan_properties():
    sys.path.insert(0, ROOT)
    from prichs_b200 import ep
    rng = np.random.default_rng(0)
    for world in (1, 2, 4, 8):
        cmat = rng.integers(0, 400, size=(world, 8))
        cmat[:, 3] = 0  # an expert nobody selected
        plans = [ep.plan(cmat, r) for r in range(world)]
        El = 8 // world
        for e in range(8):
            o = e // El
            # the ranks' slices tile the expert's segment without gaps or overlap, in rank order
            offs = [int(plans[r]["src_off"][e]) for r in range(world)]
            assert offs == np.concatenate([[0], np.cumsum(cmat[:-1, e])]).tolist()
            assert all(int(pl["seg_base"][e]) == int(plans[o]["seg_base"][e]) for pl in plans)
            assert plans[o]["seg_base"][e] % 256 == 0
        assert sum(pl["recv_rows"] for pl in plans) == int(cmat.sum())


# ---- failure detection on the host: a rank that never posts its counts -------------------------------------------
def _lost_peer_worker(rank, world, port, ret):
    """Rank 0 starts the counts all-gather of a wave and waits for it under the library's watchdog
    (prichs_ep_wait_or_abort through the C-ABI); rank 1 takes part in the first exchange and then stops answering
    (it never posts the counts of the second one). Rank 0 must get PRICHS_OK for the first, PRICHS_ERR_COMM for the
    second after the timeout, with its abort callback called exactly once. No GPU is involved."""
    sys.path.insert(0, ROOT)
    import ctypes as C
    import time
    import torch
    import torch.distributed as dist
    from prichs_b200 import _capi
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    L = _capi.lib()
    QUERY = C.CFUNCTYPE(C.c_int, C.c_void_p)
    ABORT = C.CFUNCTYPE(None, C.c_void_p)
    state = {"work": None, "aborted": 0}
    query = QUERY(lambda ctx: 0 if state["work"].is_completed() else 1)

    def _abort(ctx):
        state["aborted"] += 1
    abort = ABORT(_abort)

    def gather_counts(counts):
        out = [torch.zeros(8, dtype=torch.int32) for _ in range(world)]
        state["work"] = dist.all_gather(out, torch.tensor(counts, dtype=torch.int32), async_op=True)
        return out

    # healthy exchange: both ranks post
    out = gather_counts([rank + 1] * 8)
    rc_ok = L.prichs_ep_wait_or_abort(C.cast(query, C.c_void_p), C.cast(abort, C.c_void_p), None, 20000, 200)
    healthy = rc_ok == _capi.OK and int(out[1 - rank][0]) == (1 - rank) + 1 and state["aborted"] == 0
    if rank == 1:
        # the lost peer: it never posts its counts of the next wave
        ret[rank] = bool(healthy)
        time.sleep(4.0)
        os._exit(0)
    gather_counts([7] * 8)
    t0 = time.time()
    rc = L.prichs_ep_wait_or_abort(C.cast(query, C.c_void_p), C.cast(abort, C.c_void_p), None, 500, 200)
    waited = time.time() - t0
    msg = _capi.last_error()
    ret[rank] = bool(healthy and rc == _capi.ERR_COMM and state["aborted"] == 1 and 0.4 <= waited < 3.0 and "never joined" in msg)
    # a query that reports failure ends the wait at once, without the abort callback
    failed = QUERY(lambda ctx: 5)
    ret["failed_query"] = L.prichs_ep_wait_or_abort(C.cast(failed, C.c_void_p), C.cast(abort, C.c_void_p), None, 500, 200) == _capi.ERR_COMM \
        and state["aborted"] == 1
    os._exit(0)  # the process group still holds the collective that will never finish: leave without tearing it down


def test_rank_that_never_posts_its_counts_is_detected_by_the_watchdog():
    import time
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29810 + os.getpid() % 150
    ctx = mp.spawn(_lost_peer_worker, args=(world, port, ret), nprocs=world, join=False)
    deadline = time.time() + 120
    while not ctx.join(timeout=2):
        assert time.time() < deadline, "ranks did not finish"
    assert dict(ret) == {0: True, 1: True, "failed_query": True}


# ---- readiness-flag protocol on CPU ranks ---------------------------------------------------------------------------
def _flag_worker(rank, world, port, ret):
    """Host model of the expert-parallel exchange's readiness flags (route::ep_signal_kernel / ep_wait_kernel) with the
    process group's key-value store standing in for peer-mapped memory: "store rows into the owner's receive region,
    then store the forward's sequence number into slot [kind][wave][source] of the owner's flag array"; the owner polls
    its own slots with a budget and only then reads the rows. Three forwards of two waves: the rows a rank reads after a
    successful wait belong to that forward or a later one, never an earlier one (sequence numbers only grow, nothing is
    reset); a withheld signal makes every rank's wait run out and report a timeout, and the next forward works again;
    a signal of an older forward never satisfies a wait for a newer one."""
    sys.path.insert(0, ROOT)
    import time
    import torch.distributed as dist
    from prichs_b200 import ep
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    store = dist.distributed_c10d._get_default_store()
    board = ep.FlagBoard(store, rank, world)
    ok = True
    for seq in (1, 2, 3):
        for wave in (0, 1):
            for dst in range(world):  # "dispatch": this rank's rows of the wave land in every owner's region ...
                store.set(f"rows/{dst}/{wave}/{rank}", f"{seq}:{rank}")
                withheld = seq == 2 and wave == 1 and rank == 1
                if not withheld:          # ... and only then the signal is stored
                    board.signal(0, wave, seq, dst)
            status = board.wait(0, wave, seq, budget_s=0.5 if seq == 2 else 20.0)
            if seq == 2 and wave == 1:
                ok = ok and status == ep.FlagBoard.TIMEOUT  # every rank misses rank 1's signal
            else:
                ok = ok and status == ep.FlagBoard.OK
                for src in range(world):  # the rows seen after the wait are at least this forward's
                    s_, r_ = store.get(f"rows/{rank}/{wave}/{src}").decode().split(":")
                    ok = ok and int(s_) >= seq and int(r_) == src
        dist.barrier()
    # a signal from an OLDER forward never satisfies a wait for a newer one; a newer one does (wrap-safe comparison)
    ok = ok and board.wait(0, 0, 4, budget_s=0.2) == ep.FlagBoard.TIMEOUT
    ok = ok and ep.FlagBoard.reached(5 - 2 ** 32, 2 ** 31 - 3 - 2 ** 32) is False and ep.FlagBoard.reached(-2 ** 31 + 1, 2 ** 31 - 1) is True
    ret[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_readiness_flag_protocol_gloo():
    import time
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29400 + os.getpid() % 150
    ctx = mp.spawn(_flag_worker, args=(world, port, ret), nprocs=world, join=False)
    deadline = time.time() + 120
    while not ctx.join(timeout=2):
        assert time.time() < deadline, "ranks did not finish"
    assert dict(ret) == {0: True, 1: True}
