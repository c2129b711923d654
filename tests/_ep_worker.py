"""Expert-parallel parity worker, one process per GPU (launched by tests/test_gpu_zep.py through
torch.distributed.run). Every rank routes its own seeded tokens, the experts are partitioned over the ranks,
and each rank checks its outputs against the CPU oracle run on the full (unpartitioned) layer."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    import torch
    import torch.distributed as dist
    from prichs_b200 import MoELayer, ep, synth
    from oracle import oracle as O
    from _util import assert_close

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    O.set_num_threads(max(1, (os.cpu_count() or 8) // world))  # the ranks share the host's cores for the oracle
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    # (d, f, E, k, T, bias range, waves): the last two cases cut the batch into token waves
    # (d, f, E, k, T, bias range, waves, skew): the later cases cut the batch into token waves; `skew` scales the
    # router columns so that the first experts attract most tokens (the shape of the Zipf-skewed config)
    cases = [(512, 384, 8, 2, 1000, (-0.1, 0.1), 1, False), (1536, 1280, 8, 2, 2048, None, 1, False),
             (512, 384, 8, 2, 3000, (-0.1, 0.1), 3, False), (1536, 1280, 8, 2, 4096, None, 4, False),
             (512, 384, 8, 2, 2500, None, 2, True),
             (512, 384, 8, 2, 40, (-0.1, 0.1), 4, False),       # fewer tokens than waves x 16: some waves are empty
             (512, 384, 8, 2, 700, (-0.1, 0.1), 2, "f32"),      # fp32-fidelity mode across ranks
             (512, 384, world, 2, 1800, (-0.1, 0.1), 3, False),   # one expert per rank, whatever the group size
             # the multi-GPU configurations of the baseline at their real size: T = 32768 tokens per GPU, production
             # dimensions, default waves; uniform routing and the Zipf(1.2)-skewed router. Routing is checked on every
             # token, outputs on a seeded sample of 1024 tokens per rank.
             (1536, 1280, 8, 2, 32768, None, 0, "big"), (1536, 1280, 8, 2, 32768, None, 0, "zipf")]
    for d, f, E, k, T, brange, waves, skew in cases:
        f32 = skew == "f32"
        big = skew in ("big", "zipf")
        zipf = skew == "zipf"
        skew = skew is True
        Tr = T + 37 * rank  # ragged: every rank brings a different number of tokens
        ws = synth.layer_weights(3, d, f, E, std=0.02 if big else 0.03, bf16=not f32)
        bias = synth.router_bias(3, E, *brange) if brange else np.zeros(E, np.float32)
        if zipf:
            import bench
            ws[0], _, zshare, ztarget = bench.zipf_router(ws[0], 4)
        if skew:
            ws[0] = synth.round_bf16(np.abs(ws[0]) * np.array([6, 4, 3, 2, 1.5, 1, 1, 1], np.float32)[None, :] *
                                     np.sign(synth.normal(5, 1, ws[0].shape)))
            bias = np.array([0.6, 0.3, 0.15, 0, 0, 0, 0, 0], np.float32)
        x = synth.tokens(3000 + rank, Tr, d, bf16=not f32)
        El = E // world
        m = MoELayer.from_weights(ws, k, ep_world=world, ep_rank=rank, device=local, ep_waves=waves, mode="f32" if f32 else "bf16")
        for e in range(E):  # experts owned by other ranks are not uploaded here
            if e // El != rank:
                m.experts[e].gate_proj = m.experts[e].up_proj = m.experts[e].down_proj = None
        m.router_bias = bias
        ep.connect(m, dist, max_tokens=T + 37 * world)
        if f32:
            xd = torch.from_numpy(x).cuda()
        else:
            xd = torch.from_numpy(synth.to_bf16_bits(x).view(np.int16)).view(torch.bfloat16).cuda()
        for rep in range(2):  # twice: buffers are reused across calls
            y = m.forward(xd).float().cpu().numpy()
            m.sync_status()
        st = m.last_stash()
        given = O.route(None, ws[0], bias, k, logits=st.router_logits)
        sel = st.selected_experts.reshape(Tr, k)
        assert np.array_equal(sel, given["selected"]), "top-k differs from the oracle on the GPU's logits"
        assert np.array_equal(st.expert_token_counts, given["counts"])
        # device plan against the host restatement
        cm = torch.tensor(st.expert_token_counts, device="cuda")
        allc = [torch.zeros_like(cm) for _ in range(world)]
        dist.all_gather(allc, cm)
        cmat = np.stack([c.cpu().numpy() for c in allc])
        hp = ep.plan(cmat, rank)
        meta = m.debug_buffer(5, 4 * 100).view(np.int32)
        if waves == 1:  # with several waves every wave has a plan of its own; the summary keeps the sums
            assert np.array_equal(meta[8:8 + E], hp["seg_base"]), (meta[8:16], hp["seg_base"])
            assert np.array_equal(meta[16:16 + E], hp["src_off"])
            assert meta[32] == hp["n_mtiles"]
        assert np.array_equal(meta[24:24 + E], hp["total"])
        assert meta[33] == hp["recv_rows"] and meta[34] == 0
        assert np.array_equal(meta[36:36 + 8 * world].reshape(world, 8)[:, :E], cmat)
        # outputs against the oracle of the whole layer on this rank's tokens
        mask = None
        if big:
            mask = np.zeros(Tr, bool)
            mask[np.random.default_rng(77 + rank).choice(Tr, size=1024, replace=False)] = True
        ref = O.moe_forward_train(ws, bias, k, x, token_mask=mask)
        ok = np.all(ref["selected"] == sel, axis=1)
        assert (~ok).sum() <= max(2, Tr // 200)
        if mask is not None:
            ok &= mask
        rep_ = assert_close(y[ok], ref["out"][ok], 1e-3 if f32 else 2e-2, f"EP output rank {rank}")
        # bias update from the global counts: identical on every rank, equal to the oracle's
        total_tokens = sum(T + 37 * r for r in range(world))
        m.update_bias_from_last(1e-3, total_tokens=total_tokens)  # ragged ranks: the global total is given
        exp = O.update_aux_free_bias(bias, cmat.sum(axis=0), total_tokens, 1e-3, k)
        assert np.array_equal(m.router_bias, exp)
        if skew or zipf:
            share = cmat.sum(axis=0) / cmat.sum()
            assert share.max() > 1.5 / E, f"routing is not skewed: {share}"
        if big and not zipf:
            # the host-buffer entry point feeds an expert-parallel batch through in chunks (every rank the same number
            # of chunks, each a collective forward): same result, same counts, and the stash covers the whole batch
            counts_dev = st.expert_token_counts.copy()
            yh = m.forward(x.astype(np.float32))
            m.sync_status()
            assert_close(yh[ok], ref["out"][ok], 2e-2, f"EP output through host buffers, rank {rank}")
            assert np.abs(yh - y).max() <= 1e-2 * (np.abs(y).max() + 1.0)
            st2 = m.last_stash()
            assert np.array_equal(st2.expert_token_counts, counts_dev)
            assert np.array_equal(st2.selected_experts, st.selected_experts)
        print(f"EP_OK rank={rank} d={d} T={Tr} waves={waves} max_rel={rep_['max_rel']:.3e} recv_rows={hp['recv_rows']}", flush=True)
        dist.barrier()
        m.close()
        dist.barrier()
    # capacity: a receive region that is too small is detected on every rank, reported once, and nothing is
    # written out of bounds; the handle stays usable
    from prichs_b200 import PrichsError
    d, f, E, k, T = 512, 384, 8, 2, 1500
    ws = synth.layer_weights(3, d, f, E, std=0.03, bf16=True)
    m = MoELayer.from_weights(ws, k, ep_world=world, ep_rank=rank, device=local, ep_waves=1, ep_max_recv_rows=64)
    El = E // world
    for e in range(E):
        if e // El != rank:
            m.experts[e].gate_proj = m.experts[e].up_proj = m.experts[e].down_proj = None
    ep.connect(m, dist, max_tokens=T)
    xd = torch.from_numpy(synth.to_bf16_bits(synth.tokens(3100 + rank, T, d, bf16=True)).view(np.int16)).view(torch.bfloat16).cuda()
    m.forward(xd)
    try:
        m.sync_status()
        raise AssertionError("the overflow was not reported")
    except PrichsError as e:
        assert e.code == -2, e
    m.sync_status()  # cleared after the report
    assert int(m.last_counts().sum()) == T * k
    print(f"EP_OK rank={rank} capacity overflow reported", flush=True)
    dist.barrier()
    m.close()
    dist.barrier()
    # readiness flags: rank 0 withholds its "rows landed" signal of wave 0 (test knob); every rank's bounded wait for it
    # runs out after about a millisecond, the forward ends in an orderly way and reports PRICHS_ERR_TIMEOUT; with the
    # knob cleared the same handles work again. Nothing faults or hangs. The NCCL-barrier variant must give the same
    # output as the flag variant.
    ws = synth.layer_weights(3, d, f, E, std=0.03, bf16=True)
    outs = []
    for nccl_barriers in (0, 1):
        m = MoELayer.from_weights(ws, k, ep_world=world, ep_rank=rank, device=local, ep_waves=2, ep_nccl_barriers=nccl_barriers,
                                  ep_dispatch_kernel=nccl_barriers)  # second pass: also the warp-per-token dispatch kernel
        for e in range(E):
            if e // El != rank:
                m.experts[e].gate_proj = m.experts[e].up_proj = m.experts[e].down_proj = None
        ep.connect(m, dist, max_tokens=T)
        outs.append(m.forward(xd).float().cpu().numpy())
        m.sync_status()
        if nccl_barriers == 0:
            m.debug_set(1, 2_000_000)
            if rank == 0:
                m.debug_set(2, 1 + 0 * 4 + 0)
            m.forward(xd)
            try:
                m.sync_status()
                raise AssertionError("the missing readiness signal was not reported")
            except PrichsError as e:
                assert e.code == -5, e
            m.debug_set(2, 0)
            m.debug_set(1, 4_000_000_000)
            dist.barrier()
            again = m.forward(xd).float().cpu().numpy()
            m.sync_status()
            assert np.array_equal(again, outs[0])
            print(f"EP_OK rank={rank} readiness wait ran out and was reported", flush=True)
        dist.barrier()
        m.close()
        dist.barrier()
    assert np.array_equal(outs[0], outs[1]), "flag and NCCL-barrier variants differ"
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
