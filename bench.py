#!/usr/bin/env python
"""Benchmark of the PRICHS MoE-layer forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward pass of the MoE layer over one batch of synthetic tokens.
N = 1: config 1 of the baseline -- T = 16384 tokens (8 x 2048), d = 1536, f = 1280, 1 shared + 8 routed
       experts, top-2, bf16, seed 1, router bias ~ U(-0.1, 0.1).
N > 1: config 3 -- expert parallel, T = 32768 tokens per GPU (weak scaling), bias 0.
Prints ONE JSON line (rank 0): `value` = tokens/s with inputs resident in HBM (CUDA events, max over ranks),
`e2e` = the same metric through the host-buffer entry point (pinned fp32 host tensors, copies inside the
timed region), `roofline` for the dominant kernel, `cpu_baseline` = the CPU oracle on the host cores.
`--impl reference` times the CPU restatement of the reference path (the Rust original cannot be built here).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D, F, E, K = 1536, 1280, 8, 2
FLOPS_PER_TOKEN = 18 * D * F           # 3 expert MLPs x 6 d f
GATE_UP_FLOPS_PER_TOKEN = 12 * D * F   # first GEMM: 3 experts x (gate + up)
DOWN_FLOPS_PER_TOKEN = 6 * D * F
ROUTER_BYTES = D * 2 + K * 4 + K * 4
DISPATCH_BYTES = D * 2 + K * D * 2 + K * 4 + K * 4
COMBINE_BYTES_NORES = (K + 1) * D * 2 + D * 2 + K * 4 + K * 4  # no residual in the benchmarked call


def roofline_sum(T, gemm_rows, ms_step, peaks, world=1):
    """Lower bound of one forward from the rooflines of its stages, and the measured step against it:
    GEMM flops / tensor peak + (router + dispatch + combine bytes) / HBM peak, plus, for an expert-parallel group,
    the dispatch and combine rows that cross NVLink at 900 GB/s per direction (un-overlapped: summed; overlapped: the
    larger of the exchange and everything else)."""
    t_gemm = gemm_rows * 6 * D * F / (peaks["tf"] * 1e12)
    t_hbm = T * (ROUTER_BYTES + DISPATCH_BYTES + COMBINE_BYTES_NORES) / (peaks["hbm"] * 1e9)
    t_comm = 2 * T * K * D * 2 * (world - 1) / world / 900e9 if world > 1 else 0.0
    serial = (t_gemm + t_hbm + t_comm) * 1e3
    overlapped = max(t_gemm + t_hbm, t_comm) * 1e3
    out = {"ms": serial, "frac": serial / ms_step, "gemm_ms": t_gemm * 1e3, "hbm_ms": t_hbm * 1e3}
    if world > 1:
        out.update({"comm_ms": t_comm * 1e3, "ms_overlapped": overlapped, "frac_overlapped": overlapped / ms_step})
    return out


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return dict(hbm=float(j["hbm_gbs"]), tf=float(j["bf16_tflops"]), tf_sustained=float(j.get("bf16_tflops_sustained", 0)),
                    source="measured")
    return dict(hbm=6650.0, tf=1590.0, tf_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz, self._stop, self._t = [], set(), None, threading.Event(), None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    r = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    r = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self.nv:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._t:
            self._t.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": []}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def cpu_baseline(ws, bias, x_f32, target_seconds=12.0, max_tokens=None):
    """The CPU oracle (a port of the reference's CPU path) on a bounded sample of the workload."""
    from oracle import oracle as O
    T = x_f32.shape[0] if max_tokens is None else min(max_tokens, x_f32.shape[0])
    probe = min(256, T)
    t0 = time.perf_counter()
    O.moe_forward_train(ws, bias, K, x_f32[:probe])
    dt = time.perf_counter() - t0
    n = int(min(T, max(probe, target_seconds / max(dt, 1e-6) * probe)))
    n = max(16, n // 16 * 16)
    t0 = time.perf_counter()
    O.moe_forward_train(ws, bias, K, x_f32[:n])
    dt = time.perf_counter() - t0
    return {"value": n / dt, "unit": "tokens/s", "cores": O.num_threads(), "kind": "port",
            "sample": f"first {n} tokens of the batch, one full layer forward (routing + shared + routed experts + combine), {dt:.2f} s"}


def parity_check(layer, ws, bias, x_host, x_dev, n_sample, seed):
    """This rank's forward of one timed batch against the CPU oracle, outside every timed region: top-2 indices, gates
    and per-expert counts bit-exact on ALL tokens when the oracle's top-k is fed the GPU's own fp32 logits (ties go to
    the lower index), logits within 1e-4, and the layer output of a seeded sample of tokens within the bf16 tolerance
    2e-2 (|a - b| <= tol * (|b| + rms(b))). Tokens whose own-logit routing differs from the GPU's (near-ties of two
    selection logits) are left out of the output comparison and counted."""
    from oracle import oracle as O
    T = x_host.shape[0]
    y = layer.forward(x_dev).float().cpu().numpy()
    layer.sync_status()
    st = layer.last_stash()
    given = O.route(None, ws[0], bias, K, logits=st.router_logits)
    own = O.route(x_host, ws[0], bias, K)
    sel = st.selected_experts.reshape(T, K)
    routing_ok = bool(np.array_equal(sel, given["selected"]) and np.array_equal(st.expert_token_counts, given["counts"])
                      and np.allclose(st.gating_weights.reshape(T, K), given["gating"], rtol=2e-6, atol=1e-7)
                      and int(st.expert_token_counts.sum()) == T * K)
    logit_err = float(np.abs(st.router_logits - own["logits"]).max())
    agree = np.all(sel == own["selected"], axis=1)
    rng = np.random.default_rng(seed)
    mask = np.zeros(T, bool)
    mask[rng.choice(T, size=min(n_sample, T), replace=False)] = True
    mask &= agree
    ref = O.moe_forward_train(ws, bias, K, x_host, token_mask=mask)["out"]
    rms = float(np.sqrt(np.mean(ref[mask].astype(np.float64) ** 2)))
    rel = np.abs(y[mask] - ref[mask]) / (np.abs(ref[mask]) + rms)
    return {"routing_bit_exact": routing_ok, "logits_max_abs_err": logit_err, "max_rel": float(rel.max()),
            "tokens_checked": int(mask.sum()), "tokens_routed": T, "near_tie_tokens_skipped": int((~agree).sum())}


def skew_measure(args, dist, dev, rank, world, local_rank, steps=20):
    """Config 4 as an object of the multi-GPU line: the shapes of config 3 with W_r scaled so that expert selection
    follows Zipf(1.2) (seed 4), timed like the headline (barrier, CUDA events, max over ranks), checked against the
    oracle like the headline, then one aux-loss-free bias step from the global counts (gamma = 1e-3 on load
    fractions, i.e. gamma / (T * world) per token of deviation in count form)."""
    import torch
    from prichs_b200 import MoELayer, ep, synth
    seed, T = 4, (args.tokens or 32768)
    ws = synth.layer_weights(seed, D, F, E, bf16=True)
    ws[0], sigma, share, target = zipf_router(ws[0], seed)
    bias = np.zeros(E, np.float32)
    layer = MoELayer.from_weights(ws, K, max_tokens=T, device=local_rank, ep_world=world, ep_rank=rank, ep_waves=args.ep_waves,
                                  ep_nccl_barriers=args.ep_nccl_barriers, ep_reserve_sms=args.ep_reserve_sms,
                                  ep_dispatch_kernel=args.ep_dispatch_kernel, ep_shared_copy_sms=args.ep_shared_copy_sms)
    for e in range(E):
        if e // (E // world) != rank:
            layer.experts[e].gate_proj = layer.experts[e].up_proj = layer.experts[e].down_proj = None
    ep.connect(layer, dist, max_tokens=T)
    layer.router_bias = bias
    xh = [synth.tokens(seed * 1000 + rank + 7919 * i, T, D, bf16=True) for i in range(2)]
    xs = [torch.from_numpy(synth.to_bf16_bits(x).view(np.int16)).view(torch.bfloat16).to(dev) for x in xh]
    y = torch.empty_like(xs[0])
    for i in range(5):
        layer.forward(xs[i % 2], out=y)
    torch.cuda.synchronize(dev)
    layer.sync_status()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        layer.forward(xs[i % 2], out=y)
    e1.record()
    torch.cuda.synchronize(dev)
    dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    par = parity_check(layer, ws, bias, xh[0], xs[0], 4096 if rank == 0 else 512, 4321 + rank)
    tt = torch.tensor([0.0 if par["routing_bit_exact"] else 1.0, par["max_rel"], par["logits_max_abs_err"]], device=dev, dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    nn = torch.tensor([par["tokens_checked"], par["tokens_routed"]], device=dev, dtype=torch.int64)
    dist.all_reduce(nn)
    gcounts = torch.tensor(layer.last_counts(), device=dev)
    dist.all_reduce(gcounts)
    import ctypes as C
    from prichs_b200 import _capi
    rr = C.c_int64()
    _capi.lib().prichs_moe_ep_recv_rows(layer._h, C.byref(rr))
    rr2 = torch.tensor([int(rr.value)], device=dev, dtype=torch.int64)
    allrows = [torch.zeros_like(rr2) for _ in range(world)]
    dist.all_gather(allrows, rr2)
    layer.update_bias_from_last(1e-3, total_tokens=T * world)
    bias_after = [float(v) for v in layer.router_bias]
    gc = gcounts.cpu().numpy().astype(np.float64)
    out = {"workload": f"config 4: config 3's shapes with a Zipf(1.2)-skewed router (seed 4), {world} GPUs",
           "ms_per_step": ms, "tokens_per_s": T * world / (ms * 1e-3), "steps": steps,
           "parity": {"routing_bit_exact": float(tt[0]) == 0.0, "max_rel": float(tt[1]), "logits_max_abs_err": float(tt[2]),
                      "tokens_checked": int(nn[0]), "tokens_routed": int(nn[1]), "tolerance": 2e-2,
                      "ok": bool(float(tt[0]) == 0.0 and float(tt[1]) <= 2e-2 and float(tt[2]) <= 1e-3)},
           "zipf_alpha": ZIPF_ALPHA, "sigma": [float(v) for v in sigma], "top1_share_sample": [float(v) for v in share],
           "top1_share_target": [float(v) for v in target], "global_counts": [int(v) for v in gc],
           "imbalance_max_over_mean": float(gc.max() / gc.mean()), "recv_rows_per_gpu": [int(v.item()) for v in allrows],
           "bias_after_step": bias_after, "gamma": 1e-3}
    layer.close()
    return out


def run_reference(args):
    """The reference arm: the reference's CPU path (C++ restatement; no Rust toolchain on this image) on the
    host cores, all threads, each step a bounded sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from prichs_b200 import synth
    from oracle import oracle as O
    O.build()
    n_gpus = args.gpus
    seed, T_full = (1, 16384) if n_gpus == 1 else (3, 32768)
    ws = synth.layer_weights(seed, D, F, E, bf16=True)
    bias = synth.router_bias(seed, E, -0.1, 0.1) if n_gpus == 1 else np.zeros(E, np.float32)
    n = 512  # tokens per step: ~18 GFLOP, a fraction of a second on a multi-core host
    x = synth.tokens(seed, n, D, bf16=True)
    for _ in range(args.warmup):
        O.moe_forward_train(ws, bias, K, x)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.moe_forward_train(ws, bias, K, x)
    dt = time.perf_counter() - t0
    v = n * args.steps / dt
    sample = f"{n} tokens per step (first rows of the T={T_full} batch), full layer forward on the CPU"
    line = {
        "impl": "reference", "metric": "MoE-layer tokens/sec", "value": v, "unit": "tokens/s", "n_gpus": n_gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(n_gpus),
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": O.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def workload_config(n_gpus):
    if n_gpus == 1:
        return {"workload": "config 1: MoE layer forward, T=16384 (8x2048), d=1536, f=1280, 1 shared + 8 routed experts, "
                            "top-2, bf16, seed 1, bias~U(-0.1,0.1)",
                "tokens_per_step": 16384, "parallelism": "single GPU",
                "l2": "inputs rotate over 4 distinct batches (201 MB) and the per-step working set (~0.6 GB) exceeds the 126 MB L2"}
    return {"workload": f"config 3: expert-parallel MoE layer forward, T=32768 tokens per GPU, {E // n_gpus} routed experts per GPU, "
                        "shared expert replicated, bf16, seed 3, bias 0",
            "tokens_per_step": 32768 * n_gpus, "parallelism": f"ep{n_gpus}",
            "l2": "per-GPU working set (~1.2 GB) exceeds the 126 MB L2; inputs rotate over 2 batches"}


ZIPF_ALPHA = 1.2


def zipf_router(ws_router, seed, n_sample=65536, iters=60):
    """Config 4: per-expert column factors sigma_i for W_r, found by a host-side fixed-point iteration on a
    token sample, such that expert i's share of top-1 selections follows Zipf(alpha = 1.2)."""
    from prichs_b200 import synth
    target = 1.0 / np.arange(1, E + 1) ** ZIPF_ALPHA
    target /= target.sum()
    xs = synth.tokens(seed * 100 + 77, n_sample, D, bf16=True)
    base = xs @ ws_router  # [n, E] logits at sigma = 1
    sigma = np.ones(E, np.float64)
    share = None
    for _ in range(iters):
        share = np.bincount(np.argmax(base * sigma[None, :].astype(np.float32), axis=1), minlength=E) / n_sample
        if np.all(np.abs(share - target) <= 0.01 * target + 1e-4):
            break
        sigma *= (target / np.maximum(share, 1e-6)) ** 0.5
        sigma /= sigma[-1]
    return synth.round_bf16((ws_router * sigma[None, :].astype(np.float32))), sigma, share, target


def decode_measure(n_layers, steps, warmup, stream_counts, use_graph=True, **tuning):
    """Config 2 (decode shape, bandwidth bound): `n_layers` independent MoE layers of the production dimensions, each
    with its own seeded weights (seed 2 + layer), applied to the same T = 64 tokens; one step = all layer forwards.
    The layers are independent by the config's definition, so they may be spread over several streams: the small
    routing kernels of one layer then overlap the weight streaming of others. Measured for every entry of
    `stream_counts` (1 = all layers back to back on one stream). Returns one dict per stream count."""
    import torch
    from prichs_b200 import MoELayer, _capi, synth
    dev = torch.device("cuda", torch.cuda.current_device())
    T = 64
    x_host = synth.tokens(2, T, D, bf16=True)
    x = torch.from_numpy(synth.to_bf16_bits(x_host).view(np.int16)).view(torch.bfloat16).to(dev)
    layers = []
    for l in range(n_layers):
        m = MoELayer.from_weights(synth.layer_weights(2 + l, D, F, E, bf16=True), K, max_tokens=T, device=dev.index, **tuning)
        m.forward(x)  # creates the handle and uploads the weights
        m.router = m.shared_expert = None  # the host copies are not needed any more
        m.experts = []
        layers.append(m)
    L = _capi.lib()
    peaks = measured_peaks()
    wbytes = n_layers * 9 * 3 * D * F * 2  # every expert of every layer is hit with probability ~1 at 128 assignments
    results = []
    for nstreams in stream_counts:
        lanes = [torch.cuda.Stream(dev) for _ in range(nstreams)] if nstreams > 1 else []
        ys = [torch.empty_like(x) for _ in range(max(1, nstreams))]

        def step():
            if not lanes:
                st = torch.cuda.current_stream(dev).cuda_stream
                for m in layers:
                    rc = L.prichs_moe_forward(m._h, x.data_ptr(), _capi.DTYPE_BF16, None, None, 0, ys[0].data_ptr(), _capi.DTYPE_BF16, T, st)
                    assert rc == 0, _capi.last_error()
                return
            cur = torch.cuda.current_stream(dev)
            for ln in lanes:
                ln.wait_stream(cur)
            for i, m in enumerate(layers):
                ln = lanes[i % nstreams]
                rc = L.prichs_moe_forward(m._h, x.data_ptr(), _capi.DTYPE_BF16, None, None, 0, ys[i % nstreams].data_ptr(),
                                          _capi.DTYPE_BF16, T, ln.cuda_stream)
                assert rc == 0, _capi.last_error()
            for ln in lanes:
                cur.wait_stream(ln)

        for _ in range(max(warmup, 3)):
            step()
        torch.cuda.synchronize(dev)
        # the small launches of a step are replayed as one CUDA graph (the forward neither allocates nor synchronises,
        # so it can be captured)
        graph, launches_per_step = None, None
        if use_graph:
            side = torch.cuda.Stream(dev)
            with torch.cuda.stream(side):
                graph = torch.cuda.CUDAGraph()
                l0 = L.prichs_kernel_launches()
                with torch.cuda.graph(graph, stream=side):
                    step()
                launches_per_step = int(L.prichs_kernel_launches() - l0)
            torch.cuda.synchronize(dev)
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize(dev)
        with ClockSampler(dev.index) as clocks:
            l0 = L.prichs_kernel_launches()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                graph.replay() if graph is not None else step()
            e1.record()
            torch.cuda.synchronize(dev)
            launches = int(L.prichs_kernel_launches() - l0) if graph is None else launches_per_step * steps
        ms = e0.elapsed_time(e1) / steps
        gbs = wbytes / (ms * 1e-3) / 1e9
        results.append({"streams": nstreams, "ms_per_step": ms, "us_per_layer": ms * 1e3 / n_layers, "weight_GBps": gbs,
                        "frac_hbm": gbs / peaks["hbm"], "gpu_launches": launches, "cuda_graph": graph is not None,
                        "clocks": clocks.summary(), "tokens_per_s": T * n_layers / (ms * 1e-3), "weight_bytes_per_step": wbytes})
    for m in layers:
        m.close()
    return results


def run_decode(args):
    """`--config 2`: the decode configuration as a bench line of its own."""
    import torch
    torch.cuda.set_device(0)
    peaks = measured_peaks()
    r = decode_measure(args.layers, args.steps, args.warmup, [max(1, args.streams)], use_graph=not args.no_graph,
                       route_kernel=args.route_kernel, pdl=args.pdl, gemm_kernel=args.gemm_kernel)[0]
    line = {"metric": "MoE-layer tokens/sec", "value": r["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"config 2: decode, {args.layers} independent MoE layers (seed 2+layer), T=64 tokens each, bf16; "
                                   f"a step is all layer forwards, spread over {r['streams']} stream(s)", "layers": args.layers,
                       "l2": f"the step streams {r['weight_bytes_per_step'] / 1e6:.0f} MB of weights, far more than the 126 MB L2"},
            "decode": {k: r[k] for k in ("ms_per_step", "us_per_layer", "weight_GBps", "frac_hbm")},
            "roofline": {"kernel": "whole decode step (weight streaming through the grouped GEMMs)", "bound": "hbm",
                         "achieved": r["weight_GBps"], "peak": peaks["hbm"], "unit": "GB/s", "frac": r["frac_hbm"], "traffic": None},
            "gpu_launches": r["gpu_launches"], "cuda_graph": r["cuda_graph"], "streams": r["streams"], "clocks": r["clocks"]}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of this run's own result (profiling)")
    ap.add_argument("--ep-waves", type=int, default=0, help="expert-parallel token waves (0 = library default)")
    ap.add_argument("--tokens", type=int, default=0,
                    help="override T (profiling of a small case only; the line is then not the baseline's config)")
    ap.add_argument("--config", type=int, default=0, choices=[0, 1, 2, 3, 4],
                    help="baseline config to run (0 = 1 for one GPU, 3 for several); 2 = decode, 4 = Zipf-skewed routing")
    ap.add_argument("--layers", type=int, default=24, help="layers of the decode config")
    ap.add_argument("--no-graph", action="store_true", help="decode config: plain launches instead of a CUDA graph")
    ap.add_argument("--streams", type=int, default=8, help="decode config: streams the independent layers are spread over")
    ap.add_argument("--no-decode", action="store_true", help="one GPU: skip the decode object (config 2) after the headline run")
    ap.add_argument("--no-skew", action="store_true", help="several GPUs: skip the skewed-routing object (config 4) after the headline run")
    ap.add_argument("--no-same-t", action="store_true", help="several GPUs: skip rank 0's one-GPU run at the same T")
    ap.add_argument("--ep-nccl-barriers", type=int, default=0, choices=[0, 1], help="1 = NCCL all-gathers as barriers instead of readiness flags")
    ap.add_argument("--ep-dispatch-kernel", type=int, default=0, choices=[0, 1], help="0 = bulk-copy dispatch, 1 = warp-per-token dispatch")
    ap.add_argument("--ep-shared-copy-sms", type=int, default=0, choices=[0, 1], help="1 = dispatch / combine may share SMs with GEMM CTAs")
    ap.add_argument("--ep-reserve-sms", type=int, default=0, help="SMs the expert-parallel GEMM launches leave free (0 = default, -1 = none)")
    ap.add_argument("--route-kernel", type=int, default=0, choices=[0, 1, 2],
                    help="single GPU: 0 = library default, 1 = single-pass routing kernel, 2 = router / scan / dispatch launches")
    ap.add_argument("--gemm-kernel", type=int, default=0, choices=[0, 1, 2], help="0 = CTA-pair kernel (small batches: one-CTA kernel), 1 = one-CTA kernel, 2 = as 0 with 128-column down tiles for small batches")
    ap.add_argument("--pdl", type=int, default=0, choices=[0, 1, 2], help="programmatic dependent launch: 0/1 = on (default), 2 = off")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.config == 2:
        return run_decode(args)

    import torch
    from prichs_b200 import MoELayer, _capi, synth

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    n_gpus = args.gpus
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {n_gpus}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    peaks = measured_peaks()
    L = _capi.lib()

    if n_gpus == 1:
        seed, T = 1, (args.tokens or 16384)
        ws = synth.layer_weights(seed, D, F, E, bf16=True)
        bias = synth.router_bias(seed, E, -0.1, 0.1)
        layer = MoELayer.from_weights(ws, K, max_tokens=T, device=local_rank, route_kernel=args.route_kernel,
                                      gemm_kernel=args.gemm_kernel, pdl=args.pdl)
    else:
        from prichs_b200 import ep
        skew = args.config == 4
        seed, T = (4 if skew else 3), (args.tokens or 32768)
        ws = synth.layer_weights(seed, D, F, E, bf16=True)
        if skew:
            ws[0], zipf_sigma, zipf_share, zipf_target = zipf_router(ws[0], seed)
        bias = np.zeros(E, np.float32)
        same_T = None
        if rank == 0 and not args.no_same_t:
            # like-for-like baseline of the scaling figure: the same T tokens on ONE GPU with all eight experts local
            # (the driver's own efficiency divides by the config-1 value, measured at T = 16384)
            solo = MoELayer.from_weights(ws, K, max_tokens=T, device=local_rank)
            solo.router_bias = bias
            xsolo = [torch.from_numpy(synth.to_bf16_bits(synth.tokens(seed * 1000 + 7919 * i, T, D, bf16=True)).view(np.int16)).view(torch.bfloat16).to(dev)
                     for i in range(2)]
            ysolo = torch.empty_like(xsolo[0])
            for i in range(5):
                solo.forward(xsolo[i % 2], out=ysolo)
            torch.cuda.synchronize(dev)
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for i in range(30):
                solo.forward(xsolo[i % 2], out=ysolo)
            s1.record()
            torch.cuda.synchronize(dev)
            solo.sync_status()
            ms1 = s0.elapsed_time(s1) / 30
            same_T = {"tokens": T, "ms_per_step": ms1, "tokens_per_s": T / (ms1 * 1e-3), "steps": 30}
            solo.close()
            del solo, xsolo, ysolo
            torch.cuda.empty_cache()
        layer = MoELayer.from_weights(ws, K, max_tokens=T, device=local_rank, ep_world=world, ep_rank=rank, ep_waves=args.ep_waves,
                                      ep_nccl_barriers=args.ep_nccl_barriers, ep_reserve_sms=args.ep_reserve_sms,
                                      ep_dispatch_kernel=args.ep_dispatch_kernel, ep_shared_copy_sms=args.ep_shared_copy_sms)
        for e in range(E):  # only the experts this rank owns are uploaded
            if e // (E // world) != rank:
                layer.experts[e].gate_proj = layer.experts[e].up_proj = layer.experts[e].down_proj = None
        ep.connect(layer, dist, max_tokens=T)
    layer.router_bias = bias

    nbatch = 4 if n_gpus == 1 else 2
    xseed = seed if n_gpus == 1 else seed * 1000 + rank  # config 3: per-rank token seed 3000 + rank
    xs_host = [synth.tokens(xseed + 7919 * i, T, D, bf16=True) for i in range(nbatch)]
    xs = [torch.from_numpy(synth.to_bf16_bits(x).view(np.int16)).view(torch.bfloat16).to(dev) for x in xs_host]
    y = torch.empty_like(xs[0])
    stream = torch.cuda.current_stream(dev)

    def step(i):
        layer.forward(xs[i % nbatch], out=y)

    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize(dev)
    layer.sync_status()

    # ---- device-resident timing (value) + per-stage times ---------------------------------------------
    with ClockSampler(local_rank) as clocks:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
        launches0 = L.prichs_kernel_launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(args.steps):
            step(i)
        e1.record(stream)
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        launches = int(L.prichs_kernel_launches() - launches0)
        ms_total = e0.elapsed_time(e1)
        # stage breakdown: the library records CUDA events on the launching stream between its kernels
        stage, timeline = None, None
        if world > 1:
            import ctypes as C
            L.prichs_moe_enable_timing(layer._h, 1)
            for i in range(3):
                step(i)
            tlb = (C.c_float * 34)()
            if L.prichs_moe_get_ep_timeline(layer._h, tlb, 34) == 0:
                v = [round(float(x), 4) for x in tlb]
                nw = args.ep_waves or max(1, min(4, T // 8192))
                timeline = {"ms_since_router": {"shared_gate_up": v[0], "shared_down": v[1]},
                            "marks": ["scan", "plan", "dispatched", "rows_landed", "gate_up", "down", "outputs_ready", "combined"],
                            "waves": [v[2 + 8 * w: 10 + 8 * w] for w in range(nw)]}
            L.prichs_moe_enable_timing(layer._h, 0)
            torch.cuda.synchronize(dev)
        if world == 1:  # (the expert-parallel forward overlaps its kernels on several streams: no per-stage split)
            L.prichs_moe_enable_timing(layer._h, 1)
            stage = np.zeros(6, np.float64)
            nstage = min(args.steps, 20)
            import ctypes as C
            buf = (C.c_float * 6)()
            for i in range(nstage):
                # the measured forward is the last of a back-to-back group, so that the GPU is as busy (and as
                # power-limited) around it as in the timed region above
                for r in range(5):
                    step(5 * i + r)
                L.prichs_moe_get_stage_ms(layer._h, buf)
                stage += np.array(list(buf), np.float64)
            stage /= nstage
            L.prichs_moe_enable_timing(layer._h, 0)

        # ---- end to end through the host-buffer entry point ------------------------------------------
        xh = [torch.from_numpy(x).pin_memory() for x in xs_host[:2]]
        yh = torch.empty((T, D), dtype=torch.float32).pin_memory()
        for i in range(3):
            layer.forward(xh[i % 2].numpy(), out=yh.numpy())
        t0 = time.perf_counter()
        e2e_steps = max(5, min(args.steps, 30))
        for i in range(e2e_steps):
            layer.forward(xh[i % 2].numpy(), out=yh.numpy())
        e2e_dt = time.perf_counter() - t0
    layer.sync_status()

    ms_step = ms_total / args.steps
    # host link rate each rank saw in its own end-to-end loop (bytes of one direction / its wall time)
    my_gbs = T * D * 4 * e2e_steps / e2e_dt / 1e9
    rank_gbs = [my_gbs]
    if world > 1:
        g = torch.tensor([my_gbs], device=dev, dtype=torch.float64)
        allg = [torch.zeros_like(g) for _ in range(world)]
        dist.all_gather(allg, g)
        rank_gbs = [float(v[0]) for v in allg]
        t = torch.tensor([ms_step, e2e_dt], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step, e2e_dt = float(t[0]), float(t[1])
    tokens = T * n_gpus
    value = tokens / (ms_step * 1e-3)

    # rows the GEMMs of THIS rank processed: its T shared rows plus the routed rows its experts received
    rows = T * (1 + K)
    if world > 1:
        import ctypes as C2
        rr = C2.c_int64()
        L.prichs_moe_ep_recv_rows(layer._h, C2.byref(rr))
        rows = T + int(rr.value)
    gu_flops = rows * 4 * D * F
    if stage is not None:
        names = ["router", "scan", "dispatch", "gate_up_gemm", "down_gemm", "combine"]
        stage_ms = dict(zip(names, [float(v) for v in stage]))
        gu_tf = gu_flops / (stage_ms["gate_up_gemm"] * 1e-3) / 1e12
        dn_tf = rows * 2 * D * F / (stage_ms["down_gemm"] * 1e-3) / 1e12
        single_pass = stage_ms["dispatch"] < 0.008  # one kernel routed, placed and dispatched: no scan / dispatch stages
        if single_pass:
            routing = {"route_dispatch": {"ms": stage_ms["router"], "GB/s": T * (ROUTER_BYTES + DISPATCH_BYTES) / stage_ms["router"] / 1e6,
                                          "bound": "hbm", "kernel": "route_dispatch_kernel (router + prefix + dispatch in one pass)",
                                          "algorithmic_bytes_per_token": ROUTER_BYTES + DISPATCH_BYTES,
                                          "bytes_moved_per_token": ROUTER_BYTES + DISPATCH_BYTES - D * 2}}
        else:
            routing = {"router": {"ms": stage_ms["router"], "GB/s": T * ROUTER_BYTES / stage_ms["router"] / 1e6, "bound": "hbm"},
                       "scan": {"ms": stage_ms["scan"]},
                       "dispatch": {"ms": stage_ms["dispatch"], "GB/s": T * DISPATCH_BYTES / stage_ms["dispatch"] / 1e6, "bound": "hbm"}}
        stages = {
            **routing,
            "gate_up_gemm": {"ms": stage_ms["gate_up_gemm"], "TFLOP/s": gu_tf, "bound": "tensor"},
            "down_gemm": {"ms": stage_ms["down_gemm"], "TFLOP/s": dn_tf, "bound": "tensor"},
            "combine": {"ms": stage_ms["combine"], "GB/s": T * COMBINE_BYTES_NORES / stage_ms["combine"] / 1e6, "bound": "hbm"},
        }
        for s in stages.values():
            if "GB/s" in s:
                s["frac"] = s["GB/s"] / peaks["hbm"]
            if "TFLOP/s" in s:
                s["frac"] = s["TFLOP/s"] / peaks["tf"]
        roofline = {"kernel": "expert_gemm_pair_kernel<EPI_SWIGLU> (gate|up GEMM + SwiGLU, shared + 8 routed experts in one launch)",
                    "bound": "tensor", "achieved": gu_tf, "peak": peaks["tf"], "unit": "TFLOP/s", "frac": gu_tf / peaks["tf"],
                    # dram__bytes_read + dram__bytes_write of one launch at this size, from the one-pass ncu capture
                    # summarised in profiles/traffic_config1_full_size.md (bytes); only valid for config 1
                    "traffic": 328.0e6 if not args.tokens else None,
                    "peak_source": f"{peaks['source']} bf16_tflops (burst; the timed region lasts well under a second)",
                    "frac_of_sustained_peak": gu_tf / peaks["tf_sustained"] if peaks["tf_sustained"] else None,
                    "algorithmic_flops_per_launch": gu_flops}
    else:
        # Expert-parallel step: the GEMM launches of the waves overlap the exchange of other waves on several
        # streams, so one kernel cannot be timed alone; the figure is this rank's GEMM flops over the WHOLE step.
        stages = None
        tf = rows * 6 * D * F / (ms_step * 1e-3) / 1e12
        roofline = {"kernel": "expert_gemm_pair_kernel (all GEMM launches of one rank) over the whole expert-parallel step",
                    "bound": "tensor", "achieved": tf, "peak": peaks["tf"], "unit": "TFLOP/s", "frac": tf / peaks["tf"],
                    "traffic": None, "peak_source": f"{peaks['source']} bf16_tflops (burst)",
                    "algorithmic_flops_per_launch": rows * 6 * D * F}

    line = {
        "metric": "MoE-layer tokens/sec", "value": value, "unit": "tokens/s", "n_gpus": n_gpus, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(n_gpus) if not args.tokens else {"workload": f"NOT the baseline config: T={T} override for profiling"},
        "e2e": {"value": tokens * e2e_steps / e2e_dt, "unit": "tokens/s", "h2d_bytes_per_step": T * D * 4 * n_gpus,
                "d2h_bytes_per_step": T * D * 4 * n_gpus, "bytes_per_rank_and_direction": T * D * 4, "steps": e2e_steps,
                "h2d_gbs": [round(v, 2) for v in rank_gbs], "d2h_gbs": [round(v, 2) for v in rank_gbs],
                "api": "MoELayer.forward(numpy fp32 [T,d]) -> prichs_moe_forward_host, pinned host buffers"},
        "gpu_launches": launches, "roofline": roofline, "stages": stages, "ep_timeline": timeline,
        "layer_tflops": tokens * FLOPS_PER_TOKEN / (ms_step * 1e-3) / 1e12,
        "roofline_sum": roofline_sum(T, rows, ms_step, peaks, world),
        "clocks": clocks.summary(),
    }
    if world > 1 and rank == 0 and same_T is not None:
        same_T["efficiency_vs_same_T"] = value / (n_gpus * same_T["tokens_per_s"])
        line["single_gpu_same_T"] = same_T
    # ---- parity of this run's own result against the CPU oracle (every rank; outside the timed regions) -------------
    if not args.no_parity:
        par = parity_check(layer, ws, bias, xs_host[0], xs[0], 4096 if rank == 0 else 512, 1234 + rank)
        if world > 1:
            t = torch.tensor([0.0 if par["routing_bit_exact"] else 1.0, par["max_rel"], par["logits_max_abs_err"]], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            n = torch.tensor([par["tokens_checked"], par["tokens_routed"], par["near_tie_tokens_skipped"]], device=dev, dtype=torch.int64)
            dist.all_reduce(n)
            par = {"routing_bit_exact": float(t[0]) == 0.0, "logits_max_abs_err": float(t[2]), "max_rel": float(t[1]),
                   "tokens_checked": int(n[0]), "tokens_routed": int(n[1]), "near_tie_tokens_skipped": int(n[2]), "ranks": world}
        par["tolerance"] = 2e-2
        par["ok"] = bool(par["routing_bit_exact"] and par["max_rel"] <= 2e-2 and par["logits_max_abs_err"] <= 1e-3)
        line["parity"] = par
    if world > 1 and args.config == 4:
        # one aux-loss-free bias step from the global counts of the last forward: b_i += gamma (k/E - count_i/total);
        # gamma = 1e-3 on load fractions equals a count-form step of gamma / (T * world) per token of deviation
        gcounts = torch.tensor(layer.last_counts(), device=dev)
        dist.all_reduce(gcounts)
        rr2 = torch.tensor([rows - T], device=dev, dtype=torch.int64)
        allrows = [torch.zeros_like(rr2) for _ in range(world)]
        dist.all_gather(allrows, rr2)
        layer.update_bias_from_last(1e-3, total_tokens=T * world)
        gc = gcounts.cpu().numpy().astype(np.float64)
        line["skew"] = {"zipf_alpha": ZIPF_ALPHA, "sigma": [float(v) for v in zipf_sigma],
                        "top1_share_sample": [float(v) for v in zipf_share], "top1_share_target": [float(v) for v in zipf_target],
                        "global_counts": [int(v) for v in gc], "imbalance_max_over_mean": float(gc.max() / gc.mean()),
                        "recv_rows_per_gpu": [int(t.item()) for t in allrows],
                        "bias_after_step": [float(v) for v in layer.router_bias], "gamma": 1e-3}
        line["config"]["workload"] = line["config"]["workload"].replace("config 3", "config 4 (Zipf(1.2)-skewed router, seed 4)")
    if world > 1 and args.config != 4 and not args.no_skew:
        layer.close()
        del xs, y
        torch.cuda.empty_cache()
        line["skew"] = skew_measure(args, dist, dev, rank, world, local_rank)
    if n_gpus == 1 and not args.no_decode and not args.tokens:
        # config 2 (decode) after the headline measurement, as a short object of the same line: 8 streams and 1 stream
        layer.close()
        del xs, y
        torch.cuda.empty_cache()
        dec = decode_measure(24, 30, 5, [8, 1])
        line["decode"] = {"workload": "config 2: 24 independent MoE layers (seed 2+layer), T=64 tokens each, bf16, CUDA-graph replay; "
                                      "weight-streaming GB/s = weight bytes of a step / time",
                          "ms_per_step": dec[0]["ms_per_step"], "weight_GBps": dec[0]["weight_GBps"], "frac_hbm": dec[0]["frac_hbm"],
                          "streams": dec[0]["streams"], "one_stream_ms": dec[1]["ms_per_step"], "one_stream_frac_hbm": dec[1]["frac_hbm"],
                          "weight_bytes_per_step": dec[0]["weight_bytes_per_step"], "steps": 30,
                          "gpu_launches_per_step": dec[0]["gpu_launches"] // 30}
    if rank == 0:
        if not args.no_cpu_baseline and n_gpus == 1:
            line["cpu_baseline"] = cpu_baseline(ws, bias, xs_host[0])
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    if "parity" in line and not line["parity"]["ok"]:
        raise SystemExit("parity check against the CPU oracle failed: " + json.dumps(line["parity"]))
    if "skew" in line and not line["skew"]["parity"]["ok"]:
        raise SystemExit("parity check of the skewed configuration failed: " + json.dumps(line["skew"]["parity"]))


if __name__ == "__main__":
    main()
