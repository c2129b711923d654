"""Seeded synthetic tensors for the benchmark and the tests (no dataset is involved anywhere).

Counter-based generator, vectorised in numpy: u = splitmix64(key + idx), key = splitmix64(splitmix64(seed) + tensor_id) with the low 32 bits cleared, gives
two 24-bit uniforms per element; normals follow the reference's own Box-Muller form
(crates/prichs-core/src/tensor.rs:57-59): z = sqrt(-2 ln max(u1, 1e-7)) * cos(2 pi u2).
tensor_id order: 0 = x, 1 = router, 2..4 = shared gate/up/down, 5 + 3e + {0,1,2} = expert e gate/up/down,
1000 = router bias.
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = (z + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def _stream(seed: int, tensor_id: int, lo: int, hi: int) -> np.ndarray:
    """64 random bits for elements lo..hi-1 of tensor `tensor_id` under `seed`."""
    with np.errstate(over="ignore"):
        key = _splitmix64(_splitmix64(np.array([seed], np.uint64)) + np.uint64(tensor_id))[0]
        key = key & np.uint64(0xFFFFFFFF00000000)  # element index occupies the low 32 bits
        return _splitmix64(key + np.arange(lo, hi, dtype=np.uint64))


def normal(seed: int, tensor_id: int, shape, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    n = int(np.prod(shape))
    out = np.empty(n, np.float32)
    step = 1 << 22
    for lo in range(0, n, step):
        m = min(step, n - lo)
        b = _stream(seed, tensor_id, lo, lo + m)
        u1 = ((b >> np.uint64(40)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / (1 << 24))
        u2 = ((b >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.float32) * np.float32(1.0 / (1 << 24))
        u1 = np.maximum(u1, np.float32(1e-7))
        z = np.sqrt(np.float32(-2.0) * np.log(u1)) * np.cos(np.float32(2.0 * np.pi) * u2)
        out[lo:lo + m] = np.float32(mean) + z.astype(np.float32) * np.float32(std)
    return out.reshape(shape)


def uniform(seed: int, tensor_id: int, shape, lo: float, hi: float) -> np.ndarray:
    n = int(np.prod(shape))
    b = _stream(seed, tensor_id, 0, n)
    u = (b >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / (1 << 24))
    return (np.float32(lo) + u * np.float32(hi - lo)).astype(np.float32).reshape(shape)


def round_bf16(a: np.ndarray) -> np.ndarray:
    """Round fp32 values to the nearest bf16 (ties to even), returned widened to fp32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = a.view(np.uint32).astype(np.uint64)
    r = ((b + np.uint64(0x7FFF) + ((b >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)) << np.uint64(16)
    return r.astype(np.uint32).view(np.float32).reshape(a.shape)


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns (uint16), round to nearest even."""
    return (round_bf16(a).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


def layer_weights(seed: int, d: int, f: int, E: int, std: float = 0.02, bf16: bool = False, threads: int = 0):
    """Weights of one MoE layer in the reference's parameter order (crates/prichs-model/src/model.rs:353-361):
    [router [d,E], shared gate [d,f], up [d,f], down [f,d], expert0 gate, up, down, ...], all ~ N(0, std).
    The tensors are independent streams of the counter-based generator, so they are generated on a thread pool
    (numpy releases the interpreter lock inside its array operations); the values do not depend on `threads`."""
    import os
    from concurrent.futures import ThreadPoolExecutor
    jobs = [(1, (d, E))]
    tid = 2
    for _ in range(1 + E):
        jobs += [(tid, (d, f)), (tid + 1, (d, f)), (tid + 2, (f, d))]
        tid += 3

    def make(job):
        w = normal(seed, job[0], job[1], 0.0, std)
        return round_bf16(w) if bf16 else w

    n = threads or min(len(jobs), os.cpu_count() or 1)
    if n <= 1:
        return [make(j) for j in jobs]
    with ThreadPoolExecutor(max_workers=n) as pool:
        return list(pool.map(make, jobs))


def tokens(seed: int, T: int, d: int, bf16: bool = False) -> np.ndarray:
    x = normal(seed, 0, (T, d), 0.0, 1.0)
    return round_bf16(x) if bf16 else x


def router_bias(seed: int, E: int, lo: float, hi: float) -> np.ndarray:
    return uniform(seed, 1000, (E,), lo, hi)
