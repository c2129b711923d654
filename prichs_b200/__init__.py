"""prichs_b200 -- B200 (sm_100a) implementation of the PRICHS MoE-layer forward path.

The product is the C-ABI library libprichs_moe.so (include/prichs_moe.h, sources under prichs_b200/csrc).
This package is the thin host side above it: `MoELayer` mirrors the reference's
crates/prichs-model/src/moe.rs API, `synth` makes the seeded synthetic tensors the benchmark and tests use.
There is no CPU fallback: without the built library or without a CUDA device the layer raises.
"""
from .moe import Expert, ExpertForwardStash, MoELayer, MoEStash, PrichsError  # noqa: F401

__all__ = ["Expert", "ExpertForwardStash", "MoELayer", "MoEStash", "PrichsError"]
