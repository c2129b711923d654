"""Generates tests/golden/moe_small.npz: the C++ oracle's outputs for the integer-hashed grid inputs of
tests/_util.py:golden_small_inputs (the inputs are regenerated, not stored).

The reference (Rust) cannot be built or imported on this image, so these vectors are a regression pin of the
oracle, produced by `python tests/golden/make_golden.py` from the repository root. The closed-form
known-answer cases derived from the reference's own fixture constants live in tests/test_oracle.py.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import oracle as O  # noqa: E402
from _util import golden_small_inputs  # noqa: E402


def main():
    g = golden_small_inputs()
    r = O.moe_forward_train(g["ws"], g["bias"], g["top_k"], g["x"], concept_bias=g["concept_bias"])
    np.savez_compressed(os.path.join(os.path.dirname(__file__), "moe_small.npz"), out=r["out"], logits=r["logits"],
                        selected=r["selected"], gating=r["gating"], counts=r["counts"], shared_out=r["shared_out"])
    print("wrote moe_small.npz", {k2: v.shape for k2, v in r.items()}, r["counts"])


if __name__ == "__main__":
    main()
