"""The tiny Qwen2-shaped model behind tests/golden/engine_hf.npz: shapes, seeds and weight construction shared by the
script that writes the fixture (make_engine_golden.py: a random-init Hugging Face Qwen2 whose block linears are
replaced by reference-decoded codebook matrices, run on the CPU in fp32) and by the GPU test that rebuilds the same
model in the packed format.  Everything is derived from seeds, so the fixture itself holds only tokens and logits.

The reference pins its own engine the same way (tests/test_runtime.py:18-89 of the reference)."""
from __future__ import annotations

import numpy as np

from oracle import cbl_oracle as orc

H, I, NH, NKV, HD, V, NL, MAX_LEN, THETA, EPS = 512, 1024, 4, 2, 128, 1024, 2, 64, 1e6, 1e-6
LINEARS = {"q": (NH * HD, H), "k": (NKV * HD, H), "v": (NKV * HD, H), "o": (H, NH * HD), "gate": (I, H), "up": (I, H), "down": (H, I)}
TOKENS = [5, 17, 300, 2, 911, 64, 7, 1000, 3, 512, 88, 41, 650, 9]


def matrix(layer: int, name: str, books: int = 1, M: int = 1) -> dict:
    """The packed matrix of one block linear (oracle.synth_matrix: seeded tags, N(0,1) fp16 book, row scales 0.01-0.03)."""
    R, C = LINEARS[name]
    return orc.synth_matrix(R, C, seed=1000 * layer + sorted(LINEARS).index(name) + 77, books=books, M=M)


def small_tensors() -> dict:
    """Norm weights (1 +- 0.1), q/k/v biases (~0.1), embedding and head (~0.05), rounded to fp16."""
    rng = np.random.RandomState(20240)
    f16 = lambda a: a.astype(np.float16)                                  # noqa: E731
    out = {"embed": f16(rng.randn(V, H) * 0.05), "head": f16(rng.randn(V, H) * 0.05), "final_norm": f16(1 + 0.1 * rng.randn(H))}
    for li in range(NL):
        out[f"ln1_{li}"], out[f"ln2_{li}"] = f16(1 + 0.1 * rng.randn(H)), f16(1 + 0.1 * rng.randn(H))
        for n in "qkv":
            out[f"b{n}_{li}"] = f16(0.1 * rng.randn(LINEARS[n][0]))
    return out
