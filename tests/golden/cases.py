"""Seeded input generators shared by the golden-fixture script and the tests.

Inputs follow the synthetic distribution of the build's benchmark configs:
K ~ N(0,1) with four fixed outlier channels per head scaled x8, V ~ N(0,1),
q ~ N(0,1), all rounded to fp16.  `slots` is an identity map or a seeded
permutation of whole pages plus a ragged tail.
"""
from __future__ import annotations

import numpy as np

OUTLIER_CHANNELS = (3, 17, 64, 101)

CASES = [
    # small, ragged last page, identity slots
    dict(name="small_h2", n=37, h=2, nq=3, seed=1, permute=False, store_inputs=True),
    # four kv heads, pages handed out in a seeded order
    dict(name="perm_h4", n=50, h=4, nq=2, seed=2, permute=True, store_inputs=True),
    # one full page exactly
    dict(name="page_h8", n=16, h=8, nq=1, seed=3, permute=False, store_inputs=True),
    # the CPU-plumbing config: 1143 tokens, 2 kv heads, 16 q heads (GQA 8:1) -> 8 query rows
    dict(name="cfg1_1143", n=1143, h=2, nq=8, seed=0, permute=False, store_inputs=False),
]


def make_kv(rng: np.random.Generator, n: int, h: int, d: int = 128):
    key = rng.standard_normal((n, h, d)).astype(np.float32)
    key[:, :, list(OUTLIER_CHANNELS)] *= 8.0
    value = rng.standard_normal((n, h, d)).astype(np.float32)
    return key.astype(np.float16), value.astype(np.float16)


def make_slots(rng: np.random.Generator, n: int, permute: bool, block: int = 16,
               extra_pages: int = 0) -> np.ndarray:
    pages = (n + block - 1) // block
    order = np.arange(pages + extra_pages)
    if permute:
        order = rng.permutation(pages + extra_pages)
    t = np.arange(n)
    return (order[t // block] * block + t % block).astype(np.int32)


def make_inputs(case: dict):
    rng = np.random.default_rng(case["seed"])
    key, value = make_kv(rng, case["n"], case["h"])
    query = rng.standard_normal((case["nq"], case["h"], 128)).astype(np.float16)
    slots = make_slots(rng, case["n"], case["permute"], extra_pages=1 if case["permute"] else 0)
    return key, value, query, slots
