"""Shared builders for test inputs: KAT decoding and the seeded synthetic generator.

Every config draws weights and activations once from numpy's PCG64
(``default_rng(seed).standard_normal`` scaled, cast to f32) and hands the same raw
buffers to the CPU oracle and to the CUDA path.
"""
from __future__ import annotations

import numpy as np

from oracle import kbref

TERNARY, QUATERNARY = kbref.TERNARY, kbref.QUATERNARY


def kind_id(name: str) -> int:
    return TERNARY if name.startswith("tern") else QUATERNARY


def rule(expr: str, count: int) -> np.ndarray:
    """Evaluate one of the reference tests' arithmetic generators over i = 0..count-1."""
    i = np.arange(count, dtype=np.int64)
    table = {
        "(i%3)-1": (i % 3).astype(np.float32) - np.float32(1.0),
        "(i%5)*0.2": (i % 5).astype(np.float32) * np.float32(0.2),
        "(i%7)-3": (i % 7).astype(np.float32) - np.float32(3.0),
        "(i%5)*0.1": (i % 5).astype(np.float32) * np.float32(0.1),
        "(i%4)*2-3": (i % 4).astype(np.float32) * np.float32(2.0) - np.float32(3.0),
        "i*0.1": i.astype(np.float32) * np.float32(0.1),
    }
    return table[expr].astype(np.float32)


def packed_from_kat(case: dict) -> np.ndarray:
    """Wire-format bytes of a 'matmul_packed' KAT (given as bytes, trits or quat codes)."""
    if "packed" in case:
        return np.array(case["packed"], np.uint8)
    if "trits" in case:
        return np.concatenate([kbref.pack_ternary(np.array(r, np.int8)) for r in case["trits"]])
    rows = []
    for r in case["codes"]:
        codes = np.zeros(((len(r) + 3) // 4) * 4, np.uint8)  # tail slots stay code 0
        codes[: len(r)] = r
        rows.append(kbref.pack_quaternary(codes))
    return np.concatenate(rows)


def gaussian(seed: int, shape, sigma: float) -> np.ndarray:
    return (np.random.default_rng(seed).standard_normal(shape) * sigma).astype(np.float32)


def make_weights(kind: int, quantiser: str, w: np.ndarray, threshold: float = 0.3):
    """f32 [M,K] -> reference wire format (packed, scales) through the oracle's packers."""
    m, k = w.shape
    if kind == TERNARY:
        if quantiser == "absmean":
            return kbref.pack_weights_ternary_absmean(w, m, k)
        return kbref.pack_weights_ternary(w, m, k, threshold)
    return kbref.pack_weights_quaternary(w, m, k)


def integer_activations(seed: int, n: int, k: int) -> np.ndarray:
    """Integer-valued f32 activations whose rows all have max|x| = 127, so the per-token
    scale is exactly 1.0 and the int8 quantiser is the identity."""
    rng = np.random.default_rng(seed)
    x = rng.integers(-127, 128, size=(n, k)).astype(np.float32)
    x[:, 0] = 127.0
    return x
