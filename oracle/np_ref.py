"""Second, independent restatement of the path in numpy (test infrastructure only).

It exists to cross-check ``kbref.c``: two restatements written separately that agree
bit-for-bit are much less likely to share a misreading of the reference.  The R-level
loops are pure Python over K (small cases only); the Q level is vectorised.

Reference locations restated here:
  crates/kore-btes/src/encoder.rs:50-110           codecs
  crates/kore-kernels/src/cpu_ternary_matmul.rs:105-124, 198-240
  crates/kore-kernels/src/cpu_quat_matmul.rs:74-108, 174-214
"""
from __future__ import annotations

import numpy as np

f32 = np.float32
QUAT_VALUES = np.array([-3.0, -1.0, 1.0, 3.0], dtype=f32)


def ternary_lut() -> np.ndarray:
    """[256,5] int8: byte -> five trits, trit 0 least significant, >=243 -> zeros."""
    lut = np.zeros((256, 5), np.int8)
    for b in range(243):
        v = b
        for j in range(5):
            lut[b, j] = (v % 3) - 1
            v //= 3
    return lut


def decode_ternary(packed: np.ndarray, m: int, k: int) -> np.ndarray:
    kp = (k + 4) // 5
    rows = np.asarray(packed, np.uint8)[: m * kp].reshape(m, kp)
    return ternary_lut()[rows].reshape(m, kp * 5)[:, :k]


def decode_quaternary_codes(packed: np.ndarray, m: int, k: int) -> np.ndarray:
    kp = (k + 3) // 4
    rows = np.asarray(packed, np.uint8)[: m * kp].reshape(m, kp)
    codes = np.stack([(rows >> (2 * i)) & 3 for i in range(4)], axis=-1).reshape(m, kp * 4)
    return codes[:, :k]


def encode_ternary(trits: np.ndarray) -> np.ndarray:
    """[m,k] int8 trits -> [m,ceil(k/5)] base-243 bytes (pad with zero trits)."""
    m, k = trits.shape
    kp = (k + 4) // 5
    pad = np.zeros((m, kp * 5), np.int64)
    pad[:, :k] = trits
    digits = (pad + 1).reshape(m, kp, 5)
    return (digits * np.array([1, 3, 9, 27, 81])).sum(-1).astype(np.uint8)


def pack_weights_ternary(w: np.ndarray, thr: float):
    w = np.asarray(w, f32)
    am = np.abs(w).max(axis=1)
    scale = np.where(am < f32(1e-8), f32(1.0), am).astype(f32)
    nrm = (w / scale[:, None]).astype(f32)
    tr = np.where(nrm > f32(thr), 1, np.where(nrm < -f32(thr), -1, 0)).astype(np.int8)
    return encode_ternary(tr).ravel(), scale


def pack_weights_quaternary(w: np.ndarray):
    w = np.asarray(w, f32)
    m, k = w.shape
    am = np.abs(w).max(axis=1)
    scale = np.where(am < f32(1e-8), f32(1.0), (am / f32(3.0)).astype(f32)).astype(f32)
    nrm = (w / scale[:, None]).astype(f32)
    code = np.where(nrm < -2, 0, np.where(nrm < 0, 1, np.where(nrm < 2, 2, 3))).astype(np.uint8)
    kp = (k + 3) // 4
    pad = np.zeros((m, kp * 4), np.uint8)
    pad[:, :k] = code
    g = pad.reshape(m, kp, 4)
    return (g[..., 0] | (g[..., 1] << 2) | (g[..., 2] << 4) | (g[..., 3] << 6)).astype(np.uint8).ravel(), scale


def absmean_ternarise(w: np.ndarray):
    """Benchmark-specified: s = mean|W| (f64, row sums then sum of rows), rne, clip."""
    w = np.asarray(w, f32)
    total = 0.0
    for r in range(w.shape[0]):
        rs = 0.0
        for v in np.abs(w[r]).astype(np.float64):
            rs += float(v)
        total += rs
    s = f32(total / float(w.size))
    if s < f32(1e-8):
        s = f32(1.0)
    q = np.rint((w / s).astype(f32))
    return np.clip(q, -1, 1).astype(np.int8), s


def ternary_matmul(packed, scales, b, m, n, k):
    """f32 sequential accumulation, zero trits skipped, scale after the sum."""
    tr = decode_ternary(packed, m, k)
    b = np.asarray(b, f32).reshape(k, n)
    c = np.zeros((m, n), f32)
    for ki in range(k):
        t = tr[:, ki].astype(f32)[:, None]
        upd = (c + (t * b[ki][None, :]).astype(f32)).astype(f32)
        c = np.where(t != 0, upd, c)
    return (c * np.asarray(scales, f32)[:m, None]).astype(f32)


def quat_matmul(packed, scales, b, m, n, k):
    """scale folded into the weight first, then mul-then-add over ascending k."""
    codes = decode_quaternary_codes(packed, m, k)
    b = np.asarray(b, f32).reshape(k, n)
    s = np.asarray(scales, f32)[:m]
    c = np.zeros((m, n), f32)
    for ki in range(k):
        wv = (QUAT_VALUES[codes[:, ki]] * s).astype(f32)[:, None]
        c = (c + (wv * b[ki][None, :]).astype(f32)).astype(f32)
    return c


def quantize_act_i8(x: np.ndarray):
    x = np.asarray(x, f32)
    am = np.abs(x).max(axis=1)
    s = np.where(am < f32(1e-8), f32(1.0), (am / f32(127.0)).astype(f32)).astype(f32)
    q = np.rint((x / s[:, None]).astype(f32))
    q = np.clip(q, -127, 127).astype(np.int8)
    return q, s, q.astype(np.int32).sum(axis=1).astype(np.int32)


def acc_i32(w_i8: np.ndarray, xq: np.ndarray) -> np.ndarray:
    return (xq.astype(np.int64) @ w_i8.astype(np.int64).T).astype(np.int32)


def dequant(acc, sw, sx, bias=None):
    y = (acc.astype(f32) * np.asarray(sw, f32)[None, :]).astype(f32)
    y = (y * np.asarray(sx, f32)[:, None]).astype(f32)
    if bias is not None:
        y = (y + np.asarray(bias, f32)[None, :]).astype(f32)
    return y


def qlora_forward(base_out, x, lora_a, lora_b, alpha, rank, bias=None):
    """QLoraLinear::forward after the base projection (crates/kore-nn/src/lora.rs:296-317):
    output = base_out + ((x @ A^T) @ B^T) * (alpha / rank), then + bias.  f32 throughout; the
    two dense products are summed in numpy's order, so comparisons against another f32
    implementation of them need a tolerance."""
    f32 = np.float32
    scaling = f32(alpha) / f32(rank)
    lora = ((np.asarray(x, f32) @ np.asarray(lora_a, f32).T).astype(f32) @ np.asarray(lora_b, f32).T).astype(f32) * scaling
    out = (np.asarray(base_out, f32) + lora.astype(f32)).astype(f32)
    if bias is not None:
        out = (out + np.asarray(bias, f32)).astype(f32)
    return out


def lora_a_init(rank, in_features):
    """lora.rs:219-225 with Python integers (pure loop; small sizes only)"""
    a_scale = np.sqrt(np.float32(1.0) / np.float32(in_features)).astype(np.float32)
    out = np.zeros(rank * in_features, np.float32)
    for i in range(rank * in_features):
        x = np.float32((i * 2654435761 + 1013904223) & 0xFFFFFF) / np.float32(0xFFFFFF)
        out[i] = (x * np.float32(2.0) - np.float32(1.0)) * a_scale
    return out.reshape(rank, in_features)
