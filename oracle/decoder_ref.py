"""CPU restatement (numpy) of the decoder step around the quantized-linear path.

TEST INFRASTRUCTURE ONLY (see kbref.h).  Parity status: the reference's decoder loop
(``crates/kore-edge/src/runtime.rs:106-294``) has no recorded end-to-end outputs and cannot
be run here, so this restatement is pinned operator by operator against every known answer
the reference's own unit tests hold for them (``tests/golden/decoder_kats.json``, checked in
``tests/test_decoder_ref_cpu.py``): RMSNorm (``crates/kore-edge/src/ops/norm.rs:43-49``,
``crates/kore-kernels/src/cpu_fused.rs:264-276``), the fused RMSNorm + projection and
RMSNorm x SiLU-gate references (``cpu_fused.rs:309-370,451-489``), RoPE
(``crates/kore-edge/src/ops/rope.rs:43-75``), attention (``ops/attention.rs:142-207``), SiLU
and softmax (``ops/activation.rs:87-119``); every projection goes through the pinned
``kbref.q_forward``.  Projections use the W2A8 arithmetic (per-token int8 activations), as
the GPU path does.
"""
from __future__ import annotations

import numpy as np

from . import kbref

f32 = np.float32


def rmsnorm(x, gamma, eps):
    """(x * (1 / sqrt(mean(x^2) + eps))) * gamma  — cpu_fused.rs:176-184"""
    x = np.asarray(x, f32)
    ss = (x * x).sum(axis=-1, dtype=f32)
    rms = np.sqrt((ss / f32(x.shape[-1]) + f32(eps)).astype(f32)).astype(f32)
    inv = (f32(1.0) / rms).astype(f32)
    return ((x * inv[..., None]).astype(f32) * np.asarray(gamma, f32)).astype(f32)


def silu_mul(g, u):
    """(g / (1 + exp(-g))) * u — ops/activation.rs:21-26, runtime.rs:249-252"""
    g = np.asarray(g, f32)
    return ((g / (f32(1.0) + np.exp(-g).astype(f32))).astype(f32) * np.asarray(u, f32)).astype(f32)


def silu(x):
    """x / (1 + exp(-x)) — ops/activation.rs:21-26"""
    x = np.asarray(x, f32)
    return (x / (f32(1.0) + np.exp(-x).astype(f32))).astype(f32)


def softmax(x):
    """over the last axis, max subtracted first — ops/activation.rs:37-56"""
    x = np.asarray(x, f32)
    e = np.exp((x - x.max(axis=-1, keepdims=True)).astype(f32)).astype(f32)
    return (e * (f32(1.0) / e.sum(axis=-1, keepdims=True, dtype=f32))).astype(f32)


def rope_tables(head_dim, max_len, base):
    """cos/sin [max_len, head_dim/2]: freq_i = 1 / base^(2i/head_dim), angle = pos * freq_i (ops/rope.rs:24-27)"""
    i = np.arange(head_dim // 2, dtype=f32)
    freq = (f32(1.0) / np.power(f32(base), (f32(2.0) * i / f32(head_dim)).astype(f32))).astype(f32)
    ang = (np.arange(max_len, dtype=f32)[:, None] * freq[None, :]).astype(f32)
    return np.cos(ang).astype(f32), np.sin(ang).astype(f32)


def rope(x, positions, cos, sin):
    """x [N, H, hd]; pairs (i, i + hd/2) — ops/rope.rs:17-35"""
    x = np.asarray(x, f32)
    half = x.shape[-1] // 2
    c = cos[positions][:, None, :]
    s = sin[positions][:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return np.concatenate([(x0 * c).astype(f32) - (x1 * s).astype(f32), (x0 * s).astype(f32) + (x1 * c).astype(f32)], axis=-1).astype(f32)


def attention(q, k, v, start_pos):
    """q [T, H, hd], k/v [L, H, hd] with L = start_pos + T; query i sees keys <= start_pos + i
    (ops/attention.rs:99-133 with the mask of layered/engine.rs:734-751)."""
    t, h, hd = q.shape
    L = k.shape[0]
    scale = f32(1.0) / np.sqrt(f32(hd))
    out = np.zeros_like(q)
    for hh in range(h):
        sc = (q[:, hh, :] @ k[:, hh, :].T).astype(f32) * scale
        mask = np.arange(L)[None, :] > (start_pos + np.arange(t))[:, None]
        sc = np.where(mask, -np.inf, sc).astype(f32)
        sc = sc - sc.max(axis=1, keepdims=True)
        e = np.exp(sc).astype(f32)
        p = (e / e.sum(axis=1, keepdims=True)).astype(f32)
        out[:, hh, :] = (p @ v[:, hh, :]).astype(f32)
    return out


def project(w, x, resid=None, threads=4):
    packed, scales, m, k = w
    y, _ = kbref.q_forward(kbref.TERNARY, packed, scales, None, m, k, np.ascontiguousarray(x, f32), threads=threads)
    return (y + resid).astype(f32) if resid is not None else y


class DecoderRef:
    """Single-sequence decoder with a KV cache."""

    def __init__(self, cfg, weights, cos, sin):
        self.cfg, self.w, self.cos, self.sin = cfg, weights, cos, sin
        self.k = [np.zeros((0, cfg.n_heads, cfg.head_dim), f32) for _ in range(cfg.n_layers)]
        self.v = [np.zeros((0, cfg.n_heads, cfg.head_dim), f32) for _ in range(cfg.n_layers)]
        self.pos = 0

    def forward(self, tokens):
        """tokens: list of ids (prompt chunk or a single decode token) -> logits of the last one"""
        cfg, W = self.cfg, self.w
        t = len(tokens)
        H, hd = cfg.n_heads, cfg.head_dim
        hidden = W["embed"][np.asarray(tokens)].astype(f32)
        positions = np.arange(self.pos, self.pos + t)
        for li, lw in enumerate(W["layers"]):
            xn = rmsnorm(hidden, lw["norm1"], cfg.eps)
            q = project(lw["q"], xn).reshape(t, H, hd)
            k = project(lw["k"], xn).reshape(t, H, hd)
            v = project(lw["v"], xn).reshape(t, H, hd)
            q = rope(q, positions, self.cos, self.sin)
            k = rope(k, positions, self.cos, self.sin)
            self.k[li] = np.concatenate([self.k[li], k])
            self.v[li] = np.concatenate([self.v[li], v])
            a = attention(q, self.k[li], self.v[li], self.pos).reshape(t, H * hd)
            hidden = project(lw["o"], a, resid=hidden)
            xn = rmsnorm(hidden, lw["norm2"], cfg.eps)
            g = project(lw["gate"], xn)
            u = project(lw["up"], xn)
            hidden = project(lw["down"], silu_mul(g, u), resid=hidden)
        self.pos += t
        xn = rmsnorm(hidden[-1:], W["norm_f"], cfg.eps)
        return (xn @ W["lm_head"].T.astype(f32)).astype(f32)[0]
