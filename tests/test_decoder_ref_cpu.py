"""CPU checks of the numpy decoder restatement used to verify the GPU decoder."""
import numpy as np

from kore_b200.decoder import DecoderConfig, rope_tables
from oracle import decoder_ref as dr


def test_rmsnorm_formula():
    x = np.array([[3.0, 4.0]], np.float32)
    out = dr.rmsnorm(x, np.array([1.0, 2.0], np.float32), 0.0)
    rms = np.sqrt(np.float32(12.5))
    assert np.allclose(out, [[3.0 / rms, 8.0 / rms]], rtol=1e-6)


def test_rope_identity_at_position_zero_and_norm_preserved():
    cfg = DecoderConfig(n_layers=1, d_model=8, n_heads=2, d_ff=16, vocab=11, max_len=16)
    cos, sin = rope_tables(cfg)
    assert cos.shape == (16, 2) and np.all(cos[0] == 1.0) and np.all(sin[0] == 0.0)
    x = np.arange(16, dtype=np.float32).reshape(2, 2, 4) + 1
    assert (dr.rope(x, np.array([0, 0]), cos, sin) == x).all()
    y = dr.rope(x, np.array([3, 7]), cos, sin)
    assert np.allclose((y ** 2).sum(-1), (x ** 2).sum(-1), rtol=1e-5)
    # first frequency is 1 rad per position: pair (0, half) rotates by pos radians
    assert np.allclose(y[0, 0, 0], x[0, 0, 0] * np.cos(3.0) - x[0, 0, 2] * np.sin(3.0), rtol=1e-5)


def test_attention_causal_against_direct_softmax():
    rng = np.random.default_rng(0)
    q = rng.standard_normal((3, 2, 4)).astype(np.float32)
    k = rng.standard_normal((5, 2, 4)).astype(np.float32)
    v = rng.standard_normal((5, 2, 4)).astype(np.float32)
    out = dr.attention(q, k, v, start_pos=2)
    for i in range(3):
        for h in range(2):
            s = (k[: 2 + i + 1, h] @ q[i, h]) / 2.0
            p = np.exp(s - s.max())
            p /= p.sum()
            assert np.allclose(out[i, h], p @ v[: 2 + i + 1, h], rtol=1e-5, atol=1e-6)


def test_silu_mul():
    g = np.array([0.0, 1.0, -2.0], np.float32)
    u = np.array([5.0, 2.0, 3.0], np.float32)
    ref = g / (1 + np.exp(-g)) * u
    assert np.allclose(dr.silu_mul(g, u), ref, rtol=1e-6)
