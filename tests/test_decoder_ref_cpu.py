"""CPU checks of the numpy decoder restatement used to verify the GPU decoder."""
import json
import os

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


# ---- the reference's own known answers for these operators (tests/golden/decoder_kats.json) ----
def _kats():
    root = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(root, "golden", "decoder_kats.json")) as fh:
        return json.load(fh)


def _check_props(case, out):
    out = np.asarray(out, np.float32).ravel()
    for idx, (lo, hi) in case.get("between", {}).items():
        assert lo < out[int(idx)] < hi, (case["name"], out)
    for idx, v in case.get("greater", {}).items():
        assert out[int(idx)] > v, (case["name"], out)
    for idx, v in case.get("abs_less", {}).items():
        assert abs(out[int(idx)]) < v, (case["name"], out)


def test_reference_known_answers_rmsnorm_silu_softmax():
    k = _kats()
    for c in k["rmsnorm"]:
        _check_props(c, dr.rmsnorm(np.array([c["x"]], np.float32), np.array(c["gamma"], np.float32), c["eps"]))
    for c in k["silu"]:
        _check_props(c, dr.silu(np.array(c["x"], np.float32)))
    for c in k["softmax"]:
        p = dr.softmax(np.array(c["x"], np.float32))
        assert abs(float(p.sum(dtype=np.float32)) - c["sum"]) < c["tol"] and np.isfinite(p).all()
        if c.get("increasing"):
            assert p[2] > p[1] > p[0]
    c = k["rmsnorm_proj"][0]
    x = np.array(c["x"], np.float32).reshape(c["batch"], c["hidden"])
    normed = dr.rmsnorm(x, np.array(c["gamma"], np.float32), c["eps"])
    assert np.abs(normed.ravel() - np.array(c["normed"], np.float32)).max() < c["tol"]
    w = np.array(c["w"], np.float32).reshape(c["out_dim"], c["hidden"])
    assert np.abs((normed @ w.T).ravel() - np.array(c["expect"], np.float32)).max() < c["tol"]
    c = k["rmsnorm_silu_gate"][0]
    x = np.array(c["x"], np.float32).reshape(c["rows"], c["cols"])
    z = np.array(c["z"], np.float32).reshape(c["rows"], c["cols"])
    out = dr.silu_mul(z, dr.rmsnorm(x, np.array(c["gamma"], np.float32), c["eps"]))
    assert np.isfinite(out).all() and abs(out.ravel()[c["zero_index"]]) < c["tol"]
    assert np.abs(out.ravel() - np.array(c["expect"], np.float32)).max() < c["tol"]


def test_reference_known_answers_rope():
    for c in _kats()["rope"]:
        hd, H = c["head_dim"], c["n_heads"]
        cos, sin = dr.rope_tables(hd, 16, c["base"])
        x = np.array(c["data"], np.float32).reshape(1, H, hd)
        y = dr.rope(x, np.array([c["pos"]]), cos, sin).ravel()
        if "expect" in c:
            assert np.abs(y - np.array(c["expect"], np.float32)).max() < c["tol"]
        if "changes_by_more_than" in c:
            assert np.abs(y - x.ravel()).max() > c["changes_by_more_than"]
        if "pair" in c:
            a, b = c["pair"]
            assert abs(float(np.sqrt(y[a] * y[a] + y[b] * y[b])) - c["pair_norm"]) < c["tol"]
    # the tables the GPU decoder uses are the same function of (head_dim, base)
    cfg = DecoderConfig(n_layers=1, d_model=8, n_heads=2, d_ff=16, vocab=11, max_len=16)
    cos, sin = rope_tables(cfg)
    cr, sr = dr.rope_tables(cfg.head_dim, cfg.max_len, cfg.rope_base)
    assert (cos == cr).all() and (sin == sr).all()


def test_reference_known_answers_attention():
    for c in _kats()["attention"]:
        seq, H, hd = c["seq"], c["n_heads"], c["head_dim"]
        q = np.array(c["q"], np.float32).reshape(seq, H, hd)
        kk = np.array(c["k"], np.float32).reshape(seq, H, hd)
        v = np.array(c["v"], np.float32).reshape(seq, H, hd)
        if c["causal"]:
            out = dr.attention(q, kk, v, start_pos=0)
        else:  # every query sees every key: one query row at a time at the end of the sequence
            out = np.concatenate([dr.attention(q[i:i + 1], kk, v, start_pos=seq - 1) for i in range(seq)])
        if "expect_all" in c:
            assert np.abs(out - c["expect_all"]).max() < c["tol"]
        if "expect_row0" in c:
            assert np.abs(out[0].ravel() - np.array(c["expect_row0"], np.float32)).max() < c["tol"]
