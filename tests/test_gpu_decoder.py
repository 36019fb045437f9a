"""Decoder-step kernels and the small end-to-end decoder against the CPU restatement."""
import ctypes as C

import numpy as np
import pytest

from oracle import decoder_ref as dr
from oracle import kbref
from tests import cases

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch

    from kore_b200 import _cabi, decoder, nn

    assert torch.cuda.is_available()
    return type("E", (), {"torch": torch, "cabi": _cabi, "lib": _cabi.lib(), "decoder": decoder, "nn": nn,
                          "sp": torch.cuda.current_stream().cuda_stream})


@pytest.mark.parametrize("n,d", [(1, 3200), (5, 128), (3, 8640), (2, 77)])
def test_rmsnorm_quant(env, n, d):
    t = env.torch
    x = cases.gaussian(n + d, (n, d), 1.5)
    g = (1.0 + cases.gaussian(7, (d,), 0.1)).astype(np.float32)
    ld = int(env.lib.kb_act_ld(d))
    xd, gd = t.from_numpy(x).cuda(), t.from_numpy(g).cuda()
    xn = t.empty((n, d), device="cuda")
    xq = t.empty((n, ld), dtype=t.int8, device="cuda")
    sx = t.empty(n, device="cuda")
    sm = t.empty(n, dtype=t.int32, device="cuda")
    env.cabi.check(env.lib.kb_rmsnorm_quant(xd.data_ptr(), gd.data_ptr(), n, d, C.c_float(1e-5), xn.data_ptr(), xq.data_ptr(), ld,
                                            sx.data_ptr(), sm.data_ptr(), env.sp))
    xn_h = xn.cpu().numpy()
    ref = dr.rmsnorm(x, g, 1e-5)
    # float reduction order differs from the sequential CPU sum: 1e-5 relative to the row's largest value
    assert (np.abs(xn_h - ref) <= 1e-5 * np.abs(ref).max(axis=1, keepdims=True)).all()
    # the quantiser applied to the kernel's own normalised values is exact
    q_ref, s_ref, sum_ref = kbref.quantize_act_i8(xn_h, ldq=ld)
    assert (xq.cpu().numpy() == q_ref).all() and (sx.cpu().numpy() == s_ref).all() and (sm.cpu().numpy() == sum_ref).all()


@pytest.mark.parametrize("n,f", [(1, 8640), (4, 256), (2, 100)])
def test_swiglu_quant(env, n, f):
    t = env.torch
    gu = cases.gaussian(n * f, (n, 2 * f), 2.0)
    ld = int(env.lib.kb_act_ld(f))
    gud = t.from_numpy(gu).cuda()
    h = t.empty((n, f), device="cuda")
    xq = t.empty((n, ld), dtype=t.int8, device="cuda")
    sx = t.empty(n, device="cuda")
    sm = t.empty(n, dtype=t.int32, device="cuda")
    env.cabi.check(env.lib.kb_swiglu_quant(gud.data_ptr(), n, f, 2 * f, h.data_ptr(), xq.data_ptr(), ld, sx.data_ptr(), sm.data_ptr(), env.sp))
    h_h = h.cpu().numpy()
    ref = dr.silu_mul(gu[:, :f], gu[:, f:])
    assert (np.abs(h_h - ref) <= 2e-6 * np.abs(ref).max() + 1e-7).all()  # expf differs from libm in the last bits
    q_ref, s_ref, sum_ref = kbref.quantize_act_i8(h_h, ldq=ld)
    assert (xq.cpu().numpy() == q_ref).all() and (sx.cpu().numpy() == s_ref).all() and (sm.cpu().numpy() == sum_ref).all()


@pytest.mark.parametrize("n,f", [(1, 8640), (3, 130)])
def test_swiglu_quant_pairs_equals_halves(env, n, f):
    """the interleaved-row variant computes exactly what the [gate | up] variant does"""
    t = env.torch
    gu = cases.gaussian(5 + n * f, (n, 2 * f), 2.0)
    inter = np.empty_like(gu)
    inter[:, 0::2], inter[:, 1::2] = gu[:, :f], gu[:, f:]
    ld = int(env.lib.kb_act_ld(f))
    outs = []
    for fn, src in ((env.lib.kb_swiglu_quant, gu), (env.lib.kb_swiglu_quant_pairs, inter)):
        d_in = t.from_numpy(src).cuda()
        h = t.empty((n, f), device="cuda")
        xq = t.empty((n, ld), dtype=t.int8, device="cuda")
        sx = t.empty(n, device="cuda")
        sm = t.empty(n, dtype=t.int32, device="cuda")
        env.cabi.check(fn(d_in.data_ptr(), n, f, 2 * f, h.data_ptr(), xq.data_ptr(), ld, sx.data_ptr(), sm.data_ptr(), env.sp))
        t.cuda.synchronize()
        outs.append((h.cpu().numpy(), xq.cpu().numpy(), sx.cpu().numpy(), sm.cpu().numpy()))
    for a, b in zip(*outs):
        assert (a == b).all()


@pytest.mark.parametrize("n,m,k", [(1, 9600, 3200), (2, 300, 640), (5, 64, 256)])
def test_projection_with_rmsnorm_prologue(env, n, m, k):
    """kb_linear_forward_rmsnorm == kb_rmsnorm_quant followed by the projection, up to the order
    of the row's sum of squares; against the restatement: normalise, then the exact W2A8 forward"""
    t = env.torch
    x = cases.gaussian(300 + n + k, (n, k), 1.5)
    g = (1.0 + cases.gaussian(8, (k,), 0.1)).astype(np.float32)
    w = cases.gaussian(301 + m, (m, k), 0.02)
    packed, scales = kbref.pack_weights_ternary_absmean(w, m, k)
    lay = env.nn.BitLinear.from_packed(packed, scales, None, k, m)
    xd, gd = t.from_numpy(x).cuda(), t.from_numpy(g).cuda()
    y = t.empty((n, m), device="cuda")
    env.cabi.check(env.lib.kb_linear_forward_rmsnorm(lay.handle, xd.data_ptr(), gd.data_ptr(), C.c_float(1e-5), n, y.data_ptr(),
                                                     0, 0, None, env.sp))
    t.cuda.synchronize()
    # two-kernel path on the GPU: the normalised rows may differ in the last bit (sum order), and a
    # code flips only where a value sits on a rounding boundary, so compare through the restatement
    xn = dr.rmsnorm(x, g, 1e-5)
    y_ref = kbref.q_forward(kbref.TERNARY, packed, scales, None, m, k, xn, threads=2)[0]
    tol = 2e-3 * np.abs(y_ref).max(axis=1, keepdims=True)
    assert (np.abs(y.cpu().numpy() - y_ref) <= tol).all()
    # and it is exact when the kernel's own normalised row is quantised by the restatement
    xn_gpu = t.empty((n, k), device="cuda")
    env.cabi.check(env.lib.kb_rmsnorm_quant(xd.data_ptr(), gd.data_ptr(), n, k, C.c_float(1e-5), xn_gpu.data_ptr(), None, 0, None,
                                            None, env.sp))
    t.cuda.synchronize()
    y_two = kbref.q_forward(kbref.TERNARY, packed, scales, None, m, k, xn_gpu.cpu().numpy(), threads=2)[0]
    frac_equal = float((y.cpu().numpy() == y_two).mean())
    assert frac_equal > 0.5  # identical unless the two reductions rounded the row's scale differently
    lay.close()


@pytest.mark.parametrize("n,f,k", [(1, 8640, 3200), (2, 8640, 3200), (2, 150, 256), (1, 4096, 512)])
def test_swiglu_epilogue_and_prescaled_projection(env, n, f, k):
    """gate/up projection with interleaved rows + SwiGLU epilogue + atomic max|h|, then the down
    projection quantising with that maximum: equal to the separate kernels bit for bit"""
    t = env.torch
    x = cases.gaussian(400 + n + k, (n, k), 1.0)
    g = (1.0 + cases.gaussian(9, (k,), 0.1)).astype(np.float32)
    wg, wu = cases.gaussian(401, (f, k), 0.02), cases.gaussian(402, (f, k), 0.02)
    wd = cases.gaussian(403, (k, f), 0.02)
    pg, sg = kbref.pack_weights_ternary_absmean(wg, f, k)
    pu, su = kbref.pack_weights_ternary_absmean(wu, f, k)
    pd, sd = kbref.pack_weights_ternary_absmean(wd, k, f)
    inter = env.decoder._interleave_rows((pg, sg, f, k), (pu, su, f, k))
    gu = env.nn.BitLinear.from_packed(inter[0], inter[1], None, k, 2 * f)
    down = env.nn.BitLinear.from_packed(pd, sd, None, f, k)
    xd, gd = t.from_numpy(x).cuda(), t.from_numpy(g).cuda()
    resid = cases.gaussian(404, (n, k), 1.0)
    # fused: norm+gu+swiglu -> h, absmax; down with known absmax (+ residual), clearing the other slot
    h = t.empty((n, f), device="cuda")
    am = t.zeros((2, n), device="cuda")
    am[1].fill_(7.0)
    y = t.from_numpy(resid).cuda()
    env.cabi.check(env.lib.kb_linear_forward_rmsnorm(gu.handle, xd.data_ptr(), gd.data_ptr(), C.c_float(1e-5), n, h.data_ptr(), 0, 1,
                                                     am[0].data_ptr(), env.sp))
    env.cabi.check(env.lib.kb_linear_forward_scaled(down.handle, h.data_ptr(), am[0].data_ptr(), n, y.data_ptr(), y.data_ptr(), 0,
                                                    am[1].data_ptr(), env.sp))
    t.cuda.synchronize()
    h_h = h.cpu().numpy()
    assert (am[0].cpu().numpy() == np.abs(h_h).max(axis=1)).all()
    assert (am[1].cpu().numpy() == 0).all()
    # separate kernels on the same normalised input
    gu_out = t.empty((n, 2 * f), device="cuda")
    env.cabi.check(env.lib.kb_linear_forward_rmsnorm(gu.handle, xd.data_ptr(), gd.data_ptr(), C.c_float(1e-5), n, gu_out.data_ptr(),
                                                     0, 0, None, env.sp))
    t.cuda.synchronize()
    go = gu_out.cpu().numpy()
    # restated SiLU * up from the kernel's own gate/up values (expf differs from libm in the last bits)
    ref_h = dr.silu_mul(go[:, 0::2], go[:, 1::2])
    assert (np.abs(h_h - ref_h) <= 2e-6 * np.abs(ref_h).max() + 1e-7).all()
    # down projection: exact W2A8 forward of the kernel's h, plus the residual
    y_ref = kbref.q_forward(kbref.TERNARY, pd, sd, None, k, f, h_h, threads=2)[0]
    assert (y.cpu().numpy() == (y_ref + resid).astype(np.float32)).all()
    gu.close()
    down.close()


@pytest.mark.parametrize("d_model", [128, 120])  # head_dim 32 (128-bit key/value loads) and 30 (scalar loads)
def test_rope_kv_and_attention(env, d_model):
    t = env.torch
    cfg = env.decoder.DecoderConfig(n_layers=1, d_model=d_model, n_heads=4, d_ff=256, vocab=50, max_len=24)
    cos, sin = env.decoder.rope_tables(cfg)
    H, hd, d = cfg.n_heads, cfg.head_dim, cfg.d_model
    batch, lmax = 3, cfg.max_len
    kc = t.zeros((batch, H, lmax, hd), device="cuda")  # head-major caches
    vc = t.zeros((batch, H, lmax, hd), device="cuda")
    cosd, sind = t.from_numpy(cos).cuda(), t.from_numpy(sin).cuda()
    lens = [5, 1, 9]
    k_ref = [np.zeros((0, H, hd), np.float32) for _ in range(batch)]
    v_ref = [np.zeros((0, H, hd), np.float32) for _ in range(batch)]
    q_last = np.zeros((batch, H, hd), np.float32)
    for b in range(batch):  # fill each sequence token by token
        for pos in range(lens[b]):
            qkv = cases.gaussian(1000 * b + pos, (1, 3 * d), 1.0)
            q_out = t.empty((1, d), device="cuda")
            qkv_d = t.from_numpy(qkv).cuda()  # named: a temporary would be freed before the kernel runs
            pos_d = t.tensor([pos], dtype=t.int32, device="cuda")
            row_d = t.tensor([b * lmax + pos], dtype=t.int64, device="cuda")
            env.cabi.check(env.lib.kb_rope_kv(qkv_d.data_ptr(), pos_d.data_ptr(), row_d.data_ptr(), cosd.data_ptr(),
                                              sind.data_ptr(), 1, H, hd, lmax, q_out.data_ptr(), kc.data_ptr(), vc.data_ptr(), env.sp))
            t.cuda.synchronize()
            q_r = dr.rope(qkv[:, :d].reshape(1, H, hd), np.array([pos]), cos, sin)
            k_r = dr.rope(qkv[:, d:2 * d].reshape(1, H, hd), np.array([pos]), cos, sin)
            assert (q_out.cpu().numpy().reshape(1, H, hd) == q_r).all()  # same table, same roundings
            k_ref[b] = np.concatenate([k_ref[b], k_r])
            v_ref[b] = np.concatenate([v_ref[b], qkv[:, 2 * d:].reshape(1, H, hd)])
            q_last[b] = q_r[0]
        assert (kc[b, :, :lens[b]].transpose(0, 1).cpu().numpy() == k_ref[b]).all()
        assert (vc[b, :, :lens[b]].transpose(0, 1).cpu().numpy() == v_ref[b]).all()
    out = t.empty((batch, d), device="cuda")
    q_d = t.from_numpy(q_last.reshape(batch, d)).cuda()
    lens_d = t.tensor(lens, dtype=t.int32, device="cuda")
    nbytes = int(env.lib.kb_attn_decode_scratch_bytes(batch, H))
    scratch = t.zeros(nbytes, dtype=t.uint8, device="cuda")
    for use_scratch in (True, True, False):  # split path twice (counters must reset), then one CTA per head
        out.zero_()
        env.cabi.check(env.lib.kb_attn_decode(q_d.data_ptr(), kc.data_ptr(), vc.data_ptr(), lens_d.data_ptr(), batch, H, hd, lmax,
                                              out.data_ptr(), scratch.data_ptr() if use_scratch else None,
                                              nbytes if use_scratch else 0, env.sp))
        for b in range(batch):
            ref = dr.attention(q_last[b:b + 1], k_ref[b], v_ref[b], start_pos=lens[b] - 1).reshape(d)
            assert np.abs(out[b].cpu().numpy() - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("n", [1, 4, 40])
def test_fused_forward_with_residual(env, n):
    t = env.torch
    m, k = 200, 384
    w = cases.gaussian(5, (m, k), 0.02)
    packed, scales = cases.make_weights(kbref.TERNARY, "absmean", w)
    lay = env.nn.BitLinear.from_packed(packed, scales, None, k, m)
    x = cases.gaussian(6 + n, (n, k), 1.0)
    resid = cases.gaussian(7, (n, m), 1.0)
    y_ref = (kbref.q_forward(kbref.TERNARY, packed, scales, None, m, k, x)[0] + resid).astype(np.float32)
    ws_bytes = int(env.lib.kb_linear_workspace_bytes(lay.handle, n))
    ws = t.empty(ws_bytes + 256, dtype=t.uint8, device="cuda")
    ws_ptr = (ws.data_ptr() + 255) // 256 * 256
    # f32 input, residual updated in place
    hid = t.from_numpy(resid).cuda()
    x_d = t.from_numpy(x).cuda()
    env.cabi.check(env.lib.kb_linear_forward_fused(lay.handle, x_d.data_ptr(), None, 0, None, None, n,
                                                   hid.data_ptr(), hid.data_ptr(), 0, env.cabi.PATH_AUTO, ws_ptr, ws_bytes, env.sp))
    assert (hid.cpu().numpy() == y_ref).all()
    # pre-quantised input, separate output, both kernels
    from kore_b200 import kernels
    xq, sx, sm = kernels.quantize_act_i8(x_d)
    resid_d = t.from_numpy(resid).cuda()
    for path in (env.cabi.PATH_GEMV, env.cabi.PATH_GEMM_TC):
        y = t.empty((n, m), device="cuda")
        env.cabi.check(env.lib.kb_linear_forward_fused(lay.handle, None, xq.data_ptr(), xq.stride(0), sx.data_ptr(), sm.data_ptr(), n,
                                                       resid_d.data_ptr(), y.data_ptr(), 0, path, None, 0, env.sp))
        assert (y.cpu().numpy() == y_ref).all()


def test_small_decoder_against_cpu_restatement(env):
    t = env.torch
    cfg = env.decoder.DecoderConfig(n_layers=2, d_model=128, n_heads=4, d_ff=256, vocab=97, max_len=32)
    weights = env.decoder.random_weights(cfg, seed=4000)
    cos, sin = env.decoder.rope_tables(cfg)
    prompt = np.array([[5, 17, 3, 90, 41, 8], [1, 2, 3, 4, 5, 6]], np.int64)
    dec = env.decoder.BitNetDecoder(cfg, weights, batch=2)
    logits = dec.prefill(t.from_numpy(prompt).cuda()).cpu().numpy()
    refs = [dr.DecoderRef(cfg, weights, cos, sin) for _ in range(2)]
    ref_logits = np.stack([refs[b].forward(list(prompt[b])) for b in range(2)])
    # int8 activation codes are discontinuous in the f32 inputs, so a last-bit difference in a
    # norm or softmax can flip a code: tolerance is 2 % of the largest logit
    tol = 0.02 * np.abs(ref_logits).max()
    assert np.abs(logits - ref_logits).max() <= tol
    toks = logits.argmax(axis=1)
    dec.tokens.copy_(t.from_numpy(toks).cuda())
    for step in range(3):
        dec.decode_step(use_graph=(step > 0))
        ref_logits = np.stack([refs[b].forward([int(toks[b])]) for b in range(2)])
        got = dec.logits.cpu().numpy()
        assert np.abs(got - ref_logits).max() <= tol, step
        toks = dec.tokens.cpu().numpy()
    dec.close()


def test_fused_projection_argument_checks(env):
    """the decode-step projections refuse what they cannot run instead of falling back"""
    t = env.torch
    m, k = 64, 256
    w = cases.gaussian(500, (m, k), 0.02)
    packed, scales = kbref.pack_weights_ternary_absmean(w, m, k)
    lay = env.nn.BitLinear.from_packed(packed, scales, None, k, m)
    x = t.zeros((16, k), device="cuda")
    g = t.ones(k, device="cuda")
    y = t.zeros((16, m), device="cuda")
    am = t.zeros(16, device="cuda")
    lib, E = env.lib, env.cabi
    assert lib.kb_linear_forward_rmsnorm(lay.handle, x.data_ptr(), g.data_ptr(), C.c_float(1e-5), 9, y.data_ptr(), 0, 0, None, env.sp) == E.ERR_UNSUPPORTED
    assert lib.kb_linear_forward_rmsnorm(lay.handle, x.data_ptr(), g.data_ptr(), C.c_float(1e-5), 3, y.data_ptr(), 0, 1, am.data_ptr(), env.sp) == E.ERR_UNSUPPORTED
    assert "tokens" in lib.kb_last_error().decode()
    assert lib.kb_linear_forward_rmsnorm(lay.handle, None, g.data_ptr(), C.c_float(1e-5), 1, y.data_ptr(), 0, 0, None, env.sp) == E.ERR_INVALID
    assert lib.kb_linear_forward_rmsnorm(lay.handle, x.data_ptr(), g.data_ptr(), C.c_float(1e-5), 1, y.data_ptr(), m - 1, 0, None, env.sp) == E.ERR_INVALID
    assert lib.kb_linear_forward_scaled(lay.handle, x.data_ptr(), am.data_ptr(), 9, None, y.data_ptr(), 0, None, env.sp) == E.ERR_UNSUPPORTED
    assert lib.kb_linear_forward_scaled(lay.handle, x.data_ptr(), None, 1, None, y.data_ptr(), 0, None, env.sp) == E.ERR_INVALID
    assert lib.kb_linear_forward_rmsnorm(None, x.data_ptr(), g.data_ptr(), C.c_float(1e-5), 1, y.data_ptr(), 0, 0, None, env.sp) == E.ERR_BAD_HANDLE
    # zero tokens is a no-op
    assert lib.kb_linear_forward_rmsnorm(lay.handle, x.data_ptr(), g.data_ptr(), C.c_float(1e-5), 0, y.data_ptr(), 0, 0, None, env.sp) == 0
    # a SwiGLU epilogue needs an even number of rows
    w3 = cases.gaussian(501, (63, k), 0.02)
    p3, s3 = kbref.pack_weights_ternary_absmean(w3, 63, k)
    odd = env.nn.BitLinear.from_packed(p3, s3, None, k, 63)
    assert lib.kb_linear_forward_rmsnorm(odd.handle, x.data_ptr(), g.data_ptr(), C.c_float(1e-5), 1, y.data_ptr(), 0, 1, am.data_ptr(), env.sp) == E.ERR_UNSUPPORTED
    t.cuda.synchronize()
    lay.close()
    odd.close()


# ---- the reference's own known answers for these operators, on the GPU kernels ----------------
def _decoder_kats():
    import json
    import os

    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "decoder_kats.json")) as fh:
        return json.load(fh)


def _gpu_rmsnorm(env, x, gamma, eps):
    t = env.torch
    n, d = x.shape
    xd, gd = t.from_numpy(np.ascontiguousarray(x, np.float32)).cuda(), t.from_numpy(np.asarray(gamma, np.float32)).cuda()
    xn = t.empty((n, d), device="cuda")
    env.cabi.check(env.lib.kb_rmsnorm_quant(xd.data_ptr(), gd.data_ptr(), n, d, C.c_float(eps), xn.data_ptr(), None, 0, None, None,
                                            env.sp))
    t.cuda.synchronize()
    return xn.cpu().numpy()


def _gpu_swiglu(env, gate, up):
    t = env.torch
    n, f = gate.shape
    gu = t.from_numpy(np.concatenate([gate, up], axis=1).astype(np.float32)).cuda()
    h = t.empty((n, f), device="cuda")
    env.cabi.check(env.lib.kb_swiglu_quant(gu.data_ptr(), n, f, 2 * f, h.data_ptr(), None, 0, None, None, env.sp))
    t.cuda.synchronize()
    return h.cpu().numpy()


def test_reference_known_answers_norm_and_gate_kernels(env):
    k = _decoder_kats()
    for c in k["rmsnorm"]:
        out = _gpu_rmsnorm(env, np.array([c["x"]], np.float32), c["gamma"], c["eps"]).ravel()
        for idx, (lo, hi) in c.get("between", {}).items():
            assert lo < out[int(idx)] < hi
        for idx, v in c.get("greater", {}).items():
            assert out[int(idx)] > v
    c = k["rmsnorm_proj"][0]
    x = np.array(c["x"], np.float32).reshape(c["batch"], c["hidden"])
    assert np.abs(_gpu_rmsnorm(env, x, c["gamma"], c["eps"]).ravel() - np.array(c["normed"], np.float32)).max() < c["tol"]
    c = k["silu"][0]
    out = _gpu_swiglu(env, np.array([c["x"]], np.float32), np.ones((1, len(c["x"])), np.float32)).ravel()
    assert abs(out[0]) < c["abs_less"]["0"] and out[1] > c["greater"]["1"]
    c = k["rmsnorm_silu_gate"][0]
    x = np.array(c["x"], np.float32).reshape(c["rows"], c["cols"])
    z = np.array(c["z"], np.float32).reshape(c["rows"], c["cols"])
    out = _gpu_swiglu(env, z, _gpu_rmsnorm(env, x, c["gamma"], c["eps"])).ravel()
    assert np.isfinite(out).all() and abs(out[c["zero_index"]]) < c["tol"]
    assert np.abs(out - np.array(c["expect"], np.float32)).max() < c["tol"]


def test_reference_known_answers_rope_and_attention_kernels(env):
    t = env.torch
    k = _decoder_kats()
    for c in k["rope"]:
        H, hd = c["n_heads"], c["head_dim"]
        d = H * hd
        cos, sin = dr.rope_tables(hd, 16, c["base"])
        data = np.array(c["data"], np.float32)
        qkv = t.from_numpy(np.concatenate([data, data, data])[None, :]).cuda()  # q = k = v = the case's row
        q_out = t.empty((1, d), device="cuda")
        kc, vc = t.zeros((1, H, 1, hd), device="cuda"), t.zeros((1, H, 1, hd), device="cuda")
        pos = t.tensor([c["pos"]], dtype=t.int32, device="cuda")
        row = t.tensor([0], dtype=t.int64, device="cuda")
        cosd, sind = t.from_numpy(cos).cuda(), t.from_numpy(sin).cuda()
        env.cabi.check(env.lib.kb_rope_kv(qkv.data_ptr(), pos.data_ptr(), row.data_ptr(), cosd.data_ptr(), sind.data_ptr(), 1, H, hd,
                                          1, q_out.data_ptr(), kc.data_ptr(), vc.data_ptr(), env.sp))
        t.cuda.synchronize()
        for y in (q_out.cpu().numpy().ravel(), kc.cpu().numpy().ravel()):  # q and the cached k are both rotated
            if "expect" in c:
                assert np.abs(y - np.array(c["expect"], np.float32)).max() < c["tol"]
            if "changes_by_more_than" in c:
                assert np.abs(y - data).max() > c["changes_by_more_than"]
            if "pair" in c:
                a, b = c["pair"]
                assert abs(float(np.sqrt(y[a] * y[a] + y[b] * y[b])) - c["pair_norm"]) < c["tol"]
        assert (vc.cpu().numpy().ravel() == data).all()  # v goes to the cache untouched
    for c in k["attention"]:
        seq, H, hd = c["seq"], c["n_heads"], c["head_dim"]
        d = H * hd
        q = np.array(c["q"], np.float32).reshape(seq, d)
        kk = np.array(c["k"], np.float32).reshape(seq, d)
        v = np.array(c["v"], np.float32).reshape(seq, d)
        # the decode kernel serves one query per sequence: query i becomes sequence i over the same
        # cache, seeing i + 1 positions (causal) or all of them
        # [sequence][head][position][hd]
        kc = t.from_numpy(np.broadcast_to(kk.reshape(seq, H, hd).transpose(1, 0, 2), (seq, H, seq, hd)).copy()).cuda()
        vc = t.from_numpy(np.broadcast_to(v.reshape(seq, H, hd).transpose(1, 0, 2), (seq, H, seq, hd)).copy()).cuda()
        lens = t.tensor([i + 1 if c["causal"] else seq for i in range(seq)], dtype=t.int32, device="cuda")
        out = t.empty((seq, d), device="cuda")
        nbytes = int(env.lib.kb_attn_decode_scratch_bytes(seq, H))
        scratch = t.zeros(max(nbytes, 4), dtype=t.uint8, device="cuda")
        qd = t.from_numpy(q).cuda()
        env.cabi.check(env.lib.kb_attn_decode(qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), lens.data_ptr(), seq, H, hd, seq,
                                              out.data_ptr(), scratch.data_ptr(), nbytes, env.sp))
        t.cuda.synchronize()
        o = out.cpu().numpy()
        if "expect_all" in c:
            assert np.abs(o - c["expect_all"]).max() < c["tol"]
        if "expect_row0" in c:
            assert np.abs(o[0] - np.array(c["expect_row0"], np.float32)).max() < c["tol"]
        ref = dr.attention(q.reshape(seq, H, hd), kk.reshape(seq, H, hd), v.reshape(seq, H, hd), 0).reshape(seq, d) if c["causal"] else None
        if ref is not None:
            assert np.abs(o - ref).max() < 1e-5


@pytest.mark.parametrize("batch", [1, 2])
def test_persistent_decode_step_matches_the_separate_kernels(env, batch):
    """One cooperative launch per step (kb_decoder_step) against the step built from the separate kernels:
    same tokens, logits within the tolerance the int8 activation codes allow, clean status word."""
    t = env.torch
    cfg = env.decoder.DecoderConfig(n_layers=3, d_model=256, n_heads=4, d_ff=640, vocab=301, max_len=48)
    weights = env.decoder.random_weights(cfg, seed=4100)
    prompt = t.from_numpy(np.array([[7, 300, 12, 99, 150, 3, 42, 8, 250][: 9 - b] + [1] * b for b in range(batch)], np.int64)).cuda()
    outs = []
    for persistent in (True, False):
        dec = env.decoder.BitNetDecoder(cfg, weights, batch=batch, persistent=persistent)
        assert (dec.persistent is not None) == persistent
        logits = dec.prefill(prompt)
        t.argmax(logits, dim=1, out=dec.tokens)
        toks, lgs = [dec.tokens.cpu().numpy().copy()], []
        for _ in range(8):
            dec.decode_step()
            toks.append(dec.tokens.cpu().numpy().copy())
            lgs.append(dec.logits.cpu().numpy().copy())
        dec.check_status()
        assert int(dec.positions[0]) == prompt.shape[1] + 8 and int(dec.lens[0]) == prompt.shape[1] + 9
        outs.append((np.stack(toks), np.stack(lgs)))
        dec.close()
    (tok_p, lg_p), (tok_s, lg_s) = outs
    assert (tok_p == tok_s).all()
    assert np.abs(lg_p - lg_s).max() <= 0.02 * np.abs(lg_s).max()


@pytest.mark.parametrize("n,d,vocab", [(1, 256, 301), (5, 3200, 1000), (16, 3200, 3001), (9, 128, 77), (8, 4096, 515)])
def test_lm_head_argmax_and_advance(env, n, d, vocab):
    """The library's dense f32 head: logits against a float64 product, the argmax keys against numpy's argmax of the
    kernel's own logits (first index among equal maxima), and the launch that ends a greedy step."""
    t = env.torch
    x = cases.gaussian(600 + n + d, (n, d), 1.0)
    w = cases.gaussian(601 + vocab, (vocab, d), 0.05)
    w[vocab // 3] = w[vocab // 2]  # two identical rows: equal logits for every token
    x[0] = w[vocab // 2] * 5.0     # ... and token 0 points at them, so its maximum is a tie
    xd, wd = t.from_numpy(x).cuda(), t.from_numpy(w).cuda()
    logits = t.zeros((n, vocab), device="cuda")
    keys = t.zeros(n, dtype=t.int64, device="cuda")
    tokens = t.full((n,), -1, dtype=t.int64, device="cuda")
    pos = t.arange(n, dtype=t.int32, device="cuda")
    lens = t.arange(n, dtype=t.int32, device="cuda") + 1
    rows = t.arange(n, dtype=t.int64, device="cuda") * 100
    for rep in range(2):  # the second pass checks that the keys were cleared
        env.cabi.check(env.lib.kb_lm_head_argmax(xd.data_ptr(), n, d, wd.data_ptr(), vocab, logits.data_ptr(), keys.data_ptr(), env.sp))
        env.cabi.check(env.lib.kb_decode_advance(keys.data_ptr(), n, tokens.data_ptr(), pos.data_ptr(), lens.data_ptr(), rows.data_ptr(), env.sp))
        t.cuda.synchronize()
        lg = logits.cpu().numpy()
        ref = x.astype(np.float64) @ w.astype(np.float64).T
        assert np.abs(lg - ref).max() <= 1e-5 * np.abs(ref).max()
        assert (tokens.cpu().numpy() == lg.argmax(axis=1)).all()
        assert int(tokens[0]) == min(vocab // 3, vocab // 2)
        assert (keys.cpu().numpy() == 0).all()
        assert (pos.cpu().numpy() == np.arange(n) + rep + 1).all() and (lens.cpu().numpy() == np.arange(n) + rep + 2).all()
        assert (rows.cpu().numpy() == np.arange(n) * 100 + rep + 1).all()
    # without a logits buffer the keys are the same
    env.cabi.check(env.lib.kb_lm_head_argmax(xd.data_ptr(), n, d, wd.data_ptr(), vocab, None, keys.data_ptr(), env.sp))
    env.cabi.check(env.lib.kb_decode_advance(keys.data_ptr(), n, tokens.data_ptr(), None, None, None, env.sp))
    t.cuda.synchronize()
    assert (tokens.cpu().numpy() == logits.cpu().numpy().argmax(axis=1)).all()
