"""Parity of the CUDA path against the CPU oracle, through the C ABI (needs a B200).

Bar: int32 accumulators equal (==), f32 outputs equal bit for bit where the fixed
epilogue order applies, and within 1e-5 of each output row's largest magnitude against
the reference arithmetic (R level) fed the dequantised activations.
"""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import kbref
from tests import cases

pytestmark = pytest.mark.gpu

T, Q = kbref.TERNARY, kbref.QUATERNARY
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def torch():
    import torch

    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch


@pytest.fixture(scope="module")
def kb():
    import kore_b200
    from kore_b200 import kernels, nn

    return type("KB", (), {"nn": nn, "kernels": kernels, "cabi": kore_b200._cabi})


def _layer(kb, kind, packed, scales, bias, m, k):
    cls = kb.nn.BitLinear if kind == T else kb.nn.QuatLinear
    return cls.from_packed(packed, scales, bias, k, m)


# ---- activation quantiser ------------------------------------------------------
@pytest.mark.parametrize("n,k", [(1, 4096), (32, 256), (3, 77), (5, 1), (2, 8640), (7, 130), (1, 11008)])
def test_act_quant_bit_exact(torch, kb, n, k):
    x = cases.gaussian(10 * n + k, (n, k), 1.0)
    if n > 2:
        x[1] = 0.0
        x[2] *= 1e-10
    xq_ref, sx_ref, sum_ref = kbref.quantize_act_i8(x, ldq=kb.kernels.act_ld(k))
    xq, sx, sumq = kb.kernels.quantize_act_i8(torch.from_numpy(x).cuda())
    assert (xq.cpu().numpy() == xq_ref).all()
    assert (sx.cpu().numpy() == sx_ref).all()
    assert (sumq.cpu().numpy() == sum_ref).all()


def test_act_quant_rounding_ties_and_neighbours(torch, kb):
    """Values placed on and next to rounding ties (j + 0.5) * s: the kernel's
    multiply-by-reciprocal shortcut must still agree with the IEEE division everywhere."""
    rows = []
    for amax in (127.0, 1.0, 3.3333, 0.017, 1234.567, 2.0 ** -20):
        s = np.float32(np.float32(amax) / np.float32(127.0))
        j = np.arange(-127, 127, dtype=np.float32)
        tie = ((j + np.float32(0.5)) * s).astype(np.float32)
        vals = np.concatenate([tie, np.nextafter(tie, np.float32(np.inf)), np.nextafter(tie, np.float32(-np.inf)),
                               (j * s).astype(np.float32)])
        vals = np.clip(vals, -np.float32(amax), np.float32(amax))
        vals[0] = np.float32(amax)
        rows.append(vals.astype(np.float32))
    x = np.stack(rows)
    xq_ref, sx_ref, sum_ref = kbref.quantize_act_i8(x, ldq=kb.kernels.act_ld(x.shape[1]))
    xq, sx, sumq = kb.kernels.quantize_act_i8(torch.from_numpy(x).cuda())
    assert (sx.cpu().numpy() == sx_ref).all()
    assert (xq.cpu().numpy() == xq_ref).all()
    assert (sumq.cpu().numpy() == sum_ref).all()
    # the same rows through the fused GEMV prologue (identity-like layer exposes the codes)
    k = x.shape[1]
    w = np.zeros((k, k), np.float32)
    np.fill_diagonal(w, 1.0)
    lay = kb.nn.BitLinear.new(w, None, 0.3)
    for r in range(x.shape[0]):
        _, acc = lay.forward(torch.from_numpy(x[r:r + 1]).cuda(), path=kb.cabi.PATH_GEMV, return_acc=True)
        assert (acc.cpu().numpy()[0] == xq_ref[r, :k].astype(np.int32)).all()


def test_act_quant_unaligned_rows(torch, kb):
    # a view whose rows start 4 bytes off a 16-byte boundary takes the scalar-load path
    big = torch.from_numpy(cases.gaussian(5, (1, 3 * 256 + 1), 1.0)).cuda()
    x = big[0, 1:].reshape(3, 256)
    xq, sx, sumq = kb.kernels.quantize_act_i8(x)
    xq_ref, sx_ref, sum_ref = kbref.quantize_act_i8(x.cpu().numpy())
    assert (xq.cpu().numpy() == xq_ref).all() and (sx.cpu().numpy() == sx_ref).all()


# ---- load-time formats -----------------------------------------------------------
@pytest.mark.parametrize("kind", [T, Q])
@pytest.mark.parametrize("m,k", [(128, 256), (3, 5), (2, 7), (8, 20), (130, 1000), (1, 1)])
def test_wire_format_roundtrip_and_dequantize(kb, kind, m, k):
    w = cases.gaussian(m * 31 + k, (m, k), 0.02)
    packed, scales = cases.make_weights(kind, "reference", w)
    lay = _layer(kb, kind, packed, scales, None, m, k)
    assert (lay.packed_weights() == packed).all()
    assert (lay.scales() == scales).all()
    assert (lay.dequantize_weights() == kbref.dequantize_weights(kind, packed, scales, m, k)).all()
    ref_bytes = m * kbref.k_packed(kind, k) + 4 * m
    assert lay.weight_memory_bytes() == ref_bytes
    assert abs(lay.compression_ratio() - m * k * 4 / ref_bytes) < 1e-3


def test_bytes_above_242_decode_to_zero_trits(kb):
    packed = np.array([250, 121, 243, 255], np.uint8)  # 2 rows x 2 bytes, K = 10
    lay = kb.nn.BitLinear.from_packed(packed, np.ones(2, np.float32), None, 10, 2)
    assert not lay.dequantize_weights().any()


@pytest.mark.parametrize("kind,quantiser", [(T, "reference"), (T, "absmean"), (Q, "reference")])
@pytest.mark.parametrize("m,k", [(128, 256), (5, 13), (64, 1000)])
def test_device_quantiser_matches_oracle(kb, kind, quantiser, m, k):
    w = cases.gaussian(m + 7 * k, (m, k), 0.02)
    w[m // 2] = 0.0  # an all-zero row gets scale 1.0
    packed, scales = cases.make_weights(kind, quantiser, w)
    if kind == T:
        lay = kb.nn.BitLinear.new(w, None, 0.3, quantiser=quantiser)
    else:
        lay = kb.nn.QuatLinear.new(w)
    assert (lay.scales() == scales).all()
    assert (lay.packed_weights() == packed).all()


def test_pack_weights_functions(kb):
    w = cases.gaussian(99, (24, 50), 0.02)
    p, s = kb.kernels.pack_weights_ternary(w, 24, 50, 0.3)
    pr, sr = kbref.pack_weights_ternary(w, 24, 50, 0.3)
    assert (p == pr).all() and (s == sr).all()
    p, s = kb.kernels.pack_weights_quaternary(w, 24, 50)
    pr, sr = kbref.pack_weights_quaternary(w, 24, 50)
    assert (p == pr).all() and (s == sr).all()


# ---- forward: both kernels against the Q oracle -----------------------------------
SHAPES = [
    # m, k, n
    (128, 256, 1), (128, 256, 32), (8, 20, 4), (2, 7, 3), (16, 32, 16), (1, 1, 1), (130, 1000, 5),
    (300, 4096, 2), (257, 2304, 8), (64, 5, 9), (200, 640, 70), (129, 384, 130), (256, 512, 300),
    # GEMV with more row groups than one round of the persistent grid (grid-stride rounds, ragged last one)
    (14400, 256, 1), (14270, 130, 2), (14500, 384, 8), (28800, 128, 4),
    # small-batch kernel: K steps fewer / more than its 16 warps, ragged rows and tokens
    (50, 8640, 16), (3200, 3200, 12), (17, 4352, 27),
    # CTA-pair GEMM edges: odd number of 128-row blocks, odd number of 128-byte K slabs, ragged tokens
    (384, 640, 520), (130, 128, 257),
    # medium-batch GEMM with K split over CTAs (few row tiles, long rows): ragged last split, both token tiles
    (300, 8640, 100), (3200, 2048, 64), (1000, 4224, 40),
]


@pytest.mark.parametrize("path", ["gemv", "gemv_shared", "gemv_mma", "gemv_stream", "gemm_tc"])
@pytest.mark.parametrize("kind,quantiser", [(T, "reference"), (T, "absmean"), (Q, "reference")])
@pytest.mark.parametrize("m,k,n", SHAPES)
def test_forward_bit_exact(torch, kb, path, kind, quantiser, m, k, n):
    if path.startswith("gemv") and n > 40:
        pytest.skip("decode kernel is exercised up to a few token groups")
    if path in ("gemv_mma", "gemv_stream") and n > 32:
        pytest.skip("small-batch kernels take up to 32 tokens")
    if path == "gemv_stream" and n > 8 and k > 8192:
        pytest.skip("more than 8 tokens of K > 8192 do not fit in the streaming kernel's shared memory")
    w = cases.gaussian(1000 + m + k, (m, k), 0.02)
    packed, scales = cases.make_weights(kind, quantiser, w)
    bias = cases.gaussian(3, (m,), 0.1) if (m + n) % 2 else None
    x = cases.gaussian(2000 + n + k, (n, k), 1.0)
    y_ref, acc_ref = kbref.q_forward(kind, packed, scales, bias, m, k, x, threads=4)
    lay = _layer(kb, kind, packed, scales, bias, m, k)
    p = {"gemv": kb.cabi.PATH_GEMV, "gemv_shared": kb.cabi.PATH_GEMV_SHARED, "gemv_mma": kb.cabi.PATH_GEMV_MMA,
         "gemv_stream": kb.cabi.PATH_GEMV_STREAM, "gemm_tc": kb.cabi.PATH_GEMM_TC}[path]
    y, acc = lay.forward(torch.from_numpy(x).cuda(), path=p, return_acc=True)
    torch.cuda.synchronize()
    st = C.c_int(0)
    assert kb.cabi.lib().kb_linear_last_device_status(lay.handle, None, C.byref(st)) == 0, st.value
    assert (acc.cpu().numpy() == acc_ref).all()
    assert (y.cpu().numpy() == y_ref).all()
    # 1e-5 relative (to the row's largest output) against the reference arithmetic on the
    # dequantised activations
    xq, sx, _ = kbref.quantize_act_i8(x)
    y_r = kbref.linear_forward(kind, packed, scales, bias, m, k, (xq.astype(np.float32) * sx[:, None]).astype(np.float32))
    tol = 1e-5 * np.abs(y_r).max(axis=1, keepdims=True) + 1e-7
    assert (np.abs(y.cpu().numpy() - y_r) <= tol).all()


# ---- the benchmark specification's full sizes: size-independent properties + sampled exact rows ---------
FULL_SIZES = [
    # name, m, k, n, kind
    ("decode_4096x4096_b1", 4096, 4096, 1, T),
    ("decode_4096x4096_b16_quat", 4096, 4096, 16, Q),
    ("prefill_up_2048tok", 11008, 4096, 2048, T),
    ("prefill_down_2048tok", 4096, 11008, 2048, T),
    ("ffn70b_8192x28672_b1", 28672, 8192, 1, T),
    ("ffn70b_8192x28672_b8", 28672, 8192, 8, T),
    ("ffn70b_8192x28672_b16", 28672, 8192, 16, T),
    ("ffn70b_8192x28672_b64", 28672, 8192, 64, T),
    ("ffn70b_8192x28672_b512", 28672, 8192, 512, T),
    # the decoder configuration's projections: q|k|v concatenated, gate/up interleaved, down (K = 8640
    # is a multiple of 64 but not of 128: the last K tile is masked)
    ("decoder_qkv_9600x3200_b1", 9600, 3200, 1, T),
    ("decoder_qkv_9600x3200_b16", 9600, 3200, 16, T),
    ("decoder_gate_up_17280x3200_b1", 17280, 3200, 1, T),
    ("decoder_gate_up_17280x3200_b16", 17280, 3200, 16, T),
    ("decoder_down_3200x8640_b1", 3200, 8640, 1, T),
    ("decoder_down_3200x8640_b16", 3200, 8640, 16, T),
]


@pytest.mark.parametrize("name,m,k,n,kind", FULL_SIZES)
def test_full_size_checksum_and_sampled_rows(torch, kb, name, m, k, n, kind):
    """At full size the oracle cannot afford every output, so: (1) checksum of checksums —
    sum over output features of the int32 accumulators equals xq . (column sums of W), an
    identity that touches every weight and every activation; (2) 48 sampled output features
    are compared exactly (accumulators and f32 outputs) against the oracle for all tokens."""
    g = torch.Generator().manual_seed(sum(name.encode()) % 1000)
    w = (torch.randn((m, k), generator=g) * 0.02).numpy()
    x = torch.randn((n, k), generator=g).numpy()
    if kind == T:
        lay = kb.nn.BitLinear.new(w, None, 0.3, quantiser="absmean")
    else:
        lay = kb.nn.QuatLinear.new(w)
    del w
    packed, scales = lay.packed_weights(), lay.scales()
    y, acc = lay.forward(torch.from_numpy(x).cuda(), return_acc=True)
    torch.cuda.synchronize()
    st = C.c_int(0)
    assert kb.cabi.lib().kb_linear_last_device_status(lay.handle, None, C.byref(st)) == 0, st.value
    acc_h, y_h = acc.cpu().numpy(), y.cpu().numpy()
    xq, sx, _ = kbref.quantize_act_i8(x)
    w_i8 = kbref.decode_weights_i8(kind, packed, m, k)
    colsum = w_i8.sum(axis=0, dtype=np.int64)
    assert (acc_h.astype(np.int64).sum(axis=1) == xq.astype(np.int64) @ colsum).all()
    rows = np.random.default_rng(1).choice(m, size=48, replace=False)
    acc_ref = kbref.acc_i32(np.ascontiguousarray(w_i8[rows]), xq, threads=8)
    assert (acc_h[:, rows] == acc_ref).all()
    assert (y_h[:, rows] == kbref.dequant_epilogue(acc_ref, scales[rows], sx)).all()
    assert np.isfinite(y_h).all()


# token counts x K at which the decode GEMV's activation stage is exactly 48 KiB (the default
# shared-memory limit once the kernel's static arrays are added) or just beside it
@pytest.mark.parametrize("n,k", [(3, 11008), (4, 12288), (8, 6144), (5, 5120), (2, 24576), (8, 5000)])
@pytest.mark.parametrize("kind", [T, Q])
def test_gemv_at_the_shared_memory_opt_in_boundary(torch, kb, kind, n, k):
    m = 200
    w = cases.gaussian(31 * n + k, (m, k), 0.02)
    packed, scales = cases.make_weights(kind, "absmean" if kind == T else "reference", w)
    bias = cases.gaussian(4, (m,), 0.1)
    x = cases.gaussian(77 + n, (n, k), 1.0)
    y_ref, acc_ref = kbref.q_forward(kind, packed, scales, bias, m, k, x, threads=4)
    lay = _layer(kb, kind, packed, scales, bias, m, k)
    xd = torch.from_numpy(x).cuda()
    for p in (kb.cabi.PATH_GEMV, kb.cabi.PATH_AUTO):
        y, acc = lay.forward(xd, path=p, return_acc=True)
        assert (acc.cpu().numpy() == acc_ref).all() and (y.cpu().numpy() == y_ref).all()
    xq, sx, sumq = kb.kernels.quantize_act_i8(xd)
    assert (kb.kernels.forward_q8(lay, xq, sx, sumq, path=kb.cabi.PATH_GEMV).cpu().numpy() == y_ref).all()
    # the allocation-free entry point takes the same kernel for up to 8 tokens
    ys = torch.empty((n, m), dtype=torch.float32, device="cuda")
    kb.cabi.check(kb.cabi.lib().kb_linear_forward_static(lay.handle, xd.data_ptr(), n, k, ys.data_ptr(), None))
    assert (ys.cpu().numpy() == y_ref).all()


# ---- ReLU in the epilogue (cuda/ops.rs:828-878 in layer form) -----------------------------
@pytest.mark.parametrize("kind", [T, Q])
@pytest.mark.parametrize("m,k,n", [(128, 256, 1), (130, 1000, 5), (257, 2304, 12), (200, 640, 70), (384, 640, 300)])
def test_relu_epilogue(torch, kb, kind, m, k, n):
    w = cases.gaussian(500 + m + k, (m, k), 0.02)
    packed, scales = cases.make_weights(kind, "reference", w)
    bias = cases.gaussian(6, (m,), 0.1)
    x = cases.gaussian(600 + n, (n, k), 1.0)
    y_ref = np.maximum(kbref.q_forward(kind, packed, scales, bias, m, k, x, threads=4)[0], np.float32(0.0))
    assert (y_ref == 0).any() and (y_ref > 0).any()
    lay = _layer(kb, kind, packed, scales, bias, m, k)
    paths = [kb.cabi.PATH_AUTO, kb.cabi.PATH_GEMM_TC] + ([kb.cabi.PATH_GEMV] if n <= 8 else []) + ([kb.cabi.PATH_GEMV_MMA] if n <= 32 else [])
    for p in paths:
        y = lay.forward_relu(torch.from_numpy(x).cuda(), path=p)
        assert (y.cpu().numpy() == y_ref).all(), p
    if kind == Q:
        # kernel-shaped one-shot: b [K,N] in, c [M,N] out, bias per weight row
        c = kb.kernels.quat_matmul_bias_relu(packed, scales, np.ascontiguousarray(x.T), bias, m, n, k)
        assert (c == y_ref.T).all()
        with pytest.raises(kb.nn.KoreError) as e:
            kb.kernels.quat_matmul_bias_relu(packed, scales, np.ascontiguousarray(x.T), bias[:-1], m, n, k)
        assert e.value.code == kb.cabi.ERR_STORAGE


def test_auto_path_matches_and_host_entry(torch, kb):
    m, k = 384, 1024
    w = cases.gaussian(42, (m, k), 0.02)
    packed, scales = cases.make_weights(T, "absmean", w)
    lay = _layer(kb, T, packed, scales, None, m, k)
    for n in (1, 8, 9, 64, 200):
        x = cases.gaussian(n, (n, k), 1.0)
        y_ref, _ = kbref.q_forward(T, packed, scales, None, m, k, x, threads=4)
        assert (lay(x) == y_ref).all()  # numpy in -> host entry point
        assert (lay(torch.from_numpy(x).cuda()).cpu().numpy() == y_ref).all()
    # n-d and 1-d inputs keep their leading shape (bit_linear.rs:193-234)
    x3 = cases.gaussian(77, (2, 3, k), 1.0)
    y3 = lay(x3)
    assert y3.shape == (2, 3, m)
    assert (y3.reshape(6, m) == kbref.q_forward(T, packed, scales, None, m, k, x3.reshape(6, k))[0]).all()
    assert lay(x3[0, 0]).shape == (m,)


# ---- the reference's own known answers, on the GPU ---------------------------------
def test_reference_kats_exact_through_q8_entry(torch, kb, kats):
    """Integer-valued activations go in as int8 codes with unit scales, so the kernels
    must return the reference tests' exact answers."""
    for c in kats["matmul_packed"]:
        kind = cases.kind_id(c["kind"])
        m, n, k = c["m"], c["n"], c["k"]
        b = np.array(c["b"], np.float32).reshape(k, n)
        assert (b == np.rint(b)).all() and np.abs(b).max() <= 127
        lay = _layer(kb, kind, cases.packed_from_kat(c), np.array(c["scales"], np.float32), None, m, k)
        ld = kb.kernels.act_ld(k)
        xq = np.zeros((n, ld), np.int8)
        xq[:, :k] = b.T.astype(np.int8)
        for p in (kb.cabi.PATH_GEMV, kb.cabi.PATH_GEMM_TC):
            y = kb.kernels.forward_q8(lay, torch.from_numpy(xq).cuda(), torch.ones(n, device="cuda"),
                                      torch.from_numpy(xq.astype(np.int32).sum(1).astype(np.int32)).cuda(), path=p)
            got = y.cpu().numpy().T  # [M,N] like the reference kernels
            assert (got == np.array(c["expect"], np.float32).reshape(m, n)).all(), (c["name"], p, got)


def test_reference_kats_with_reference_tolerances(kb, kats):
    """Through the f32 entry points (activations quantised to int8 on the way) the loosely
    toleranced reference assertions still hold."""
    for c in kats["matmul_from_f32"]:
        kind = cases.kind_id(c["kind"])
        m, n, k = c["m"], c["n"], c["k"]
        w = np.array(c["w"], np.float32).reshape(m, k)
        if kind == T:
            p, s = kb.kernels.pack_weights_ternary(w, m, k, c["threshold"])
            got = kb.kernels.ternary_matmul(p, s, np.array(c["b"], np.float32).reshape(k, n), m, n, k)
        else:
            p, s = kb.kernels.pack_weights_quaternary(w, m, k)
            got = kb.kernels.quat_matmul(p, s, np.array(c["b"], np.float32).reshape(k, n), m, n, k)
        assert np.abs(got - np.array(c["expect"], np.float32).reshape(m, n)).max() < c["tol"]
    c = kats["layer"][0]
    lay = kb.nn.BitLinear.new(np.array(c["w"], np.float32).reshape(c["m"], c["k"]), None, c["threshold"])
    y = lay(np.array(c["x"], np.float32).reshape(c["x_shape"]))
    assert np.abs(y.ravel() - np.array(c["expect"])).max() < c["tol"]
    c = kats["layer"][1]
    lay = kb.nn.BitLinear.new(np.array(c["w"], np.float32).reshape(c["m"], c["k"]), np.array(c["bias"], np.float32), c["threshold"])
    y = lay(np.array(c["x"], np.float32).reshape(c["x_shape"]))
    assert (y.ravel() > np.array(c["greater_than"])).all()
    assert [p[0] for p in lay.named_parameters()] == ["bias"] and len(lay.parameters()) == 1


def test_generator_cases_and_config1_against_golden(torch, kb, kats):
    rec = np.load(os.path.join(ROOT, "tests", "golden", "recorded.npz"))
    for c in kats["generator_cases"]:
        kind = cases.kind_id(c["kind"])
        m, n, k = c["m"], c["n"], c["k"]
        w = cases.rule(c["w_rule"], m * k).reshape(m, k)
        b = cases.rule(c["b_rule"], k * n).reshape(k, n)
        packed, scales = cases.make_weights(kind, "reference", w, c.get("threshold", 0.3))
        fn = kb.kernels.ternary_matmul if kind == T else kb.kernels.quat_matmul
        got = fn(packed, scales, b, m, n, k)
        assert got.shape == (m, n) and np.isfinite(got).all()
        assert (got.T == rec[f"gen_{c['name']}_q_y"]).all()
    w = cases.gaussian(1001, (128, 256), 0.02)
    x = cases.gaussian(1002, (32, 256), 1.0)
    for name, kind, quantiser in (("tern_ref", T, "reference"), ("tern_absmean", T, "absmean"), ("quat", Q, "reference")):
        lay = kb.nn.BitLinear.new(w, None, 0.3, quantiser=quantiser) if kind == T else kb.nn.QuatLinear.new(w)
        for p in (kb.cabi.PATH_GEMV, kb.cabi.PATH_GEMM_TC):
            y, acc = lay.forward(torch.from_numpy(x).cuda(), path=p, return_acc=True)
            assert (acc.cpu().numpy() == rec[f"cfg1_{name}_q_acc"]).all()
            assert (y.cpu().numpy() == rec[f"cfg1_{name}_q_y"]).all()


# ---- errors and module surface --------------------------------------------------------
def test_errors_mirror_the_reference(torch, kb):
    lay = kb.nn.BitLinear(16, 8, bias=False)
    with pytest.raises(kb.nn.KoreError) as e:
        lay(np.ones((4, 17), np.float32))
    assert e.value.code == kb.cabi.ERR_SHAPE
    with pytest.raises(kb.nn.KoreError):
        lay(np.float32(1.0))
    with pytest.raises(kb.nn.KoreError) as e:
        lay(torch.ones(4, 16, device="cuda", dtype=torch.float16))
    assert e.value.code == kb.cabi.ERR_DTYPE
    p, s = kbref.pack_weights_ternary(np.ones((4, 10), np.float32), 4, 10, 0.3)
    with pytest.raises(kb.nn.KoreError) as e:
        kb.kernels.ternary_matmul(p[:-1], s, np.ones((10, 2), np.float32), 4, 2, 10)
    assert e.value.code == kb.cabi.ERR_STORAGE and "a_packed too small: need 8 bytes, got 7" in str(e.value)
    with pytest.raises(kb.nn.KoreError) as e:
        kb.kernels.quat_matmul(p, s[:-1], np.ones((10, 2), np.float32), 4, 2, 10)
    assert e.value.code == kb.cabi.ERR_STORAGE
    with pytest.raises(kb.nn.KoreError) as e:
        kb.kernels.ternary_matmul(p, s, np.ones((10, 2), np.float64), 4, 2, 10)
    assert e.value.code == kb.cabi.ERR_DTYPE
    with pytest.raises(AssertionError):
        kb.nn.BitLinear.new(np.ones(5, np.float32))


def test_module_surface(kb, kats):
    for which, cls in (("bitlinear", kb.nn.BitLinear), ("quatlinear", kb.nn.QuatLinear)):
        c = kats["shapes"][which]
        lay = cls.random(c["in"], c["out"], False)
        for shp, out in zip(c["inputs"], c["outputs"]):
            assert list(lay(np.ones(shp, np.float32)).shape) == out
        assert lay.parameters() == [] and lay.state_dict()["weight"].shape == (c["out"], c["in"])
        assert which[:4].lower() in repr(lay).lower() and str(c["in"]) in repr(lay)
        assert lay.compression_ratio() > 5.0
        lay.train(True)
        assert lay.is_training()
    big = kb.nn.BitLinear.random(4096, 4096, False)
    assert big.compression_ratio() > 10.0  # bit_linear.rs:356-362
    c = kats["compression"]["bitlinear_256_128"]
    assert abs(kb.nn.BitLinear(256, 128).compression_ratio() - c["ratio"]) < 1e-3
    c = kats["compression"]["quatlinear_256_128"]
    assert abs(kb.nn.QuatLinear(256, 128).compression_ratio() - c["ratio"]) < 1e-3


def test_concurrent_forward_from_many_threads(torch, kb):
    """Module is Send + Sync in the reference: many host threads may call one layer."""
    import threading

    m, k = 256, 512
    w = cases.gaussian(8, (m, k), 0.02)
    packed, scales = cases.make_weights(T, "absmean", w)
    lay = _layer(kb, T, packed, scales, None, m, k)
    xs = [cases.gaussian(100 + i, (1 + 20 * (i % 3), k), 1.0) for i in range(8)]
    refs = [kbref.q_forward(T, packed, scales, None, m, k, x)[0] for x in xs]
    outs = [None] * 8

    def work(i):
        for _ in range(5):
            outs[i] = lay(xs[i])

    ts = [threading.Thread(target=work, args=(i,)) for i in range(8)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    for o, r in zip(outs, refs):
        assert (o == r).all()


# ---- both operands ternary (cpu_ternary_matmul.rs:131-193) ---------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(2, 2, 2), (8, 4, 20), (16, 16, 32), (130, 70, 1000), (300, 3, 77), (64, 200, 640), (5, 1, 1)])
def test_ternary_ternary_matmul(kb, m, n, k):
    a = cases.gaussian(7000 + m + k, (m, k), 0.02)
    b = cases.gaussian(7100 + n + k, (n, k), 0.02)
    if (m, n, k) == (2, 2, 2):  # the reference's own case (:293-307)
        a = np.array([[1.0, -1.0], [0.0, 1.0]], np.float32)
        b = np.array([[1.0, 0.0], [-1.0, 1.0]], np.float32)
    pa, sa = kbref.pack_weights_ternary(a, m, k, 0.3)
    pb, sb = kbref.pack_weights_ternary(b, n, k, 0.3)
    c_ref = kbref.ternary_ternary_matmul(pa, sa, pb, sb, m, n, k)
    c = kb.kernels.ternary_ternary_matmul(pa, sa, pb, sb, m, n, k)
    assert c.shape == (m, n)
    assert (c == c_ref).all()
    if (m, n, k) == (2, 2, 2):
        assert (c == np.array([[1, -2], [0, 1]], np.float32)).all()


@pytest.mark.gpu
def test_ternary_ternary_matmul_errors(kb):
    from kore_b200 import KoreError

    pa, sa = kbref.pack_weights_ternary(cases.gaussian(1, (4, 10), 0.02), 4, 10, 0.3)
    with pytest.raises(KoreError) as e:
        kb.kernels.ternary_ternary_matmul(pa[:-1], sa, pa, sa, 4, 4, 10)
    assert "packed arrays too small" in str(e.value)  # :142-146
