"""Pins the CPU oracle against the known answers held by the reference's own unit tests
(tests/golden/reference_kats.json) and cross-checks the C restatement against the
independent numpy restatement."""
import numpy as np
import pytest

from oracle import kbref, np_ref
from tests import cases

T, Q = kbref.TERNARY, kbref.QUATERNARY


# ---- codecs -------------------------------------------------------------------
def test_all_zero_trits_is_121(kats):
    c = kats["codec"]["all_zero_trits_byte"]
    assert kbref.encode_trits5(c["trits"]) == c["byte"]
    assert list(kbref.decode_trits5(c["byte"])) == c["trits"]


def test_trit_roundtrip(kats):
    tr = kats["codec"]["trit_roundtrip"]["trits"]
    assert list(kbref.decode_trits5(kbref.encode_trits5(tr))) == tr


def test_every_byte_roundtrips(kats):
    r = kats["codec"]["byte_roundtrip_range"]
    for b in range(r["lo"], r["hi"] + 1):
        assert kbref.encode_trits5(kbref.decode_trits5(b)) == b


def test_bytes_above_242_decode_to_zero():
    for b in range(243, 256):
        assert not kbref.decode_trits5(b).any()


def test_lut_matches_numpy_restatement():
    lut = np_ref.ternary_lut()
    for b in range(256):
        assert (kbref.decode_trits5(b) == lut[b]).all()


def test_quat_pack_unpack_and_values(kats):
    q = kats["codec"]["quat_roundtrip"]
    byte = kbref.pack_quats4(q["codes"])
    assert byte == 0b11100100
    assert list(kbref.unpack_quats4(byte)) == q["codes"]
    assert [kbref.quat_value(c) for c in q["codes"]] == q["values"]


def test_pack_sizes(kats):
    p = kats["codec"]["pack_sizes"]
    assert kbref.pack_ternary(np.ones(p["n_trits"], np.int8)).size == p["trit_bytes"]
    assert kbref.pack_quaternary(np.full(p["n_quats"], 2, np.uint8)).size == p["quat_bytes"]


# ---- quantisers ---------------------------------------------------------------
def test_quantize_ternary_kat(kats):
    c = kats["quantize"]["ternary"]
    tr, s = kbref.quantize_ternary(c["w"], c["threshold"])
    assert list(tr[:3]) == c["first_trits"] and s > 0


def test_quantize_quaternary_kat(kats):
    c = kats["quantize"]["quaternary"]
    codes, s = kbref.quantize_quaternary(c["w"])
    assert codes[0] == c["code0"] and codes[3] == c["code3"] and s > 0


def test_quat_roundtrip_within_tol(kats):
    c = kats["quantize"]["quat_roundtrip"]
    codes, s = kbref.quantize_quaternary(c["w"])
    rec = np.array([kbref.quat_value(x) * s for x in codes])
    assert np.abs(rec - np.array(c["w"])).max() < c["tol"]


def test_ternary_roundtrip_signs(kats):
    c = kats["quantize"]["ternary_roundtrip"]
    tr, s = kbref.quantize_ternary(c["w"], c["threshold"])
    assert list(np.sign(tr[:3] * s).astype(int)) == c["signs"]


def test_quat_pack_unit_scales(kats):
    c = kats["quantize"]["quat_pack_unit_scales"]
    packed, scales = kbref.pack_weights_quaternary(np.array(c["w"], np.float32), c["m"], c["k"])
    assert packed.size == c["packed_len"]
    assert np.abs(scales - np.array(c["scales"])).max() < c["tol"]
    assert list(packed) == [0b11100100, 0b00011011]


def test_ternary_pack_len(kats):
    c = kats["quantize"]["ternary_pack_len"]
    packed, scales = kbref.pack_weights_ternary(np.array(c["w"], np.float32), c["m"], c["k"], c["threshold"])
    assert packed.size == c["packed_len"] and scales.size == 2 and scales[0] > 0


def test_zero_row_gets_unit_scale():
    w = np.zeros((2, 7), np.float32)
    assert (kbref.pack_weights_ternary(w, 2, 7, 0.3)[1] == 1.0).all()
    assert (kbref.pack_weights_quaternary(w, 2, 7)[1] == 1.0).all()
    assert (kbref.pack_weights_ternary_absmean(w, 2, 7)[1] == 1.0).all()


# ---- matmul known answers -----------------------------------------------------
def _run_r(kind, packed, scales, b, m, n, k):
    if kind == T:
        return kbref.ternary_matmul(packed, scales, b, m, n, k)
    return kbref.quat_matmul(packed, scales, b, m, n, k)


@pytest.mark.parametrize("idx", range(7))
def test_matmul_packed_kats(kats, idx):
    c = kats["matmul_packed"][idx]
    kind = cases.kind_id(c["kind"])
    packed = cases.packed_from_kat(c)
    m, n, k = c["m"], c["n"], c["k"]
    b = np.array(c["b"], np.float32).reshape(k, n)
    expect = np.array(c["expect"], np.float32).reshape(m, n)
    got = _run_r(kind, packed, c["scales"], b, m, n, k)
    assert np.abs(got - expect).max() < c["tol"]
    # every matmul KAT has an exactly representable answer: the oracle must hit it exactly
    assert (got == expect).all()
    # scale-after-sum statements (edge runtime, CUDA kernel) agree on these inputs
    edge = (kbref.edge_matmul_ternary if kind == T else kbref.edge_matmul_quaternary)(packed, c["scales"], b, m, n, k)
    assert (edge == expect).all()
    # independent numpy restatement agrees bit for bit
    ref2 = (np_ref.ternary_matmul if kind == T else np_ref.quat_matmul)(packed, c["scales"], b, m, n, k)
    assert (ref2 == got).all()


def test_dequant_4x8x3(kats):
    c = kats["dequant_4x8x3"]
    m, k, n = c["m"], c["k"], c["n"]
    packed = np.concatenate([kbref.pack_quaternary(np.array(c["codes_row"], np.uint8))] * m)
    scales = np.full(m, c["scale"], np.float32)
    b = cases.rule(c["b_rule"], k * n).reshape(k, n)
    vals = np.array([kbref.quat_value(x) for x in c["codes_row"]], np.float32)
    expect = np.zeros((m, n), np.float32)
    for i in range(m):
        for j in range(n):
            acc = np.float32(0)
            for p in range(k):
                acc = np.float32(acc + np.float32(vals[p] * b[p, j]))
            expect[i, j] = acc * scales[i]
    got_edge = kbref.edge_matmul_quaternary(packed, scales, b, m, n, k)
    assert (got_edge == expect).all()
    got = kbref.quat_matmul(packed, scales, b, m, n, k)  # scale 0.5 is a power of two: same bits
    assert np.abs(got - expect).max() < c["tol"] and (got == expect).all()


@pytest.mark.parametrize("idx", range(3))
def test_matmul_from_f32_kats(kats, idx):
    c = kats["matmul_from_f32"][idx]
    kind = cases.kind_id(c["kind"])
    m, n, k = c["m"], c["n"], c["k"]
    w = np.array(c["w"], np.float32).reshape(m, k)
    packed, scales = cases.make_weights(kind, "reference", w, c.get("threshold", 0.3))
    b = np.array(c["b"], np.float32).reshape(k, n)
    got = _run_r(kind, packed, scales, b, m, n, k)
    assert np.abs(got - np.array(c["expect"], np.float32).reshape(m, n)).max() < c["tol"]


@pytest.mark.parametrize("idx", range(3))
def test_generator_cases_finite_and_cross_checked(kats, idx):
    c = kats["generator_cases"][idx]
    kind = cases.kind_id(c["kind"])
    m, n, k = c["m"], c["n"], c["k"]
    w = cases.rule(c["w_rule"], m * k).reshape(m, k)
    b = cases.rule(c["b_rule"], k * n).reshape(k, n)
    packed, scales = cases.make_weights(kind, "reference", w, c.get("threshold", 0.3))
    got = _run_r(kind, packed, scales, b, m, n, k)
    assert got.shape == (m, n) and np.isfinite(got).all()
    if kind == T:
        p2, s2 = np_ref.pack_weights_ternary(w, c["threshold"])
        ref2 = np_ref.ternary_matmul(p2, s2, b, m, n, k)
    else:
        p2, s2 = np_ref.pack_weights_quaternary(w)
        ref2 = np_ref.quat_matmul(p2, s2, b, m, n, k)
    assert (p2 == packed).all() and (s2 == scales).all() and (ref2 == got).all()


# ---- layer level --------------------------------------------------------------
def test_bitlinear_approximates_linear(kats):
    c = kats["layer"][0]
    w = np.array(c["w"], np.float32).reshape(c["m"], c["k"])
    packed, scales = kbref.pack_weights_ternary(w, c["m"], c["k"], c["threshold"])
    y = kbref.linear_forward(T, packed, scales, None, c["m"], c["k"], np.array(c["x"], np.float32).reshape(c["x_shape"]))
    assert y.shape == (1, 2) and (y.ravel() == np.array(c["expect"], np.float32)).all()


def test_bitlinear_bias(kats):
    c = kats["layer"][1]
    w = np.array(c["w"], np.float32).reshape(c["m"], c["k"])
    packed, scales = kbref.pack_weights_ternary(w, c["m"], c["k"], c["threshold"])
    y = kbref.linear_forward(T, packed, scales, np.array(c["bias"], np.float32), c["m"], c["k"],
                             np.array(c["x"], np.float32).reshape(c["x_shape"]))
    assert (y.ravel() > np.array(c["greater_than"])).all()
    assert list(y.ravel()) == [11.0, 21.0]


@pytest.mark.parametrize("which", ["bitlinear", "quatlinear"])
def test_forward_shapes(kats, which):
    c = kats["shapes"][which]
    kind = T if which == "bitlinear" else Q
    w = cases.gaussian(7, (c["out"], c["in"]), 1.0)
    packed, scales = cases.make_weights(kind, "reference", w)
    for shp, out in zip(c["inputs"], c["outputs"]):
        y = kbref.linear_forward(kind, packed, scales, None, c["out"], c["in"], np.ones(shp, np.float32))
        assert list(y.shape) == out
    y = kbref.linear_forward(kind, packed, scales, None, c["out"], c["in"], np.ones((2, 3, c["in"]), np.float32))
    assert y.shape == (2, 3, c["out"])
    with pytest.raises(kbref.OracleError) as e:
        kbref.linear_forward(kind, packed, scales, None, c["out"], c["in"], np.ones((2, c["in"] + 1), np.float32))
    assert e.value.code == kbref.ERR_SHAPE


def test_storage_errors():
    packed, scales = kbref.pack_weights_ternary(np.ones((4, 10), np.float32), 4, 10, 0.3)
    b = np.ones((10, 2), np.float32)
    with pytest.raises(kbref.OracleError) as e:
        kbref.ternary_matmul(packed[:-1], scales, b, 4, 2, 10)
    assert e.value.code == kbref.ERR_STORAGE
    with pytest.raises(kbref.OracleError):
        kbref.ternary_matmul(packed, scales[:-1], b, 4, 2, 10)
    pq, sq = kbref.pack_weights_quaternary(np.ones((4, 10), np.float32), 4, 10)
    with pytest.raises(kbref.OracleError):
        kbref.quat_matmul(pq[:-1], sq, b, 4, 2, 10)


def test_compression_ratio_formula(kats):
    for name, kind in (("bitlinear_256_128", T), ("quatlinear_256_128", Q)):
        c = kats["compression"][name]
        bytes_ = c["m"] * kbref.k_packed(kind, c["k"]) + 4 * c["m"]
        assert abs(c["m"] * c["k"] * 4 / bytes_ - c["ratio"]) < 1e-4


def test_dequantize_matches_quantiser():
    w = cases.gaussian(11, (5, 13), 0.02)
    p, s = kbref.pack_weights_ternary(w, 5, 13, 0.3)
    d = kbref.dequantize_weights(T, p, s, 5, 13)
    assert (d == np_ref.decode_ternary(p, 5, 13).astype(np.float32) * s[:, None]).all()
    p, s = kbref.pack_weights_quaternary(w, 5, 13)
    d = kbref.dequantize_weights(Q, p, s, 5, 13)
    assert (d == np_ref.QUAT_VALUES[np_ref.decode_quaternary_codes(p, 5, 13)] * s[:, None]).all()


def test_threaded_rows_match_serial():
    w = cases.gaussian(3, (64, 50), 0.02)
    p, s = kbref.pack_weights_ternary(w, 64, 50, 0.3)
    b = cases.gaussian(4, (50, 5), 1.0)
    assert (kbref.ternary_matmul(p, s, b, 64, 5, 50, threads=4) == kbref.ternary_matmul(p, s, b, 64, 5, 50, threads=1)).all()


def test_ternary_ternary_matmul():
    a = np.array([1.0, -1.0, 0.0, 1.0], np.float32).reshape(2, 2)
    b = np.array([1.0, 0.0, -1.0, 1.0], np.float32).reshape(2, 2)
    pa, sa = kbref.pack_weights_ternary(a, 2, 2, 0.3)
    pb, sb = kbref.pack_weights_ternary(b, 2, 2, 0.3)
    c = kbref.ternary_ternary_matmul(pa, sa, pb, sb, 2, 2, 2)
    assert (c == np.array([[1, -2], [0, 1]], np.float32)).all()
