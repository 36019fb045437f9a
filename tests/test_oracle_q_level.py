"""Q level (W2A8) of the oracle: quantisers, int32 accumulation and the bridge identity
that ties it to the reference's f32 matmul.

Bridge: the reference's f32 accumulation of weight x activation is exact integer
arithmetic when activations are integer-valued with |x| <= 127 and
127*max|w|*K < 2^24.  Feeding its ternary_matmul / quat_matmul the int8-quantised
activations cast to f32, with unit row scales, therefore returns exactly the int32
accumulators.
"""
import numpy as np
import pytest

from oracle import kbref, np_ref
from tests import cases

T, Q = kbref.TERNARY, kbref.QUATERNARY


def test_act_quant_matches_numpy_and_edge_cases():
    x = cases.gaussian(21, (9, 77), 1.0)
    x[3] = 0.0  # all-zero token -> scale 1.0, all codes 0
    x[4, 5] = 1e4  # outlier token
    x[5] = 1e-9  # below the 1e-8 guard
    xq, sx, sumq = kbref.quantize_act_i8(x, ldq=80)
    q2, s2, sum2 = np_ref.quantize_act_i8(x)
    assert (xq[:, :77] == q2).all() and (xq[:, 77:] == 0).all()
    assert (sx == s2).all() and (sumq == sum2).all()
    assert sx[3] == 1.0 and not xq[3].any() and sx[5] == 1.0
    assert np.abs(xq).max() == 127 and xq.min() >= -127


def test_act_quant_rounds_half_to_even():
    x = np.array([[127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 63.5]], np.float32)
    xq, sx, _ = kbref.quantize_act_i8(x)
    assert sx[0] == 1.0
    assert list(xq[0]) == [127, 0, 2, 2, 0, -2, -2, 64]


def test_absmean_matches_numpy_and_zero_fraction():
    w = cases.gaussian(31, (48, 200), 0.02)
    packed, scales = kbref.pack_weights_ternary_absmean(w, 48, 200)
    tr2, s2 = np_ref.absmean_ternarise(w)
    assert (scales == s2).all()
    assert (np_ref.decode_ternary(packed, 48, 200) == tr2).all()
    zero_frac = (tr2 == 0).mean()
    assert 0.27 < zero_frac < 0.36  # |w| < s/2 for a half-normal: about 31 %


@pytest.mark.parametrize("kind,quantiser", [(T, "reference"), (T, "absmean"), (Q, "reference")])
@pytest.mark.parametrize("m,k,n", [(128, 256, 32), (16, 5, 3), (33, 1000, 1), (8, 20, 4)])
def test_bridge_identity(kind, quantiser, m, k, n):
    w = cases.gaussian(100 + m + k, (m, k), 0.02)
    packed, scales = cases.make_weights(kind, quantiser, w)
    x = cases.gaussian(200 + n, (n, k), 1.0)
    xq, sx, sumq = kbref.quantize_act_i8(x)
    w_i8 = kbref.decode_weights_i8(kind, packed, m, k)
    acc = kbref.acc_i32(w_i8, xq, threads=2)
    assert (acc == np_ref.acc_i32(w_i8, xq)).all()
    ones = np.ones(m, np.float32)
    b = np.ascontiguousarray(xq.astype(np.float32).T)  # [K,N]
    fn = kbref.ternary_matmul if kind == T else kbref.quat_matmul
    c = fn(packed, ones, b, m, n, k)
    assert (c == acc.T.astype(np.float32)).all()
    # sum-of-codes identity used by the kernels: acc = mul*sum(code*x) - off*sum(x)
    codes = (w_i8.astype(np.int32) + 1) if kind == T else ((w_i8.astype(np.int32) + 3) // 2)
    mul, off = (1, 1) if kind == T else (2, 3)
    s_code = xq.astype(np.int64) @ codes.astype(np.int64).T
    assert (mul * s_code - off * sumq[:, None] == acc).all()


@pytest.mark.parametrize("kind", [T, Q])
def test_q_forward_against_r_on_dequantised_activations(kind):
    """f32 outputs of the integer path agree with the reference arithmetic fed the
    dequantised activations to 1e-5 of each output row's largest magnitude."""
    m, k, n = 128, 256, 32
    w = cases.gaussian(1001, (m, k), 0.02)
    packed, scales = cases.make_weights(kind, "reference", w)
    bias = cases.gaussian(5, (m,), 0.1)
    x = cases.gaussian(1002, (n, k), 1.0)
    y, acc = kbref.q_forward(kind, packed, scales, bias, m, k, x, threads=2)
    xq, sx, _ = kbref.quantize_act_i8(x)
    assert (y == np_ref.dequant(acc, scales, sx, bias)).all()
    x_deq = (xq.astype(np.float32) * sx[:, None]).astype(np.float32)
    y_r = kbref.linear_forward(kind, packed, scales, bias, m, k, x_deq)
    tol = 1e-5 * np.abs(y_r).max(axis=1, keepdims=True)
    assert (np.abs(y - y_r) <= tol + 1e-7).all()


def test_q_forward_exact_on_integer_activations():
    """With integer activations and max|x| = 127 the activation quantiser is the identity,
    so the integer path reproduces the reference's BitLinear forward bit for bit."""
    m, k, n = 24, 50, 6
    w = cases.gaussian(77, (m, k), 0.02)
    packed, scales = kbref.pack_weights_ternary(w, m, k, 0.3)
    x = cases.integer_activations(78, n, k)
    y, _ = kbref.q_forward(T, packed, scales, None, m, k, x)
    assert (y == kbref.linear_forward(T, packed, scales, None, m, k, x)).all()
