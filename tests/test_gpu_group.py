"""Grouped decode launch (`kb_linear_group_forward_q8`) against the CPU oracle: row i of the
output equals layer i applied to token i, bit for bit (needs a B200)."""
import ctypes as C

import numpy as np
import pytest

from oracle import kbref
from tests import cases

pytestmark = pytest.mark.gpu

T, Q = kbref.TERNARY, kbref.QUATERNARY


@pytest.fixture(scope="module")
def torch():
    import torch

    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch


def _make(kind, quantiser, count, m, k, with_bias, seed):
    from kore_b200 import nn

    cls = nn.BitLinear if kind == T else nn.QuatLinear
    layers, raw = [], []
    for i in range(count):
        w = cases.gaussian(seed + 10 * i, (m, k), 0.02)
        packed, scales = cases.make_weights(kind, quantiser, w)
        # only some members carry a bias: the kernel looks the pointer up per layer
        bias = cases.gaussian(seed + 10 * i + 1, (m,), 0.1) if with_bias and i % 2 == 0 else None
        layers.append(cls.from_packed(packed, scales, bias, k, m))
        raw.append((packed, scales, bias))
    return layers, raw


# (count, m, k): ranges inside one layer, ranges spanning many small layers, ragged M and K,
# a single member, two 2048-element chunks per row
SHAPES = [(5, 300, 1000), (1, 130, 77), (40, 8, 64), (7, 33, 4100), (3, 1024, 4096), (150, 4, 16), (12, 1, 5)]


@pytest.mark.parametrize("count,m,k", SHAPES)
@pytest.mark.parametrize("kind,quantiser", [(T, "reference"), (T, "absmean"), (Q, "reference")])
def test_group_matches_oracle_per_layer(torch, kind, quantiser, count, m, k):
    from kore_b200 import nn

    layers, raw = _make(kind, quantiser, count, m, k, True, 1000 + count + m)
    grp = nn.LinearGroup(layers)
    assert len(grp) == count
    from kore_b200 import kernels

    x = cases.gaussian(7 + count, (count, k), 1.0)
    xd = torch.from_numpy(x).cuda()
    y = grp(xd).cpu().numpy()  # f32 in: quantiser in the kernel's prologue
    y_q8 = grp.forward_q8(*kernels.quantize_act_i8(xd)).cpu().numpy()  # quantised beforehand
    assert (y == y_q8).all()
    assert (grp(x) == y).all()  # numpy in: host entry point
    for i, (packed, scales, bias) in enumerate(raw):
        y_ref, _ = kbref.q_forward(kind, packed, scales, bias, m, k, x[i : i + 1], threads=2)
        assert (y[i] == y_ref[0]).all(), f"layer {i}"
    # the same through the per-layer entry point
    for i in (0, count - 1):
        yi = layers[i](torch.from_numpy(x[i : i + 1]).cuda()).cpu().numpy()
        assert (yi[0] == y[i]).all()
    grp.close()


def test_group_strided_output_and_repeat(torch):
    from kore_b200 import kernels, nn

    count, m, k = 9, 200, 520
    layers, raw = _make(T, "absmean", count, m, k, False, 77)
    grp = nn.LinearGroup(layers)
    x = torch.from_numpy(cases.gaussian(3, (count, k), 1.0)).cuda()
    xq, sx, sumq = kernels.quantize_act_i8(x)
    wide = torch.full((count, m + 24), -7.0, dtype=torch.float32, device="cuda")
    out = wide[:, :m]
    for _ in range(3):
        grp.forward_q8(xq, sx, sumq, out=out)
    torch.cuda.synchronize()
    ref = grp.forward_q8(xq, sx, sumq)
    assert (out == ref).all()
    assert (wide[:, m:] == -7.0).all()  # nothing written past a row's end
    grp.close()


def test_group_full_size_pool(torch):
    """The bench's shape: many 4096 x 4096 layers; a checksum of checksums plus sampled rows."""
    from kore_b200 import kernels, nn

    count, m, k = 24, 4096, 4096
    w = cases.gaussian(5, (m, k), 0.02)
    packed, scales = cases.make_weights(T, "absmean", w)
    layers = [nn.BitLinear.from_packed(packed, scales, None, k, m) for _ in range(count)]
    grp = nn.LinearGroup(layers)
    x = cases.gaussian(6, (count, k), 1.0)
    xd = torch.from_numpy(x).cuda()
    y = grp(xd).cpu().numpy()
    xq, sx, sumq = kernels.quantize_act_i8(xd)
    for i in (0, 11, count - 1):
        yi = kernels.forward_q8(layers[i], xq[i : i + 1], sx[i : i + 1], sumq[i : i + 1]).cpu().numpy()
        assert (yi[0] == y[i]).all()
    y_ref, _ = kbref.q_forward(T, packed, scales, None, m, k, x, threads=8)
    assert (y == y_ref).all()
    grp.close()


def test_group_errors(torch):
    from kore_b200 import _cabi, nn

    a, _ = _make(T, "reference", 2, 64, 128, False, 1)
    b, _ = _make(T, "reference", 1, 64, 256, False, 2)
    q, _ = _make(Q, "reference", 1, 64, 128, False, 3)
    with pytest.raises(_cabi.KoreError) as e:
        nn.LinearGroup(a + b)
    assert e.value.code == _cabi.ERR_SHAPE and "shape mismatch" in str(e.value)
    with pytest.raises(_cabi.KoreError):
        nn.LinearGroup(a + q)
    with pytest.raises(_cabi.KoreError):
        nn.LinearGroup([])
    grp = nn.LinearGroup(a)
    with pytest.raises(_cabi.KoreError) as e:
        grp(torch.zeros((3, 128), device="cuda"))
    assert e.value.code == _cabi.ERR_SHAPE
    lib = _cabi.lib()
    assert lib.kb_linear_group_forward_q8(None, None, 0, None, None, None, 0, None) == _cabi.ERR_BAD_HANDLE
    assert lib.kb_linear_group_forward_q8(grp.handle, None, 0, None, None, None, 0, None) == _cabi.ERR_INVALID
    assert lib.kb_linear_group_count(grp.handle) == 2
    assert lib.kb_linear_group_forward(grp.handle, None, 0, None, 0, None) == _cabi.ERR_INVALID
    assert lib.kb_linear_group_forward_host(grp.handle, None, None) == _cabi.ERR_INVALID
    assert lib.kb_linear_group_forward_host(None, None, None) == _cabi.ERR_BAD_HANDLE
    xs = torch.zeros((2, 128), device="cuda")
    ys = torch.zeros((2, 64), device="cuda")
    assert lib.kb_linear_group_forward(grp.handle, xs.data_ptr(), 100, ys.data_ptr(), 0, None) == _cabi.ERR_SHAPE
    assert lib.kb_linear_group_forward(grp.handle, xs.data_ptr(), 0, ys.data_ptr(), 10, None) == _cabi.ERR_SHAPE
    grp.close()
    lib.kb_linear_group_destroy(None)  # harmless


def test_group_f32_input_strided_and_unaligned(torch):
    """Rows of x that are neither contiguous nor 16-byte aligned take the scalar path of the prologue."""
    from kore_b200 import nn

    count, m, k = 6, 96, 333
    layers, raw = _make(Q, "reference", count, m, k, True, 400)
    grp = nn.LinearGroup(layers)
    x = cases.gaussian(9, (count, k), 1.0)
    wide = torch.zeros((count, k + 3), dtype=torch.float32, device="cuda")
    wide[:, 1 : k + 1] = torch.from_numpy(x).cuda()
    y = grp(wide[:, 1 : k + 1]).cpu().numpy()
    for i, (packed, scales, bias) in enumerate(raw):
        y_ref, _ = kbref.q_forward(Q, packed, scales, bias, m, k, x[i : i + 1], threads=2)
        assert (y[i] == y_ref[0]).all(), f"layer {i}"
    # an all-zero row quantises with scale 1 (the reference's 1e-8 rule)
    x[2] = 0.0
    y = grp(torch.from_numpy(x).cuda()).cpu().numpy()
    y_ref, _ = kbref.q_forward(Q, raw[2][0], raw[2][1], raw[2][2], m, k, x[2:3], threads=2)
    assert (y[2] == y_ref[0]).all()
    grp.close()
