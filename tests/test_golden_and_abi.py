"""CPU-side checks: the oracle reproduces the committed golden vectors, and the C-ABI
library loads and exports every symbol its header declares (no compute without a GPU)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from oracle import kbref
from tests import cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def recorded():
    return np.load(os.path.join(ROOT, "tests", "golden", "recorded.npz"))


def test_oracle_reproduces_recorded_generator_cases(kats, recorded):
    for c in kats["generator_cases"]:
        kind = cases.kind_id(c["kind"])
        m, n, k = c["m"], c["n"], c["k"]
        w = cases.rule(c["w_rule"], m * k).reshape(m, k)
        b = cases.rule(c["b_rule"], k * n).reshape(k, n)
        packed, scales = cases.make_weights(kind, "reference", w, c.get("threshold", 0.3))
        fn = kbref.ternary_matmul if kind == kbref.TERNARY else kbref.quat_matmul
        assert (fn(packed, scales, b, m, n, k) == recorded[f"gen_{c['name']}_r"]).all()
        y, acc = kbref.q_forward(kind, packed, scales, None, m, k, np.ascontiguousarray(b.T))
        assert (acc == recorded[f"gen_{c['name']}_q_acc"]).all() and (y == recorded[f"gen_{c['name']}_q_y"]).all()


def test_oracle_reproduces_recorded_config1(recorded):
    w = cases.gaussian(1001, (128, 256), 0.02)
    x = cases.gaussian(1002, (32, 256), 1.0)
    for name, kind, quantiser in (("tern_ref", kbref.TERNARY, "reference"), ("tern_absmean", kbref.TERNARY, "absmean"),
                                  ("quat", kbref.QUATERNARY, "reference")):
        packed, scales = cases.make_weights(kind, quantiser, w)
        assert (kbref.linear_forward(kind, packed, scales, None, 128, 256, x) == recorded[f"cfg1_{name}_r"]).all()
        y, acc = kbref.q_forward(kind, packed, scales, None, 128, 256, x, threads=2)
        assert (acc == recorded[f"cfg1_{name}_q_acc"]).all() and (y == recorded[f"cfg1_{name}_q_y"]).all()
        # W2A8 output stays close to what the reference computes from f32 activations
        r = recorded[f"cfg1_{name}_r"]
        assert np.abs(y - r).max() < 0.02 * np.abs(r).max()


def _header_functions():
    text = open(os.path.join(ROOT, "include", "kore_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from kore_b200 import _cabi

    lib = _cabi.lib()
    names = _header_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/kore_b200.h but not exported"
        assert n in _cabi.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_cabi.SIGNATURES) == names


def test_host_side_argument_checks_need_no_gpu():
    from kore_b200 import _cabi

    lib = _cabi.lib()
    assert lib.kb_version().startswith(b"kore_b200")
    assert lib.kb_act_ld(4096) == 4096 and lib.kb_act_ld(5) == 128 and lib.kb_act_ld(8640) == 8704
    # a null handle is reported, never dereferenced; destroy is null-tolerant
    assert lib.kb_linear_forward(None, None, 1, None, None) == _cabi.ERR_BAD_HANDLE
    assert lib.kb_linear_info(None, None, None, None, None, None) == _cabi.ERR_BAD_HANDLE
    lib.kb_linear_destroy(None)
    # buffer-length checks happen before any CUDA call and use the reference's wording
    packed = np.zeros(51, np.uint8)
    scales = np.ones(1, np.float32)
    h = C.c_void_p()
    rc = lib.kb_linear_create_from_ref_packed(_cabi.TERNARY, packed.ctypes.data, packed.size, scales.ctypes.data, 1,
                                              None, 1, 256, 0, C.byref(h))
    assert rc == _cabi.ERR_STORAGE and b"a_packed too small: need 52 bytes, got 51" in lib.kb_last_error()
    packed = np.zeros(52, np.uint8)
    rc = lib.kb_linear_create_from_ref_packed(_cabi.TERNARY, packed.ctypes.data, packed.size, scales.ctypes.data, 0,
                                              None, 1, 256, 0, C.byref(h))
    assert rc == _cabi.ERR_STORAGE and b"a_scales too small: need 1, got 0" in lib.kb_last_error()
    rc = lib.kb_linear_create_from_f32(_cabi.QUATERNARY, _cabi.QUANT_ABSMEAN, packed.ctypes.data, None, 1, 13,
                                       C.c_float(0.3), 0, C.byref(h))
    assert rc == _cabi.ERR_INVALID
    with pytest.raises(_cabi.KoreError) as e:
        _cabi.check(rc)
    assert e.value.code == _cabi.ERR_INVALID


def test_product_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "kore_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".hpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text and "kbref" not in text, f"{f} refers to the oracle"
