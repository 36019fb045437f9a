"""ctypes front-end of the CPU oracle ``libkbref.so`` (see ``kbref.h``).

TEST INFRASTRUCTURE ONLY.  Imported by the test-suite, by the smoke check and by
the CPU-baseline leg of the benchmark; the shipped package never imports it.

Parity status: pinned against the known answers in the reference's unit tests
(transcribed in ``tests/golden/reference_kats.json``); the reference itself is
Rust and cannot be built without cargo/rustc, so no reference binary was run.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libkbref.so")

TERNARY, QUATERNARY = 0, 1
OK, ERR_SHAPE, ERR_STORAGE = 0, 1, 2


def build(force: bool = False) -> str:
    """Compile the oracle with gcc through its Makefile; returns the library path."""
    src_m = max(os.path.getmtime(os.path.join(_HERE, f)) for f in ("kbref.c", "kbref.h", "Makefile"))
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < src_m:
        subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _declare(_lib)
    return _lib


_u8p = C.POINTER(C.c_uint8)
_i8p = C.POINTER(C.c_int8)
_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int32)
_sz = C.c_size_t


def _declare(L):
    L.kbref_encode_trits5.restype = C.c_uint8
    L.kbref_encode_trits5.argtypes = [_i8p]
    L.kbref_decode_trits5.argtypes = [C.c_uint8, _i8p]
    L.kbref_pack_quats4.restype = C.c_uint8
    L.kbref_pack_quats4.argtypes = [_u8p]
    L.kbref_unpack_quats4.argtypes = [C.c_uint8, _u8p]
    L.kbref_quat_value.restype = C.c_float
    L.kbref_quat_value.argtypes = [C.c_uint8]
    L.kbref_pack_ternary.restype = _sz
    L.kbref_pack_ternary.argtypes = [_i8p, _sz, _u8p]
    L.kbref_pack_quaternary.restype = _sz
    L.kbref_pack_quaternary.argtypes = [_u8p, _sz, _u8p]
    L.kbref_quantize_ternary.restype = C.c_float
    L.kbref_quantize_ternary.argtypes = [_f32p, _sz, C.c_float, _i8p]
    L.kbref_quantize_quaternary.restype = C.c_float
    L.kbref_quantize_quaternary.argtypes = [_f32p, _sz, _u8p]
    L.kbref_pack_weights_ternary.argtypes = [_f32p, _sz, _sz, C.c_float, _u8p, _f32p]
    L.kbref_pack_weights_quaternary.argtypes = [_f32p, _sz, _sz, _u8p, _f32p]
    L.kbref_pack_weights_ternary_absmean.argtypes = [_f32p, _sz, _sz, _u8p, _f32p]
    L.kbref_ternary_matmul.argtypes = [_u8p, _sz, _f32p, _sz, _f32p, _f32p, _sz, _sz, _sz, C.c_int]
    L.kbref_quat_matmul.argtypes = [_u8p, _sz, _f32p, _sz, _f32p, _f32p, _sz, _sz, _sz, C.c_int]
    L.kbref_ternary_ternary_matmul.argtypes = [_u8p, _sz, _f32p, _u8p, _sz, _f32p, _f32p, _sz, _sz, _sz]
    L.kbref_edge_matmul_ternary.argtypes = [_u8p, _f32p, _f32p, _f32p, _sz, _sz, _sz]
    L.kbref_edge_matmul_quaternary.argtypes = [_u8p, _f32p, _f32p, _f32p, _sz, _sz, _sz]
    L.kbref_bitlinear_forward.argtypes = [_u8p, _f32p, _f32p, _sz, _sz, _f32p, _sz, _sz, _f32p, C.c_int]
    L.kbref_quatlinear_forward.argtypes = [_u8p, _f32p, _f32p, _sz, _sz, _f32p, _sz, _sz, _f32p]
    L.kbref_dequantize_ternary.argtypes = [_u8p, _f32p, _sz, _sz, _f32p]
    L.kbref_dequantize_quaternary.argtypes = [_u8p, _f32p, _sz, _sz, _f32p]
    L.kbref_quantize_act_i8.argtypes = [_f32p, _sz, _sz, _i8p, _sz, _f32p, _i32p]
    L.kbref_decode_weights_i8.argtypes = [C.c_int, _u8p, _sz, _sz, _i8p]
    L.kbref_acc_i32.argtypes = [_i8p, _sz, _sz, _i8p, _sz, _sz, _i32p, C.c_int]
    L.kbref_dequant_epilogue.argtypes = [_i32p, _f32p, _f32p, _f32p, _sz, _sz, _f32p]
    L.kbref_q_forward.argtypes = [C.c_int, _u8p, _f32p, _f32p, _sz, _sz, _f32p, _sz, _f32p, _i32p, C.c_int]


def _p(a, typ):
    return a.ctypes.data_as(typ) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


def max_threads() -> int:
    return int(lib().kbref_max_threads())


def host_cores() -> int:
    """Cores this process may run on.  Every entry point here takes its thread count as an
    argument (``num_threads`` clauses in kbref.c), so passing this value uses all of them even
    where a launcher has set OMP_NUM_THREADS=1 for its workers (torch.distributed.run does)."""
    import os

    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def k_packed(kind: int, k: int) -> int:
    return (k + 4) // 5 if kind == TERNARY else (k + 3) // 4


# ---- codecs -----------------------------------------------------------------
def encode_trits5(trits) -> int:
    t = np.ascontiguousarray(trits, dtype=np.int8)
    assert t.size == 5
    return int(lib().kbref_encode_trits5(_p(t, _i8p)))


def decode_trits5(byte: int):
    out = np.zeros(5, np.int8)
    lib().kbref_decode_trits5(C.c_uint8(byte), _p(out, _i8p))
    return out


def pack_quats4(codes) -> int:
    c = _u8(codes)
    return int(lib().kbref_pack_quats4(_p(c, _u8p)))


def unpack_quats4(byte: int):
    out = np.zeros(4, np.uint8)
    lib().kbref_unpack_quats4(C.c_uint8(byte), _p(out, _u8p))
    return out


def quat_value(code: int) -> float:
    return float(lib().kbref_quat_value(C.c_uint8(code)))


def pack_ternary(trits):
    t = np.ascontiguousarray(trits, dtype=np.int8)
    out = np.zeros((t.size + 4) // 5, np.uint8)
    lib().kbref_pack_ternary(_p(t, _i8p), t.size, _p(out, _u8p))
    return out


def pack_quaternary(codes):
    c = _u8(codes)
    out = np.zeros((c.size + 3) // 4, np.uint8)
    lib().kbref_pack_quaternary(_p(c, _u8p), c.size, _p(out, _u8p))
    return out


# ---- quantisers -------------------------------------------------------------
def quantize_ternary(w, threshold: float):
    w = _f32(w).ravel()
    tr = np.zeros(w.size, np.int8)
    s = lib().kbref_quantize_ternary(_p(w, _f32p), w.size, C.c_float(threshold), _p(tr, _i8p))
    return tr, float(s)


def quantize_quaternary(w):
    w = _f32(w).ravel()
    codes = np.zeros(w.size, np.uint8)
    s = lib().kbref_quantize_quaternary(_p(w, _f32p), w.size, _p(codes, _u8p))
    return codes, float(s)


def pack_weights_ternary(w, m: int, k: int, threshold: float):
    w = _f32(w).reshape(m, k)
    packed = np.zeros(m * k_packed(TERNARY, k), np.uint8)
    scales = np.zeros(m, np.float32)
    lib().kbref_pack_weights_ternary(_p(w, _f32p), m, k, C.c_float(threshold), _p(packed, _u8p), _p(scales, _f32p))
    return packed, scales


def pack_weights_quaternary(w, m: int, k: int):
    w = _f32(w).reshape(m, k)
    packed = np.zeros(m * k_packed(QUATERNARY, k), np.uint8)
    scales = np.zeros(m, np.float32)
    lib().kbref_pack_weights_quaternary(_p(w, _f32p), m, k, _p(packed, _u8p), _p(scales, _f32p))
    return packed, scales


def pack_weights_ternary_absmean(w, m: int, k: int):
    w = _f32(w).reshape(m, k)
    packed = np.zeros(m * k_packed(TERNARY, k), np.uint8)
    scales = np.zeros(m, np.float32)
    lib().kbref_pack_weights_ternary_absmean(_p(w, _f32p), m, k, _p(packed, _u8p), _p(scales, _f32p))
    return packed, scales


# ---- R level ----------------------------------------------------------------
class OracleError(RuntimeError):
    def __init__(self, code):
        super().__init__({ERR_SHAPE: "ShapeMismatch", ERR_STORAGE: "StorageError"}.get(code, str(code)))
        self.code = code


def ternary_matmul(a_packed, a_scales, b, m, n, k, threads: int = 1):
    a_packed, a_scales, b = _u8(a_packed), _f32(a_scales), _f32(b)
    c = np.zeros((m, n), np.float32)
    rc = lib().kbref_ternary_matmul(_p(a_packed, _u8p), a_packed.size, _p(a_scales, _f32p), a_scales.size,
                                    _p(b, _f32p), _p(c, _f32p), m, n, k, threads)
    if rc:
        raise OracleError(rc)
    return c


def quat_matmul(a_packed, a_scales, b, m, n, k, use_fma: bool = False):
    a_packed, a_scales, b = _u8(a_packed), _f32(a_scales), _f32(b)
    c = np.zeros((m, n), np.float32)
    rc = lib().kbref_quat_matmul(_p(a_packed, _u8p), a_packed.size, _p(a_scales, _f32p), a_scales.size,
                                 _p(b, _f32p), _p(c, _f32p), m, n, k, int(use_fma))
    if rc:
        raise OracleError(rc)
    return c


def ternary_ternary_matmul(a_packed, a_scales, b_packed, b_scales, m, n, k):
    a_packed, b_packed = _u8(a_packed), _u8(b_packed)
    a_scales, b_scales = _f32(a_scales), _f32(b_scales)
    c = np.zeros((m, n), np.float32)
    rc = lib().kbref_ternary_ternary_matmul(_p(a_packed, _u8p), a_packed.size, _p(a_scales, _f32p),
                                            _p(b_packed, _u8p), b_packed.size, _p(b_scales, _f32p),
                                            _p(c, _f32p), m, n, k)
    if rc:
        raise OracleError(rc)
    return c


def edge_matmul_ternary(a_packed, a_scales, b, m, n, k):
    a_packed, a_scales, b = _u8(a_packed), _f32(a_scales), _f32(b)
    c = np.zeros((m, n), np.float32)
    lib().kbref_edge_matmul_ternary(_p(a_packed, _u8p), _p(a_scales, _f32p), _p(b, _f32p), _p(c, _f32p), m, n, k)
    return c


def edge_matmul_quaternary(a_packed, a_scales, b, m, n, k):
    a_packed, a_scales, b = _u8(a_packed), _f32(a_scales), _f32(b)
    c = np.zeros((m, n), np.float32)
    lib().kbref_edge_matmul_quaternary(_p(a_packed, _u8p), _p(a_scales, _f32p), _p(b, _f32p), _p(c, _f32p), m, n, k)
    return c


def linear_forward(kind, packed, scales, bias, m, k, x, threads: int = 1):
    """Module-level forward (BitLinear kind=0 / QuatLinear kind=1); x is [..., in]."""
    x = _f32(x)
    if x.ndim == 0:
        raise OracleError(ERR_SHAPE)
    in_dim = x.shape[-1]
    lead = x.shape[:-1]
    nt = int(np.prod(lead)) if x.ndim > 1 else 1
    x2 = x.reshape(nt, in_dim)
    packed, scales = _u8(packed), _f32(scales)
    bias = _f32(bias) if bias is not None else None
    y = np.zeros((nt, m), np.float32)
    if kind == TERNARY:
        rc = lib().kbref_bitlinear_forward(_p(packed, _u8p), _p(scales, _f32p), _p(bias, _f32p), m, k,
                                           _p(x2, _f32p), nt, in_dim, _p(y, _f32p), threads)
    else:
        rc = lib().kbref_quatlinear_forward(_p(packed, _u8p), _p(scales, _f32p), _p(bias, _f32p), m, k,
                                            _p(x2, _f32p), nt, in_dim, _p(y, _f32p))
    if rc:
        raise OracleError(rc)
    return y.reshape(*lead, m) if x.ndim > 1 else y.reshape(m)


def dequantize_weights(kind, packed, scales, m, k):
    packed, scales = _u8(packed), _f32(scales)
    w = np.zeros((m, k), np.float32)
    fn = lib().kbref_dequantize_ternary if kind == TERNARY else lib().kbref_dequantize_quaternary
    fn(_p(packed, _u8p), _p(scales, _f32p), m, k, _p(w, _f32p))
    return w


# ---- Q level ----------------------------------------------------------------
def quantize_act_i8(x, ldq: int | None = None):
    x = _f32(x)
    nt, k = x.shape
    ldq = k if ldq is None else ldq
    xq = np.zeros((nt, ldq), np.int8)
    sx = np.zeros(nt, np.float32)
    sumq = np.zeros(nt, np.int32)
    lib().kbref_quantize_act_i8(_p(x, _f32p), nt, k, _p(xq, _i8p), ldq, _p(sx, _f32p), _p(sumq, _i32p))
    return xq, sx, sumq


def decode_weights_i8(kind, packed, m, k):
    packed = _u8(packed)
    w = np.zeros((m, k), np.int8)
    lib().kbref_decode_weights_i8(kind, _p(packed, _u8p), m, k, _p(w, _i8p))
    return w


def acc_i32(w_i8, xq, threads: int = 1):
    w_i8 = np.ascontiguousarray(w_i8, dtype=np.int8)
    xq = np.ascontiguousarray(xq, dtype=np.int8)
    m, k = w_i8.shape
    nt, ldq = xq.shape
    assert ldq >= k
    acc = np.zeros((nt, m), np.int32)
    lib().kbref_acc_i32(_p(w_i8, _i8p), m, k, _p(xq, _i8p), ldq, nt, _p(acc, _i32p), threads)
    return acc


def dequant_epilogue(acc, sw, sx, bias=None):
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    nt, m = acc.shape
    sw, sx = _f32(sw), _f32(sx)
    bias = _f32(bias) if bias is not None else None
    y = np.zeros((nt, m), np.float32)
    lib().kbref_dequant_epilogue(_p(acc, _i32p), _p(sw, _f32p), _p(sx, _f32p), _p(bias, _f32p), nt, m, _p(y, _f32p))
    return y


def q_forward(kind, packed, scales, bias, m, k, x, threads: int = 1):
    """W2A8 forward from wire-format weights: returns (y[N,M] f32, acc[N,M] int32)."""
    x = _f32(x).reshape(-1, k)
    nt = x.shape[0]
    packed, scales = _u8(packed), _f32(scales)
    bias = _f32(bias) if bias is not None else None
    y = np.zeros((nt, m), np.float32)
    acc = np.zeros((nt, m), np.int32)
    lib().kbref_q_forward(kind, _p(packed, _u8p), _p(scales, _f32p), _p(bias, _f32p), m, k, _p(x, _f32p), nt,
                          _p(y, _f32p), _p(acc, _i32p), threads)
    return y, acc
