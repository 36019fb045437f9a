"""ctypes binding of ``libkore_b200.so`` — the same C ABI a Rust/cgo/JNI caller binds.

The library is built ahead of time into ``kore_b200/_lib`` (see ``_build.py``).  There
is no fallback: if the shared library is missing, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

from . import _build

OK, ERR_SHAPE, ERR_STORAGE, ERR_DTYPE, ERR_CUDA = 0, 1, 2, 3, 4
ERR_TIMEOUT, ERR_BAD_HANDLE, ERR_INVALID, ERR_UNSUPPORTED = 6, 7, 8, 9
TERNARY, QUATERNARY = 0, 1
QUANT_REFERENCE, QUANT_ABSMEAN = 0, 1
ACT_NONE, ACT_RELU = 0, 1
PATH_AUTO, PATH_GEMV, PATH_GEMM_TC, PATH_GEMV_SHARED, PATH_GEMV_MMA, PATH_GEMV_STREAM = 0, 1, 2, 3, 4, 5

_u8p, _i8p = C.POINTER(C.c_uint8), C.POINTER(C.c_int8)
_f32p, _i32p = C.POINTER(C.c_float), C.POINTER(C.c_int32)
_sz, _vp = C.c_size_t, C.c_void_p

# name -> (restype, argtypes); one entry per symbol declared in include/kore_b200.h
SIGNATURES = {
    "kb_version": (C.c_char_p, []),
    "kb_last_error": (C.c_char_p, []),
    "kb_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "kb_linear_create_from_ref_packed": (C.c_int, [C.c_int, _vp, _sz, _vp, _sz, _vp, _sz, _sz, C.c_int, C.POINTER(_vp)]),
    "kb_linear_create_from_f32": (C.c_int, [C.c_int, C.c_int, _vp, _vp, _sz, _sz, C.c_float, C.c_int, C.POINTER(_vp)]),
    "kb_linear_destroy": (None, [_vp]),
    "kb_linear_info": (C.c_int, [_vp, C.POINTER(_sz), C.POINTER(_sz), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(_sz)]),
    "kb_linear_scales": (C.c_int, [_vp, _vp, _sz]),
    "kb_linear_packed_weights": (C.c_int, [_vp, _vp, _sz]),
    "kb_linear_dequantize_weights": (C.c_int, [_vp, _vp, _sz]),
    "kb_quantize_act_i8": (C.c_int, [_vp, _sz, _sz, _vp, _sz, _vp, _vp, _vp]),
    "kb_act_ld": (_sz, [_sz]),
    "kb_linear_forward": (C.c_int, [_vp, _vp, _sz, _vp, _vp]),
    "kb_linear_forward_ex": (C.c_int, [_vp, _vp, _sz, _sz, _vp, _sz, _vp, C.c_int, _vp, _sz, _vp]),
    "kb_linear_forward_act": (C.c_int, [_vp, _vp, _sz, _sz, _vp, _sz, C.c_int, C.c_int, _vp, _sz, _vp]),
    "kb_linear_workspace_bytes": (_sz, [_vp, _sz]),
    "kb_linear_forward_q8": (C.c_int, [_vp, _vp, _sz, _vp, _vp, _sz, _vp, _sz, _vp, C.c_int, _vp]),
    "kb_linear_forward_fused": (C.c_int, [_vp, _vp, _vp, _sz, _vp, _vp, _sz, _vp, _vp, _sz, C.c_int, _vp, _sz, _vp]),
    "kb_rmsnorm_quant": (C.c_int, [_vp, _vp, _sz, _sz, C.c_float, _vp, _vp, _sz, _vp, _vp, _vp]),
    "kb_swiglu_quant": (C.c_int, [_vp, _sz, _sz, _sz, _vp, _vp, _sz, _vp, _vp, _vp]),
    "kb_swiglu_quant_pairs": (C.c_int, [_vp, _sz, _sz, _sz, _vp, _vp, _sz, _vp, _vp, _vp]),
    "kb_rope_kv": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _sz, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp, _vp]),
    "kb_attn_decode": (C.c_int, [_vp, _vp, _vp, _vp, _sz, C.c_int, C.c_int, C.c_int, _vp, _vp, _sz, _vp]),
    "kb_attn_decode_scratch_bytes": (_sz, [_sz, C.c_int]),
    "kb_lm_head_argmax": (C.c_int, [_vp, _sz, _sz, _vp, _sz, _vp, _vp, _vp]),
    "kb_decode_advance": (C.c_int, [_vp, _sz, _vp, _vp, _vp, _vp, _vp]),
    "kb_decoder_create": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, C.c_float, _vp, _vp, _vp, _vp, _vp,
                                    C.POINTER(_vp)]),
    "kb_decoder_destroy": (None, [_vp]),
    "kb_decoder_step": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "kb_decoder_status": (C.c_int, [_vp, _vp, C.POINTER(C.c_int)]),
    "kb_linear_forward_host": (C.c_int, [_vp, _vp, _sz, _sz, _vp]),
    "kb_linear_forward_static": (C.c_int, [_vp, _vp, _sz, _sz, _vp, _vp]),
    "kb_linear_group_create": (C.c_int, [_vp, _sz, _vp]),
    "kb_linear_group_destroy": (None, [_vp]),
    "kb_linear_group_count": (_sz, [_vp]),
    "kb_linear_group_forward_q8": (C.c_int, [_vp, _vp, _sz, _vp, _vp, _vp, _sz, _vp]),
    "kb_linear_group_forward": (C.c_int, [_vp, _vp, _sz, _vp, _sz, _vp]),
    "kb_linear_group_forward_host": (C.c_int, [_vp, _vp, _vp]),
    "kb_static_scratch_bytes": (_sz, []),
    "kb_ternary_matmul": (C.c_int, [_vp, _sz, _vp, _sz, _vp, _vp, _sz, _sz, _sz]),
    "kb_linear_forward_rmsnorm": (C.c_int, [_vp, _vp, _vp, C.c_float, _sz, _vp, _sz, C.c_int, _vp, _vp]),
    "kb_linear_forward_scaled": (C.c_int, [_vp, _vp, _vp, _sz, _vp, _vp, _sz, _vp, _vp]),
    "kb_quat_matmul": (C.c_int, [_vp, _sz, _vp, _sz, _vp, _vp, _sz, _sz, _sz]),
    "kb_quat_matmul_bias_relu": (C.c_int, [_vp, _sz, _vp, _sz, _vp, _vp, _sz, _vp, _sz, _sz, _sz]),
    "kb_ternary_ternary_matmul": (C.c_int, [_vp, _sz, _vp, _vp, _sz, _vp, _vp, _sz, _sz, _sz]),
    "kb_pack_weights_ternary": (C.c_int, [_vp, _sz, _sz, C.c_float, _vp, _sz, _vp, _sz, C.c_int]),
    "kb_pack_weights_quaternary": (C.c_int, [_vp, _sz, _sz, _vp, _sz, _vp, _sz, C.c_int]),
    "kb_linear_forward_sharded": (C.c_int, [_vp, _vp, _sz, _sz, _vp, C.c_int, C.c_int, _sz, _sz, C.c_int, _vp, _sz, _vp, _vp, _vp]),
    "kb_linear_forward_sharded_q8": (C.c_int, [_vp, _vp, _sz, _vp, _vp, _sz, _vp, C.c_int, C.c_int, _sz, _sz, C.c_int, _vp, _vp, _vp]),
    "kb_linear_forward_sharded_chain_q8": (C.c_int, [_vp, _vp, _sz, _vp, _vp, _sz, _vp, C.c_int, C.c_int, _sz, _sz, _vp, _vp, _vp]),
    "kb_peer_wait": (C.c_int, [_vp, C.c_int, C.c_int, _vp, _vp, _vp]),
    "kb_linear_forward_sharded_flagged": (C.c_int, [_vp, _vp, C.c_int, _sz, _sz, _sz, _vp, C.c_int, C.c_int, _sz, _sz, C.c_int,
                                                   C.c_int, _vp, _sz, _vp, _vp]),
    "kb_linear_forward_sharded_flagged_q8": (C.c_int, [_vp, _vp, _sz, _vp, _vp, _sz, _vp, C.c_int, C.c_int, _sz, _sz, C.c_int, _vp,
                                                      _vp]),
    "kb_flagged_unpack": (C.c_int, [_vp, _sz, _sz, _sz, _vp, _sz, C.c_int, _vp, _vp]),
    "kb_peer_barrier": (C.c_int, [_vp, C.c_int, C.c_int, _vp, _vp, _vp]),
    "kb_symm_alloc": (C.c_int, [_sz, C.POINTER(_vp)]),
    "kb_symm_free": (C.c_int, [_vp]),
    "kb_ipc_export": (C.c_int, [_vp, _vp]),
    "kb_ipc_open": (C.c_int, [_vp, C.POINTER(_vp)]),
    "kb_ipc_close": (C.c_int, [_vp]),
    "kb_linear_device_ptrs": (C.c_int, [_vp, C.POINTER(_vp), C.POINTER(_sz), C.POINTER(_vp), C.POINTER(_vp)]),
    "kb_linear_last_device_status": (C.c_int, [_vp, _vp, C.POINTER(C.c_int)]),
}

_lib = None


class KoreError(RuntimeError):
    """Mirror of KoreError / CudaError: ``code`` is the KB_* status, the message the
    library's thread-local error string."""

    NAMES = {ERR_SHAPE: "ShapeMismatch", ERR_STORAGE: "StorageError", ERR_DTYPE: "UnsupportedDType",
             ERR_CUDA: "CudaError", ERR_TIMEOUT: "Timeout", ERR_BAD_HANDLE: "BadHandle",
             ERR_INVALID: "InvalidArgument", ERR_UNSUPPORTED: "Unsupported"}

    def __init__(self, code: int, message: str):
        super().__init__(f"{self.NAMES.get(code, code)}: {message}")
        self.code = code
        self.message = message


def lib_path() -> str:
    return _build.LIB_PATH


def lib() -> C.CDLL:
    """Load the shared library (raises if it has not been built)."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: the CUDA extension has not been built "
                "(run `python -m kore_b200._build`); there is no CPU fallback")
        L = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc: int) -> None:
    if rc != OK:
        raise KoreError(rc, lib().kb_last_error().decode("utf-8", "replace"))
