"""Function-level mirror of the kore-kernels quantized-matmul entry points over the C ABI.

Signatures follow ``crates/kore-kernels/src/cpu_ternary_matmul.rs:29-36,198-203`` and
``cpu_quat_matmul.rs:22-29,174``: ``a_packed`` is the reference wire format, ``b`` is
``[K,N]`` f32, the result is ``[M,N]`` f32.  Everything is computed by the CUDA library.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _cabi
from ._cabi import KoreError  # noqa: F401


def _one_shot(fn, a_packed, a_scales, b, m, n, k):
    a = np.ascontiguousarray(a_packed, dtype=np.uint8).ravel()
    s = np.ascontiguousarray(a_scales, dtype=np.float32).ravel()
    b = np.asarray(b)
    if b.dtype != np.float32:
        # ternary_matmul returns UnsupportedDType for non-f32 activations (:38-40)
        raise KoreError(_cabi.ERR_DTYPE, f"unsupported dtype {b.dtype}")
    b = np.ascontiguousarray(b).reshape(k, n)
    c = np.zeros((m, n), np.float32)
    _cabi.check(fn(a.ctypes.data, a.size, s.ctypes.data, s.size, b.ctypes.data, c.ctypes.data, m, n, k))
    return c


def ternary_matmul(a_packed, a_scales, b, m: int, n: int, k: int) -> np.ndarray:
    """C[M,N] = ternary(A)[M,K] @ B[K,N] * scales[M]  (base-243 packed A)."""
    return _one_shot(_cabi.lib().kb_ternary_matmul, a_packed, a_scales, b, m, n, k)


def quat_matmul(a_packed, a_scales, b, m: int, n: int, k: int) -> np.ndarray:
    """C[M,N] = quat(A)[M,K] @ B[K,N] * scales[M]  (2-bit LSB-first packed A)."""
    return _one_shot(_cabi.lib().kb_quat_matmul, a_packed, a_scales, b, m, n, k)


def quat_matmul_bias_relu(a_packed, a_scales, b, bias, m: int, n: int, k: int) -> np.ndarray:
    """C[M,N] = max(0, quat(A)[M,K] @ B[K,N] * scales[M] + bias[M])  (cuda/ops.rs:828-878); bias is
    per output feature (weight row)."""
    a = np.ascontiguousarray(a_packed, dtype=np.uint8).ravel()
    s = np.ascontiguousarray(a_scales, dtype=np.float32).ravel()
    bi = np.ascontiguousarray(bias, dtype=np.float32).ravel()
    b = np.asarray(b)
    if b.dtype != np.float32:
        raise KoreError(_cabi.ERR_DTYPE, f"unsupported dtype {b.dtype}")
    b = np.ascontiguousarray(b).reshape(k, n)
    c = np.zeros((m, n), np.float32)
    _cabi.check(_cabi.lib().kb_quat_matmul_bias_relu(a.ctypes.data, a.size, s.ctypes.data, s.size, b.ctypes.data,
                                                     bi.ctypes.data, bi.size, c.ctypes.data, m, n, k))
    return c


def ternary_ternary_matmul(a_packed, a_scales, b_packed, b_scales, m: int, n: int, k: int) -> np.ndarray:
    """C[M,N] = (ternary(A)[M,K] . ternary(B)[N,K]) * a_scales[M] * b_scales[N], integer dot products
    (both operands base-243 rows; cpu_ternary_matmul.rs:131-193)."""
    a = np.ascontiguousarray(a_packed, dtype=np.uint8).ravel()
    b = np.ascontiguousarray(b_packed, dtype=np.uint8).ravel()
    sa = np.ascontiguousarray(a_scales, dtype=np.float32).ravel()
    sb = np.ascontiguousarray(b_scales, dtype=np.float32).ravel()
    if sa.size < m or sb.size < n:
        raise KoreError(_cabi.ERR_STORAGE, "scales too small")
    c = np.zeros((m, n), np.float32)
    _cabi.check(_cabi.lib().kb_ternary_ternary_matmul(a.ctypes.data, a.size, sa.ctypes.data, b.ctypes.data, b.size,
                                                      sb.ctypes.data, c.ctypes.data, m, n, k))
    return c


def pack_weights_ternary(weights, m: int, k: int, threshold: float, device: int = 0):
    """(packed base-243 bytes [M*ceil(K/5)], scales [M]) computed on the device."""
    w = np.ascontiguousarray(weights, dtype=np.float32).reshape(m, k)
    packed = np.zeros(m * ((k + 4) // 5), np.uint8)
    scales = np.zeros(m, np.float32)
    _cabi.check(_cabi.lib().kb_pack_weights_ternary(w.ctypes.data, m, k, C.c_float(threshold), packed.ctypes.data,
                                                    packed.size, scales.ctypes.data, scales.size, device))
    return packed, scales


def pack_weights_quaternary(weights, m: int, k: int, device: int = 0):
    """(packed 2-bit bytes [M*ceil(K/4)], scales [M]) computed on the device."""
    w = np.ascontiguousarray(weights, dtype=np.float32).reshape(m, k)
    packed = np.zeros(m * ((k + 3) // 4), np.uint8)
    scales = np.zeros(m, np.float32)
    _cabi.check(_cabi.lib().kb_pack_weights_quaternary(w.ctypes.data, m, k, packed.ctypes.data, packed.size,
                                                       scales.ctypes.data, scales.size, device))
    return packed, scales


def act_ld(k: int) -> int:
    return int(_cabi.lib().kb_act_ld(k))


def quantize_act_i8(x):
    """Per-token absmax int8 quantiser on a CUDA float32 tensor [N,K].
    Returns (xq int8 [N, act_ld(K)], sx f32 [N], sumq int32 [N]) as CUDA tensors."""
    import torch

    if not x.is_cuda or x.dtype != torch.float32 or x.dim() != 2:
        raise KoreError(_cabi.ERR_DTYPE, "expected a 2-D CUDA float32 tensor")
    x = x.contiguous()
    n, k = x.shape
    ld = act_ld(k)
    xq = torch.empty((n, ld), dtype=torch.int8, device=x.device)
    sx = torch.empty((n,), dtype=torch.float32, device=x.device)
    sumq = torch.empty((n,), dtype=torch.int32, device=x.device)
    _cabi.check(_cabi.lib().kb_quantize_act_i8(x.data_ptr(), n, k, xq.data_ptr(), ld, sx.data_ptr(), sumq.data_ptr(),
                                               torch.cuda.current_stream(x.device.index).cuda_stream))
    return xq, sx, sumq


def forward_q8(layer, xq, sx, sumq, path: int = _cabi.PATH_AUTO, return_acc: bool = False):
    """Forward of a BitLinear/QuatLinear from pre-quantised activations (CUDA tensors)."""
    import torch

    n = xq.shape[0]
    y = torch.empty((n, layer.out_features), dtype=torch.float32, device=xq.device)
    acc = torch.empty((n, layer.out_features), dtype=torch.int32, device=xq.device) if return_acc else None
    _cabi.check(_cabi.lib().kb_linear_forward_q8(
        layer.handle, xq.data_ptr(), xq.stride(0), sx.data_ptr(), sumq.data_ptr(), n, y.data_ptr(), 0,
        None if acc is None else acc.data_ptr(), path, torch.cuda.current_stream(xq.device.index).cuda_stream))
    return (y, acc) if return_acc else y
