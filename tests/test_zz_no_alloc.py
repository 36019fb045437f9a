"""kb_linear_forward_static — the forward for callers that cannot allocate device memory
(fixed-footprint real-time loops, plugins living under someone else's allocator, engines
whose pools are frozen).  Its quantised activations live in a fixed 1 MiB array inside the
library instead of freshly allocated scratch, so this file checks, through the C ABI, that
it returns exactly what the regular entry point returns — and what the CPU oracle computes
from the same packed weights — twice in a row on the shared array, and that it refuses
work that does not fit.

Collected last on purpose (file name): a run that stops at the first failure has then
already exercised every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _gauss(seed, shape, sigma):
    return (np.random.default_rng(seed).standard_normal(shape) * sigma).astype(np.float32)


def test_static_scratch_forward_matches_regular_forward_twice():
    import torch

    from kore_b200 import _cabi, nn
    from oracle import kbref

    assert torch.cuda.is_available()
    lib = _cabi.lib()
    limit = lib.kb_static_scratch_bytes()
    assert limit == 1 << 20
    stream = torch.cuda.current_stream().cuda_stream

    lay_a_bias = _gauss(2, (384,), 0.1)
    lay_a = nn.BitLinear.new(_gauss(1, (384, 1000), 0.02), lay_a_bias, 0.3, quantiser="absmean")
    lay_b = nn.QuatLinear.new(_gauss(3, (200, 4096), 0.02))
    # two calls in a row on the shared array: the second is smaller in both dimensions, so
    # it runs over bytes the first call left behind; then a decode-sized call (GEMV branch)
    for lay, n, seed in ((lay_a, 300, 10), (lay_b, 37, 11), (lay_a, 3, 12), (lay_b, 1, 13)):
        k, m = lay.in_features, lay.out_features
        x = torch.from_numpy(_gauss(seed, (n, k), 1.0)).cuda()
        y_static = torch.full((n, m), float("nan"), device="cuda")
        y_regular = torch.full((n, m), float("nan"), device="cuda")
        _cabi.check(lib.kb_linear_forward_static(lay.handle, x.data_ptr(), n, k, y_static.data_ptr(), stream))
        path = _cabi.PATH_GEMV if n <= 8 else _cabi.PATH_GEMM_TC
        _cabi.check(lib.kb_linear_forward_ex(lay.handle, x.data_ptr(), n, k, y_regular.data_ptr(), 0, None, path,
                                             None, 0, stream))
        torch.cuda.synchronize()
        # same kernels, same arithmetic: the comparison is exact, like every other parity test here
        assert torch.equal(y_static, y_regular)
        assert torch.isfinite(y_static).all()
        # and the checker that shares no code with either entry point
        kind = kbref.TERNARY if lay is lay_a else kbref.QUATERNARY
        bias = lay_a_bias if lay is lay_a else None
        y_ref = kbref.q_forward(kind, lay.packed_weights(), lay.scales(), bias, m, k, x.cpu().numpy(), threads=4)[0]
        assert (y_static.cpu().numpy() == y_ref).all()


def test_static_scratch_rejects_oversized_and_bad_arguments():
    import torch

    from kore_b200 import _cabi, nn

    lib = _cabi.lib()
    lay = nn.BitLinear.new(_gauss(5, (128, 4096), 0.02), None, 0.3)
    stream = torch.cuda.current_stream().cuda_stream
    n = 300  # 300 x 4096 codes alone exceed 1 MiB
    x = torch.zeros((n, 4096), device="cuda")
    y = torch.zeros((n, 128), device="cuda")
    rc = lib.kb_linear_forward_static(lay.handle, x.data_ptr(), n, 4096, y.data_ptr(), stream)
    assert rc == _cabi.ERR_UNSUPPORTED
    msg = lib.kb_last_error().decode()
    assert "static scratch too small" in msg and str(1 << 20) in msg
    assert lib.kb_linear_forward_static(lay.handle, x.data_ptr(), 4, 4095, y.data_ptr(), stream) == _cabi.ERR_SHAPE
    assert lib.kb_linear_forward_static(None, x.data_ptr(), 4, 4096, y.data_ptr(), stream) == _cabi.ERR_BAD_HANDLE
    # largest request that fits: 255 tokens x 4096 codes + two 1 KiB vectors
    assert 255 * 4096 + 2 * 1024 <= (1 << 20)
    _cabi.check(lib.kb_linear_forward_static(lay.handle, x.data_ptr(), 255, 4096, y.data_ptr(), stream))
    torch.cuda.synchronize()
    assert not y[:255].any()  # zero activations -> zero outputs (no bias)


def test_static_scratch_forward_takes_no_device_memory_where_the_regular_path_would():
    """A layer of few row tiles with long rows: the regular entry splits K over CTAs and creates a scratch buffer on
    first use; the static entry must not, and still returns the same values (integer partial sums are exact)."""
    import torch

    from kore_b200 import _cabi, nn

    lib = _cabi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    lay = nn.QuatLinear.new(_gauss(21, (200, 8192), 0.02))
    n, k, m = 40, 8192, 200
    x = torch.from_numpy(_gauss(22, (n, k), 1.0)).cuda()
    y_static = torch.full((n, m), float("nan"), device="cuda")
    y_regular = torch.full((n, m), float("nan"), device="cuda")
    _cabi.check(lib.kb_linear_forward_static(lay.handle, x.data_ptr(), n, k, y_static.data_ptr(), stream))  # warm-up: loads the kernels
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    _cabi.check(lib.kb_linear_forward_static(lay.handle, x.data_ptr(), n, k, y_static.data_ptr(), stream))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    _cabi.check(lib.kb_linear_forward_ex(lay.handle, x.data_ptr(), n, k, y_regular.data_ptr(), 0, None, _cabi.PATH_GEMM_TC, None, 0, stream))
    torch.cuda.synchronize()
    assert torch.equal(y_static, y_regular)
