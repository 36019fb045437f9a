"""QLoraLinear (crates/kore-nn/src/lora.rs:190-372): deterministic adapter init, forward as
base + adapters, the reference's own test cases (:456-482)."""
import numpy as np
import pytest

from oracle import kbref, np_ref
from tests import cases


def test_lora_a_init_matches_formula():
    from kore_b200 import nn

    for rank, k in ((4, 16), (8, 64), (3, 7)):
        a = nn.lora_a_init(rank, k)
        assert a.shape == (rank, k)
        assert (a == np_ref.lora_a_init(rank, k)).all()
        assert np.abs(a).max() <= np.sqrt(np.float32(1.0) / np.float32(k))
    # first element: ((0 * c + 1013904223) & 0xFFFFFF) / 0xFFFFFF
    x0 = np.float32(1013904223 & 0xFFFFFF) / np.float32(0xFFFFFF)
    assert nn.lora_a_init(1, 16)[0, 0] == (x0 * np.float32(2) - np.float32(1)) * np.sqrt(np.float32(1 / 16))


@pytest.mark.gpu
def test_qlora_reference_cases_and_parity():
    import torch
    from kore_b200 import QLoraLinear

    # :456-461  creation
    w = cases.gaussian(81, (32, 64), 0.2)
    q = QLoraLinear.from_linear(w, None, 8, 8.0, 0.3)
    assert q.rank == 8 and q.base_compression_ratio() > 5.0
    assert "QLoraLinear" in repr(q) and "rank=8" in repr(q) and "alpha=8," in repr(q)
    assert q.trainable_params() == 8 * 64 + 32 * 8
    # :463-473  forward shape on ones, finite; lora_b starts at zero, so the output is the base's
    w = cases.gaussian(82, (8, 16), 0.2)
    q = QLoraLinear.from_linear(w, None, 4, 4.0, 0.3)
    y = q(torch.ones((3, 16), device="cuda"))
    assert tuple(y.shape) == (3, 8) and bool(torch.isfinite(y).all())
    packed, scales = kbref.pack_weights_ternary(w, 8, 16, 0.3)
    base_ref = kbref.q_forward(kbref.TERNARY, packed, scales, None, 8, 16, np.ones((3, 16), np.float32), threads=1)[0]
    assert (y.cpu().numpy() == base_ref).all()

    # trained adapters + bias, small batch and a batch that takes the GEMM path
    m, k, r, alpha = 200, 333, 16, 32.0
    w = cases.gaussian(83, (m, k), 0.05)
    bias = cases.gaussian(84, (m,), 0.1)
    q = QLoraLinear.from_linear(w, bias, r, alpha, 0.3)
    b_np = cases.gaussian(85, (m, r), 0.05)
    q.lora_b.copy_(torch.from_numpy(b_np))
    packed, scales = kbref.pack_weights_ternary(w, m, k, 0.3)
    for n in (2, 70):
        x = cases.gaussian(86 + n, (n, k), 1.0)
        y = q(torch.from_numpy(x).cuda()).cpu().numpy()
        base_ref = kbref.q_forward(kbref.TERNARY, packed, scales, None, m, k, x, threads=2)[0]
        y_ref = np_ref.qlora_forward(base_ref, x, q.lora_a.cpu().numpy(), b_np, alpha, r, bias)
        # the quantized base is exact; the two dense f32 products are summed in a different order
        tol = 1e-5 * np.abs(y_ref).max(axis=1, keepdims=True) + 1e-6
        assert (np.abs(y - y_ref) <= tol).all()
    # n-D input keeps its leading dimensions
    y3 = q(torch.from_numpy(cases.gaussian(90, (2, 3, k), 1.0)).cuda())
    assert tuple(y3.shape) == (2, 3, m)
    assert [n for n, _ in q.named_parameters()] == ["lora_a", "lora_b", "bias"]
