"""Regenerates tests/golden/recorded.npz from the CPU oracle.

The reference's own tests only assert "finite" for its generator cases and hold no
seeded vectors at all (its RNG is unseeded), so the recorded outputs of the pinned
oracle are the golden vectors for those cases and for the 256->128 configuration.

    python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import kbref  # noqa: E402
from tests import cases  # noqa: E402


def main():
    out = {}
    with open(os.path.join(ROOT, "tests", "golden", "reference_kats.json")) as f:
        kats = json.load(f)
    # generator cases of the reference's tests, R level (what the reference computes)
    for c in kats["generator_cases"]:
        kind = cases.kind_id(c["kind"])
        m, n, k = c["m"], c["n"], c["k"]
        w = cases.rule(c["w_rule"], m * k).reshape(m, k)
        b = cases.rule(c["b_rule"], k * n).reshape(k, n)
        packed, scales = cases.make_weights(kind, "reference", w, c.get("threshold", 0.3))
        fn = kbref.ternary_matmul if kind == kbref.TERNARY else kbref.quat_matmul
        out[f"gen_{c['name']}_r"] = fn(packed, scales, b, m, n, k)
        y, acc = kbref.q_forward(kind, packed, scales, None, m, k, np.ascontiguousarray(b.T))
        out[f"gen_{c['name']}_q_y"] = y
        out[f"gen_{c['name']}_q_acc"] = acc
    # configuration 1: BitLinear(256 -> 128), 32 tokens, seeds 1001 / 1002
    w = cases.gaussian(1001, (128, 256), 0.02)
    x = cases.gaussian(1002, (32, 256), 1.0)
    for name, kind, quantiser in (("tern_ref", kbref.TERNARY, "reference"), ("tern_absmean", kbref.TERNARY, "absmean"),
                                  ("quat", kbref.QUATERNARY, "reference")):
        packed, scales = cases.make_weights(kind, quantiser, w)
        out[f"cfg1_{name}_r"] = kbref.linear_forward(kind, packed, scales, None, 128, 256, x)
        y, acc = kbref.q_forward(kind, packed, scales, None, 128, 256, x)
        out[f"cfg1_{name}_q_y"] = y
        out[f"cfg1_{name}_q_acc"] = acc
        out[f"cfg1_{name}_packed_crc"] = np.array([int(packed.astype(np.uint64).sum()), int(np.bitwise_xor.reduce(packed))])
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "recorded.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
