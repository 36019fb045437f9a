"""Writes tests/golden/decoder_kats.json: the exact-valued cases that KORE's own unit tests hold for the
operators around the quantized-linear path (RMSNorm, RoPE, attention, SiLU / softmax, and the fused
RMSNorm references), transcribed with their inputs, the property each test asserts and its tolerance.

Where a reference test compares two in-test formulas instead of stating numbers (the fused RMSNorm +
projection and RMSNorm x SiLU-gate references), the formula is evaluated here in sequential float32 — the
order of the Rust loops — and the values are recorded beside the inputs.  Paths are relative to KORE's
source tree.  Run once; the JSON is committed.
"""
import json
import os

import numpy as np

f32 = np.float32


def seq_sum(vals):
    acc = f32(0.0)
    for v in vals:
        acc = f32(acc + f32(v))
    return acc


def rms_rows(x, gamma, eps):
    """x / rms(x) * gamma, the loop of crates/kore-kernels/src/cpu_fused.rs:176-184"""
    out = np.zeros_like(x)
    for b in range(x.shape[0]):
        ss = seq_sum([f32(v * v) for v in x[b]])
        inv = f32(f32(1.0) / f32(np.sqrt(f32(f32(ss / f32(x.shape[1])) + f32(eps)))))
        for i in range(x.shape[1]):
            out[b, i] = f32(f32(x[b, i] * inv) * gamma[i])
    return out


def main():
    cases = {"_comment": "Known answers of KORE's unit tests for the decoder-step operators; see make_decoder_golden.py"}
    cases["attention"] = [
        {"name": "uniform_single_head", "src": "crates/kore-edge/src/ops/attention.rs:142-158", "seq": 3, "n_heads": 1, "head_dim": 4,
         "causal": False, "q": [1.0] * 12, "k": [1.0] * 12, "v": [1.0] * 12, "expect_all": 1.0, "tol": 1e-4},
        {"name": "causal_first_row_sees_itself", "src": "crates/kore-edge/src/ops/attention.rs:160-177", "seq": 3, "n_heads": 1,
         "head_dim": 2, "causal": True, "q": [1.0] * 6, "k": [1.0] * 6, "v": [float(i) for i in range(6)],
         "expect_row0": [0.0, 1.0], "tol": 1e-4},
        {"name": "uniform_two_heads", "src": "crates/kore-edge/src/ops/attention.rs:179-207", "seq": 2, "n_heads": 2, "head_dim": 2,
         "causal": False, "q": [1.0] * 8, "k": [1.0] * 8, "v": [1.0] * 8, "expect_all": 1.0, "tol": 1e-4},
    ]
    cases["rope"] = [
        {"name": "position_zero_is_identity", "src": "crates/kore-edge/src/ops/rope.rs:43-52", "data": [1.0, 2.0, 3.0, 4.0],
         "n_heads": 1, "head_dim": 4, "pos": 0, "base": 10000.0, "expect": [1.0, 2.0, 3.0, 4.0], "tol": 1e-5},
        {"name": "position_five_changes_values", "src": "crates/kore-edge/src/ops/rope.rs:54-65", "data": [1.0, 2.0, 3.0, 4.0],
         "n_heads": 1, "head_dim": 4, "pos": 5, "base": 10000.0, "changes_by_more_than": 1e-5},
        {"name": "rotation_preserves_pair_norm", "src": "crates/kore-edge/src/ops/rope.rs:67-75", "data": [3.0, 4.0, 1.0, 2.0],
         "n_heads": 1, "head_dim": 4, "pos": 7, "base": 10000.0, "pair": [0, 2], "pair_norm": float(np.sqrt(f32(10.0))), "tol": 1e-4},
    ]
    cases["rmsnorm"] = [
        {"name": "edge_rms_norm", "src": "crates/kore-edge/src/ops/norm.rs:43-49", "x": [1.0, 2.0, 3.0], "gamma": [1.0, 1.0, 1.0],
         "eps": 1e-5, "between": {"0": [0.0, 1.0]}, "greater": {"2": 1.0}},
        {"name": "fused_rms_norm", "src": "crates/kore-kernels/src/cpu_fused.rs:264-276", "x": [1.0, 2.0, 3.0], "gamma": [1.0, 1.0, 1.0],
         "eps": 1e-5, "between": {"0": [0.0, 1.0]}, "greater": {"2": 1.0}},
    ]
    cases["silu"] = [{"name": "silu", "src": "crates/kore-edge/src/ops/activation.rs:87-93", "x": [0.0, 1.0, -1.0],
                      "abs_less": {"0": 1e-5}, "greater": {"1": 0.7}}]
    cases["softmax"] = [
        {"name": "softmax", "src": "crates/kore-edge/src/ops/activation.rs:104-111", "x": [1.0, 2.0, 3.0], "sum": 1.0, "tol": 1e-6,
         "increasing": True},
        {"name": "softmax_stability", "src": "crates/kore-edge/src/ops/activation.rs:113-119", "x": [1000.0, 1001.0, 1002.0], "sum": 1.0,
         "tol": 1e-6, "finite": True},
    ]
    # fused RMSNorm + projection reference (cpu_fused.rs:309-370): two-step and fused forms agree to 1e-5
    hidden, out_dim, batch = 8, 4, 2
    x = np.array([f32(f32(i) * f32(0.3)) - f32(1.0) for i in range(batch * hidden)], f32).reshape(batch, hidden)
    gamma = np.array([f32(1.0) + f32(i) * f32(0.1) for i in range(hidden)], f32)
    w = np.array([f32(f32(i) * f32(0.1)) - f32(0.5) for i in range(out_dim * hidden)], f32).reshape(out_dim, hidden)
    normed = rms_rows(x, gamma, 1e-6)
    proj = np.zeros((batch, out_dim), f32)
    for b in range(batch):
        for j in range(out_dim):
            proj[b, j] = seq_sum([f32(normed[b, kk] * w[j, kk]) for kk in range(hidden)])
    cases["rmsnorm_proj"] = [{"name": "fused_rms_norm_proj_cpu_reference", "src": "crates/kore-kernels/src/cpu_fused.rs:309-370",
                              "x": x.ravel().tolist(), "gamma": gamma.tolist(), "w": w.ravel().tolist(), "batch": batch, "hidden": hidden,
                              "out_dim": out_dim, "eps": 1e-6, "normed": normed.ravel().tolist(), "expect": proj.ravel().tolist(),
                              "tol": 1e-5}]
    # RMSNorm x SiLU gate reference (cpu_fused.rs:451-489): element 5 is zero (SiLU(0) = 0), all finite
    xg = np.arange(1, 9, dtype=f32).reshape(2, 4)
    z = np.array([0.5, 1.0, -0.5, 2.0, -1.0, 0.0, 1.5, -2.0], f32).reshape(2, 4)
    ng = rms_rows(xg, np.ones(4, f32), 1e-6)
    gate = np.zeros_like(ng)
    for b in range(2):
        for c in range(4):
            s = f32(z[b, c] / f32(f32(1.0) + f32(np.exp(f32(-z[b, c])))))
            gate[b, c] = f32(ng[b, c] * s)
    cases["rmsnorm_silu_gate"] = [{"name": "fused_rms_norm_silu_gate_cpu_reference", "src": "crates/kore-kernels/src/cpu_fused.rs:451-489",
                                   "x": xg.ravel().tolist(), "gamma": [1.0] * 4, "z": z.ravel().tolist(), "rows": 2, "cols": 4,
                                   "eps": 1e-6, "expect": gate.ravel().tolist(), "zero_index": 5, "tol": 1e-5}]
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "decoder_kats.json")
    with open(path, "w") as fh:
        json.dump(cases, fh, indent=1)
    print(path)


if __name__ == "__main__":
    main()
