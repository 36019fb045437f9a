#!/usr/bin/env python
"""Benchmark of the BitLinear / QuatLinear forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload (N = 1): the batch-1 decode GEMV of the benchmark specification's second configuration —
ternary 4096x4096 weights (absmean-ternarised N(0, 0.02^2), seed 2001), one f32 activation row N(0,1)
(seed 2002) per layer.  A "step" is one pass over a pool of POOL separately allocated copies of that layer
(POOL * 4 MiB > the 126 MB L2, so every weight byte comes from HBM), every layer with its own input row:
ONE kb_linear_group_forward launch — the per-token int8 quantiser runs in the kernel's prologue, then the
streaming GEMV over all layers — captured in a CUDA graph.  value = algorithmic bytes of the step / device
time.  Beside it, at the same level of the JSON line:

  e2e            the same step through kb_linear_group_forward_host (host buffers, copies timed)
  e2e_drop_in    the same pool as POOL synchronous kb_linear_forward_host calls: what a caller of the
                 reference's forward gets without restructuring into a group
  drop_in_chain  the pool as one stream-ordered chain of per-layer launches (dependent layers of a decoder)
  prefill        2048-token GEMMs (4096 -> 11008, 11008 -> 4096) with their own tensor roofline object
  decoder        BitNet-3B-shaped decoder, 512-token prompt + 128 greedy steps, batch 1 and 16
  cpu_baseline   the CPU port of the reference's ternary_matmul on the same packed weights, all host cores

With N > 1 the layers of the pool are independent units, so every rank runs the N = 1 step on its own pool
(weak scaling, no exchange; value = all ranks' bytes / max time over ranks).  What does need an exchange is
reported at the top level as `sharded_projection`: the 8192 -> 28672 projection split by output features
over the ranks at batch 1 / 8 / 64 / 512, every rank ending with the full output, checked against the
unsharded layer and timed next to it in the same run (exchanges: flagged (value, epoch) words, peer stores
with fence and flag barrier, NCCL all-gather), and a chain of dependent sharded layers on the flagged words
(`dependent_chain_flagged`).

`--impl reference` times the CPU port (oracle/kbref.c, a restatement of the reference's CPU code: the
reference is Rust and no Rust toolchain exists here) on the same workload and config; a step there is a
bounded sample of the pool (SAMPLE_LAYERS layers), all host cores.

All inputs are synthetic (no dataset or checkpoint exists for this path).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M_DEC, K_DEC = 4096, 4096
POOL = 160  # 160 x 4 MiB = 640 MiB of packed weights, five times the L2
STREAMS = 16
SAMPLE_LAYERS = 8  # layers of the pool one CPU-arm step runs
METRIC, UNIT = "bitlinear_gemv_hbm_gbs", "GB/s"
WORKLOAD = "decode_gemv_ternary_4096x4096_batch1"


def headline_config(pool_n):
    """What is measured, in the same words for both arms (the driver compares the two dicts)."""
    return {"workload": WORKLOAD, "pool": pool_n, "pool_bytes": pool_n * M_DEC * K_DEC // 4,
            "weights": "ternary 4096x4096, absmean per-tensor scale, N(0, 0.02^2), seed 2001",
            "activations": "f32 [1, 4096] N(0, 1) per layer, seed 2002",
            "l2": "inputs larger than L2 (pool of separately allocated weight copies)"}


def gemv_bytes(m, k, n):
    """Algorithmic bytes of one decode GEMV launch: packed 2-bit weights + scales
    + f32 activations in + f32 outputs out."""
    return m * k // 4 + 4 * m + 4 * k * n + 4 * m * n


def gaussian(seed, shape, sigma):
    return (np.random.default_rng(seed).standard_normal(shape) * sigma).astype(np.float32)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "src": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- CPU arm
def cpu_prepare():
    """The headline layer in the reference wire format (base-243, per-row scales): the same absmean-ternarised
    weights the GPU arm uploads, so both arms run one workload."""
    from oracle import kbref

    w = gaussian(2001, (M_DEC, K_DEC), 0.02)
    x = gaussian(2002, (1, K_DEC), 1.0)
    packed, scales = kbref.pack_weights_ternary_absmean(w, M_DEC, K_DEC)
    return kbref, packed, scales, x


def cpu_step(kbref, packed, scales, x, layers, threads):
    """`layers` forwards of the 4096x4096 layer as the reference runs them today: BitLinear::forward ->
    ternary_matmul with per-call row decode, both transposes, rows in parallel over `threads` cores."""
    t0 = time.perf_counter()
    for _ in range(layers):
        kbref.linear_forward(kbref.TERNARY, packed, scales, None, M_DEC, K_DEC, x, threads=threads)
    return time.perf_counter() - t0


def cpu_reference_arm(steps: int, warmup: int, layers: int = SAMPLE_LAYERS):
    kbref, packed, scales, x = cpu_prepare()
    threads = kbref.host_cores()  # not OMP_NUM_THREADS: torch.distributed.run pins that to 1 for its workers
    for _ in range(max(1, warmup)):
        cpu_step(kbref, packed, scales, x, layers, threads)
    times = [cpu_step(kbref, packed, scales, x, layers, threads) for _ in range(max(1, steps))]
    sec = float(np.mean(times))
    return {"value": layers * gemv_bytes(M_DEC, K_DEC, 1) / sec / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{len(times)} steps of {layers} forwards of the 4096x4096 batch-1 layer (of the pool's {POOL}), "
                      f"{sec / layers * 1e3:.3f} ms per forward; the GPU arm's absmean-ternarised weights in the reference "
                      "wire format, f32 activations, the reference's ternary_matmul restated in C",
            "ms_per_step": sec * 1e3, "ms_per_forward": sec / layers * 1e3}


def run_reference_impl(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    pool_n = args.pool + (args.pool & 1)
    base = cpu_reference_arm(args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": headline_config(pool_n),
        "step": f"{SAMPLE_LAYERS} layers of the pool per step (bounded sample); a whole pool would take "
                f"{base['ms_per_forward'] * pool_n:.1f} ms (extrapolated)",
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def time_graph(torch, fn, steps, warmup, stream, hold_s=0.0):
    """Capture fn() (one step) into a CUDA graph, replay warmup + steps, return seconds per step.
    hold_s > 0 keeps the same graph replaying (untimed) for that long before and after the
    timed steps, so that a clock sampler running alongside sees the GPU under this load."""
    g = torch.cuda.CUDAGraph()

    def hold():
        t_end = time.perf_counter() + hold_s
        while hold_s > 0 and time.perf_counter() < t_end:
            for _ in range(20):
                g.replay()
            stream.synchronize()

    with torch.cuda.stream(stream):
        fn()  # eager warm-up (also sets function attributes outside capture)
        stream.synchronize()
        with torch.cuda.graph(g, stream=stream):
            fn()
        for _ in range(warmup):
            g.replay()
        stream.synchronize()
        hold()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            g.replay()
        e1.record(stream)
        stream.synchronize()
        hold()
    return e0.elapsed_time(e1) / 1e3 / steps, g


class StreamFan:
    """Round-robin fan-out of independent launches over several CUDA streams, fork/join'd
    on a main stream so that the whole step can be captured into one CUDA graph."""

    def __init__(self, torch, main, count):
        self.torch, self.main = torch, main
        self.side = [torch.cuda.Stream(device=main.device) for _ in range(count)] if count > 1 else [main]

    def fork(self):
        if len(self.side) > 1:
            ev = self.torch.cuda.Event()
            ev.record(self.main)
            for st in self.side:
                st.wait_event(ev)

    def join(self):
        if len(self.side) > 1:
            for st in self.side:
                ev = self.torch.cuda.Event()
                ev.record(st)
                self.main.wait_event(ev)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="kore_b200")
    ap.add_argument("--no-extras", action="store_true", help="skip the prefill / quaternary / batch side measurements")
    ap.add_argument("--pool", type=int, default=POOL)
    ap.add_argument("--streams", type=int, default=STREAMS)
    ap.add_argument("--fused-quant", action="store_true",
                    help="N=1: run the activation quantiser inside the GEMV prologue (one launch per layer)")
    ap.add_argument("--no-decoder", action="store_true", help="skip the BitNet-3B-shaped decoder measurement")
    ap.add_argument("--launch", default="grouped", choices=["grouped", "streams"],
                    help="headline step: one grouped launch over the pool of independent layers (default), or one "
                         "quantiser + one GEMV launch per layer spread over --streams streams")
    ap.add_argument("--only", default=None, choices=["gemv_big", "gemv_4096", "group_4096", "small_batch", "medium_batch", "prefill_up", "prefill_down",
                             "decode_step", "decode_step_graph", "decode_step_batch16", "attn_decode", "medium_batch_few_tiles", "flagged_chain", "stream_batch8"],
                    help="run one small case and print its own JSON line (used for ncu captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference_impl(args)

    import torch

    from kore_b200 import _cabi, kernels, nn

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"  # keep NCCL's version banner off stdout (one JSON line only)
        import torch.distributed as dist_

        dist = dist_
        dist.init_process_group("nccl", device_id=dev)
    lib = _cabi.lib()
    if args.only:
        return single_case(torch, lib, _cabi, nn, kernels, dev, args)
    pool_n = args.pool + (args.pool & 1)  # even: the sharded double buffering repeats per replay
    peaks = measured_peaks()

    # ---- weights: one seeded layer, POOL separately allocated copies of this rank's shard
    w = gaussian(2001 + rank, (M_DEC, K_DEC), 0.02)
    proto = nn.BitLinear.new(w, None, 0.3, quantiser="absmean", device=local_rank)
    packed, scales = proto.packed_weights(), proto.scales()
    pool = [proto] + [nn.BitLinear.from_packed(packed, scales, None, K_DEC, M_DEC, device=local_rank) for _ in range(pool_n - 1)]
    x_host = gaussian(2002, (1, K_DEC), 1.0)
    x_pin = torch.from_numpy(x_host).pin_memory()
    x_dev = x_pin.to(dev)
    m_total = M_DEC * world
    main_stream = torch.cuda.Stream(device=dev)
    ld = kernels.act_ld(K_DEC)

    # The headline units are independent layers, so at N > 1 every rank runs the same step on its own
    # pool (no exchange); the column-sharded variants, which do exchange, are measured under `extra`.
    n_streams = max(1, args.streams)
    fan = StreamFan(torch, main_stream, n_streams)
    ys = [torch.zeros((1, M_DEC), dtype=torch.float32, device=dev) for _ in fan.side]
    xqs = [torch.zeros((1, ld), dtype=torch.int8, device=dev) for _ in fan.side]
    sxs = [torch.zeros(1, dtype=torch.float32, device=dev) for _ in fan.side]
    sms = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in fan.side]

    # several independent layers are in flight at once: the GEMV grid sized for sharing the SMs
    gemv_path = _cabi.PATH_GEMV_SHARED if n_streams > 1 else _cabi.PATH_GEMV

    def step():
        fan.fork()
        for j, lay in enumerate(pool):
            i = j % len(fan.side)
            sp = fan.side[i].cuda_stream
            if args.fused_quant:  # quantiser in the GEMV prologue: one launch per layer
                _cabi.check(lib.kb_linear_forward_ex(lay.handle, x_dev.data_ptr(), 1, K_DEC, ys[i].data_ptr(), 0, None,
                                                     gemv_path, None, 0, sp))
                continue
            _cabi.check(lib.kb_quantize_act_i8(x_dev.data_ptr(), 1, K_DEC, xqs[i].data_ptr(), ld, sxs[i].data_ptr(),
                                               sms[i].data_ptr(), sp))
            _cabi.check(lib.kb_linear_forward_q8(lay.handle, xqs[i].data_ptr(), ld, sxs[i].data_ptr(), sms[i].data_ptr(),
                                                 1, ys[i].data_ptr(), 0, None, gemv_path, sp))
        fan.join()

    launches_per_step = (1 if args.fused_quant else 2) * pool_n
    y_view = lambda: ys[(pool_n - 1) % len(fan.side)][0]
    step_streams = step

    # Grouped launch: the pool's layers are independent, so one quantiser launch over the [pool, K]
    # matrix of their inputs and ONE kernel that streams all their weights replace 2 * pool launches.
    grouped = args.launch == "grouped" and not args.fused_quant
    group = None
    if grouped:
        group = nn.LinearGroup(pool)
        x_all = x_dev.expand(pool_n, K_DEC).contiguous()  # every layer gets its own input row (same values)
        xq_all = torch.zeros((pool_n, ld), dtype=torch.int8, device=dev)
        sx_all = torch.zeros(pool_n, dtype=torch.float32, device=dev)
        sm_all = torch.zeros(pool_n, dtype=torch.int32, device=dev)
        y_all = torch.zeros((pool_n, M_DEC), dtype=torch.float32, device=dev)

        def group_only():
            _cabi.check(lib.kb_linear_group_forward_q8(group.handle, xq_all.data_ptr(), ld, sx_all.data_ptr(), sm_all.data_ptr(),
                                                       y_all.data_ptr(), 0, main_stream.cuda_stream))

        def step():  # f32 inputs in: the per-token quantiser runs in the kernel's prologue
            _cabi.check(lib.kb_linear_group_forward(group.handle, x_all.data_ptr(), K_DEC, y_all.data_ptr(), 0,
                                                    main_stream.cuda_stream))

        _cabi.check(lib.kb_quantize_act_i8(x_all.data_ptr(), pool_n, K_DEC, xq_all.data_ptr(), ld, sx_all.data_ptr(),
                                           sm_all.data_ptr(), main_stream.cuda_stream))  # inputs of group_only
        launches_per_step = 1
        y_view = lambda: y_all[pool_n - 1]

    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(local_rank) as clocks:
        sec_per_step, graph = time_graph(torch, step, args.steps, args.warmup, main_stream, hold_s=0.7)
    torch.cuda.synchronize()
    if dist is not None:
        t = torch.tensor([sec_per_step], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec_per_step = float(t.item())
    step_bytes = pool_n * gemv_bytes(M_DEC, K_DEC, 1) * world
    value = step_bytes / sec_per_step / 1e9
    y_chk = y_view().cpu().numpy().copy()  # what the timed path produced for the last layer
    group_sec = streams_sec = None
    if grouped:
        group_sec, _ = time_graph(torch, group_only, args.steps, args.warmup, main_stream)
        if not args.no_extras:
            streams_sec, _ = time_graph(torch, step_streams, max(5, args.steps // 2), args.warmup, main_stream)
            assert (ys[(pool_n - 1) % len(fan.side)][0].cpu().numpy() == y_chk).all(), "grouped and per-layer launches disagree"

    # ---- end to end: host buffers through the C ABI, copies inside the timed region
    y_host = np.zeros((1, M_DEC), np.float32)
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_step():
        for lay in pool:
            _cabi.check(lib.kb_linear_forward_host(lay.handle, x_pin.data_ptr(), 1, K_DEC, y_host.ctypes.data))

    for _ in range(2):
        e2e_step()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_sec = (time.perf_counter() - t0) / e2e_steps
    if dist is not None:
        t = torch.tensor([e2e_sec], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_sec = float(t.item())
    e2e = {"value": step_bytes / e2e_sec / 1e9, "unit": UNIT, "h2d_bytes_per_step": pool_n * 4 * K_DEC,
           "d2h_bytes_per_step": pool_n * 4 * M_DEC, "ms_per_step": e2e_sec * 1e3,
           "note": "kb_linear_forward_host per layer: pinned x -> device, quantiser + GEMV, y -> host, synchronise"}
    if grouped:
        # the same step through the group's host entry point: one call copies the pool's inputs from pinned
        # memory, runs the grouped launch, copies the outputs back and synchronises
        per_layer = dict(e2e)
        xg_pin = x_pin.expand(pool_n, K_DEC).contiguous().pin_memory()
        yg_pin = torch.zeros((pool_n, M_DEC), dtype=torch.float32).pin_memory()

        def e2e_group_step():
            _cabi.check(lib.kb_linear_group_forward_host(group.handle, xg_pin.data_ptr(), yg_pin.data_ptr()))

        for _ in range(3):
            e2e_group_step()
        if dist is not None:
            dist.barrier()
        ge_steps = max(5, min(args.steps, 20))
        t0 = time.perf_counter()
        for _ in range(ge_steps):
            e2e_group_step()
        ge_sec = (time.perf_counter() - t0) / ge_steps
        if dist is not None:
            t = torch.tensor([ge_sec], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ge_sec = float(t.item())
        assert (yg_pin[pool_n - 1].numpy() == y_chk).all(), "group host entry point and graph replay disagree"
        e2e = {"value": step_bytes / ge_sec / 1e9, "unit": UNIT, "h2d_bytes_per_step": pool_n * 4 * K_DEC,
               "d2h_bytes_per_step": pool_n * 4 * M_DEC, "ms_per_step": ge_sec * 1e3,
               "note": "kb_linear_group_forward_host: pinned x [pool, K] -> device, grouped launches, y [pool, M] -> "
                       "pinned host, synchronise (inside the call a pipeline over four chunks of the pool); wall clock "
                       "around the calls"}
        e2e_drop_in = per_layer
    else:
        e2e_drop_in = dict(e2e)
    e2e_drop_in["us_per_call"] = e2e_drop_in["ms_per_step"] * 1e3 / pool_n
    assert (y_host[0] == y_chk).all(), "host entry point and graph replay disagree"

    sharded_extra = sharded_step_extra = None
    if world > 1 and not args.no_extras:
        try:
            sharded_step_extra = column_sharded_step(torch, lib, _cabi, dist, dev, main_stream, rank, local_rank, world, pool,
                                                     x_dev, x_pin, args)
        except Exception as exc:
            sharded_step_extra = {"error": repr(exc)}
        try:
            sharded_extra = sharded_projection(torch, lib, _cabi, nn, dist, dev, main_stream, rank, world, peaks)
        except Exception as exc:
            sharded_extra = {"error": repr(exc)}

    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    kernel_name = "gemv_stream_kernel<grouped,dp4a>"
    if grouped:
        # the step IS one launch of the dominant kernel: its launch duration is the step time
        achieved = pool_n * gemv_bytes(M_DEC, K_DEC, 1) / sec_per_step / 1e9
        pre_q = pool_n * gemv_bytes(M_DEC, K_DEC, 1) / group_sec / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["src"], "kernel": kernel_name,
                    "us_per_launch": sec_per_step * 1e6, "us_per_layer": sec_per_step / pool_n * 1e6,
                    "frac_of_nominal_8000": achieved / 8000.0,
                    "note": "one launch per step: algorithmic bytes of the launch / its duration in the timed region "
                            "(graph replays held under load for 0.7 s before and after, clocks in `clocks`)",
                    "prequantised_inputs_short_run": {"achieved": pre_q, "frac": pre_q / peaks["hbm_gbs"],
                                                      "note": "kb_linear_group_forward_q8 alone, timed without the "
                                                              "sustained-load hold (burst clocks)"}}
    else:
        per_launch_s = sec_per_step / pool_n
        achieved = gemv_bytes(M_DEC, K_DEC, 1) / per_launch_s / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["src"],
                    "kernel": "gemv_kernel<1,4,2>", "us_per_layer": per_launch_s * 1e6,
                    "note": "step time / layers: launches of independent layers overlap across streams",
                    "frac_of_nominal_8000": achieved / 8000.0}
    tpath = os.path.join(ROOT, "profiles", "gemv_traffic.json")
    if os.path.exists(tpath):
        with open(tpath) as f:
            tj = json.load(f)
        per_layer_traffic = tj.get("dram_bytes_per_layer", {}).get(kernel_name if grouped else "gemv_kernel")
        if per_layer_traffic:
            # captured on a smaller pool; the kernel's traffic grows in proportion to the number of layers
            roofline["traffic"] = per_layer_traffic * pool_n
            roofline["traffic_source"] = tj.get("source")

    cpu = cpu_reference_arm(steps=40, warmup=2) if world == 1 else None

    extras = {}
    prefill_obj = decoder_obj = chain_obj = None
    if not args.no_extras and world == 1:
        try:
            extras = side_measurements(torch, lib, _cabi, nn, kernels, dev, main_stream, peaks, args, pool, x_dev)
        except Exception as exc:  # side numbers must never cost the headline line
            extras = {"error": repr(exc)}
        chain_obj = extras.pop("drop_in_chain", None)
        prefill_obj = extras.pop("prefill", None)

    if streams_sec:
        gbs = pool_n * gemv_bytes(M_DEC, K_DEC, 1) / streams_sec / 1e9
        extras[f"gemv_4096x4096_batch1_{n_streams}_streams_2_launches_per_layer"] = {
            "GB/s": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "us_per_layer": streams_sec / pool_n * 1e6,
            "launches_per_step": 2 * pool_n}
    config = headline_config(pool_n)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec_per_step * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic", "config": config,
        "step": ("one grouped launch (kb_linear_group_forward) over the pool's independent layers, f32 inputs [pool, K] "
                 "quantised per token in its prologue; CUDA events around CUDA-graph replays") if grouped else
                f"per layer one quantiser and one GEMV launch, {n_streams} streams",
        "ranks": ("every rank runs the step on its own pool of independent layers, no exchange; the layer that needs "
                  "an exchange is under sharded_projection") if world > 1 else None,
        "roofline": roofline, "e2e": e2e, "e2e_drop_in": e2e_drop_in,
        "gpu_launches": launches_per_step * args.steps * world, "clocks": clocks.summary(),
    }
    if chain_obj:
        line["drop_in_chain"] = chain_obj
    if prefill_obj:
        line["prefill"] = prefill_obj
    if cpu is not None:
        line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if world == 1 and not args.no_extras and not args.no_decoder:
        del pool
        torch.cuda.empty_cache()
        try:
            line["decoder"] = decoder_measurement(torch, dev, peaks)
        except Exception as exc:
            line["decoder"] = {"error": repr(exc)}
    if sharded_step_extra:
        extras["column_sharded_4096_rows_per_rank_step"] = sharded_step_extra
    if sharded_extra:
        line["sharded_projection"] = sharded_extra
    if extras:
        line["extra"] = extras
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def decoder_case(torch, lib, _cabi, dev, args):
    """Small cases of the decoder kernels for ncu: the persistent decode step on an 8-layer slice of the decoder
    configuration (batch 1, 512-token prompt), the graph of separate kernels on a 4-layer slice at batch 16, or the
    batch-16 decode attention kernel on one layer's cache."""
    from kore_b200 import decoder

    if args.only in ("decode_step", "decode_step_graph", "decode_step_batch16"):
        batch = 16 if args.only == "decode_step_batch16" else 1
        cfg = decoder.DecoderConfig(n_layers=8 if batch == 1 else 4)
        weights = decoder.random_weights(cfg, seed=4000, device=dev.index)
        # decode_step: the persistent kernel (the decoder's choice for one sequence); decode_step_graph: the same step as
        # a CUDA graph of the separate kernels
        dec = decoder.BitNetDecoder(cfg, weights, batch=batch, device=dev.index,
                                    persistent=False if args.only == "decode_step_graph" else None)
        prompt = torch.randint(0, cfg.vocab, (batch, 512), generator=torch.Generator().manual_seed(4999)).to(dev)
        torch.argmax(dec.prefill(prompt), dim=1, out=dec.tokens)
        for _ in range(max(1, args.warmup)):
            dec.decode_step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            dec.decode_step()
        e1.record()
        torch.cuda.synchronize()
        dec.check_status()
        per = e0.elapsed_time(e1) / 1e3 / args.steps
        wbytes = cfg.n_layers * (4 * cfg.d_model ** 2 + 3 * cfg.d_model * cfg.d_ff) // 4 + cfg.vocab * cfg.d_model * 4
        print(json.dumps({"case": args.only, "layers": cfg.n_layers, "us_per_step": per * 1e6, "weight_GB/s": wbytes / per / 1e9}), flush=True)
        return
    cfg = decoder.DecoderConfig()
    batch, H, hd, lmax, length = 16, cfg.n_heads, cfg.head_dim, cfg.max_len, 576
    kc = torch.randn((batch, H, lmax, hd), device=dev)
    vc = torch.randn((batch, H, lmax, hd), device=dev)
    q = torch.randn((batch, H * hd), device=dev)
    out = torch.empty((batch, H * hd), device=dev)
    lens = torch.full((batch,), length, dtype=torch.int32, device=dev)
    nbytes = int(lib.kb_attn_decode_scratch_bytes(batch, H))
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    sp = torch.cuda.current_stream().cuda_stream

    def once():
        _cabi.check(lib.kb_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), lens.data_ptr(), batch, H, hd, lmax, out.data_ptr(),
                                       scratch.data_ptr(), nbytes, sp))

    for _ in range(max(1, args.warmup)):
        once()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        once()
    e1.record()
    torch.cuda.synchronize()
    per = e0.elapsed_time(e1) / 1e3 / args.steps
    kv = batch * 2 * length * H * hd * 4
    print(json.dumps({"case": args.only, "batch": batch, "len": length, "us_per_launch": per * 1e6, "GB/s": kv / per / 1e9}), flush=True)


def single_case(torch, lib, _cabi, nn, kernels, dev, args):
    """One kernel on one small case, a handful of eager launches: the command profiled with ncu."""
    if args.only in ("decode_step", "decode_step_graph", "decode_step_batch16", "attn_decode"):
        return decoder_case(torch, lib, _cabi, dev, args)
    if args.only == "flagged_chain":
        return flagged_chain_case(torch, lib, _cabi, nn, dev, args)
    shapes = {"gemv_big": (28672, 8192, 1, 3), "gemv_4096": (4096, 4096, 1, 40), "group_4096": (4096, 4096, 1, 40),
              "small_batch": (28672, 8192, 16, 3), "stream_batch8": (28672, 8192, 8, 3),
              "medium_batch": (28672, 8192, 64, 3),
              "medium_batch_few_tiles": (3584, 8192, 64, 20),  # an eighth of the big layer: K split over CTAs
              "prefill_up": (11008, 4096, 2048, 1), "prefill_down": (4096, 11008, 2048, 1)}
    m, k, n, copies = shapes[args.only]
    w = (torch.randn((m, k), generator=torch.Generator().manual_seed(7)) * 0.02).numpy()
    first = nn.BitLinear.new(w, None, 0.3, quantiser="absmean", device=dev.index)
    del w
    pk, sc = first.packed_weights(), first.scales()
    layers = [first] + [nn.BitLinear.from_packed(pk, sc, None, k, m, device=dev.index) for _ in range(copies - 1)]
    x = torch.from_numpy(gaussian(8, (n, k), 1.0)).to(dev)
    y = torch.empty((n, m), dtype=torch.float32, device=dev)
    xq, sx, sumq = kernels.quantize_act_i8(x)
    path = _cabi.PATH_GEMV if n == 1 else (_cabi.PATH_GEMV_MMA if n <= 32 else _cabi.PATH_GEMM_TC)
    if args.only == "stream_batch8":
        path = _cabi.PATH_GEMV_STREAM
    sp = torch.cuda.current_stream().cuda_stream

    def once():
        for lay in layers:
            _cabi.check(lib.kb_linear_forward_q8(lay.handle, xq.data_ptr(), xq.stride(0), sx.data_ptr(), sumq.data_ptr(), n,
                                                 y.data_ptr(), 0, None, path, sp))

    if args.only == "group_4096":  # the headline launch on a 40-layer pool (160 MiB > L2): one launch per step
        group = nn.LinearGroup(layers)
        xg = x.expand(copies, k).contiguous()
        yg = torch.empty((copies, m), dtype=torch.float32, device=dev)

        def once():  # noqa: F811
            _cabi.check(lib.kb_linear_group_forward(group.handle, xg.data_ptr(), k, yg.data_ptr(), 0, sp))

    for _ in range(max(1, args.warmup)):
        once()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        once()
    e1.record()
    torch.cuda.synchronize()
    per = e0.elapsed_time(e1) / 1e3 / (args.steps * copies)
    if args.only == "group_4096":
        per *= copies  # one launch covers all copies
        print(json.dumps({"case": args.only, "m": m, "k": k, "layers": copies, "us_per_launch": per * 1e6,
                          "GB/s": copies * gemv_bytes(m, k, 1) / per / 1e9}), flush=True)
        return
    print(json.dumps({"case": args.only, "m": m, "k": k, "n": n, "copies": copies, "us_per_launch": per * 1e6,
                      "GB/s": gemv_bytes(m, k, n) / per / 1e9, "TOPS": 2.0 * m * k * n / per / 1e12}), flush=True)


def flagged_chain_case(torch, lib, _cabi, nn, dev, args):
    """The kernels of the flagged exchange on one GPU (a sharded layer with a single rank): a chain of dependent
    8192 -> 3584 -> 8192 layers at one token — every link's forward writes (value, epoch) words, the next link's
    cluster quantiser waits for them — ended by one unpack.  Shapes of an eighth of the 8192 <-> 28672 pair."""
    import ctypes as C

    k, m, pairs = 8192, 3584, 12
    ups, downs = [], []
    wu = (torch.randn((m, k), generator=torch.Generator().manual_seed(7)) * 0.02).numpy()
    wd = (torch.randn((k, m), generator=torch.Generator().manual_seed(8)) * 0.02).numpy()
    u0 = nn.BitLinear.new(wu, None, 0.3, quantiser="absmean", device=dev.index)
    d0 = nn.BitLinear.new(wd, None, 0.3, quantiser="absmean", device=dev.index)
    del wu, wd
    ups = [u0] + [nn.BitLinear.from_packed(u0.packed_weights(), u0.scales(), None, k, m, device=dev.index) for _ in range(pairs - 1)]
    downs = [d0] + [nn.BitLinear.from_packed(d0.packed_weights(), d0.scales(), None, m, k, device=dev.index) for _ in range(pairs - 1)]
    x = torch.from_numpy(gaussian(8, (1, k), 1.0)).to(dev)
    bufs = [torch.zeros((1, k), dtype=torch.int64, device=dev) for _ in range(2)]
    sync = torch.zeros(8, dtype=torch.int32, device=dev)
    ws = torch.empty(1 << 20, dtype=torch.uint8, device=dev)
    y = torch.empty((1, k), dtype=torch.float32, device=dev)
    sp = torch.cuda.current_stream().cuda_stream

    def once():
        seq, src, flagged, width = 0, x, 0, k
        for i in range(pairs):
            for lay, out_dim in ((ups[i], m), (downs[i], k)):
                dst = bufs[seq & 1]
                table = (C.c_void_p * 1)(dst.data_ptr())
                seq += 1
                _cabi.check(lib.kb_linear_forward_sharded_flagged(lay.handle, src.data_ptr(), flagged, width, 1, width, table, 1, 0,
                                                                  out_dim, 0, seq, 0, ws.data_ptr(), ws.numel(), sync.data_ptr(), sp))
                src, flagged, width = dst, 1, out_dim
        _cabi.check(lib.kb_flagged_unpack(src.data_ptr(), k, 1, k, y.data_ptr(), k, seq, sync.data_ptr(), sp))

    for _ in range(max(1, args.warmup)):
        once()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        once()
    e1.record()
    torch.cuda.synchronize()
    per = e0.elapsed_time(e1) / 1e3 / (args.steps * 2 * pairs)
    print(json.dumps({"case": args.only, "links": 2 * pairs, "us_per_link": per * 1e6, "status": int(sync[2].item())}), flush=True)


def column_sharded_step(torch, lib, _cabi, dist, dev, main_stream, rank, local_rank, world, pool, x_dev, x_pin, args):
    """The pool as column-sharded layers: every rank owns a 4096-row shard of a 4096 * world-row layer
    and all ranks end every layer with the full output (epilogue peer stores over NVLink + the flag
    barrier fused into the GEMV tail).  Per layer one quantiser launch and one sharded GEMV, one
    exchange context per stream.  Aggregate GB/s over all ranks, max over ranks."""
    from kore_b200 import kernels, sharded

    pool_n = len(pool)
    m_total = M_DEC * world
    ld = kernels.act_ld(K_DEC)
    n_streams = max(1, min(args.streams, 32))
    while pool_n % (2 * n_streams):
        n_streams -= 1
    fan = StreamFan(torch, main_stream, n_streams)
    ctxs = [sharded.ShardContext(rank, world, m_total, 8, local_rank, dist) for _ in fan.side]
    xqs = [torch.zeros((1, ld), dtype=torch.int8, device=dev) for _ in fan.side]
    sxs = [torch.zeros(1, dtype=torch.float32, device=dev) for _ in fan.side]
    sms = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in fan.side]
    last = [0, 0]

    def step():
        fan.fork()
        for j, lay in enumerate(pool):
            i = j % len(fan.side)
            c = ctxs[i]
            par = c.next_parity()
            last[0], last[1] = i, par
            sp = fan.side[i].cuda_stream
            _cabi.check(lib.kb_quantize_act_i8(x_dev.data_ptr(), 1, K_DEC, xqs[i].data_ptr(), ld, sxs[i].data_ptr(),
                                               sms[i].data_ptr(), sp))
            _cabi.check(lib.kb_linear_forward_sharded_q8(lay.handle, xqs[i].data_ptr(), ld, sxs[i].data_ptr(),
                                                         sms[i].data_ptr(), 1, c.y_tables_host[par], world, rank,
                                                         m_total, rank * M_DEC, _cabi.PATH_GEMV_SHARED,
                                                         c.flag_table.data_ptr(), c.sync_words.data_ptr(), sp))
        fan.join()

    dist.barrier()
    torch.cuda.synchronize()
    sec, _ = time_graph(torch, step, args.steps, args.warmup, main_stream)
    torch.cuda.synchronize()
    t = torch.tensor([sec], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sec = float(t.item())
    for c in ctxs:
        c.check_status()
    # this rank's slice of the last layer against the host entry point
    y_host = np.zeros((1, M_DEC), np.float32)
    _cabi.check(lib.kb_linear_forward_host(pool[-1].handle, x_pin.data_ptr(), 1, K_DEC, y_host.ctypes.data))
    mine = ctxs[last[0]].local_y[last[1]][0, rank * M_DEC:(rank + 1) * M_DEC].cpu().numpy()
    ok = bool((mine == y_host[0]).all())
    dist.barrier()
    for c in ctxs:
        c.close()
    gbs = pool_n * gemv_bytes(M_DEC, K_DEC, 1) * world / sec / 1e9
    return {"GB/s_all_ranks": gbs, "ms_per_step": sec * 1e3, "us_per_layer": sec / pool_n * 1e6, "streams": n_streams,
            "matches_host_entry_point": ok, "exchange": "epilogue peer stores over NVLink + flag barrier fused into the GEMV tail"}


def sharded_projection(torch, lib, _cabi, nn, dist, dev, stream, rank, world, peaks):
    """Sharded-projection configuration of the benchmark specification: ternary K=8192 x M=28672 split by output
    features over the ranks (strong scaling: the layer is fixed), batch 1 / 8 / 64 / 512, every rank ends with the
    full y.  Exchange: epilogue peer stores + flag barrier (p2p), and the NCCL all-gather variant beside it.  A pool of
    separately allocated copies of the shard (> L2 in total) is cycled.  Rank 0 also keeps the unsharded layer: its
    output is the check (every value of rank 0's gathered y, ==) and its time, measured in the same run, the yardstick."""
    from kore_b200 import kernels, sharded

    m, k = 28672, 8192
    w = (torch.randn((m, k), generator=torch.Generator().manual_seed(5001)) * 0.02).numpy()
    full = nn.BitLinear.new(w, None, 0.3, quantiser="absmean", device=dev.index)  # scale from the full tensor
    del w
    packed, scales = full.packed_weights(), full.scales()
    full_pool = None
    if rank == 0:
        full_pool = [full] + [nn.BitLinear.from_packed(packed, scales, None, k, m, device=dev.index) for _ in range(3)]
    else:
        full.close()
    shard_bytes = (m // world) * k // 4
    copies = max(2, int(160e6 // shard_bytes) + 1)
    copies += copies & 1
    ctx = sharded.ShardContext(rank, world, m, 512, dev.index, dist)
    layers = [sharded.ShardedLinear(0, packed, scales, None, k, m, rank, world, device=dev.index, ctx=ctx, dist=dist,
                                    exchange="p2p") for _ in range(copies)]
    sp = stream.cuda_stream
    link_gbs = 770.0  # measured peer-copy bandwidth per direction on this pool
    out = {"world": world, "shard_copies": copies, "layer": "ternary 8192 -> 28672, absmean", "exchange": "p2p = epilogue peer "
           "stores over NVLink + fence + flag barrier; flagged = (value, epoch) words + unpack, no fence or barrier (the "
           "library's default up to 8 tokens); nccl = local slice then all_gather_into_tensor",
           "matches_unsharded": True}
    for nb in (1, 8, 64, 512):
        x_host = gaussian(5002, (nb, k), 1.0)
        x = torch.from_numpy(x_host).to(dev)
        entry = {}
        y_full = None
        if rank == 0:  # the unsharded layer on this GPU, same run
            y_full = torch.empty((nb, m), dtype=torch.float32, device=dev)
            xq, sx, sm = kernels.quantize_act_i8(x)

            def step_full():
                for lay in full_pool:
                    _cabi.check(lib.kb_linear_forward_q8(lay.handle, xq.data_ptr(), xq.stride(0), sx.data_ptr(), sm.data_ptr(),
                                                         nb, y_full.data_ptr(), 0, None, _cabi.PATH_AUTO, sp))

            sec_full, _ = time_graph(torch, step_full, 5, 3, stream)
            entry["us_unsharded_1gpu_same_run"] = sec_full / len(full_pool) * 1e6
            y_chk = np.zeros((nb, m), np.float32)
            _cabi.check(lib.kb_linear_forward_host(full.handle, x_host.ctypes.data, nb, k, y_chk.ctypes.data))
        dist.barrier()

        for lay in layers:
            lay.use_flagged = False  # the fence-and-flag form first; the flagged form (the default up to 8 tokens) below

        xq_c, sx_c, sm_c = kernels.quantize_act_i8(x)  # every sharded form below starts from these, like the unsharded layer

        def step_p2p():
            for lay in layers:
                lay.forward_q8(xq_c, sx_c, sm_c, stream_ptr=sp)

        sec, _ = time_graph(torch, step_p2p, 5, 3, stream)
        t = torch.tensor([sec / copies], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        per = float(t.item())
        y_p2p = layers[-1].forward(x, stream_ptr=sp)  # one more forward (from f32) whose result is read back
        stream.synchronize()
        ok_p2p = bool((y_p2p.cpu().numpy() == y_chk).all()) if rank == 0 else True
        entry.update({"us_per_forward_p2p": per * 1e6, "GB/s": gemv_bytes(m, k, nb) / per / 1e9,
                      "frac_of_measured_hbm_one_gpu": gemv_bytes(m, k, nb) / per / 1e9 / peaks["hbm_gbs"],
                      "TOPS": 2.0 * nb * m * k / per / 1e12,
                      "ingress_bound_us": (world - 1) / world * nb * m * 4 / (link_gbs * 1e9) * 1e6})
        layers[-1].forward(x, stream_ptr=sp)  # keep the parity sequence even
        # chain form (pre-quantised activations, up to 32 tokens): every link waits only for the peers' PREVIOUS
        # publication, behind its own weight stream; one wait ends the chain
        if nb <= 32:
            def step_chain():
                for lay in layers:
                    lay.forward_chain_q8(xq_c, sx_c, sm_c, stream_ptr=sp)
                ctx.wait(sp)

            dist.barrier()
            sec_c, _ = time_graph(torch, step_chain, 5, 3, stream)
            t = torch.tensor([sec_c / copies], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            y_chain = layers[-1].forward_chain_q8(xq_c, sx_c, sm_c, stream_ptr=sp)
            ctx.wait(sp)
            stream.synchronize()
            ok_chain = bool((y_chain.cpu().numpy() == y_chk).all()) if rank == 0 else True
            layers[-1].forward_chain_q8(xq_c, sx_c, sm_c, stream_ptr=sp)  # even parity sequence again
            ctx.wait(sp)
            stream.synchronize()
            entry["us_per_forward_p2p_chain"] = float(t.item()) * 1e6
            entry["chain_matches_unsharded"] = ok_chain
            if rank == 0:
                out["matches_unsharded"] = out["matches_unsharded"] and ok_chain
        for lay in layers:
            lay.use_flagged = True
        # flagged exchange (up to 128 tokens): every value crosses NVLink as an 8-byte (value, epoch) word, nothing
        # is fenced and the producer does not wait; the unpack that follows every forward waits per word and leaves
        # the plain y [nb, m] on every rank
        if nb <= 128:
            y_fl = torch.empty((nb, m), dtype=torch.float32, device=dev)

            def step_flagged():
                for lay in layers:
                    ctx.unpack(lay.forward_flagged_q8(xq_c, sx_c, sm_c, stream_ptr=sp), sp, out=y_fl)

            dist.barrier()
            sec_f, _ = time_graph(torch, step_flagged, 5, 3, stream)
            t = torch.tensor([sec_f / copies], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            y_fl.zero_()
            ctx.unpack(layers[-1].forward_flagged_q8(xq_c, sx_c, sm_c, stream_ptr=sp), sp, out=y_fl)
            ctx.unpack(layers[-1].forward_flagged_q8(xq_c, sx_c, sm_c, stream_ptr=sp), sp, out=y_fl)
            stream.synchronize()
            ok_fl = bool((y_fl.cpu().numpy() == y_chk).all()) if rank == 0 else True
            entry["us_per_forward_flagged"] = float(t.item()) * 1e6
            entry["flagged_matches_unsharded"] = ok_fl
            if rank == 0:
                out["matches_unsharded"] = out["matches_unsharded"] and ok_fl
        # NCCL all-gather variant (eager launches; collectives are not captured here)
        for lay in layers:
            lay.exchange = "collective"
        torch.cuda.synchronize()
        dist.barrier()
        with torch.cuda.stream(stream):
            for lay in layers[:2]:
                y_nccl = lay.forward(x, stream_ptr=sp)
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(3):
                for lay in layers:
                    lay.forward(x, stream_ptr=sp)
            e1.record(stream)
            stream.synchronize()
        ok_nccl = bool((y_nccl.cpu().numpy() == y_chk).all()) if rank == 0 else True
        t = torch.tensor([e0.elapsed_time(e1) / 1e3 / (3 * copies)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        entry["us_per_forward_nccl_allgather"] = float(t.item()) * 1e6
        for lay in layers:
            lay.exchange = "p2p"
        if rank == 0:
            entry["matches_unsharded"] = {"p2p": ok_p2p, "nccl": ok_nccl, "compared": f"all {nb} x {m} outputs of rank 0, =="}
            best = min(entry["us_per_forward_p2p"], entry.get("us_per_forward_p2p_chain", 1e30),
                       entry.get("us_per_forward_flagged", 1e30))
            entry["speedup_vs_unsharded"] = entry["us_unsharded_1gpu_same_run"] / best
            out["matches_unsharded"] = out["matches_unsharded"] and ok_p2p and ok_nccl
        out[f"batch{nb}"] = entry
    ctx.check_status()
    for lay in layers:
        lay.layer.close()
    # dependent chain: up (8192 -> 28672) and down (28672 -> 8192) projections alternate, both sharded by output
    # features, every link reading the previous link's flagged words (the wait sits in its quantiser prologue, behind
    # its own weight stream); one unpack ends the chain.  Rank 0 runs the same chain unsharded in the same run.
    wd = (torch.randn((k, m), generator=torch.Generator().manual_seed(5003)) * 0.02).numpy()
    full_d = nn.BitLinear.new(wd, None, 0.3, quantiser="absmean", device=dev.index)
    del wd
    packed_d, scales_d = full_d.packed_weights(), full_d.scales()
    pairs = max(2, copies // 2)
    ups = [sharded.ShardedLinear(0, packed, scales, None, k, m, rank, world, device=dev.index, ctx=ctx, dist=dist)
           for _ in range(pairs)]
    downs = [sharded.ShardedLinear(0, packed_d, scales_d, None, m, k, rank, world, device=dev.index, ctx=ctx, dist=dist)
             for _ in range(pairs)]
    chain = {"links": 2 * pairs, "layers": "ternary 8192 -> 28672 -> 8192 -> ... (absmean), batch 1 and 2, f32 in, f32 out"}
    for nb in (1, 2):
        x_host = gaussian(5004, (nb, k), 1.0)
        x = torch.from_numpy(x_host).to(dev)
        y_end = torch.empty((nb, k), dtype=torch.float32, device=dev)
        entry = {}
        if rank == 0:
            fu = [full] + [nn.BitLinear.from_packed(packed, scales, None, k, m, device=dev.index) for _ in range(2)]
            fd = [full_d] + [nn.BitLinear.from_packed(packed_d, scales_d, None, m, k, device=dev.index) for _ in range(2)]
            mid = torch.empty((nb, m), dtype=torch.float32, device=dev)
            y_one = torch.empty((nb, k), dtype=torch.float32, device=dev)
            for name, path in (("auto", _cabi.PATH_AUTO), ("streaming_kernel", _cabi.PATH_GEMV_STREAM)):
                def step_one():
                    src = x
                    for i in range(pairs):
                        _cabi.check(lib.kb_linear_forward_ex(fu[i % 3].handle, src.data_ptr(), nb, k, mid.data_ptr(), m, None,
                                                             path, None, 0, sp))
                        _cabi.check(lib.kb_linear_forward_ex(fd[i % 3].handle, mid.data_ptr(), nb, m, y_one.data_ptr(), k, None,
                                                             path, None, 0, sp))
                        src = y_one

                sec_one, _ = time_graph(torch, step_one, 5, 3, stream)
                entry[f"us_per_link_unsharded_1gpu_{name}"] = sec_one / (2 * pairs) * 1e6
            stream.synchronize()
            y_chk = y_one.cpu().numpy().copy()
            for lay in fu[1:] + fd[1:]:
                lay.close()
        dist.barrier()

        ok = True
        # where the consumer waits for the words: 0 = the library's choice (here the cluster quantiser), 1 = in the
        # forward kernel's own prologue (every CTA reads the whole row)
        for name, fuse in (("us_per_link_flagged", 0), ("us_per_link_flagged_wait_in_prologue", 1)):
            def step_links():
                f = ups[0].forward_flagged(x, False, sp)
                f = downs[0].forward_flagged(f, True, sp, fuse)
                for i in range(1, pairs):
                    f = ups[i].forward_flagged(f, True, sp, fuse)
                    f = downs[i].forward_flagged(f, True, sp, fuse)
                ctx.unpack(f, sp, out=y_end)

            y_end.zero_()
            dist.barrier()
            sec_l, _ = time_graph(torch, step_links, 5, 3, stream)
            t = torch.tensor([sec_l / (2 * pairs)], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            stream.synchronize()
            entry[name] = float(t.item()) * 1e6
            if rank == 0:
                ok = ok and bool((y_end.cpu().numpy() == y_chk).all())
        if rank == 0:
            entry["matches_unsharded_chain"] = ok
            entry["speedup_vs_unsharded"] = min(entry["us_per_link_unsharded_1gpu_auto"],
                                                entry["us_per_link_unsharded_1gpu_streaming_kernel"]) / entry["us_per_link_flagged"]
            out["matches_unsharded"] = out["matches_unsharded"] and ok
        chain[f"batch{nb}"] = entry
    out["dependent_chain_flagged"] = chain
    ctx.check_status()
    for lay in ups + downs:
        lay.layer.close()
    ctx.close()
    return out


def decoder_measurement(torch, dev, peaks):
    """Decoder configuration of the benchmark specification: BitNet-b1.58-3B-shaped decoder (26 layers, d 3200, 32 heads,
    FFN 8640, vocab 32000), random init, 512-token prompt then 128 greedy steps, batch 1 and 16.
    Decode steps are CUDA-graph replays timed with CUDA events.  The roofline object counts the bytes a step must
    move: packed projections, the dense f32 lm_head, and the f32 KV cache at the mean sequence length."""
    from kore_b200 import decoder

    cfg = decoder.DecoderConfig()
    t0 = time.perf_counter()
    weights = decoder.random_weights(cfg, seed=4000, device=dev.index)
    build_s = time.perf_counter() - t0
    wbytes = cfg.n_layers * (4 * cfg.d_model ** 2 + 3 * cfg.d_model * cfg.d_ff) // 4
    head_bytes = cfg.vocab * cfg.d_model * 4
    out = {"weights_build_s": build_s, "packed_weight_bytes_per_token": wbytes, "lm_head_bytes": head_bytes,
           "dense_parts": "embedding and lm_head are dense f32", "prompt": 512, "steps": 128}
    for batch in (1, 16):
        dec = decoder.BitNetDecoder(cfg, weights, batch=batch, device=dev.index)
        g = torch.Generator().manual_seed(4999)
        prompt = torch.randint(0, cfg.vocab, (batch, 512), generator=g).to(dev)
        torch.cuda.synchronize()
        e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(2))
        logits = dec.prefill(prompt)
        torch.argmax(logits, dim=1, out=dec.tokens)
        torch.cuda.synchronize()
        dec.decode_step()  # builds the graph (one eager step + capture), then first replay
        torch.cuda.synchronize()
        steps = 127
        e1.record()
        for _ in range(steps):
            dec.decode_step()
        e2.record()
        torch.cuda.synchronize()
        dec_s = e1.elapsed_time(e2) / 1e3
        mean_len = 512 + 1 + steps / 2
        kv_bytes = batch * cfg.n_layers * 2 * cfg.d_model * 4 * mean_len
        step_bytes = wbytes + head_bytes + kv_bytes
        gbs = step_bytes * steps / dec_s / 1e9
        entry = {"decode_tok_per_s": batch * steps / dec_s, "ms_per_step": dec_s / steps * 1e3,
                 "weight_stream_GB/s": wbytes * steps / dec_s / 1e9,
                 "launches_per_step": dec.launches_per_step,
                 "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                              "frac": gbs / peaks["hbm_gbs"], "bytes_per_step": step_bytes,
                              "bytes": "packed projections + f32 lm_head + f32 KV cache at the mean length"}}
        # prefill timed on a second, fresh pass (buffers already allocated)
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        dec.prefill(prompt)
        p1.record()
        torch.cuda.synchronize()
        entry["prefill_ms"] = p0.elapsed_time(p1)
        entry["prefill_tok_per_s"] = batch * 512 / (entry["prefill_ms"] / 1e3)
        out[f"batch{batch}"] = entry
        dec.close()
        del dec
        torch.cuda.empty_cache()
    return out


def side_measurements(torch, lib, _cabi, nn, kernels, dev, stream, peaks, args, pool, x_dev):
    """Other configurations of the benchmark specification, measured briefly.  Returns a dict whose entries
    "drop_in_chain" and "prefill" are lifted to the top level of the JSON line."""
    from oracle import kbref  # CPU port timed beside the small cases (the checker, never the measured GPU path)

    out = {}
    sptr = stream.cuda_stream
    steps, warm = 10, 3
    hbm = peaks["hbm_gbs"]

    # the headline pool as one stream-ordered chain (each layer waits for the previous one)
    y1 = torch.empty((1, M_DEC), dtype=torch.float32, device=dev)
    xq, sx, sumq = kernels.quantize_act_i8(x_dev)

    def chain_fused():
        for lay in pool:
            _cabi.check(lib.kb_linear_forward(lay.handle, x_dev.data_ptr(), 1, y1.data_ptr(), sptr))

    def chain_q8():
        for lay in pool:
            _cabi.check(lib.kb_linear_forward_q8(lay.handle, xq.data_ptr(), xq.stride(0), sx.data_ptr(), sumq.data_ptr(), 1,
                                                 y1.data_ptr(), 0, None, _cabi.PATH_AUTO, sptr))

    chain = {"bound": "hbm", "peak": hbm, "unit": "GB/s",
             "note": "the pool as ONE dependent chain of kb_linear_forward launches (a decoder's layers), CUDA-graph replays"}
    for name, fn in (("f32_input", chain_fused), ("prequantised_input", chain_q8)):
        sec, _ = time_graph(torch, fn, steps, warm, stream)
        gbs = len(pool) * gemv_bytes(M_DEC, K_DEC, 1) / sec / 1e9
        chain[name] = {"us_per_layer": sec / len(pool) * 1e6, "achieved": gbs, "frac": gbs / hbm}
    chain["achieved"], chain["frac"] = chain["f32_input"]["achieved"], chain["f32_input"]["frac"]
    out["drop_in_chain"] = chain

    # the 70B-class FFN shape on one GPU (58.7 MB per layer: launch overheads amortise)
    wbig = (torch.randn((28672, 8192), generator=torch.Generator().manual_seed(5001)) * 0.02).numpy()
    big = nn.BitLinear.new(wbig, None, 0.3, quantiser="absmean", device=dev.index)
    bp, bs = big.packed_weights(), big.scales()
    bigpool = [big] + [nn.BitLinear.from_packed(bp, bs, None, 8192, 28672, device=dev.index) for _ in range(3)]
    del wbig
    for nb in (1, 8, 16, 32, 64):
        xb = torch.from_numpy(gaussian(5002, (nb, 8192), 1.0)).to(dev)
        yb = torch.empty((nb, 28672), dtype=torch.float32, device=dev)
        xqb, sxb, smb = kernels.quantize_act_i8(xb)

        def bigstep():
            for lay in bigpool:
                _cabi.check(lib.kb_linear_forward_q8(lay.handle, xqb.data_ptr(), xqb.stride(0), sxb.data_ptr(), smb.data_ptr(),
                                                     nb, yb.data_ptr(), 0, None, _cabi.PATH_AUTO, sptr))

        sec, _ = time_graph(torch, bigstep, steps, warm, stream)
        gbs = len(bigpool) * gemv_bytes(28672, 8192, nb) / sec / 1e9
        out[f"gemv_8192x28672_batch{nb}_chain_prequantised"] = {"GB/s": gbs, "frac_of_measured_hbm": gbs / hbm,
                                                                "us_per_layer": sec / len(bigpool) * 1e6}
    del bigpool, big

    # quaternary twin of the headline layer: per-layer chain, and the pool through the grouped launch
    w = gaussian(2001, (M_DEC, K_DEC), 0.02)
    qproto = nn.QuatLinear.new(w, device=dev.index)
    qp, qs = qproto.packed_weights(), qproto.scales()
    qpool = [qproto] + [nn.QuatLinear.from_packed(qp, qs, None, K_DEC, M_DEC, device=dev.index) for _ in range(63)]
    for nb in (1, 8):
        x = torch.from_numpy(gaussian(2002, (nb, K_DEC), 1.0)).to(dev)
        y = torch.empty((nb, M_DEC), dtype=torch.float32, device=dev)
        ws_bytes = max(int(lib.kb_linear_workspace_bytes(qproto.handle, nb)), 256)
        ws = torch.empty(ws_bytes + 256, dtype=torch.uint8, device=dev)
        ws_ptr = (ws.data_ptr() + 255) // 256 * 256

        def qstep():
            for lay in qpool:
                _cabi.check(lib.kb_linear_forward_ex(lay.handle, x.data_ptr(), nb, K_DEC, y.data_ptr(), 0, None,
                                                     _cabi.PATH_AUTO, ws_ptr, ws_bytes, sptr))

        sec, _ = time_graph(torch, qstep, steps, warm, stream)
        gbs = len(qpool) * gemv_bytes(M_DEC, K_DEC, nb) / sec / 1e9
        out[f"quat_gemv_4096x4096_batch{nb}_chain"] = {"GB/s": gbs, "frac_of_measured_hbm": gbs / hbm,
                                                        "us_per_launch": sec / len(qpool) * 1e6}
    qgroup = nn.LinearGroup(qpool)
    xg = torch.from_numpy(gaussian(2002, (1, K_DEC), 1.0)).to(dev).expand(len(qpool), K_DEC).contiguous()
    yg = torch.empty((len(qpool), M_DEC), dtype=torch.float32, device=dev)

    def qgroup_step():
        _cabi.check(lib.kb_linear_group_forward(qgroup.handle, xg.data_ptr(), K_DEC, yg.data_ptr(), 0, sptr))

    sec, _ = time_graph(torch, qgroup_step, 20, warm, stream)
    gbs = len(qpool) * gemv_bytes(M_DEC, K_DEC, 1) / sec / 1e9
    out["quat_gemv_4096x4096_batch1_grouped_64_layers"] = {"GB/s": gbs, "frac_of_measured_hbm": gbs / hbm,
                                                            "us_per_launch": sec * 1e6, "note": "256 MiB pool (2x L2)"}
    qgroup.close()
    del qpool

    # prefill GEMM
    prefill = {"bound": "tensor", "unit": "TOP/s", "peak": 4500.0,
               "peak_source": "nominal dense int8 (no int8 figure among the measured peaks); 2x the measured bf16 burst "
                              f"= {2 * peaks['bf16_tflops']:.0f} and a library int8 GEMM timed in the same run are given per shape"}
    for name, m, k, seed in (("up_4096_to_11008", 11008, 4096, 3001), ("down_11008_to_4096", 4096, 11008, 3003)):
        n = 2048
        wg = torch.Generator(device="cpu").manual_seed(seed)
        w = (torch.randn((m, k), generator=wg) * 0.02).numpy()
        lay = nn.BitLinear.new(w, None, 0.3, quantiser="absmean", device=dev.index)
        x = torch.from_numpy(gaussian(3002, (n, k), 1.0)).to(dev)
        y = torch.empty((n, m), dtype=torch.float32, device=dev)
        xq, sx, sumq = kernels.quantize_act_i8(x)

        def gemm_only():
            _cabi.check(lib.kb_linear_forward_q8(lay.handle, xq.data_ptr(), xq.stride(0), sx.data_ptr(), sumq.data_ptr(),
                                                 n, y.data_ptr(), 0, None, _cabi.PATH_GEMM_TC, sptr))

        def full():
            _cabi.check(lib.kb_linear_forward_ex(lay.handle, x.data_ptr(), n, k, y.data_ptr(), 0, None,
                                                 _cabi.PATH_GEMM_TC, None, 0, sptr))

        sec_g, _ = time_graph(torch, gemm_only, 20, 5, stream)
        sec_f, _ = time_graph(torch, full, 20, 5, stream)
        st = C.c_int(0)
        rc = lib.kb_linear_last_device_status(lay.handle, None, C.byref(st))
        ops = 2.0 * n * m * k
        entry = {"gemm_TOPS": ops / sec_g / 1e12, "gemm_ms": sec_g * 1e3, "with_act_quant_TOPS": ops / sec_f / 1e12,
                 "with_act_quant_ms": sec_f * 1e3, "device_status": int(st.value), "status_rc": int(rc),
                 "frac_of_nominal_int8_4500": ops / sec_g / 1e12 / 4500.0,
                 "frac_of_2x_measured_bf16": ops / sec_g / 1e12 / (2 * peaks["bf16_tflops"])}
        try:  # library int8 GEMM on the same shape as a local ceiling
            a8 = torch.randint(-127, 127, (n, k), dtype=torch.int8, device=dev)
            b8 = torch.randint(-1, 2, (k, m), dtype=torch.int8, device=dev)
            with torch.cuda.stream(stream):
                for _ in range(3):
                    torch._int_mm(a8, b8)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(20):
                    torch._int_mm(a8, b8)
                e1.record(stream)
                stream.synchronize()
            lib_s = e0.elapsed_time(e1) / 1e3 / 20
            entry["library_int8_gemm_TOPS"] = ops / lib_s / 1e12
            entry["frac_of_library_int8"] = sec_g and (lib_s / sec_g)
        except Exception as exc:
            entry["library_int8_gemm_TOPS"] = None
            entry["library_error"] = repr(exc)[:200]
        prefill[name] = entry
        del lay
    worst = min(prefill["up_4096_to_11008"]["gemm_TOPS"], prefill["down_11008_to_4096"]["gemm_TOPS"])
    prefill["achieved"], prefill["frac"] = worst, worst / prefill["peak"]
    prefill["kernel"] = "gemm_tc2_kernel (tcgen05.mma.cta_group::2.kind::i8)"
    prefill["note"] = "achieved = the slower of the two 2048-token shapes, GEMM alone on pre-quantised activations"
    out["prefill"] = prefill

    # first configuration of the specification: BitLinear(256 -> 128), 32 tokens — too small for a bandwidth
    # figure, so time only, with the CPU port beside it
    w1, x1 = gaussian(1001, (128, 256), 0.02), gaussian(1002, (32, 256), 1.0)
    lay1 = nn.BitLinear.new(w1, None, 0.3, quantiser="absmean", device=dev.index)
    x1d = torch.from_numpy(x1).to(dev)
    y1d = torch.empty((32, 128), dtype=torch.float32, device=dev)
    ws_b = max(int(lib.kb_linear_workspace_bytes(lay1.handle, 32)), 256)
    ws1 = torch.empty(ws_b + 256, dtype=torch.uint8, device=dev)
    ws1_ptr = (ws1.data_ptr() + 255) // 256 * 256

    def cfg1():
        for _ in range(16):
            _cabi.check(lib.kb_linear_forward_ex(lay1.handle, x1d.data_ptr(), 32, 256, y1d.data_ptr(), 0, None, _cabi.PATH_AUTO,
                                                 ws1_ptr, ws_b, sptr))

    sec, _ = time_graph(torch, cfg1, steps, warm, stream)
    p1, s1 = lay1.packed_weights(), lay1.scales()
    threads = kbref.host_cores()
    t0 = time.perf_counter()
    for _ in range(20):
        kbref.linear_forward(kbref.TERNARY, p1, s1, None, 128, 256, x1, threads=threads)
    cpu_us = (time.perf_counter() - t0) / 20 * 1e6
    y_host = np.zeros((32, 128), np.float32)
    t0 = time.perf_counter()
    for _ in range(20):
        _cabi.check(lib.kb_linear_forward_host(lay1.handle, x1.ctypes.data, 32, 256, y_host.ctypes.data))
    out["bitlinear_256_to_128_32_tokens"] = {"us_per_forward_device": sec / 16 * 1e6,
                                             "us_per_forward_host_buffers": (time.perf_counter() - t0) / 20 * 1e6,
                                             "us_per_forward_cpu_port": cpu_us, "cpu_cores": threads}

    # the reference's own benchmark: quat_matmul at square sizes (benches/matmul_bench.rs:42-78), GF/s = 2 n^3 / t
    sq = {"note": "quaternary, M = N = K; device = resident layer + device buffers (graph replays); host = kb_quat_matmul "
                  "one-shot with host buffers (uploads and repacks the weights every call, like the reference's signature); "
                  "cpu = the reference's single-threaded quat_matmul restated in C"}
    for nsq in (64, 128, 256, 512, 1024):
        wq = gaussian(60 + nsq, (nsq, nsq), 0.02)
        bq = gaussian(61 + nsq, (nsq, nsq), 1.0)
        layq = nn.QuatLinear.new(wq, device=dev.index)
        pq, sq_scales = layq.packed_weights(), layq.scales()
        xd = torch.from_numpy(np.ascontiguousarray(bq.T)).to(dev)
        yd = torch.empty((nsq, nsq), dtype=torch.float32, device=dev)
        wsb = max(int(lib.kb_linear_workspace_bytes(layq.handle, nsq)), 256)
        wsq = torch.empty(wsb + 256, dtype=torch.uint8, device=dev)
        wsq_ptr = (wsq.data_ptr() + 255) // 256 * 256

        def sq_step():
            for _ in range(8):
                _cabi.check(lib.kb_linear_forward_ex(layq.handle, xd.data_ptr(), nsq, nsq, yd.data_ptr(), 0, None, _cabi.PATH_AUTO,
                                                     wsq_ptr, wsb, sptr))

        sec, _ = time_graph(torch, sq_step, steps, warm, stream)
        dev_s = sec / 8
        kernels.quat_matmul(pq, sq_scales, bq, nsq, nsq, nsq)
        t0 = time.perf_counter()
        for _ in range(3):
            kernels.quat_matmul(pq, sq_scales, bq, nsq, nsq, nsq)
        host_s = (time.perf_counter() - t0) / 3
        reps = 3 if nsq <= 512 else 1
        t0 = time.perf_counter()
        for _ in range(reps):
            kbref.quat_matmul(pq, sq_scales, bq, nsq, nsq, nsq)
        cpu_s = (time.perf_counter() - t0) / reps
        fl = 2.0 * nsq ** 3
        sq[str(nsq)] = {"device_us": dev_s * 1e6, "device_GF/s": fl / dev_s / 1e9, "host_one_shot_us": host_s * 1e6,
                        "host_one_shot_GF/s": fl / host_s / 1e9, "cpu_port_us": cpu_s * 1e6, "cpu_port_GF/s": fl / cpu_s / 1e9}
        del layq
    out["reference_bench_quat_matmul_square"] = sq
    return out


if __name__ == "__main__":
    main()
