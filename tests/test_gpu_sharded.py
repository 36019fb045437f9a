"""Column-sharded forward on 2 GPUs (skipped with fewer): both exchanges reproduce the
unsharded oracle result bit for bit on every rank, for decode (GEMV) and prefill (GEMM)."""
import os
import socket

import numpy as np
import pytest

from oracle import kbref
from tests import cases

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ok, msgs = True, []
    try:
        from kore_b200 import sharded

        m, k = 640, 1000
        ctx = sharded.ShardContext(rank, world, m, 256, rank, dist)
        for kind, quantiser in ((kbref.TERNARY, "absmean"), (kbref.QUATERNARY, "reference")):
            w = cases.gaussian(21, (m, k), 0.02)
            packed, scales = cases.make_weights(kind, quantiser, w)
            bias = cases.gaussian(22, (m,), 0.1)
            for exchange in ("p2p", "collective"):
                lay = sharded.ShardedLinear(kind, packed, scales, bias, k, m, rank, world, device=rank, ctx=ctx,
                                            dist=dist, exchange=exchange)
                for n in (1, 3, 5, 16, 64, 200):  # GEMV with fused barrier, small-batch kernel, both GEMMs
                    for rep in range(3):  # repeated calls exercise the double buffering and epochs
                        x = cases.gaussian(100 * n + rep, (n, k), 1.0)
                        y = lay.forward(torch.from_numpy(x).cuda())
                        torch.cuda.synchronize()
                        y_ref = kbref.q_forward(kind, packed, scales, bias, m, k, x, threads=2)[0]
                        same = bool((y.cpu().numpy() == y_ref).all())
                        ok &= same
                        if not same:
                            msgs.append(f"rank {rank} kind {kind} {exchange} n={n} rep={rep} differs")
                if exchange == "p2p":  # the same layer on activations quantised beforehand
                    from kore_b200 import kernels

                    for n in (1, 2, 7, 40):
                        x = cases.gaussian(900 + n, (n, k), 1.0)
                        xq, sx, sumq = kernels.quantize_act_i8(torch.from_numpy(x).cuda())
                        y = lay.forward_q8(xq, sx, sumq)
                        torch.cuda.synchronize()
                        y_ref = kbref.q_forward(kind, packed, scales, bias, m, k, x, threads=2)[0]
                        if not bool((y.cpu().numpy() == y_ref).all()):
                            ok = False
                            msgs.append(f"rank {rank} kind {kind} q8 n={n} differs")
                    # chain form: every link waits for the peers' previous publication only; one wait at the end
                    sp = torch.cuda.current_stream().cuda_stream
                    for n in (1, 2, 5, 20):
                        x = cases.gaussian(950 + n, (n, k), 1.0)
                        xq, sx, sumq = kernels.quantize_act_i8(torch.from_numpy(x).cuda())
                        y_ref = kbref.q_forward(kind, packed, scales, bias, m, k, x, threads=2)[0]
                        outs = [lay.forward_chain_q8(xq, sx, sumq) for _ in range(5)]
                        ctx.wait(sp)
                        torch.cuda.synchronize()
                        for i in (3, 4):  # the two buffers still hold the last two links' outputs
                            if not bool((outs[i].cpu().numpy() == y_ref).all()):
                                ok = False
                                msgs.append(f"rank {rank} kind {kind} chain n={n} link {i} differs")
                        dist.barrier()
        ctx.check_status()
        ctx.close()
    except Exception as exc:  # report instead of hanging the peers
        ok = False
        msgs.append(f"rank {rank}: {exc!r}")
    finally:
        q.put((rank, ok, msgs))
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_sharded_forward_two_gpus():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctxm = mp.get_context("spawn")
    q = ctxm.Queue()
    port = _free_port()
    procs = [ctxm.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in procs]
    results = [q.get(timeout=600) for _ in range(2)]
    [p.join(timeout=120) for p in procs]
    for rank, ok, msgs in results:
        assert ok, msgs
