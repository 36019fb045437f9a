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
                for n in (1, 3, 5, 16, 64, 100, 200):  # flagged words / GEMV with fused barrier, small-batch kernel, both GEMMs
                    for rep in range(4):  # repeated calls exercise the double buffering and epochs
                        lay.use_flagged = rep < 2  # up to 8 tokens: flagged words first, then peer stores + fence + barrier
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
        # flagged exchange: a dependent chain 1000 -> 640 -> 1000 -> 640 ... in which every link reads the previous
        # link's (value, epoch) words and waits per word; one unpack at the end; against the oracle's chain
        m, k = 640, 1000
        ctx = sharded.ShardContext(rank, world, max(m, k), 128, rank, dist)
        kind = kbref.TERNARY
        wa, wb = cases.gaussian(31, (m, k), 0.02), cases.gaussian(32, (k, m), 0.02)
        pa, sa = cases.make_weights(kind, "absmean", wa)
        pb, sb = cases.make_weights(kind, "absmean", wb)
        la = sharded.ShardedLinear(kind, pa, sa, None, k, m, rank, world, device=rank, ctx=ctx, dist=dist)
        lb = sharded.ShardedLinear(kind, pb, sb, None, m, k, rank, world, device=rank, ctx=ctx, dist=dist)
        for n in (1, 2, 3, 8, 40, 100):  # streaming kernel up to 8 tokens, the medium-batch GEMM beyond
            for rep in range(2):
                x = cases.gaussian(700 + 10 * n + rep, (n, k), 1.0)
                ref = x
                fuse = 1 + rep  # the wait in the forward kernel's prologue / in the separate cluster quantiser
                f = la.forward_flagged(torch.from_numpy(x).cuda())
                ref = kbref.q_forward(kind, pa, sa, None, m, k, ref, threads=2)[0]
                for link in range(3):
                    f = lb.forward_flagged(f, x_is_flagged=True, fuse=fuse)
                    ref = kbref.q_forward(kind, pb, sb, None, k, m, ref, threads=2)[0]
                    f = la.forward_flagged(f, x_is_flagged=True, fuse=fuse)
                    ref = kbref.q_forward(kind, pa, sa, None, m, k, ref, threads=2)[0]
                y = ctx.unpack(f)
                torch.cuda.synchronize()
                if not bool((y.cpu().numpy() == ref).all()):
                    ok = False
                    msgs.append(f"rank {rank} flagged chain n={n} rep={rep} differs")
            # stand-alone: pre-quantised input, unpack after every forward
            x = cases.gaussian(800 + n, (n, k), 1.0)
            xq, sx, sumq = kernels.quantize_act_i8(torch.from_numpy(x).cuda())
            y_ref = kbref.q_forward(kind, pa, sa, None, m, k, x, threads=2)[0]
            for rep in range(4):
                y = ctx.unpack(la.forward_flagged_q8(xq, sx, sumq))
                torch.cuda.synchronize()
                if not bool((y.cpu().numpy() == y_ref).all()):
                    ok = False
                    msgs.append(f"rank {rank} flagged q8 n={n} rep={rep} differs")
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


@pytest.mark.parametrize("k,m", [(1000, 640), (8192, 384), (28672, 96)])
def test_flagged_words_single_rank(k, m):
    """The flagged form with one rank (no peers): the producer writes (value, epoch) words, the next forward's
    prologue waits for them per word and quantises them, the unpack strips them; every step against the oracle.
    Covers both forms of the flagged prologue (one cell per thread held in registers; rows read twice)."""
    import ctypes as C

    import torch

    from kore_b200 import _cabi, nn

    lib = _cabi.lib()
    kind = kbref.TERNARY
    wa, wb = cases.gaussian(41, (m, k), 0.02), cases.gaussian(42, (k, m), 0.02)
    pa, sa = cases.make_weights(kind, "absmean", wa)
    pb, sb = cases.make_weights(kind, "absmean", wb)
    ba = cases.gaussian(43, (m,), 0.1)
    la = nn.BitLinear.from_packed(pa, sa, ba, k, m, device=0)
    lb = nn.BitLinear.from_packed(pb, sb, None, m, k, device=0)
    dev = torch.device("cuda", 0)
    sync = torch.zeros(8, dtype=torch.int32, device=dev)
    sp = torch.cuda.current_stream().cuda_stream
    # few tokens: streaming kernel (the staged rows must fit in shared memory); more: the medium-batch GEMM, which
    # needs rows of at least 128 packed bytes in both layers of the chain
    tokens = (1, 2, 5, 8) if k <= 8192 else (1, 2, 3)
    if min(k, m) >= 512:
        tokens += (40, 100)
    for n in tokens:
        fa = torch.zeros((n, m), dtype=torch.int64, device=dev)
        fb = torch.zeros((n, k), dtype=torch.int64, device=dev)
        x = cases.gaussian(500 + n, (n, k), 1.0)
        xd = torch.from_numpy(x).cuda()

        for fuse in (1, 2):  # the wait in the forward kernel's prologue / in the separate cluster quantiser
            seq = [0]

            def fwd(layer, src, flagged_in, dst, in_dim, out_dim):
                table = (C.c_void_p * 1)(dst.data_ptr())
                seq[0] += 1
                _cabi.check(lib.kb_linear_forward_sharded_flagged(layer.handle, src.data_ptr(), 1 if flagged_in else 0,
                                                                  src.stride(0), n, in_dim, table, 1, 0, out_dim, 0, seq[0],
                                                                  fuse, None, 0, sync.data_ptr(), sp))

            round_before = int(sync[3].item())
            fwd(la, xd, False, fa, k, m)
            ref = kbref.q_forward(kind, pa, sa, ba, m, k, x, threads=2)[0]
            for link in range(2):
                fwd(lb, fa, True, fb, m, k)
                ref = kbref.q_forward(kind, pb, sb, None, k, m, ref, threads=2)[0]
                fwd(la, fb, True, fa, k, m)
                ref = kbref.q_forward(kind, pa, sa, ba, m, k, ref, threads=2)[0]
            y = torch.empty((n, m), dtype=torch.float32, device=dev)
            _cabi.check(lib.kb_flagged_unpack(fa.data_ptr(), fa.stride(0), n, m, y.data_ptr(), m, seq[0], sync.data_ptr(), sp))
            torch.cuda.synchronize()
            assert int(sync[2].item()) == 0
            assert int(sync[3].item()) == round_before + 1  # the unpack advanced the round
            words = fa.cpu().numpy()
            assert ((words >> 32) & 0xffffffff == ((round_before << 8) | seq[0])).all()  # every word carries its epoch
            assert (y.cpu().numpy() == ref).all(), f"n={n} fuse={fuse}"
    for lay in (la, lb):
        st = C.c_int(-1)
        assert lib.kb_linear_last_device_status(lay.handle, None, C.byref(st)) == 0 and st.value == 0, st.value


def test_flagged_unpack_reports_a_word_that_never_arrives():
    """A flag that nothing sets: the bounded wait ends with the status code, the context stays usable."""
    import torch

    from kore_b200 import _cabi

    lib = _cabi.lib()
    dev = torch.device("cuda", 0)
    sync = torch.zeros(8, dtype=torch.int32, device=dev)
    f = torch.zeros((1, 64), dtype=torch.int64, device=dev)  # holds epoch 0; the unpack expects (0 << 8) | 1
    y = torch.empty((1, 64), dtype=torch.float32, device=dev)
    _cabi.check(lib.kb_flagged_unpack(f.data_ptr(), 64, 1, 64, y.data_ptr(), 64, 1, sync.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert int(sync[2].item()) == 110
    assert float((torch.ones(4, device=dev) * 2).sum().item()) == 8.0
