"""Host logic of the column-sharded layer on CPU: partition, wire-format slicing and the
gather layout, run as two gloo ranks with the oracle standing in for the CUDA compute."""
import os
import socket

import numpy as np
import pytest

from kore_b200 import sharded
from oracle import kbref
from tests import cases


def test_row_partition_properties():
    for m in (1, 31, 32, 33, 4096, 8640, 28672, 11008, 100):
        for world in (1, 2, 3, 4, 8):
            parts = sharded.row_partition(m, world)
            assert len(parts) == world and parts[0][0] == 0
            assert sum(s for _, s in parts) == m
            for (a, sa), (b, _) in zip(parts, parts[1:]):
                assert a + sa == b
            assert all(st % 32 == 0 for st, sz in parts if sz > 0)
    assert sharded.row_partition(28672, 8) == [(i * 3584, 3584) for i in range(8)]
    with pytest.raises(ValueError):
        sharded.row_partition(64, 9)


def test_slice_wire_rows_matches_packing_the_slice():
    w = cases.gaussian(3, (96, 50), 0.02)
    for kind in (kbref.TERNARY, kbref.QUATERNARY):
        packed, scales = cases.make_weights(kind, "reference", w)
        p, s, _ = sharded.slice_wire_rows(kind, packed, scales, None, 96, 50, 32, 64)
        p2, s2 = cases.make_weights(kind, "reference", w[32:96])
        assert (p == p2).all() and (s == s2).all()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_shard_class():
    """ShardedLinear with this rank's CUDA layer replaced by the oracle (the test's own stand-in:
    the package has no CPU compute), so that partition, slicing and gather layout run under gloo."""
    import torch

    class OracleShard(sharded.ShardedLinear):
        def _build_local(self, kind, packed, scales, bias, k, m_local, device):
            return (packed.copy(), scales.copy(), None if bias is None else bias.copy())

        def _local_forward(self, x, n, smax, path, stream_ptr):
            p, s, b = self.layer
            y = kbref.q_forward(self.kind, p, s, b, self.size, self.k, x.numpy())[0]
            stage = torch.zeros((n, smax), dtype=torch.float32)
            stage[:, :self.size] = torch.from_numpy(y)
            return stage

        def _all_gather(self, stage):
            chunks = [torch.empty_like(stage) for _ in range(self.world)]
            self.dist.all_gather(chunks, stage)
            return torch.stack(chunks)

    return OracleShard


def _rank_main(rank, world, port, kind, m, k, n, q):
    import torch
    import torch.distributed as dist

    _OracleShard = _oracle_shard_class()

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = cases.gaussian(11, (m, k), 0.02)
        quantiser = "absmean" if kind == kbref.TERNARY else "reference"
        packed, scales = cases.make_weights(kind, quantiser, w)  # scale from the FULL tensor
        bias = cases.gaussian(12, (m,), 0.1)
        x = cases.gaussian(13, (n, k), 1.0)

        lay = _OracleShard(kind, packed, scales, bias, k, m, rank, world, dist=dist, exchange="collective")
        y = lay.forward(torch.from_numpy(x)).numpy()
        y_ref = kbref.q_forward(kind, packed, scales, bias, m, k, x)[0]
        q.put((rank, bool((y == y_ref).all()), y.shape))
    except Exception as exc:  # report instead of leaving the parent waiting on the queue
        q.put((rank, False, repr(exc)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind", [kbref.TERNARY, kbref.QUATERNARY])
@pytest.mark.parametrize("m,k,n", [(256, 96, 3), (100, 64, 1)])
def test_two_gloo_ranks_reproduce_the_unsharded_result(kind, m, k, n):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, kind, m, k, n, q)) for r in range(2)]
    [p.start() for p in procs]
    results = [q.get(timeout=120) for _ in range(2)]
    [p.join(timeout=60) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    for rank, same, shape in results:
        assert same, f"rank {rank} disagrees with the unsharded oracle: {shape}"
        assert tuple(shape) == (n, m)


def test_layer_too_small_for_the_ranks_is_rejected_on_every_rank():
    """64 features over 4 ranks would leave two ranks without a slice: every rank must fail at
    construction (before any exchange), not only the empty ones."""
    cls = _oracle_shard_class()
    w = cases.gaussian(5, (64, 32), 0.02)
    packed, scales = cases.make_weights(kbref.TERNARY, "absmean", w)
    for rank in range(4):
        with pytest.raises(ValueError, match="without a slice"):
            cls(kbref.TERNARY, packed, scales, None, 32, 64, rank, 4, exchange="collective")
    # 64 features over 2 ranks is fine
    cls(kbref.TERNARY, packed, scales, None, 32, 64, 1, 2, exchange="collective")
