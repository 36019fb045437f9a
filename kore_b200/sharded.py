"""Column-sharded BitLinear / QuatLinear across the GPUs of one box (one process per GPU).

Output features are independent, so rank r keeps weight rows
``[start_r, start_r + size_r)`` of the packed layer and every rank ends up with the full
``y[N, M]``.  Two exchanges are provided:

* ``"p2p"`` (default on GPUs): the GEMV / GEMM epilogue stores each value into every
  rank's output buffer (peer stores over NVLink to IPC-mapped ``cudaMalloc`` memory), then
  a one-CTA barrier kernel publishes completion and waits, bounded, for the peers.  Output
  buffers are double-buffered by call parity so a fast rank never overwrites data a slow
  rank is still reading (a captured CUDA graph should hold an even number of forwards so
  that the parity sequence repeats from replay to replay).
* ``"collective"``: each rank computes ``[N, M/g]`` and the slices are exchanged with
  ``torch.distributed.all_gather_into_tensor`` (NCCL on GPUs; gloo in the CPU tests),
  then laid out as ``[N, M]``.

The reference has nothing distributed; the per-tensor absmean scale is computed on the
full tensor before splitting so that results do not depend on the number of ranks.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import _cabi
from ._cabi import QUATERNARY, TERNARY

MAX_PEERS = 8


# ---- pure host logic (exercised on CPU with gloo) ---------------------------------------
def row_partition(m: int, world: int) -> List[Tuple[int, int]]:
    """(start, size) of every rank's block of output features: sizes differ by at most one
    32-feature granule so every slice but the last starts on a 128-byte boundary of y."""
    if world < 1 or world > MAX_PEERS:
        raise ValueError(f"world size {world} outside 1..{MAX_PEERS}")
    granule = 32
    units = (m + granule - 1) // granule
    base, rem = divmod(units, world)
    out, start = [], 0
    for r in range(world):
        size = min((base + (1 if r < rem else 0)) * granule, max(0, m - start))
        out.append((start, size))
        start += size
    assert start == m
    return out


def wire_row_bytes(kind: int, k: int) -> int:
    return (k + 4) // 5 if kind == TERNARY else (k + 3) // 4


def slice_wire_rows(kind: int, packed, scales, bias, m: int, k: int, start: int, size: int):
    """Rows [start, start+size) of a layer in the reference wire format (row-major, so a
    slice of rows is a contiguous slice of bytes)."""
    rb = wire_row_bytes(kind, k)
    packed = np.ascontiguousarray(packed, dtype=np.uint8).ravel()
    scales = np.ascontiguousarray(scales, dtype=np.float32).ravel()
    if packed.size < m * rb or scales.size < m:
        raise ValueError("packed / scales shorter than the full layer")
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32).ravel()[start:start + size]
    return packed[start * rb:(start + size) * rb], scales[start:start + size], b


def assemble_gathered(chunks: Sequence, sizes: Sequence[int]):
    """[g] x [N, size_r] -> [N, M] (works for numpy arrays and torch tensors)."""
    first = chunks[0]
    if hasattr(first, "numpy") or type(first).__module__.startswith("torch"):
        import torch

        return torch.cat([c[:, :s] for c, s in zip(chunks, sizes)], dim=1)
    return np.concatenate([c[:, :s] for c, s in zip(chunks, sizes)], axis=1)


# ---- symmetric buffers --------------------------------------------------------------------
class _DevView:
    """Exposes a raw device pointer to torch through __cuda_array_interface__."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False),
                                         "version": 3, "strides": None}


class ShardContext:
    """Per-process exchange state shared by all sharded layers: two output buffers
    [max_tokens, m_total] f32 and a flag array per rank, each mapped into every peer."""

    def __init__(self, rank: int, world: int, m_total: int, max_tokens: int, device: int, dist):
        import torch

        self.rank, self.world, self.m_total, self.max_tokens = rank, world, m_total, max_tokens
        self.device, self.dist = device, dist
        self.lib = _cabi.lib()
        self.epoch = 0
        torch.cuda.set_device(device)
        self.y_bytes = (max_tokens * m_total * 4 + 255) // 256 * 256
        # flagged exchange (a few tokens): two buffers of [flagged_tokens, m_total] 8-byte (value, epoch) words
        self.flagged_tokens = min(max_tokens, 128)
        self.f_bytes = (self.flagged_tokens * m_total * 8 + 255) // 256 * 256
        self.f_offset = 2 * self.y_bytes + 256
        total = self.f_offset + 2 * self.f_bytes
        base = C.c_void_p()
        _cabi.check(self.lib.kb_symm_alloc(total, C.byref(base)))
        self.local_base = base.value
        handle = np.zeros(64, np.uint8)
        _cabi.check(self.lib.kb_ipc_export(self.local_base, handle.ctypes.data))
        gathered = [None] * world
        dist.all_gather_object(gathered, handle.tobytes())
        self.peer_bases = []
        for q in range(world):
            if q == rank:
                self.peer_bases.append(self.local_base)
            else:
                p = C.c_void_p()
                h = np.frombuffer(gathered[q], np.uint8).copy()
                _cabi.check(self.lib.kb_ipc_open(h.ctypes.data, C.byref(p)))
                self.peer_bases.append(p.value)
        dev = torch.device("cuda", device)
        # device-side pointer tables: [2][world] output bases, [world] flag arrays
        ybases = [[b + par * self.y_bytes for b in self.peer_bases] for par in range(2)]
        self.y_tables = [torch.tensor(t, dtype=torch.int64, device=dev) for t in ybases]
        self.y_tables_host = [(C.c_void_p * world)(*t) for t in ybases]
        self.flag_table = torch.tensor([b + 2 * self.y_bytes for b in self.peer_bases], dtype=torch.int64, device=dev)
        self.f_tables_host = [(C.c_void_p * world)(*[b + self.f_offset + par * self.f_bytes for b in self.peer_bases])
                              for par in range(2)]
        # {epoch counter, CTA-done counter, status, round of the flagged chains, CTA counter of the unpack, spare}
        self.sync_words = torch.zeros(8, dtype=torch.int32, device=dev)
        self.flag_seq = 0  # position of the last flagged forward in its chain (0: no chain open)
        self.flag_ws = None
        self.epoch_counter = self.sync_words[0:1]
        self.status = self.sync_words[2:3]
        self.local_y = [torch.as_tensor(_DevView(self.local_base + par * self.y_bytes, (max_tokens, m_total), "<f4"),
                                        device=dev) for par in range(2)]
        dist.barrier()

    def close(self):
        if getattr(self, "local_base", None):
            import torch

            torch.cuda.synchronize(self.device)
            self.dist.barrier()
            for q, b in enumerate(self.peer_bases):
                if q != self.rank:
                    self.lib.kb_ipc_close(b)
            self.dist.barrier()
            self.lib.kb_symm_free(self.local_base)
            self.local_base = None

    def next_parity(self) -> int:
        self.epoch += 1
        return self.epoch & 1

    def barrier(self, stream_ptr: int):
        _cabi.check(self.lib.kb_peer_barrier(self.flag_table.data_ptr(), self.world, self.rank,
                                             self.epoch_counter.data_ptr(), self.status.data_ptr(), stream_ptr))

    def wait(self, stream_ptr: int):
        """Waits (on the stream, bounded) until every rank has published as many forwards as this one: ends a
        chain of ``forward_chain_q8`` calls before the last output is read."""
        _cabi.check(self.lib.kb_peer_wait(self.flag_table.data_ptr(), self.world, self.rank, self.epoch_counter.data_ptr(),
                                          self.status.data_ptr(), stream_ptr))

    def local_flagged(self, par: int, n: int, m: int):
        """This rank's flagged buffer of the given parity as an int64 tensor [n, m] (value bits in the low half of
        every word, epoch in the high half)."""
        import torch

        return torch.as_tensor(_DevView(self.local_base + self.f_offset + par * self.f_bytes, (n, m), "<i8"),
                               device=torch.device("cuda", self.device))

    def flagged_workspace(self, n: int, kp: int):
        """(pointer, bytes) of the two-half scratch of the separate flagged quantiser, grown on demand."""
        import torch

        need = 2 * ((n * kp + 255) // 256 * 256 + 2 * ((4 * n + 255) // 256 * 256))
        if self.flag_ws is None or self.flag_ws.numel() < need:  # sized generously once, so that it rarely moves
            self.flag_ws = torch.empty(max(need, 4 << 20), dtype=torch.uint8, device=torch.device("cuda", self.device))
        return self.flag_ws.data_ptr(), self.flag_ws.numel()

    def unpack(self, flagged, stream_ptr: Optional[int] = None, out=None):
        """Ends a chain of flagged forwards: flagged words [n, m] (the view the last one returned) -> plain f32
        [n, m]; waits on the stream, bounded, until every rank's slice has arrived."""
        import torch

        n, m = flagged.shape
        if self.flag_seq < 1:
            raise _cabi.KoreError(_cabi.ERR_INVALID, "no flagged forward to unpack")
        if out is None:
            out = torch.empty((n, m), dtype=torch.float32, device=flagged.device)
        if stream_ptr is None:
            stream_ptr = torch.cuda.current_stream(self.device).cuda_stream
        _cabi.check(self.lib.kb_flagged_unpack(flagged.data_ptr(), flagged.stride(0), n, m, out.data_ptr(), out.stride(0),
                                               self.flag_seq, self.sync_words.data_ptr(), stream_ptr))
        self.flag_seq = 0
        return out

    def check_status(self):
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise _cabi.KoreError(_cabi.ERR_TIMEOUT, f"peer barrier gave up waiting (device code {code})")


class ShardedLinear:
    """One rank's share of a column-sharded layer (CUDA only: the local slice is a
    ``BitLinear`` / ``QuatLinear`` on this rank's GPU).

    Every rank must own at least one output feature: a layer with fewer than ``32 * world``
    features would leave some ranks without a slice, and those ranks would have no launch to
    join the exchange from, so construction fails on every rank alike (the partition is a pure
    function of ``out_features`` and ``world``)."""

    def __init__(self, kind: int, packed, scales, bias, in_features: int, out_features: int, rank: int, world: int,
                 *, device: int = 0, ctx: Optional[ShardContext] = None, dist=None, exchange: str = "p2p"):
        self.kind, self.k, self.m_total = kind, in_features, out_features
        self.rank, self.world = rank, world
        self.parts = row_partition(out_features, world)
        empty = [r for r, (_, size) in enumerate(self.parts) if size == 0]
        if empty:
            raise ValueError(f"{out_features} output features over {world} ranks leave rank(s) {empty} without a slice "
                             f"(slices are multiples of 32 features): use at most {max(1, (out_features + 31) // 32)} ranks")
        self.start, self.size = self.parts[rank]
        self.exchange, self.ctx, self.dist = exchange, ctx, (dist if dist is not None else (ctx.dist if ctx else None))
        # p2p exchange of up to eight tokens: flagged words + unpack instead of peer stores + fence + flag barrier
        # (12.4 against 25.5 us for one token of 8192 -> 28672 on two GPUs)
        self.use_flagged = True
        p, s, b = slice_wire_rows(kind, packed, scales, bias, out_features, in_features, self.start, self.size)
        self.layer = self._build_local(kind, p, s, b, in_features, self.size, device)
        if exchange == "p2p" and ctx is None:
            raise ValueError("the p2p exchange needs a ShardContext")

    def _build_local(self, kind, packed, scales, bias, k, m_local, device):
        from . import nn

        cls = nn.BitLinear if kind == TERNARY else nn.QuatLinear
        return cls.from_packed(packed, scales, bias, k, m_local, device=device)

    # -- product path -------------------------------------------------------------------------
    def forward(self, x, path: int = _cabi.PATH_AUTO, stream_ptr: Optional[int] = None):
        """x: CUDA f32 [N, K] (replicated on every rank) -> y [N, M] on this rank."""
        import torch

        n = x.shape[0]
        if stream_ptr is None and x.is_cuda:
            stream_ptr = torch.cuda.current_stream(x.device.index).cuda_stream
        if self.exchange == "p2p":
            ctx = self.ctx
            if n > ctx.max_tokens or self.m_total != ctx.m_total:
                raise _cabi.KoreError(_cabi.ERR_UNSUPPORTED, "tokens or features exceed the shard context")
            if self._flagged_ok(n, path):
                f = self.forward_flagged(x, False, stream_ptr)
                return ctx.unpack(f, stream_ptr, out=ctx.local_y[ctx.epoch & 1][:n])
            par = ctx.next_parity()
            _cabi.check(ctx.lib.kb_linear_forward_sharded(
                self.layer.handle, x.data_ptr(), n, x.shape[1], ctx.y_tables_host[par], self.world, self.rank,
                self.m_total, self.start, path, None, 0, ctx.flag_table.data_ptr(), ctx.sync_words.data_ptr(),
                stream_ptr))
            return ctx.local_y[par][:n]
        # collective: equal-sized staging blocks, all-gather, then [g, N, s] -> [N, M]
        smax = max(s for _, s in self.parts)
        stage = self._local_forward(x, n, smax, path, stream_ptr)
        out = self._all_gather(stage)
        if n == 1 and all(s == smax for _, s in self.parts):
            return out.reshape(1, self.world * smax)
        return assemble_gathered([out[q] for q in range(self.world)], [s for _, s in self.parts])

    def _flagged_ok(self, n: int, path: int) -> bool:
        ctx = self.ctx
        if not (self.use_flagged and path == _cabi.PATH_AUTO and ctx.flag_seq == 0 and self.m_total == ctx.m_total
                and self.m_total % 2 == 0 and n <= ctx.flagged_tokens):
            return False
        # more tokens can travel as flagged words too (forward_flagged, up to 128), but from 64 tokens on the exchange
        # is bound by NVLink bytes, of which the words carry twice as many (8192 -> 28672 at 64 tokens: 40.1 against
        # 36.7 us on two GPUs, 41.9 against 41.7 on eight)
        return n <= 8 and n * ((self.k + 1023) // 1024 * 1024 + 64) <= 96 * 1024

    def forward_chain_q8(self, xq, sx, sumq, stream_ptr: Optional[int] = None):
        """One link of a chain of sharded layers on pre-quantised activations: the launch waits for the peers'
        PREVIOUS publication after it has started streaming its weights, and publishes its own slice without
        waiting.  Call ``ctx.wait(stream)`` after the last link before reading its output (returned view)."""
        import torch

        ctx, n = self.ctx, xq.shape[0]
        if self.exchange != "p2p" or ctx is None:
            raise _cabi.KoreError(_cabi.ERR_UNSUPPORTED, "forward_chain_q8 uses the p2p exchange")
        if n > ctx.max_tokens or self.m_total != ctx.m_total:
            raise _cabi.KoreError(_cabi.ERR_UNSUPPORTED, "tokens or features exceed the shard context")
        if stream_ptr is None:
            stream_ptr = torch.cuda.current_stream(xq.device.index).cuda_stream
        par = ctx.next_parity()
        _cabi.check(ctx.lib.kb_linear_forward_sharded_chain_q8(
            self.layer.handle, xq.data_ptr(), xq.stride(0), sx.data_ptr(), sumq.data_ptr(), n, ctx.y_tables_host[par],
            self.world, self.rank, self.m_total, self.start, ctx.flag_table.data_ptr(), ctx.sync_words.data_ptr(), stream_ptr))
        return ctx.local_y[par][:n]

    def forward_flagged(self, x, x_is_flagged: bool = False, stream_ptr: Optional[int] = None, fuse: int = 0):
        """One link of a chain of dependent sharded layers (1..8 tokens) on the flagged exchange.  The first link
        takes plain f32 x [N, K]; every later one the flagged view the previous link returned (any layer of the
        same context).  The result is this rank's flagged buffer [N, M]: feed it to the next link, or end the
        chain with ``ctx.unpack``.  Nothing waits in the producer; the consumer waits per word, behind its own
        weight stream (fuse: 0 automatic, 1 in the forward kernel's prologue, 2 in a separate cluster kernel)."""
        import torch

        ctx, n = self.ctx, x.shape[0]
        if self.exchange != "p2p" or ctx is None:
            raise _cabi.KoreError(_cabi.ERR_UNSUPPORTED, "forward_flagged uses the p2p exchange")
        if n > ctx.flagged_tokens or self.m_total > ctx.m_total or self.m_total % 2:
            raise _cabi.KoreError(_cabi.ERR_UNSUPPORTED, "tokens or features exceed the shard context's flagged buffers")
        if bool(x_is_flagged) != (ctx.flag_seq >= 1):
            raise _cabi.KoreError(_cabi.ERR_INVALID, "a chain starts on plain activations and continues on flagged ones")
        if stream_ptr is None:
            stream_ptr = torch.cuda.current_stream(ctx.device).cuda_stream
        ws, ws_bytes = ctx.flagged_workspace(n, (self.k + 127) // 128 * 128)  # for the separate quantiser, where one runs
        par = ctx.next_parity()  # consecutive flagged forwards, across chains too, alternate between the two buffers
        _cabi.check(ctx.lib.kb_linear_forward_sharded_flagged(
            self.layer.handle, x.data_ptr(), 1 if x_is_flagged else 0, x.stride(0), n, self.k, ctx.f_tables_host[par],
            self.world, self.rank, self.m_total, self.start, ctx.flag_seq + 1, fuse, ws, ws_bytes, ctx.sync_words.data_ptr(),
            stream_ptr))
        ctx.flag_seq += 1
        return ctx.local_flagged(par, n, self.m_total)

    def forward_flagged_q8(self, xq, sx, sumq, stream_ptr: Optional[int] = None):
        """First link of a flagged chain on activations that are already quantised (up to 32 tokens)."""
        import torch

        ctx, n = self.ctx, xq.shape[0]
        if self.exchange != "p2p" or ctx is None:
            raise _cabi.KoreError(_cabi.ERR_UNSUPPORTED, "forward_flagged_q8 uses the p2p exchange")
        if n > ctx.flagged_tokens or self.m_total > ctx.m_total or self.m_total % 2:
            raise _cabi.KoreError(_cabi.ERR_UNSUPPORTED, "tokens or features exceed the shard context's flagged buffers")
        if ctx.flag_seq:
            raise _cabi.KoreError(_cabi.ERR_INVALID, "pre-quantised activations start a chain: unpack the open one first")
        if stream_ptr is None:
            stream_ptr = torch.cuda.current_stream(ctx.device).cuda_stream
        par = ctx.next_parity()
        _cabi.check(ctx.lib.kb_linear_forward_sharded_flagged_q8(
            self.layer.handle, xq.data_ptr(), xq.stride(0), sx.data_ptr(), sumq.data_ptr(), n, ctx.f_tables_host[par],
            self.world, self.rank, self.m_total, self.start, 1, ctx.sync_words.data_ptr(), stream_ptr))
        ctx.flag_seq = 1
        return ctx.local_flagged(par, n, self.m_total)

    def _local_forward(self, x, n, smax, path, stream_ptr):
        """This rank's slice of the output in a [N, smax] staging block (columns beyond the slice stay zero)."""
        import torch

        stage = torch.zeros((n, smax), dtype=torch.float32, device=x.device)
        _cabi.check(_cabi.lib().kb_linear_forward_ex(self.layer.handle, x.data_ptr(), n, x.shape[1], stage.data_ptr(),
                                                     smax, None, path, None, 0, stream_ptr))
        return stage

    def _all_gather(self, stage):
        """[N, smax] per rank -> [world, N, smax] on every rank (NCCL)."""
        import torch

        out = torch.empty((self.world,) + tuple(stage.shape), dtype=stage.dtype, device=stage.device)
        self.dist.all_gather_into_tensor(out, stage)
        return out

    __call__ = forward

    def forward_q8(self, xq, sx, sumq, path: int = _cabi.PATH_AUTO, stream_ptr: Optional[int] = None):
        """The p2p exchange on activations that are already quantised (int8 [N, ld], scales [N],
        code sums [N], all CUDA tensors replicated on every rank) -> y [N, M] on this rank."""
        import torch

        ctx, n = self.ctx, xq.shape[0]
        if self.exchange != "p2p" or ctx is None:
            raise _cabi.KoreError(_cabi.ERR_UNSUPPORTED, "forward_q8 uses the p2p exchange")
        if n > ctx.max_tokens or self.m_total != ctx.m_total:
            raise _cabi.KoreError(_cabi.ERR_UNSUPPORTED, "tokens or features exceed the shard context")
        if stream_ptr is None:
            stream_ptr = torch.cuda.current_stream(xq.device.index).cuda_stream
        if self._flagged_ok(n, path):
            f = self.forward_flagged_q8(xq, sx, sumq, stream_ptr)
            return ctx.unpack(f, stream_ptr, out=ctx.local_y[ctx.epoch & 1][:n])
        par = ctx.next_parity()
        _cabi.check(ctx.lib.kb_linear_forward_sharded_q8(
            self.layer.handle, xq.data_ptr(), xq.stride(0), sx.data_ptr(), sumq.data_ptr(), n, ctx.y_tables_host[par],
            self.world, self.rank, self.m_total, self.start, path, ctx.flag_table.data_ptr(), ctx.sync_words.data_ptr(),
            stream_ptr))
        return ctx.local_y[par][:n]
