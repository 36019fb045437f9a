"""LLaMA-style decoder whose seven projections per layer are BitLinear (ternary) layers —
the harness around the quantized-linear path for the BitNet-b1.58-3B-shaped workload.

Structure follows the reference's decoder loop (``crates/kore-edge/src/runtime.rs:106-294``):
pre-norm (RMSNorm), q/k/v projections, half-split RoPE, KV cache, causal attention, output
projection + residual, RMSNorm, SwiGLU feed-forward + residual, final RMSNorm, dense
lm_head, greedy argmax.  q/k/v share one launch (their packed rows are concatenated, each
keeping its own per-tensor scale through the per-row scale vector) and so do gate/up.
RMSNorm and SwiGLU end in the per-token int8 quantiser, the residual adds live in the
projection epilogues.  Embedding and lm_head are dense f32 (in a decode step of up to 16
sequences the head is the library's own streaming kernel with the argmax folded in; in prefill
it is torch's matmul); prefill attention uses torch's scaled_dot_product_attention, decode
attention the library's own kernel.

For one sequence a decode step is ONE launch of the library's persistent decode-step kernel
(``kb_decoder_step``: every phase of every layer, the lm_head GEMV and the argmax inside one
cooperative grid; it also takes two sequences, ``persistent=True``, where the graph is a few
percent faster); larger batches run the step as a CUDA graph of the separate kernels.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np

from . import _cabi, nn


@dataclass
class DecoderConfig:
    n_layers: int = 26
    d_model: int = 3200
    n_heads: int = 32
    d_ff: int = 8640
    vocab: int = 32000
    eps: float = 1e-5
    rope_base: float = 10000.0
    max_len: int = 640

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads


def rope_tables(cfg: DecoderConfig):
    """cos/sin [max_len, head_dim/2] in f32: freq_i = 1 / base^(2i/head_dim), angle = pos * freq_i
    (crates/kore-edge/src/ops/rope.rs:24-27), evaluated once on the host so that every
    consumer multiplies by identical table entries."""
    half = cfg.head_dim // 2
    i = np.arange(half, dtype=np.float32)
    freq = (np.float32(1.0) / np.power(np.float32(cfg.rope_base), (np.float32(2.0) * i / np.float32(cfg.head_dim)).astype(np.float32))).astype(np.float32)
    pos = np.arange(cfg.max_len, dtype=np.float32)[:, None]
    ang = (pos * freq[None, :]).astype(np.float32)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def random_weights(cfg: DecoderConfig, seed: int = 4000, device: int = 0) -> Dict:
    """Random-init weights of the configured shape: projections N(0, 0.02^2) ternarised by
    per-tensor absmean on the device and returned in the reference wire format (so a CPU
    checker and the GPU decoder read identical packed bytes), norms at 1, dense embedding and
    lm_head N(0, 0.02^2)."""
    import torch

    d, f = cfg.d_model, cfg.d_ff
    shapes = {"q": (d, d), "k": (d, d), "v": (d, d), "o": (d, d), "gate": (f, d), "up": (f, d), "down": (d, f)}
    layers = []
    for li in range(cfg.n_layers):
        entry = {}
        for pi, (name, (m, k)) in enumerate(shapes.items()):
            g = torch.Generator().manual_seed(seed + li * 10 + pi)
            w = (torch.randn((m, k), generator=g) * 0.02).numpy()
            lay = nn.BitLinear.new(w, None, 0.3, quantiser="absmean", device=device)
            entry[name] = (lay.packed_weights(), lay.scales(), m, k)
            lay.close()
        entry["norm1"] = np.ones(d, np.float32)
        entry["norm2"] = np.ones(d, np.float32)
        layers.append(entry)
    g = torch.Generator().manual_seed(seed + 999)
    embed = (torch.randn((cfg.vocab, d), generator=g) * 0.02).numpy()
    lm_head = (torch.randn((cfg.vocab, d), generator=g) * 0.02).numpy()
    return {"layers": layers, "embed": embed, "lm_head": lm_head, "norm_f": np.ones(d, np.float32)}


def _concat_rows(parts):
    """Several (packed, scales, m, k) layers with the same k -> one layer of sum(m) rows."""
    k = parts[0][3]
    assert all(p[3] == k for p in parts)
    return (np.concatenate([p[0] for p in parts]), np.concatenate([p[1] for p in parts]), sum(p[2] for p in parts), k)


def _interleave_rows(a, b):
    """Two (packed, scales, m, k) layers of equal shape -> one layer whose rows alternate a_0, b_0,
    a_1, b_1, ...: gate and up rows side by side, so one warp of the GEMV holds both values of a
    SwiGLU output."""
    (pa, sa, m, k), (pb, sb, m2, k2) = a, b
    assert (m, k) == (m2, k2)
    row = pa.size // m
    packed = np.empty((2 * m, row), np.uint8)
    packed[0::2], packed[1::2] = pa.reshape(m, row), pb.reshape(m, row)
    scales = np.empty(2 * m, np.float32)
    scales[0::2], scales[1::2] = sa, sb
    return (packed.reshape(-1), scales, 2 * m, k)


class BitNetDecoder:
    def __init__(self, cfg: DecoderConfig, weights: Dict, batch: int, device: int = 0, max_prefill_tokens: int = 0,
                 persistent: Optional[bool] = None):
        import torch

        self.cfg, self.batch, self.device = cfg, batch, device
        self.torch = torch
        self.lib = _cabi.lib()
        self.dev = torch.device("cuda", device)
        d, f, v = cfg.d_model, cfg.d_ff, cfg.vocab
        self.layers = []
        for lw in weights["layers"]:
            qkv = _concat_rows([lw["q"], lw["k"], lw["v"]])
            gu = _interleave_rows(lw["gate"], lw["up"])
            mk = lambda t: nn.BitLinear.from_packed(t[0], t[1], None, t[3], t[2], device=device)
            self.layers.append({
                "qkv": mk(qkv), "o": mk(lw["o"]), "gu": mk(gu), "down": mk(lw["down"]),
                "norm1": torch.from_numpy(lw["norm1"]).to(self.dev), "norm2": torch.from_numpy(lw["norm2"]).to(self.dev)})
        self.embed = torch.from_numpy(weights["embed"]).to(self.dev)
        self.lm_head = torch.from_numpy(weights["lm_head"]).to(self.dev).contiguous()  # [vocab, d] row-major
        self.norm_f = torch.from_numpy(weights["norm_f"]).to(self.dev)
        cos, sin = rope_tables(cfg)
        self.cos, self.sin = torch.from_numpy(cos).to(self.dev), torch.from_numpy(sin).to(self.dev)
        # KV caches are head-major, [batch, heads, max_len, head_dim]: a head's keys and values are contiguous
        kv_shape = (batch, cfg.n_heads, cfg.max_len, cfg.head_dim)
        self.kc = [torch.zeros(kv_shape, dtype=torch.float32, device=self.dev) for _ in range(cfg.n_layers)]
        self.vc = [torch.zeros(kv_shape, dtype=torch.float32, device=self.dev) for _ in range(cfg.n_layers)]
        self.ld_d, self.ld_f = int(self.lib.kb_act_ld(d)), int(self.lib.kb_act_ld(f))
        self._bufs = {}
        self._alloc(batch)
        if max_prefill_tokens:
            self._alloc(max_prefill_tokens)
        self.positions = torch.zeros(batch, dtype=torch.int32, device=self.dev)
        self.lens = torch.ones(batch, dtype=torch.int32, device=self.dev)
        self.cache_rows = (torch.arange(batch, dtype=torch.int64, device=self.dev) * cfg.max_len)
        self.tokens = torch.zeros(batch, dtype=torch.int64, device=self.dev)
        self.logits = torch.zeros((batch, v), dtype=torch.float32, device=self.dev)
        self.att_bytes = int(self.lib.kb_attn_decode_scratch_bytes(batch, cfg.n_heads))
        self.att_scratch = torch.zeros(self.att_bytes, dtype=torch.uint8, device=self.dev)
        self.graph = None
        self.launches_per_step = 0
        # persistent decode step (one launch per step) where the library supports the shape
        self.persistent = None
        self.hidden_step = torch.zeros((batch, d), dtype=torch.float32, device=self.dev)
        self.head_keys = torch.zeros(batch, dtype=torch.int64, device=self.dev)  # argmax keys of the library's head
        if persistent is None:
            persistent = batch == 1
        if batch <= 2 and persistent:
            n = cfg.n_layers
            arr = lambda ptrs: (C.c_void_p * n)(*ptrs)
            h = C.c_void_p()
            rc = self.lib.kb_decoder_create(
                arr([L["qkv"].handle.value for L in self.layers]), arr([L["o"].handle.value for L in self.layers]),
                arr([L["gu"].handle.value for L in self.layers]), arr([L["down"].handle.value for L in self.layers]),
                arr([L["norm1"].data_ptr() for L in self.layers]), arr([L["norm2"].data_ptr() for L in self.layers]),
                arr([t.data_ptr() for t in self.kc]), arr([t.data_ptr() for t in self.vc]), n, batch, cfg.n_heads, cfg.max_len,
                cfg.vocab, C.c_float(cfg.eps), self.embed.data_ptr(), self.lm_head.data_ptr(), self.norm_f.data_ptr(),
                self.cos.data_ptr(), self.sin.data_ptr(), C.byref(h))
            if rc == _cabi.OK:
                self.persistent = h
            elif rc != _cabi.ERR_UNSUPPORTED:
                _cabi.check(rc)

    def close(self):
        if self.persistent is not None:
            self.lib.kb_decoder_destroy(self.persistent)
            self.persistent = None
        for lay in self.layers:
            for name in ("qkv", "o", "gu", "down"):
                lay[name].close()

    def _alloc(self, n):
        torch, cfg = self.torch, self.cfg
        d, f = cfg.d_model, cfg.d_ff
        z = lambda shape, dt=torch.float32: torch.zeros(shape, dtype=dt, device=self.dev)
        ws_bytes = max(int(self.lib.kb_linear_workspace_bytes(self.layers[0]["o"].handle, n)), 256)
        self._bufs[n] = {
            "hidden": z((n, d)), "qkv": z((n, 3 * d)), "q": z((n, d)), "attn": z((n, d)), "gu": z((n, 2 * f)),
            "xn": z((n, d)), "xq_d": z((n, self.ld_d), torch.int8), "xq_f": z((n, self.ld_f), torch.int8),
            "sx": z(n), "sum": z(n, torch.int32), "ws": z(ws_bytes + 256, torch.uint8), "ws_bytes": ws_bytes,
            "h": z((n, f)) if n <= 2 else None, "absmax": z((2, n)) if n <= 2 else None}

    # ---- one pass over all layers for n tokens ----------------------------------------------
    def _layers(self, n, tokens, positions, cache_rows, lens, prefill_shape=None):
        torch, cfg, lib, B = self.torch, self.cfg, self.lib, self._bufs[n]
        sp = torch.cuda.current_stream(self.device).cuda_stream
        d, f, H, hd = cfg.d_model, cfg.d_ff, cfg.n_heads, cfg.head_dim
        ck = _cabi.check
        ws_ptr = (B["ws"].data_ptr() + 255) // 256 * 256
        torch.index_select(self.embed, 0, tokens, out=B["hidden"])
        launches = 1
        # one or two decode tokens: norms and the SwiGLU ride in the projections' prologue / epilogue
        fused = prefill_shape is None and n <= 2
        for li, L in enumerate(self.layers):
            if fused:
                ck(lib.kb_linear_forward_rmsnorm(L["qkv"].handle, B["hidden"].data_ptr(), L["norm1"].data_ptr(),
                                                 C.c_float(cfg.eps), n, B["qkv"].data_ptr(), 0, 0, None, sp))
            else:
                ck(lib.kb_rmsnorm_quant(B["hidden"].data_ptr(), L["norm1"].data_ptr(), n, d, C.c_float(cfg.eps), None,
                                        B["xq_d"].data_ptr(), self.ld_d, B["sx"].data_ptr(), B["sum"].data_ptr(), sp))
                ck(lib.kb_linear_forward_fused(L["qkv"].handle, None, B["xq_d"].data_ptr(), self.ld_d, B["sx"].data_ptr(),
                                               B["sum"].data_ptr(), n, None, B["qkv"].data_ptr(), 0, _cabi.PATH_AUTO, None, 0, sp))
            ck(lib.kb_rope_kv(B["qkv"].data_ptr(), positions.data_ptr(), cache_rows.data_ptr(), self.cos.data_ptr(),
                              self.sin.data_ptr(), n, H, hd, cfg.max_len, B["q"].data_ptr(), self.kc[li].data_ptr(),
                              self.vc[li].data_ptr(), sp))
            if prefill_shape is None:
                ck(lib.kb_attn_decode(B["q"].data_ptr(), self.kc[li].data_ptr(), self.vc[li].data_ptr(), lens.data_ptr(),
                                      n, H, hd, cfg.max_len, B["attn"].data_ptr(), self.att_scratch.data_ptr(),
                                      self.att_bytes, sp))
                launches += 2
            else:
                b, t = prefill_shape
                qh = B["q"].view(b, t, H, hd).transpose(1, 2)
                kh = self.kc[li][:b, :, :t]
                vh = self.vc[li][:b, :, :t]
                o = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=True)
                B["attn"].view(b, t, H, hd).copy_(o.transpose(1, 2))
                launches += 4
            ck(lib.kb_linear_forward_fused(L["o"].handle, B["attn"].data_ptr(), None, 0, None, None, n, B["hidden"].data_ptr(),
                                           B["hidden"].data_ptr(), 0, _cabi.PATH_AUTO, ws_ptr, B["ws_bytes"], sp))
            if fused:
                am = B["absmax"]
                ck(lib.kb_linear_forward_rmsnorm(L["gu"].handle, B["hidden"].data_ptr(), L["norm2"].data_ptr(),
                                                 C.c_float(cfg.eps), n, B["h"].data_ptr(), 0, 1, am[li & 1].data_ptr(), sp))
                ck(lib.kb_linear_forward_scaled(L["down"].handle, B["h"].data_ptr(), am[li & 1].data_ptr(), n,
                                                B["hidden"].data_ptr(), B["hidden"].data_ptr(), 0, am[(li + 1) & 1].data_ptr(), sp))
                launches += 4
            else:
                ck(lib.kb_rmsnorm_quant(B["hidden"].data_ptr(), L["norm2"].data_ptr(), n, d, C.c_float(cfg.eps), None,
                                        B["xq_d"].data_ptr(), self.ld_d, B["sx"].data_ptr(), B["sum"].data_ptr(), sp))
                ck(lib.kb_linear_forward_fused(L["gu"].handle, None, B["xq_d"].data_ptr(), self.ld_d, B["sx"].data_ptr(),
                                               B["sum"].data_ptr(), n, None, B["gu"].data_ptr(), 0, _cabi.PATH_AUTO, None, 0, sp))
                ck(lib.kb_swiglu_quant_pairs(B["gu"].data_ptr(), n, f, 2 * f, None, B["xq_f"].data_ptr(), self.ld_f,
                                             B["sx"].data_ptr(), B["sum"].data_ptr(), sp))
                ck(lib.kb_linear_forward_fused(L["down"].handle, None, B["xq_f"].data_ptr(), self.ld_f, B["sx"].data_ptr(),
                                               B["sum"].data_ptr(), n, B["hidden"].data_ptr(), B["hidden"].data_ptr(), 0,
                                               _cabi.PATH_AUTO, None, 0, sp))
                launches += 7 + (1 if n > 4 else 0)
        self.launches_per_step = launches + 3
        return B

    def _head(self, hidden_rows):
        """final RMSNorm + dense lm_head on the given rows -> logits"""
        torch, cfg, lib = self.torch, self.cfg, self.lib
        n = hidden_rows.shape[0]
        sp = torch.cuda.current_stream(self.device).cuda_stream
        xn = self._bufs[self.batch]["xn"][:n]
        _cabi.check(lib.kb_rmsnorm_quant(hidden_rows.data_ptr(), self.norm_f.data_ptr(), n, cfg.d_model, C.c_float(cfg.eps),
                                         xn.data_ptr(), None, 0, None, None, sp))
        torch.matmul(xn, self.lm_head.t(), out=self.logits[:n])
        return self.logits[:n]

    # ---- public API --------------------------------------------------------------------------
    def prefill(self, prompt):
        """prompt: int64 [batch, T] (CUDA).  Fills the KV caches and returns the logits of the
        last prompt token, [batch, vocab]."""
        torch = self.torch
        b, t = prompt.shape
        n = b * t
        if n not in self._bufs:
            self._alloc(n)
        pos = torch.arange(t, dtype=torch.int32, device=self.dev).repeat(b)
        rows = (torch.arange(b, dtype=torch.int64, device=self.dev)[:, None] * self.cfg.max_len
                + torch.arange(t, dtype=torch.int64, device=self.dev)[None, :]).reshape(-1)
        B = self._layers(n, prompt.reshape(-1), pos, rows, None, prefill_shape=(b, t))
        last = B["hidden"].view(b, t, -1)[:, -1].contiguous()
        logits = self._head(last)
        self.positions.fill_(t)
        self.lens.fill_(t + 1)
        self.cache_rows.copy_(torch.arange(b, dtype=torch.int64, device=self.dev) * self.cfg.max_len + t)
        return logits

    def _decode_body(self):
        B = self._layers(self.batch, self.tokens, self.positions, self.cache_rows, self.lens)
        if self.batch <= 16 and self.cfg.d_model % 4 == 0 and self.cfg.d_model <= 4096:
            # the library's own head: final norm, streaming f32 lm_head with the argmax folded in, then one launch that
            # stores the tokens and advances positions, lengths and cache rows
            torch, cfg, lib, n = self.torch, self.cfg, self.lib, self.batch
            sp = torch.cuda.current_stream(self.device).cuda_stream
            xn = self._bufs[n]["xn"][:n]
            _cabi.check(lib.kb_rmsnorm_quant(B["hidden"].data_ptr(), self.norm_f.data_ptr(), n, cfg.d_model, C.c_float(cfg.eps),
                                             xn.data_ptr(), None, 0, None, None, sp))
            _cabi.check(lib.kb_lm_head_argmax(xn.data_ptr(), n, cfg.d_model, self.lm_head.data_ptr(), cfg.vocab,
                                              self.logits.data_ptr(), self.head_keys.data_ptr(), sp))
            _cabi.check(lib.kb_decode_advance(self.head_keys.data_ptr(), n, self.tokens.data_ptr(), self.positions.data_ptr(),
                                              self.lens.data_ptr(), self.cache_rows.data_ptr(), sp))
            return
        logits = self._head(B["hidden"])
        self.torch.argmax(logits, dim=1, out=self.tokens)
        self.positions.add_(1)
        self.lens.add_(1)
        self.cache_rows.add_(1)

    def decode_step(self, use_graph: bool = True):
        """One greedy decode step for every sequence: consumes self.tokens (the tokens chosen
        by the previous step), leaves the next tokens in self.tokens and logits in self.logits."""
        torch = self.torch
        if self.persistent is not None:
            sp = torch.cuda.current_stream(self.device).cuda_stream
            _cabi.check(self.lib.kb_decoder_step(self.persistent, self.tokens.data_ptr(), self.positions.data_ptr(),
                                                 self.lens.data_ptr(), self.cache_rows.data_ptr(), self.hidden_step.data_ptr(),
                                                 self.logits.data_ptr(), sp))
            self.launches_per_step = 1
            return
        if not use_graph:
            return self._decode_body()
        if self.graph is None:
            saved = [t.clone() for t in (self.tokens, self.positions, self.lens, self.cache_rows)]
            s = torch.cuda.Stream(device=self.dev)
            s.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(s):
                self._decode_body()  # warm-up outside capture (function attributes, cuBLAS handles)
                s.synchronize()
                for dst, src in zip((self.tokens, self.positions, self.lens, self.cache_rows), saved):
                    dst.copy_(src)
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph, stream=s):
                    self._decode_body()
            torch.cuda.current_stream(self.device).wait_stream(s)
            for dst, src in zip((self.tokens, self.positions, self.lens, self.cache_rows), saved):
                dst.copy_(src)
        self.graph.replay()

    def check_status(self):
        """Raises KoreError(Timeout) if a bounded wait inside a persistent decode step gave up."""
        if self.persistent is not None:
            st = C.c_int(0)
            _cabi.check(self.lib.kb_decoder_status(self.persistent, None, C.byref(st)))

    def generate(self, prompt, steps: int, use_graph: bool = True):
        """Greedy generation: returns int64 [batch, steps] of new tokens."""
        torch = self.torch
        logits = self.prefill(prompt)
        torch.argmax(logits, dim=1, out=self.tokens)
        out = [self.tokens.clone()]
        for _ in range(steps - 1):
            self.decode_step(use_graph)
            out.append(self.tokens.clone())
        return torch.stack(out, dim=1)
