"""Batched decode: one new token for each of B sequences per step.

The reference has no serving loop of its own; a batch reaches its operator as the tokens of one
``linear`` call, and every token count below the prefill threshold goes to the decode GEMV with one grid
row per token (``texelator/cuda/texelator_cuda.cu:1438-1468``), which streams the whole matrix once per
token.  Here the B rows of a step go through the multi-token decode kernel, which reads the matrix once
for all of them (K ranges per CTA, so that the B activation rows of a range fit in shared memory), and the
steps between the linears are the library's glue kernels with a batch dimension:

    add_rmsnorm [B, hidden] -> qkv linear -> attention_step_batch (RoPE, cache append, attention of every
    sequence at its own position) -> o linear (+ all-reduce) -> add_rmsnorm -> gate/up linear ->
    silu_mul_pairs -> down linear (+ all-reduce)

Tensor-parallel runs all-reduce the [B, hidden] partial sums of the row-parallel linears with NCCL inside
the captured graph; the vocabulary-parallel output head gathers one (score, token) pair per sequence and rank.
Weights, sharding and the packing of the projections are ``modeling.BC4Decoder``'s.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .modeling import BC4Decoder, DecoderConfig, _rmsnorm


class BatchedBC4Decoder(BC4Decoder):
    """``BC4Decoder`` with ``batch`` independent sequences: caches ``[layers, B, kv_heads, max_len, head_dim]``,
    per-sequence positions, static ``[B, ...]`` buffers for a captured step."""

    def __init__(self, config: DecoderConfig, device, max_len: int, batch: int, **kwargs):
        super().__init__(config, device, max_len=16, **kwargs)      # the parent's one-sequence caches stay tiny
        if not self.fused:
            raise ValueError(f"{config.name}: batched decode needs the library's glue kernels (head_dim 128, group <= 8)")
        c, self.batch, self.max_len = config, batch, max_len
        kv_heads, q_heads = c.kv_heads // self.world, c.q_heads // self.world
        if batch < 1 or batch * kv_heads > 4096:
            raise ValueError("batch * kv heads per rank must be between 1 and 4096")
        bf = dict(dtype=torch.bfloat16, device=self.device)
        with torch.cuda.device(self.device):
            from .modeling import _rope_tables
            self.cos, self.sin = _rope_tables(c, max_len, self.device)
            self.k_cache = torch.zeros(c.layers, batch, kv_heads, max_len, c.head_dim, **bf)
            self.v_cache = torch.zeros_like(self.k_cache)
            self.tok = torch.zeros(batch, dtype=torch.int64, device=self.device)
            self.pos = torch.zeros(batch, dtype=torch.int64, device=self.device)
            self.next_tok = torch.zeros(batch, dtype=torch.int64, device=self.device)
            self.last_hidden = torch.zeros(batch, c.hidden, **bf)
            self.buf_h = torch.zeros(batch, c.hidden, **bf)
            self.buf_x = torch.zeros(batch, c.hidden, **bf)
            self.buf_qkv = torch.zeros(batch, self.q_loc + 2 * self.kv_loc, **bf)
            self.buf_attn = torch.zeros(batch, self.q_loc, **bf)
            self.buf_o = torch.zeros(batch, c.hidden, **bf)
            self.buf_gu = torch.zeros(batch, 2 * self.i_loc, **bf)
            self.buf_act = torch.zeros(batch, self.i_loc, **bf)
            self.buf_down = torch.zeros(batch, c.hidden, **bf)
            self.attn_scratch = torch.zeros(batch * self.ext.attention_step_scratch_floats(q_heads, max_len),
                                            dtype=torch.float32, device=self.device)
            if self.vocab_parallel:
                self.best_local = torch.zeros(batch, 2, dtype=torch.float32, device=self.device)
                self.best_all = torch.zeros(self.world, batch, 2, dtype=torch.float32, device=self.device)
            # a step's B rows go to the multi-token decode kernel (weights read once for all rows); prompts stay on
            # the tensor-core tiles
            from .runtime import PREFILL_THRESHOLD, PREFILL_TILE_ROWS
            for handle in self.handles:
                self.ext.set_prefill(handle, max(PREFILL_THRESHOLD, batch + 1), PREFILL_TILE_ROWS)
        self.single = False
        self.graph = None

    # -- which kernel serves a step's B rows -------------------------------------------------------------
    @torch.no_grad()
    def tune_decode_kernel(self, repeats: int = 3) -> dict:
        """For batches at or above the reference's prefill threshold (16), time every projection's B-row linear
        through the multi-token decode kernel and through the two narrow tensor-core tiles, over all layers (so
        the weights come from HBM), and keep the fastest per projection -- the per-shape selection the reference's
        autotuner makes for prompts (texelator/autotune.py:170-193), applied to the decode batch.  All ranks of a
        tensor-parallel run take rank 0's choice.  Returns {projection: (kernel, microseconds per call)}."""
        from .autotune import CANDIDATES
        from .runtime import PREFILL_THRESHOLD, PREFILL_TILE_ROWS
        ext, chosen = self.ext, {}
        if self.batch < PREFILL_THRESHOLD:
            return chosen
        options = [("gemv", self.batch + 1, CANDIDATES["umma_128x64x128"]), ("umma_128x64x128", PREFILL_THRESHOLD, CANDIDATES["umma_128x64x128"]),
                   ("umma_128x128x128", PREFILL_THRESHOLD, CANDIDATES["umma_128x128x128"])]
        groups = (("qkv", self.h_qkv, self.buf_x, self.buf_qkv), ("o", self.h_o, self.buf_attn, self.buf_o),
                  ("gate_up", self.h_gu, self.buf_x, self.buf_gu), ("down", self.h_down, self.buf_act, self.buf_down))
        for name, handles, x, y in groups:
            timings = []
            for _, threshold, backend in options:
                for handle in handles:
                    ext.set_prefill(handle, threshold, PREFILL_TILE_ROWS)
                    ext.set_prefill_backend(handle, backend)
                for handle in handles:                  # warm-up pass (first launches set kernel attributes)
                    ext.linear_out(handle, x, y)
                begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                begin.record()
                for _ in range(repeats):
                    for handle in handles:
                        ext.linear_out(handle, x, y)
                end.record()
                end.synchronize()
                timings.append(begin.elapsed_time(end) * 1000 / (repeats * len(handles)))
            best = torch.tensor([min(range(len(options)), key=timings.__getitem__)], device=self.device)
            if self.world > 1:
                torch.distributed.broadcast(best, src=0, group=self.group)
            pick = int(best.item())
            for handle in handles:
                ext.set_prefill(handle, options[pick][1], PREFILL_TILE_ROWS)
                ext.set_prefill_backend(handle, options[pick][2])
            chosen[name] = (options[pick][0], timings[pick], dict(zip((o[0] for o in options), timings)))
        return chosen

    # -- prompt --------------------------------------------------------------------------------------
    @torch.no_grad()
    def prefill_sequence(self, sequence: int, ids: torch.Tensor, dense: bool = False) -> torch.Tensor:
        """Run one sequence's prompt from position 0 (the linears take the tensor-core path from the prefill
        threshold on), fill its cache rows, set its position; returns the final hidden states ``[T, hidden]``."""
        tokens = ids.numel()
        index = torch.arange(tokens, device=self.device)
        cos, sin = self.cos[:tokens], self.sin[:tokens]
        k_all, v_all = self.k_cache, self.v_cache
        self.k_cache, self.v_cache = k_all[:, sequence], v_all[:, sequence]       # views: _layer indexes [layer]
        try:
            def attend(layer, q):
                k = self.k_cache[layer][:, :tokens].unsqueeze(0)
                v = self.v_cache[layer][:, :tokens].unsqueeze(0)
                return F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)

            h = self.embed.index_select(0, ids.to(self.device).reshape(-1))
            for layer in range(self.config.layers):
                h = self._layer(layer, h, cos, sin, index, attend, dense)
        finally:
            self.k_cache, self.v_cache = k_all, v_all
        self.pos[sequence] = tokens
        return _rmsnorm(h, self.final_norm, self.config.rms_eps)

    @torch.no_grad()
    def fill_context(self, sequence: int, first: int, last: int, seed: int = 0) -> None:
        """Synthetic context: cache rows ``first..last-1`` of one sequence get seeded random keys and values with
        the statistics of real ones (unit-variance rows), and the position moves to ``last``.  Decode speed depends
        on the length of the context, not on its content."""
        generator = torch.Generator(device=self.device).manual_seed(seed * 1000003 + sequence)
        shape = (self.config.layers, self.k_cache.shape[2], last - first, self.config.head_dim)
        self.k_cache[:, sequence, :, first:last] = torch.randn(shape, device=self.device, generator=generator).bfloat16()
        self.v_cache[:, sequence, :, first:last] = torch.randn(shape, device=self.device, generator=generator).bfloat16()
        self.pos[sequence] = last

    # -- decode --------------------------------------------------------------------------------------
    def _all_reduce(self, t: torch.Tensor) -> None:
        if self.world > 1:
            torch.distributed.all_reduce(t, group=self.group)

    def _pick_tokens(self, hidden: torch.Tensor) -> None:
        logits = (hidden @ self.lm_head.T).float()
        if not self.vocab_parallel:
            self.next_tok.copy_(logits.argmax(-1))
            return
        score, index = logits.max(-1)
        self.best_local[:, 0].copy_(score)
        self.best_local[:, 1].copy_(index + self.vocab_offset)             # token ids are exact in fp32 (< 2^24)
        torch.distributed.all_gather_into_tensor(self.best_all, self.best_local, group=self.group)
        winner = self.best_all[:, :, 0].argmax(0, keepdim=True)                                      # [1, B]
        self.next_tok.copy_(torch.gather(self.best_all[:, :, 1], 0, winner).reshape(-1).long())

    @torch.no_grad()
    def decode_step(self) -> None:
        """One token for every sequence, library kernels only (this is what ``capture`` records)."""
        c, ext = self.config, self.ext
        q_heads, kv_heads = c.q_heads // self.world, c.kv_heads // self.world
        torch.index_select(self.embed, 0, self.tok, out=self.buf_h)
        delta = None
        for layer in range(c.layers):
            ext.add_rmsnorm(self.buf_h, delta, self.norm1[layer], self.buf_x, c.rms_eps)
            ext.linear_out(self.h_qkv[layer], self.buf_x, self.buf_qkv)
            ext.attention_step_batch(self.buf_qkv, self.cos, self.sin, self.pos, self.k_cache[layer], self.v_cache[layer],
                                     self.attn_scratch, self.buf_attn, q_heads, kv_heads, c.head_dim)
            ext.linear_out(self.h_o[layer], self.buf_attn, self.buf_o)
            self._all_reduce(self.buf_o)
            ext.add_rmsnorm(self.buf_h, self.buf_o, self.norm2[layer], self.buf_x, c.rms_eps)
            ext.linear_out(self.h_gu[layer], self.buf_x, self.buf_gu)
            ext.silu_mul_pairs(self.buf_gu, self.buf_act)
            ext.linear_out(self.h_down[layer], self.buf_act, self.buf_down)
            self._all_reduce(self.buf_down)
            delta = self.buf_down
        ext.add_rmsnorm(self.buf_h, delta, self.final_norm, self.buf_x, c.rms_eps)
        self.last_hidden.copy_(self.buf_x)
        self._pick_tokens(self.buf_x)
        self.tok.copy_(self.next_tok)
        self.pos.add_(1)

    @torch.no_grad()
    def decode_step_reference(self, dense: bool = False) -> None:
        """The same step, sequence by sequence, through PyTorch glue (``dense``: and dense ``bf16(pal*scale)`` weights)."""
        c = self.config
        hidden = []
        for b in range(self.batch):
            position = self.pos[b:b + 1]
            cos, sin = self.cos.index_select(0, position), self.sin.index_select(0, position)
            k_all, v_all = self.k_cache, self.v_cache
            self.k_cache, self.v_cache = k_all[:, b], v_all[:, b]
            try:
                length = int(position) + 1

                def attend(layer, q):
                    k, v = self.k_cache[layer][:, :length].unsqueeze(0), self.v_cache[layer][:, :length].unsqueeze(0)
                    return F.scaled_dot_product_attention(q, k, v, enable_gqa=True)

                h = self.embed.index_select(0, self.tok[b:b + 1])
                for layer in range(c.layers):
                    h = self._layer(layer, h, cos, sin, position, attend, dense)
            finally:
                self.k_cache, self.v_cache = k_all, v_all
            hidden.append(_rmsnorm(h, self.final_norm, c.rms_eps))
        hidden = torch.cat(hidden)
        self.last_hidden.copy_(hidden)
        self._pick_tokens(hidden)
        self.tok.copy_(self.next_tok)
        self.pos.add_(1)

    @torch.no_grad()
    def capture(self) -> None:
        """Record ``decode_step`` in a CUDA graph (NCCL all-reduces included when tensor-parallel)."""
        stream = torch.cuda.Stream(self.device)
        saved = (self.tok.clone(), self.pos.clone())     # the warm-up steps write cache rows that the real steps rewrite
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            for _ in range(2):
                self.decode_step()
            self.tok.copy_(saved[0]); self.pos.copy_(saved[1])
            stream.synchronize()
            before = self.ext.launch_count()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                self.decode_step()
            self.launches_per_step = self.ext.launch_count() - before
            self.tok.copy_(saved[0]); self.pos.copy_(saved[1])
            stream.synchronize()
        torch.cuda.current_stream(self.device).wait_stream(stream)
        self.graph, self.stream = graph, stream

    def decode_graph(self) -> None:
        self.graph.replay()

