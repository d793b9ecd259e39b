"""Dense decoder harness around the BC4 linear operator.

The reference drives Hugging Face models (``texelator/modeling.py:9-31`` loads them,
``texelator/cli.py:189-219`` calls ``generate``) and replaces their seven projection
linears per layer.  Checkpoints are not available here, so this module builds the
same architecture family (Qwen2/Llama-style: RMSNorm, RoPE, grouped-query attention,
SwiGLU) from a config with random-init weights, BC4-encodes the projections, and
runs a CUDA-graphed batch-1 decode loop so that tokens/s reflects the operator and
not Python.  q/k/v and gate/up are packed as one BC4 matrix each (rows concatenated;
row scales are per row, so fusing changes no value).

Tensor parallelism (new; the reference is single-GPU, README.md:145-148): q/k/v and
gate/up are split by output rows, o and down by 16-column blocks with the full row
scale vector, followed by an all-reduce over ``torch.distributed`` (NCCL).

``input_device`` keeps the reference's helper (modeling.py:26-31).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import runtime


@dataclass(frozen=True)
class DecoderConfig:
    name: str
    hidden: int
    layers: int
    q_heads: int
    kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    rope_theta: float = 1e6
    rms_eps: float = 1e-6
    qkv_bias: bool = False

    @property
    def q_rows(self) -> int:
        return self.q_heads * self.head_dim

    @property
    def kv_rows(self) -> int:
        return self.kv_heads * self.head_dim

    def bc4_bytes_per_token(self) -> int:
        """BC4 blocks + fp32 row scales read per decoded token (all seven projections)."""
        h, i = self.hidden, self.intermediate
        shapes = [(self.q_rows, h), (self.kv_rows, h), (self.kv_rows, h), (h, self.q_rows), (i, h), (i, h), (h, i)]
        return self.layers * sum(m * k // 2 + 4 * m for m, k in shapes)


CONFIGS = {
    # BASELINE.json configs[1], [3], [4] and a toy model for tests
    "qwen2.5-3b-shaped": DecoderConfig("qwen2.5-3b-shaped", 2048, 36, 16, 2, 128, 11008, 151936, qkv_bias=True),
    "27b-class": DecoderConfig("27b-class", 5120, 64, 40, 8, 128, 17408, 151936),
    "70b-class": DecoderConfig("70b-class", 8192, 80, 64, 8, 128, 28672, 128256, rope_theta=5e5),
    "toy": DecoderConfig("toy", 256, 2, 4, 2, 64, 512, 1024, qkv_bias=True),
    "toy128": DecoderConfig("toy128", 512, 3, 8, 2, 128, 1024, 2048, qkv_bias=True),
    "toy128x8": DecoderConfig("toy128x8", 1024, 2, 16, 8, 128, 2048, 4096, qkv_bias=True),      # splits 8 ways
}


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Rows of a fused gate/up projection in the pair order of ``tx_linear_fused``'s SwiGLU: every group of
    16 rows holds 8 gate rows followed by the 8 up rows of the same output columns."""
    rows = gate.shape[0]
    if rows % 8 or up.shape != gate.shape:
        raise ValueError("gate and up must have the same shape with a multiple of 8 rows")
    return torch.stack([gate.reshape(rows // 8, 8, -1), up.reshape(rows // 8, 8, -1)], 1).reshape(2 * rows, -1)


def input_device(model) -> torch.device:
    embedding = model.get_input_embeddings()
    device = getattr(embedding, "output_device", embedding.weight.device)
    if device.type == "meta":
        raise RuntimeError("input embedding remains on a meta device")
    return device


# ---------------------------------------------------------------------------
# GPU-side min/max BC4 encoder for synthetic weights (the initialisation step of
# texelator/encoder.py:46-51 without the endpoint search; throughput inputs only).
# ---------------------------------------------------------------------------

def software_palette_table(device) -> torch.Tensor:
    """``[255, 255, 8]`` fp32 software BC4-SNORM palette, ``lut[e1+127, e0+127, s]``."""
    e = torch.arange(-127, 128, device=device, dtype=torch.int32)
    e0, e1 = e[None, :, None], e[:, None, None]
    g8 = torch.tensor([0, 7, 1, 2, 3, 4, 5, 6], device=device, dtype=torch.int32)[None, None, :]
    g6 = torch.tensor([0, 5, 1, 2, 3, 4, 0, 0], device=device, dtype=torch.int32)[None, None, :]
    p8 = ((7 - g8) * e0 + g8 * e1).float() / 889.0
    p6 = ((5 - g6) * e0 + g6 * e1).float() / 635.0
    p6[:, :, 6] = -1.0
    p6[:, :, 7] = 1.0
    return torch.where(e0 > e1, p8, p6).contiguous()


@torch.no_grad()
def encode_minmax_cuda(weight: torch.Tensor, lut: torch.Tensor, rows_per_chunk: int = 2048):
    """BC4-encode a CUDA fp32/bf16 ``[M, K]`` matrix; returns (blocks uint8 ``[M*K/2]``, scales fp32 ``[M]``)."""
    m, k = weight.shape
    blocks = torch.empty((m, k // 16, 8), dtype=torch.uint8, device=weight.device)
    scales = torch.empty(m, dtype=torch.float32, device=weight.device)
    shifts = (3 * torch.arange(16, device=weight.device, dtype=torch.int64))[None, :]
    for start in range(0, m, rows_per_chunk):
        rows = weight[start:start + rows_per_chunk].float()
        sc = rows.abs().amax(1).clamp_min(1e-12)
        v = (rows / sc[:, None]).clamp(-1, 1).reshape(-1, 16)
        e0 = torch.round(v.max(1).values * 127).clamp(-127, 127).long()
        e1 = torch.round(v.min(1).values * 127).clamp(-127, 127).long()
        pal = lut[e1 + 127, e0 + 127]                                  # [n, 8]
        sel = (v[:, :, None] - pal[:, None, :]).abs().argmin(2)        # [n, 16]
        word = (sel << shifts).sum(1)                                   # 48-bit selector word
        out = blocks[start:start + rows_per_chunk].reshape(-1, 8)
        out[:, 0] = (e0 & 255).to(torch.uint8)
        out[:, 1] = (e1 & 255).to(torch.uint8)
        for byte in range(6):
            out[:, 2 + byte] = ((word >> (8 * byte)) & 255).to(torch.uint8)
        scales[start:start + rows_per_chunk] = sc
    return blocks.reshape(-1), scales


def _rope_tables(config: DecoderConfig, max_len: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    half = config.head_dim // 2
    inv = 1.0 / (config.rope_theta ** (torch.arange(0, half, device=device, dtype=torch.float32) / half))
    ang = torch.arange(max_len, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


def _apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x ``[T, heads, d]``; cos/sin ``[T, d/2]`` (rotate-half convention of Qwen2/Llama)."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half].float(), x[..., half:].float()
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def _rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)


class BC4Decoder:
    """Random-init dense decoder whose projections are BC4 handles.

    ``tp_world > 1`` builds this rank's shard of every projection (see module docstring) and
    all-reduces after o/down over ``group``.  ``keep_dense`` also keeps ``bf16(pal*scale)``
    copies of every projection (from ``ext.dequant``) so that ``forward(..., dense=True)`` runs
    the same model through ``torch.matmul`` -- the dequantise-then-matmul comparison.
    """

    def __init__(self, config: DecoderConfig, device, max_len: int, seed: int = 0, tp_rank: int = 0,
                 tp_world: int = 1, group=None, lookahead: int = 3, keep_dense: bool = False,
                 weight_std: float = 0.02, prefill_backend: int = 5, encoder: str = "minmax"):
        self.config, self.device, self.max_len = config, torch.device(device), max_len
        self.rank, self.world, self.group = tp_rank, tp_world, group
        if encoder not in ("minmax", "e3"):
            raise ValueError("encoder must be 'minmax' (endpoints at the block's extremes) or 'e3' (the reference's endpoint search)")
        self.encoder = encoder
        self.ext = runtime.extension()
        c = config
        if c.q_heads % tp_world or c.kv_heads % tp_world or (c.intermediate // 16) % tp_world or (c.q_rows // 16) % tp_world:
            raise ValueError(f"{c.name} cannot be split {tp_world}-way (heads and 16-column blocks must divide)")
        self.q_loc, self.kv_loc, self.i_loc = c.q_rows // tp_world, c.kv_rows // tp_world, c.intermediate // tp_world
        gen = torch.Generator(device=self.device).manual_seed(seed)
        lut = software_palette_table(self.device)
        self.handles: list[int] = []
        self.h_qkv, self.h_o, self.h_gu, self.h_down = [], [], [], []
        self.dense = [] if keep_dense else None
        self.norm1, self.norm2 = [], []

        def randn(rows, cols):
            return torch.randn(rows, cols, device=self.device, generator=gen) * weight_std

        def rows_of(mat, per):          # this rank's slice of the output rows
            return mat[tp_rank * per:(tp_rank + 1) * per]

        with torch.cuda.device(self.device):
            for _ in range(c.layers):
                wq, wk, wv = randn(c.q_rows, c.hidden), randn(c.kv_rows, c.hidden), randn(c.kv_rows, c.hidden)
                wqkv = torch.cat([rows_of(wq, self.q_loc), rows_of(wk, self.kv_loc), rows_of(wv, self.kv_loc)])
                del wq, wk, wv
                bias = None
                if c.qkv_bias:
                    # drawn for the whole projection and then sliced, so every rank of a tensor-parallel
                    # model sees the weights of the one-GPU model made from the same seed
                    whole = (torch.randn(c.q_rows + 2 * c.kv_rows, device=self.device, generator=gen) * 0.02).bfloat16()
                    bq, bk, bv = whole[:c.q_rows], whole[c.q_rows:c.q_rows + c.kv_rows], whole[c.q_rows + c.kv_rows:]
                    bias = torch.cat([rows_of(bq, self.q_loc), rows_of(bk, self.kv_loc), rows_of(bv, self.kv_loc)]).contiguous()
                self.h_qkv.append(self._pack_rows(wqkv, lut, bias))
                del wqkv
                self.h_o.append(self._pack_columns(randn(c.hidden, c.q_rows), lut))
                wg, wu = randn(c.intermediate, c.hidden), randn(c.intermediate, c.hidden)
                wgu = interleave_gate_up(rows_of(wg, self.i_loc), rows_of(wu, self.i_loc))
                del wg, wu
                self.h_gu.append(self._pack_rows(wgu, lut, None))
                del wgu
                self.h_down.append(self._pack_columns(randn(c.hidden, c.intermediate), lut))
                self.norm1.append((1 + 0.1 * torch.randn(c.hidden, device=self.device, generator=gen)).bfloat16())
                self.norm2.append((1 + 0.1 * torch.randn(c.hidden, device=self.device, generator=gen)).bfloat16())
            self.final_norm = torch.ones(c.hidden, device=self.device, dtype=torch.bfloat16)
            self.embed = (torch.randn(c.vocab, c.hidden, device=self.device, generator=gen) * 0.02).bfloat16()
            lm_head = (torch.randn(c.vocab, c.hidden, device=self.device, generator=gen) * 0.02).bfloat16()
            # vocabulary-parallel output head: each rank scores its slice of the vocabulary and the ranks
            # exchange one (score, token) pair per step instead of every rank reading all 1.5 GB
            self.vocab_parallel = tp_world > 1 and c.vocab % tp_world == 0
            if self.vocab_parallel:
                per = c.vocab // tp_world
                self.vocab_offset = tp_rank * per
                self.lm_head = lm_head[self.vocab_offset:self.vocab_offset + per].clone()
                self.best_local = torch.zeros(2, dtype=torch.float32, device=self.device)
                self.best_all = torch.zeros(tp_world, 2, dtype=torch.float32, device=self.device)
            else:
                self.lm_head = lm_head
            del lm_head
            for h in self.handles:
                self.ext.set_lookahead(h, lookahead)
                self.ext.set_prefill_backend(h, prefill_backend)
            self.cos, self.sin = _rope_tables(c, max_len, self.device)
            kv_heads = c.kv_heads // tp_world
            self.k_cache = torch.zeros(c.layers, kv_heads, max_len, c.head_dim, device=self.device, dtype=torch.bfloat16)
            self.v_cache = torch.zeros_like(self.k_cache)
            # static decode state (CUDA graph)
            self.tok = torch.zeros(1, dtype=torch.int64, device=self.device)
            self.pos = torch.zeros(1, dtype=torch.int64, device=self.device)
            self.mask = torch.zeros(1, 1, 1, max_len, dtype=torch.bool, device=self.device)
            self.next_tok = torch.zeros(1, dtype=torch.int64, device=self.device)
            self.last_hidden = torch.zeros(1, c.hidden, dtype=torch.bfloat16, device=self.device)
            # static buffers of the fused decode step
            q_heads = c.q_heads // tp_world
            bf = dict(dtype=torch.bfloat16, device=self.device)
            self.buf_h = torch.zeros(1, c.hidden, **bf)
            self.buf_h2 = torch.zeros(1, c.hidden, **bf)
            self.buf_x = torch.zeros(1, c.hidden, **bf)
            self.buf_qkv = torch.zeros(1, self.q_loc + 2 * self.kv_loc, **bf)
            self.buf_attn = torch.zeros(1, self.q_loc, **bf)
            self.buf_o = torch.zeros(1, c.hidden, **bf)
            self.buf_gu = torch.zeros(1, 2 * self.i_loc, **bf)
            self.buf_act = torch.zeros(1, self.i_loc, **bf)
            self.buf_down = torch.zeros(1, c.hidden, **bf)
            self.attn_scratch = torch.zeros(max(q_heads * ((max_len + 127) // 128) * (c.head_dim + 2),
                                                self.ext.attention_step_scratch_floats(q_heads, max_len)),
                                            dtype=torch.float32, device=self.device)
            self.fused = c.head_dim == 128 and (c.q_heads // c.kv_heads) <= 8 and c.hidden <= 18432 and self.i_loc % 8 == 0
            # single-token decode path (tx_linear_single): the norm kernels hand the qkv and gate/up linears their
            # token in staged form, the o and down linears leave K-split fp32 partial sums that the next norm adds
            info = [self.ext.linear_single_info(h) for h in self.handles]
            self.single = self.fused and c.hidden <= 16384 and c.hidden % 128 == 0 and all(i[0] for i in info)
            self.k_split = False
            if self.single:
                self.split_o = self.ext.linear_single_info(self.h_o[0])[1]
                self.split_down = self.ext.linear_single_info(self.h_down[0])[1]
                stride = (c.hidden + 31) // 32 * 32
                self.part_o = torch.zeros(self.split_o, stride, dtype=torch.float32, device=self.device)
                self.part_down = torch.zeros(self.split_down, stride, dtype=torch.float32, device=self.device)
                self.staged_h = torch.zeros(self.ext.linear_single_info(self.h_qkv[0])[2], dtype=torch.uint8, device=self.device)
        # tensor parallelism: the all-reduce of the o/down partials fused into the next residual add + norm
        # over peer memory (tp.PeerExchange); None keeps the NCCL all-reduce
        self.peers = None
        # residual add + RMSNorm inside the qkv and gate/up linears instead of separate launches: every CTA
        # of the linear then repeats the norm, which measured slower than the two small kernels on a B200
        self.fuse_norm = False
        self.graph = None
        self.launches_per_step = 0

    # -- packing ---------------------------------------------------------------
    def _register(self, handle, bias=None):
        self.handles.append(handle)
        if self.dense is not None:
            self.dense.append((handle, self.ext.dequant(handle, runtime.DEQUANT_SCALED_BF16), bias))
        return handle

    def _encode(self, weight, lut):
        """BC4 blocks and row scales of one projection: ``minmax`` is the start of the reference's encoder
        (texelator/encoder.py:46-51) written with torch ops; ``e3`` its whole activation-weighted endpoint search
        (:34-102) on the GPU (``tx_encode``), weighted by the second moments of 64 seeded N(0,1) calibration rows
        (drawn per K from a generator of their own, so every rank of a tensor-parallel model uses the same)."""
        if self.encoder == "minmax":
            return encode_minmax_cuda(weight, lut)
        k = weight.shape[1]
        calibration = torch.randn(64, k, device=self.device, generator=torch.Generator(device=self.device).manual_seed(1000003 + k))
        return self.ext.encode(weight.float().contiguous(), (calibration * calibration).mean(0), lut)

    def _pack_rows(self, weight, lut, bias):
        blocks, scales = self._encode(weight, lut)
        return self._register(self.ext.pack_encoded_device(blocks, scales, bias), bias)

    def _pack_columns(self, weight, lut):
        """Row-parallel shard: encode the full matrix (row scales come from full rows), keep this
        rank's 16-column blocks of every row."""
        blocks, scales = self._encode(weight, lut)
        if self.world > 1:
            m, k = weight.shape
            per = (k // 16) // self.world
            blocks = blocks.reshape(m, k // 16, 8)[:, self.rank * per:(self.rank + 1) * per].contiguous().reshape(-1)
        return self._register(self.ext.pack_encoded_device(blocks, scales, None))

    # -- forward -----------------------------------------------------------------
    def _linear(self, handle, x, dense):
        if not dense:
            return self.ext.linear(handle, x)
        _, w, bias = next(item for item in self.dense if item[0] == handle)
        # dense=True: fp32 GEMM on the same bf16(pal*scale) matrix; dense="bf16": the library's bf16 GEMM (fp32
        # accumulation in another order), which shows how far rounding alone moves a model's output
        y = (x @ w.T).float() if dense == "bf16" else x.float() @ w.float().T
        return (y + bias.float() if bias is not None else y).to(x.dtype)

    def _reduce(self, t):
        if self.world > 1:
            torch.distributed.all_reduce(t, group=self.group)
        return t

    def _layer(self, layer, h, cos, sin, write_index, attend, dense=False):
        c = self.config
        tokens = h.shape[0]
        x = _rmsnorm(h, self.norm1[layer], c.rms_eps)
        qkv = self._linear(self.h_qkv[layer], x, dense)
        q = qkv[:, :self.q_loc].reshape(tokens, -1, c.head_dim)
        k = qkv[:, self.q_loc:self.q_loc + self.kv_loc].reshape(tokens, -1, c.head_dim)
        v = qkv[:, self.q_loc + self.kv_loc:].reshape(tokens, -1, c.head_dim)
        q, k = _apply_rope(q, cos, sin), _apply_rope(k, cos, sin)
        self.k_cache[layer].index_copy_(1, write_index, k.transpose(0, 1))
        self.v_cache[layer].index_copy_(1, write_index, v.transpose(0, 1))
        out = attend(layer, q.transpose(0, 1).unsqueeze(0))                     # [1, Hq, T, d]
        out = out.squeeze(0).transpose(0, 1).reshape(tokens, self.q_loc).contiguous()
        h = h + self._reduce(self._linear(self.h_o[layer], out, dense))
        x = _rmsnorm(h, self.norm2[layer], c.rms_eps)
        gu = self._linear(self.h_gu[layer], x, dense).view(tokens, self.i_loc // 8, 2, 8)     # (gate, up) row pairs
        act = (F.silu(gu[:, :, 0].float()) * gu[:, :, 1].float()).to(h.dtype).reshape(tokens, self.i_loc)
        return h + self._reduce(self._linear(self.h_down[layer], act, dense))

    @torch.no_grad()
    def prefill(self, ids: torch.Tensor, dense: bool = False) -> torch.Tensor:
        """Run a prompt from position 0, fill the KV cache, return the final hidden states ``[T, hidden]``."""
        tokens = ids.numel()
        index = torch.arange(tokens, device=self.device)
        cos, sin = self.cos[:tokens], self.sin[:tokens]

        def attend(layer, q):
            k = self.k_cache[layer][:, :tokens].unsqueeze(0)
            v = self.v_cache[layer][:, :tokens].unsqueeze(0)
            return F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)

        h = self.embed.index_select(0, ids.to(self.device).reshape(-1))
        for layer in range(self.config.layers):
            h = self._layer(layer, h, cos, sin, index, attend, dense)
        h = _rmsnorm(h, self.final_norm, self.config.rms_eps)
        self.pos.fill_(tokens)
        self.mask.zero_()
        self.mask[..., :tokens] = True
        return h

    def _decode_step(self, dense: bool = False):
        cos, sin = self.cos.index_select(0, self.pos), self.sin.index_select(0, self.pos)
        self.mask.index_fill_(3, self.pos, True)

        def attend(layer, q):
            return F.scaled_dot_product_attention(q, self.k_cache[layer].unsqueeze(0), self.v_cache[layer].unsqueeze(0),
                                                  attn_mask=self.mask, enable_gqa=True)

        h = self.embed.index_select(0, self.tok)
        for layer in range(self.config.layers):
            h = self._layer(layer, h, cos, sin, self.pos, attend, dense)
        h = _rmsnorm(h, self.final_norm, self.config.rms_eps)
        self.last_hidden.copy_(h)
        self._pick_token(h)
        self.tok.copy_(self.next_tok)
        self.pos.add_(1)

    def _pick_token(self, hidden):
        """Greedy next token from the final hidden state (bf16 output head, fp32 argmax)."""
        logits = (hidden @ self.lm_head.T).float()
        if not self.vocab_parallel:
            self.next_tok.copy_(logits.argmax(-1))
            return
        score, index = logits.max(-1)
        if self.peers is not None and self.single:
            self.ext.peer_best_token(score.contiguous(), index.contiguous(), self.vocab_offset, self.peers, self.next_tok)
            return
        self.best_local[0:1].copy_(score)
        self.best_local[1:2].copy_(index + self.vocab_offset)          # token ids are exact in fp32 (< 2^24)
        torch.distributed.all_gather_into_tensor(self.best_all, self.best_local, group=self.group)
        winner = self.best_all[:, 0].argmax().reshape(1)
        self.next_tok.copy_(torch.index_select(self.best_all[:, 1], 0, winner).long())   # no host round trip

    def _add_norm(self, residual, delta, weight):
        """residual += delta (all-reduced first when it is a tensor-parallel partial); buf_x = rmsnorm(residual) * weight."""
        if delta is not None and self.peers is not None and not self.fuse_norm:
            self.ext.allreduce_add_rmsnorm(residual, delta, weight, self.buf_x, self.config.rms_eps, self.peers)
        else:
            self.ext.add_rmsnorm(residual, delta, weight, self.buf_x, self.config.rms_eps)

    def enable_peer_exchange(self) -> bool:
        """Switch the fused decode step of a tensor-parallel model from NCCL all-reduces to the all-reduce
        fused into the norm kernel (collective call).  Returns False, keeping NCCL, when symmetric memory
        cannot be set up on this system."""
        if self.world == 1:
            return False
        from .tp import PeerExchange
        try:
            self.peers = PeerExchange(self.config.hidden, self.device, self.group)
        except Exception as error:  # noqa: BLE001 - any set-up failure means "keep NCCL"
            print(f"[texelator_b200] peer exchange unavailable, keeping NCCL all-reduce: {error}", flush=True)
            self.peers = None
        # all ranks must agree, or the call sequences diverge
        flag = torch.tensor([1 if self.peers is not None else 0], device=self.device)
        torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 0:
            self.peers = None
        return self.peers is not None

    def _decode_step_single(self):
        """One decode step on the single-token path, eight launches per layer (the attention step is two: splits, merge).  The norm kernels write their
        output in the staged form of ``tx_linear_single`` (the qkv and gate/up linears then copy 11 KB instead
        of each CTA scanning and converting the row).  On one GPU the o and down linears, whose inputs come
        from many CTAs, stage for themselves in the general decode kernel (``self.k_split`` lets them leave
        K-split fp32 partial sums for the next norm instead).  Tensor-parallel, they push their partial rows
        into every rank's packet inbox from their epilogue and the next norm (one thread-block cluster) polls
        and adds the packets of all ranks; the output head exchanges one (score, token) packet per rank."""
        c, ext = self.config, self.ext
        q_heads, kv_heads = c.q_heads // self.world, c.kv_heads // self.world
        peers = self.peers if self.world > 1 else None
        torch.index_select(self.embed, 0, self.tok, out=self.buf_h)

        def norm(weight, pending, **outputs):
            if peers is not None:
                ext.peer_reduce_rmsnorm(self.buf_h, weight, c.rms_eps, peers=peers if pending else None, **outputs)
            else:
                ext.add_rmsnorm_single(self.buf_h, weight, c.rms_eps, **pending, **outputs)

        def row_parallel(handle, x, out, partials):
            if peers is not None:
                ext.linear_single_push(handle, x, peers)
                return dict(pushed=True)
            if self.k_split:
                ext.linear_single(handle, x, None, partials=partials)
                return dict(partials=partials)
            ext.linear_out(handle, x, out)
            return dict(delta=out)

        pending = {}
        for layer in range(c.layers):
            norm(self.norm1[layer], pending, staged=self.staged_h)
            ext.linear_single(self.h_qkv[layer], None, self.buf_qkv, staged=self.staged_h)
            ext.attention_step(self.buf_qkv, self.cos, self.sin, self.pos, self.k_cache[layer], self.v_cache[layer],
                               self.attn_scratch, self.buf_attn, q_heads, kv_heads, c.head_dim)
            pending = row_parallel(self.h_o[layer], self.buf_attn, self.buf_o, self.part_o)
            norm(self.norm2[layer], pending, staged=self.staged_h)
            ext.linear_single(self.h_gu[layer], None, self.buf_act, staged=self.staged_h, swiglu=True)
            pending = row_parallel(self.h_down[layer], self.buf_act, self.buf_down, self.part_down)
        norm(self.final_norm, pending, y=self.buf_x)
        self.last_hidden.copy_(self.buf_x)
        self._pick_token(self.buf_x)
        self.tok.copy_(self.next_tok)
        self.mask.index_fill_(3, self.pos, True)
        self.pos.add_(1)

    def _decode_step_fused(self):
        """One decode step with the library's fused kernels, six launches per layer with ``fuse_norm`` (eight without): qkv linear (with the
        residual add and RMSNorm in its activation staging), attention step (RoPE, cache append, attention,
        split merge), o linear, gate/up linear (add + norm in front, SwiGLU behind), down linear."""
        c, ext = self.config, self.ext
        q_heads, kv_heads = c.q_heads // self.world, c.kv_heads // self.world
        torch.index_select(self.embed, 0, self.tok, out=self.buf_h)
        residual, spare = self.buf_h, self.buf_h2       # the fused linears write x + delta to the other buffer
        delta = None
        for layer in range(c.layers):
            if not self.fuse_norm:
                self._add_norm(residual, delta, self.norm1[layer])
                ext.linear_out(self.h_qkv[layer], self.buf_x, self.buf_qkv)
            elif delta is None:
                ext.linear_fused_out(self.h_qkv[layer], residual, self.buf_qkv, norm_weight=self.norm1[layer], eps=c.rms_eps)
            else:
                ext.linear_fused_out(self.h_qkv[layer], residual, self.buf_qkv, norm_weight=self.norm1[layer], delta=delta,
                                     eps=c.rms_eps, residual_out=spare)
                residual, spare = spare, residual
            ext.attention_step(self.buf_qkv, self.cos, self.sin, self.pos, self.k_cache[layer], self.v_cache[layer],
                               self.attn_scratch, self.buf_attn, q_heads, kv_heads, c.head_dim)
            ext.linear_out(self.h_o[layer], self.buf_attn, self.buf_o)
            if self.fuse_norm or self.peers is None:
                self._reduce(self.buf_o)
            if self.fuse_norm:
                ext.linear_fused_out(self.h_gu[layer], residual, self.buf_act, norm_weight=self.norm2[layer], delta=self.buf_o,
                                     eps=c.rms_eps, residual_out=spare, swiglu=True)
                residual, spare = spare, residual
            else:
                self._add_norm(residual, self.buf_o, self.norm2[layer])
                ext.linear_fused_out(self.h_gu[layer], self.buf_x, self.buf_act, swiglu=True)
            ext.linear_out(self.h_down[layer], self.buf_act, self.buf_down)
            if self.fuse_norm or self.peers is None:
                self._reduce(self.buf_down)
            delta = self.buf_down
        if residual is not self.buf_h:
            self.buf_h.copy_(residual)
        self._add_norm(self.buf_h, delta, self.final_norm)
        self.last_hidden.copy_(self.buf_x)
        self._pick_token(self.buf_x)
        self.tok.copy_(self.next_tok)
        self.mask.index_fill_(3, self.pos, True)
        self.pos.add_(1)

    def prefer_single(self) -> bool:
        """Which fused step a captured graph runs.  On one GPU the general decode kernel wins end to end
        (measured on the 27B-class shapes: 194 tok/s against 186 with staged activations), so the
        single-token path is the default only where it is needed: tensor-parallel runs whose row-parallel
        linears push their partial rows to the peers from their epilogue."""
        return self.world > 1 and self.peers is not None

    @torch.no_grad()
    def decode_eager(self, dense: bool = False, fused: bool = False, single: bool = False) -> None:
        if single:
            self._decode_step_single()
        elif fused:
            self._decode_step_fused()
        else:
            self._decode_step(dense)

    @torch.no_grad()
    def capture(self, fused: bool | None = None) -> None:
        """Capture one decode step (all layers, lm_head, argmax, position update) in a CUDA graph.
        ``fused`` (default: when the shapes allow) uses the library's glue kernels instead of PyTorch ops."""
        use_fused = self.fused if fused is None else fused
        step = self._decode_step if not use_fused else (self._decode_step_single if self.single and fused is None and not self.fuse_norm and self.prefer_single() else self._decode_step_fused)
        stream = torch.cuda.Stream(self.device)
        saved = (self.tok.clone(), self.pos.clone(), self.mask.clone())
        # the capture stream is non-blocking: everything queued so far (the prompt's cache writes, the clones
        # above) has to be ordered before the first warm-up step on it
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            for _ in range(2):
                step()
            self.tok.copy_(saved[0]); self.pos.copy_(saved[1]); self.mask.copy_(saved[2])
            stream.synchronize()
            before = self.ext.launch_count()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=stream):
                step()
            self.launches_per_step = self.ext.launch_count() - before
            self.tok.copy_(saved[0]); self.pos.copy_(saved[1]); self.mask.copy_(saved[2])
            stream.synchronize()
        torch.cuda.current_stream(self.device).wait_stream(stream)
        self.stream = stream

    def decode_graph(self) -> None:
        self.graph.replay()

    def check_status(self) -> None:
        """Raise if any kernel of this rank gave up on a bounded wait (a peer that never delivered, a pipeline
        barrier that never completed): whatever was decoded since the last check cannot be trusted then.
        Synchronises the device; call it at host synchronisation points (every few tokens, or when a
        sequence ends), not per launch."""
        code = self.ext.kernel_status(clear=True, device=self.device.index)
        if code:
            raise RuntimeError(f"a device-side bounded wait ran out (status {code}); the tokens decoded since the last check are invalid")

    def decode_tokens(self, count: int, check_every: int = 16) -> list[int]:
        """Replay the captured step ``count`` times; the device status word is checked every ``check_every``
        tokens and at the end."""
        tokens = []
        for index in range(count):
            self.graph.replay()
            if (index + 1) % check_every == 0 or index + 1 == count:
                self.stream.synchronize()
                self.check_status()
            tokens.append(self.next_tok.clone())
        return [int(t) for t in torch.cat(tokens).tolist()]

    def free(self) -> None:
        runtime.free(self.handles)
        self.handles = []
