"""Tensor-parallel sharding of BC4 linears across the GPUs of one node.

The reference is single-GPU (README.md:145-148).  Sharding an encoded matrix is byte slicing,
never a re-encode:

* column-parallel (q/k/v/gate/up): rank r keeps output rows ``[r*M/P, (r+1)*M/P)`` of the blocks
  and of the row scales;
* row-parallel (o/down): rank r keeps 16-column blocks ``[r*K/(16P), (r+1)*K/(16P))`` of every
  row together with the FULL row-scale vector (the scale belongs to the output row), and the
  ``[tokens, M]`` partial results are summed with an all-reduce.

One process per GPU; ``torch.distributed`` (NCCL over NVLink on the GPU box, gloo in CPU tests)
carries the all-reduce.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
from torch import nn

from .adapters import resolve_parent
from .runtime import PREFILL_THRESHOLD, PREFILL_TILE_ROWS, extension, free

COLUMN_PARALLEL_OPS = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")
ROW_PARALLEL_OPS = ("o_proj", "down_proj")


def shard_ranges(m: int, k: int, op: str, rank: int, world: int) -> tuple[tuple[int, int], tuple[int, int]]:
    """(row range, 16-column-block range) that ``rank`` owns for a linear of kind ``op``."""
    if not 0 <= rank < world:
        raise ValueError("rank outside the tensor-parallel group")
    blocks_per_row = k // 16
    if op in COLUMN_PARALLEL_OPS:
        if m % world:
            raise ValueError(f"M={m} is not divisible by the tensor-parallel size {world}")
        per = m // world
        return (rank * per, (rank + 1) * per), (0, blocks_per_row)
    if op in ROW_PARALLEL_OPS:
        if blocks_per_row % world:
            raise ValueError(f"K={k} has {blocks_per_row} BC4 blocks per row, not divisible by {world}")
        per = blocks_per_row // world
        return (0, m), (rank * per, (rank + 1) * per)
    raise ValueError(f"no tensor-parallel rule for linear {op!r}")


def shard_bytes(blocks: np.ndarray, scales: np.ndarray, m: int, k: int, op: str, rank: int, world: int):
    """Host-side slice of an encoded matrix: returns (blocks_u8, scales_f32) of the shard."""
    (r0, r1), (b0, b1) = shard_ranges(m, k, op, rank, world)
    raw = np.asarray(blocks, dtype=np.uint8).reshape(m, k // 16, 8)
    return np.ascontiguousarray(raw[r0:r1, b0:b1]).reshape(-1), np.ascontiguousarray(scales[r0:r1])


def pack_entry_shard(weights: Path, entry: dict, rank: int, world: int, bias: torch.Tensor | None = None,
                     lookahead: int = 1) -> int:
    """Pack this rank's shard of one ``metadata.json`` entry straight from the files."""
    m, k = int(entry["M"]), int(entry["K"])
    rows, kblocks = shard_ranges(m, k, entry["op"], rank, world)
    blocks = torch.from_numpy(np.fromfile(Path(weights) / entry["blocks_file"], dtype=np.uint8))
    scales = torch.from_numpy(np.fromfile(Path(weights) / entry["scales_file"], dtype="<f4").copy())
    ext = extension()
    # a row-parallel shard adds its bias on rank 0 only (the all-reduce would add it P times)
    use_bias = bias if (entry["op"] in COLUMN_PARALLEL_OPS or rank == 0) else None
    handle = ext.pack_encoded_shard(blocks, scales, m, k, rows, kblocks, use_bias)
    ext.set_lookahead(handle, lookahead)
    ext.set_prefill(handle, PREFILL_THRESHOLD, PREFILL_TILE_ROWS)
    return handle


class TensorParallelLinear(nn.Module):
    """A BC4 linear shard.  Column-parallel shards return their slice of the output; row-parallel
    shards take the matching slice of the input features and all-reduce the partial sums."""

    def __init__(self, handle: int, op: str, group=None):
        super().__init__()
        self.handle, self.op, self.group = handle, op, group
        self.row_parallel = op in ROW_PARALLEL_OPS

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = extension().linear(self.handle, x.contiguous())
        if self.row_parallel and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(y, group=self.group)
        return y


def install_tp(model: nn.Module, weights: Path, rank: int, world: int, group=None, lookahead: int = 1) -> list[int]:
    """Tensor-parallel counterpart of ``runtime.install``: replaces every listed linear with this
    rank's shard.  The surrounding model code must already split heads / intermediate features."""
    metadata = json.loads((Path(weights) / "metadata.json").read_text())
    handles: list[int] = []
    try:
        for entry in metadata["entries"]:
            parent, child = resolve_parent(model, entry["module_name"])
            original = getattr(parent, child)
            bias = original.bias if getattr(original, "bias", None) is not None else None
            handle = pack_entry_shard(weights, entry, rank, world, bias=bias, lookahead=lookahead)
            setattr(parent, child, TensorParallelLinear(handle, entry["op"], group))
            handles.append(handle)
    except Exception:
        free(handles)
        raise
    model._texelator_handles = handles
    return handles


class PeerExchange:
    """Peer-mapped buffers of the fused tensor-parallel exchanges, in symmetric memory
    (``torch.distributed._symmetric_memory``: plain peer mappings over NVLink, no multicast object is bound):

    * ``packet_inbox``: ``2 * world * hidden / 4`` 16-byte packets for ``tx_linear_single_push`` /
      ``tx_aux_peer_reduce_rmsnorm`` with the epoch word ``packet_epoch``;
    * ``token_inbox``: ``2 * world`` packets for ``tx_aux_peer_best_token`` with ``token_epoch``;
    * ``inbox`` / ``flags`` / ``epoch``: the first-generation layout of ``tx_aux_allreduce_add_rmsnorm``.

    ``*_ptrs`` are ctypes arrays with the address of every rank's buffer as seen from this rank.
    Construction is collective over ``group`` and raises when symmetric memory cannot be set up, in which
    case callers keep the NCCL all-reduce.
    """

    def __init__(self, hidden: int, device: torch.device, group=None):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("the fused all-reduce handles up to 8 ranks")
        with torch.cuda.device(device):
            self.inbox = symm_mem.empty(2 * self.world * hidden, dtype=torch.bfloat16, device=device)
            self.flags = symm_mem.empty(2 * self.world, dtype=torch.int32, device=device)
            self.packet_inbox = symm_mem.empty(2 * self.world * (hidden // 4) * 4, dtype=torch.int32, device=device)
            self.token_inbox = symm_mem.empty(2 * self.world * 4, dtype=torch.int32, device=device)
            self.inbox.zero_()
            self.flags.zero_()
            self.packet_inbox.zero_()
            self.token_inbox.zero_()
            inbox_handle = symm_mem.rendezvous(self.inbox, group)
            flag_handle = symm_mem.rendezvous(self.flags, group)
            packet_handle = symm_mem.rendezvous(self.packet_inbox, group)
            token_handle = symm_mem.rendezvous(self.token_inbox, group)
            self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
            self.packet_epoch = torch.zeros(1, dtype=torch.int32, device=device)
            self.token_epoch = torch.zeros(1, dtype=torch.int32, device=device)
            torch.cuda.synchronize(device)
        dist.barrier(group)            # every rank's zeroes are in place before anyone publishes a flag
        pointers = ctypes.c_void_p * self.world
        self.inbox_ptrs = pointers(*[int(p) for p in inbox_handle.buffer_ptrs])
        self.flag_ptrs = pointers(*[int(p) for p in flag_handle.buffer_ptrs])
        self.packet_ptrs = pointers(*[int(p) for p in packet_handle.buffer_ptrs])
        self.token_ptrs = pointers(*[int(p) for p in token_handle.buffer_ptrs])
        self._handles = (inbox_handle, flag_handle, packet_handle, token_handle)     # keep the mappings alive
