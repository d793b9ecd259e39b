"""Tensor-parallel path with two CPU ranks over gloo: every rank slices the encoded bytes with
``tp.shard_bytes``, evaluates its shard with the oracle, and the row-parallel partials are summed
with an all-reduce -- the exchange the GPU path performs over NCCL."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import bc4_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, golden, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from texelator_b200 import tp
    lut = O.software_palette()
    z = np.load(golden)
    m, k = z["scales"].shape[0], z["weight"].shape[1]
    x = z["x_bf16"].astype(np.float64)
    # row-parallel (down/o): this rank's K slice, full scales, partial sums all-reduced
    blocks, scales = tp.shard_bytes(z["blocks"], z["scales"], m, k, "down_proj", rank, world)
    (_, _), (b0, b1) = tp.shard_ranges(m, k, "down_proj", rank, world)
    w = O.dequant_weights(blocks, scales, lut).astype(np.float64)
    partial = torch.from_numpy(x[:, b0 * 16:b1 * 16] @ w.T)
    dist.all_reduce(partial)
    # column-parallel (gate/up): this rank's rows, gathered
    blocks_c, scales_c = tp.shard_bytes(z["blocks"], z["scales"], m, k, "up_proj", rank, world)
    mine = torch.from_numpy(x @ O.dequant_weights(blocks_c, scales_c, lut).astype(np.float64).T)
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    if rank == 0:
        np.savez(out, row=partial.numpy(), col=torch.cat(parts, 1).numpy())
    dist.destroy_process_group()


def test_two_rank_tensor_parallel_linear(tmp_path, golden_dir, lut):
    golden = str(golden_dir / "small_48x256.npz")
    out = str(tmp_path / "tp.npz")
    mp.spawn(_worker, args=(2, _free_port(), golden, out), nprocs=2, join=True)
    z = np.load(golden)
    full = z["x_bf16"].astype(np.float64) @ O.dequant_weights(z["blocks"], z["scales"], lut).astype(np.float64).T
    got = np.load(out)
    assert np.allclose(got["row"], full, rtol=0, atol=1e-9)     # only the summation order differs
    assert np.array_equal(got["col"], full)
