"""Tensor-parallel host logic on CPU: two gloo ranks, the CPU checker standing in for the kernels."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from tattletale_b200 import FMT_Q4_K, SHARD_COLUMN, SHARD_COLUMN_GATED, SHARD_ROW, tp

H, INTER, M = 512, 1024, 3


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make():
    rng = np.random.default_rng(77)
    gate_up = oracle.quantize(oracle.Q4_K, rng.normal(0, 0.02, (2 * INTER, H)).astype(np.float32))
    down = oracle.quantize(oracle.Q4_K, rng.normal(0, 0.02, (H, INTER)).astype(np.float32))
    x = oracle.to_bf16_bits(rng.normal(0, 1, (M, H)).astype(np.float32))
    return gate_up, down, x


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    gate_up, down, x = _make()
    # column-parallel gate|up (gated split keeps silu_and_mul local), then row-parallel down + all-reduce
    gu_l, n_l, _ = tp.shard_blocks(FMT_Q4_K, torch.from_numpy(gate_up), H, SHARD_COLUMN_GATED, rank, world)
    assert n_l == 2 * INTER // world
    act_l = oracle.silu_and_mul(oracle.linear(oracle.Q4_K, gu_l.numpy(), x, oracle.BF16))
    d_l, _, k_l = tp.shard_blocks(FMT_Q4_K, torch.from_numpy(down), INTER, SHARD_ROW, rank, world)
    assert k_l == INTER // world
    y = torch.from_numpy(oracle.linear(oracle.Q4_K, d_l.numpy(), act_l.astype(np.float32), oracle.F32))
    tp.all_reduce_sum(y)
    # plain column split: gathered slices are the full output
    c_l, _, _ = tp.shard_blocks(FMT_Q4_K, torch.from_numpy(down), INTER, SHARD_COLUMN, rank, world)
    full_act = oracle.silu_and_mul(oracle.linear(oracle.Q4_K, gate_up, x, oracle.BF16))
    yc = torch.from_numpy(oracle.linear(oracle.Q4_K, c_l.numpy(), full_act, oracle.F32))
    parts = [torch.empty_like(yc) for _ in range(world)]
    dist.all_gather(parts, yc)
    if rank == 0:
        want = oracle.linear(oracle.Q4_K, down, full_act, oracle.F32)
        out["row_err"] = float(np.abs(y.numpy() - want).max() / np.abs(want).max())
        out["col_equal"] = bool(np.array_equal(torch.cat(parts, dim=1).numpy(), want))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_mlp_matches_single_rank():
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
        assert out["col_equal"]
        assert out["row_err"] < 1e-5  # only the order of the fp32 partial sums differs


def test_shard_shapes_and_errors():
    blocks = torch.zeros((64, 1024 // 256 * 144), dtype=torch.uint8)
    b, n, k = tp.shard_blocks(FMT_Q4_K, blocks, 1024, SHARD_ROW, 1, 2)
    assert (tuple(b.shape), n, k) == ((64, 288), 64, 512)
    b, n, k = tp.shard_blocks(FMT_Q4_K, blocks, 1024, SHARD_COLUMN, 0, 4)
    assert (tuple(b.shape), n, k) == ((16, 576), 16, 1024)
    import pytest

    with pytest.raises(ValueError):
        tp.shard_blocks(FMT_Q4_K, blocks, 1024, SHARD_ROW, 0, 8)  # 128 weights per rank < one block
    with pytest.raises(ValueError):
        tp.shard_blocks(FMT_Q4_K, blocks, 1024, SHARD_COLUMN, 0, 3)
