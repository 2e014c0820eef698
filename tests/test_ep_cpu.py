"""Expert-parallel dispatch / combine on CPU: two and three gloo ranks, the CPU checker standing in for the
grouped GEMM of each rank.  The gathered result must equal the single-process checker on all tokens."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from tattletale_b200 import tp

H, INTER, E, TOPK, T = 256, 256, 6, 2, 20


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make():
    rng = np.random.default_rng(123)
    gu = [oracle.quantize(oracle.Q4_K, rng.normal(0, 0.05, (2 * INTER, H)).astype(np.float32)) for _ in range(E)]
    dn = [oracle.quantize(oracle.Q4_K, rng.normal(0, 0.05, (H, INTER)).astype(np.float32)) for _ in range(E)]
    x = torch.from_numpy(rng.normal(0, 1, (T, H)).astype(np.float32)).to(torch.bfloat16)
    logits = rng.normal(0, 1, (T, E))
    ids = np.argsort(-logits, axis=1)[:, :TOPK].astype(np.int32)
    w = rng.uniform(0.1, 1.0, (T, TOPK)).astype(np.float32)
    ids[3, 1] = -1  # a dropped choice
    return gu, dn, x, ids, w


def _bits(x):
    return x.contiguous().view(torch.int16).numpy().view(np.uint16)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    gu, dn, x, ids, w = _make()
    epr = E // world
    lo = rank * epr

    def local_forward(rows, local_ids):
        lid = local_ids.numpy().reshape(-1, 1)
        y = oracle.moe(oracle.Q4_K, gu[lo:lo + epr], dn[lo:lo + epr], _bits(rows), oracle.BF16, lid,
                       np.ones_like(lid, dtype=np.float32))
        return torch.from_numpy(y).to(torch.bfloat16)

    layer = tp.ExpertParallelMoE(local_forward, epr, 1)
    # uneven token slices: rank r takes tokens r, r + world, ...
    mine = np.arange(rank, T, world)
    y = layer.forward(x[mine], torch.from_numpy(ids[mine]), torch.from_numpy(w[mine]))
    parts = [None] * world
    dist.all_gather_object(parts, (mine, y.float().numpy()))
    if rank == 0:
        got = np.zeros((T, H), dtype=np.float32)
        for idx, val in parts:
            got[idx] = val
        want = oracle.moe(oracle.Q4_K, gu, dn, _bits(x), oracle.BF16, ids, w)
        out["err"] = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    dist.barrier()
    dist.destroy_process_group()


def _run(world):
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
        return out["err"]


def test_two_ranks():
    # the expert outputs cross the wire in bf16 (as on the GPU), the checker sums fp16-rounded outputs
    assert _run(2) < 5e-3


def test_three_ranks():
    assert _run(3) < 5e-3


def test_plan_dispatch_order_and_counts():
    ids = torch.tensor([[0, 5], [4, -1], [2, 3], [7, 1]], dtype=torch.int32)  # 8 experts, 4 ranks of 2
    order, counts = tp.plan_dispatch(ids, 2, 4)
    assert counts.tolist() == [2, 2, 2, 1]
    assert order.tolist() == [0, 7, 4, 5, 1, 2, 6]
    order, counts = tp.plan_dispatch(torch.full((3, 2), -1, dtype=torch.int32), 2, 4)
    assert order.numel() == 0 and counts.tolist() == [0, 0, 0, 0]
