"""Row-parallel linear with the fused peer-memory all-reduce, on two GPUs (skipped on single-GPU boxes)."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

N, K = 512, 2048


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    import torch.distributed as dist

    import oracle
    import tattletale_b200 as ttq
    from tattletale_b200 import tp

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ctx = ttq.Context(rank)
    rng = np.random.default_rng(900)
    blocks = oracle.quantize(oracle.Q4_K, rng.normal(0, 0.02, (N, K)).astype(np.float32))
    bias = torch.from_numpy(rng.normal(0, 0.1, N).astype(np.float32)).cuda()
    lin = ttq.QuantLinear(ctx, ttq.FMT_Q4_K, torch.from_numpy(blocks), K, bias=bias, shard=(ttq.SHARD_ROW, rank, world))
    comm = tp.Communicator(ctx, n_cap=N, m_cap=16)
    kl = K // world
    errs, agree = [], []
    # consecutive exchanges reuse both parities of the buffers; 1..2 rows: integer decode kernel, 3..16: fp16 kernel
    for call, m in enumerate((1, 4, 2, 1, 3, 16, 9, 1)):
        x = torch.from_numpy(rng.normal(0, 1, (m, K)).astype(np.float32)).to(torch.bfloat16)
        y = lin.forward_allreduce(x[:, rank * kl:(rank + 1) * kl].cuda(), comm, out_dtype=torch.float32)
        ctx.check_device_status()
        want = oracle.linear(oracle.Q4_K, blocks, x.view(torch.int16).numpy().view(np.uint16), oracle.BF16, bias.cpu().numpy())
        errs.append(float(np.linalg.norm(y.cpu().numpy() - want) / np.linalg.norm(want)))
        ys = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(ys, y)
        agree.append(all(torch.equal(ys[0], t) for t in ys))
    # a batch larger than the exchange buffer falls back to forward + library all-reduce
    # (the bias stays on: the fallback must add it once, after the sum over ranks)
    x = torch.from_numpy(rng.normal(0, 1, (24, K)).astype(np.float32)).to(torch.bfloat16)
    y = lin.forward_allreduce(x[:, rank * kl:(rank + 1) * kl].cuda(), comm, out_dtype=torch.float32)
    want = oracle.linear(oracle.Q4_K, blocks, x.view(torch.int16).numpy().view(np.uint16), oracle.BF16, bias.cpu().numpy())
    errs.append(float(np.linalg.norm(y.cpu().numpy() - want) / np.linalg.norm(want)))
    if rank == 0:
        out["errs"], out["agree"] = errs, agree
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)  # leave without tearing the communicators down (ranks exit between steps, nothing in flight)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_allreduce_matches_full_matrix():
    import torch.multiprocessing as mp

    world = 2
    ctxmp = mp.get_context("spawn")
    with ctxmp.Manager() as mgr:
        out = mgr.dict()
        procs = [ctxmp.Process(target=_worker, args=(r, world, port, out)) for port in [_free_port()] for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=180)
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        assert all(e < 1e-3 for e in out["errs"]), out["errs"]
        assert all(out["agree"]), "ranks disagree on the reduced result"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_contexts_in_one_process():
    """One process, one context per device: every device gets its own kernel configuration (shared-memory opt-in)."""
    import oracle
    import tattletale_b200 as ttq

    rng = np.random.default_rng(77)
    blocks = oracle.quantize(oracle.Q4_K, rng.normal(0, 0.02, (N, K)).astype(np.float32))
    for m in (1, 64):  # decode kernel and tensor-core GEMM
        x = torch.from_numpy(rng.normal(0, 1, (m, K)).astype(np.float32)).to(torch.bfloat16)
        want = oracle.linear(oracle.Q4_K, blocks, x.view(torch.int16).numpy().view(np.uint16), oracle.BF16)
        for dev in (0, 1):
            with torch.cuda.device(dev):
                ctx = ttq.Context(dev)
                lin = ttq.QuantLinear(ctx, ttq.FMT_Q4_K, torch.from_numpy(blocks), K)
                y = lin.forward(x.to(f"cuda:{dev}"), out_dtype=torch.float32)
                ctx.check_device_status()
                err = float(np.linalg.norm(y.cpu().numpy() - want) / np.linalg.norm(want))
                assert err < 1e-3, (dev, m, err)
                lin.close()
                ctx.close()
