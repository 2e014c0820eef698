"""Tensor-parallel helpers: which slice of a packed weight a rank keeps, and the reduction a
row-parallel linear needs.  The reference has no parallelism; the split is the usual column/row scheme
(include/ttq.h, ``ttq_shard``).  ``shard_blocks`` is the host-side statement of what
``ttq_weight_create(..., shard)`` uploads, usable without a GPU."""
from __future__ import annotations

import torch

from ._lib import SHARD_COLUMN, SHARD_COLUMN_GATED, SHARD_NONE, SHARD_ROW
from .formats import BLOCK_BYTES, BLOCK_ELEMS


def shard_blocks(fmt: int, blocks: torch.Tensor, in_features: int, kind: int, rank: int, world: int):
    """Returns (local_blocks, local_out_features, local_in_features) of a canonical block matrix."""
    n, k = blocks.shape[0], in_features
    be, bb = BLOCK_ELEMS[fmt], BLOCK_BYTES[fmt]
    if kind == SHARD_NONE or world == 1:
        return blocks, n, k
    if not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if kind == SHARD_COLUMN:
        if n % world:
            raise ValueError("out_features not divisible by world")
        nl = n // world
        return blocks[rank * nl:(rank + 1) * nl], nl, k
    if kind == SHARD_COLUMN_GATED:
        if n % (2 * world):
            raise ValueError("out_features not divisible by 2*world")
        half, hl = n // 2, n // (2 * world)
        return torch.cat([blocks[rank * hl:(rank + 1) * hl], blocks[half + rank * hl:half + (rank + 1) * hl]]), 2 * hl, k
    if kind == SHARD_ROW:
        if k % (world * be):
            raise ValueError("in_features / world must be a multiple of the block length")
        kl = k // world
        bpr = kl // be * bb
        return blocks[:, rank * bpr:(rank + 1) * bpr].contiguous(), n, kl
    raise ValueError(f"unknown shard kind {kind}")


def all_reduce_sum(y: torch.Tensor) -> torch.Tensor:
    """Sum of the partial outputs of a row-parallel linear over all ranks (in place)."""
    import torch.distributed as dist

    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(y)
    return y


class Communicator:
    """Exchange buffers of a tensor-parallel group for ``QuantLinear.forward_allreduce`` (one process per GPU).

    Built on the C ABI (``ttq_comm_create`` / ``ttq_comm_connect``): each rank allocates its buffer, the
    64-byte CUDA IPC handles are all-gathered with ``torch.distributed`` and every rank maps its peers.
    """

    def __init__(self, ctx, n_cap: int, m_cap: int = 4, group=None):
        import ctypes

        import torch.distributed as dist

        from ._lib import check

        self.ctx = ctx
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.m_cap, self.n_cap = m_cap, n_cap
        lib = ctx._lib
        h = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        check(ctx.handle, lib.ttq_comm_create(ctx.handle, self.rank, self.world, n_cap, m_cap, ctypes.byref(h), handle))
        self.handle = h
        mine = torch.frombuffer(bytearray(handle.raw), dtype=torch.uint8).to(ctx.device)
        gathered = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(gathered, mine, group=group)
        blob = b"".join(bytes(t.cpu().numpy().tobytes()) for t in gathered)
        check(ctx.handle, lib.ttq_comm_connect(h, blob))
        dist.barrier(group=group)  # every buffer is zeroed and mapped before anyone writes into it

    def close(self):
        if getattr(self, "handle", None):
            self.ctx._lib.ttq_comm_destroy(self.handle)
            self.handle = None
