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
        self.group = group
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


def plan_dispatch(topk_ids: torch.Tensor, experts_per_rank: int, world: int):
    """Send order of the (token, choice) pairs of one rank for expert-parallel dispatch.

    Pairs go to the rank that holds their expert (``id // experts_per_rank``), grouped by destination in
    ascending rank, original order kept inside a group.  Returns ``(order, send_counts)``: ``order[i]`` is the
    flat pair index (``token * top_k + choice``) sent at position i; pairs with an id outside the global
    expert range are not sent.  Pure tensor code: runs on CPU or GPU.
    """
    flat = topk_ids.reshape(-1).to(torch.int64)
    valid = (flat >= 0) & (flat < experts_per_rank * world)
    dest = torch.where(valid, flat // experts_per_rank, torch.full_like(flat, world))
    order = torch.sort(dest, stable=True).indices
    counts = torch.bincount(dest, minlength=world + 1)
    order = order[: int(counts[:world].sum())]
    return order, counts[:world]


class ExpertParallelMoE:
    """Expert-parallel mixture-of-experts layer: rank r holds experts ``[r * E/P, (r + 1) * E/P)`` and its own
    slice of the tokens.  One forward is dispatch (all-to-all of the routed rows to the ranks that own their
    experts), the local grouped GEMM layer with one choice per received row, and combine (all-to-all back,
    weighted sum at the source in fp32, ascending choice order).

    ``local_forward(rows, local_ids)`` is the layer that runs the received rows through local expert
    ``local_ids[i]`` -- ``MoELayer`` on the GPU (``from_layer``), any callable in host-side tests.  The
    all-to-alls are ``torch.distributed.all_to_all_single`` (NCCL over NVLink on GPUs, gloo on CPU); the
    split sizes travel first, which costs one host synchronisation per forward.
    """

    def __init__(self, local_forward, experts_per_rank: int, top_k: int, group=None):
        import torch.distributed as dist

        self.dist, self.group = dist, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.local_forward, self.epr, self.top_k = local_forward, experts_per_rank, top_k

    @classmethod
    def from_layer(cls, layer, group=None):
        """``layer``: a MoELayer built with top_k = 1 over this rank's experts, sized for the rows it may receive."""
        if layer.top_k != 1:
            raise ValueError("the local layer of an expert-parallel group takes one expert per received row")

        def run(rows, local_ids):
            ones = torch.ones((rows.shape[0], 1), dtype=torch.float32, device=rows.device)
            return layer.forward(rows, local_ids.reshape(-1, 1), ones)

        return cls(run, layer.n_experts, 1, group)

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        dist, P = self.dist, self.world
        t, k = topk_ids.shape
        order, send_counts = plan_dispatch(topk_ids, self.epr, P)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        send_splits, recv_splits = send_counts.tolist(), recv_counts.tolist()
        n_recv = sum(recv_splits)
        send_rows = x.reshape(t, -1)[order // k].contiguous()
        send_ids = (topk_ids.reshape(-1)[order].to(torch.int64) % self.epr).to(torch.int32).contiguous()
        recv_rows = torch.empty((n_recv, send_rows.shape[1]), dtype=x.dtype, device=x.device)
        recv_ids = torch.empty((n_recv,), dtype=torch.int32, device=x.device)
        dist.all_to_all_single(recv_rows, send_rows, recv_splits, send_splits, group=self.group)
        dist.all_to_all_single(recv_ids, send_ids, recv_splits, send_splits, group=self.group)
        out_rows = self.local_forward(recv_rows, recv_ids) if n_recv else recv_rows
        back = torch.empty_like(send_rows)
        dist.all_to_all_single(back, out_rows.contiguous(), send_splits, recv_splits, group=self.group)
        # place every returned row at its (token, choice) slot, then the weighted sum over the choices
        slots = torch.zeros((t * k, back.shape[1]), dtype=torch.float32, device=x.device)
        slots[order] = back.float()
        y = (slots.view(t, k, -1) * topk_weights.reshape(t, k, 1).float()).sum(dim=1)
        return y.to(x.dtype)


def shard_trellis(packed: torch.Tensor, out_features: int, in_features: int, kind: int, rank: int, world: int):
    """Tensor-parallel slice of a trellis-coded (TTQ_FMT_TQ3) buffer: returns (local buffer, local N, local K).

    COLUMN keeps rows ``[rank * N/P, (rank + 1) * N/P)`` (tiles and out_scale of those rows, all of in_sign);
    ROW keeps the K columns of the rank (tile columns and in_sign of the slice, all of out_scale) -- the output
    rotation and scale are linear, so the ranks' results simply add.  Slices must be multiples of 128, the
    Hadamard block, so that a shard rotates locally.
    """
    n, k = out_features, in_features
    tiles_end = n * k * 3 // 8
    tiles = packed[:tiles_end].reshape(n // 16, k // 16, 96)
    scale = packed[tiles_end:tiles_end + 2 * n]
    sign = packed[tiles_end + 2 * n:]
    if kind == SHARD_NONE or world == 1:
        return packed, n, k
    if not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if kind == SHARD_COLUMN:
        if n % (128 * world):
            raise ValueError("out_features / world must be a multiple of 128")
        nl = n // world
        t = tiles[rank * nl // 16:(rank + 1) * nl // 16]
        return torch.cat((t.reshape(-1), scale[2 * rank * nl:2 * (rank + 1) * nl], sign)), nl, k
    if kind == SHARD_ROW:
        if k % (128 * world):
            raise ValueError("in_features / world must be a multiple of 128")
        kl = k // world
        t = tiles[:, rank * kl // 16:(rank + 1) * kl // 16]
        return torch.cat((t.reshape(-1), scale, sign[rank * kl // 8:(rank + 1) * kl // 8])), n, kl
    raise ValueError(f"shard kind {kind} does not apply to the trellis format")
