"""Llama-style decoder stack wired from QuantLinear layers, for the decode-throughput benchmark.

The linears, silu_and_mul and (by default) the steps between them -- residual add + RMSNorm, RoPE + KV-cache
append, single-query attention -- run in libttq; ``fused_glue=False`` runs those steps as plain torch ops
instead.  They stand for the reference's own layers (workspace/transformers/src/layers: norm.nim:23-38,
rope.nim:29-92, attn.nim:56-88,149-189).  Dataflow of one layer follows the reference's long-residual block
(transformer.nim:122-156): attn_norm -> attention -> residual -> mlp_norm -> gated MLP -> residual.

Weights are synthetic: every rank draws its own tensor-parallel shard (N(0, 0.02), quantized on the
device) -- q/kv heads and FFN rows split over ranks, O and down split along K with a sum over ranks.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import quantize as Q
from ._lib import FMT_Q4_K, FMT_Q6_K
from .layers import Context, QuantLinear, add_rmsnorm, decode_attention, rope_kv_append, silu_and_mul


@dataclass
class DecoderConfig:
    """Llama-3-8B geometry."""
    n_layers: int = 32
    hidden: int = 4096
    n_q_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5
    context: int = 2048


def synthetic_blocks(fmt, n, k, seed, dev):
    """Canonical blocks of a seeded N(0, 0.02) matrix, quantized on the device (what the stack's linears hold)."""
    g = torch.Generator(device=dev).manual_seed(seed)
    w = torch.randn(n, k, generator=g, device=dev) * 0.02
    return Q.quantize(fmt, w)


def _qlinear(ctx, fmt, n, k, seed, dev):
    return QuantLinear(ctx, fmt, synthetic_blocks(fmt, n, k, seed, dev), k)


class DecoderStack:
    def __init__(self, ctx: Context, cfg: DecoderConfig, batch: int, rank: int = 0, world: int = 1, seed: int = 3000, comm=None,
                 fused_glue: bool = True):
        assert cfg.n_q_heads % world == 0 and cfg.n_kv_heads % world == 0 and cfg.ffn % (256 * world) == 0
        self.ctx, self.cfg, self.batch, self.rank, self.world = ctx, cfg, batch, rank, world
        self.comm = comm  # tp.Communicator: row-parallel sums fused into the linears when the batch fits
        self.fused_glue = fused_glue
        dev = ctx.device
        self.dev = dev
        hq, hkv, d = cfg.n_q_heads // world, cfg.n_kv_heads // world, cfg.head_dim
        self.hq, self.hkv = hq, hkv
        ffn_l = cfg.ffn // world
        self.layers = []
        for layer in range(cfg.n_layers):
            s = seed + 16 * layer + 1000 * rank
            self.layers.append({
                "qkv": _qlinear(ctx, FMT_Q4_K, (hq + 2 * hkv) * d, cfg.hidden, s + 0, dev),     # column parallel (heads)
                "o": _qlinear(ctx, FMT_Q4_K, cfg.hidden, hq * d, s + 1, dev),                   # row parallel
                "gate_up": _qlinear(ctx, FMT_Q4_K, 2 * ffn_l, cfg.hidden, s + 2, dev),          # column parallel, [gate; up]
                "down": _qlinear(ctx, FMT_Q4_K, cfg.hidden, ffn_l, s + 3, dev),                 # row parallel
                "attn_norm": (1.0 + 0.02 * torch.randn(cfg.hidden, device=dev)).to(torch.bfloat16),
                "mlp_norm": (1.0 + 0.02 * torch.randn(cfg.hidden, device=dev)).to(torch.bfloat16),
                # KV cache prefilled to the full context with N(0,1) values: [batch, kv heads, context, head_dim]
                "k": torch.randn(batch, hkv, cfg.context, d, device=dev).to(torch.bfloat16),
                "v": torch.randn(batch, hkv, cfg.context, d, device=dev).to(torch.bfloat16),
            })
        vocab_l = cfg.vocab // world
        self.lm_head = _qlinear(ctx, FMT_Q6_K, vocab_l, cfg.hidden, seed + 900 + rank, dev)     # column parallel
        # embedding: the full vocabulary as Q6_K rows, expanded once at load time to bf16 (the lookup reads only
        # `batch` rows per step); built in slabs so that the fp32 expansion stays small
        self.emb_rows = torch.empty((cfg.vocab, cfg.hidden), dtype=torch.bfloat16, device=dev)
        slab = 16032
        for r0 in range(0, cfg.vocab, slab):
            rows = min(slab, cfg.vocab - r0)
            emb_q = _qlinear(ctx, FMT_Q6_K, rows, cfg.hidden, seed + 901 + r0, dev)
            self.emb_rows[r0:r0 + rows] = emb_q.dequantize().to(torch.bfloat16)
            emb_q.close()
        self.final_norm = torch.ones(cfg.hidden, device=dev, dtype=torch.bfloat16)
        pos = cfg.context - 1
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2, device=dev, dtype=torch.float64) / d))
        ang = pos * inv
        self.cos = torch.cat([ang.cos(), ang.cos()]).to(torch.bfloat16)
        self.sin = torch.cat([ang.sin(), ang.sin()]).to(torch.bfloat16)
        self.pos = pos
        self.weight_bytes = sum(l[k].weight_bytes for l in self.layers for k in ("qkv", "o", "gate_up", "down")) + self.lm_head.weight_bytes

    def _rms(self, x, w):
        return torch.nn.functional.rms_norm(x, (x.shape[-1],), w, self.cfg.rms_eps)

    def _rope(self, t):
        d = t.shape[-1]
        rot = torch.cat([-t[..., d // 2:], t[..., :d // 2]], dim=-1)
        return t * self.cos + rot * self.sin

    def _row_parallel(self, lin, x):
        if self.world == 1:
            return lin.forward(x)
        if self.comm is not None:
            return lin.forward_allreduce(x, self.comm)
        return lin.forward_reduce(x)

    def _step_fused(self, token_ids: torch.Tensor) -> torch.Tensor:
        """The layer loop with the library's decode-step kernels: 9 launches per layer besides the linears' own."""
        cfg, B, d, ctx = self.cfg, token_ids.shape[0], self.cfg.head_dim, self.ctx  # any batch up to the one the caches hold
        h = self.emb_rows[token_ids].contiguous()
        delta = None
        # up to two rows the linears run the integer decode kernel, whose activation planes the norm kernel can write
        # itself: one launch and one dependent hand-over less for the QKV and gate|up projections
        prep = B <= 2 and cfg.hidden % 256 == 0 and cfg.hidden <= 8192
        for L in self.layers:
            x = add_rmsnorm(ctx, h, delta, L["attn_norm"], cfg.rms_eps, prepare=prep)
            qkv = L["qkv"].forward_prepared(B, x.dtype) if prep else L["qkv"].forward(x)
            q = rope_kv_append(ctx, qkv, self.hq, self.hkv, d, self.cos, self.sin, L["k"], L["v"], self.pos)
            att = decode_attention(ctx, q, L["k"], L["v"], cfg.context)
            o = self._row_parallel(L["o"], att.view(B, self.hq * d))
            x = add_rmsnorm(ctx, h, o, L["mlp_norm"], cfg.rms_eps, prepare=prep)
            gu = L["gate_up"].forward_prepared(B, x.dtype) if prep else L["gate_up"].forward(x)
            if self.world == 1:
                delta = L["down"].forward_gated(gu)  # silu(gate) * up folded into the projection's input conversion
            else:
                delta = self._row_parallel(L["down"], silu_and_mul(ctx, gu))
        return add_rmsnorm(ctx, h, delta, self.final_norm, cfg.rms_eps)

    def step(self, token_ids: torch.Tensor) -> torch.Tensor:
        """One decode step for `batch` sequences at position context-1; returns next token ids."""
        if self.fused_glue:
            return self._pick(self.lm_head.forward(self._step_fused(token_ids), out_dtype=torch.float32))
        cfg, B, d = self.cfg, token_ids.shape[0], self.cfg.head_dim
        h = self.emb_rows[token_ids]
        for L in self.layers:
            x = self._rms(h, L["attn_norm"])
            qkv = L["qkv"].forward(x)
            q = qkv[:, : self.hq * d].view(B, self.hq, 1, d)
            k = qkv[:, self.hq * d:(self.hq + self.hkv) * d].view(B, self.hkv, 1, d)
            v = qkv[:, (self.hq + self.hkv) * d:].view(B, self.hkv, 1, d)
            q, k = self._rope(q), self._rope(k)
            L["k"][:B, :, self.pos:self.pos + 1] = k
            L["v"][:B, :, self.pos:self.pos + 1] = v
            att = torch.nn.functional.scaled_dot_product_attention(q, L["k"][:B], L["v"][:B], enable_gqa=True)
            o = self._row_parallel(L["o"], att.reshape(B, self.hq * d))
            h = h + o
            x = self._rms(h, L["mlp_norm"])
            gu = L["gate_up"].forward(x)
            act = silu_and_mul(self.ctx, gu)
            h = h + self._row_parallel(L["down"], act)
        return self._pick(self.lm_head.forward(self._rms(h, self.final_norm), out_dtype=torch.float32))

    def _pick(self, logits: torch.Tensor) -> torch.Tensor:
        """Greedy token over the (vocabulary-parallel) logits."""
        if self.world > 1:
            import torch.distributed as dist

            val, idx = logits.max(dim=-1)
            vals = [torch.empty_like(val) for _ in range(self.world)]
            idxs = [torch.empty_like(idx) for _ in range(self.world)]
            dist.all_gather(vals, val)
            dist.all_gather(idxs, idx + self.rank * logits.shape[-1])
            best = torch.stack(vals).argmax(dim=0)
            return torch.stack(idxs).gather(0, best.unsqueeze(0)).squeeze(0)
        return logits.argmax(dim=-1)
