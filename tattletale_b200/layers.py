"""Operator objects with the reference's surface: plain objects with ``init``-style constructors
and a ``forward`` method, no base class (workspace/transformers/src/layers/all.nim:8-15)."""
from __future__ import annotations

import ctypes
import enum
from typing import Optional

import torch

from . import _lib
from ._lib import Shard, TtqError, check
from .formats import BLOCK_BYTES, BLOCK_ELEMS, packed_bytes

_TORCH_DT = {torch.bfloat16: _lib.DT_BF16, torch.float16: _lib.DT_F16, torch.float32: _lib.DT_F32}


def _dt(t: torch.dtype) -> int:
    try:
        return _TORCH_DT[t]
    except KeyError:
        raise TtqError(_lib.OK + 1, f"unsupported dtype {t}") from None


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class Context:
    """One per (host thread, device): owns the library's scratch.  ``ttq_init`` / ``ttq_destroy``."""

    def __init__(self, device: int | torch.device = 0):
        self._lib = _lib.load()
        dev = torch.device(device) if not isinstance(device, int) else torch.device("cuda", device)
        self.device = dev
        h = ctypes.c_void_p()
        st = self._lib.ttq_init(dev.index or 0, ctypes.byref(h))
        check(None, st)
        self.handle = h

    def close(self) -> None:
        if getattr(self, "handle", None):
            self._lib.ttq_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def host_sync(self) -> None:
        """Waits for the calls enqueued with ``forward_host(..., wait=False)``; raises if one of their kernels gave up a wait."""
        check(self.handle, self._lib.ttq_host_sync(self.handle))

    def check_device_status(self) -> None:
        """Synchronises the current stream; raises TtqError(TIMEOUT) if a kernel gave up a bounded wait."""
        check(self.handle, self._lib.ttq_device_status(self.handle, _stream_ptr(self.device)))

    def read_trace(self, max_entries: int = 8192):
        """Device timeline entries recorded since the last read (needs TTQ_TRACE=1 at creation): int64 [n, 8]."""
        buf = torch.zeros((max_entries, 8), dtype=torch.int64)
        n = ctypes.c_int64()
        check(self.handle, self._lib.ttq_trace_read(self.handle, buf.data_ptr(), max_entries, ctypes.byref(n)))
        return buf[: n.value]

    @property
    def launch_count(self) -> int:
        return int(self._lib.ttq_launch_count(self.handle))


class HostBatch:
    """Independent linears recorded once (``ttq_host_batch_create``) and run with one foreign call and one wait per
    step.  ``items``: (QuantLinear, x, y) with x and y contiguous tensors of decode size, either pinned CPU tensors or
    tensors on the context's device.  The linears must not depend on each other (no y is another's x): the activations
    of all decode-size linears are converted by one launch and those linears run side by side.  After ``run()`` returns
    every y holds its linear's result.  The batch runs on the context's own stream: synchronise the stream that wrote
    device inputs before ``run()``.  A linear's bias (a device tensor) is added as in ``forward``."""

    def __init__(self, ctx: "Context", items):
        self.ctx = ctx
        self._keep = list(items)
        arr = (_lib.HostLinear * len(self._keep))()
        for slot, (lin, x, y) in zip(arr, self._keep):
            x2 = x.reshape(-1, lin.in_features)
            y2 = y.reshape(-1, lin.out_features)
            if x2.data_ptr() != x.data_ptr() or y2.data_ptr() != y.data_ptr() or not x2.is_contiguous() or not y2.is_contiguous():
                raise TtqError(1, "x and y must be contiguous host tensors")
            slot.w, slot.x_host, slot.x_dt, slot.M, slot.ldx = lin.handle, x2.data_ptr(), _dt(x2.dtype), x2.shape[0], lin.in_features
            if lin.bias is not None:
                slot.bias_host, slot.bias_dt = lin.bias.data_ptr(), _dt(lin.bias.dtype)
            else:
                slot.bias_host, slot.bias_dt = None, _lib.DT_F32
            slot.y_host, slot.y_dt, slot.ldy = y2.data_ptr(), _dt(y2.dtype), lin.out_features
        handle = ctypes.c_void_p()
        check(ctx.handle, ctx._lib.ttq_host_batch_create(ctx.handle, arr, len(self._keep), ctypes.byref(handle)))
        self.handle = handle

    def run(self) -> None:
        check(self.ctx.handle, self.ctx._lib.ttq_host_batch_run(self.handle))

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.ctx._lib.ttq_host_batch_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class QuantLinear:
    """Quantized ``Linear`` (linear.nim:14-57): ``y = x @ W^T + bias`` with W held as packed blocks.

    ``blocks`` is a uint8 tensor of canonical row-major blocks, shape ``[out_features, bytes_per_row]``,
    on the host (uploaded and repacked) or already on the device.  ``bias`` is an optional device
    tensor of ``out_features`` elements.  ``forward`` accepts ``x`` of shape ``(..., in_features)`` in
    bf16 or f16 on the context's device and returns ``(..., out_features)`` in ``out_dtype`` (the
    input dtype by default, as ATen linear does).
    """

    def __init__(self, ctx: Context, fmt: int, blocks: torch.Tensor, in_features: int,
                 bias: Optional[torch.Tensor] = None, shard: Optional[tuple[int, int, int]] = None,
                 out_features: Optional[int] = None):
        if fmt == _lib.FMT_TQ3:
            # one flat buffer (tiles | out_scale | in_sign): the row count cannot be read off its shape
            if blocks.dtype != torch.uint8 or blocks.dim() != 1 or out_features is None:
                raise TtqError(1, "the trellis format takes a 1-D uint8 buffer and out_features")
        elif blocks.dtype != torch.uint8 or blocks.dim() != 2:
            raise TtqError(1, "blocks must be a 2-D uint8 tensor [out_features, bytes_per_row]")
        self.ctx, self.fmt = ctx, fmt
        lib = ctx._lib
        n, k = int(out_features if fmt == _lib.FMT_TQ3 else blocks.shape[0]), int(in_features)
        blocks = blocks.contiguous()
        h = ctypes.c_void_p()
        if blocks.is_cuda:
            if shard is not None:
                raise TtqError(3, "sharding is applied while uploading host blocks")
            st = lib.ttq_weight_create_device(ctx.handle, fmt, n, k, blocks.data_ptr(), blocks.numel(),
                                              _stream_ptr(blocks.device), ctypes.byref(h))
            check(ctx.handle, st)
            torch.cuda.current_stream(blocks.device).synchronize()  # blocks may be freed by the caller
        else:
            sh = None if shard is None else ctypes.byref(Shard(*shard))
            st = lib.ttq_weight_create(ctx.handle, fmt, n, k, blocks.data_ptr(), blocks.numel(), sh,
                                       ctypes.byref(h))
            check(ctx.handle, st)
        self.handle = h
        f, nn, kk = ctypes.c_int32(), ctypes.c_int64(), ctypes.c_int64()
        check(ctx.handle, lib.ttq_weight_info(h, ctypes.byref(f), ctypes.byref(nn), ctypes.byref(kk)))
        self.out_features, self.in_features = int(nn.value), int(kk.value)
        if bias is not None and bias.numel() != self.out_features:
            raise TtqError(2, f"bias has {bias.numel()} elements, expected {self.out_features}")
        self.bias = None if bias is None else bias.contiguous()

    @classmethod
    def init(cls, ctx: Context, fmt: int, blocks: torch.Tensor, in_features: int,
             bias: Optional[torch.Tensor] = None, shard=None) -> "QuantLinear":
        """Spelling of the reference constructor (``Linear.init``, linear.nim:29)."""
        return cls(ctx, fmt, blocks, in_features, bias, shard)

    @property
    def weight_bytes(self) -> int:
        return int(self.ctx._lib.ttq_weight_bytes(self.handle))

    def dequantize(self) -> torch.Tensor:
        """fp32 ``[out_features, in_features]`` expansion of the device layout (test hook)."""
        out = torch.empty((self.out_features, self.in_features), dtype=torch.float32, device=self.ctx.device)
        st = self.ctx._lib.ttq_dequantize(self.ctx.handle, self.handle, out.data_ptr(), self.in_features,
                                          _stream_ptr(self.ctx.device))
        check(self.ctx.handle, st)
        return out

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                out: Optional[torch.Tensor] = None, use_bias: bool = True) -> torch.Tensor:
        if not x.is_cuda:
            raise TtqError(1, "x must live on the context's CUDA device (use forward_host for host buffers)")
        if x.shape[-1] != self.in_features:
            raise TtqError(2, f"x has {x.shape[-1]} input features, the layer has {self.in_features}")
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        m = x2.shape[0]
        odt = out_dtype or x.dtype
        if out is None:
            out = torch.empty((m, self.out_features), dtype=odt, device=x.device)
        y2 = out.reshape(-1, self.out_features)
        b = self.bias if use_bias else None
        st = self.ctx._lib.ttq_linear_forward(
            self.ctx.handle, self.handle, x2.data_ptr(), _dt(x2.dtype), m, x2.stride(0) if m > 1 else self.in_features,
            None if b is None else b.data_ptr(), _lib.DT_F32 if b is None else _dt(b.dtype),
            y2.data_ptr(), _dt(y2.dtype), y2.stride(0) if m > 1 else self.out_features, _stream_ptr(x.device))
        check(self.ctx.handle, st)
        return out.reshape(*lead, self.out_features)

    __call__ = forward

    def forward_prepared(self, m: int, out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None,
                         use_bias: bool = True) -> torch.Tensor:
        """``forward`` on the ``m`` rows the last ``add_rmsnorm(..., prepare=True)`` left in the context (same stream);
        bit-identical to ``forward`` on that call's result, without the conversion pass."""
        if out is None:
            out = torch.empty((m, self.out_features), dtype=out_dtype, device=self.ctx.device)
        y2 = out.reshape(-1, self.out_features)
        b = self.bias if use_bias else None
        st = self.ctx._lib.ttq_linear_forward_prepared(
            self.ctx.handle, self.handle, m, None if b is None else b.data_ptr(), _lib.DT_F32 if b is None else _dt(b.dtype),
            y2.data_ptr(), _dt(y2.dtype), y2.stride(0) if m > 1 else self.out_features, _stream_ptr(self.ctx.device))
        check(self.ctx.handle, st)
        return out

    def forward_gated(self, gate_up: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``forward(silu(gate) * up)`` for ``gate_up = [gate | up]`` of ``2 * in_features`` columns: the activation
        of the gated MLP (mlp.nim:56-60) folded into the input conversion of this (down) projection."""
        if gate_up.shape[-1] != 2 * self.in_features:
            raise TtqError(2, f"gate_up has {gate_up.shape[-1]} columns, expected {2 * self.in_features}")
        x2 = gate_up.reshape(-1, 2 * self.in_features)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        m = x2.shape[0]
        if out is None:
            out = torch.empty((m, self.out_features), dtype=out_dtype or gate_up.dtype, device=gate_up.device)
        y2 = out.reshape(-1, self.out_features)
        b = self.bias
        st = self.ctx._lib.ttq_linear_forward_gated(
            self.ctx.handle, self.handle, x2.data_ptr(), _dt(x2.dtype), m, x2.stride(0) if m > 1 else 2 * self.in_features,
            None if b is None else b.data_ptr(), _lib.DT_F32 if b is None else _dt(b.dtype),
            y2.data_ptr(), _dt(y2.dtype), y2.stride(0) if m > 1 else self.out_features, _stream_ptr(gate_up.device))
        check(self.ctx.handle, st)
        return out.reshape(*gate_up.shape[:-1], self.out_features)

    def forward_allreduce(self, x: torch.Tensor, comm, out_dtype: Optional[torch.dtype] = None,
                          out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Row-parallel forward: this rank's K shard, summed over all ranks.  Decode-size batches go through the
        fused peer-memory all-reduce of the library; anything larger falls back to forward + NCCL all-reduce."""
        x2 = x.reshape(-1, self.in_features)
        m = x2.shape[0]
        odt = out_dtype or x.dtype
        if out is None:
            out = torch.empty((m, self.out_features), dtype=odt, device=x.device)
        if m > comm.m_cap or self.out_features > comm.n_cap:
            return self.forward_reduce(x, getattr(comm, "group", None), out=out)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        y2 = out.reshape(-1, self.out_features)
        b = self.bias
        st = self.ctx._lib.ttq_linear_forward_allreduce(
            self.ctx.handle, self.handle, x2.data_ptr(), _dt(x2.dtype), m, x2.stride(0) if m > 1 else self.in_features,
            None if b is None else b.data_ptr(), _lib.DT_F32 if b is None else _dt(b.dtype),
            y2.data_ptr(), _dt(y2.dtype), y2.stride(0) if m > 1 else self.out_features, comm.handle, _stream_ptr(x.device))
        check(self.ctx.handle, st)
        return out.reshape(*x.shape[:-1], self.out_features)

    def forward_reduce(self, x: torch.Tensor, group=None, out_dtype: Optional[torch.dtype] = None,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Row-parallel forward through a library all-reduce: the rank's partial product without the bias, summed over
        ``group`` in fp32, the bias added once after the sum (what the fused exchange does inside the kernel)."""
        import torch.distributed as dist

        part = self.forward(x, out_dtype=torch.float32, use_bias=False)
        dist.all_reduce(part, group=group)
        if self.bias is not None:
            part += self.bias.to(torch.float32)
        if out is None:
            return part.to(out_dtype or x.dtype)
        out.reshape(part.shape).copy_(part)
        return out.reshape(*x.shape[:-1], self.out_features)

    def forward_host(self, x: torch.Tensor, y: torch.Tensor, wait: bool = True) -> torch.Tensor:
        """Host-buffer call: x and y are CPU tensors (pinned for speed); copies are part of the call.

        ``wait=False`` only enqueues the call (pinned buffers of decode size required); ``Context.host_sync()`` then
        waits for all enqueued calls at once, and y must not be read before it returns."""
        x2 = x.reshape(-1, self.in_features)
        y2 = y.reshape(-1, self.out_features)
        m = x2.shape[0]
        fn = self.ctx._lib.ttq_linear_forward_host if wait else self.ctx._lib.ttq_linear_forward_host_async
        st = fn(
            self.ctx.handle, self.handle, x2.data_ptr(), _dt(x2.dtype), m, self.in_features, None, _lib.DT_F32,
            y2.data_ptr(), _dt(y2.dtype), self.out_features)
        check(self.ctx.handle, st)
        return y

    def host_call(self, x: torch.Tensor, y: torch.Tensor, wait: bool = True):
        """A zero-argument callable that runs ``forward_host(x, y, wait)`` on these very buffers with every argument
        bound ahead (a decode loop reuses its buffers: this leaves one foreign call per linear and step).  The
        callable keeps x and y alive; it raises like ``forward_host``."""
        x2 = x.reshape(-1, self.in_features)
        y2 = y.reshape(-1, self.out_features)
        if x2.data_ptr() != x.data_ptr() or y2.data_ptr() != y.data_ptr():
            raise TtqError(1, "x and y must be contiguous host tensors")
        fn = self.ctx._lib.ttq_linear_forward_host if wait else self.ctx._lib.ttq_linear_forward_host_async
        args = (self.ctx.handle, self.handle, x2.data_ptr(), _dt(x2.dtype), x2.shape[0], self.in_features, None, _lib.DT_F32,
                y2.data_ptr(), _dt(y2.dtype), self.out_features)
        ctx_handle = self.ctx.handle

        def call(_keep=(x, y, self)):
            st = fn(*args)
            if st != 0:
                check(ctx_handle, st)
        return call

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.ctx._lib.ttq_weight_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ActivationKind(enum.IntEnum):
    """kernels/activations.nim:10-12"""
    kSilu = 0


def silu_and_mul(ctx: Context, x: torch.Tensor) -> torch.Tensor:
    """``silu(x[..., :H]) * x[..., H:]`` (kernels/activations.nim:14-38); the gate is the first half."""
    h = x.shape[-1] // 2
    x2 = x.reshape(-1, 2 * h)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    out = torch.empty((x2.shape[0], h), dtype=x.dtype, device=x.device)
    st = ctx._lib.ttq_silu_and_mul(ctx.handle, x2.data_ptr(), _dt(x.dtype), x2.shape[0], h,
                                   x2.stride(0) if x2.shape[0] > 1 else 2 * h, out.data_ptr(), h,
                                   _stream_ptr(x.device))
    check(ctx.handle, st)
    return out.reshape(*x.shape[:-1], h)


class GatedMLP:
    """Gated MLP (mlp.nim:14-60): fused gate|up projection, silu_and_mul, down projection.

    The reference concatenates dense gate and up weights along dim 0 at init (mlp.nim:39); packed
    blocks are row-major, so the same concatenation of the two block matrices is the fused weight.
    """

    def __init__(self, ctx: Context, fmt: int, gate_blocks: torch.Tensor, up_blocks: torch.Tensor,
                 down_blocks: torch.Tensor, hidden_size: int, intermediate_size: int,
                 activation: ActivationKind = ActivationKind.kSilu):
        self.ctx = ctx
        self.gate_up_proj = QuantLinear(ctx, fmt, torch.cat([gate_blocks, up_blocks], 0), hidden_size)
        self.down_proj = QuantLinear(ctx, fmt, down_blocks, intermediate_size)
        self.activation = activation

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gate_up = self.gate_up_proj.forward(x)
        if self.activation != ActivationKind.kSilu:
            raise TtqError(3, f"activation {self.activation} is not implemented")
        return self.down_proj.forward(silu_and_mul(self.ctx, gate_up))

    __call__ = forward


class MoELayer:
    """Mixture of gated-MLP experts on the grouped Q4_K GEMM (``ttq_moe_*``).

    ``gate_up_blocks[e]`` is expert e's fused gate|up block matrix ``[2 * intermediate, bytes_per_row]``
    (gate rows first, as GatedMLP fuses them), ``down_blocks[e]`` its ``[hidden, bytes_per_row]`` down
    projection.  ``forward(x, topk_ids, topk_weights)`` computes, for every token t,
    ``sum_j topk_weights[t, j] * mlp_{topk_ids[t, j]}(x[t])``; router and top-k selection are the caller's.
    An id outside ``0..E-1`` drops that choice.
    """

    def __init__(self, ctx: Context, fmt: int, gate_up_blocks, down_blocks, hidden_size: int, intermediate_size: int,
                 top_k: int, max_tokens: int):
        if len(gate_up_blocks) != len(down_blocks) or not gate_up_blocks:
            raise TtqError(2, "gate_up_blocks and down_blocks must be equally long, non-empty lists")
        self.ctx, self.hidden, self.inter, self.top_k, self.max_tokens = ctx, hidden_size, intermediate_size, top_k, max_tokens
        self.gate_up = [QuantLinear(ctx, fmt, b, hidden_size) for b in gate_up_blocks]
        self.down = [QuantLinear(ctx, fmt, b, intermediate_size) for b in down_blocks]
        n = len(self.gate_up)
        self.n_experts = n
        arr_t = ctypes.c_void_p * n
        gu = arr_t(*[w.handle.value for w in self.gate_up])
        dn = arr_t(*[w.handle.value for w in self.down])
        h = ctypes.c_void_p()
        check(ctx.handle, ctx._lib.ttq_moe_create(ctx.handle, n, gu, dn, max_tokens, top_k, ctypes.byref(h)))
        self.handle = h

    @property
    def weight_bytes(self) -> int:
        return sum(w.weight_bytes for w in self.gate_up) + sum(w.weight_bytes for w in self.down)

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if not x.is_cuda:
            raise TtqError(1, "x must live on the context's CUDA device")
        x2 = x.reshape(-1, self.hidden)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        t = x2.shape[0]
        ids = topk_ids.reshape(t, self.top_k).to(torch.int32).contiguous()
        wts = topk_weights.reshape(t, self.top_k).to(torch.float32).contiguous()
        if out is None:
            out = torch.empty((t, self.hidden), dtype=x.dtype, device=x.device)
        st = self.ctx._lib.ttq_moe_forward(
            self.ctx.handle, self.handle, x2.data_ptr(), _dt(x2.dtype), t, x2.stride(0) if t > 1 else self.hidden,
            ids.data_ptr(), wts.data_ptr(), out.data_ptr(), _dt(out.dtype), out.stride(0) if t > 1 else self.hidden,
            _stream_ptr(x.device))
        check(self.ctx.handle, st)
        return out.reshape(x.shape)

    __call__ = forward

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.ctx._lib.ttq_moe_destroy(self.handle)
            self.handle = None
            for w in self.gate_up + self.down:
                w.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def add_rmsnorm(ctx: Context, h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: Optional[torch.Tensor] = None, prepare: bool = False) -> torch.Tensor:
    """``h += delta`` in place (skipped when ``delta`` is None), returns ``rmsnorm(h) * weight``
    (norm.nim:23-38, ``forward_with_residual`` fused).  2-D contiguous 16-bit tensors.

    ``prepare=True`` (1 or 2 rows, hidden size a multiple of 256) also leaves the rows in the context in the form
    the decode kernel reads: the linear that consumes the result may then be called as
    ``QuantLinear.forward_prepared`` and skips its own conversion pass."""
    m, hid = h.shape
    if out is None:
        out = torch.empty_like(h)
    fn = ctx._lib.ttq_add_rmsnorm_prepare if prepare else ctx._lib.ttq_add_rmsnorm
    st = fn(ctx.handle, h.data_ptr(), None if delta is None else delta.data_ptr(), weight.data_ptr(),
            _dt(h.dtype), m, hid, h.stride(0), hid if delta is None else delta.stride(0), eps,
            out.data_ptr(), out.stride(0), _stream_ptr(h.device))
    check(ctx.handle, st)
    return out


def rope_kv_append(ctx: Context, qkv: torch.Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int, cos: torch.Tensor,
                   sin: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: int,
                   q_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rotate the q and k heads of fused qkv rows for position ``pos`` (rope.nim:29-92, rotate-half), append k and v
    to the caches ``[B, kv heads, context, head_dim]``; returns q ``[B, q heads, head_dim]``."""
    b = qkv.shape[0]
    if q_out is None:
        q_out = torch.empty((b, n_q_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    st = ctx._lib.ttq_rope_kv_append(ctx.handle, qkv.data_ptr(), _dt(qkv.dtype), b, qkv.stride(0), n_q_heads, n_kv_heads, head_dim,
                                     cos.data_ptr(), sin.data_ptr(), q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                     k_cache.shape[2], pos, _stream_ptr(qkv.device))
    check(ctx.handle, st)
    return q_out


def decode_attention(ctx: Context, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, n_ctx: int,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Single-query grouped-query attention over cache positions ``0 .. n_ctx-1`` (attn.nim:149-189 for one new
    token): q ``[B, q heads, 128]``, caches ``[B, kv heads, context, 128]`` -> ``[B, q heads, 128]``."""
    b, hq, d = q.shape
    if out is None:
        out = torch.empty_like(q)
    st = ctx._lib.ttq_decode_attention(ctx.handle, q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), _dt(q.dtype), b, hq,
                                       k_cache.shape[1], d, k_cache.shape[2], n_ctx, out.data_ptr(), _stream_ptr(q.device))
    check(ctx.handle, st)
    return out
