## QuantLinear -- drop-in for `Linear` (workspace/transformers/src/layers/linear.nim) whose weight
## is a block-quantized matrix served by libttq (include/ttq.h).
##
## Same surface as the reference layer: a plain object, `init` from existing weights, `forward(x)`.
## Compile with `nim cpp` like the rest of the workspace; link with `--passL:-lttq`.
## This file is the whole host-side integration: every call goes through the C ABI, no libtorch call
## is made on this path except `data_ptr` to obtain device pointers.

import
  std/options,
  workspace/libtorch as F

{.passL: "-lttq".}

type
  TtqCtx* {.importc: "ttq_ctx", header: "ttq.h", incompleteStruct.} = object
  TtqWeight* {.importc: "ttq_weight", header: "ttq.h", incompleteStruct.} = object
  TtqStatus* = cint
  TtqComm* {.importc: "ttq_comm", header: "ttq.h", incompleteStruct.} = object
  TtqMoe* {.importc: "ttq_moe", header: "ttq.h", incompleteStruct.} = object
  TtqFormat* {.size: sizeof(cint).} = enum
    kQ8_0 = 0, kQ4_K = 1, kQ6_K = 2, kTQ3 = 3
  TtqDtype* {.size: sizeof(cint).} = enum
    kTtqBF16 = 0, kTtqF16 = 1, kTtqF32 = 2
  TtqShard* {.importc: "ttq_shard", header: "ttq.h", bycopy.} = object
    kind*, rank*, world*: int32
  TtqHostBatch* {.importc: "ttq_host_batch", header: "ttq.h", incompleteStruct.} = object
  TtqHostLinear* {.importc: "ttq_host_linear", header: "ttq.h", bycopy.} = object
    w*: ptr TtqWeight
    x_host*: pointer
    x_dt*: int32
    M*, ldx*: int64
    bias_host*: pointer
    bias_dt*: int32
    y_host*: pointer
    y_dt*: int32
    ldy*: int64

proc ttq_init(device: cint, ctx: ptr ptr TtqCtx): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_destroy(ctx: ptr TtqCtx): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_last_error(ctx: ptr TtqCtx): cstring {.importc, cdecl, header: "ttq.h".}
proc ttq_weight_create(ctx: ptr TtqCtx, fmt: TtqFormat, N, K: int64, hostBlocks: pointer, nbytes: csize_t,
                       shard: ptr TtqShard, w: ptr ptr TtqWeight): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_weight_destroy(w: ptr TtqWeight): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_linear_forward(ctx: ptr TtqCtx, w: ptr TtqWeight, x: pointer, xDt: TtqDtype, M, ldx: int64,
                        bias: pointer, biasDt: TtqDtype, y: pointer, yDt: TtqDtype, ldy: int64,
                        stream: pointer): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_silu_and_mul(ctx: ptr TtqCtx, inp: pointer, dt: TtqDtype, M, H, ldIn: int64, outp: pointer,
                      ldOut: int64, stream: pointer): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_linear_forward_gated(ctx: ptr TtqCtx, w: ptr TtqWeight, gateUp: pointer, xDt: TtqDtype, M, ldGateUp: int64,
                              bias: pointer, biasDt: TtqDtype, y: pointer, yDt: TtqDtype, ldy: int64,
                              stream: pointer): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_add_rmsnorm(ctx: ptr TtqCtx, h, delta, weight: pointer, dt: TtqDtype, M, H, ldH, ldDelta: int64,
                     eps: cfloat, outp: pointer, ldOut: int64, stream: pointer): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_add_rmsnorm_prepare(ctx: ptr TtqCtx, h, delta, weight: pointer, dt: TtqDtype, M, H, ldH, ldDelta: int64,
                             eps: cfloat, outp: pointer, ldOut: int64, stream: pointer): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_linear_forward_prepared(ctx: ptr TtqCtx, w: ptr TtqWeight, M: int64, bias: pointer, biasDt: TtqDtype, y: pointer,
                                 yDt: TtqDtype, ldy: int64, stream: pointer): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_rope_kv_append(ctx: ptr TtqCtx, qkv: pointer, dt: TtqDtype, B, ldQkv: int64, hq, hkv, d: int32,
                        cosv, sinv, qOut, kCache, vCache: pointer, ctxLen, pos: int64,
                        stream: pointer): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_decode_attention(ctx: ptr TtqCtx, q, kCache, vCache: pointer, dt: TtqDtype, B: int64, hq, hkv, d: int32,
                          ctxLen, nCtx: int64, outp: pointer, stream: pointer): TtqStatus {.importc, cdecl, header: "ttq.h".}

# -- the rest of the C ABI (include/ttq.h), bound one to one ------------------------------------------------
proc ttq_status_string(s: TtqStatus): cstring {.importc, cdecl, header: "ttq.h".}
proc ttq_version(): cstring {.importc, cdecl, header: "ttq.h".}
proc ttq_block_elems(fmt: TtqFormat): int64 {.importc, cdecl, header: "ttq.h".}
proc ttq_block_bytes(fmt: TtqFormat): int64 {.importc, cdecl, header: "ttq.h".}
proc ttq_packed_bytes(fmt: TtqFormat, N, K: int64): int64 {.importc, cdecl, header: "ttq.h".}
proc ttq_weight_create_device(ctx: ptr TtqCtx, fmt: TtqFormat, N, K: int64, devBlocks: pointer, nbytes: csize_t,
                              stream: pointer, w: ptr ptr TtqWeight): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_weight_info(w: ptr TtqWeight, fmt: ptr int32, N, K: ptr int64): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_weight_bytes(w: ptr TtqWeight): int64 {.importc, cdecl, header: "ttq.h".}
proc ttq_dequantize(ctx: ptr TtqCtx, w: ptr TtqWeight, devOut: ptr cfloat, ld: int64,
                    stream: pointer): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_linear_forward_host(ctx: ptr TtqCtx, w: ptr TtqWeight, xHost: pointer, xDt: TtqDtype, M, ldx: int64,
                             biasHost: pointer, biasDt: TtqDtype, yHost: pointer, yDt: TtqDtype,
                             ldy: int64): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_linear_forward_host_async(ctx: ptr TtqCtx, w: ptr TtqWeight, xHost: pointer, xDt: TtqDtype, M, ldx: int64,
                                   biasHost: pointer, biasDt: TtqDtype, yHost: pointer, yDt: TtqDtype,
                                   ldy: int64): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_host_sync(ctx: ptr TtqCtx): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_host_batch_create(ctx: ptr TtqCtx, linears: ptr TtqHostLinear, n: cint,
                            batch: ptr ptr TtqHostBatch): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_host_batch_run(batch: ptr TtqHostBatch): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_host_batch_destroy(batch: ptr TtqHostBatch): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_device_status(ctx: ptr TtqCtx, stream: pointer): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_linear_forward_static(w: ptr TtqWeight, x: pointer, xDt: TtqDtype, M, ldx: int64, bias: pointer,
                               biasDt: TtqDtype, y: pointer, yDt: TtqDtype, ldy: int64, stream: pointer,
                               errbuf: cstring, errbufLen: csize_t): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_static_status(stream: pointer, errbuf: cstring, errbufLen: csize_t): TtqStatus {.importc, cdecl, header: "ttq.h".}
# tensor parallelism: exchange buffers and the row-parallel linear with the sum over ranks fused in
proc ttq_comm_create(ctx: ptr TtqCtx, rank, world: cint, nCap: int64, mCap: cint, comm: ptr ptr TtqComm,
                     ipcHandleOut: pointer): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_comm_connect(comm: ptr TtqComm, allHandles: pointer): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_comm_local_buffer(comm: ptr TtqComm, baseOut: ptr pointer, bytesOut: ptr csize_t): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_comm_connect_pointers(comm: ptr TtqComm, bases: ptr pointer): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_comm_set_wait_limit(comm: ptr TtqComm, polls: int64): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_comm_destroy(comm: ptr TtqComm): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_linear_forward_allreduce(ctx: ptr TtqCtx, w: ptr TtqWeight, x: pointer, xDt: TtqDtype, M, ldx: int64,
                                  bias: pointer, biasDt: TtqDtype, y: pointer, yDt: TtqDtype, ldy: int64,
                                  comm: ptr TtqComm, stream: pointer): TtqStatus {.importc, cdecl, header: "ttq.h".}
# mixture-of-experts layer on the grouped Q4_K GEMM
proc ttq_moe_create(ctx: ptr TtqCtx, nExperts: int32, gateUp, down: ptr ptr TtqWeight, maxTokens: int64, topK: int32,
                    moe: ptr ptr TtqMoe): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_moe_destroy(moe: ptr TtqMoe): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_moe_forward(ctx: ptr TtqCtx, moe: ptr TtqMoe, x: pointer, xDt: TtqDtype, T, ldx: int64, topkIds: ptr int32,
                     topkWeights: ptr cfloat, y: pointer, yDt: TtqDtype, ldy: int64,
                     stream: pointer): TtqStatus {.importc, cdecl, header: "ttq.h".}
# introspection
proc ttq_trace_read(ctx: ptr TtqCtx, outp: ptr uint64, maxEntries: int64, nEntries: ptr int64): TtqStatus {.importc, cdecl, header: "ttq.h".}
proc ttq_launch_count(ctx: ptr TtqCtx): int64 {.importc, cdecl, header: "ttq.h".}

template check(ctx: ptr TtqCtx, rc: TtqStatus) =
  ## Non-zero status -> ValueError, the exception style of the reference's own loaders
  ## (workspace/safetensors/src/safetensors.nim:17-25).
  if rc != 0:
    raise newException(ValueError, "ttq: " & $ttq_last_error(ctx))

type
  TtqContext* = object
    ## One per host thread and device (value type holding the raw handle; never a module-level global).
    handle*: ptr TtqCtx

  QuantLinear* = object
    ## Quantized linear layer.
    ##
    ## Input:
    ##   - An externally provided `x` of shape [..., in_features], bf16 or f16, on the context's device
    ##   - A local packed weight of logical shape [out_features, in_features]
    ##   - Optionally a local bias of shape [out_features]
    ##
    ## Return:
    ##   - x @ weight^T + bias, shape [..., out_features], dtype of x
    ctx*: ptr TtqCtx
    weight*: ptr TtqWeight
    bias*: Option[TorchTensor]
    in_features*: int
    out_features*: int

proc init*(_: type TtqContext, device = 0): TtqContext =
  check(nil, ttq_init(device.cint, addr result.handle))

proc close*(c: var TtqContext) =
  discard ttq_destroy(c.handle)
  c.handle = nil

proc init*(_: type QuantLinear, ctx: TtqContext, fmt: TtqFormat, blocks: pointer, nbytes: int,
           out_features, in_features: int, bias = none(TorchTensor)): QuantLinear =
  ## Creates a quantized linear layer from canonical blocks in host memory (for instance the
  ## `MemSlice` returned by `getMmapView`, workspace/safetensors/src/safetensors.nim:256-274).
  ## The blocks are uploaded and repacked once; the host buffer can be unmapped afterwards.
  result = QuantLinear(ctx: ctx.handle, bias: bias, in_features: in_features, out_features: out_features)
  check(ctx.handle, ttq_weight_create(ctx.handle, fmt, out_features.int64, in_features.int64, blocks,
                                      nbytes.csize_t, nil, addr result.weight))

proc close*(self: var QuantLinear) =
  discard ttq_weight_destroy(self.weight)
  self.weight = nil

func ttqDtype(k: ScalarKind): TtqDtype =
  case k
  of kBFloat16: kTtqBF16
  of kFloat16: kTtqF16
  of kFloat32: kTtqF32
  else: raise newException(ValueError, "ttq: unsupported dtype " & $k)

proc forward*(self: QuantLinear, x: TorchTensor, stream: pointer = nil): TorchTensor =
  ## Forward pass for inference.
  ##
  ## Args:
  ##   x: Input tensor of shape (..., in_features), contiguous in its last dimension
  ##
  ## Returns:
  ##   Output tensor of shape (..., out_features)
  let x2 = x.reshape([-1, self.in_features]).contiguous()
  let M = x2.size(0)
  var outShape = x.sizes().asNimView().toSeq()
  outShape[^1] = self.out_features
  result = F.empty(outShape, x.options())
  let biasPtr = if self.bias.isSome: self.bias.get().data_ptr(byte) else: nil
  let biasDt = if self.bias.isSome: ttqDtype(self.bias.get().scalarType()) else: kTtqF32
  check(self.ctx, ttq_linear_forward(self.ctx, self.weight, x2.data_ptr(byte), ttqDtype(x2.scalarType()),
                                     M.int64, self.in_features.int64, biasPtr, biasDt,
                                     result.data_ptr(byte), ttqDtype(result.scalarType()),
                                     self.out_features.int64, stream))

proc silu_and_mul*(ctx: TtqContext, x: TorchTensor, stream: pointer = nil): TorchTensor =
  ## Fused form of workspace/transformers/src/kernels/activations.nim:14-38.
  let H = x.size(-1) div 2
  let x2 = x.reshape([-1, 2 * H]).contiguous()
  var outShape = x.sizes().asNimView().toSeq()
  outShape[^1] = H
  result = F.empty(outShape, x.options())
  check(ctx.handle, ttq_silu_and_mul(ctx.handle, x2.data_ptr(byte), ttqDtype(x2.scalarType()), x2.size(0).int64,
                                     H.int64, (2 * H).int64, result.data_ptr(byte), H.int64, stream))


proc forward_gated*(self: QuantLinear, gate_up: TorchTensor, stream: pointer = nil): TorchTensor =
  ## ``down_proj.forward(silu_and_mul(gate_up))`` of GatedMLP.forward (workspace/transformers/src/layers/mlp.nim:56-60)
  ## in one call: the activation is computed inside the projection's input conversion.
  let g2 = gate_up.reshape([-1, 2 * self.in_features]).contiguous()
  var outShape = gate_up.sizes().asNimView().toSeq()
  outShape[^1] = self.out_features
  result = F.empty(outShape, gate_up.options())
  let biasPtr = if self.bias.isSome: self.bias.get().data_ptr(byte) else: nil
  let biasDt = if self.bias.isSome: ttqDtype(self.bias.get().scalarType()) else: kTtqF32
  check(self.ctx, ttq_linear_forward_gated(self.ctx, self.weight, g2.data_ptr(byte), ttqDtype(g2.scalarType()),
                                           g2.size(0).int64, (2 * self.in_features).int64, biasPtr, biasDt,
                                           result.data_ptr(byte), ttqDtype(result.scalarType()),
                                           self.out_features.int64, stream))

proc add_rmsnorm*(ctx: TtqContext, h: var TorchTensor, delta: Option[TorchTensor], weight: TorchTensor, eps: float32,
                  stream: pointer = nil): TorchTensor =
  ## ``RmsNorm.forward_with_residual`` (workspace/transformers/src/layers/norm.nim:27-38) as one kernel:
  ## h += delta in place, returns rmsnorm(h) * weight.  h is 2-D and contiguous.
  result = F.empty_like(h)
  let dPtr = if delta.isSome: delta.get().data_ptr(byte) else: nil
  check(ctx.handle, ttq_add_rmsnorm(ctx.handle, h.data_ptr(byte), dPtr, weight.data_ptr(byte), ttqDtype(h.scalarType()),
                                    h.size(0).int64, h.size(1).int64, h.size(1).int64, h.size(1).int64, eps.cfloat,
                                    result.data_ptr(byte), h.size(1).int64, stream))
