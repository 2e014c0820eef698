/*
 * ttq.h -- C ABI of the B200 (sm_100a) quantized-linear library.
 *
 * This is the boundary a host program binds against (Nim `{.importc, cdecl.}`, C++, ctypes).  Plain
 * pointers and sizes only: no torch, no C++ types.  Every function returns a ttq_status (0 = OK),
 * never throws and never aborts; a human-readable reason for the last failure on a context is
 * available from ttq_last_error().
 *
 * The operator replaced is the reference's `Linear` (workspace/transformers/src/layers/linear.nim):
 *   Linear.init(weight[out,in], bias)   -> ttq_weight_create*()      (linear.nim:29-43)
 *   Linear.forward(x[..., in])          -> ttq_linear_forward()       (linear.nim:45-57)
 * whose only callee is ATen's linear (workspace/libtorch/src/abi/neural_nets.nim:64-81).  Here the
 * weight is a block-quantized matrix (GGUF-style Q8_0 / Q4_K / Q6_K) that the library repacks once,
 * at creation, into a tiled device layout; forward never allocates.
 *
 * Conventions
 *  - A ttq_ctx is bound to ONE CUDA device and is not thread-safe: one context per host thread and
 *    device, as in the reference's single-threaded model.
 *  - The caller owns x, y, bias and the stream.  The library owns repacked weights and its scratch.
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *  - Device-pointer entry points are asynchronous on `stream`; *_host entry points copy in, run,
 *    copy out and synchronise before returning.
 *  - Shapes: W is [N = out_features][K = in_features]; x is [M][ldx] (ldx >= K, in elements);
 *    y is [M][ldy] (ldy >= N).  K must be a multiple of the format's block length.
 */
#ifndef TTQ_H
#define TTQ_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define TTQ_API __attribute__((visibility("default")))
#else
#define TTQ_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ttq_ctx ttq_ctx;
typedef struct ttq_weight ttq_weight;
typedef struct ttq_comm ttq_comm;
typedef struct ttq_moe ttq_moe;
typedef struct ttq_host_batch ttq_host_batch;

typedef enum ttq_status {
    TTQ_OK = 0,
    TTQ_ERR_INVALID_ARG = 1, /* null pointer, negative size, unknown enum value */
    TTQ_ERR_SHAPE = 2,       /* K not a multiple of the block length, nbytes mismatch, ld too small */
    TTQ_ERR_UNSUPPORTED = 3, /* valid request this build cannot serve */
    TTQ_ERR_CUDA = 4,        /* a CUDA runtime call failed; see ttq_last_error */
    TTQ_ERR_OOM = 5,         /* device or host allocation failed */
    TTQ_ERR_DEVICE = 6,      /* no sm_100 device / wrong device current */
    TTQ_ERR_LIMIT = 7,       /* request exceeds a fixed capacity (scratch, static buffers) */
    TTQ_ERR_TIMEOUT = 8      /* a kernel gave up a bounded wait (copy pipeline, tensor-core pipeline, absent peer); results invalid */
} ttq_status;

typedef enum ttq_format {
    TTQ_FMT_Q8_0 = 0, /* 32 weights / 34 B: fp16 d, 32 x int8 */
    TTQ_FMT_Q4_K = 1, /* 256 weights / 144 B: fp16 d, fp16 dmin, 12 B of 6-bit scales+mins, 128 B nibbles */
    TTQ_FMT_Q6_K = 2, /* 256 weights / 210 B: 128 B low nibbles, 64 B high 2 bits, 16 x int8 scales, fp16 d */
    /* Trellis-coded 3 bits per weight, Hadamard-rotated input and output (this library's own format in the
     * family a reference configuration fixture names, tests/fixtures/configs/config-GLM-4.7-EXL3-3.84bpw.json:43-54;
     * not interchangeable with other tools' checkpoints).  N and K multiples of 128.  One buffer of
     * N*K*3/8 + 2N + K/8 bytes: tiles [N/16][K/16][96 B] | out_scale [N] fp16 | in_sign [K/8] bytes.
     * Weight t = 16 r + c of a 16x16 tile is coded by the 16-bit window at bit 3t of the tile's 768-bit
     * little-endian stream (zero beyond its end): h = window * 2654435761 mod 2^32,
     * q = (byte0(h) + byte1(h) + byte2(h) + byte3(h) - 510) / 147.8.  The operator is
     * y = out_scale * H_N(q . H_K(in_sign * x)) + bias, H = orthonormal Hadamard transform on blocks of 128.
     * ttq_dequantize returns q (the decoded codes).  ttq_shard is not applied to this format: shard the
     * buffer on the host (rows in multiples of 128, columns in multiples of 128). */
    TTQ_FMT_TQ3 = 3
} ttq_format;

typedef enum ttq_dtype { TTQ_DT_BF16 = 0, TTQ_DT_F16 = 1, TTQ_DT_F32 = 2 } ttq_dtype;

/* Which slice of the full [N][K] matrix a rank keeps (tensor parallelism).  There is no reference
 * counterpart (the reference has no parallelism); the split follows the usual column/row scheme:
 *  COLUMN       rows    [rank*N/world, (rank+1)*N/world)                    -- no collective after
 *  COLUMN_GATED as COLUMN but applied to each half of a fused gate|up weight (mlp.nim:39), so the
 *               shard is [gate_rank ; up_rank] and silu_and_mul stays local
 *  ROW          columns [rank*K/world, (rank+1)*K/world), K/world a multiple of the block length;
 *               outputs of all ranks must be summed (all-reduce) by the caller */
typedef enum ttq_shard_kind {
    TTQ_SHARD_NONE = 0,
    TTQ_SHARD_COLUMN = 1,
    TTQ_SHARD_COLUMN_GATED = 2,
    TTQ_SHARD_ROW = 3
} ttq_shard_kind;

typedef struct ttq_shard {
    int32_t kind; /* ttq_shard_kind */
    int32_t rank;
    int32_t world;
} ttq_shard;

/* ---- context ------------------------------------------------------------------------------ */

/* Creates a context on CUDA device `device` (made current for the call).  Allocates the fixed
 * scratch used by forward.  Fails with TTQ_ERR_DEVICE when the device is not compute capability
 * 10.x: there is no fallback path. */
TTQ_API ttq_status ttq_init(int device, ttq_ctx **out);
TTQ_API ttq_status ttq_destroy(ttq_ctx *ctx);
/* Message of the last failure on this context ("" if none).  Valid until the next call on ctx. */
TTQ_API const char *ttq_last_error(const ttq_ctx *ctx);
TTQ_API const char *ttq_status_string(ttq_status s);
/* Library version, "major.minor.patch". */
TTQ_API const char *ttq_version(void);

/* ---- format facts (host only, no device needed) --------------------------------------------- */

TTQ_API int64_t ttq_block_elems(ttq_format fmt); /* weights per block, 0 for an unknown format */
TTQ_API int64_t ttq_block_bytes(ttq_format fmt); /* bytes per block,   0 for an unknown format */
/* Bytes of canonical blocks for an [N][K] matrix (= the algorithmic weight bytes of one forward). */
TTQ_API int64_t ttq_packed_bytes(ttq_format fmt, int64_t N, int64_t K);

/* ---- weights: Linear.init (linear.nim:29-43) ------------------------------------------------ */

/* host_blocks: canonical row-major blocks, [N][K / block_elems] blocks of block_bytes each (for
 * instance a view into an mmap'ed file, cf. safetensors.nim:256-274 getMmapView); nbytes must equal
 * ttq_packed_bytes(fmt, N, K).  The blocks are uploaded and repacked on the device into the tiled
 * layout; the call returns after the repack finished, the host buffer may then be released.
 * `shard` may be NULL (whole matrix); otherwise only the rank's slice is uploaded and the
 * resulting weight has the slice's N and K. */
TTQ_API ttq_status ttq_weight_create(ttq_ctx *ctx, ttq_format fmt, int64_t N, int64_t K, const void *host_blocks,
                             size_t nbytes, const ttq_shard *shard, ttq_weight **out);
/* Same, with the canonical blocks already in device memory (whole matrix).  Repack runs on
 * `stream`; dev_blocks may be released once the stream has passed this point. */
TTQ_API ttq_status ttq_weight_create_device(ttq_ctx *ctx, ttq_format fmt, int64_t N, int64_t K,
                                    const void *dev_blocks, size_t nbytes, void *stream,
                                    ttq_weight **out);
TTQ_API ttq_status ttq_weight_destroy(ttq_weight *w);
TTQ_API ttq_status ttq_weight_info(const ttq_weight *w, int32_t *fmt, int64_t *N, int64_t *K);
/* Canonical (algorithmic) byte count of this weight, ttq_packed_bytes of its own N and K. */
TTQ_API int64_t ttq_weight_bytes(const ttq_weight *w);

/* Test hook: expands the tiled device layout back to canonical order, fp32 [N][ld] in device
 * memory.  Must reproduce a CPU dequantization of the original blocks bit for bit. */
TTQ_API ttq_status ttq_dequantize(ttq_ctx *ctx, const ttq_weight *w, float *dev_out, int64_t ld, void *stream);

/* ---- forward: Linear.forward (linear.nim:45-57) -------------------------------------------- */

/* y[m][n] = sum_k x[m][k] * W[n][k] (+ bias[n]).  x: bf16 or f16 device matrix; bias: NULL or a
 * device vector of N elements of bias_dt; y: f32, bf16 or f16 device matrix.  Any M >= 0.
 * Decode batches use exact integer products with scales applied in fp32; larger batches expand the weights
 * to fp16 for the tensor cores (fp32 accumulation).  Asynchronous on `stream`, allocates nothing: every
 * scratch buffer was sized when the context and the weights were created -- so create ALL weights before
 * capturing forwards into a CUDA graph (creating a larger Q8_0 / Q6_K / trellis weight later may move the
 * context's expansion scratch, which an already captured graph would still address). */
TTQ_API ttq_status ttq_linear_forward(ttq_ctx *ctx, const ttq_weight *w, const void *x_dev, ttq_dtype x_dt,
                              int64_t M, int64_t ldx, const void *bias_dev, ttq_dtype bias_dt,
                              void *y_dev, ttq_dtype y_dt, int64_t ldy, void *stream);

/* Host-buffer form of the same call, synchronous like the reference's `Linear.forward`
 * (workspace/libtorch/src/workspace/layers/module.nim:8-24 on CPU tensors).  Page-locked buffers of up to 1 MiB in
 * total (decode sizes) are read and written in place through their device mappings; pageable or larger buffers go
 * through the context's pinned staging area (TTQ_ERR_LIMIT beyond its capacity).  Runs on the context's own host
 * stream, waits for it and reports a kernel that gave up a bounded wait (TTQ_ERR_TIMEOUT). */
TTQ_API ttq_status ttq_linear_forward_host(ttq_ctx *ctx, const ttq_weight *w, const void *x_host, ttq_dtype x_dt,
                                   int64_t M, int64_t ldx, const void *bias_host, ttq_dtype bias_dt,
                                   void *y_host, ttq_dtype y_dt, int64_t ldy);

/* The same call without the wait (no counterpart in the reference, whose forward is synchronous): it only enqueues
 * the work on the context's host stream, so that a caller with several linears to run pays one wait per batch
 * of calls instead of one per call.  x, bias and y must be page-locked and at most 1 MiB in total
 * (TTQ_ERR_INVALID_ARG for pageable memory, TTQ_ERR_LIMIT for size); they must stay valid, and y unread, until
 * ttq_host_sync returns.  Calls execute in the order they were made. */
TTQ_API ttq_status ttq_linear_forward_host_async(ttq_ctx *ctx, const ttq_weight *w, const void *x_host, ttq_dtype x_dt,
                                         int64_t M, int64_t ldx, const void *bias_host, ttq_dtype bias_dt,
                                         void *y_host, ttq_dtype y_dt, int64_t ldy);

/* One host-buffer linear of a recorded batch: the arguments of ttq_linear_forward_host. */
typedef struct ttq_host_linear {
    const ttq_weight *w;
    const void *x_host;
    int32_t x_dt;
    int64_t M, ldx;
    const void *bias_host; /* may be NULL */
    int32_t bias_dt;
    void *y_host;
    int32_t y_dt;
    int64_t ldy;
} ttq_host_linear;

/* Records `n` host-buffer linears (a decode step's worth) once, as a CUDA graph on the context's host stream, for
 * callers that run the same linears on the same buffers step after step (no counterpart in the reference).  The
 * buffers are page-locked host memory or device memory; the linears of a batch must not depend on each other (no y
 * of one is the x of another): the decode-size ones run side by side.  The batch runs on the context's own host
 * stream: device buffers must have been written (their producing stream synchronised) before ttq_host_batch_run, and
 * may be read once it has returned.  Same limits per linear as ttq_linear_forward_host_async.  The linears run once during the call
 * (every kernel is configured before the recording starts).  The activations of ALL decode-size linears
 * of the batch (one row; two rows below K = 8192; block formats) are converted by one launch at the head of the
 * graph, straight from the host buffers, so those linears run without an activation pass of their own; the
 * activations of the other linears are copied to the device by one gather launch (Q4_K linears of up to 16 rows then
 * run side by side as well, each forked stream with a K-split workspace of its own; larger ones run in order).  Either way all reads over the host
 * link are in flight together.  Allocates the device storage for both; the results are written to the host buffers
 * by the linears themselves.  Weights and buffers must outlive the batch; create
 * every weight of the context before recording (see ttq_linear_forward on scratch that may move). */
TTQ_API ttq_status ttq_host_batch_create(ttq_ctx *ctx, const ttq_host_linear *linears, int n, ttq_host_batch **out);
/* Runs the recorded linears in order, waits, and reports a kernel that gave up a bounded wait (TTQ_ERR_TIMEOUT):
 * when it returns TTQ_OK every y of the batch is in host memory. */
TTQ_API ttq_status ttq_host_batch_run(ttq_host_batch *batch);
TTQ_API ttq_status ttq_host_batch_destroy(ttq_host_batch *batch);

/* Waits for everything the host entry points have enqueued on this context; TTQ_ERR_TIMEOUT if a kernel of those
 * calls gave up a bounded wait (the results of the batch are invalid then; the flag is cleared). */
TTQ_API ttq_status ttq_host_sync(ttq_ctx *ctx);

/* Synchronises `stream` and reports whether any kernel launched through this context since the last
 * check gave up a bounded device-side wait (TTQ_ERR_TIMEOUT; the flag is cleared).  The *_host entry
 * points perform this check themselves. */
TTQ_API ttq_status ttq_device_status(ttq_ctx *ctx, void *stream);

/* ---- row-parallel linear with the all-reduce fused in (tensor parallelism) --------------------
 * No reference counterpart (the reference has no parallelism).  One process per GPU (or one process driving
 * several, see ttq_comm_connect_pointers).  For a ROW shard the outputs of all ranks must be summed; for
 * decode-size batches the sum is done inside the linear's own kernel: the warp that finishes a 16-row tile
 * writes its partial sums into the exchange buffers of ALL ranks over NVLink as single 8-byte stores of
 * {value, epoch} (plain peer stores on mapped memory, no multicast, no fence, no separate flag: the epoch that
 * validates a value arrives with it), then polls -- bounded -- its own buffer until every rank's cells carry
 * this exchange's epoch and adds them in rank order, so every rank ends with the same full result in y.
 *   ttq_comm_create   allocates this rank's exchange buffer (sized for N <= n_cap, M <= m_cap <= 16) and
 *                     returns its 64-byte CUDA IPC handle in ipc_handle_out;
 *   ttq_comm_connect  takes the handles of ALL ranks (world x 64 bytes, in rank order; exchanged by the
 *                     host, e.g. with an all-gather) and maps the peers' buffers.  All ranks must pass a
 *                     host barrier after connecting and before the first forward;
 *   ttq_linear_forward_allreduce  as ttq_linear_forward on the rank's ROW shard, y = sum over ranks
 *                     (+ bias, added once).  Every rank must issue the same sequence of calls.  Returns
 *                     TTQ_ERR_UNSUPPORTED when M or N exceed the buffer: fall back to ttq_linear_forward
 *                     plus a library all-reduce.  A peer that never arrives ends the wait after a set
 *                     number of polls (ttq_comm_set_wait_limit) and is reported as TTQ_ERR_TIMEOUT by
 *                     ttq_device_status; the kernel returns and the context stays usable. */
TTQ_API ttq_status ttq_comm_create(ttq_ctx *ctx, int rank, int world, int64_t n_cap, int m_cap, ttq_comm **out,
                                   void *ipc_handle_out);
TTQ_API ttq_status ttq_comm_connect(ttq_comm *comm, const void *all_handles);
/* Single-process form of the connection (the reference is one application without a launcher): ttq_comm_local_buffer returns this rank's exchange
 * buffer and its size; ttq_comm_connect_pointers takes, in rank order, device pointers through which THIS
 * rank's device can reach every rank's buffer (peer access enabled by the host; the own entry is ignored).
 * No reference counterpart. */
TTQ_API ttq_status ttq_comm_local_buffer(ttq_comm *comm, void **base_out, size_t *bytes_out);
TTQ_API ttq_status ttq_comm_connect_pointers(ttq_comm *comm, void *const *bases);
/* Number of polls of a peer's cell after which the fused exchange gives up (default 2^22, a few
 * seconds); the give-up is reported as TTQ_ERR_TIMEOUT by ttq_device_status and the context stays usable.
 * No reference counterpart. */
TTQ_API ttq_status ttq_comm_set_wait_limit(ttq_comm *comm, int64_t polls);
TTQ_API ttq_status ttq_comm_destroy(ttq_comm *comm);
TTQ_API ttq_status ttq_linear_forward_allreduce(ttq_ctx *ctx, const ttq_weight *w, const void *x_dev, ttq_dtype x_dt,
                                                int64_t M, int64_t ldx, const void *bias_dev, ttq_dtype bias_dt,
                                                void *y_dev, ttq_dtype y_dt, int64_t ldy, ttq_comm *comm, void *stream);

/* The decode linear for hosts that cannot allocate device memory.  No counterpart in the reference.
 * Some hosts are not allowed to call cudaMalloc at all: a server that has given every byte of device
 * memory to its own pool, or a plug-in under a framework that forbids allocation after start-up.  Such
 * a host cannot create a ttq_ctx (ttq_init allocates scratch and staging buffers).  This call needs no
 * context and allocates nothing: its activation scratch is a fixed 157,760-byte array inside the
 * library image, present on every GPU that loads the library until the process exits.
 *   Limits: M <= 4 and K <= 16384; larger requests return TTQ_ERR_LIMIT (message in errbuf).
 *   The weight's device must be the current device.  x, bias, y and the weight (created elsewhere,
 *   e.g. while loading, by code that may allocate) are passed as for ttq_linear_forward.
 *   The first call on a device looks up the array's device address (cudaGetSymbolAddress, checked)
 *   and the SM count; make that first call before starting any stream capture.
 *   All calls share the one array, which keeps the previous call's contents; every call rewrites what
 *   it reads.  Calls that overlap on the GPU (two streams, two threads) race on it: keep them on one
 *   stream.  Not thread-safe on the host either.
 *   A kernel that gives up a bounded device-side wait records it in a status word inside the array and
 *   carries on with invalid data; the call itself has long returned TTQ_OK by then.  Read the word with
 *   ttq_static_status (below) before trusting y -- after every call, or once per batch of calls.
 *   errbuf (optional) receives a message when the status is not TTQ_OK. */
TTQ_API ttq_status ttq_linear_forward_static(const ttq_weight *w, const void *x_dev, ttq_dtype x_dt, int64_t M,
                                             int64_t ldx, const void *bias_dev, ttq_dtype bias_dt, void *y_dev,
                                             ttq_dtype y_dt, int64_t ldy, void *stream, char *errbuf,
                                             size_t errbuf_len);

/* Companion of ttq_linear_forward_static, equally allocation-free and context-free (no counterpart in the
 * reference): synchronises `stream`, reads the status word of the static array on the current device with one
 * 4-byte copy and returns TTQ_ERR_TIMEOUT (clearing the word) if any ttq_linear_forward_static kernel since
 * the last check gave up a wait, TTQ_OK otherwise. */
TTQ_API ttq_status ttq_static_status(void *stream, char *errbuf, size_t errbuf_len);

/* The down projection of a gated MLP with the activation folded into its input conversion
 * (GatedMLP.forward, workspace/transformers/src/layers/mlp.nim:56-60: silu_and_mul then down_proj):
 * gate_up_dev is [M][ld_gate_up] with 2K used columns [gate | up], y = (silu(gate) * up) . W^T + b.
 * Same conventions as ttq_linear_forward; block formats only (TTQ_ERR_UNSUPPORTED for TTQ_FMT_TQ3). */
TTQ_API ttq_status ttq_linear_forward_gated(ttq_ctx *ctx, const ttq_weight *w, const void *gate_up_dev, ttq_dtype x_dt,
                                            int64_t M, int64_t ld_gate_up, const void *bias_dev, ttq_dtype bias_dt,
                                            void *y_dev, ttq_dtype y_dt, int64_t ldy, void *stream);

/* ---- adjacent step: silu_and_mul (kernels/activations.nim:14-38) ---------------------------- */

/* out[m][h] = silu(in[m][h]) * in[m][H + h]; in is [M][ld_in] with 2H used columns, out [M][ld_out].
 * Same dtype in and out (bf16, f16 or f32). */
TTQ_API ttq_status ttq_silu_and_mul(ttq_ctx *ctx, const void *in_dev, ttq_dtype dt, int64_t M, int64_t H,
                            int64_t ld_in, void *out_dev, int64_t ld_out, void *stream);

/* ---- adjacent steps of a decode layer: residual + RMSNorm, RoPE + KV-cache append, attention ----------
 * 16-bit tensors only (bf16 or f16, one dtype per call), fp32 arithmetic, asynchronous on `stream`. */

/* h[m][:] += delta[m][:] when delta != NULL (the sum is stored back, rounded), then
 * out[m][:] = h[m][:] * rsqrt(mean(h[m][:]^2) + eps) * weight[:].  RmsNorm.forward and forward_with_residual,
 * workspace/transformers/src/layers/norm.nim:23-38 (the reference runs add and norm as separate ops, TODO at :35).
 * H a multiple of 8, rows and weight 16-byte aligned. */
TTQ_API ttq_status ttq_add_rmsnorm(ttq_ctx *ctx, void *h_dev, const void *delta_dev, const void *weight_dev, ttq_dtype dt,
                                   int64_t M, int64_t H, int64_t ld_h, int64_t ld_delta, float eps, void *out_dev,
                                   int64_t ld_out, void *stream);

/* The same step, which in addition converts the M <= 2 output rows into the context's activation scratch in the form
 * the decode kernel reads, so that the linear consuming `out` can be called as ttq_linear_forward_prepared and skip
 * its own conversion pass (one launch and one dependent hand-over less per linear in a decode layer: RmsNorm.forward
 * followed by Linear.forward, transformer.nim:122-156).  H a multiple of 256, at most 8192.  The prepared rows stay
 * valid until the next ttq_linear_forward* / ttq_linear_forward_allreduce call on the context that is not the
 * prepared form (those rewrite the scratch); several prepared linears may consume the same rows.  No reference
 * counterpart: the reference has no quantized activations. */
TTQ_API ttq_status ttq_add_rmsnorm_prepare(ttq_ctx *ctx, void *h_dev, const void *delta_dev, const void *weight_dev, ttq_dtype dt,
                                           int64_t M, int64_t H, int64_t ld_h, int64_t ld_delta, float eps, void *out_dev,
                                           int64_t ld_out, void *stream);

/* Linear.forward (linear.nim:45-57) on the rows the last ttq_add_rmsnorm_prepare on `ctx` left in the scratch:
 * y [M][ldy] = x . W^T + bias with x = that call's `out`.  Block formats only; M and K must match the prepared rows
 * (TTQ_ERR_SHAPE otherwise, TTQ_ERR_INVALID_ARG when nothing is prepared).  Must run on the same stream, after the
 * prepare call.  Results are bit-identical to ttq_linear_forward on `out`. */
TTQ_API ttq_status ttq_linear_forward_prepared(ttq_ctx *ctx, const ttq_weight *w, int64_t M, const void *bias_dev, ttq_dtype bias_dt,
                                               void *y_dev, ttq_dtype y_dt, int64_t ldy, void *stream);

/* Rotary embedding in the rotate-half form (workspace/transformers/src/layers/rope.nim:29-92) of the q and k heads
 * of fused qkv rows [B][ld_qkv] = [hq q heads | hkv k heads | hkv v heads] x d, for ONE position `pos` whose
 * cos / sin vectors [d] the caller supplies; q goes to q_out [B][hq][d], k and v into the caches
 * [B][hkv][ctx_len][d] at `pos` (the preallocated-cache form of attn.nim:97-104). */
TTQ_API ttq_status ttq_rope_kv_append(ttq_ctx *ctx, const void *qkv_dev, ttq_dtype dt, int64_t B, int64_t ld_qkv, int32_t hq,
                                      int32_t hkv, int32_t d, const void *cos_dev, const void *sin_dev, void *q_out_dev,
                                      void *k_cache_dev, void *v_cache_dev, int64_t ctx_len, int64_t pos, void *stream);

/* One query per sequence, grouped-query attention over cache positions 0 .. n_ctx-1 (attn.nim:149-189 at a
 * single new token): out[b][h][:] = softmax_p(q[b][h] . k[b][h / (hq/hkv)][p] / sqrt(d)) . v.  d = 128,
 * hq / hkv in {1, 2, 4, 8}.  TTQ_ERR_LIMIT when B * hq * ceil(n_ctx / 128) exceeds the context's scratch. */
TTQ_API ttq_status ttq_decode_attention(ttq_ctx *ctx, const void *q_dev, const void *k_cache_dev, const void *v_cache_dev,
                                        ttq_dtype dt, int64_t B, int32_t hq, int32_t hkv, int32_t d, int64_t ctx_len,
                                        int64_t n_ctx, void *out_dev, void *stream);

/* ---- mixture-of-experts layer (grouped quantized GEMM) -----------------------------------------
 * No reference counterpart: the reference has dense gated MLPs only
 * (workspace/transformers/src/layers/mlp.nim:31-60).  The layer applies that gated MLP per expert:
 *     y[t] = sum_j w[t][j] * down_e( silu(gate_e x[t]) * up_e x[t] ),  e = topk_ids[t][j]
 * with E experts of identical shape, gate|up fused as one [2I][H] matrix (gate rows first) and down
 * [H][I], all Q4_K.  Router, softmax and top-k selection stay with the caller, who passes the chosen
 * expert ids and their weights.  Routing tables, the routed activation images and the intermediates
 * live in a workspace allocated by ttq_moe_create for up to max_tokens tokens; the forward call
 * allocates nothing, copies nothing to the host and is asynchronous on `stream`.  The handle keeps
 * the experts' device pointers: destroy it before the weights. */
TTQ_API ttq_status ttq_moe_create(ttq_ctx *ctx, int32_t n_experts, const ttq_weight *const *gate_up,
                                  const ttq_weight *const *down, int64_t max_tokens, int32_t top_k, ttq_moe **out);
TTQ_API ttq_status ttq_moe_destroy(ttq_moe *moe);

/* x: [T][ldx] bf16|f16 device rows of H values; topk_ids: [T][top_k] int32 (an id outside 0..E-1
 * drops that choice, which is how an expert-parallel rank skips experts it does not hold);
 * topk_weights: [T][top_k] f32; y: [T][ldy] of H values.  TTQ_ERR_LIMIT when T > max_tokens. */
TTQ_API ttq_status ttq_moe_forward(ttq_ctx *ctx, ttq_moe *moe, const void *x_dev, ttq_dtype x_dt, int64_t T,
                                   int64_t ldx, const int32_t *topk_ids_dev, const float *topk_weights_dev,
                                   void *y_dev, ttq_dtype y_dt, int64_t ldy, void *stream);

/* ---- optional device timeline (tracing) -------------------------------------------------------
 * The reference meters host procedures (workspace/probes/src/tracer.nim:72-133, enabled by a
 * compile-time switch); the counterpart here is a device-side timeline enabled by setting the
 * environment variable TTQ_TRACE=1 before ttq_init.  Every kernel then records, from its first block,
 * eight 64-bit words: kind (1 activation pass, 2 GEMV), start, after the dependency wait, activations
 * ready, first weight tile ready, end of block 0 (all in globaltimer nanoseconds), grid size, N.
 * The tensor-core GEMM records kind 3: start, ns its MMA lane waited for operands, ns it waited for the
 * epilogue, stages issued, end, grid size, N.
 * ttq_trace_read synchronises the device, copies up to max_entries entries (8 words each) into `out`,
 * stores their number in *n_entries and clears the buffer.  With tracing off it reports 0 entries. */
TTQ_API ttq_status ttq_trace_read(ttq_ctx *ctx, uint64_t *out, int64_t max_entries, int64_t *n_entries);

/* ---- introspection for benchmarks ----------------------------------------------------------- */

/* Number of kernels this context has launched since creation (forward, repack, dequantize ...). */
TTQ_API int64_t ttq_launch_count(const ttq_ctx *ctx);

#ifdef __cplusplus
}
#endif
#endif /* TTQ_H */
