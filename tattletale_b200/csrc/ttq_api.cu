// C-ABI entry points of libttq: argument validation, context and weight lifetime, dispatch.
// Nothing here touches weights on the host beyond copying the caller's canonical blocks to the
// device; there is no CPU compute path.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include <vector>

#include "ttq_internal.cuh"

using namespace ttq;

struct ttq_ctx {
    int device;
    char err[512];
    int64_t launches;
    // scratch for the activation planes of the non-fused GEMV path (M <= 16)
    XqView xq;
    int64_t xq_capacity_k;
    void *xq_base;
    int64_t prepared_m, prepared_k;  // rows and row length of the planes ttq_add_rmsnorm_prepare left in `xq` (0: none)
    int sms;          // multiprocessor count of the device
    int *dev_status;  // device word the kernels OR failure bits into (bit 0: a bounded wait gave up)
    int *host_status; // pinned, device-mapped host words: [0] raised by a failing kernel (see report_failure), [1] copy of the status word
    // device mappings of the page-locked host buffers most recently passed to the host entry points
    struct { const void *host; void *dev; } map_cache[1024];  // direct-mapped by address bits
    unsigned long long *trace;  // device timeline buffer, allocated only when TTQ_TRACE=1 is set at init
    float *tq_x1, *tq_y1;       // TQ3: rotated activations [TQ3_SLAB][K] and raw results [TQ3_SLAB][N] (fp32; x1 also
    int64_t tq_x1_cap, tq_y1_cap;  //   holds the fp16 form for the GEMM); capacities in floats, grown at weight creation
    float *att_part;            // partial results of the decode attention slices (fixed at init)
    int64_t att_part_cap;       // in floats
    __half *wimg;               // fp16 expansion of one whole weight (plain GEMM mode of the formats without a
    int64_t wimg_capacity;      //   fused dequant GEMM); in halves, grown when such a weight is created
    __half *xh;                 // fp16 activation scratch of the tcgen05 GEMM path
    int64_t xh_capacity;        // in halves
    float *split_ws;            // fp32 partial sums of decode linears whose K is split across CTAs (fixed at init)
    size_t split_ws_bytes;
    unsigned *split_counters;   // their per-row-tile arrival counters, zero between launches
    int64_t split_counters_cap;
    // device staging for the *_host entry points
    uint8_t *stage_x, *stage_y, *stage_b;
    size_t stage_x_bytes, stage_y_bytes, stage_b_bytes;
    cudaStream_t host_stream;
};

// Exchange area of one tensor-parallel group member (see CommView).
struct ttq_comm {
    ttq_ctx *ctx;
    CommView view;
    void *local;    // this rank's buffer of {value, epoch} cells, exported through CUDA IPC
    size_t bytes;
    void *peer_map[TTQ_MAX_RANKS];  // IPC mappings of the peers' buffers (nullptr for the own rank)
};

// Mixture-of-experts layer: expert weight tables and the workspace of one call (sized at creation).
struct ttq_moe {
    ttq_ctx *ctx;
    int E, top_k;
    int64_t H, I, max_tokens;
    int64_t NT1, SBp1, NT2, SBp2;  // gate|up: [2I][H], down: [H][I]
    int64_t rows_cap;              // routed row capacity: max_tokens * top_k + E * 256
    const uint8_t **d_gate_up, **d_down;  // device arrays of the experts' tiled matrices
    MoeRouting route;
    void *ws;                      // one allocation: routing tables, activation images, intermediates
    __half *xh1, *h1, *xh2, *o2;
};

namespace {

constexpr int64_t XQ_CAPACITY_K = 65536;          // largest K (padded to 256) the scratch planes hold
constexpr size_t STAGE_X_BYTES = 64u << 20;       // host-entry staging: activations
constexpr size_t STAGE_Y_BYTES = 128u << 20;      // host-entry staging: outputs
constexpr size_t STAGE_B_BYTES = 4u << 20;        // host-entry staging: bias
constexpr int64_t XH_CAPACITY = 32ll << 20;       // halves (64 MB): fp16 activations of one GEMM slab
constexpr size_t SPLIT_WS_BYTES = 16u << 20;      // K-split partial sums: 8 slices x 16 rows x 32768 outputs of fp32
constexpr int64_t SPLIT_COUNTERS = 1 << 16;       // row tiles (N <= 1M) a K-split decode linear may have
constexpr int DEFAULT_PEER_WAIT_LIMIT = 1 << 22;  // polls of a peer's counter in the fused row-parallel exchange

ttq_status fail(ttq_ctx *ctx, ttq_status s, const char *fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
        va_end(ap);
    }
    return s;
}

ttq_status cuda_fail(ttq_ctx *ctx, cudaError_t e, const char *what) {
    ttq_status s = (e == cudaErrorMemoryAllocation) ? TTQ_ERR_OOM : TTQ_ERR_CUDA;
    return fail(ctx, s, "%s: %s", what, cudaGetErrorString(e));
}

#define TTQ_CUDA(ctx, call)                                       \
    do {                                                          \
        cudaError_t e__ = (call);                                 \
        if (e__ != cudaSuccess) return cuda_fail(ctx, e__, #call); \
    } while (0)

bool valid_fmt(int f) { return f == TTQ_FMT_Q8_0 || f == TTQ_FMT_Q4_K || f == TTQ_FMT_Q6_K || f == TTQ_FMT_TQ3; }
constexpr int64_t TQ3_GEMV_MAX_M = 4;
constexpr int64_t TQ3_MMA_MAX_M = 64;  // up to here the tensor-core decode kernel beats expansion + GEMM
constexpr int64_t TQ3_SLAB = 512;  // rows of rotated activations / raw results the TQ3 scratch holds
bool valid_dt(int d) { return d == TTQ_DT_BF16 || d == TTQ_DT_F16 || d == TTQ_DT_F32; }
int dt_size(int d) { return d == TTQ_DT_F32 ? 4 : 2; }

ttq_status alloc_weight(ttq_ctx *ctx, int fmt, int64_t N, int64_t K, ttq_weight **out) {
    ttq_weight *w = new (std::nothrow) ttq_weight();
    if (!w) return fail(ctx, TTQ_ERR_OOM, "host allocation of weight handle failed");
    w->ctx = ctx;
    w->device = ctx->device;
    w->fmt = fmt;
    w->N = N;
    w->K = K;
    w->NT = (N + TILE_ROWS - 1) / TILE_ROWS;
    w->SBp = (K + TILE_K - 1) / TILE_K;
    w->tiled_bytes = fmt == TTQ_FMT_TQ3 ? (size_t)tq3_packed_bytes(N, K) : (size_t)w->NT * w->SBp * tile_bytes(fmt);
    w->tiles = nullptr;
    cudaError_t e = cudaMalloc(&w->tiles, w->tiled_bytes);
    if (e != cudaSuccess) {
        delete w;
        return cuda_fail(ctx, e, "cudaMalloc(tiled weight)");
    }
    if (!gemm_supported(fmt)) {
        // (the trellis format) batches beyond the decode kernels run as expansion to fp16 + plain tensor-core GEMM:
        // make sure the context's expansion scratch holds this matrix (load time; forward never allocates)
        const int64_t need = gemm_wimg_rows(N) * w->SBp * TILE_K;
        if (need > ctx->wimg_capacity) {
            cudaDeviceSynchronize();
            cudaFree(ctx->wimg);
            ctx->wimg = nullptr;
            ctx->wimg_capacity = 0;
            e = cudaMalloc(&ctx->wimg, (size_t)need * sizeof(__half));
            if (e != cudaSuccess) {
                cudaFree(w->tiles);
                delete w;
                return cuda_fail(ctx, e, "cudaMalloc(fp16 expansion scratch)");
            }
            ctx->wimg_capacity = need;
        }
    }
    if (fmt == TTQ_FMT_TQ3) {
        auto grow = [&](float **buf, int64_t *cap, int64_t need) -> cudaError_t {
            if (need <= *cap) return cudaSuccess;
            cudaDeviceSynchronize();
            cudaFree(*buf);
            *buf = nullptr;
            *cap = 0;
            cudaError_t ge = cudaMalloc(buf, (size_t)need * sizeof(float));
            if (ge == cudaSuccess) *cap = need;
            return ge;
        };
        e = grow(&ctx->tq_x1, &ctx->tq_x1_cap, TQ3_SLAB * K);
        if (e == cudaSuccess) e = grow(&ctx->tq_y1, &ctx->tq_y1_cap, TQ3_SLAB * N);
        if (e != cudaSuccess) {
            cudaFree(w->tiles);
            delete w;
            return cuda_fail(ctx, e, "cudaMalloc(rotation scratch)");
        }
    }
    *out = w;
    return TTQ_OK;
}

ttq_status check_create_args(ttq_ctx *ctx, int fmt, int64_t N, int64_t K, const void *blocks, size_t nbytes,
                             ttq_weight **out) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    if (!out) return fail(ctx, TTQ_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    if (!blocks) return fail(ctx, TTQ_ERR_INVALID_ARG, "blocks pointer is NULL");
    if (!valid_fmt(fmt)) return fail(ctx, TTQ_ERR_INVALID_ARG, "unknown format %d", fmt);
    if (N <= 0 || K <= 0) return fail(ctx, TTQ_ERR_SHAPE, "N and K must be positive (N=%lld K=%lld)", (long long)N, (long long)K);
    if (K % block_elems(fmt)) return fail(ctx, TTQ_ERR_SHAPE, "K=%lld is not a multiple of the block length %d", (long long)K, block_elems(fmt));
    if (fmt == TTQ_FMT_TQ3 && N % 128) return fail(ctx, TTQ_ERR_SHAPE, "N=%lld is not a multiple of 128 (output rotation block)", (long long)N);
    if ((int64_t)nbytes != ttq_packed_bytes((ttq_format)fmt, N, K))
        return fail(ctx, TTQ_ERR_SHAPE, "nbytes=%zu but an [%lld][%lld] matrix of this format has %lld bytes", nbytes,
                    (long long)N, (long long)K, (long long)ttq_packed_bytes((ttq_format)fmt, N, K));
    return TTQ_OK;
}

// y = out_scale * H_N(q . H_K(in_sign * x)) + bias in slabs of TQ3_SLAB rows: rotate in, multiply (decode kernel
// up to 4 rows, tensor-core decode kernel up to 64, whole-weight expansion + plain tensor-core GEMM beyond), rotate out.
ttq_status tq3_forward(ttq_ctx *ctx, const ttq_weight *w, const void *x_dev, int x_dt, int64_t M, int64_t ldx, const void *bias_dev,
                       int bias_dt, void *y_dev, int y_dt, int64_t ldy, cudaStream_t st) {
    const int64_t N = w->N, K = w->K;
    const uint8_t *packed = w->tiles;
    const __half *oscale = reinterpret_cast<const __half *>(packed + N * K * 3 / 8);
    const uint8_t *isign = packed + N * K * 3 / 8 + 2 * N;
    if (TQ3_SLAB * K > ctx->tq_x1_cap || TQ3_SLAB * N > ctx->tq_y1_cap)
        return fail(ctx, TTQ_ERR_LIMIT, "rotation scratch smaller than this weight needs");
    static const bool use_gemm = []() {
        const char *v = getenv("TTQ_GEMM");
        return !(v && v[0] == '0');
    }();
    // the decode-and-multiply kernel re-decodes every weight per 8 rows; beyond TQ3_GEMV_MAX_M rows one expansion
    // to fp16 and the tensor-core GEMM is cheaper
    // 5 to TQ3_MMA_MAX_M rows: the tensor-core decode kernel (every weight decoded once, no expansion); TTQ_TQ3_MMA=0
    // switches it off
    static const bool use_mma = env_flag("TTQ_TQ3_MMA", true);
    const bool mma = use_mma && M > TQ3_GEMV_MAX_M && M <= TQ3_MMA_MAX_M;
    const bool gemm = !mma && M > TQ3_GEMV_MAX_M && use_gemm && ctx->wimg != nullptr &&
                      gemm_wimg_rows(N) * w->SBp * TILE_K <= ctx->wimg_capacity;
    cudaError_t e;
    if (gemm) {
        e = launch_tq3_wimg(packed, N, K, ctx->wimg, st);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "weight expansion launch");
        ctx->launches++;
    }
    for (int64_t m0 = 0; m0 < M; m0 += TQ3_SLAB) {
        const int64_t Ms = (M - m0) < TQ3_SLAB ? (M - m0) : TQ3_SLAB;
        const uint8_t *xs = reinterpret_cast<const uint8_t *>(x_dev) + (size_t)m0 * ldx * dt_size(x_dt);
        uint8_t *ys = reinterpret_cast<uint8_t *>(y_dev) + (size_t)m0 * ldy * dt_size(y_dt);
        e = launch_tq3_rotate(xs, x_dt, Ms, K, ldx, isign, nullptr, nullptr, TTQ_DT_F32, ctx->tq_x1, (gemm || mma) ? TTQ_DT_F16 : TTQ_DT_F32, K, st, mma);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "input rotation launch");
        ctx->launches++;
        if (gemm) {
            LinearArgs a;
            a.tiles = nullptr;
            a.N = N; a.K = K; a.NT = w->NT; a.SBp = w->SBp;
            a.x = ctx->tq_x1; a.x_dt = TTQ_DT_F16; a.M = Ms; a.ldx = K;
            a.bias = nullptr; a.bias_dt = TTQ_DT_F32;
            a.y = ctx->tq_y1; a.y_dt = TTQ_DT_F32; a.ldy = N;
            int launches = 0;
            e = launch_gemm(w->fmt, a, ctx->xh, ctx->xh_capacity, ctx->sms, ctx->dev_status, ctx->trace, st, &launches, ctx->wimg);
            ctx->launches += launches;
            if (e != cudaSuccess) return cuda_fail(ctx, e, "linear forward (plain GEMM) launch");
        } else if (mma) {
            e = launch_tq3_mma(packed, N, K, reinterpret_cast<const __half *>(ctx->tq_x1), (int)Ms, ctx->tq_y1, st);
            if (e != cudaSuccess) return cuda_fail(ctx, e, "tensor-core decode-and-multiply launch");
            ctx->launches++;
        } else {
            for (int64_t r0 = 0; r0 < Ms; r0 += TQ3_GEMV_MAX_M) {
                const int rows = (int)((Ms - r0) < TQ3_GEMV_MAX_M ? (Ms - r0) : TQ3_GEMV_MAX_M);
                e = launch_tq3_gemv(packed, N, K, ctx->tq_x1 + r0 * K, rows, ctx->tq_y1 + r0 * N, st);
                if (e != cudaSuccess) return cuda_fail(ctx, e, "decode-and-multiply launch");
                ctx->launches++;
            }
        }
        e = launch_tq3_rotate(ctx->tq_y1, TTQ_DT_F32, Ms, N, N, nullptr, oscale, bias_dev, bias_dt, ys, y_dt, ldy, st);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "output rotation launch");
        ctx->launches++;
    }
    return TTQ_OK;
}

}  // namespace

extern "C" {

const char *ttq_version(void) { return "0.1.0"; }

const char *ttq_status_string(ttq_status s) {
    switch (s) {
    case TTQ_OK: return "ok";
    case TTQ_ERR_INVALID_ARG: return "invalid argument";
    case TTQ_ERR_SHAPE: return "shape or size mismatch";
    case TTQ_ERR_UNSUPPORTED: return "unsupported request";
    case TTQ_ERR_CUDA: return "CUDA error";
    case TTQ_ERR_OOM: return "out of memory";
    case TTQ_ERR_DEVICE: return "no usable sm_100 device";
    case TTQ_ERR_LIMIT: return "fixed capacity exceeded";
    case TTQ_ERR_TIMEOUT: return "device-side wait timed out";
    }
    return "unknown status";
}

int64_t ttq_block_elems(ttq_format fmt) { return valid_fmt(fmt) ? block_elems(fmt) : 0; }
int64_t ttq_block_bytes(ttq_format fmt) { return valid_fmt(fmt) ? block_bytes(fmt) : 0; }
int64_t ttq_packed_bytes(ttq_format fmt, int64_t N, int64_t K) {
    if (!valid_fmt(fmt) || N < 0 || K < 0 || K % block_elems(fmt)) return 0;
    if (fmt == TTQ_FMT_TQ3) return N % 128 ? 0 : tq3_packed_bytes(N, K);
    return N * (K / block_elems(fmt)) * block_bytes(fmt);
}

const char *ttq_last_error(const ttq_ctx *ctx) { return ctx ? ctx->err : "null context"; }
int64_t ttq_launch_count(const ttq_ctx *ctx) { return ctx ? ctx->launches : 0; }

ttq_status ttq_init(int device, ttq_ctx **out) {
    if (!out) return TTQ_ERR_INVALID_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        cudaGetLastError();
        return TTQ_ERR_DEVICE;
    }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return TTQ_ERR_DEVICE;
    if (prop.major != 10) return TTQ_ERR_DEVICE;  // kernels are built for sm_100a only
    if (cudaSetDevice(device) != cudaSuccess) return TTQ_ERR_DEVICE;
    ttq_ctx *ctx = new (std::nothrow) ttq_ctx();
    if (!ctx) return TTQ_ERR_OOM;
    memset(ctx, 0, sizeof(*ctx));
    ctx->device = device;
    ctx->sms = prop.multiProcessorCount;
    // scratch: planes [2*16][Kcap] int8, sum16 [16][Kcap/16], sum32 [16][Kcap/32], sx [16][Kcap/256]
    const int64_t Kc = XQ_CAPACITY_K, MP = MAX_GEMV_M;
    const size_t planes_b = (size_t)2 * MP * Kc, s16_b = (size_t)MP * (Kc / 16) * 4, s32_b = (size_t)MP * (Kc / 32) * 4,
                 sx_b = (size_t)MP * (Kc / 256 + 4) * 4;
    cudaError_t e = cudaMalloc(&ctx->xq_base, planes_b + s16_b + s32_b + sx_b);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->dev_status, 1024);  // status word, then 768 zero bytes
    if (e == cudaSuccess) e = cudaMemset(ctx->dev_status, 0, 1024);
    if (e == cudaSuccess) e = cudaHostAlloc(&ctx->host_status, 2 * sizeof(int), cudaHostAllocMapped);
    if (e == cudaSuccess) {
        // words 2..3 of the status area: device-visible address of the host flag
        ctx->host_status[0] = ctx->host_status[1] = 0;
        void *flag_dev = nullptr;
        e = cudaHostGetDevicePointer(&flag_dev, ctx->host_status, 0);
        if (e == cudaSuccess) e = cudaMemcpy(ctx->dev_status + 2, &flag_dev, sizeof(void *), cudaMemcpyHostToDevice);
    }
    const char *tr = getenv("TTQ_TRACE");
    if (e == cudaSuccess && tr && tr[0] == '1') {
        const size_t tb = (size_t)(8 + 8 * TTQ_TRACE_ENTRIES) * sizeof(unsigned long long);
        e = cudaMalloc(&ctx->trace, tb);
        if (e == cudaSuccess) e = cudaMemset(ctx->trace, 0, tb);
    }
    if (e == cudaSuccess) e = cudaMalloc(&ctx->xh, (size_t)XH_CAPACITY * sizeof(__half));
    if (e == cudaSuccess) e = cudaMalloc(&ctx->split_ws, SPLIT_WS_BYTES);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->split_counters, (size_t)SPLIT_COUNTERS * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMemset(ctx->split_counters, 0, (size_t)SPLIT_COUNTERS * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMalloc(&ctx->stage_x, STAGE_X_BYTES);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->stage_y, STAGE_Y_BYTES);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->stage_b, STAGE_B_BYTES);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->host_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        cudaGetLastError();
        ttq_destroy(ctx);
        return e == cudaErrorMemoryAllocation ? TTQ_ERR_OOM : TTQ_ERR_CUDA;
    }
    uint8_t *b = reinterpret_cast<uint8_t *>(ctx->xq_base);
    ctx->xq.planes = reinterpret_cast<int8_t *>(b);
    ctx->xq.sum16 = reinterpret_cast<float *>(b + planes_b);
    ctx->xq.sum32 = reinterpret_cast<float *>(b + planes_b + s16_b);
    ctx->xq.sx = reinterpret_cast<float *>(b + planes_b + s16_b + s32_b);
    ctx->xq_capacity_k = Kc;
    ctx->xh_capacity = XH_CAPACITY;
    ctx->split_ws_bytes = SPLIT_WS_BYTES;
    ctx->split_counters_cap = SPLIT_COUNTERS;
    ctx->att_part_cap = 8ll << 20;  // 32 MB: e.g. 32 sequences x 32 heads x 64 slices of 128 positions
    if (cudaMalloc(&ctx->att_part, (size_t)ctx->att_part_cap * sizeof(float)) != cudaSuccess) {
        ctx->att_part = nullptr;
        ctx->att_part_cap = 0;
        cudaGetLastError();
    }
    ctx->stage_x_bytes = STAGE_X_BYTES;
    ctx->stage_y_bytes = STAGE_Y_BYTES;
    ctx->stage_b_bytes = STAGE_B_BYTES;
    *out = ctx;
    return TTQ_OK;
}

ttq_status ttq_destroy(ttq_ctx *ctx) {
    if (!ctx) return TTQ_OK;
    cudaSetDevice(ctx->device);
    if (ctx->host_stream) cudaStreamDestroy(ctx->host_stream);
    cudaFree(ctx->xq_base);
    cudaFree(ctx->dev_status);
    cudaFreeHost(ctx->host_status);
    cudaFree(ctx->trace);
    cudaFree(ctx->xh);
    cudaFree(ctx->split_ws);
    cudaFree(ctx->split_counters);
    cudaFree(ctx->wimg);
    cudaFree(ctx->tq_x1);
    cudaFree(ctx->tq_y1);
    cudaFree(ctx->att_part);
    cudaFree(ctx->stage_x);
    cudaFree(ctx->stage_y);
    cudaFree(ctx->stage_b);
    delete ctx;
    return TTQ_OK;
}

ttq_status ttq_weight_create_device(ttq_ctx *ctx, ttq_format fmt, int64_t N, int64_t K, const void *dev_blocks,
                                    size_t nbytes, void *stream, ttq_weight **out) {
    ttq_status s = check_create_args(ctx, fmt, N, K, dev_blocks, nbytes, out);
    if (s != TTQ_OK) return s;
    TTQ_CUDA(ctx, cudaSetDevice(ctx->device));
    ttq_weight *w = nullptr;
    if ((s = alloc_weight(ctx, fmt, N, K, &w)) != TTQ_OK) return s;
    if (fmt == TTQ_FMT_TQ3) {
        // kept as it is: tiles of a 16-row band are already contiguous along K
        cudaError_t ce = cudaMemcpyAsync(w->tiles, dev_blocks, w->tiled_bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
        if (ce != cudaSuccess) {
            ttq_weight_destroy(w);
            return cuda_fail(ctx, ce, "copy of the packed buffer");
        }
        *out = w;
        return TTQ_OK;
    }
    cudaError_t e = launch_repack(fmt, reinterpret_cast<const uint8_t *>(dev_blocks), w->tiles, N, K, w->NT, w->SBp,
                                  (cudaStream_t)stream);
    if (e != cudaSuccess) {
        ttq_weight_destroy(w);
        return cuda_fail(ctx, e, "repack launch");
    }
    ctx->launches++;
    *out = w;
    return TTQ_OK;
}

ttq_status ttq_weight_create(ttq_ctx *ctx, ttq_format fmt, int64_t N, int64_t K, const void *host_blocks,
                             size_t nbytes, const ttq_shard *shard, ttq_weight **out) {
    ttq_status s = check_create_args(ctx, fmt, N, K, host_blocks, nbytes, out);
    if (s != TTQ_OK) return s;
    TTQ_CUDA(ctx, cudaSetDevice(ctx->device));
    if (fmt == TTQ_FMT_TQ3) {
        if (shard && shard->kind != TTQ_SHARD_NONE)
            return fail(ctx, TTQ_ERR_UNSUPPORTED, "ttq_shard is not applied to the trellis format: shard the buffer on the host");
        ttq_weight *tw = nullptr;
        if ((s = alloc_weight(ctx, fmt, N, K, &tw)) != TTQ_OK) return s;
        cudaError_t ce = cudaMemcpyAsync(tw->tiles, host_blocks, nbytes, cudaMemcpyHostToDevice, ctx->host_stream);
        if (ce == cudaSuccess) ce = cudaStreamSynchronize(ctx->host_stream);
        if (ce != cudaSuccess) {
            ttq_weight_destroy(tw);
            return cuda_fail(ctx, ce, "upload of the packed buffer");
        }
        *out = tw;
        return TTQ_OK;
    }
    const int64_t be = block_elems(fmt), bb = block_bytes(fmt);
    const int64_t row_bytes = (K / be) * bb;
    const uint8_t *src = reinterpret_cast<const uint8_t *>(host_blocks);
    int64_t Nl = N, Kl = K;
    int kind = shard ? shard->kind : TTQ_SHARD_NONE;
    if (kind != TTQ_SHARD_NONE) {
        if (shard->world <= 0 || shard->rank < 0 || shard->rank >= shard->world)
            return fail(ctx, TTQ_ERR_INVALID_ARG, "bad shard rank %d of %d", shard->rank, shard->world);
        const int64_t P = shard->world;
        if (kind == TTQ_SHARD_COLUMN) {
            if (N % P) return fail(ctx, TTQ_ERR_SHAPE, "N=%lld not divisible by world %lld", (long long)N, (long long)P);
            Nl = N / P;
        } else if (kind == TTQ_SHARD_COLUMN_GATED) {
            if (N % (2 * P)) return fail(ctx, TTQ_ERR_SHAPE, "N=%lld not divisible by 2*world", (long long)N);
            Nl = N / P;
        } else if (kind == TTQ_SHARD_ROW) {
            if (K % (P * be)) return fail(ctx, TTQ_ERR_SHAPE, "K=%lld: K/world must be a multiple of the block length %lld", (long long)K, (long long)be);
            Kl = K / P;
        } else {
            return fail(ctx, TTQ_ERR_INVALID_ARG, "unknown shard kind %d", kind);
        }
    }
    const size_t local_bytes = (size_t)Nl * (Kl / be) * bb;
    uint8_t *staging = nullptr;
    TTQ_CUDA(ctx, cudaMalloc(&staging, local_bytes));
    cudaError_t e = cudaSuccess;
    // All copies are ordered on the same stream as the repack kernel that consumes them.
    cudaStream_t up = ctx->host_stream;
    if (kind == TTQ_SHARD_NONE) {
        e = cudaMemcpyAsync(staging, src, local_bytes, cudaMemcpyHostToDevice, up);
    } else if (kind == TTQ_SHARD_COLUMN) {
        e = cudaMemcpyAsync(staging, src + (size_t)shard->rank * Nl * row_bytes, local_bytes, cudaMemcpyHostToDevice, up);
    } else if (kind == TTQ_SHARD_COLUMN_GATED) {
        const int64_t half = N / 2, hl = Nl / 2;
        e = cudaMemcpyAsync(staging, src + (size_t)(shard->rank * hl) * row_bytes, (size_t)hl * row_bytes,
                            cudaMemcpyHostToDevice, up);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(staging + (size_t)hl * row_bytes, src + (size_t)(half + shard->rank * hl) * row_bytes,
                                (size_t)hl * row_bytes, cudaMemcpyHostToDevice, up);
    } else {
        const size_t lrow = (size_t)(Kl / be) * bb;
        e = cudaMemcpy2DAsync(staging, lrow, src + (size_t)shard->rank * lrow, row_bytes, lrow, (size_t)N,
                              cudaMemcpyHostToDevice, up);
    }
    if (e != cudaSuccess) {
        cudaFree(staging);
        return cuda_fail(ctx, e, "upload of canonical blocks");
    }
    ttq_weight *w = nullptr;
    if ((s = alloc_weight(ctx, fmt, Nl, Kl, &w)) != TTQ_OK) {
        cudaFree(staging);
        return s;
    }
    e = launch_repack(fmt, staging, w->tiles, Nl, Kl, w->NT, w->SBp, ctx->host_stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->host_stream);
    cudaFree(staging);
    if (e != cudaSuccess) {
        ttq_weight_destroy(w);
        return cuda_fail(ctx, e, "repack");
    }
    ctx->launches++;
    *out = w;
    return TTQ_OK;
}

ttq_status ttq_weight_destroy(ttq_weight *w) {
    if (!w) return TTQ_OK;
    if (w->ctx) cudaSetDevice(w->ctx->device);
    cudaFree(w->tiles);
    delete w;
    return TTQ_OK;
}

ttq_status ttq_weight_info(const ttq_weight *w, int32_t *fmt, int64_t *N, int64_t *K) {
    if (!w) return TTQ_ERR_INVALID_ARG;
    if (fmt) *fmt = w->fmt;
    if (N) *N = w->N;
    if (K) *K = w->K;
    return TTQ_OK;
}

int64_t ttq_weight_bytes(const ttq_weight *w) { return w ? ttq_packed_bytes((ttq_format)w->fmt, w->N, w->K) : 0; }

ttq_status ttq_dequantize(ttq_ctx *ctx, const ttq_weight *w, float *dev_out, int64_t ld, void *stream) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    if (!w || !dev_out) return fail(ctx, TTQ_ERR_INVALID_ARG, "weight or output pointer is NULL");
    if (w->ctx != ctx) return fail(ctx, TTQ_ERR_INVALID_ARG, "weight belongs to another context");
    if (ld < w->K) return fail(ctx, TTQ_ERR_SHAPE, "ld=%lld < K=%lld", (long long)ld, (long long)w->K);
    cudaError_t e = w->fmt == TTQ_FMT_TQ3 ? launch_tq3_decode(w->tiles, w->N, w->K, dev_out, ld, (cudaStream_t)stream)
                                          : launch_dequant(w->fmt, w->tiles, dev_out, ld, w->N, w->K, w->SBp, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "dequantize launch");
    ctx->launches++;
    return TTQ_OK;
}

static ttq_status linear_forward_impl(ttq_ctx *ctx, const ttq_weight *w, const void *x_dev, ttq_dtype x_dt, int64_t M,
                              int64_t ldx, const void *bias_dev, ttq_dtype bias_dt, void *y_dev, ttq_dtype y_dt,
                              int64_t ldy, void *stream, bool gated) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    ctx->prepared_m = 0;  // the activation scratch may be rewritten below
    if (!w) return fail(ctx, TTQ_ERR_INVALID_ARG, "weight is NULL");
    if (w->ctx != ctx) return fail(ctx, TTQ_ERR_INVALID_ARG, "weight belongs to another context");
    if (M < 0) return fail(ctx, TTQ_ERR_SHAPE, "M=%lld is negative", (long long)M);
    if (M == 0) return TTQ_OK;
    if (!x_dev || !y_dev) return fail(ctx, TTQ_ERR_INVALID_ARG, "x or y pointer is NULL");
    if (x_dt != TTQ_DT_BF16 && x_dt != TTQ_DT_F16) return fail(ctx, TTQ_ERR_INVALID_ARG, "x dtype must be bf16 or f16");
    if (!valid_dt(y_dt)) return fail(ctx, TTQ_ERR_INVALID_ARG, "unknown y dtype %d", (int)y_dt);
    if (bias_dev && !valid_dt(bias_dt)) return fail(ctx, TTQ_ERR_INVALID_ARG, "unknown bias dtype %d", (int)bias_dt);
    if (ldx < (gated ? 2 : 1) * w->K)
        return fail(ctx, TTQ_ERR_SHAPE, "ldx=%lld < %s=%lld", (long long)ldx, gated ? "2K" : "K", (long long)((gated ? 2 : 1) * w->K));
    if (gated && w->fmt == TTQ_FMT_TQ3) return fail(ctx, TTQ_ERR_UNSUPPORTED, "the gated form serves the block formats");
    if (ldy < w->N) return fail(ctx, TTQ_ERR_SHAPE, "ldy=%lld < N=%lld", (long long)ldy, (long long)w->N);
    if (w->SBp * TILE_K > ctx->xq_capacity_k)
        return fail(ctx, TTQ_ERR_LIMIT, "K=%lld exceeds the activation scratch capacity %lld", (long long)w->K,
                    (long long)ctx->xq_capacity_k);
    cudaStream_t st = (cudaStream_t)stream;
    if (w->fmt == TTQ_FMT_TQ3) return tq3_forward(ctx, w, x_dev, x_dt, M, ldx, bias_dev, bias_dt, y_dev, y_dt, ldy, st);
    LinearArgs a;
    a.tiles = w->tiles;
    a.N = w->N; a.K = w->K; a.NT = w->NT; a.SBp = w->SBp;
    a.x_dt = x_dt; a.ldx = ldx;
    a.bias = bias_dev; a.bias_dt = bias_dt;
    a.y_dt = y_dt; a.ldy = ldy;
    a.gated = gated;
    static const bool use_gemm = []() {
        const char *v = getenv("TTQ_GEMM");
        return !(v && v[0] == '0');
    }();
    // Q4_K, up to 8 rows: the integer tensor-memory kernel (TTQ_Q4K_UMMA=1; the maximum batch it takes is
    // TTQ_Q4K_UMMA_MAX_M, default 8)
    static const bool use_umma = env_flag("TTQ_Q4K_UMMA", false);
    static const int64_t umma_max_m = []() -> int64_t {
        const char *v = getenv("TTQ_Q4K_UMMA_MAX_M");
        const int64_t n = v ? atoll(v) : 8;
        return n < 0 ? 0 : (n > 8 ? 8 : n);
    }();
    if (w->fmt == TTQ_FMT_Q4_K && use_umma && M <= umma_max_m) {
        a.x = x_dev; a.M = M; a.y = y_dev;
        int launches = 0;
        cudaError_t e = launch_q4k_umma(a, ctx->xq, ctx->xq_capacity_k, ctx->sms, ctx->dev_status, ctx->trace, ctx->split_ws,
                                        ctx->split_ws_bytes, ctx->split_counters, ctx->split_counters_cap, st, &launches);
        ctx->launches += launches;
        if (e == cudaSuccess) return TTQ_OK;
        if (e != cudaErrorNotSupported) return cuda_fail(ctx, e, "linear forward (Q4_K tensor-memory decode) launch");
    }
    // Q4_K batches of 3 to 16 rows: one kernel (fp16 tensor-core instructions on exact integer operands, activations
    // converted inside the kernel).  Up to 2 rows the integer decode kernel below is faster, beyond 16 the tcgen05 path.
    // TTQ_Q4K_MMA=0 switches the kernel off.
    static const bool use_mma = env_flag("TTQ_Q4K_MMA", true);
    // (two rows of a long K -- 8192 and more -- also go there: their planes leave room for one small CTA per SM only in
    // the integer kernel; measured 17.3 against 21.1 us on 14336 -> 4096)
    constexpr int64_t MMA_MIN_M = 3, MMA_MAX_M = 16;
    if (w->fmt == TTQ_FMT_Q4_K && use_mma && (M >= MMA_MIN_M || (M == 2 && w->SBp >= 32)) && M <= MMA_MAX_M) {
        a.x = x_dev; a.M = M; a.y = y_dev;
        int launches = 0;
        cudaError_t e = launch_q4k_mma(a, ctx->sms, ctx->dev_status, ctx->trace, ctx->split_ws, ctx->split_ws_bytes, ctx->split_counters,
                                       ctx->split_counters_cap, st, &launches);
        ctx->launches += launches;
        if (e == cudaSuccess) return TTQ_OK;
        if (e != cudaErrorNotSupported) return cuda_fail(ctx, e, "linear forward (Q4_K decode) launch");
        // shape outside the kernel's plans: the other paths below
    }
    // crossover between the decode kernel of the other formats (per-row MMA sets) and the tensor-core path
    // (TTQ_GEMM_MIN_M overrides)
    static const int64_t GEMM_MIN_M = []() -> int64_t {
        const char *v = getenv("TTQ_GEMM_MIN_M");
        const int64_t n = v ? atoll(v) : 0;
        return n >= 1 ? n : 5;
    }();
    // Q8_0 / Q6_K: the integer decode kernel serves 16 rows per pass; from 9 rows the fused tensor-core GEMM is used
    const int64_t gemm_min_m = w->fmt == TTQ_FMT_Q4_K ? GEMM_MIN_M : (GEMM_MIN_M > 9 ? GEMM_MIN_M : 9);
    if (M >= gemm_min_m && use_gemm && gemm_supported(w->fmt)) {
        // prefill / larger batches: tensor-core path
        a.x = x_dev; a.M = M; a.y = y_dev;
        int launches = 0;
        cudaError_t e = launch_gemm(w->fmt, a, ctx->xh, ctx->xh_capacity, ctx->sms, ctx->dev_status, ctx->trace, st, &launches);
        ctx->launches += launches;
        if (e != cudaSuccess) return cuda_fail(ctx, e, "linear forward (GEMM) launch");
        return TTQ_OK;
    }
    // decode path; more rows than one pass holds are processed in groups of MAX_GEMV_M
    for (int64_t m0 = 0; m0 < M; m0 += MAX_GEMV_M) {
        a.x = reinterpret_cast<const uint8_t *>(x_dev) + (size_t)m0 * ldx * dt_size(x_dt);
        a.M = (M - m0) < MAX_GEMV_M ? (M - m0) : MAX_GEMV_M;
        a.y = reinterpret_cast<uint8_t *>(y_dev) + (size_t)m0 * ldy * dt_size(y_dt);
        int launches = 0;
        cudaError_t e = launch_gemv(w->fmt, a, ctx->xq, ctx->xq_capacity_k, reinterpret_cast<const uint8_t *>(ctx->dev_status) + 256, ctx->sms,
                                    ctx->dev_status, ctx->trace, st, &launches);
        ctx->launches += launches;
        if (e != cudaSuccess) return cuda_fail(ctx, e, "linear forward launch");
    }
    return TTQ_OK;
}

ttq_status ttq_linear_forward(ttq_ctx *ctx, const ttq_weight *w, const void *x_dev, ttq_dtype x_dt, int64_t M, int64_t ldx,
                              const void *bias_dev, ttq_dtype bias_dt, void *y_dev, ttq_dtype y_dt, int64_t ldy, void *stream) {
    return linear_forward_impl(ctx, w, x_dev, x_dt, M, ldx, bias_dev, bias_dt, y_dev, y_dt, ldy, stream, false);
}

ttq_status ttq_linear_forward_gated(ttq_ctx *ctx, const ttq_weight *w, const void *gate_up_dev, ttq_dtype x_dt, int64_t M,
                                    int64_t ld_gate_up, const void *bias_dev, ttq_dtype bias_dt, void *y_dev, ttq_dtype y_dt,
                                    int64_t ldy, void *stream) {
    return linear_forward_impl(ctx, w, gate_up_dev, x_dt, M, ld_gate_up, bias_dev, bias_dt, y_dev, y_dt, ldy, stream, true);
}

namespace {

// Device-side addresses of the buffers of the host entry points: the mapping of a page-locked host buffer, a device
// pointer as it is (nullptr for pageable memory).  The driver query costs about a
// microsecond per pointer: buffers that come back call after call are remembered.
void *host_mapping(ttq_ctx *ctx, const void *p) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    auto &slot = ctx->map_cache[((a >> 6) ^ (a >> 16)) & 1023];
    if (slot.host == p) return slot.dev;
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    // page-locked host memory through its device mapping; device (or managed) memory as it is
    if (at.type != cudaMemoryTypeHost && at.type != cudaMemoryTypeDevice && at.type != cudaMemoryTypeManaged) return nullptr;
    slot = {p, at.devicePointer};
    return at.devicePointer;
}

// Waits for the context's host stream; a kernel that gave up a bounded wait has raised the mapped host flag by then.
ttq_status host_stream_sync(ttq_ctx *ctx) {
    cudaStream_t st = ctx->host_stream;
    TTQ_CUDA(ctx, cudaStreamSynchronize(st));
    if (*reinterpret_cast<volatile int *>(ctx->host_status) != 0) {
        ctx->host_status[0] = 0;
        TTQ_CUDA(ctx, cudaMemcpyAsync(ctx->host_status + 1, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost, st));
        TTQ_CUDA(ctx, cudaStreamSynchronize(st));
        const int seen = ctx->host_status[1];
        cudaMemsetAsync(ctx->dev_status, 0, sizeof(int), st);
        cudaMemsetAsync(ctx->split_counters, 0, (size_t)ctx->split_counters_cap * sizeof(unsigned), st);
        return fail(ctx, TTQ_ERR_TIMEOUT, "a kernel gave up a bounded wait (status word 0x%x); results of that call are invalid", seen);
    }
    return TTQ_OK;
}

// Shared body of the host-buffer entry points.  `wait`: synchronise before returning (pageable buffers are allowed
// then and go through the staging copies); without it the buffers must be page-locked and small enough to be read
// and written in place over the host link.
ttq_status forward_host_impl(ttq_ctx *ctx, const ttq_weight *w, const void *x_host, ttq_dtype x_dt, int64_t M, int64_t ldx,
                             const void *bias_host, ttq_dtype bias_dt, void *y_host, ttq_dtype y_dt, int64_t ldy, bool wait) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    if (!w) return fail(ctx, TTQ_ERR_INVALID_ARG, "weight is NULL");
    if (M < 0) return fail(ctx, TTQ_ERR_SHAPE, "M=%lld is negative", (long long)M);
    if (M == 0) return TTQ_OK;
    if (!x_host || !y_host) return fail(ctx, TTQ_ERR_INVALID_ARG, "x or y pointer is NULL");
    if (!valid_dt(x_dt) || !valid_dt(y_dt)) return fail(ctx, TTQ_ERR_INVALID_ARG, "unknown dtype");
    if (ldx < w->K || ldy < w->N) return fail(ctx, TTQ_ERR_SHAPE, "leading dimension smaller than the row length");
    const size_t xb = (size_t)M * ldx * dt_size(x_dt), yb = (size_t)M * ldy * dt_size(y_dt);
    const size_t bbytes = bias_host ? (size_t)w->N * dt_size(bias_dt) : 0;
    if (xb > ctx->stage_x_bytes || yb > ctx->stage_y_bytes || bbytes > ctx->stage_b_bytes)
        return fail(ctx, TTQ_ERR_LIMIT, "host-entry staging capacity exceeded (x %zu B, y %zu B)", xb, yb);
    TTQ_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaStream_t st = ctx->host_stream;
    // Decode-size calls on page-locked buffers skip the staging copies: the kernels read x and write y through
    // the buffers' device mappings (8-60 KB over the host link), which leaves one small copy (the status word)
    // and one synchronisation per call.  Pageable buffers and larger transfers go through the staging copies.
    const void *x_map = nullptr, *b_map = nullptr;
    void *y_map = nullptr;
    bool direct = xb + yb + bbytes <= (1u << 20);
    if (direct) {
        x_map = host_mapping(ctx, x_host);
        y_map = host_mapping(ctx, y_host);
        if (bias_host) b_map = host_mapping(ctx, bias_host);
        direct = x_map && y_map && (!bias_host || b_map);
    }
    if (!wait && !direct)
        return fail(ctx, xb + yb + bbytes <= (1u << 20) ? TTQ_ERR_INVALID_ARG : TTQ_ERR_LIMIT,
                    "the asynchronous host entry needs page-locked buffers of at most 1 MiB in total (x %zu B, y %zu B)", xb, yb);
    ttq_status s;
    if (direct) {
        s = ttq_linear_forward(ctx, w, x_map, x_dt, M, ldx, b_map, bias_dt, y_map, y_dt, ldy, st);
        if (s != TTQ_OK) return s;
    } else {
        TTQ_CUDA(ctx, cudaMemcpyAsync(ctx->stage_x, x_host, xb, cudaMemcpyHostToDevice, st));
        if (bias_host) TTQ_CUDA(ctx, cudaMemcpyAsync(ctx->stage_b, bias_host, bbytes, cudaMemcpyHostToDevice, st));
        s = ttq_linear_forward(ctx, w, ctx->stage_x, x_dt, M, ldx, bias_host ? ctx->stage_b : nullptr, bias_dt, ctx->stage_y, y_dt,
                               ldy, st);
        if (s != TTQ_OK) return s;
        TTQ_CUDA(ctx, cudaMemcpyAsync(y_host, ctx->stage_y, yb, cudaMemcpyDeviceToHost, st));
    }
    return wait ? host_stream_sync(ctx) : TTQ_OK;
}

}  // namespace

ttq_status ttq_linear_forward_host(ttq_ctx *ctx, const ttq_weight *w, const void *x_host, ttq_dtype x_dt, int64_t M,
                                   int64_t ldx, const void *bias_host, ttq_dtype bias_dt, void *y_host, ttq_dtype y_dt,
                                   int64_t ldy) {
    return forward_host_impl(ctx, w, x_host, x_dt, M, ldx, bias_host, bias_dt, y_host, y_dt, ldy, true);
}

ttq_status ttq_linear_forward_host_async(ttq_ctx *ctx, const ttq_weight *w, const void *x_host, ttq_dtype x_dt, int64_t M,
                                         int64_t ldx, const void *bias_host, ttq_dtype bias_dt, void *y_host, ttq_dtype y_dt,
                                         int64_t ldy) {
    return forward_host_impl(ctx, w, x_host, x_dt, M, ldx, bias_host, bias_dt, y_host, y_dt, ldy, false);
}

struct ttq_host_batch {
    ttq_ctx *ctx;
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    void *stage;   // device copies of the activations of the linears that run their own activation pass (gather kernel)
    void *table;   // device array of HostGatherItem
    void *planes;  // converted activations of the decode-size linears (batched activation pass)
    void *xitems;  // device array of XprepBatchItem
    void *side_ws;        // per side stream: K-split partial sums of the one-launch Q4_K decode kernel ...
    void *side_counters;  // ... and its arrival counters (zero between launches)
};

namespace {

struct HostGatherItem {
    const void *src;  // device mapping of a page-locked host buffer
    void *dst;        // its place in the batch's staging area
    unsigned long long bytes;
};

// grid (pieces, items): the activations of all linears of a recorded batch come over the host link in one kernel, with
// every read in flight at once, instead of one dependent round trip at the start of each linear's activation pass.
__global__ void __launch_bounds__(256) host_gather_kernel(const HostGatherItem *__restrict__ items) {
    const HostGatherItem it = items[blockIdx.y];
    const bool vec = ((reinterpret_cast<uintptr_t>(it.src) | reinterpret_cast<uintptr_t>(it.dst) | it.bytes) & 15) == 0;
    if (vec) {
        const unsigned long long n16 = it.bytes / 16;
        for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (unsigned long long)gridDim.x * blockDim.x)
            reinterpret_cast<uint4 *>(it.dst)[i] = reinterpret_cast<const uint4 *>(it.src)[i];
    } else {
        for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < it.bytes; i += (unsigned long long)gridDim.x * blockDim.x)
            reinterpret_cast<uint8_t *>(it.dst)[i] = reinterpret_cast<const uint8_t *>(it.src)[i];
    }
}

void host_batch_free(ttq_host_batch *b) {
    if (b->exec) cudaGraphExecDestroy(b->exec);
    if (b->graph) cudaGraphDestroy(b->graph);
    cudaFree(b->stage);
    cudaFree(b->table);
    cudaFree(b->planes);
    cudaFree(b->xitems);
    cudaFree(b->side_ws);
    cudaFree(b->side_counters);
    delete b;
}

}  // namespace

ttq_status ttq_host_batch_create(ttq_ctx *ctx, const ttq_host_linear *linears, int n, ttq_host_batch **out) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    if (!out) return fail(ctx, TTQ_ERR_INVALID_ARG, "output pointer is NULL");
    *out = nullptr;
    if (!linears || n <= 0 || n > 65535) return fail(ctx, TTQ_ERR_INVALID_ARG, "a batch holds 1 to 65535 linears");
    TTQ_CUDA(ctx, cudaSetDevice(ctx->device));
    // first pass outside the recording, straight on the host buffers: argument errors surface here, every kernel's
    // attributes are set, and every buffer's device mapping is known afterwards
    for (int i = 0; i < n; i++) {
        const ttq_host_linear &l = linears[i];
        ttq_status s = forward_host_impl(ctx, l.w, l.x_host, (ttq_dtype)l.x_dt, l.M, l.ldx, l.bias_host, (ttq_dtype)l.bias_dt, l.y_host,
                                         (ttq_dtype)l.y_dt, l.ldy, false);
        if (s != TTQ_OK) return s;
    }
    ttq_status s = host_stream_sync(ctx);
    if (s != TTQ_OK) return s;
    ttq_host_batch *b = new (std::nothrow) ttq_host_batch();
    if (!b) return fail(ctx, TTQ_ERR_OOM, "out of host memory");
    b->ctx = ctx;
    // Decode-size linears of the block formats (the ones ttq_linear_forward serves with the GEMV) get their activations
    // converted by ONE launch for the whole batch, straight from the host buffers; the others get theirs copied to a
    // staging area by one gather launch and run their own activation pass.
    std::vector<HostGatherItem> items;
    std::vector<XprepBatchItem> xitems;
    std::vector<int> slot((size_t)n);  // index into xitems (>= 0) or -1 - index into items
    std::vector<char> one_launch((size_t)n, 0);  // Q4_K batches of the one-launch decode kernel: staged x, side stream
    std::vector<size_t> offs;
    size_t stage_total = 0, longest = 0, planes_total = 0;
    int total_units = 0;
    auto take = [](size_t &total, size_t bytes) {
        const size_t at = total;
        total += (bytes + 255) & ~(size_t)255;
        return at;
    };
    for (int i = 0; i < n; i++) {
        const ttq_host_linear &l = linears[i];
        const void *x_map = host_mapping(ctx, l.x_host);  // (the first pass has already refused pageable buffers)
        const size_t xb = (size_t)l.M * l.ldx * dt_size((ttq_dtype)l.x_dt);
        // one row always; two rows below K = 8192 (as in ttq_linear_forward); three and four rows only for weights of up to
        // 24 MB, where the small GEMV CTAs of neighbouring launches share the SMs (measured in batches: 4096 -> 4096 at four
        // rows 5.7 against 8.9 us with the one-launch kernel, 4096 -> 28672 27.8 against 22.5)
        const size_t packed = l.w->tiled_bytes;
        const bool decode = (l.M == 1 || (l.M == 2 && l.w->SBp < 32) || (l.M <= 4 && l.w->SBp < 32 && packed <= (24u << 20))) &&
                            gemv_prepared_supported(l.w->fmt, l.M, l.w->SBp);
        if (decode) {
            const int64_t Kp = l.w->SBp * TILE_K;
            XprepBatchItem it;
            it.x = x_map; it.x_dt = l.x_dt; it.M = (int)l.M; it.K = l.w->K; it.ldx = l.ldx; it.SBp = l.w->SBp;
            // (offsets for now; turned into pointers once the buffer exists)
            it.xq.planes = reinterpret_cast<int8_t *>(take(planes_total, (size_t)2 * l.M * Kp));
            it.xq.sum16 = reinterpret_cast<float *>(take(planes_total, (size_t)l.M * (Kp / 16) * sizeof(float)));
            it.xq.sum32 = reinterpret_cast<float *>(take(planes_total, (size_t)l.M * (Kp / 32) * sizeof(float)));
            it.xq.sx = reinterpret_cast<float *>(take(planes_total, (size_t)l.M * sx_stride(l.w->SBp) * sizeof(float)));
            it.unit0 = total_units;
            total_units += (int)(l.M * l.w->SBp);
            slot[i] = (int)xitems.size();
            xitems.push_back(it);
        } else {
            HostGatherItem it;
            it.src = x_map;
            it.dst = reinterpret_cast<void *>(take(stage_total, xb));
            it.bytes = xb;
            longest = xb > longest ? xb : longest;
            slot[i] = -1 - (int)items.size();
            items.push_back(it);
            one_launch[i] = l.w->fmt == TTQ_FMT_Q4_K && l.M <= 16 && (l.M >= 3 || (l.M == 2 && l.w->SBp >= 32));
        }
    }
    bool any_one_launch = false;
    for (int i = 0; i < n; i++) any_one_launch = any_one_launch || one_launch[i];
    cudaError_t e = cudaSuccess;
    if (!items.empty()) {
        e = cudaMalloc(&b->stage, stage_total);
        if (e == cudaSuccess) e = cudaMalloc(&b->table, items.size() * sizeof(HostGatherItem));
        for (auto &it : items) it.dst = reinterpret_cast<uint8_t *>(b->stage) + reinterpret_cast<uintptr_t>(it.dst);
        if (e == cudaSuccess) e = cudaMemcpy(b->table, items.data(), items.size() * sizeof(HostGatherItem), cudaMemcpyHostToDevice);
    }
    if (e == cudaSuccess && !xitems.empty()) {
        e = cudaMalloc(&b->planes, planes_total);
        if (e == cudaSuccess) e = cudaMalloc(&b->xitems, xitems.size() * sizeof(XprepBatchItem));
        uint8_t *base = reinterpret_cast<uint8_t *>(b->planes);
        for (auto &it : xitems) {
            it.xq.planes = reinterpret_cast<int8_t *>(base + reinterpret_cast<uintptr_t>(it.xq.planes));
            it.xq.sum16 = reinterpret_cast<float *>(base + reinterpret_cast<uintptr_t>(it.xq.sum16));
            it.xq.sum32 = reinterpret_cast<float *>(base + reinterpret_cast<uintptr_t>(it.xq.sum32));
            it.xq.sx = reinterpret_cast<float *>(base + reinterpret_cast<uintptr_t>(it.xq.sx));
        }
        if (e == cudaSuccess) e = cudaMemcpy(b->xitems, xitems.data(), xitems.size() * sizeof(XprepBatchItem), cudaMemcpyHostToDevice);
    }
    if (e != cudaSuccess) {
        host_batch_free(b);
        return cuda_fail(ctx, e, "host batch staging");
    }
    // side streams of the recording (see below) and what they need, settled before the recording starts
    static const int n_side_env = []() {
        const char *v = getenv("TTQ_HOST_BATCH_STREAMS");
        return v ? atoi(v) : 4;
    }();
    constexpr int MAX_SIDE = 8;
    int side_work = (int)xitems.size();
    for (int i = 0; i < n; i++) side_work += one_launch[i];
    const int n_side = side_work < 2 ? 1 : (n_side_env < 1 ? 1 : (n_side_env > MAX_SIDE ? MAX_SIDE : n_side_env));
    if (any_one_launch && n_side > 1) {
        // the one-launch decode kernel sums K-split partials through a workspace: one per side stream (the linears of a
        // stream run in order)
        e = cudaMalloc(&b->side_ws, (size_t)n_side * SPLIT_WS_BYTES);
        if (e == cudaSuccess) e = cudaMalloc(&b->side_counters, (size_t)n_side * SPLIT_COUNTERS * sizeof(unsigned));
        if (e == cudaSuccess) e = cudaMemsetAsync(b->side_counters, 0, (size_t)n_side * SPLIT_COUNTERS * sizeof(unsigned), nullptr);
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        if (e != cudaSuccess) {
            host_batch_free(b);
            return cuda_fail(ctx, e, "host batch workspaces");
        }
    }
    e = cudaStreamBeginCapture(ctx->host_stream, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) {
        host_batch_free(b);
        return fail(ctx, TTQ_ERR_CUDA, "cudaStreamBeginCapture: %s", cudaGetErrorString(e));
    }
    s = TTQ_OK;
    if (!items.empty()) {
        const unsigned pieces = (unsigned)((longest / 16 + 255) / 256 > 0 ? (longest / 16 + 255) / 256 : 1);
        host_gather_kernel<<<dim3(pieces < 64 ? pieces : 64, (unsigned)items.size()), 256, 0, ctx->host_stream>>>(
            reinterpret_cast<const HostGatherItem *>(b->table));
    }
    if (!xitems.empty()) {
        e = launch_xprep_batch(reinterpret_cast<const XprepBatchItem *>(b->xitems), (int)xitems.size(), total_units, ctx->host_stream);
        if (e != cudaSuccess) s = cuda_fail(ctx, e, "batched activation pass launch");
    }
    // The decode-size linears depend on the batched activation pass only, not on each other (their planes and outputs are
    // their own): they are recorded round-robin on a few side streams that fork from the head of the graph, so that the
    // last CTAs of one linear and the first of the next run side by side instead of a dependent launch apart.
    // TTQ_HOST_BATCH_STREAMS (default 4, 1 = one chain).  The other linears share the context's scratch and stay in line.
    cudaStream_t side[MAX_SIDE] = {};
    cudaEvent_t fork_ev = nullptr, join_ev[MAX_SIDE] = {};
    if (n_side > 1) {
        e = cudaEventCreateWithFlags(&fork_ev, cudaEventDisableTiming);
        for (int k = 0; e == cudaSuccess && k < n_side; k++) {
            e = cudaStreamCreateWithFlags(&side[k], cudaStreamNonBlocking);
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&join_ev[k], cudaEventDisableTiming);
        }
        if (e == cudaSuccess) e = cudaEventRecord(fork_ev, ctx->host_stream);
        for (int k = 0; e == cudaSuccess && k < n_side; k++) e = cudaStreamWaitEvent(side[k], fork_ev, 0);
        if (e != cudaSuccess) s = cuda_fail(ctx, e, "host batch side streams");
    }
    int next_side = 0;
    for (int i = 0; s == TTQ_OK && i < n; i++) {
        const ttq_host_linear &l = linears[i];
        const void *b_map = l.bias_host ? host_mapping(ctx, l.bias_host) : nullptr;
        void *y_map = host_mapping(ctx, l.y_host);
        if (slot[i] >= 0) {
            const XprepBatchItem &it = xitems[(size_t)slot[i]];
            LinearArgs a;
            a.tiles = l.w->tiles;
            a.N = l.w->N; a.K = l.w->K; a.NT = l.w->NT; a.SBp = l.w->SBp;
            a.x = nullptr; a.x_dt = TTQ_DT_BF16; a.M = l.M; a.ldx = l.w->K;
            a.bias = b_map; a.bias_dt = l.bias_dt;
            a.y = y_map; a.y_dt = l.y_dt; a.ldy = l.ldy;
            a.gated = false;
            int launches = 0;
            cudaStream_t lst = n_side > 1 ? side[next_side++ % n_side] : ctx->host_stream;
            e = launch_gemv(l.w->fmt, a, it.xq, l.w->SBp * TILE_K, reinterpret_cast<const uint8_t *>(ctx->dev_status) + 256, ctx->sms,
                            ctx->dev_status, nullptr, lst, &launches, nullptr, true);
            if (e != cudaSuccess) s = cuda_fail(ctx, e, "linear forward (batched activations) launch");
        } else {
            const void *xs = items[(size_t)(-1 - slot[i])].dst;
            bool done = false;
            if (one_launch[i] && n_side > 1 && b->side_ws != nullptr) {
                const int k = next_side++ % n_side;
                LinearArgs a;
                a.tiles = l.w->tiles;
                a.N = l.w->N; a.K = l.w->K; a.NT = l.w->NT; a.SBp = l.w->SBp;
                a.x = xs; a.x_dt = l.x_dt; a.M = l.M; a.ldx = l.ldx;
                a.bias = b_map; a.bias_dt = l.bias_dt;
                a.y = y_map; a.y_dt = l.y_dt; a.ldy = l.ldy;
                a.gated = false;
                int launches = 0;
                e = launch_q4k_mma(a, ctx->sms, ctx->dev_status, nullptr, reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(b->side_ws) + (size_t)k * SPLIT_WS_BYTES),
                                   SPLIT_WS_BYTES, reinterpret_cast<unsigned *>(b->side_counters) + (size_t)k * SPLIT_COUNTERS, SPLIT_COUNTERS, side[k],
                                   &launches);
                if (e == cudaSuccess) done = true;
                else if (e != cudaErrorNotSupported) s = cuda_fail(ctx, e, "linear forward (batched, one-launch decode) launch");
            }
            if (!done && s == TTQ_OK)
                s = ttq_linear_forward(ctx, l.w, xs, (ttq_dtype)l.x_dt, l.M, l.ldx, b_map, (ttq_dtype)l.bias_dt, y_map, (ttq_dtype)l.y_dt, l.ldy,
                                       ctx->host_stream);
        }
    }
    if (n_side > 1) {
        // join: the recording ends on the host stream with every side chain merged back (also after an error, so that the
        // recording can end)
        for (int k = 0; k < n_side; k++) {
            if (side[k] == nullptr || join_ev[k] == nullptr) continue;
            cudaError_t je = cudaEventRecord(join_ev[k], side[k]);
            if (je == cudaSuccess) je = cudaStreamWaitEvent(ctx->host_stream, join_ev[k], 0);
            if (je != cudaSuccess && s == TTQ_OK) s = cuda_fail(ctx, je, "host batch join");
        }
    }
    e = cudaStreamEndCapture(ctx->host_stream, &b->graph);  // always ends the recording, also after an error
    for (int k = 0; k < MAX_SIDE; k++) {
        if (join_ev[k]) cudaEventDestroy(join_ev[k]);
        if (side[k]) cudaStreamDestroy(side[k]);
    }
    if (fork_ev) cudaEventDestroy(fork_ev);
    if (s != TTQ_OK || e != cudaSuccess) {
        host_batch_free(b);
        cudaGetLastError();
        return s != TTQ_OK ? s : fail(ctx, TTQ_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
    }
    e = cudaGraphInstantiate(&b->exec, b->graph, 0);
    if (e != cudaSuccess) {
        b->exec = nullptr;
        host_batch_free(b);
        return fail(ctx, TTQ_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
    }
    *out = b;
    return TTQ_OK;
}

ttq_status ttq_host_batch_run(ttq_host_batch *batch) {
    if (!batch) return TTQ_ERR_INVALID_ARG;
    ttq_ctx *ctx = batch->ctx;
    TTQ_CUDA(ctx, cudaSetDevice(ctx->device));
    TTQ_CUDA(ctx, cudaGraphLaunch(batch->exec, ctx->host_stream));
    return host_stream_sync(ctx);
}

ttq_status ttq_host_batch_destroy(ttq_host_batch *batch) {
    if (!batch) return TTQ_OK;
    cudaSetDevice(batch->ctx->device);
    cudaStreamSynchronize(batch->ctx->host_stream);
    host_batch_free(batch);
    return TTQ_OK;
}

ttq_status ttq_host_sync(ttq_ctx *ctx) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    TTQ_CUDA(ctx, cudaSetDevice(ctx->device));
    return host_stream_sync(ctx);
}

ttq_status ttq_device_status(ttq_ctx *ctx, void *stream) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    int host = 0;
    TTQ_CUDA(ctx, cudaMemcpyAsync(&host, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    TTQ_CUDA(ctx, cudaStreamSynchronize((cudaStream_t)stream));
    if (host != 0) {
        ctx->host_status[0] = 0;
        cudaMemsetAsync(ctx->dev_status, 0, sizeof(int), (cudaStream_t)stream);
        // a kernel that gave up may have left K-split arrival counters behind
        cudaMemsetAsync(ctx->split_counters, 0, (size_t)ctx->split_counters_cap * sizeof(unsigned), (cudaStream_t)stream);
        return fail(ctx, TTQ_ERR_TIMEOUT, "a kernel gave up a bounded wait (status word 0x%x); results of that call are invalid", host);
    }
    return TTQ_OK;
}

ttq_status ttq_comm_create(ttq_ctx *ctx, int rank, int world, int64_t n_cap, int m_cap, ttq_comm **out, void *ipc_handle_out) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    if (!out || !ipc_handle_out) return fail(ctx, TTQ_ERR_INVALID_ARG, "out or handle pointer is NULL");
    *out = nullptr;
    if (world < 2 || world > TTQ_MAX_RANKS || rank < 0 || rank >= world)
        return fail(ctx, TTQ_ERR_INVALID_ARG, "rank %d of %d: world must be 2..%d", rank, world, TTQ_MAX_RANKS);
    if (n_cap <= 0 || m_cap <= 0 || m_cap > MAX_GEMV_M) return fail(ctx, TTQ_ERR_SHAPE, "bad capacity (n_cap=%lld m_cap=%d)", (long long)n_cap, m_cap);
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    TTQ_CUDA(ctx, cudaSetDevice(ctx->device));
    ttq_comm *c = new (std::nothrow) ttq_comm();
    if (!c) return fail(ctx, TTQ_ERR_OOM, "host allocation failed");
    memset(c, 0, sizeof(*c));
    c->ctx = ctx;
    const int64_t nt_cap = (n_cap + TILE_ROWS - 1) / TILE_ROWS;
    n_cap = nt_cap * TILE_ROWS;
    c->bytes = (size_t)2 * world * m_cap * n_cap * sizeof(uint2);
    cudaError_t e = cudaMalloc(&c->local, c->bytes);
    if (e == cudaSuccess) e = cudaMemset(c->local, 0, c->bytes);
    if (e == cudaSuccess) e = cudaMalloc(&c->view.sent, (size_t)nt_cap * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(c->view.sent, 0, (size_t)nt_cap * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t *>(ipc_handle_out), c->local);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(c->local);
        cudaFree(c->view.sent);
        delete c;
        return cuda_fail(ctx, e, "exchange buffer set-up");
    }
    c->view.rank = rank;
    c->view.world = world;
    c->view.wait_limit = DEFAULT_PEER_WAIT_LIMIT;
    c->view.nt_cap = (int)nt_cap;
    c->view.m_cap = m_cap;
    c->view.n_cap = n_cap;
    *out = c;
    return TTQ_OK;
}

ttq_status ttq_comm_connect(ttq_comm *c, const void *all_handles) {
    if (!c || !all_handles) return TTQ_ERR_INVALID_ARG;
    ttq_ctx *ctx = c->ctx;
    TTQ_CUDA(ctx, cudaSetDevice(ctx->device));
    const cudaIpcMemHandle_t *h = reinterpret_cast<const cudaIpcMemHandle_t *>(all_handles);
    for (int r = 0; r < c->view.world; r++) {
        void *base = c->local;
        if (r != c->view.rank) {
            TTQ_CUDA(ctx, cudaIpcOpenMemHandle(&c->peer_map[r], h[r], cudaIpcMemLazyEnablePeerAccess));
            base = c->peer_map[r];
        }
        c->view.cells[r] = reinterpret_cast<uint2 *>(base);
    }
    return TTQ_OK;
}

ttq_status ttq_comm_local_buffer(ttq_comm *c, void **base_out, size_t *bytes_out) {
    if (!c || !base_out) return TTQ_ERR_INVALID_ARG;
    *base_out = c->local;
    if (bytes_out) *bytes_out = c->bytes;
    return TTQ_OK;
}

ttq_status ttq_comm_connect_pointers(ttq_comm *c, void *const *bases) {
    if (!c || !bases) return TTQ_ERR_INVALID_ARG;
    ttq_ctx *ctx = c->ctx;
    for (int r = 0; r < c->view.world; r++) {
        void *base = r == c->view.rank ? c->local : bases[r];
        if (!base) return fail(ctx, TTQ_ERR_INVALID_ARG, "exchange buffer of rank %d is NULL", r);
        if (reinterpret_cast<uintptr_t>(base) & 255) return fail(ctx, TTQ_ERR_INVALID_ARG, "exchange buffer of rank %d is not 256-byte aligned", r);
        c->view.cells[r] = reinterpret_cast<uint2 *>(base);
    }
    return TTQ_OK;
}

ttq_status ttq_comm_set_wait_limit(ttq_comm *c, int64_t polls) {
    if (!c) return TTQ_ERR_INVALID_ARG;
    if (polls < 1 || polls > (1ll << 30)) return fail(c->ctx, TTQ_ERR_INVALID_ARG, "polls=%lld outside 1..2^30", (long long)polls);
    c->view.wait_limit = (int)polls;
    return TTQ_OK;
}

ttq_status ttq_comm_destroy(ttq_comm *c) {
    if (!c) return TTQ_OK;
    cudaSetDevice(c->ctx->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < TTQ_MAX_RANKS; r++)
        if (c->peer_map[r]) cudaIpcCloseMemHandle(c->peer_map[r]);
    cudaFree(c->local);
    cudaFree(c->view.sent);
    delete c;
    return TTQ_OK;
}

ttq_status ttq_linear_forward_allreduce(ttq_ctx *ctx, const ttq_weight *w, const void *x_dev, ttq_dtype x_dt, int64_t M, int64_t ldx,
                                        const void *bias_dev, ttq_dtype bias_dt, void *y_dev, ttq_dtype y_dt, int64_t ldy,
                                        ttq_comm *comm, void *stream) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    ctx->prepared_m = 0;  // the activation scratch may be rewritten below
    if (!w || !comm) return fail(ctx, TTQ_ERR_INVALID_ARG, "weight or communicator is NULL");
    if (w->ctx != ctx || comm->ctx != ctx) return fail(ctx, TTQ_ERR_INVALID_ARG, "weight or communicator belongs to another context");
    if (comm->view.cells[comm->view.world - 1] == nullptr) return fail(ctx, TTQ_ERR_INVALID_ARG, "communicator is not connected");
    if (M < 0) return fail(ctx, TTQ_ERR_SHAPE, "M=%lld is negative", (long long)M);
    if (M == 0) return TTQ_OK;
    if (!x_dev || !y_dev) return fail(ctx, TTQ_ERR_INVALID_ARG, "x or y pointer is NULL");
    if (x_dt != TTQ_DT_BF16 && x_dt != TTQ_DT_F16) return fail(ctx, TTQ_ERR_INVALID_ARG, "x dtype must be bf16 or f16");
    if (!valid_dt(y_dt) || (bias_dev && !valid_dt(bias_dt))) return fail(ctx, TTQ_ERR_INVALID_ARG, "unknown dtype");
    if (ldx < w->K || ldy < w->N) return fail(ctx, TTQ_ERR_SHAPE, "leading dimension smaller than the row length");
    if (w->fmt == TTQ_FMT_TQ3)
        return fail(ctx, TTQ_ERR_UNSUPPORTED, "the fused exchange serves the block formats: use ttq_linear_forward and a library all-reduce");
    if (M > comm->view.m_cap || w->N > comm->view.n_cap)
        return fail(ctx, TTQ_ERR_UNSUPPORTED, "M=%lld / N=%lld exceed the exchange buffer (m_cap=%d, n_cap=%lld): use ttq_linear_forward and a library all-reduce",
                    (long long)M, (long long)w->N, comm->view.m_cap, (long long)comm->view.n_cap);
    LinearArgs a;
    a.tiles = w->tiles;
    a.N = w->N; a.K = w->K; a.NT = w->NT; a.SBp = w->SBp;
    a.x = x_dev; a.x_dt = x_dt; a.M = M; a.ldx = ldx;
    a.bias = bias_dev; a.bias_dt = bias_dt;
    a.y = y_dev; a.y_dt = y_dt; a.ldy = ldy;
    int launches = 0;
    cudaError_t e = cudaErrorNotSupported;
    static const bool use_mma = env_flag("TTQ_Q4K_MMA", true);
    if (w->fmt == TTQ_FMT_Q4_K && use_mma && M >= 3) {
        e = launch_q4k_mma(a, ctx->sms, ctx->dev_status, ctx->trace, ctx->split_ws, ctx->split_ws_bytes, ctx->split_counters,
                           ctx->split_counters_cap, (cudaStream_t)stream, &launches, &comm->view);
        ctx->launches += launches;
    }
    if (e == cudaErrorNotSupported) {
        if (M > MAX_GEMV_M) return fail(ctx, TTQ_ERR_UNSUPPORTED, "M=%lld exceeds the decode kernel's %d rows", (long long)M, MAX_GEMV_M);
        e = launch_gemv(w->fmt, a, ctx->xq, ctx->xq_capacity_k, reinterpret_cast<const uint8_t *>(ctx->dev_status) + 256, ctx->sms,
                        ctx->dev_status, ctx->trace, (cudaStream_t)stream, &launches, &comm->view);
        ctx->launches += launches;
    }
    if (e != cudaSuccess) return cuda_fail(ctx, e, "row-parallel linear launch");
    return TTQ_OK;
}

ttq_status ttq_trace_read(ttq_ctx *ctx, uint64_t *out, int64_t max_entries, int64_t *n_entries) {
    if (!ctx || !out || !n_entries) return TTQ_ERR_INVALID_ARG;
    *n_entries = 0;
    if (!ctx->trace) return TTQ_OK;
    TTQ_CUDA(ctx, cudaDeviceSynchronize());
    unsigned long long count = 0;
    TTQ_CUDA(ctx, cudaMemcpy(&count, ctx->trace, sizeof(count), cudaMemcpyDeviceToHost));
    int64_t n = (int64_t)(count < (unsigned long long)TTQ_TRACE_ENTRIES ? count : TTQ_TRACE_ENTRIES);
    if (n > max_entries) n = max_entries;
    if (n > 0) TTQ_CUDA(ctx, cudaMemcpy(out, ctx->trace + 8, (size_t)n * 8 * sizeof(uint64_t), cudaMemcpyDeviceToHost));
    TTQ_CUDA(ctx, cudaMemset(ctx->trace, 0, sizeof(unsigned long long)));
    *n_entries = n;
    return TTQ_OK;
}

ttq_status ttq_silu_and_mul(ttq_ctx *ctx, const void *in_dev, ttq_dtype dt, int64_t M, int64_t H, int64_t ld_in,
                            void *out_dev, int64_t ld_out, void *stream) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    if (M < 0 || H < 0) return fail(ctx, TTQ_ERR_SHAPE, "negative size");
    if (M == 0 || H == 0) return TTQ_OK;
    if (!in_dev || !out_dev) return fail(ctx, TTQ_ERR_INVALID_ARG, "input or output pointer is NULL");
    if (!valid_dt(dt)) return fail(ctx, TTQ_ERR_INVALID_ARG, "unknown dtype %d", (int)dt);
    if (ld_in < 2 * H || ld_out < H) return fail(ctx, TTQ_ERR_SHAPE, "leading dimension smaller than the row length");
    cudaError_t e = launch_silu_and_mul(in_dev, dt, M, H, ld_in, out_dev, ld_out, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "silu_and_mul launch");
    ctx->launches++;
    return TTQ_OK;
}

ttq_status ttq_moe_create(ttq_ctx *ctx, int32_t n_experts, const ttq_weight *const *gate_up, const ttq_weight *const *down,
                          int64_t max_tokens, int32_t top_k, ttq_moe **out) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    if (!out) return fail(ctx, TTQ_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    if (!gate_up || !down) return fail(ctx, TTQ_ERR_INVALID_ARG, "expert weight table is NULL");
    if (n_experts <= 0 || n_experts > 4096) return fail(ctx, TTQ_ERR_SHAPE, "n_experts=%d out of range 1..4096", n_experts);
    if (top_k <= 0 || top_k > n_experts) return fail(ctx, TTQ_ERR_SHAPE, "top_k=%d out of range 1..%d", top_k, n_experts);
    if (max_tokens <= 0) return fail(ctx, TTQ_ERR_SHAPE, "max_tokens must be positive");
    for (int e = 0; e < n_experts; e++) {
        const ttq_weight *a = gate_up[e], *b = down[e];
        if (!a || !b) return fail(ctx, TTQ_ERR_INVALID_ARG, "expert %d: weight is NULL", e);
        if (a->ctx != ctx || b->ctx != ctx) return fail(ctx, TTQ_ERR_INVALID_ARG, "expert %d: weight belongs to another context", e);
        if (a->fmt != TTQ_FMT_Q4_K || b->fmt != TTQ_FMT_Q4_K)
            return fail(ctx, TTQ_ERR_UNSUPPORTED, "expert %d: the grouped path takes Q4_K weights", e);
        if (a->N != gate_up[0]->N || a->K != gate_up[0]->K || b->N != down[0]->N || b->K != down[0]->K)
            return fail(ctx, TTQ_ERR_SHAPE, "expert %d: shape differs from expert 0", e);
    }
    const int64_t H = gate_up[0]->K, I = down[0]->K;
    if (gate_up[0]->N != 2 * I || down[0]->N != H)
        return fail(ctx, TTQ_ERR_SHAPE, "gate|up must be [2I][H] and down [H][I] (got [%lld][%lld] and [%lld][%lld])",
                    (long long)gate_up[0]->N, (long long)H, (long long)down[0]->N, (long long)I);
    if (H % 8 || I % 8) return fail(ctx, TTQ_ERR_SHAPE, "H and I must be multiples of 8");
    if (max_tokens * top_k + (int64_t)n_experts * 256 > (1ll << 30)) return fail(ctx, TTQ_ERR_LIMIT, "routed row capacity too large");
    ttq_moe *m = new (std::nothrow) ttq_moe();
    if (!m) return fail(ctx, TTQ_ERR_OOM, "host allocation failed");
    m->ctx = ctx; m->E = n_experts; m->top_k = top_k; m->H = H; m->I = I; m->max_tokens = max_tokens;
    m->NT1 = gate_up[0]->NT; m->SBp1 = gate_up[0]->SBp; m->NT2 = down[0]->NT; m->SBp2 = down[0]->SBp;
    m->rows_cap = ((max_tokens * top_k + (int64_t)n_experts * 256 + 255) / 256) * 256;
    const int64_t pairs = max_tokens * top_k;
    auto up256 = [](size_t b) { return (b + 255) & ~(size_t)255; };
    const size_t b_tab = up256(sizeof(void *) * (size_t)n_experts);
    const size_t b_e = up256(sizeof(int) * (size_t)n_experts);
    const size_t b_mt = up256(sizeof(int) * (size_t)(m->rows_cap / 64));
    const size_t b_rows = up256(sizeof(int) * (size_t)m->rows_cap);
    const size_t b_pairs = up256(sizeof(int) * (size_t)pairs);
    const size_t b_xh1 = up256(sizeof(__half) * (size_t)m->rows_cap * (size_t)(m->SBp1 * TILE_K));
    const size_t b_o2 = up256(sizeof(__half) * (size_t)m->rows_cap * (size_t)H);
    const size_t b_a = b_xh1 > b_o2 ? b_xh1 : b_o2;  // the routed input images and the routed outputs are never live together
    const size_t b_h1 = up256(sizeof(__half) * (size_t)m->rows_cap * (size_t)(2 * I));
    const size_t b_xh2 = up256(sizeof(__half) * (size_t)m->rows_cap * (size_t)(m->SBp2 * TILE_K));
    const size_t total = 2 * b_tab + 3 * b_e + 256 + 3 * b_mt + b_rows + b_pairs + b_a + b_h1 + b_xh2;
    cudaError_t e = cudaMalloc(&m->ws, total);
    if (e != cudaSuccess) {
        delete m;
        return cuda_fail(ctx, e, "cudaMalloc(mixture-of-experts workspace)");
    }
    uint8_t *q = reinterpret_cast<uint8_t *>(m->ws);
    m->d_gate_up = reinterpret_cast<const uint8_t **>(q); q += b_tab;
    m->d_down = reinterpret_cast<const uint8_t **>(q); q += b_tab;
    m->route.counts = reinterpret_cast<int *>(q); q += b_e;
    m->route.row_start = reinterpret_cast<int *>(q); q += b_e;
    m->route.cursor = reinterpret_cast<int *>(q); q += b_e;
    m->route.n_mt = reinterpret_cast<int *>(q); q += 256;
    m->route.mt_group = reinterpret_cast<int *>(q); q += b_mt;
    m->route.mt_row0 = reinterpret_cast<int *>(q); q += b_mt;
    m->route.mt_mh = reinterpret_cast<int *>(q); q += b_mt;
    m->route.row_src = reinterpret_cast<int *>(q); q += b_rows;
    m->route.slot_of = reinterpret_cast<int *>(q); q += b_pairs;
    m->xh1 = reinterpret_cast<__half *>(q); m->o2 = m->xh1; q += b_a;
    m->h1 = reinterpret_cast<__half *>(q); q += b_h1;
    m->xh2 = reinterpret_cast<__half *>(q);
    std::vector<const uint8_t *> tab((size_t)2 * n_experts);
    for (int x = 0; x < n_experts; x++) {
        tab[x] = gate_up[x]->tiles;
        tab[(size_t)n_experts + x] = down[x]->tiles;
    }
    e = cudaMemcpy(m->d_gate_up, tab.data(), sizeof(void *) * (size_t)n_experts, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(m->d_down, tab.data() + n_experts, sizeof(void *) * (size_t)n_experts, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaFree(m->ws);
        delete m;
        return cuda_fail(ctx, e, "upload of the expert tables");
    }
    *out = m;
    return TTQ_OK;
}

ttq_status ttq_moe_destroy(ttq_moe *m) {
    if (!m) return TTQ_OK;
    cudaFree(m->ws);
    delete m;
    return TTQ_OK;
}

ttq_status ttq_moe_forward(ttq_ctx *ctx, ttq_moe *m, const void *x_dev, ttq_dtype x_dt, int64_t T, int64_t ldx,
                           const int32_t *topk_ids_dev, const float *topk_weights_dev, void *y_dev, ttq_dtype y_dt, int64_t ldy,
                           void *stream) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    if (!m) return fail(ctx, TTQ_ERR_INVALID_ARG, "layer handle is NULL");
    if (m->ctx != ctx) return fail(ctx, TTQ_ERR_INVALID_ARG, "layer belongs to another context");
    if (T < 0) return fail(ctx, TTQ_ERR_SHAPE, "T=%lld is negative", (long long)T);
    if (T == 0) return TTQ_OK;
    if (T > m->max_tokens) return fail(ctx, TTQ_ERR_LIMIT, "T=%lld exceeds max_tokens=%lld of the layer", (long long)T, (long long)m->max_tokens);
    if (!x_dev || !y_dev || !topk_ids_dev || !topk_weights_dev) return fail(ctx, TTQ_ERR_INVALID_ARG, "a device pointer is NULL");
    if (x_dt != TTQ_DT_BF16 && x_dt != TTQ_DT_F16) return fail(ctx, TTQ_ERR_INVALID_ARG, "x dtype must be bf16 or f16");
    if (!valid_dt(y_dt)) return fail(ctx, TTQ_ERR_INVALID_ARG, "unknown y dtype %d", (int)y_dt);
    if (ldx < m->H || ldy < m->H) return fail(ctx, TTQ_ERR_SHAPE, "leading dimension smaller than the hidden size %lld", (long long)m->H);
    cudaStream_t st = (cudaStream_t)stream;
    // row-tile height from the mean number of rows per expert; capacity of this call in rows
    const int64_t pairs = T * m->top_k, mean = pairs / m->E;
    // TTQ_MOE_BM=384 selects tiles of one to three 128-row blocks (rows padded to 128 only, one expansion of an
    // expert's weight rows for up to 384 of its rows); measured 5 % slower than 256-row tiles at 256 rows per
    // expert because it runs with one 128-row weight sub-tile per CTA
    int BM = mean <= 64 ? 64 : (mean <= 128 ? 128 : 256);
    static const int force_bm = []() {
        const char *v = getenv("TTQ_MOE_BM");
        return v ? atoi(v) : 0;
    }();
    if (force_bm == 64 || force_bm == 128 || force_bm == 256 || force_bm == 384) BM = force_bm;
    const int64_t unit = BM == 384 ? 128 : BM;
    int64_t Mp = ((pairs + (int64_t)m->E * unit + unit - 1) / unit) * unit;
    if (Mp > m->rows_cap) Mp = m->rows_cap / unit * unit;
    const int64_t mt_cap = BM == 384 ? pairs / 384 + m->E + 1 : Mp / BM;
    int n = 0;
    cudaError_t e = launch_moe_route(m->route, topk_ids_dev, T, m->top_k, m->E, BM, Mp, mt_cap, st, &n);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "routing launch");
    ctx->launches += n;
    GroupedArgs g;
    g.group_tiles = m->d_gate_up;
    g.N = 2 * m->I; g.K = m->H; g.NT = m->NT1; g.SBp = m->SBp1;
    g.x = x_dev; g.x_dt = x_dt; g.x_rows = T; g.ldx = ldx;
    g.row_src = m->route.row_src; g.gated = false;
    g.Mp = Mp; g.BM = BM;
    g.mt_group = m->route.mt_group; g.n_mt = m->route.n_mt;
    g.mt_row0 = m->route.mt_row0; g.mt_mh = m->route.mt_mh; g.rows_total = m->route.n_mt + 1; g.mt_cap = mt_cap;
    g.y = m->h1; g.y_dt = TTQ_DT_F16; g.ldy = 2 * m->I;
    e = launch_gemm_grouped(g, m->xh1, ctx->sms, ctx->dev_status, st, &n);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "grouped gate|up launch");
    ctx->launches += n;
    g.group_tiles = m->d_down;
    g.N = m->H; g.K = m->I; g.NT = m->NT2; g.SBp = m->SBp2;
    g.x = m->h1; g.x_dt = TTQ_DT_F16; g.x_rows = Mp; g.ldx = 2 * m->I;
    g.row_src = nullptr; g.gated = true;
    g.y = m->o2; g.y_dt = TTQ_DT_F16; g.ldy = m->H;
    e = launch_gemm_grouped(g, m->xh2, ctx->sms, ctx->dev_status, st, &n);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "grouped down launch");
    ctx->launches += n;
    e = launch_moe_combine(m->route, m->o2, TTQ_DT_F16, m->H, topk_weights_dev, T, m->top_k, m->H, y_dev, y_dt, ldy, st);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "combine launch");
    ctx->launches++;
    return TTQ_OK;
}

ttq_status ttq_add_rmsnorm(ttq_ctx *ctx, void *h_dev, const void *delta_dev, const void *weight_dev, ttq_dtype dt, int64_t M,
                           int64_t H, int64_t ld_h, int64_t ld_delta, float eps, void *out_dev, int64_t ld_out, void *stream) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    if (M < 0 || H <= 0) return fail(ctx, TTQ_ERR_SHAPE, "bad size (M=%lld H=%lld)", (long long)M, (long long)H);
    if (M == 0) return TTQ_OK;
    if (!h_dev || !weight_dev || !out_dev) return fail(ctx, TTQ_ERR_INVALID_ARG, "a device pointer is NULL");
    if (dt != TTQ_DT_BF16 && dt != TTQ_DT_F16) return fail(ctx, TTQ_ERR_INVALID_ARG, "dtype must be bf16 or f16");
    if (H % 8 || ld_h % 8 || ld_out % 8 || (delta_dev && ld_delta % 8) || ld_h < H || ld_out < H || (delta_dev && ld_delta < H))
        return fail(ctx, TTQ_ERR_SHAPE, "H and the leading dimensions must be multiples of 8 and at least H");
    if (((uintptr_t)h_dev | (uintptr_t)weight_dev | (uintptr_t)out_dev | (uintptr_t)delta_dev) & 15)
        return fail(ctx, TTQ_ERR_INVALID_ARG, "pointers must be 16-byte aligned");
    cudaError_t e = launch_add_rmsnorm(h_dev, delta_dev, weight_dev, dt, M, H, ld_h, ld_delta, eps, out_dev, ld_out, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "add_rmsnorm launch");
    ctx->launches++;
    return TTQ_OK;
}

ttq_status ttq_add_rmsnorm_prepare(ttq_ctx *ctx, void *h_dev, const void *delta_dev, const void *weight_dev, ttq_dtype dt, int64_t M,
                                   int64_t H, int64_t ld_h, int64_t ld_delta, float eps, void *out_dev, int64_t ld_out, void *stream) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    ctx->prepared_m = ctx->prepared_k = 0;
    if (M < 1 || M > 2) return fail(ctx, TTQ_ERR_LIMIT, "M=%lld: the prepared form serves 1 or 2 rows", (long long)M);
    if (H <= 0 || H % TILE_K || H > 8192 || H > ctx->xq_capacity_k)
        return fail(ctx, TTQ_ERR_SHAPE, "H=%lld: the prepared form needs a multiple of 256, at most 8192 and within the activation scratch", (long long)H);
    if (!h_dev || !weight_dev || !out_dev) return fail(ctx, TTQ_ERR_INVALID_ARG, "a device pointer is NULL");
    if (dt != TTQ_DT_BF16 && dt != TTQ_DT_F16) return fail(ctx, TTQ_ERR_INVALID_ARG, "dtype must be bf16 or f16");
    if (ld_h % 8 || ld_out % 8 || (delta_dev && ld_delta % 8) || ld_h < H || ld_out < H || (delta_dev && ld_delta < H))
        return fail(ctx, TTQ_ERR_SHAPE, "the leading dimensions must be multiples of 8 and at least H");
    if (((uintptr_t)h_dev | (uintptr_t)weight_dev | (uintptr_t)out_dev | (uintptr_t)delta_dev) & 15)
        return fail(ctx, TTQ_ERR_INVALID_ARG, "pointers must be 16-byte aligned");
    cudaError_t e = launch_add_rmsnorm(h_dev, delta_dev, weight_dev, dt, M, H, ld_h, ld_delta, eps, out_dev, ld_out, (cudaStream_t)stream, &ctx->xq);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "add_rmsnorm (prepared) launch");
    ctx->launches++;
    ctx->prepared_m = M;
    ctx->prepared_k = H;
    return TTQ_OK;
}

ttq_status ttq_linear_forward_prepared(ttq_ctx *ctx, const ttq_weight *w, int64_t M, const void *bias_dev, ttq_dtype bias_dt, void *y_dev,
                                       ttq_dtype y_dt, int64_t ldy, void *stream) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    if (!w) return fail(ctx, TTQ_ERR_INVALID_ARG, "weight is NULL");
    if (w->ctx != ctx) return fail(ctx, TTQ_ERR_INVALID_ARG, "weight belongs to another context");
    if (w->fmt == TTQ_FMT_TQ3) return fail(ctx, TTQ_ERR_UNSUPPORTED, "the prepared form serves the block formats");
    if (ctx->prepared_m == 0) return fail(ctx, TTQ_ERR_INVALID_ARG, "no prepared activations: call ttq_add_rmsnorm_prepare first");
    if (M != ctx->prepared_m || w->K != ctx->prepared_k)
        return fail(ctx, TTQ_ERR_SHAPE, "prepared activations are [%lld][%lld], the call wants [%lld][%lld]", (long long)ctx->prepared_m,
                    (long long)ctx->prepared_k, (long long)M, (long long)w->K);
    if (!y_dev) return fail(ctx, TTQ_ERR_INVALID_ARG, "y pointer is NULL");
    if (!valid_dt(y_dt) || (bias_dev && !valid_dt(bias_dt))) return fail(ctx, TTQ_ERR_INVALID_ARG, "unknown dtype");
    if (ldy < w->N) return fail(ctx, TTQ_ERR_SHAPE, "ldy=%lld is smaller than N=%lld", (long long)ldy, (long long)w->N);
    LinearArgs a;
    a.tiles = w->tiles;
    a.N = w->N; a.K = w->K; a.NT = w->NT; a.SBp = w->SBp;
    a.x = nullptr; a.x_dt = TTQ_DT_BF16; a.M = M; a.ldx = w->K;
    a.bias = bias_dev; a.bias_dt = bias_dt;
    a.y = y_dev; a.y_dt = y_dt; a.ldy = ldy;
    a.gated = false;
    int launches = 0;
    cudaError_t e = launch_gemv(w->fmt, a, ctx->xq, ctx->xq_capacity_k, reinterpret_cast<const uint8_t *>(ctx->dev_status) + 256, ctx->sms,
                                ctx->dev_status, ctx->trace, (cudaStream_t)stream, &launches, nullptr, true);
    ctx->launches += launches;
    if (e == cudaErrorNotSupported) return fail(ctx, TTQ_ERR_UNSUPPORTED, "this shape does not fit the copying mode of the decode kernel");
    if (e != cudaSuccess) return cuda_fail(ctx, e, "linear forward (prepared) launch");
    return TTQ_OK;
}

ttq_status ttq_rope_kv_append(ttq_ctx *ctx, const void *qkv_dev, ttq_dtype dt, int64_t B, int64_t ld_qkv, int32_t hq, int32_t hkv,
                              int32_t d, const void *cos_dev, const void *sin_dev, void *q_out_dev, void *k_cache_dev,
                              void *v_cache_dev, int64_t ctx_len, int64_t pos, void *stream) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    if (B < 0 || hq <= 0 || hkv <= 0 || d <= 0 || d % 2 || d > 2048) return fail(ctx, TTQ_ERR_SHAPE, "bad head geometry");
    if (B == 0) return TTQ_OK;
    if (B > 65535) return fail(ctx, TTQ_ERR_LIMIT, "B=%lld exceeds 65535", (long long)B);
    if (!qkv_dev || !cos_dev || !sin_dev || !q_out_dev || !k_cache_dev || !v_cache_dev) return fail(ctx, TTQ_ERR_INVALID_ARG, "a device pointer is NULL");
    if (dt != TTQ_DT_BF16 && dt != TTQ_DT_F16) return fail(ctx, TTQ_ERR_INVALID_ARG, "dtype must be bf16 or f16");
    if (ld_qkv < (int64_t)(hq + 2 * hkv) * d) return fail(ctx, TTQ_ERR_SHAPE, "ld_qkv smaller than (hq + 2 hkv) * d");
    if (pos < 0 || pos >= ctx_len) return fail(ctx, TTQ_ERR_SHAPE, "pos=%lld outside the cache of %lld positions", (long long)pos, (long long)ctx_len);
    if ((((uintptr_t)qkv_dev) | ((uintptr_t)q_out_dev) | ((uintptr_t)k_cache_dev) | ((uintptr_t)v_cache_dev)) & 3)
        return fail(ctx, TTQ_ERR_INVALID_ARG, "qkv, q_out and the caches must be 4-byte aligned");
    cudaError_t e = launch_rope_kv(qkv_dev, dt, B, ld_qkv, hq, hkv, d, cos_dev, sin_dev, q_out_dev, k_cache_dev, v_cache_dev, ctx_len, pos,
                                   (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "rope_kv launch");
    ctx->launches++;
    return TTQ_OK;
}

ttq_status ttq_decode_attention(ttq_ctx *ctx, const void *q_dev, const void *k_cache_dev, const void *v_cache_dev, ttq_dtype dt, int64_t B,
                                int32_t hq, int32_t hkv, int32_t d, int64_t ctx_len, int64_t n_ctx, void *out_dev, void *stream) {
    if (!ctx) return TTQ_ERR_INVALID_ARG;
    if (B < 0 || hq <= 0 || hkv <= 0 || hq % hkv) return fail(ctx, TTQ_ERR_SHAPE, "bad head counts (hq=%d hkv=%d)", hq, hkv);
    if (B == 0) return TTQ_OK;
    const int G = hq / hkv;
    if (d != 128 || (G != 1 && G != 2 && G != 4 && G != 8))
        return fail(ctx, TTQ_ERR_UNSUPPORTED, "decode attention serves d = 128 and hq / hkv in {1, 2, 4, 8}");
    if (!q_dev || !k_cache_dev || !v_cache_dev || !out_dev) return fail(ctx, TTQ_ERR_INVALID_ARG, "a device pointer is NULL");
    if (dt != TTQ_DT_BF16 && dt != TTQ_DT_F16) return fail(ctx, TTQ_ERR_INVALID_ARG, "dtype must be bf16 or f16");
    if (n_ctx <= 0 || n_ctx > ctx_len) return fail(ctx, TTQ_ERR_SHAPE, "n_ctx=%lld outside 1..ctx_len=%lld", (long long)n_ctx, (long long)ctx_len);
    if (B > 65535 || hkv > 65535) return fail(ctx, TTQ_ERR_LIMIT, "B or hkv exceeds 65535");
    if ((((uintptr_t)k_cache_dev) | ((uintptr_t)v_cache_dev) | ((uintptr_t)q_dev) | ((uintptr_t)out_dev)) & 15)
        return fail(ctx, TTQ_ERR_INVALID_ARG, "q, out and the K and V caches must be 16-byte aligned");
    if (decode_attention_scratch_floats(B, hq, n_ctx) > ctx->att_part_cap)
        return fail(ctx, TTQ_ERR_LIMIT, "B * hq * ceil(n_ctx / 128) exceeds the attention scratch of the context");
    cudaError_t e = launch_decode_attention(q_dev, k_cache_dev, v_cache_dev, dt, B, hq, hkv, d, ctx_len, n_ctx, ctx->att_part, out_dev,
                                            (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "decode attention launch");
    ctx->launches += 2;
    return TTQ_OK;
}

}  // extern "C"
