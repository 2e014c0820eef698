// Internal declarations shared by the translation units of libttq (not part of the public ABI).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdlib>
#include <stdint.h>

#include "ttq.h"

namespace ttq {

// ------------------------------------------------------------------------------------------------
// Tiled device layout.
//
// Every format is cut into tiles of TILE_ROWS weight rows x TILE_K weights along K (one Q4_K / Q6_K
// super-block, eight Q8_0 blocks).  Tiles of one row-tile are contiguous along K, so a warp that
// walks K for 16 rows reads one contiguous byte stream:
//
//     offset(tile nt, sb) = (nt * SBp + sb) * tile_bytes(fmt),   SBp = ceil(K / 256)
//
// Inside a tile the quant payload is stored in the order the integer tensor-core instruction
// (mma.sync m16n8k32, A row-major, u8|s8) wants its A operand, so that one 16-byte load per lane is a
// complete A fragment.  One instruction multiplies FOUR sub-blocks at once: its 32 K slots are four
// groups of 8, group u holding an 8-weight window of sub-block u of the current set; the activation
// operand is block-diagonal (columns 2u, 2u+1 = high/low activation plane, non-zero only in group
// u), so after the windows of a set have been accumulated, lane (g, t) holds the complete integer
// dot products of sub-block t for rows g and g+8 -- every lane owns a different (row, sub-block)
// pair when the per-sub-block scales are applied.
//
//  A chunk is 512 bytes, lane L = 4g + t owns 16 bytes = registers a0..a3; register `sl` covers
//     row = g + 8*(sl & 1),  group u = (t >> 1) + 2*(sl >> 1),  weights 4*(t & 1) .. +3 of the window.
//
//  Q4_K (2304 B = 16 x 144): set X = sub-blocks 0,2,4,6 (low nibbles), set Y = 1,3,5,7 (high nibbles)
//     [0,2048)      4 chunks, chunk n = window n (weights 8n..8n+7 of each sub-block); the byte of
//                   group u is the canonical qs byte of pair u (low nibble: sub-block 2u, high: 2u+1)
//     [2048,2304)   16 row headers x 16 B, canonical {fp16 d, fp16 dmin, 12 B 6-bit scales/mins}
//  Q8_0 (4352 B = 16 x 8 x 34): set s = blocks 4s..4s+3
//     [0,4096)      8 chunks, chunk 4s+n = window n of set s
//     [4096,4352)   fp16 d[r][b], row-major (16 B per row)
//  Q6_K (3360 B = 16 x 210): sub-blocks of 16 weights, set s = sub-blocks 4s..4s+3, windows n = 0,1
//     [0,2048)      4 chunks, chunk 2s'+n: low nibble = low 4 bits of the quant of set s', high nibble
//                   = low 4 bits of the quant at the same position of set s'+2
//     [2048,3072)   2 chunks, chunk n: bit pair s of a byte = high 2 bits of the quant of set s
//     [3072,3328)   int8 scales[r][16]
//     [3328,3360)   fp16 d[r]
//  Rows >= N and Q8_0 blocks beyond K are stored as zero bytes (they dequantize to 0).
// ------------------------------------------------------------------------------------------------
constexpr int TILE_ROWS = 16;
constexpr int TILE_K = 256;

__host__ __device__ constexpr int tile_bytes(int fmt) {
    return fmt == TTQ_FMT_Q8_0 ? 4352 : (fmt == TTQ_FMT_Q4_K ? 2304 : 3360);
}
__host__ __device__ constexpr int block_elems(int fmt) { return fmt == TTQ_FMT_Q8_0 ? 32 : (fmt == TTQ_FMT_TQ3 ? 128 : 256); }
__host__ __device__ constexpr int block_bytes(int fmt) {
    return fmt == TTQ_FMT_Q8_0 ? 34 : (fmt == TTQ_FMT_Q4_K ? 144 : 210);
}

// Activation fixed-point: per 256-chunk scale, |xq| <= XQ_MAX so that xq = 256*hi + lo with both
// planes in int8.
constexpr int XQ_MAX = 32639;
constexpr int MAX_GEMV_M = 16;

struct Weight {
    ttq_ctx *ctx;
    int device;  // CUDA device that holds `tiles`
    int fmt;
    int64_t N, K;
    int64_t NT;   // row tiles
    int64_t SBp;  // 256-wide K tiles
    uint8_t *tiles;
    size_t tiled_bytes;
};

}  // namespace ttq

struct ttq_weight : public ttq::Weight {};

namespace ttq {

// Activation planes produced by the x-prep kernel (global scratch) for the non-fused GEMV path.
struct XqView {
    int8_t *planes;   // [2*Mpad][Kp] : row 2m = high plane, 2m+1 = low plane
    float *sum16;     // [Mpad][Kp/16] sum of xq over 16-weight groups
    float *sum32;     // [Mpad][Kp/32]
    float *sx;        // [Mpad][SBp]
};

// One linear's activations in a batched activation pass (xprep_batch_kernel): M rows of K values at x, converted into xq;
// unit0 = first (row, chunk) unit of the item in the batch's numbering, ascending over the items.
struct XprepBatchItem {
    const void *x;
    int x_dt, M;
    int64_t K, ldx, SBp;
    XqView xq;
    int unit0;
};

// row pitch (floats) of XqView::sx
__host__ __device__ constexpr int sx_stride(int64_t SBp) { return (int)((SBp + 3) & ~(int64_t)3); }

// Peer-memory exchange area of a row-parallel linear (tensor parallelism).  Passed by value to the decode
// kernels; world <= 1 means "no exchange".  Every rank owns one buffer of 8-byte cells {value bits, epoch},
//   cells [2][world][m_cap][n_cap]   partial outputs pushed by rank src, double-buffered by exchange parity,
// and knows the base addresses of all ranks' buffers (its own and the peers' mappings).  A cell is written with
// ONE 8-byte store, so the value and the epoch that validates it arrive together: no fence, no separate flag.
constexpr int TTQ_MAX_RANKS = 8;
struct CommView {
    int rank, world;
    int nt_cap, m_cap;
    int wait_limit;                  // polls of a peer's cell before the wait is given up (status bit 2)
    int64_t n_cap;
    uint32_t *sent;                  // local [nt_cap]: exchanges this rank has completed per row tile
    uint2 *cells[TTQ_MAX_RANKS];     // exchange buffer of every rank
};

struct LinearArgs {
    const uint8_t *tiles;
    int64_t N, K, NT, SBp;
    const void *x;
    int x_dt;
    int64_t M, ldx;
    const void *bias;
    int bias_dt;
    void *y;
    int y_dt;
    int64_t ldy;
    bool gated = false;  // x rows hold 2K values [gate | up]; the operand is silu(gate[k]) * up[k]
};

// ---- failure reporting --------------------------------------------------------------------------------------
// A kernel that gives up a bounded wait ORs a bit into the status word it was given (bit 0: copy ring, bit 1:
// tensor-core pipeline, bit 2: peer exchange) and, when the two words behind it hold the address of a mapped host
// flag, raises that flag too, so that a host entry point learns of the failure from its own memory without a
// device-to-host copy on every call.  The static scratch array keeps those two words zero: no host flag.
__device__ __forceinline__ void report_failure(int *status, int bit) {
    atomicOr(status, bit);
    volatile int *host_flag = *reinterpret_cast<volatile int *volatile *>(status + 2);
    if (host_flag != nullptr) *host_flag = 1;
}

// ---- row-parallel exchange --------------------------------------------------------------------------------
// One 16-row tile of a row-parallel linear, called by a full warp: `value(o)` is this rank's partial sum of output
// o = m * 16 + row.  Every lane pushes its outputs into the cells of ALL ranks (its own included) with single
// 8-byte stores {value, epoch}, then polls -- bounded -- its own buffer until the cells of every rank carry this
// exchange's epoch and adds them in rank order, so all ranks end with bit-identical sums.  The epoch counts the
// exchanges of the row tile (all ranks issue the same sequence of calls); two parities of cells alternate, so a
// rank that runs one exchange ahead never overwrites cells a slower rank has yet to read.
template <class ValueFn, class StoreFn>
__device__ __forceinline__ void exchange_row_tile(const CommView &cm, int64_t rt, int M, int64_t N, int lane, int *status, ValueFn &&value,
                                                  StoreFn &&store) {
    const uint32_t epoch = cm.sent[rt] + 1u;
    const size_t slab = (size_t)cm.m_cap * cm.n_cap;
    const size_t par_off = (size_t)(epoch & 1u) * cm.world * slab;
    const int outs = M * TILE_ROWS;
    for (int o = lane; o < outs; o += 32) {
        const int row = o & 15, mm = o >> 4;
        const int64_t n = rt * TILE_ROWS + row;
        if (n < N) {
            const uint32_t bits = __float_as_uint(value(o));
            const size_t off = par_off + (size_t)cm.rank * slab + (size_t)mm * cm.n_cap + n;
            for (int q = 0; q < cm.world; q++)
                asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(cm.cells[q] + off), "r"(bits), "r"(epoch) : "memory");
        }
    }
    bool ok = true;
    const uint2 *mine = cm.cells[cm.rank] + par_off;
    for (int o = lane; o < outs; o += 32) {
        const int row = o & 15, mm = o >> 4;
        const int64_t n = rt * TILE_ROWS + row;
        if (n < N) {
            float acc = 0.f;
            for (int q = 0; q < cm.world; q++) {
                const uint2 *cell = mine + (size_t)q * slab + (size_t)mm * cm.n_cap + n;
                uint32_t bits = 0, seen = epoch - 1u;
                for (int spins = 0; ok; spins++) {
                    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(bits), "=r"(seen) : "l"(cell) : "memory");
                    if (seen == epoch) break;
                    if (spins >= cm.wait_limit) ok = false;  // bounded: give up, flag the failure, keep going
                }
                acc += __uint_as_float(bits);
            }
            store(mm, n, acc);
        }
    }
    if (!__all_sync(0xffffffffu, ok) && lane == 0) report_failure(status, 4);
    __syncwarp();
    if (lane == 0) cm.sent[rt] = epoch;
}

// ---- programmatic dependent launch ---------------------------------------------------------------------
// Kernels of a decode chain are launched with programmatic stream serialization: a kernel tells the scheduler
// early that its successor may be set up (grid_launch_dependents) and every such kernel waits for its
// predecessor's completion and memory flush (grid_dependency_wait) before it touches anything that depends on
// it -- only loads of constant data (weights) may precede the wait.  TTQ_PDL=0 launches plainly.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Multiprocessor count of the current device (cached per device); grid caps are multiples of it.
inline int device_sms() {
    static int cache[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
    if (cache[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 1;
        cache[dev] = n;
    }
    return cache[dev];
}

inline bool env_flag(const char *name, bool dflt) {
    const char *v = getenv(name);
    if (!v || !*v) return dflt;
    return v[0] != '0';
}

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    static const bool pdl = env_flag("TTQ_PDL", true);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// Grouped (mixture-of-experts) GEMM on the tensor-core path: activation rows are routed into BM-row
// tiles, each owned by one weight matrix; all matrices share N x K.
struct GroupedArgs {
    const uint8_t *const *group_tiles;  // device array: Q4_K tiled layout of every group
    int64_t N, K, NT, SBp;
    const void *x;                      // source rows
    int x_dt;
    int64_t x_rows, ldx;
    const int *row_src;                 // device [Mp]: source row of each routed row (-1 = padding) or nullptr (identity)
    bool gated;                         // source rows hold 2K values, the operand is silu(x[k]) * x[K + k]
    int64_t Mp;                         // capacity in routed rows (a multiple of 128, or of BM)
    int BM;                             // row-tile height: 64, 128, 256, or 384 = one to three 128-row blocks per tile
    const int *mt_group, *n_mt;         // device: group of each row tile, number of row tiles in use
    const int *mt_row0, *mt_mh;         // device: first routed row of each row tile; its 128-row blocks (BM = 384)
    const int *rows_total;              // device: routed rows in use (rows beyond are not converted)
    int64_t mt_cap;                     // row tiles the tables hold
    void *y;                            // [Mp][ldy] routed output rows
    int y_dt;
    int64_t ldy;
};
cudaError_t launch_gemm_grouped(const GroupedArgs &g, __half *xh, int sms, int *status, cudaStream_t st, int *launches);

// Trellis-coded 3-bit format (ttq_tq3.cu); `packed` is the canonical buffer on the device.
inline int64_t tq3_packed_bytes(int64_t N, int64_t K) { return N * K * 3 / 8 + 2 * N + K / 8; }
cudaError_t launch_tq3_decode(const uint8_t *packed, int64_t N, int64_t K, float *out, int64_t ld, cudaStream_t st);
cudaError_t launch_tq3_wimg(const uint8_t *packed, int64_t N, int64_t K, __half *wimg, cudaStream_t st);
cudaError_t launch_tq3_rotate(const void *in, int in_dt, int64_t M, int64_t C, int64_t ld_in, const uint8_t *sign, const __half *scale,
                              const void *bias, int bias_dt, void *out, int out_dt, int64_t ld_out, cudaStream_t st, bool fragments = false);
cudaError_t launch_tq3_gemv(const uint8_t *packed, int64_t N, int64_t K, const float *x1, int rows, float *y1, cudaStream_t st);
cudaError_t launch_tq3_mma(const uint8_t *packed, int64_t N, int64_t K, const __half *x1, int rows, float *y1, cudaStream_t st);

// Decode-step kernels around the linears (ttq_decode.cu).
// (`xq` != nullptr: also convert the output rows into the activation planes of a decode linear)
cudaError_t launch_add_rmsnorm(void *h, const void *delta, const void *weight, int dt, int64_t M, int64_t H, int64_t ld_h, int64_t ld_delta,
                               float eps, void *out, int64_t ld_out, cudaStream_t st, const XqView *xq = nullptr);
cudaError_t launch_rope_kv(const void *qkv, int dt, int64_t B, int64_t ld_qkv, int hq, int hkv, int d, const void *cosv, const void *sinv,
                           void *q_out, void *k_cache, void *v_cache, int64_t ctx_len, int64_t pos, cudaStream_t st);
int64_t decode_attention_scratch_floats(int64_t B, int hq, int64_t n_ctx);
cudaError_t launch_decode_attention(const void *q, const void *k_cache, const void *v_cache, int dt, int64_t B, int hq, int hkv, int d,
                                    int64_t ctx_len, int64_t n_ctx, float *part, void *out, cudaStream_t st);

// Routing and combination of a mixture-of-experts layer (ttq_moe.cu).
struct MoeRouting {
    int *counts, *row_start, *cursor;  // [E]
    int *n_mt;                         // [1] row tiles in use; [1] routed rows in use
    int *mt_group, *mt_row0, *mt_mh;   // [Mp / 64] each
    int *row_src;                      // [Mp]
    int *slot_of;                      // [T * top_k]
};
cudaError_t launch_moe_route(const MoeRouting &r, const int *topk_ids, int64_t T, int top_k, int E, int BM, int64_t Mp,
                             int64_t mt_cap, cudaStream_t st, int *launches);
cudaError_t launch_moe_combine(const MoeRouting &r, const void *o, int o_dt, int64_t ldo, const float *topk_w, int64_t T,
                               int top_k, int64_t H, void *y, int y_dt, int64_t ldy, cudaStream_t st);

// launchers (defined in the .cu files); each returns the number of kernels it launched or -1
cudaError_t launch_repack(int fmt, const uint8_t *canon, uint8_t *tiled, int64_t N, int64_t K, int64_t NT,
                          int64_t SBp, cudaStream_t st);
cudaError_t launch_dequant(int fmt, const uint8_t *tiled, float *out, int64_t ld, int64_t N, int64_t K,
                           int64_t SBp, cudaStream_t st);
// GEMV for M <= MAX_GEMV_M.  `xq` is scratch for the separate x-prep pass (used when M > fused limit).
// `prepared`: the planes of a.M rows are already in `xq` (written by the kernel that produced the activations): no
// activation pass is launched, a.x is not read.
cudaError_t launch_xprep_batch(const XprepBatchItem *items_dev, int n, int total_units, cudaStream_t st);
bool gemv_prepared_supported(int fmt, int64_t M, int64_t SBp);
cudaError_t launch_gemv(int fmt, const LinearArgs &a, const XqView &xq, int64_t xq_capacity_k, const uint8_t *zeros,
                        int sms, int *status, unsigned long long *trace, cudaStream_t st, int *launches,
                        const CommView *comm = nullptr, bool prepared = false);
// (`interleaved`: plane bytes of a sub-block in the order of the tensor-memory decode kernel, see XqRow)
cudaError_t launch_xprep(const LinearArgs &a, const XqView &xq, int64_t Mpad, unsigned long long *trace, cudaStream_t st, bool interleaved);
// Q4_K decode linear on the integer tensor-memory path (tcgen05.mma kind::i8), M <= 8: the activation pass, then one
// kernel (ttq_q4k_umma.cu).  `ws` / `counters` as for launch_q4k_mma.  cudaErrorNotSupported: take another path.
cudaError_t launch_q4k_umma(const LinearArgs &a, const XqView &xq, int64_t xq_capacity_k, int sms, int *status, unsigned long long *trace,
                            float *ws, size_t ws_bytes, unsigned *counters, int64_t counters_cap, cudaStream_t st, int *launches);
// Q4_K decode linear on fp16 tensor-core instructions, M <= 16, activations converted inside the kernel
// (ttq_q4k_mma.cu).  `ws` / `counters`: fp32 workspace and per-row-tile arrival counters (zero between launches)
// for matrices whose K is split across CTAs.  cudaErrorNotSupported: the caller takes another path.
bool q4k_mma_supported(const LinearArgs &a);
cudaError_t launch_q4k_mma(const LinearArgs &a, int sms, int *status, unsigned long long *trace, float *ws, size_t ws_bytes,
                           unsigned *counters, int64_t counters_cap, cudaStream_t st, int *launches, const CommView *comm = nullptr);
constexpr int TTQ_TRACE_ENTRIES = 8192;
// tcgen05 dequant-GEMM for M > MAX_GEMV_M (formats for which gemm_supported() is true)
bool gemm_supported(int fmt);
// `wimg` != nullptr selects the plain mode: both operands are fp16 tile images (the trellis format's expansion).
cudaError_t launch_gemm(int fmt, const LinearArgs &a, __half *xh, int64_t xh_capacity, int sms, int *status,
                        unsigned long long *trace, cudaStream_t st, int *launches, const __half *wimg = nullptr);
// rows of the fp16 tile images the plain GEMM mode reads: [Kp / 64][Np / 8][1024 B], Np = gemm_wimg_rows(N); rows >= N
// and columns >= K are zero (written by launch_tq3_wimg)
int64_t gemm_wimg_rows(int64_t N);
cudaError_t launch_silu_and_mul(const void *in, int dt, int64_t M, int64_t H, int64_t ld_in, void *out,
                                int64_t ld_out, cudaStream_t st);

// ---------------------------------------------------------------------------------------------
// small device helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float load_as_float(const void *p, int dt, int64_t i) {
    if (dt == TTQ_DT_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
    if (dt == TTQ_DT_F16) return __half2float(reinterpret_cast<const __half *>(p)[i]);
    return reinterpret_cast<const float *>(p)[i];
}
__device__ __forceinline__ void store_from_float(void *p, int dt, int64_t i, float v) {
    if (dt == TTQ_DT_BF16) reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
    else if (dt == TTQ_DT_F16) reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
    else reinterpret_cast<float *>(p)[i] = v;
}

// (a & b) | c in one instruction with both constants in registers (written with immediates the compiler emits
// two instructions; hold b and c in variables made opaque by an empty asm statement).
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Q4_K: unpack the 6-bit scale (sc) and min (m) of sub-block j from the 12 packed bytes.
__device__ __forceinline__ void q4k_scale_min(int j, const uint8_t *s, int &sc, int &m) {
    if (j < 4) {
        sc = s[j] & 63;
        m = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0x0f) | ((s[j - 4] >> 6) << 4);
        m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

}  // namespace ttq
