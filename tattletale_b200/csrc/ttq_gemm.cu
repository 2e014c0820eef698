// Prefill / batched side: y[M][N] = x . W^T on the 5th-generation tensor cores (tcgen05.mma, kind::f16,
// cta_group::1, fp32 accumulators in tensor memory).
//
// Operand roles.  The 128 rows (tensor-memory lanes) of the MMA are 128 ACTIVATION rows; its N dimension is the
// CTA's 128 * NSUB expanded weight rows, so an epilogue thread owns one output row and stores runs of 16
// consecutive features.  A row tile of BM = 64, 128 or 256 (grouped mode also 384) activation rows is MH = BM / 128
// row blocks that share one expanded weight stage.
//
// Persistent CTAs (one per SM) walk output tiles of (128 * NSUB weight rows) x (BM activation rows); K may be cut
// into `splits` work units whose fp32 partials a small kernel sums when the tiles alone cannot fill the SMs.
// 21 warps per CTA:
//   warps 0-3    epilogue: tcgen05.ld of their 32 accumulator lanes -> bias -> y (or split-K partials).  Two
//                accumulator sets in tensor memory alternate when they fit, so the epilogue of a tile overlaps the
//                next tile's MMAs.
//   warps 4-19   dequantize: with two sub-tiles every warp owns one packed row tile (16 weight rows) of the CTA's 256
//                and works on every stage; with one sub-tile two groups of 8 warps take the even and the odd
//                stages.  A warp reads one 512-byte chunk per stage straight from global memory (16 bytes per lane,
//                prefetched two stages ahead), expands nibbles to fp16 with the 1024-offset bit trick, applies the
//                sub-block scale and offset with one HFMA2 per pair, and writes the 128-byte-swizzled K-major
//                weight tile.  Lane 0 of the first of them also brings the activation tile in with a single bulk
//                async copy per stage (xh_prep_kernel stores fp16 activations as ready-made swizzled tile images).
//                In the plain mode (weights already expanded to fp16 images by another kernel) these warps idle
//                except for one producer lane that bulk-copies both operands.
//   warp 20      allocates tensor memory, issues the MMAs (one elected lane) and commits them to the stage
//                barriers.
// A stage is one window of one 256-weight super-block: 64 K values (8 from each sub-block), in the order the
// packed chunk delivers them; the activation pass applies the same K permutation, so the dequant warps never
// shuffle.  Grouped (mixture-of-experts) mode: every row tile belongs to one weight matrix, named by device-side
// tables.  Every mbarrier wait is bounded; tensor memory is always released.
#include <cstdlib>

#include "ttq_internal.cuh"

namespace ttq {

namespace {

constexpr int GEMM_EPI_WARPS = 4;
// 16 dequant warps + 1 MMA warp.  Two sub-tiles: one warp per packed row tile of the CTA's 256 weight rows, every
// warp works on every stage.  One sub-tile: the 8 row tiles are served by two groups of 8 warps that take the
// even and the odd stages, so that two stages are expanded at the same time.
__host__ __device__ constexpr int gemm_deq_warps(int) { return 16; }
__host__ __device__ constexpr int gemm_warps(int nsub) { return GEMM_EPI_WARPS + gemm_deq_warps(nsub) + 1; }
constexpr int GEMM_BN = 128;                     // weight rows per CTA = MMA M
constexpr int A_STAGE_BYTES = GEMM_BN * 128;     // 128 rows x 64 fp16
constexpr int GEMM_WAIT_LIMIT = 1 << 22;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: after GEMM_WAIT_LIMIT polls the failure is recorded and the caller carries on (with
// garbage data) so that every role still finishes and tensor memory is released.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int *status) {
    for (int i = 0; i < GEMM_WAIT_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    report_failure(status, 2);
    return false;
}
// Warp-wide form: lane 0 polls, the others park at the warp barrier (fewer shared-memory polls next to the
// tensor core's operand reads).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, int *status, int lane) {
    bool ok = true;
    if (lane == 0) ok = mbar_wait_bounded(bar, parity, status);
    __syncwarp();
    return __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes,
// 8-row atoms of 1024 bytes stacked contiguously (stride byte offset 1024), descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    const uint32_t lo = ((addr & 0x3ffffu) >> 4) | (1u << 16);          // start address, leading byte offset (unused) = 1
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);         // stride byte offset, version = 1, SWIZZLE_128B
    return ((uint64_t)hi << 32) | lo;
}
// Instruction descriptor, kind::f16: D = f32, A = B = f16, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t idesc_f16(int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((128u >> 4) << 24); }

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// The same load without the wait, and the wait: the registers pass through the wait statement so that no use of them
// is scheduled before it.
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&v)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]),
                   "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
                 :
                 : "memory");
}

// ---- activation pass: x [M][K] (bf16 | f16) -> fp16 tile images ------------------------------------
// Output layout: [stage it = 4*sb + s][row atom m/8][1024 bytes]: the 8 rows x 128 bytes of one
// swizzle atom exactly as they must sit in shared memory, so that the B tile of a stage (BM rows) is
// ONE contiguous run of BM*128 bytes.  Inside a row, 16-byte chunk j (sub-block j) sits at position
// j ^ (m & 7) and holds, at pos = 4*half + p, the activation of K index
// sb*256 + 32*j + 8*s + 4*half + perm[p], perm = {0, 2, 1, 3} -- the order in which the nibble
// expansion of the dequant warps emits a register's four weights.
//
// Grouped (mixture-of-experts) use: `row_src` (optional) names the source row of every image row
// (-1 = a padding row of zeros), `rows_used` (optional, device scalar in units of `rows_unit` rows)
// bounds the rows worth converting, and GATED = true reads a row of 2K values and emits
// silu(x[k]) * x[K + k] (the gated-MLP activation, fused into the conversion).
// `kmap` = 1 selects the Q6_K stage order: slot j of stage s = 2s' + n holds window n of the 16-wide sub-block
// 4s' + 8 (j & 1) + (j >> 1) (low nibbles: set s', high nibbles: set s' + 2 of the packed chunk).
template <bool GATED>
__global__ void __launch_bounds__(256) xh_prep_kernel(const void *__restrict__ x, int x_dt, int64_t M, int64_t Mp, int64_t K,
                                                      int64_t Kp, int64_t ldx, __half *__restrict__ xh,
                                                      const int *__restrict__ row_src, const int *__restrict__ rows_used,
                                                      int rows_unit, int kmap) {
    grid_dependency_wait();  // x, the routing tables and the image buffer belong to preceding kernels until here
    const int64_t chunks_per_row = Kp / 8;
    const int64_t total = Mp * chunks_per_row;
    const int64_t m_used = rows_used != nullptr ? (int64_t)(*rows_used) * rows_unit : Mp;
    for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < total; c += (int64_t)gridDim.x * blockDim.x) {
        // consecutive threads: consecutive j, then rows, then stages (coalesced 16-byte stores per atom)
        const int j = (int)(c & 7);
        const int64_t mi = (c >> 3) % Mp, it = (c >> 3) / Mp;
        if (mi >= m_used) continue;
        const int64_t sb = it >> 2;
        const int s = (int)(it & 3);
        const int64_t k0 = kmap == 0 ? sb * 256 + 32 * j + 8 * s : sb * 256 + 16 * (4 * (s >> 1) + 8 * (j & 1) + (j >> 1)) + 8 * (s & 1);
        // source row: the image row itself, or the row the routing table names (negative = padding)
        int64_t m = mi;
        if (row_src != nullptr) {
            const int r = row_src[mi];
            m = r < 0 ? M : (int64_t)r;
        }
        // the 8 source values are contiguous in K: one 16-byte load when the row is aligned
        __half src[8];
        const bool vec = x_dt != TTQ_DT_F32 && m < M && k0 + 8 <= K &&
                         ((reinterpret_cast<uintptr_t>(x) + (size_t)(m * ldx + k0) * 2) & 15) == 0 && (!GATED || ((K * 2) & 15) == 0);
        if (GATED) {
#pragma unroll
            for (int i = 0; i < 8; i++) src[i] = __float2half_rn(0.f);
            if (vec && x_dt == TTQ_DT_F16) {
                const __half *row = reinterpret_cast<const __half *>(x) + m * ldx + k0;
                const uint4 ga = *reinterpret_cast<const uint4 *>(row), ua = *reinterpret_cast<const uint4 *>(row + K);
                const __half2 *g2 = reinterpret_cast<const __half2 *>(&ga), *u2 = reinterpret_cast<const __half2 *>(&ua);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const float2 gv = __half22float2(g2[q]), uv = __half22float2(u2[q]);
                    src[2 * q] = __float2half_rn(gv.x / (1.f + expf(-gv.x)) * uv.x);
                    src[2 * q + 1] = __float2half_rn(gv.y / (1.f + expf(-gv.y)) * uv.y);
                }
            } else if (m < M) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    if (k0 + i < K) {
                        const float gv = load_as_float(x, x_dt, m * ldx + k0 + i), uv = load_as_float(x, x_dt, m * ldx + K + k0 + i);
                        src[i] = __float2half_rn(gv / (1.f + expf(-gv)) * uv);
                    }
                }
            }
        } else if (vec) {
            const uint4 raw = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(x) + m * ldx + k0);
            if (x_dt == TTQ_DT_F16) {
                *reinterpret_cast<uint4 *>(src) = raw;
            } else {
                const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    src[2 * q] = __float2half_rn(__uint_as_float(w[q] << 16));
                    src[2 * q + 1] = __float2half_rn(__uint_as_float(w[q] & 0xffff0000u));
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                float v = 0.f;
                if (m < M && k0 + i < K) v = load_as_float(x, x_dt, m * ldx + k0 + i);
                src[i] = __float2half_rn(v);
            }
        }
        __half out[8];
#pragma unroll
        for (int p = 0; p < 8; p++) out[p] = src[(p & 4) + ((p & 1) << 1) + ((p & 2) >> 1)];  // swap the middle two of each four
        const int64_t dst = ((it * (Mp >> 3) + (mi >> 3)) << 10) + ((mi & 7) << 7) + ((int64_t)(j ^ (int)(mi & 7)) << 4);
        *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(xh) + dst) = *reinterpret_cast<const uint4 *>(out);
    }
    // only now may the GEMM be set up: its one-per-SM CTAs would otherwise take the SMs from the waves of this
    // bandwidth-bound pass that are still queued
    grid_launch_dependents();
}

struct GemmParams {
    const uint8_t *tiles;  // Q4_K tiled layout
    int64_t N, NT, SBp;
    const __half *xh;      // tile images, see xh_prep_kernel
    int64_t M, Mp, Kp;
    const void *bias;
    int bias_dt;
    void *y;
    int y_dt;
    int64_t ldy;
    int *status;
    unsigned long long *trace;  // optional: [0] entry counter, entries of 8 words from [8] (see ttq.h)
    int splits;   // K is cut in `splits` equal runs of super-blocks, one work unit each (1 = no split)
    float *ws;    // splits > 1: fp32 partial outputs [split][Mp][N], summed by splitk_reduce_kernel
    // grouped (mixture-of-experts) mode, group_tiles != nullptr: every BM-row tile of x belongs to one
    // weight matrix (all of one shape); the number of row tiles in use is a device scalar
    // plain mode (kernel template PLAIN): the weights arrive already expanded to fp16 tile images in the layout
    // of xh_prep_kernel ([stage][row atom][1024 B], rows = output features padded to 256); `tiles` is unused
    const __half *wimg;
    int64_t Np;
    const uint8_t *const *group_tiles;  // per group: Q4_K tiled layout
    const int *mt_group;                // group of row tile mt
    const int *mt_row0;                 // first row of row tile mt in the routed row space (a multiple of 64)
    const int *mt_mh;                   // BM = 384 only: 128-row blocks of row tile mt in use (1..3)
    const int *n_mt;                    // row tiles in use (<= mt_cap)
    int64_t mt_cap;                     // row tiles the tables and the grid are sized for
};

template <int BM, int NSUB>
struct GemmCfg {
    static constexpr int A_BYTES = NSUB * A_STAGE_BYTES;
    static constexpr int B_BYTES = BM * 128;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = STAGE_BYTES > 48 * 1024 ? 3 : 4;
    // The MMA's M side is a run of 128 activation rows (tensor-memory lanes), its N side the CTA's 128 * NSUB
    // weight rows (columns): an accumulator set is MH row blocks of 128 * NSUB columns.
    static constexpr int MH = BM > 128 ? BM / 128 : 1;
    static constexpr int ACC_COLS = MH * 128 * NSUB;
    static constexpr int NACC = (2 * ACC_COLS <= 512) ? 2 : 1;   // accumulator sets in tensor memory
    static constexpr int TMEM_COLS = NACC * ACC_COLS <= 128 ? 128 : (NACC * ACC_COLS <= 256 ? 256 : 512);  // a power of two
    static constexpr int DEQ_WARPS = gemm_deq_warps(NSUB), WARPS = gemm_warps(NSUB), THREADS = WARPS * 32;
    static constexpr int HDR_BYTES = DEQ_WARPS * 1280;  // per dequant warp: 16 rows x 80 bytes
    static constexpr int BAR_BYTES = 128;
    // + 1024 slack to align the first stage to the swizzle atom
    static constexpr int TOTAL = 1024 + STAGES * STAGE_BYTES + HDR_BYTES + BAR_BYTES;
};

// MODE: which weights the CTA multiplies -- a packed format expanded by the dequant warps (GM_Q4K, GM_Q8_0, GM_Q6K)
// or fp16 tile images expanded beforehand by another kernel (GM_PLAIN).
constexpr int GM_Q4K = 0, GM_PLAIN = 1, GM_Q8_0 = 2, GM_Q6K = 3;
__host__ __device__ constexpr int gm_format(int mode) { return mode == GM_Q8_0 ? TTQ_FMT_Q8_0 : (mode == GM_Q6K ? TTQ_FMT_Q6_K : TTQ_FMT_Q4_K); }

template <int BM, int NSUB, int MODE>
__global__ void __launch_bounds__(GemmCfg<BM, NSUB>::THREADS, 1) gemm_q4k_kernel(GemmParams p) {
    constexpr bool PLAIN = MODE == GM_PLAIN;
    extern __shared__ uint8_t smem_raw[];
    using C = GemmCfg<BM, NSUB>;
    constexpr int STAGES = C::STAGES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t stages_u32 = base;
    const uint32_t hdr_u32 = base + STAGES * C::STAGE_BYTES;
    const uint32_t bars_u32 = hdr_u32 + C::HDR_BYTES;
    // barriers: full[STAGES], empty[STAGES], accum_full[2], accum_empty[2]; then the tensor-memory address slot
    const uint32_t full_bar = bars_u32, empty_bar = bars_u32 + 8 * STAGES;
    const uint32_t accf_bar = bars_u32 + 16 * STAGES, acce_bar = accf_bar + 16;
    volatile uint32_t *tmem_slot =
        reinterpret_cast<volatile uint32_t *>(base_ptr + STAGES * C::STAGE_BYTES + C::HDR_BYTES + 16 * STAGES + 32);
    const int splits = p.splits, sb_per_unit = (int)p.SBp / splits;
    const int iters = sb_per_unit * 4;  // stages per work unit (tile x K split)
    constexpr int TILE_N = GEMM_BN * NSUB;
    const bool grouped = p.group_tiles != nullptr;
    // Programmatic dependent launch: the set-up below (barriers, tensor memory) and the first loads of packed
    // weights -- constant data -- run while the preceding kernel drains; everything that touches activations,
    // routing tables or outputs comes after grid_dependency_wait.
    grid_launch_dependents();
    if (grouped) grid_dependency_wait();  // the row-tile tables are read right away
    int64_t m_tiles = p.Mp / BM;
    if (grouped) {
        const int64_t used = *p.n_mt;
        m_tiles = used < p.mt_cap ? used : p.mt_cap;
    }
    const int64_t n_tiles = (p.N + TILE_N - 1) / TILE_N, total_tiles = n_tiles * m_tiles * splits;
    // Order of the output tiles.  Dense: all row tiles of one weight tile are neighbours (few row tiles, the weights are
    // the big operand and are read once).  Grouped: all weight tiles of one row tile are neighbours, so that the CTAs
    // running together share the row tile's activation images and an expert's weights through L2 -- the routed
    // activations (hundreds of MB) would otherwise be re-read from DRAM once per weight tile.
    auto tile_n = [&](int64_t otile) -> int64_t { return grouped ? otile % n_tiles : otile / m_tiles; };
    auto tile_m = [&](int64_t otile) -> int64_t { return grouped ? otile / n_tiles : otile % m_tiles; };
    // first activation row of a row tile; 128-row blocks of it in use (variable only for the 384-row grouped tile)
    auto tile_row0 = [&](int64_t m_tile) -> int64_t { return grouped ? (int64_t)p.mt_row0[m_tile] : m_tile * BM; };
    auto tile_mh = [&](int64_t m_tile) -> int { return (grouped && BM == 384) ? p.mt_mh[m_tile] : C::MH; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full_bar + 8 * s, PLAIN ? 1 : (NSUB == 1 ? 8 : C::DEQ_WARPS) + 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(accf_bar + 8 * b, 1);
            mbar_init(acce_bar + 8 * b, GEMM_EPI_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == C::WARPS - 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_slot)),
                     "r"((uint32_t)C::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < GEMM_EPI_WARPS) {
        // ------------------------------------------------------------------ epilogue
        grid_dependency_wait();  // the output may still be read by a preceding kernel
        bool alive = true;
        int tcount = 0;
        for (int64_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, tcount++) {
            const int64_t otile = tile / splits, split = tile % splits;
            const int64_t n_tile = tile_n(otile), m_tile = tile_m(otile);
            const int buf = tcount % C::NACC, use = tcount / C::NACC;
            if (alive) alive = mbar_wait_warp(accf_bar + 8 * buf, (uint32_t)(use & 1), p.status, lane);
            tc_fence_after();
            const int64_t m0 = tile_row0(m_tile);
            const int mh = tile_mh(m_tile);
            float *wsp = p.ws + (size_t)split * p.Mp * p.N;
            const int esz = p.y_dt == TTQ_DT_F32 ? 4 : 2;
#pragma unroll 1
            for (int hb = 0; hb < mh; hb++) {
                // lane = activation row, columns = consecutive output features: 16 of them per load, stored as one run
                const int64_t m = m0 + hb * 128 + warp * 32 + lane;
                const bool row_ok = m < p.M && hb * 128 + warp * 32 + lane < BM;  // a 64-row tile fills lanes 0..63 only
#pragma unroll 1
                for (int c0 = 0; c0 < 128 * NSUB; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(buf * C::ACC_COLS + hb * 128 * NSUB + c0), v);
                    const int64_t n0 = n_tile * TILE_N + c0;
                    if (!row_ok || n0 >= p.N) continue;
                    if (splits > 1) {
                        float *dst = wsp + m * p.N + n0;
                        if (n0 + 16 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                            for (int q = 0; q < 4; q++)
                                reinterpret_cast<float4 *>(dst)[q] = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                                                                 __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; i++)
                                if (n0 + i < p.N) dst[i] = __uint_as_float(v[i]);
                        }
                        continue;
                    }
                    float f[16];
#pragma unroll
                    for (int i = 0; i < 16; i++) f[i] = __uint_as_float(v[i]);
                    if (p.bias != nullptr) {
#pragma unroll
                        for (int i = 0; i < 16; i++)
                            if (n0 + i < p.N) f[i] += load_as_float(p.bias, p.bias_dt, n0 + i);
                    }
                    uint8_t *dst = reinterpret_cast<uint8_t *>(p.y) + (size_t)(m * p.ldy + n0) * esz;
                    if (n0 + 16 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                        if (p.y_dt == TTQ_DT_F32) {
#pragma unroll
                            for (int q = 0; q < 4; q++)
                                reinterpret_cast<float4 *>(dst)[q] = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
                        } else {
                            uint32_t w[8];
#pragma unroll
                            for (int q = 0; q < 8; q++) {
                                if (p.y_dt == TTQ_DT_BF16) {
                                    const __nv_bfloat162 t2 = __floats2bfloat162_rn(f[2 * q], f[2 * q + 1]);
                                    w[q] = *reinterpret_cast<const uint32_t *>(&t2);
                                } else {
                                    const __half2 t2 = __floats2half2_rn(f[2 * q], f[2 * q + 1]);
                                    w[q] = *reinterpret_cast<const uint32_t *>(&t2);
                                }
                            }
                            reinterpret_cast<uint4 *>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                            reinterpret_cast<uint4 *>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; i++)
                            if (n0 + i < p.N) store_from_float(p.y, p.y_dt, m * p.ldy + n0 + i, f[i]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar + 8 * buf);
        }
    } else if (PLAIN && warp < GEMM_EPI_WARPS + C::DEQ_WARPS) {
        // ------------------------------------------------------------------ producer: both operands are bulk copies
        if (warp == GEMM_EPI_WARPS && lane == 0) {
            grid_dependency_wait();  // both operands are written by preceding kernels
            bool alive = true;
            int git = 0;
            const int64_t b_it_stride = (p.Mp >> 3) << 10, w_it_stride = (p.Np >> 3) << 10;
            for (int64_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
                const int64_t otile = tile / splits, split = tile % splits;
                const int64_t n_tile = tile_n(otile), m_tile = tile_m(otile);
                const uint8_t *bsrc0 = reinterpret_cast<const uint8_t *>(p.xh) + ((tile_row0(m_tile) >> 3) << 10) + split * iters * b_it_stride;
                const uint8_t *wsrc0 = reinterpret_cast<const uint8_t *>(p.wimg) + (((n_tile * TILE_N) >> 3) << 10) + split * iters * w_it_stride;
                for (int it = 0; it < iters; it++, git++) {
                    const int stage = git % STAGES;
                    if (git >= STAGES && alive)
                        alive = mbar_wait_bounded(empty_bar + 8 * stage, (uint32_t)(((git / STAGES) - 1) & 1), p.status);
                    const uint32_t a_stage = stages_u32 + stage * C::STAGE_BYTES;
                    mbar_expect_tx(full_bar + 8 * stage, C::A_BYTES + C::B_BYTES);
                    bulk_g2s(a_stage, wsrc0 + it * w_it_stride, C::A_BYTES, full_bar + 8 * stage);
                    bulk_g2s(a_stage + C::A_BYTES, bsrc0 + it * b_it_stride, C::B_BYTES, full_bar + 8 * stage);
                }
            }
        }
        __syncwarp();
    } else if (warp < GEMM_EPI_WARPS + C::DEQ_WARPS) {
        // ------------------------------------------------------------------ dequantize A
        // A stage is 64 K values of the CTA's weight rows.  For every format it is a set of 512-byte chunks of the tiled
        // layout, in which lane (g, t) holds, per register sl, four bytes of row g + 8 (sl & 1) and group
        // u = (t >> 1) + 2 (sl >> 1) at positions 4 (t & 1) .. +3 of an 8-wide window:
        //   Q4_K  stage s = window s of the 8 sub-blocks: one chunk; byte = {low nibble: sub-block 2u, high: 2u+1}
        //   Q8_0  stage s = window s of the 8 blocks: chunk s (blocks 0..3 = group u) and chunk 4 + s (blocks 4..7)
        //   Q6_K  stage (s', n) = window n of the sub-blocks of sets s' and s'+2: chunk 2s'+n of low nibbles
        //         {low: sub-block 4s'+u, high: 4s'+8+u} and chunk n of the 2-bit planes (bit pair s of a byte = set s)
        // Each register becomes runs of four fp16 values (k order 0 2 1 3) stored into 16-byte slot `j` of the row's
        // 128-byte swizzled line; xh_prep_kernel lays the activations out with the same slot -> K mapping.
        constexpr int FMT = gm_format(MODE);
        constexpr int TB = tile_bytes(FMT);
        const int dwa = warp - GEMM_EPI_WARPS;  // dequant warp index
        constexpr bool PARITY = NSUB == 1;  // two groups of 8 warps alternate over the stages of the single sub-tile
        constexpr int STRIDE = PARITY ? 2 : 1;
        const int dw = dwa & 7;                      // row tile inside the 128-row sub-tile
        const int my_sub = PARITY ? 0 : dwa >> 3;    // sub-tile
        const int grp = PARITY ? dwa >> 3 : 0;       // first stage of a tile this warp expands
        const int g = lane >> 2, t = lane & 3;
        const int r = lane & 15, h = lane >> 4;
        const uint32_t my_hdr = hdr_u32 + dwa * 1280;
        // byte offsets (inside a 128-row A sub-tile) of this lane's stores: register sl, slot pair
        const int u0 = t >> 1, u1 = 2 + (t >> 1);
        // Q4_K: lanes with t >= 2 take their four packed words in the order 2, 3, 0, 1.  A store instruction of 8 bytes per
        // lane is served half a warp at a time, and the 16 lanes of a half (rows g = 0..3) then write eight different
        // 16-byte columns of the swizzled rows instead of four, twice each: half the shared-memory wavefronts.
        const bool swp = MODE == GM_Q4K && (t & 2) != 0;
        uint32_t dst_off[4][2], hdr_off[4];
#pragma unroll
        for (int slp = 0; slp < 4; slp++) {
            const int sl = swp ? (slp ^ 2) : slp;
            const int u = (sl >> 1) ? u1 : u0;
            const int row = dw * 16 + g + 8 * (sl & 1);
            const uint32_t key = (uint32_t)(row & 7);
            // Q4_K, Q6_K: slots 2u (low nibbles) and 2u+1 (high nibbles).  Q8_0: slots u (first chunk) and 4 + u (second)
            const uint32_t j0 = MODE == GM_Q8_0 ? (uint32_t)u : (uint32_t)(2 * u), j1 = MODE == GM_Q8_0 ? (uint32_t)(4 + u) : (uint32_t)(2 * u + 1);
            dst_off[slp][0] = (uint32_t)row * 128 + ((j0 ^ key) << 4) + (uint32_t)(t & 1) * 8;
            dst_off[slp][1] = (uint32_t)row * 128 + ((j1 ^ key) << 4) + (uint32_t)(t & 1) * 8;
            // per-row scale records in the warp's header area (80-byte rows): Q4_K {scale2, offset2} per sub-block (8 B),
            // Q8_0 scale2 per block (4 B), Q6_K scale2 per 16-wide sub-block (4 B)
            hdr_off[slp] = (uint32_t)((g + 8 * (sl & 1)) * 80) + (MODE == GM_Q4K ? (uint32_t)(2 * u * 8) : (uint32_t)(u * 4));
        }
        bool alive = true;
        int git_base = 0;  // stage counter across tiles, at the start of the current tile
        const int64_t b_it_stride = (p.Mp >> 3) << 10;
        // packed row tile of this warp in an output tile: (n_tile * NSUB + my_sub) * 8 + dw
        auto tile_ptr = [&](int64_t tile, bool &have) {
            const int64_t nt = (tile_n(tile / splits) * NSUB + my_sub) * (GEMM_BN / TILE_ROWS) + dw;
            have = tile < total_tiles && nt < p.NT;
            const uint8_t *wbase = p.tiles;
            if (grouped && have) wbase = p.group_tiles[p.mt_group[tile_m(tile / splits)]];
            return wbase + ((have ? nt : 0) * p.SBp + (tile % splits) * sb_per_unit) * TB;
        };
        struct Chunks {
            uint4 a, b;  // b: second chunk of the stage (Q8_0: blocks 4..7, Q6_K: the 2-bit planes); unused for Q4_K
        };
        auto chunk_at = [&](const uint8_t *t0, bool ok, int it) {
            Chunks c;
            c.a = c.b = make_uint4(0, 0, 0, 0);
            if (ok) {
                const uint8_t *base = t0 + (int64_t)(it >> 2) * TB + lane * 16;
                const int s = it & 3;
                if constexpr (MODE == GM_Q4K) {
                    c.a = *reinterpret_cast<const uint4 *>(base + s * 512);
                } else if constexpr (MODE == GM_Q8_0) {
                    c.a = *reinterpret_cast<const uint4 *>(base + s * 512);
                    c.b = *reinterpret_cast<const uint4 *>(base + (4 + s) * 512);
                } else {
                    c.a = *reinterpret_cast<const uint4 *>(base + s * 512);  // chunk 2s' + n with s = 2s' + n
                    c.b = *reinterpret_cast<const uint4 *>(base + 2048 + (s & 1) * 512);
                }
            }
            return c;
        };
        bool have;
        Chunks next, next2;  // chunks of the next two stages stay in flight
        struct Header {
            uint4 v;      // Q4_K: the row's 16 header bytes; Q8_0: its 8 fp16 block scales; Q6_K: its 16 int8 scales
            uint32_t d;   // Q6_K: the row's fp16 super-block scale
        };
        Header hv_next;   // row header of the next super-block (loaded one super-block ahead)
        auto header_at = [&](const uint8_t *t0, bool ok, int sb) {
            Header hd;
            hd.v = make_uint4(0, 0, 0, 0);
            hd.d = 0;
            if (ok) {
                const uint8_t *tb = t0 + (int64_t)sb * TB;
                if constexpr (MODE == GM_Q4K) {
                    hd.v = *reinterpret_cast<const uint4 *>(tb + 2048 + r * 16);
                } else if constexpr (MODE == GM_Q8_0) {
                    hd.v = *reinterpret_cast<const uint4 *>(tb + 4096 + r * 16);
                } else {
                    hd.v = *reinterpret_cast<const uint4 *>(tb + 3072 + r * 16);
                    hd.d = *reinterpret_cast<const uint16_t *>(tb + 3328 + r * 2);
                }
            }
            return hd;
        };
        const uint8_t *tile0 = tile_ptr(blockIdx.x, have);
        next = chunk_at(tile0, have, grp);
        next2 = chunk_at(tile0, have && grp + STRIDE < iters, grp + STRIDE);
        hv_next = header_at(tile0, have, 0);
        grid_dependency_wait();  // the first packed chunks and headers are in flight; activations come next
        const __half2 k1032 = __float2half2_rn(1032.f), k1152 = __float2half2_rn(1152.f), k1056 = __float2half2_rn(1056.f);
        // constants of the nibble expansion, kept in registers (see and_or)
        uint32_t mask_lo = 0x000f000fu, mask_hi = 0x00f000f0u, mask_b = 0x00ff00ffu, k1024 = 0x64006400u;
        asm volatile("" : "+r"(mask_lo), "+r"(mask_hi), "+r"(mask_b), "+r"(k1024));
        const bool trd = p.trace != nullptr && blockIdx.x == 0 && dwa == 0;
        unsigned long long t_empty = 0, t_conv = 0, t_begin = trd ? global_ns() : 0;
        for (int64_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            bool have_n;
            const uint8_t *tile0_n = tile_ptr(tile + gridDim.x, have_n);
            const int64_t m_tile_b = tile_m(tile / splits);
            const uint8_t *bsrc0 = reinterpret_cast<const uint8_t *>(p.xh) + ((tile_row0(m_tile_b) >> 3) << 10) +
                                   (tile % splits) * iters * b_it_stride;
            const uint32_t b_bytes = BM == 384 ? (uint32_t)tile_mh(m_tile_b) * (128u * 128u) : (uint32_t)C::B_BYTES;
            for (int it = grp; it < iters; it += STRIDE) {
                const int git = git_base + it;  // iters is a multiple of 4: a warp group keeps its stage parity across tiles
                const int sb = it >> 2;
                const int stage = git % STAGES;
                const Chunks w = next;
                next = next2;
                if (it + 2 * STRIDE < iters) next2 = chunk_at(tile0, have, it + 2 * STRIDE);
                else next2 = chunk_at(tile0_n, have_n && (it + 2 * STRIDE - iters) < iters, it + 2 * STRIDE - iters);
                if ((it & 3) == grp) {
                    // first own stage of a super-block: lane (r, h) unpacks half h of row r's scales into the header area
                    __syncwarp();
                    {
                        const Header hd = hv_next;
                        if (sb + 1 < sb_per_unit) hv_next = header_at(tile0, have, sb + 1);
                        else hv_next = header_at(tile0_n, have_n, 0);
                        const uint4 hv = hd.v;
                        if constexpr (MODE == GM_Q4K) {
                            // sub-blocks 4h..4h+3: {scale, scale, offset, offset} halves, w = scale*(q-8) + offset (high
                            // nibbles arrive as 16*(q-8))
                            const __half2 dd = *reinterpret_cast<const __half2 *>(&hv.x);
                            const float d = __low2float(dd), dmin = __high2float(dd);
                            uint32_t scw, mw;
                            if (h == 0) {
                                scw = hv.y & 0x3f3f3f3fu;
                                mw = hv.z & 0x3f3f3f3fu;
                            } else {
                                scw = (hv.w & 0x0f0f0f0fu) | ((hv.y >> 2) & 0x30303030u);
                                mw = ((hv.w >> 4) & 0x0f0f0f0fu) | ((hv.z >> 2) & 0x30303030u);
                            }
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                const float sc = d * (float)((scw >> (8 * i)) & 0xff);
                                const float off = fmaf(8.f, sc, -dmin * (float)((mw >> (8 * i)) & 0xff));
                                const __half2 s2 = __float2half2_rn((i & 1) ? sc * 0.0625f : sc);
                                const __half2 o2 = __float2half2_rn(off);
                                asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(my_hdr + (uint32_t)(r * 80 + (4 * h + i) * 8)),
                                             "r"(*reinterpret_cast<const uint32_t *>(&s2)), "r"(*reinterpret_cast<const uint32_t *>(&o2))
                                             : "memory");
                            }
                        } else if constexpr (MODE == GM_Q8_0) {
                            // blocks 4h..4h+3: the fp16 scale d, duplicated into both halves
                            const uint32_t lo = h == 0 ? hv.x : hv.z, hi = h == 0 ? hv.y : hv.w;
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(my_hdr + (uint32_t)(r * 80 + h * 16)),
                                         "r"(__byte_perm(lo, 0, 0x1010)), "r"(__byte_perm(lo, 0, 0x3232)), "r"(__byte_perm(hi, 0, 0x1010)),
                                         "r"(__byte_perm(hi, 0, 0x3232))
                                         : "memory");
                        } else {
                            // 16-wide sub-blocks 8h..8h+7: d * sc as fp16, duplicated into both halves
                            const float d = __half2float(__ushort_as_half((unsigned short)hd.d));
                            const uint32_t lo = h == 0 ? hv.x : hv.z, hi = h == 0 ? hv.y : hv.w;
                            uint32_t sw[8];
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                const float sc = d * (float)(int)(int8_t)(((i < 4 ? lo : hi) >> (8 * (i & 3))) & 0xff);
                                const __half2 s2 = __float2half2_rn(sc);
                                sw[i] = *reinterpret_cast<const uint32_t *>(&s2);
                            }
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(my_hdr + (uint32_t)(r * 80 + h * 32)), "r"(sw[0]),
                                         "r"(sw[1]), "r"(sw[2]), "r"(sw[3])
                                         : "memory");
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(my_hdr + (uint32_t)(r * 80 + h * 32 + 16)), "r"(sw[4]),
                                         "r"(sw[5]), "r"(sw[6]), "r"(sw[7])
                                         : "memory");
                        }
                    }
                    __syncwarp();
                }
                unsigned long long tw0 = trd ? global_ns() : 0;
                if (git >= STAGES && alive)
                    alive = mbar_wait_warp(empty_bar + 8 * stage, (uint32_t)(((git / STAGES) - 1) & 1), p.status, lane);
                if (trd) {
                    tw0 = global_ns() - tw0;
                    t_empty += tw0;
                    tw0 = global_ns();
                }
                const uint32_t a_stage = stages_u32 + stage * C::STAGE_BYTES;
                if (dw == 0 && my_sub == 0 && lane == 0) {
                    // the activation tile of this stage: one bulk copy, counted on the same full barrier
                    mbar_expect_tx(full_bar + 8 * stage, b_bytes);
                    bulk_g2s(a_stage + C::A_BYTES, bsrc0 + it * b_it_stride, b_bytes, full_bar + 8 * stage);
                }
                {
                    const uint32_t wa[4] = {swp ? w.a.z : w.a.x, swp ? w.a.w : w.a.y, swp ? w.a.x : w.a.z, swp ? w.a.y : w.a.w};
                    const uint32_t a_sub = a_stage + my_sub * A_STAGE_BYTES;
                    // three phases (loads, arithmetic, stores) so that the shared-memory latencies overlap
                    __half2 res[4][4];  // per register: the two fp16 pairs of slot j0, then of slot j1
                    if constexpr (MODE == GM_Q4K) {
                        uint4 so[4];  // {scale2, offset2} of sub-blocks 2u (low nibbles) and 2u+1 (high nibbles) per slot
#pragma unroll
                        for (int sl = 0; sl < 4; sl++)
                            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                         : "=r"(so[sl].x), "=r"(so[sl].y), "=r"(so[sl].z), "=r"(so[sl].w)
                                         : "r"(my_hdr + hdr_off[sl]));
#pragma unroll
                        for (int sl = 0; sl < 4; sl++) {
                            const __half2 sc_lo = *reinterpret_cast<const __half2 *>(&so[sl].x), of_lo = *reinterpret_cast<const __half2 *>(&so[sl].y);
                            const __half2 sc_hi = *reinterpret_cast<const __half2 *>(&so[sl].z), of_hi = *reinterpret_cast<const __half2 *>(&so[sl].w);
                            const uint32_t x = wa[sl], x8 = x >> 8;
                            uint32_t v0 = and_or(x, mask_lo, k1024), v1 = and_or(x8, mask_lo, k1024);  // 1024 + q
                            uint32_t v2 = and_or(x, mask_hi, k1024), v3 = and_or(x8, mask_hi, k1024);  // 1024 + 16 q
                            res[sl][0] = __hfma2(__hsub2(*reinterpret_cast<__half2 *>(&v0), k1032), sc_lo, of_lo);
                            res[sl][1] = __hfma2(__hsub2(*reinterpret_cast<__half2 *>(&v1), k1032), sc_lo, of_lo);
                            res[sl][2] = __hfma2(__hsub2(*reinterpret_cast<__half2 *>(&v2), k1152), sc_hi, of_hi);
                            res[sl][3] = __hfma2(__hsub2(*reinterpret_cast<__half2 *>(&v3), k1152), sc_hi, of_hi);
                        }
                    } else if constexpr (MODE == GM_Q8_0) {
                        const uint32_t wb[4] = {w.b.x, w.b.y, w.b.z, w.b.w};
                        uint32_t sc0[4], sc1[4];  // scale2 of block u (first chunk) and block 4 + u (second chunk)
#pragma unroll
                        for (int sl = 0; sl < 4; sl++) {
                            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(sc0[sl]) : "r"(my_hdr + hdr_off[sl]));
                            asm volatile("ld.shared.u32 %0, [%1+16];" : "=r"(sc1[sl]) : "r"(my_hdr + hdr_off[sl]));
                        }
#pragma unroll
                        for (int sl = 0; sl < 4; sl++) {
                            // int8 -> fp16: flip the sign bit (q + 128 in 0..255), OR into the mantissa of 1024, subtract 1152
                            const uint32_t x = wa[sl] ^ 0x80808080u, y = wb[sl] ^ 0x80808080u;
                            uint32_t v0 = and_or(x, mask_b, k1024), v1 = and_or(x >> 8, mask_b, k1024);
                            uint32_t v2 = and_or(y, mask_b, k1024), v3 = and_or(y >> 8, mask_b, k1024);
                            const __half2 s0 = *reinterpret_cast<const __half2 *>(&sc0[sl]), s1 = *reinterpret_cast<const __half2 *>(&sc1[sl]);
                            res[sl][0] = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&v0), k1152), s0);
                            res[sl][1] = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&v1), k1152), s0);
                            res[sl][2] = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&v2), k1152), s1);
                            res[sl][3] = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&v3), k1152), s1);
                        }
                    } else {
                        const uint32_t wb[4] = {w.b.x, w.b.y, w.b.z, w.b.w};
                        const int sp = (it & 3) >> 1;  // set s' of the low nibbles; the high nibbles are set s' + 2
                        uint32_t sc0[4], sc1[4];       // scale2 of sub-blocks 4s'+u and 4s'+8+u
#pragma unroll
                        for (int sl = 0; sl < 4; sl++) {
                            const uint32_t ha = my_hdr + hdr_off[sl] + (uint32_t)sp * 16;
                            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(sc0[sl]) : "r"(ha));
                            asm volatile("ld.shared.u32 %0, [%1+32];" : "=r"(sc1[sl]) : "r"(ha));
                        }
#pragma unroll
                        for (int sl = 0; sl < 4; sl++) {
                            // 6-bit quant = nibble | (two plane bits << 4); OR-ed into the mantissa of 1024, minus 1024 + 32
                            const uint32_t x = wa[sl], x8 = x >> 8;
                            const uint32_t pl = wb[sl] >> (2 * sp), ph = wb[sl] >> (2 * sp + 4);  // plane bits of set s', s'+2 at bits 0..1 of each byte
                            const uint32_t a02 = (pl << 4) & 0x00300030u, a13 = (pl >> 4) & 0x00300030u;
                            const uint32_t b02 = (ph << 4) & 0x00300030u, b13 = (ph >> 4) & 0x00300030u;
                            uint32_t v0 = and_or(x, mask_lo, k1024) | a02, v1 = and_or(x8, mask_lo, k1024) | a13;
                            uint32_t v2 = and_or(x >> 4, mask_lo, k1024) | b02, v3 = and_or(x8 >> 4, mask_lo, k1024) | b13;
                            const __half2 s0 = *reinterpret_cast<const __half2 *>(&sc0[sl]), s1 = *reinterpret_cast<const __half2 *>(&sc1[sl]);
                            res[sl][0] = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&v0), k1056), s0);
                            res[sl][1] = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&v1), k1056), s0);
                            res[sl][2] = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&v2), k1056), s1);
                            res[sl][3] = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&v3), k1056), s1);
                        }
                    }
#pragma unroll
                    for (int sl = 0; sl < 4; sl++) {
                        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(a_sub + dst_off[sl][0]),
                                     "r"(*reinterpret_cast<const uint32_t *>(&res[sl][0])), "r"(*reinterpret_cast<const uint32_t *>(&res[sl][1]))
                                     : "memory");
                        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(a_sub + dst_off[sl][1]),
                                     "r"(*reinterpret_cast<const uint32_t *>(&res[sl][2])), "r"(*reinterpret_cast<const uint32_t *>(&res[sl][3]))
                                     : "memory");
                    }
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(full_bar + 8 * stage);
                if (trd) t_conv += global_ns() - tw0;
            }
            tile0 = tile0_n;
            have = have_n;
            git_base += iters;
        }
        if (trd && lane == 0) {
            // timeline entry of kind 4: dequant warp 0 -- start, time spent waiting for free stages, stages, end
            const unsigned long long slot = atomicAdd(p.trace, 1ull);
            if (slot < 8192) {
                unsigned long long *e = p.trace + 8 + slot * 8;
                e[0] = 4; e[1] = t_begin; e[2] = t_empty; e[3] = t_conv; e[4] = (unsigned long long)git_base; e[5] = global_ns();
                e[6] = gridDim.x; e[7] = (unsigned long long)p.N;
            }
        }
    } else {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            bool alive = true;
            const uint32_t idesc = idesc_f16(128 * NSUB);
            int git = 0, tcount = 0;
            const bool tr = p.trace != nullptr && blockIdx.x == 0;
            unsigned long long t_start = tr ? global_ns() : 0, t_full = 0, t_acc = 0, t_issue = 0;
            for (int64_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, tcount++) {
                const int buf = tcount % C::NACC, use = tcount / C::NACC;
                // the epilogue must have drained this accumulator set (its previous use)
                unsigned long long t0 = tr ? global_ns() : 0;
                if (use >= 1 && alive) alive = mbar_wait_bounded(acce_bar + 8 * buf, (uint32_t)((use - 1) & 1), p.status);
                if (tr) t_acc += global_ns() - t0;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * C::ACC_COLS);
                const int mh = tile_mh(tile_m(tile / splits));
                for (int it = 0; it < iters; it++, git++) {
                    const int stage = git % STAGES;
                    if (tr) t0 = global_ns();
                    if (alive) alive = mbar_wait_bounded(full_bar + 8 * stage, (uint32_t)((git / STAGES) & 1), p.status);
                    if (tr) {
                        t_full += global_ns() - t0;
                        t0 = global_ns();
                    }
                    tc_fence_after();
                    const uint32_t a_stage = stages_u32 + stage * C::STAGE_BYTES;
                    // N side: the 128 * NSUB expanded weight rows of the stage (sub-tiles are contiguous 8-row atoms)
                    const uint64_t wdesc = smem_desc_sw128(a_stage);
#pragma unroll
                    for (int hb = 0; hb < C::MH; hb++) {
                        if (hb >= mh) break;
                        // M side: 128 activation rows (a 64-row tile leaves lanes 64..127 unused)
                        const uint64_t xdesc = smem_desc_sw128(a_stage + C::A_BYTES + hb * (128 * 128));
#pragma unroll
                        for (int kk = 0; kk < 4; kk++)  // 16 K values = 32 bytes along the swizzled row per instruction
                            umma_f16(tmem_d + (uint32_t)(hb * 128 * NSUB), xdesc + (uint64_t)(2 * kk), wdesc + (uint64_t)(2 * kk), idesc,
                                     (it > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(empty_bar + 8 * stage);
                    if (tr) t_issue += global_ns() - t0;
                }
                umma_commit(accf_bar + 8 * buf);
            }
            if (tr) {
                // timeline entry of kind 3: start, end, time the MMA lane waited for operands / for the epilogue, stages issued
                const unsigned long long slot = atomicAdd(p.trace, 1ull);
                if (slot < 8192) {
                    unsigned long long *e = p.trace + 8 + slot * 8;
                    e[0] = 3; e[1] = t_start; e[2] = t_full; e[3] = t_acc; e[4] = (unsigned long long)git; e[5] = global_ns();
                    e[6] = t_issue; e[7] = (unsigned long long)p.N;
                }
            }
        }
        __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == C::WARPS - 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::TMEM_COLS) : "memory");
    }
}

// ================================================================================================================
// Two-CTA form (cta_group::2): a pair of CTAs on neighbouring SMs shares one 256 x 256 output tile.  Each CTA expands
// only HALF of the tile's weight rows (128) per stage and holds half of its activation rows (128); one
// tcgen05.mma.cta_group::2 instruction (M = 256, N = 256, issued by the pair's first CTA) reads both halves of both
// operands, and each CTA's tensor memory receives the 128 activation rows it holds x all 256 columns.  Per SM the
// conversion work per multiplied element is half that of the one-CTA kernel, which is bound by exactly that work, and
// two accumulator sets fit (2 x 256 columns), so the epilogue overlaps the next tile.
//
// Hand-shakes: `full[stage]` lives in the first CTA and counts its own conversion warps, its activation copy and ONE
// arrival for the second CTA, whose conversion warps and activation copy meet on a local barrier that its otherwise
// idle MMA warp forwards (mapa + mbarrier.arrive.release.cluster); `empty[stage]` and `acc_full[set]` exist in both
// CTAs at the same offsets and are signalled by ONE tcgen05.commit with cluster multicast (an arrive, not a load);
// `acc_empty[set]` lives in the first CTA and counts the epilogue warps of both.  No TMA or bulk load uses multicast.
// Dense Q4_K only, no K split; every wait is bounded.
// ================================================================================================================
constexpr int GP_STAGE_W = 128 * 128;   // 128 expanded weight rows x 64 fp16
constexpr int GP_STAGE_X = 2 * 128 * 128;   // two blocks of 128 activation rows x 64 fp16
constexpr int GP_STAGE = GP_STAGE_W + GP_STAGE_X;
constexpr int GP_STAGES = 4;
constexpr int GP_HDR = 16 * 1280;
constexpr int GP_BARS = 256;  // full, empty, act [GP_STAGES]; acc_full, acc_empty [2]; tensor-memory address word
constexpr int GP_TOTAL = 1024 + GP_STAGES * GP_STAGE + GP_HDR + GP_BARS;
constexpr int GP_EPI_WARPS = 4;  // one per tensor-memory lane quarter (21 warps leave 80 registers a thread)
constexpr int GP_WARPS = GP_EPI_WARPS + 16 + 1, GP_THREADS = GP_WARPS * 32;
static_assert(GP_TOTAL <= 227 * 1024, "shared memory over the limit");

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on the barrier at the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(bar), "r"(rank));
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
// bounded wait with cluster-scope acquire: the arrivals it observes come from both CTAs of the pair
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint32_t bar, uint32_t parity, int *status) {
    for (int i = 0; i < GEMM_WAIT_LIMIT; i++) {
        uint32_t ok;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    report_failure(status, 2);
    return false;
}
// instruction descriptor, kind::f16, pair form: D = f32, A = B = f16, both K-major, M = 256 over the pair, N = n
__host__ __device__ constexpr uint32_t idesc_f16_pair(int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((256u >> 4) << 24); }
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// completion of all MMAs issued so far arrives on the barrier at this offset in both CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"((uint16_t)3)
                 : "memory");
}

__global__ void __launch_bounds__(GP_THREADS, 1) gemm_q4k_pair_kernel(GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    constexpr int STAGES = GP_STAGES;
    constexpr int TB = tile_bytes(TTQ_FMT_Q4_K);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();  // 0: issues the MMAs and owns the counting barriers
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t stages_u32 = base, hdr_u32 = base + STAGES * GP_STAGE, bars_u32 = hdr_u32 + GP_HDR;
    const uint32_t full_bar = bars_u32, empty_bar = full_bar + 8 * STAGES, act_bar = empty_bar + 8 * STAGES;
    const uint32_t accf_bar = act_bar + 8 * STAGES, acce_bar = accf_bar + 16;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + STAGES * GP_STAGE + GP_HDR + 24 * STAGES + 32);
    grid_launch_dependents();
    // Output tiles: 256 weight rows x 512 activation rows; a last block of 256 activation rows makes half tiles.  All full
    // tiles come first (weight-tile column major, so that pairs running side by side share weights), the half tiles
    // after them: dealt round-robin, every pair then gets its share of both kinds.
    const int64_t m_full = p.Mp / 512, m_half = (p.Mp % 512) ? 1 : 0, n_tiles = (p.N + 255) / 256;
    const int64_t n_full = n_tiles * m_full, n_otiles = n_full + n_tiles * m_half;
    auto tile_at = [&](int64_t tile, int64_t &n_tile, int64_t &m_tile) -> int {  // returns the tile's 256-row blocks
        if (tile < n_full) {
            n_tile = tile / m_full;
            m_tile = tile % m_full;
            return 2;
        }
        n_tile = tile - n_full;
        m_tile = m_full;
        return 1;
    };
    const int64_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int iters = (int)p.SBp * 4;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            // first CTA: its 8 conversion warps of the stage, its activation copy, one forwarded arrival for the second CTA;
            // second CTA: its 8 conversion warps and its activation copy meet on `act`, which its MMA warp forwards
            mbar_init(full_bar + 8 * s, 8 + 1 + 1);
            mbar_init(empty_bar + 8 * s, 1);
            mbar_init(act_bar + 8 * s, 8 + 1);
        }
        mbar_init(accf_bar, 1);
        mbar_init(acce_bar, 2 * GP_EPI_WARPS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == GP_WARPS - 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers and tensor memory exist before anything arrives remotely
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < GP_EPI_WARPS) {
        // ------------------------------------------------------------------ epilogue: this CTA's 128 activation rows
        grid_dependency_wait();
        bool alive = true;
        int tcount = 0;
        const int esz = p.y_dt == TTQ_DT_F32 ? 4 : 2;
        for (int64_t tile = pair; tile < n_otiles; tile += n_pairs, tcount++) {
            int64_t n_tile, m_tile;
            const int mh = tile_at(tile, n_tile, m_tile);
            if (alive) alive = mbar_wait_warp(accf_bar, (uint32_t)(tcount & 1), p.status, lane);
            tc_fence_after();
            const int quad = warp & 3;  // a warp reads the 32 tensor-memory lanes of its quarter
            const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16);
            auto emit = [&](const uint32_t (&v)[16], int c) {
                // columns [256 hb, 256 hb + 256) hold activation rows 256 hb + 128 rank + lane of the tile
                const int hb = c >> 8, c0 = c & 255;
                const int64_t m = m_tile * 512 + hb * 256 + (int64_t)rank * 128 + quad * 32 + lane;
                const int64_t n0 = n_tile * 256 + c0;
                if (m >= p.M || n0 >= p.N) return;
                float f[16];
#pragma unroll
                for (int i = 0; i < 16; i++) f[i] = __uint_as_float(v[i]);
                if (p.bias != nullptr) {
#pragma unroll
                    for (int i = 0; i < 16; i++)
                        if (n0 + i < p.N) f[i] += load_as_float(p.bias, p.bias_dt, n0 + i);
                }
                uint8_t *dst = reinterpret_cast<uint8_t *>(p.y) + (size_t)(m * p.ldy + n0) * esz;
                if (n0 + 16 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                    if (p.y_dt == TTQ_DT_F32) {
#pragma unroll
                        for (int q = 0; q < 4; q++)
                            reinterpret_cast<float4 *>(dst)[q] = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
                    } else {
                        uint32_t w[8];
#pragma unroll
                        for (int q = 0; q < 8; q++) {
                            if (p.y_dt == TTQ_DT_BF16) {
                                const __nv_bfloat162 t2 = __floats2bfloat162_rn(f[2 * q], f[2 * q + 1]);
                                w[q] = *reinterpret_cast<const uint32_t *>(&t2);
                            } else {
                                const __half2 t2 = __floats2half2_rn(f[2 * q], f[2 * q + 1]);
                                w[q] = *reinterpret_cast<const uint32_t *>(&t2);
                            }
                        }
                        reinterpret_cast<uint4 *>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                        reinterpret_cast<uint4 *>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; i++)
                        if (n0 + i < p.N) store_from_float(p.y, p.y_dt, m * p.ldy + n0 + i, f[i]);
                }
            };
            // two register sets: the next 16 columns are on their way from tensor memory while these are stored
            uint32_t va[16], vb[16];
            const int c_begin = 0, c_end = mh * 256;
            tmem_ld16_issue(t_row + (uint32_t)c_begin, va);
#pragma unroll 1
            for (int c = c_begin; c < c_end; c += 32) {
                tmem_ld_wait(va);
                tmem_ld16_issue(t_row + (uint32_t)(c + 16), vb);
                emit(va, c);
                tmem_ld_wait(vb);
                if (c + 32 < c_end) tmem_ld16_issue(t_row + (uint32_t)(c + 32), va);
                emit(vb, c + 16);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acce_bar, 0);
        }
    } else if (warp < GP_EPI_WARPS + 16) {
        // ------------------------------------------------------------------ conversion: this CTA's 128 weight rows
        // two groups of 8 warps take the even and the odd stages; warp dw of a group expands packed row tile dw
        const int dwa = warp - GP_EPI_WARPS, dw = dwa & 7, grp = dwa >> 3;
        const int g = lane >> 2, t = lane & 3, r = lane & 15, h = lane >> 4;
        const uint32_t my_hdr = hdr_u32 + dwa * 1280;
        const int u0 = t >> 1, u1 = 2 + (t >> 1);
        // Lanes with t >= 2 take their four packed words in the order 2, 3, 0, 1: a store instruction of 8 bytes per lane
        // is served half a warp at a time, and the 16 lanes of a half (rows g = 0..3) then write eight different
        // 16-byte columns of the swizzled rows instead of four, twice each.
        const bool swp = (t & 2) != 0;
        uint32_t dst_off[4][2], hdr_off[4];
#pragma unroll
        for (int slp = 0; slp < 4; slp++) {
            const int sl = swp ? (slp ^ 2) : slp;
            const int u = (sl >> 1) ? u1 : u0;
            const int row = dw * 16 + g + 8 * (sl & 1);
            const uint32_t key = (uint32_t)(row & 7);
            dst_off[slp][0] = (uint32_t)row * 128 + (((uint32_t)(2 * u) ^ key) << 4) + (uint32_t)(t & 1) * 8;
            dst_off[slp][1] = (uint32_t)row * 128 + (((uint32_t)(2 * u + 1) ^ key) << 4) + (uint32_t)(t & 1) * 8;
            hdr_off[slp] = (uint32_t)((g + 8 * (sl & 1)) * 80) + (uint32_t)(2 * u * 8);
        }
        auto tile_ptr = [&](int64_t tile, bool &have) {
            int64_t n_tile = 0, m_tile = 0;
            if (tile < n_otiles) tile_at(tile, n_tile, m_tile);
            const int64_t nt = (n_tile * 2 + rank) * 8 + dw;
            have = tile < n_otiles && nt < p.NT;
            return p.tiles + (have ? nt : 0) * p.SBp * TB;
        };
        auto chunk_at = [&](const uint8_t *t0, bool ok, int it) {
            uint4 c = make_uint4(0, 0, 0, 0);
            if (ok) c = *reinterpret_cast<const uint4 *>(t0 + (int64_t)(it >> 2) * TB + lane * 16 + (it & 3) * 512);
            return c;
        };
        auto header_at = [&](const uint8_t *t0, bool ok, int sb) {
            uint4 hd = make_uint4(0, 0, 0, 0);
            if (ok) hd = *reinterpret_cast<const uint4 *>(t0 + (int64_t)sb * TB + 2048 + r * 16);
            return hd;
        };
        bool have;
        const uint8_t *tile0 = tile_ptr(pair, have);
        uint4 next = chunk_at(tile0, have, grp), next2 = chunk_at(tile0, have && grp + 2 < iters, grp + 2);
        uint4 hv_next = header_at(tile0, have, 0);
        grid_dependency_wait();
        const __half2 k1032 = __float2half2_rn(1032.f), k1152 = __float2half2_rn(1152.f);
        uint32_t mask_lo = 0x000f000fu, mask_hi = 0x00f000f0u, k1024 = 0x64006400u;
        asm volatile("" : "+r"(mask_lo), "+r"(mask_hi), "+r"(k1024));
        bool alive = true;
        int git_base = 0;
        const int64_t b_it_stride = (p.Mp >> 3) << 10;
        const bool trd = p.trace != nullptr && pair == 0 && dwa == 0;
        unsigned long long t_empty = 0, t_conv = 0, t_begin = trd ? global_ns() : 0;
        for (int64_t tile = pair; tile < n_otiles; tile += n_pairs) {
            bool have_n;
            const uint8_t *tile0_n = tile_ptr(tile + n_pairs, have_n);
            // this CTA's activation rows of a stage: 128 of each 256-row block of the tile, a contiguous 16 KB run each
            int64_t n_tile_c, m_tile_c;
            const int mh = tile_at(tile, n_tile_c, m_tile_c);
            const int64_t m_row0 = m_tile_c * 512;
            const uint8_t *bsrc0 = reinterpret_cast<const uint8_t *>(p.xh) + (((m_row0 + (int64_t)rank * 128) >> 3) << 10);
            for (int it = grp; it < iters; it += 2) {
                const int git = git_base + it, sb = it >> 2, stage = git % STAGES;
                const uint4 w = next;
                next = next2;
                if (it + 4 < iters) next2 = chunk_at(tile0, have, it + 4);
                else next2 = chunk_at(tile0_n, have_n && (it + 4 - iters) < iters, it + 4 - iters);
                if ((it & 3) == grp) {
                    // first own stage of a super-block: lane (r, h) unpacks half h of row r's scales into the header area
                    __syncwarp();
                    const uint4 hv = hv_next;
                    if (sb + 1 < (int)p.SBp) hv_next = header_at(tile0, have, sb + 1);
                    else hv_next = header_at(tile0_n, have_n, 0);
                    const __half2 dd = *reinterpret_cast<const __half2 *>(&hv.x);
                    const float d = __low2float(dd), dmin = __high2float(dd);
                    uint32_t scw, mw;
                    if (h == 0) {
                        scw = hv.y & 0x3f3f3f3fu;
                        mw = hv.z & 0x3f3f3f3fu;
                    } else {
                        scw = (hv.w & 0x0f0f0f0fu) | ((hv.y >> 2) & 0x30303030u);
                        mw = ((hv.w >> 4) & 0x0f0f0f0fu) | ((hv.z >> 2) & 0x30303030u);
                    }
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float sc = d * (float)((scw >> (8 * i)) & 0xff);
                        const float off = fmaf(8.f, sc, -dmin * (float)((mw >> (8 * i)) & 0xff));
                        const __half2 s2 = __float2half2_rn((i & 1) ? sc * 0.0625f : sc);
                        const __half2 o2 = __float2half2_rn(off);
                        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(my_hdr + (uint32_t)(r * 80 + (4 * h + i) * 8)),
                                     "r"(*reinterpret_cast<const uint32_t *>(&s2)), "r"(*reinterpret_cast<const uint32_t *>(&o2))
                                     : "memory");
                    }
                    __syncwarp();
                }
                unsigned long long tw0 = trd ? global_ns() : 0;
                if (git >= STAGES && alive) alive = mbar_wait_warp(empty_bar + 8 * stage, (uint32_t)(((git / STAGES) - 1) & 1), p.status, lane);
                if (trd) {
                    t_empty += global_ns() - tw0;
                    tw0 = global_ns();
                }
                const uint32_t w_stage = stages_u32 + stage * GP_STAGE;
                if (dw == 0 && lane == 0) {
                    // the first CTA's copy is counted on `full` itself, the second CTA's on its local barrier (forwarded below)
                    const uint32_t bar = (rank == 0 ? full_bar : act_bar) + 8 * stage;
                    mbar_expect_tx(bar, (uint32_t)mh * 16384u);
                    for (int hb = 0; hb < mh; hb++)
                        bulk_g2s(w_stage + GP_STAGE_W + hb * 16384, bsrc0 + it * b_it_stride + (int64_t)hb * (32 << 10), 16384u, bar);
                }
                {
                    const uint32_t wa[4] = {swp ? w.z : w.x, swp ? w.w : w.y, swp ? w.x : w.z, swp ? w.y : w.w};
                    uint4 so[4];
                    __half2 res[4][4];
#pragma unroll
                    for (int sl = 0; sl < 4; sl++)
                        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(so[sl].x), "=r"(so[sl].y), "=r"(so[sl].z), "=r"(so[sl].w)
                                     : "r"(my_hdr + hdr_off[sl]));
#pragma unroll
                    for (int sl = 0; sl < 4; sl++) {
                        const __half2 sc_lo = *reinterpret_cast<const __half2 *>(&so[sl].x), of_lo = *reinterpret_cast<const __half2 *>(&so[sl].y);
                        const __half2 sc_hi = *reinterpret_cast<const __half2 *>(&so[sl].z), of_hi = *reinterpret_cast<const __half2 *>(&so[sl].w);
                        const uint32_t x = wa[sl], x8 = x >> 8;
                        uint32_t v0 = and_or(x, mask_lo, k1024), v1 = and_or(x8, mask_lo, k1024);
                        uint32_t v2 = and_or(x, mask_hi, k1024), v3 = and_or(x8, mask_hi, k1024);
                        res[sl][0] = __hfma2(__hsub2(*reinterpret_cast<__half2 *>(&v0), k1032), sc_lo, of_lo);
                        res[sl][1] = __hfma2(__hsub2(*reinterpret_cast<__half2 *>(&v1), k1032), sc_lo, of_lo);
                        res[sl][2] = __hfma2(__hsub2(*reinterpret_cast<__half2 *>(&v2), k1152), sc_hi, of_hi);
                        res[sl][3] = __hfma2(__hsub2(*reinterpret_cast<__half2 *>(&v3), k1152), sc_hi, of_hi);
                    }
#pragma unroll
                    for (int sl = 0; sl < 4; sl++) {
                        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(w_stage + dst_off[sl][0]),
                                     "r"(*reinterpret_cast<const uint32_t *>(&res[sl][0])), "r"(*reinterpret_cast<const uint32_t *>(&res[sl][1]))
                                     : "memory");
                        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(w_stage + dst_off[sl][1]),
                                     "r"(*reinterpret_cast<const uint32_t *>(&res[sl][2])), "r"(*reinterpret_cast<const uint32_t *>(&res[sl][3]))
                                     : "memory");
                    }
                }
                fence_async_smem();  // (both CTAs' tensor cores read these rows; the release at cluster scope below orders them)
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive((rank == 0 ? full_bar : act_bar) + 8 * stage);
                }
                if (trd) t_conv += global_ns() - tw0;
            }
            tile0 = tile0_n;
            have = have_n;
            git_base += iters;
        }
        if (trd && lane == 0) {
            // timeline entry of kind 4: conversion warp 0 of either CTA of the first pair
            const unsigned long long slot = atomicAdd(p.trace, 1ull);
            if (slot < 8192) {
                unsigned long long *e = p.trace + 8 + slot * 8;
                e[0] = 4; e[1] = t_begin; e[2] = t_empty; e[3] = t_conv; e[4] = (unsigned long long)git_base; e[5] = global_ns();
                e[6] = gridDim.x; e[7] = (unsigned long long)p.N;
            }
        }
    } else if (rank == 0) {
        // ------------------------------------------------------------------ MMA issue (first CTA of the pair)
        if (lane == 0) {
            bool alive = true;
            constexpr uint32_t idesc = idesc_f16_pair(256);
            int git = 0, tcount = 0;
            const bool tr = p.trace != nullptr && pair == 0;
            unsigned long long t_start = tr ? global_ns() : 0, t_full = 0, t_acc = 0, t_issue = 0;
            for (int64_t tile = pair; tile < n_otiles; tile += n_pairs, tcount++) {
                // both CTAs' epilogue warps have drained the accumulators of the previous tile
                unsigned long long t0 = tr ? global_ns() : 0;
                if (tcount >= 1 && alive) alive = mbar_wait_bounded_cluster(acce_bar, (uint32_t)((tcount - 1) & 1), p.status);
                if (tr) t_acc += global_ns() - t0;
                tc_fence_after();
                int64_t n_tile_c, m_tile_c;
                const int mh = tile_at(tile, n_tile_c, m_tile_c);
                for (int it = 0; it < iters; it++, git++) {
                    const int stage = git % STAGES;
                    if (tr) t0 = global_ns();
                    if (alive) alive = mbar_wait_bounded(full_bar + 8 * stage, (uint32_t)((git / STAGES) & 1), p.status);
                    if (tr) {
                        t_full += global_ns() - t0;
                        t0 = global_ns();
                    }
                    tc_fence_after();
                    const uint32_t w_stage = stages_u32 + stage * GP_STAGE;
                    const uint64_t wdesc = smem_desc_sw128(w_stage);
                    for (int hb = 0; hb < mh; hb++) {
                        const uint64_t xdesc = smem_desc_sw128(w_stage + GP_STAGE_W + hb * 16384);
#pragma unroll
                        for (int kk = 0; kk < 4; kk++)
                            umma_f16_pair(tmem_base + (uint32_t)(hb * 256), xdesc + (uint64_t)(2 * kk), wdesc + (uint64_t)(2 * kk), idesc, (it > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(empty_bar + 8 * stage);
                    if (tr) t_issue += global_ns() - t0;
                }
                umma_commit_pair(accf_bar);
            }
            if (tr) {
                // timeline entry of kind 3, as in the one-CTA kernel
                const unsigned long long slot = atomicAdd(p.trace, 1ull);
                if (slot < 8192) {
                    unsigned long long *e = p.trace + 8 + slot * 8;
                    e[0] = 3; e[1] = t_start; e[2] = t_full; e[3] = t_acc; e[4] = (unsigned long long)git; e[5] = global_ns();
                    e[6] = t_issue; e[7] = (unsigned long long)p.N;
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ second CTA: forward the activation copies
        if (lane == 0) {
            bool alive = true;
            int git = 0;
            for (int64_t tile = pair; tile < n_otiles; tile += n_pairs) {
                for (int it = 0; it < iters; it++, git++) {
                    const int stage = git % STAGES;
                    if (alive) alive = mbar_wait_bounded(act_bar + 8 * stage, (uint32_t)((git / STAGES) & 1), p.status);
                    mbar_arrive_cluster(full_bar + 8 * stage, 0);
                }
            }
        }
        __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // nothing of the pair is in flight any more: barriers, shared and tensor memory may go
    if (warp == GP_WARPS - 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// Sum of the split-K partials (+ bias) into y.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ ws, int splits, int64_t M, int64_t Mp, int64_t N,
                                                            const void *bias, int bias_dt, void *y, int y_dt, int64_t ldy) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int64_t total = M * N;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = e / N, n = e % N;
        float acc = 0.f;
        for (int s = 0; s < splits; s++) acc += ws[((size_t)s * Mp + m) * N + n];
        if (bias != nullptr) acc += load_as_float(bias, bias_dt, n);
        store_from_float(y, y_dt, m * ldy + n, acc);
    }
}

template <int BM, int NSUB, int MODE = GM_Q4K>
cudaError_t launch_cfg(const GemmParams &p, int sms, cudaStream_t st) {
    using C = GemmCfg<BM, NSUB>;
    static bool configured[64] = {};  // per device: the shared-memory opt-in belongs to the device's copy of the function
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!configured[dev]) {
        e = cudaFuncSetAttribute(gemm_q4k_kernel<BM, NSUB, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::TOTAL);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    const int64_t tiles = ((p.N + GEMM_BN * NSUB - 1) / (GEMM_BN * NSUB)) * (p.group_tiles != nullptr ? p.mt_cap : p.Mp / BM) * p.splits;
    const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
    return launch_pdl(gemm_q4k_kernel<BM, NSUB, MODE>, dim3(grid), dim3(C::THREADS), (size_t)C::TOTAL, st, p);
}

// Pairs of CTAs the current device runs at once: the shared-memory opt-in is set on first use, and the driver is asked
// how many clusters of two fit (SM counts per GPC may leave an SM without a partner).  0: the kernel cannot run here.
int pair_slots(int sms) {
    static int slots[64] = {};
    static bool known[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (!known[dev]) {
        known[dev] = true;
        slots[dev] = 0;
        if (cudaFuncSetAttribute(gemm_q4k_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GP_TOTAL) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)(sms / 2 * 2));
            cfg.blockDim = dim3(GP_THREADS);
            cfg.dynamicSmemBytes = GP_TOTAL;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_q4k_pair_kernel, &cfg) == cudaSuccess) slots[dev] = n < sms / 2 ? n : sms / 2;
        }
        cudaGetLastError();
    }
    return slots[dev];
}

// pairs of CTAs (cluster of 2) over the output tiles; programmatic stream serialization like every other launch
cudaError_t launch_pair(const GemmParams &p, int sms, cudaStream_t st) {
    const int slots = pair_slots(sms);
    if (slots < 1) return cudaErrorNotSupported;
    const int64_t tiles = ((p.N + 255) / 256) * ((p.Mp + 511) / 512);
    const int64_t pairs = tiles < slots ? tiles : slots;
    static const bool pdl = env_flag("TTQ_PDL", true);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(GP_THREADS);
    cfg.dynamicSmemBytes = GP_TOTAL;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, gemm_q4k_pair_kernel, p);
}

}  // namespace

bool gemm_supported(int fmt) { return fmt == TTQ_FMT_Q4_K || fmt == TTQ_FMT_Q8_0 || fmt == TTQ_FMT_Q6_K; }

// Rows of the fp16 weight images the plain mode reads: output features padded to whole 256-row tiles.
int64_t gemm_wimg_rows(int64_t N) { return (N + 255) / 256 * 256; }

// x rows are processed in slabs that fit the fp16 activation scratch (capacity in halves).
cudaError_t launch_gemm(int fmt, const LinearArgs &a, __half *xh, int64_t xh_capacity, int sms, int *status,
                        unsigned long long *trace, cudaStream_t st, int *launches, const __half *wimg) {
    *launches = 0;
    const bool plain = wimg != nullptr;
    if (!plain && !gemm_supported(fmt)) return cudaErrorNotSupported;
    const int kmap = (!plain && fmt == TTQ_FMT_Q6_K) ? 1 : 0;
    const int64_t Kp = a.SBp * TILE_K;
    const int BM = a.M <= 64 ? 64 : (a.M <= 128 ? 128 : 256);
    // two 128-row sub-tiles per CTA once there are enough tiles to keep every SM busy with them
    static const int force_nsub = []() {
        const char *v = getenv("TTQ_GEMM_NSUB");
        return v ? atoi(v) : 0;
    }();
    // a CTA with two sub-tiles does twice the work per activation stage in about 1.65x the time of one (measured: five
    // rounds of one sub-tile against three of two on 4096 -> 28672 at 768 rows take 221 against 203 us; the single
    // sub-tile is expanded by two warp groups on alternating stages)
    const int64_t mt = (a.M + BM - 1) / BM;
    const int64_t tiles1 = ((a.N + 127) / 128) * mt, tiles2 = ((a.N + 255) / 256) * mt;
    const double cost1 = (double)((tiles1 + sms - 1) / sms), cost2 = 1.65 * (double)((tiles2 + sms - 1) / sms);
    int nsub = (a.N > 128 && cost2 < cost1) ? 2 : 1;
    if (force_nsub == 1 || force_nsub == 2) nsub = force_nsub;
    if (plain || fmt != TTQ_FMT_Q4_K) nsub = 2;  // plain: no conversion work to balance; Q8_0 / Q6_K: one variant
    int64_t slab = (xh_capacity / Kp) / BM * BM;  // rows per pass
    if (slab < BM) return cudaErrorInvalidValue;
    const int esz_x = a.x_dt == TTQ_DT_F32 ? 4 : 2, esz_y = a.y_dt == TTQ_DT_F32 ? 4 : 2;
    for (int64_t m0 = 0; m0 < a.M; m0 += slab) {
        const int64_t Ms = (a.M - m0) < slab ? (a.M - m0) : slab;
        const int64_t m_tiles = (Ms + BM - 1) / BM, Mp = m_tiles * BM;
        const uint8_t *xs = reinterpret_cast<const uint8_t *>(a.x) + (size_t)m0 * a.ldx * esz_x;
        const int64_t chunks = Mp * (Kp / 8);
        const unsigned grid = (unsigned)((chunks + 255) / 256 < sms * 16 ? (chunks + 255) / 256 : sms * 16);
        const int *no_tab = nullptr;
        cudaError_t e = a.gated ? launch_pdl(xh_prep_kernel<true>, dim3(grid), dim3(256), 0, st, (const void *)xs, a.x_dt, Ms, Mp, a.K, Kp, a.ldx,
                                             xh, no_tab, no_tab, 0, kmap)
                                : launch_pdl(xh_prep_kernel<false>, dim3(grid), dim3(256), 0, st, (const void *)xs, a.x_dt, Ms, Mp, a.K, Kp, a.ldx,
                                             xh, no_tab, no_tab, 0, kmap);
        if (e != cudaSuccess) return e;
        ++*launches;
        GemmParams p;
        p.tiles = a.tiles;
        p.wimg = wimg; p.Np = gemm_wimg_rows(a.N);
        p.group_tiles = nullptr; p.mt_group = nullptr; p.mt_row0 = nullptr; p.mt_mh = nullptr; p.n_mt = nullptr; p.mt_cap = 0;
        p.N = a.N; p.NT = a.NT; p.SBp = a.SBp;
        p.xh = xh;
        p.M = Ms; p.Mp = Mp; p.Kp = Kp;
        p.bias = a.bias; p.bias_dt = a.bias_dt;
        p.y = reinterpret_cast<uint8_t *>(a.y) + (size_t)m0 * a.ldy * esz_y;
        p.y_dt = a.y_dt; p.ldy = a.ldy;
        p.status = status;
        p.trace = trace;
        // K split: when the output tiles alone cannot fill the SMs, cut K into equal runs of super-blocks;
        // partials go to the tail of the activation scratch
        int splits = 1;
        {
            const int64_t tiles = ((a.N + 128 * nsub - 1) / (128 * nsub)) * m_tiles;
            const size_t xh_bytes = (size_t)Mp * Kp * sizeof(__half);
            const size_t ws_cap = (size_t)xh_capacity * sizeof(__half) > xh_bytes ? (size_t)xh_capacity * sizeof(__half) - xh_bytes : 0;
            for (int cand = 2; cand <= 8; cand++) {
                if (a.SBp % cand || a.SBp / cand < 2) continue;
                if (tiles * cand > sms) break;
                if ((size_t)cand * Mp * a.N * sizeof(float) > ws_cap) break;
                splits = cand;
            }
            p.splits = splits;
            p.ws = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(xh) + ((xh_bytes + 255) & ~(size_t)255));
        }
        auto run = [&](const GemmParams &q, bool pair) -> cudaError_t {
            if (pair) return launch_pair(q, sms, st);
            if (plain) {
                if (BM == 64) return launch_cfg<64, 2, GM_PLAIN>(q, sms, st);
                if (BM == 128) return launch_cfg<128, 2, GM_PLAIN>(q, sms, st);
                return launch_cfg<256, 2, GM_PLAIN>(q, sms, st);
            }
            if (fmt == TTQ_FMT_Q8_0) {
                // (these formats always take two sub-tiles: the single sub-tile variant pays off on the many small tiles
                // of the grouped Q4_K GEMM, which they do not serve)
                if (BM == 64) return launch_cfg<64, 2, GM_Q8_0>(q, sms, st);
                if (BM == 128) return launch_cfg<128, 2, GM_Q8_0>(q, sms, st);
                return launch_cfg<256, 2, GM_Q8_0>(q, sms, st);
            }
            if (fmt == TTQ_FMT_Q6_K) {
                if (BM == 64) return launch_cfg<64, 2, GM_Q6K>(q, sms, st);
                if (BM == 128) return launch_cfg<128, 2, GM_Q6K>(q, sms, st);
                return launch_cfg<256, 2, GM_Q6K>(q, sms, st);
            }
            if (nsub == 2) {
                if (BM == 64) return launch_cfg<64, 2>(q, sms, st);
                if (BM == 128) return launch_cfg<128, 2>(q, sms, st);
                return launch_cfg<256, 2>(q, sms, st);
            }
            if (BM == 64) return launch_cfg<64, 1>(q, sms, st);
            if (BM == 128) return launch_cfg<128, 1>(q, sms, st);
            return launch_cfg<256, 1>(q, sms, st);
        };
        auto reduce = [&](const GemmParams &q) -> cudaError_t {
            const int64_t total = Ms * q.N;
            const unsigned rg = (unsigned)((total + 255) / 256 < sms * 8 ? (total + 255) / 256 : sms * 8);
            return launch_pdl(splitk_reduce_kernel, dim3(rg), dim3(256), 0, st, (const float *)q.ws, q.splits, Ms, Mp, q.N, q.bias, q.bias_dt,
                              (void *)q.y, q.y_dt, q.ldy);
        };
        // Ragged last round: with more output tiles than SMs, the tiles left over after the last full round keep a
        // few SMs busy for a whole tile time.  The last weight-tile columns -- just enough of them that the rest fits
        // one round less -- then go to a second launch of the one-CTA kernel with K cut into runs, spread over all SMs.
        // Cost model in pipeline stages of the one-CTA kernel: a unit of iters/S stages also pays a fixed turnaround
        // (accumulator drain + fp32 partial store, about 20 stages), the second launch a ramp of about 6, and the
        // reduction pass reads every partial back.  Measured at 2048 rows: 4096 -> 28672 (896 tiles, 8 left over) gains
        // a third of a tile time with 8 runs; 4096 -> 6144 (192 tiles, 44 left over) loses with any split and is left alone.
        static const bool tail_on = env_flag("TTQ_GEMM_TAIL", true);
        const int TN = 128 * nsub;
        const int64_t n_tiles = (a.N + TN - 1) / TN, tiles = n_tiles * m_tiles;
        const double iters = (double)a.SBp * 4;
        const size_t xh_bytes = (size_t)Mp * Kp * sizeof(__half);
        const size_t ws_cap = (size_t)xh_capacity * sizeof(__half) > xh_bytes ? (size_t)xh_capacity * sizeof(__half) - xh_bytes : 0;
        auto tail_cost = [&](int64_t cols, int min_runs, int &runs) -> double {
            double best = 1e30;
            runs = 0;
            for (int cand = min_runs; cand <= 16; cand++) {
                if (a.SBp % cand || (cand > 1 && a.SBp / cand < 2)) continue;
                if (cand > 1 && (size_t)cand * Mp * cols * TN * sizeof(float) > ws_cap) break;
                const int64_t units = cols * m_tiles * cand;
                const double cost = cand > 1 ? (double)((units + sms - 1) / sms) * (iters / cand + 20.0) + 6.0 + 0.08 * (double)units
                                             : (double)((units + sms - 1) / sms) * (iters + 8.0) + 6.0;
                if (cost < best) {
                    best = cost;
                    runs = cand;
                }
            }
            return best;
        };
        int64_t tail_cols = 0;
        int tail_splits = 1;
        double cost_one = (double)((tiles + sms - 1) / sms) * (iters + 8.0);
        if (tail_on && !plain && splits == 1 && tiles > sms && tiles % sms != 0) {
            const int64_t rounds = (tiles + sms - 1) / sms;
            const int64_t cols = (tiles - (rounds - 1) * sms + m_tiles - 1) / m_tiles;  // columns that must leave the main launch
            int runs = 0;
            const double c = cols < n_tiles ? tail_cost(cols, 2, runs) : 1e30;
            if (runs > 0 && c < 0.85 * (iters + 8.0)) {
                tail_cols = cols;
                tail_splits = runs;
                cost_one = (double)(rounds - 1) * (iters + 8.0) + c;
            }
        }
        // The two-CTA kernel (dense Q4_K, more than 128 rows, no K split): a pair's tile is 256 weight rows x 512
        // activation rows, and a stage of it takes about 0.85 of the one-CTA kernel's stage for twice the work (measured
        // at 4096 -> 28672, 2048 rows); a half tile (256 rows) about 0.6.  With 74 slots the rounds are coarser, so the
        // model prices both kernels, each with its best tail, and takes the cheaper.  The pair's load is that of the
        // first pair: tiles are dealt round-robin, full tiles first.
        // TTQ_GEMM_PAIR: 0 never, 1 (default) where the model prefers it, 2 wherever it applies
        static const int pair_mode = []() {
            const char *v = getenv("TTQ_GEMM_PAIR");
            return v ? atoi(v) : 1;
        }();
        bool use_pair = false;
        if (pair_mode > 0 && !plain && fmt == TTQ_FMT_Q4_K && BM == 256 && nsub == 2 && splits == 1) {
            const int64_t slots = pair_slots(sms), m_full = Mp / 512, m_half = (Mp % 512) ? 1 : 0;
            const double c_full = 0.85 * iters + 8.0, c_half = 0.6 * iters + 6.0;
            auto makespan = [&](int64_t cols) {
                const int64_t nf = cols * m_full, nt = nf + cols * m_half;
                double t = 0;
                for (int64_t k = 0; slots > 0 && k < nt; k += slots) t += k < nf ? c_full : c_half;
                return t;
            };
            double best = makespan(n_tiles);
            int64_t best_cols = 0;
            int best_runs = 1;
            for (int64_t cols = 1; tail_on && cols <= 16 && cols < n_tiles; cols++) {
                int runs = 0;
                const double t = tail_cost(cols, 1, runs);
                if (runs == 0) continue;
                const double total = makespan(n_tiles - cols) + t;
                if (total < 0.97 * best) {
                    best = total;
                    best_cols = cols;
                    best_runs = runs;
                }
            }
            if (slots > 0 && (best < cost_one || pair_mode >= 2)) {
                use_pair = true;
                tail_cols = best_cols;
                tail_splits = best_runs;
            }
        }
        if (tail_cols > 0) {
            const int64_t n_main = (n_tiles - tail_cols) * TN;  // output features of the main launch
            GemmParams q = p;
            q.N = n_main; q.NT = n_main / TILE_ROWS;
            e = run(q, use_pair);
            if (e != cudaSuccess) return e;
            ++*launches;
            q = p;
            q.tiles = reinterpret_cast<const uint8_t *>(p.tiles) + (size_t)(n_main / TILE_ROWS) * a.SBp * tile_bytes(fmt);
            q.N = a.N - n_main; q.NT = a.NT - n_main / TILE_ROWS;
            if (a.bias != nullptr) q.bias = reinterpret_cast<const uint8_t *>(a.bias) + (size_t)n_main * (a.bias_dt == TTQ_DT_F32 ? 4 : 2);
            q.y = reinterpret_cast<uint8_t *>(p.y) + (size_t)n_main * esz_y;
            q.splits = tail_splits;
            e = run(q, false);
            if (e != cudaSuccess) return e;
            ++*launches;
            if (tail_splits > 1) {
                e = reduce(q);
                if (e != cudaSuccess) return e;
                ++*launches;
            }
            continue;
        }
        e = run(p, use_pair);
        if (e != cudaSuccess) return e;
        ++*launches;
        if (splits > 1) {
            e = reduce(p);
            if (e != cudaSuccess) return e;
            ++*launches;
        }
    }
    return cudaSuccess;
}

// Grouped GEMM: row tile mt of the (routed, padded) activation rows multiplies weight matrix
// mt_group[mt]; the tile count is read on the device, so the grid is sized for the capacity.
cudaError_t launch_gemm_grouped(const GroupedArgs &g, __half *xh, int sms, int *status, cudaStream_t st, int *launches) {
    *launches = 0;
    const int64_t Kp = g.SBp * TILE_K;
    if (g.BM != 64 && g.BM != 128 && g.BM != 256 && g.BM != 384) return cudaErrorInvalidValue;
    if (g.Mp % 128 && g.Mp % g.BM) return cudaErrorInvalidValue;
    const int64_t chunks = g.Mp * (Kp / 8);
    const unsigned grid = (unsigned)((chunks + 255) / 256 < sms * 16 ? (chunks + 255) / 256 : sms * 16);
    cudaError_t e = g.gated ? launch_pdl(xh_prep_kernel<true>, dim3(grid), dim3(256), 0, st, g.x, g.x_dt, g.x_rows, g.Mp, g.K, Kp, g.ldx, xh,
                                         g.row_src, g.rows_total, 1, 0)
                            : launch_pdl(xh_prep_kernel<false>, dim3(grid), dim3(256), 0, st, g.x, g.x_dt, g.x_rows, g.Mp, g.K, Kp, g.ldx, xh,
                                         g.row_src, g.rows_total, 1, 0);
    if (e != cudaSuccess) return e;
    ++*launches;
    GemmParams p;
    p.tiles = nullptr;
    p.wimg = nullptr; p.Np = 0;
    p.group_tiles = g.group_tiles; p.mt_group = g.mt_group; p.mt_row0 = g.mt_row0; p.mt_mh = g.mt_mh; p.n_mt = g.n_mt;
    p.mt_cap = g.mt_cap;
    p.N = g.N; p.NT = g.NT; p.SBp = g.SBp;
    p.xh = xh;
    p.M = g.Mp; p.Mp = g.Mp; p.Kp = Kp;
    p.bias = nullptr; p.bias_dt = TTQ_DT_F32;
    p.y = g.y; p.y_dt = g.y_dt; p.ldy = g.ldy;
    p.status = status;
    p.trace = nullptr;
    p.splits = 1;
    p.ws = nullptr;
    // two sub-tiles per CTA when the expected tile count still covers the SMs
    const int64_t mt_cap = g.mt_cap;
    int nsub = (g.N >= 256 && ((g.N + 255) / 256) * mt_cap >= 2 * (int64_t)sms) ? 2 : 1;
    static const int force_nsub = []() {
        const char *v = getenv("TTQ_MOE_NSUB");
        return v ? atoi(v) : 0;
    }();
    if (force_nsub == 1 || force_nsub == 2) nsub = force_nsub;
    if (g.BM == 384) {
        e = launch_cfg<384, 1>(p, sms, st);  // up to three 128-row blocks share one expansion of the weight rows
    } else if (nsub == 2) {
        if (g.BM == 64) e = launch_cfg<64, 2>(p, sms, st);
        else if (g.BM == 128) e = launch_cfg<128, 2>(p, sms, st);
        else e = launch_cfg<256, 2>(p, sms, st);
    } else {
        if (g.BM == 64) e = launch_cfg<64, 1>(p, sms, st);
        else if (g.BM == 128) e = launch_cfg<128, 1>(p, sms, st);
        else e = launch_cfg<256, 1>(p, sms, st);
    }
    if (e != cudaSuccess) return e;
    ++*launches;
    return cudaSuccess;
}

}  // namespace ttq
