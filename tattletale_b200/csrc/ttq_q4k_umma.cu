// Decode linear for Q4_K, 1 to 8 activation rows, on the integer path of the fifth-generation tensor cores
// (tcgen05.mma kind::i8, accumulators in tensor memory).
//
// Arithmetic: the same fixed point as the other decode kernels -- activations become two int8 planes per row
// (xq = 256*hi + lo, one fp32 scale per 256-wide K chunk, produced by the separate activation pass), weight quants
// stay integers.  One instruction multiplies 128 weight rows by the planes of all activation rows over ONE sub-block
// (32 weights): A = the sub-block's nibbles widened to uint8 [128 x 32], B = the planes [N x 32] (N = 8 columns for
// up to 4 rows, 16 for up to 8), D = exact int32 sums in their own N tensor-memory columns.  The eight sub-blocks
// of a super-block go to eight column groups, so the epilogue thread that owns a weight row reads, per activation
// row, eight {hi, lo} pairs, applies the 6-bit scales, the min term and the chunk scale in fp32 and keeps the
// running output in a register.
//
// Why this shape: the legacy mma.sync path costs about 45 cycles per instruction and SM sub-partition on this
// part, which puts a 16-row x 256-weight tile at about the time HBM needs to deliver it; here an instruction with
// 8 columns was measured at 60 to 75 cycles for 128 rows x 32 weights (one per tile), and the work left to the
// CUDA cores is widening nibbles to bytes and the per-row scale arithmetic.
//
// Order of K inside a sub-block: a dot product does not care, as long as both operands agree.  A lane of the
// packed layout holds, for one weight row and sub-block, weights 8 n + 4 h + i of chunk n (h = lane parity); it
// widens the four chunks into ONE 16-byte shared store, so position 16 h + 4 n + i of the sub-block's 32 operand
// bytes holds K index 8 n + 4 h + i.  The activation pass writes the planes in the same order.
//
// Work split: an item is (group of 128 weight rows, super-block).  The items of the matrix, group-major, are cut
// into gridDim.x contiguous runs, one per CTA, equal to within one item.  A CTA that covers every super-block of a
// group writes the outputs itself; otherwise it parks its partial sums in a workspace slot of its own and counts
// its arrival, and the last CTA of the group adds the slots in CTA order (deterministic) and writes the outputs.
//
// Roles (26 warps): 8 epilogue warps (two sets on alternating items; thread = weight row), 16 expansion warps (two
// sets of 8, one packed row tile each, alternating items; packed bytes go global -> registers -> shared), one warp
// that lays out the activation operand and the per-item side sums with asynchronous copies, one lane that issues
// the MMAs.  Every wait is bounded.
#include "ttq_devutil.cuh"

namespace ttq {

namespace {

constexpr int UM_EPI_WARPS = 8, UM_EXP_WARPS = 16;
constexpr int UM_B_WARP = UM_EPI_WARPS + UM_EXP_WARPS, UM_MMA_WARP = UM_B_WARP + 1;
constexpr int UM_WARPS = UM_MMA_WARP + 1, UM_THREADS = UM_WARPS * 32;
constexpr int UM_SLOTS = 5;   // slots of expanded weights (one item each)
constexpr int UM_BSLOTS = 8;  // slots of the activation operand
constexpr int UM_NACC = 4;    // accumulator sets in tensor memory
// An item's header and side sums are read by the epilogue, after its operand slots have gone back: the rings are as
// deep as the furthest the writers can run ahead of the epilogue (slots + accumulator sets + 1).
constexpr int UM_HDR = UM_SLOTS + UM_NACC + 1, UM_SIDE = 16;
static_assert(UM_SIDE >= UM_BSLOTS + UM_NACC + 1, "side ring too shallow");
constexpr int UM_A_BYTES = 32768;  // 128 rows x 256 uint8: two swizzled tiles of [128 rows][128 bytes]
constexpr int UM_GROUP_TILES = 8, UM_GROUP_ROWS = UM_GROUP_TILES * TILE_ROWS;
constexpr int UM_WAIT_LIMIT = 1 << 22;
constexpr int UM_SIDE_FLOATS = 8;  // per activation row: the 8 sub-block sums of xq

struct UmParams {
    LinearArgs a;
    XqView xq;
    float *ws;           // partial sums: slot (CTA + group) x [M][128]
    unsigned *counters;  // arrivals per group, zero between launches
    int *status;
    unsigned long long *trace;  // optional timeline buffer (nullptr = off)
    int64_t n_groups, total_items;
    int prefetch;        // pull the CTA's packed run into L2 before the dependency wait
};

__device__ __forceinline__ void um_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
// bounded wait on the tensor-core pipeline: failure bit 1 (value 2), the caller goes on so that every role ends
__device__ __forceinline__ bool um_wait(uint32_t bar, uint32_t parity, int *status) {
    for (int i = 0; i < UM_WAIT_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    report_failure(status, 2);
    return false;
}
__device__ __forceinline__ bool um_wait_warp(uint32_t bar, uint32_t parity, int *status, int lane) {
    bool ok = true;
    if (lane == 0) {
        ok = false;
        for (int i = 0; i < UM_WAIT_LIMIT; i++) {
            if (mbar_try_wait(bar, parity)) {
                ok = true;
                break;
            }
            __nanosleep(128);
        }
        if (!ok) report_failure(status, 2);
    }
    __syncwarp();
    return __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
}
__device__ __forceinline__ void um_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void um_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row atoms of 1024 bytes stacked contiguously
__device__ __forceinline__ uint64_t um_desc_sw128(uint32_t addr) {
    const uint32_t lo = ((addr & 0x3ffffu) >> 4) | (1u << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}
// kind::i8: D = s32, A = u8, B = s8, both K-major, M = 128, N = n
__host__ __device__ constexpr uint32_t um_idesc(int n) { return (2u << 4) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((128u >> 4) << 24); }
__device__ __forceinline__ void um_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%4, %4, %4, %4}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void um_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Tensor-memory load of NB columns (one per register) for this warp's 32 lanes.  Asynchronous: the registers hold
// the data only after um_tmem_wait, which names them as operands so that no use is scheduled ahead of it.
template <int NB>
__device__ __forceinline__ void um_tmem_ld(uint32_t taddr, uint32_t (&v)[NB]) {
    if constexpr (NB == 8) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                     : "r"(taddr));
    } else {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
              "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr));
    }
}
__device__ __forceinline__ void um_tmem_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
template <int NB>
__device__ __forceinline__ void um_pin(uint32_t (&v)[NB]) {
    if constexpr (NB == 8) {
        asm volatile("" : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7])::"memory");
    } else {
        asm volatile(""
                     : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]),
                       "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])::"memory");
    }
}
__device__ __forceinline__ void um_cp16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// Timeline entry of kind 6 (block 0 only): one per role -- [1] role (0 epilogue, 1 expansion, 2 operand warp, 3 MMA lane:
// waits for weights / activations / accumulators, 4 MMA lane: issue / commits), [2] start ns, [3] end ns, [4..6] SM clocks
// spent in the role's waits, [7] items
__device__ __forceinline__ void um_trace(unsigned long long *trace, int role, unsigned long long t0, unsigned long long w0,
                                         unsigned long long w1, unsigned long long w2, int items) {
    const unsigned long long slot = atomicAdd(trace, 1ull);
    if (slot >= TRACE_CAP) return;
    unsigned long long *e = trace + 8 + slot * 8;
    e[0] = 6; e[1] = (unsigned long long)role; e[2] = t0; e[3] = global_ns(); e[4] = w0; e[5] = w1; e[6] = w2; e[7] = (unsigned long long)items;
}
template <int OFF>
__device__ __forceinline__ void um_sts32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.u32 [%0+%1], %2;" ::"r"(addr), "n"(OFF), "r"(v) : "memory");
}

template <int NB>
struct UmLayout {
    static constexpr int B_BYTES = NB * 256;  // two swizzled tiles of [NB rows][128 bytes]
    static constexpr int MR = NB / 2;         // activation rows served
    static constexpr int A_OFF = 0;
    static constexpr int B_OFF = A_OFF + UM_SLOTS * UM_A_BYTES;
    static constexpr int HDR_OFF = B_OFF + UM_BSLOTS * B_BYTES;               // [UM_HDR][128 rows][16 B]
    static constexpr int SIDE_OFF = HDR_OFF + UM_HDR * UM_GROUP_ROWS * 16;    // [UM_SIDE][MR][UM_SIDE_FLOATS] f32
    static constexpr int XCH_OFF = SIDE_OFF + UM_SIDE * MR * UM_SIDE_FLOATS * 4;  // [MR][128] f32: second epilogue set -> first
    static constexpr int BAR_OFF = XCH_OFF + MR * UM_GROUP_ROWS * 4;
    // barriers: a_full, a_empty [UM_SLOTS]; b_full, b_empty [UM_BSLOTS]; acc_full, acc_empty [UM_NACC]; then the
    // tensor-memory address word and the "last CTA of the group" flag
    static constexpr int N_BARS = 2 * UM_SLOTS + 2 * UM_BSLOTS + 2 * UM_NACC;
    static_assert(BAR_OFF + N_BARS * 8 + 16 + 1024 <= 227 * 1024, "shared memory over the limit");
    static constexpr int TOTAL = BAR_OFF + N_BARS * 8 + 16 + 1024;  // + alignment slack
    static constexpr int TMEM_COLS = UM_NACC * 8 * NB;              // 256 or 512: a power of two >= 32
};

template <int NB>
__global__ void __launch_bounds__(UM_THREADS, 1) q4k_umma_kernel(UmParams p) {
    using L = UmLayout<NB>;
    constexpr int MR = L::MR;
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t a_u32 = base + L::A_OFF, b_u32 = base + L::B_OFF, hdr_u32 = base + L::HDR_OFF, side_u32 = base + L::SIDE_OFF;
    const uint32_t xch_u32 = base + L::XCH_OFF, bars = base + L::BAR_OFF;
    const uint32_t a_full = bars, a_empty = a_full + 8 * UM_SLOTS, b_full = a_empty + 8 * UM_SLOTS, b_empty = b_full + 8 * UM_BSLOTS;
    const uint32_t acc_full = b_empty + 8 * UM_BSLOTS, acc_empty = acc_full + 8 * UM_NACC;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + L::BAR_OFF + L::N_BARS * 8);
    volatile uint32_t *last_flag = tmem_slot + 1;

    const LinearArgs &a = p.a;
    const int M = (int)a.M;
    const int64_t SBp = a.SBp, T = p.total_items;
    const int64_t i0 = (int64_t)blockIdx.x * T / gridDim.x, i1 = (int64_t)(blockIdx.x + 1) * T / gridDim.x;
    const int n_items = (int)(i1 - i0);
    const int64_t g_first = i0 / SBp;
    const int sb_first = (int)(i0 - g_first * SBp);

    grid_launch_dependents();
    if (threadIdx.x == 0) {
        for (int i = 0; i < UM_SLOTS; i++) {
            mbar_init(a_full + 8 * i, UM_GROUP_TILES);  // one arrival per expansion warp of the item's set
            mbar_init(a_empty + 8 * i, 1);
        }
        for (int i = 0; i < UM_BSLOTS; i++) {
            mbar_init(b_full + 8 * i, 1);
            mbar_init(b_empty + 8 * i, 1);
        }
        for (int i = 0; i < UM_NACC; i++) {
            mbar_init(acc_full + 8 * i, 1);
            mbar_init(acc_empty + 8 * i, UM_EPI_WARPS / 2);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // the activation operand slots start as zeros: rows beyond 2M are never written again
    for (int i = threadIdx.x; i < UM_BSLOTS * L::B_BYTES / 16; i += UM_THREADS) sts128<0>(b_u32 + i * 16, 0u, 0u, 0u, 0u);
    fence_async_shared();
    if (warp == UM_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_slot)),
                     "r"((uint32_t)L::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    um_fence_before();
    __syncthreads();
    um_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < UM_EPI_WARPS) {
        // ---------------------------------------------------------------- epilogue: thread = weight row of the group
        // Set `es` (warps 4 es .. 4 es + 3, one per 32-lane quarter of tensor memory) takes the items of parity es
        // and keeps its own running sums; when the CTA's run inside a group ends, the second set hands its sums to
        // the first through shared memory and the first set writes the outputs.
        grid_dependency_wait();  // outputs, workspace and counters may still be in use by the preceding kernel
        const int es = warp >> 2, quarter = warp & 3;
        const int r = quarter * 32 + lane;
        float acc[MR];
#pragma unroll
        for (int m = 0; m < MR; m++) acc[m] = 0.f;
        bool alive = true;
        const bool tr = p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0;
        unsigned long long t_begin = tr ? global_ns() : 0, t_w0 = 0, t_w1 = 0, tt = 0;
        int64_t G = g_first;
        int sb = sb_first, run_sb0 = sb_first;  // run_sb0: first super-block of this CTA's run inside group G
        for (int li = 0; li < n_items; li++) {
            if ((li & 1) == es) {
                const int accb = li % UM_NACC, use = li / UM_NACC;
                float sxv[MR];  // chunk scales of the activation rows (requested before the wait, used after the sums)
#pragma unroll
                for (int m = 0; m < MR; m++) sxv[m] = m < M ? __ldcg(p.xq.sx + (int64_t)m * sx_stride(SBp) + sb) : 0.f;
                if (tr) tt = (unsigned long long)clock64();
                if (alive) alive = um_wait_warp(acc_full + 8 * accb, (uint32_t)(use & 1), p.status, lane);
                if (tr) t_w0 += (unsigned long long)clock64() - tt;
                um_fence_after();
                const uint4 hv = lds128<0>(hdr_u32 + (uint32_t)((li % UM_HDR) * (UM_GROUP_ROWS * 16) + r * 16));
                const __half2 dd = *reinterpret_cast<const __half2 *>(&hv.x);
                const float d = __low2float(dd), dmin = __high2float(dd);
                const uint32_t scw[2] = {hv.y & 0x3f3f3f3fu, (hv.w & 0x0f0f0f0fu) | ((hv.y >> 2) & 0x30303030u)};
                const uint32_t mnw[2] = {hv.z & 0x3f3f3f3fu, ((hv.w >> 4) & 0x0f0f0f0fu) | ((hv.z >> 2) & 0x30303030u)};
                const uint32_t side = side_u32 + (uint32_t)((li % UM_SIDE) * (MR * UM_SIDE_FLOATS * 4));
                float sa[MR], sm[MR];
#pragma unroll
                for (int m = 0; m < MR; m++) sa[m] = sm[m] = 0.f;
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(accb * 8 * NB);
                // sub-blocks in batches of JB: all loads of a batch are in flight before the one wait
                constexpr int JB = 16 / NB;
#pragma unroll
                for (int jb = 0; jb < 8; jb += JB) {
                    uint32_t v[JB][NB];
#pragma unroll
                    for (int jj = 0; jj < JB; jj++) um_tmem_ld<NB>(taddr + (uint32_t)((jb + jj) * NB), v[jj]);
                    um_tmem_wait();
#pragma unroll
                    for (int jj = 0; jj < JB; jj++) um_pin<NB>(v[jj]);
#pragma unroll
                    for (int jj = 0; jj < JB; jj++) {
                        const int j = jb + jj;
                        const float sc = (float)((scw[j >> 2] >> (8 * (j & 3))) & 0xffu), mn = (float)((mnw[j >> 2] >> (8 * (j & 3))) & 0xffu);
#pragma unroll
                        for (int m = 0; m < MR; m++) {
                            if (m < M) {
                                const float tq = fmaf(256.f, (float)(int)v[jj][2 * m], (float)(int)v[jj][2 * m + 1]);  // exact: below 2^24
                                sa[m] = fmaf(sc, tq, sa[m]);
                                float s32;
                                asm volatile("ld.shared.f32 %0, [%1];" : "=f"(s32) : "r"(side + (uint32_t)((m * UM_SIDE_FLOATS + j) * 4)));
                                sm[m] = fmaf(mn, s32, sm[m]);
                            }
                        }
                    }
                }
#pragma unroll
                for (int m = 0; m < MR; m++)
                    if (m < M) acc[m] = fmaf(d * sxv[m], sa[m], fmaf(-dmin * sxv[m], sm[m], acc[m]));
                um_fence_before();
                __syncwarp();
                if (lane == 0) um_arrive(acc_empty + 8 * accb);
            }
            if (sb == SBp - 1 || li == n_items - 1) {
                // ---- the run inside group G ends here (both sets pass through, whichever took the last item)
                if (tr) tt = (unsigned long long)clock64();
                if (es == 1) {
#pragma unroll
                    for (int m = 0; m < MR; m++)
                        if (m < M) stsf<0>(xch_u32 + (uint32_t)((m * UM_GROUP_ROWS + r) * 4), acc[m]);
                }
                named_barrier(1, UM_EPI_WARPS * 32);
                if (es == 0) {
#pragma unroll
                    for (int m = 0; m < MR; m++)
                        if (m < M) acc[m] += ldsf<0>(xch_u32 + (uint32_t)((m * UM_GROUP_ROWS + r) * 4));
                    const int64_t n = G * UM_GROUP_ROWS + r;
                    const bool whole = run_sb0 == 0 && sb == SBp - 1;
                    bool finish = whole;
                    int64_t c_first = blockIdx.x, c_last = blockIdx.x;
                    if (!whole) {
                        // owner of item I: the largest c with c * T / grid <= I
                        c_first = ((G * SBp + 1) * (int64_t)gridDim.x - 1) / T;
                        c_last = (((G + 1) * SBp) * (int64_t)gridDim.x - 1) / T;
                        float *slot = p.ws + ((int64_t)blockIdx.x + G) * M * UM_GROUP_ROWS;
#pragma unroll
                        for (int m = 0; m < MR; m++)
                            if (m < M) __stcg(slot + m * UM_GROUP_ROWS + r, acc[m]);
                        __threadfence();
                        named_barrier(2, UM_EPI_WARPS * 16);
                        if (r == 0) {
                            const unsigned old = atomicAdd(p.counters + G, 1u);
                            const bool last = old == (unsigned)(c_last - c_first);
                            if (last) p.counters[G] = 0u;  // ready for the next launch
                            *last_flag = last ? 1u : 0u;
                        }
                        named_barrier(2, UM_EPI_WARPS * 16);
                        finish = *last_flag != 0u;
                        if (finish) __threadfence();
                    }
                    if (finish && n < a.N) {
#pragma unroll
                        for (int m = 0; m < MR; m++) {
                            if (m < M) {
                                float v = acc[m];
                                if (!whole) {
                                    v = 0.f;
                                    for (int64_t c = c_first; c <= c_last; c++) v += __ldcg(p.ws + ((c + G) * M + m) * UM_GROUP_ROWS + r);
                                }
                                if (a.bias != nullptr) v += load_as_float(a.bias, a.bias_dt, n);
                                store_from_float(a.y, a.y_dt, m * a.ldy + n, v);
                            }
                        }
                    }
                }
                named_barrier(1, UM_EPI_WARPS * 32);  // the exchange area and the flag word are free again
#pragma unroll
                for (int m = 0; m < MR; m++) acc[m] = 0.f;
                if (tr) t_w1 += (unsigned long long)clock64() - tt;  // time in the group flush
            }
            if (++sb == SBp) {
                sb = 0;
                run_sb0 = 0;
                G++;
            }
        }
        if (tr) um_trace(p.trace, 0, t_begin, t_w0, t_w1, 0, n_items);
    } else if (warp < UM_B_WARP) {
        // ---------------------------------------------------------------- expansion: nibbles -> uint8 operand rows
        const int ew = warp - UM_EPI_WARPS, set = ew >> 3, tau = ew & 7;
        // This lane takes piece (g, t) of every 512-byte chunk, with g = bits 0 and 1 of lane >> 2 exchanged (so that
        // the eight lanes of a shared-store phase cover eight different 16-byte slot positions).  Register `sl` of a
        // chunk covers row g + 8 (sl & 1) of the row tile and sub-block pair u = th + 2 (sl >> 1): low nibbles =
        // sub-block 2u, high nibbles = sub-block 2u + 1, weights 8 n + 4 (t & 1) .. +3 in chunk n.  The four chunks of a
        // register make the 16 bytes of half t & 1 of the sub-block's operand row.  The slot is two [128][128 B] tiles
        // (sub-blocks 0..3 and 4..7, i.e. sl >> 1), a row's 16-byte slots XOR-ed with row & 7.
        const int gl = lane >> 2, g = (gl & 4) | ((gl & 1) << 1) | ((gl >> 1) & 1), t = lane & 3, th = t >> 1;
        const uint32_t row_off = (uint32_t)((tau * 16 + g) * 128);
        const uint32_t off_lo = row_off + (uint32_t)((((4 * th + (t & 1)) ^ g)) << 4), off_hi = row_off + (uint32_t)((((4 * th + 2 + (t & 1)) ^ g)) << 4);
        uint32_t mask = 0x0f0f0f0fu;
        asm volatile("" : "+r"(mask));
        struct Packed {
            uint4 c[4];
            uint4 h;  // lanes 0..15: the header of row `lane`
        };
        int64_t G = g_first;
        int sb = sb_first;
        auto advance = [&](int by) {
            sb += by;
            while (sb >= SBp) {
                sb -= (int)SBp;
                G++;
            }
        };
        auto load = [&](bool ok) {
            Packed q;
#pragma unroll
            for (int c = 0; c < 4; c++) q.c[c] = make_uint4(0, 0, 0, 0);
            q.h = make_uint4(0, 0, 0, 0);
            const int64_t rt = G * UM_GROUP_TILES + tau;
            if (ok && rt < a.NT) {
                const uint8_t *tp = a.tiles + (rt * SBp + sb) * (int64_t)tile_bytes(TTQ_FMT_Q4_K);
#pragma unroll
                for (int c = 0; c < 4; c++) q.c[c] = __ldg(reinterpret_cast<const uint4 *>(tp + c * 512 + (4 * g + t) * 16));
                if (lane < 16) q.h = __ldg(reinterpret_cast<const uint4 *>(tp + 2048 + lane * 16));
            }
            return q;
        };
        advance(set);
        Packed nxt = load(set < n_items);
        bool alive = true;
        const bool tr = p.trace != nullptr && blockIdx.x == 0 && ew == 0 && lane == 0;
        unsigned long long t_begin = tr ? global_ns() : 0, t_w0 = 0, tt = 0;
        for (int li = set; li < n_items; li += 2) {
            const Packed cur = nxt;
            advance(2);
            nxt = load(li + 2 < n_items);
            const int slot = li % UM_SLOTS, use = li / UM_SLOTS;
            if (tr) tt = (unsigned long long)clock64();
            if (use >= 1 && alive) alive = um_wait_warp(a_empty + 8 * slot, (uint32_t)((use - 1) & 1), p.status, lane);
            if (tr) t_w0 += (unsigned long long)clock64() - tt;
            if (lane < 16)
                sts128<0>(hdr_u32 + (uint32_t)((li % UM_HDR) * (UM_GROUP_ROWS * 16) + (tau * 16 + lane) * 16), cur.h.x, cur.h.y, cur.h.z, cur.h.w);
            const uint32_t alo = a_u32 + (uint32_t)(slot * UM_A_BYTES) + off_lo, ahi = a_u32 + (uint32_t)(slot * UM_A_BYTES) + off_hi;
            // register sl: + 1024 for rows g + 8, + 16384 for sub-blocks 4..7
            sts128<0>(alo, cur.c[0].x & mask, cur.c[1].x & mask, cur.c[2].x & mask, cur.c[3].x & mask);
            sts128<0>(ahi, (cur.c[0].x >> 4) & mask, (cur.c[1].x >> 4) & mask, (cur.c[2].x >> 4) & mask, (cur.c[3].x >> 4) & mask);
            sts128<1024>(alo, cur.c[0].y & mask, cur.c[1].y & mask, cur.c[2].y & mask, cur.c[3].y & mask);
            sts128<1024>(ahi, (cur.c[0].y >> 4) & mask, (cur.c[1].y >> 4) & mask, (cur.c[2].y >> 4) & mask, (cur.c[3].y >> 4) & mask);
            sts128<16384>(alo, cur.c[0].z & mask, cur.c[1].z & mask, cur.c[2].z & mask, cur.c[3].z & mask);
            sts128<16384>(ahi, (cur.c[0].z >> 4) & mask, (cur.c[1].z >> 4) & mask, (cur.c[2].z >> 4) & mask, (cur.c[3].z >> 4) & mask);
            sts128<17408>(alo, cur.c[0].w & mask, cur.c[1].w & mask, cur.c[2].w & mask, cur.c[3].w & mask);
            sts128<17408>(ahi, (cur.c[0].w >> 4) & mask, (cur.c[1].w >> 4) & mask, (cur.c[2].w >> 4) & mask, (cur.c[3].w >> 4) & mask);
            fence_async_shared();
            __syncwarp();
            if (lane == 0) um_arrive(a_full + 8 * slot);
        }
        if (tr) um_trace(p.trace, 1, t_begin, t_w0, 0, 0, n_items);
    } else if (warp == UM_B_WARP) {
        // ---------------------------------------------------------------- activation operand and side sums
        if (p.prefetch) {
            // this CTA's packed run, one request per (group, row tile): contiguous along K
            int64_t G = g_first;
            int sb0 = sb_first, left = n_items;
            while (left > 0) {
                const int nsb = (int)(SBp - sb0) < left ? (int)(SBp - sb0) : left;
                const int64_t rt = G * UM_GROUP_TILES + lane;
                if (lane < UM_GROUP_TILES && rt < a.NT) {
                    const uint8_t *tp = a.tiles + (rt * SBp + sb0) * (int64_t)tile_bytes(TTQ_FMT_Q4_K);
                    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(tp), "r"((uint32_t)(nsb * tile_bytes(TTQ_FMT_Q4_K))) : "memory");
                }
                left -= nsb;
                sb0 = 0;
                G++;
            }
        }
        grid_dependency_wait();  // the planes and their sums are written by the activation pass
        const int64_t Kp = SBp * TILE_K;
        bool alive = true;
        int sb = sb_first;
        // Asynchronous 16-byte copies, one group per item; an item is handed to the MMA lane two iterations after
        // its copies were issued, when its group has landed.
        const bool tr = p.trace != nullptr && blockIdx.x == 0 && lane == 0;
        unsigned long long t_begin = tr ? global_ns() : 0, t_w0 = 0, t_w1 = 0, tt = 0;
        auto hand_over = [&](int item) {
            fence_async_shared();
            __syncwarp();
            if (lane == 0) um_arrive(b_full + 8 * (item % UM_BSLOTS));
        };
        for (int li = 0; li < n_items; li++) {
            if (li >= 2) {
                if (tr) tt = (unsigned long long)clock64();
                asm volatile("cp.async.wait_group 1;" ::: "memory");
                if (tr) t_w1 += (unsigned long long)clock64() - tt;
                hand_over(li - 2);
            }
            const int slot = li % UM_BSLOTS, use = li / UM_BSLOTS;
            if (tr) tt = (unsigned long long)clock64();
            if (use >= 1 && alive) alive = um_wait_warp(b_empty + 8 * slot, (uint32_t)((use - 1) & 1), p.status, lane);
            if (tr) t_w0 += (unsigned long long)clock64() - tt;
            // row n = 2m + plane of the operand: 256 bytes = 16 slots; slot s goes to tile s >> 3, position (s & 7) ^ (n & 7)
            const uint32_t bs = b_u32 + (uint32_t)(slot * L::B_BYTES);
            for (int idx = lane; idx < 2 * M * 16; idx += 32) {
                const int n = idx >> 4, s = idx & 15;
                um_cp16(bs + (uint32_t)((s >> 3) * (NB * 128) + n * 128 + (((s & 7) ^ (n & 7)) << 4)),
                        p.xq.planes + (int64_t)n * Kp + (int64_t)sb * TILE_K + s * 16);
            }
            // the eight sub-block sums of every activation row (32 bytes each)
            const uint32_t side = side_u32 + (uint32_t)((li % UM_SIDE) * (MR * UM_SIDE_FLOATS * 4));
            if (lane < 2 * M) um_cp16(side + (uint32_t)((lane >> 1) * UM_SIDE_FLOATS * 4 + (lane & 1) * 16),
                                      p.xq.sum32 + (int64_t)(lane >> 1) * (Kp / 32) + sb * 8 + (lane & 1) * 4);
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (++sb == SBp) sb = 0;
        }
        if (n_items >= 2) {
            asm volatile("cp.async.wait_group 1;" ::: "memory");
            hand_over(n_items - 2);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        hand_over(n_items - 1);
        if (tr) um_trace(p.trace, 2, t_begin, t_w0, t_w1, 0, n_items);
    } else {
        // ---------------------------------------------------------------- MMA issue
        {
            bool alive = true;
            constexpr uint32_t idesc = um_idesc(NB);
            const bool tr = p.trace != nullptr && blockIdx.x == 0 && lane == 0;
            unsigned long long t_begin = tr ? global_ns() : 0, t_w0 = 0, t_w1 = 0, t_w2 = 0, tt = 0, t_i = 0, t_c = 0;
            for (int li = 0; li < n_items; li++) {
                const int slot = li % UM_SLOTS, bslot = li % UM_BSLOTS, accb = li % UM_NACC;
                if (tr) tt = (unsigned long long)clock64();
                if (alive) alive = um_wait(a_full + 8 * slot, (uint32_t)((li / UM_SLOTS) & 1), p.status);
                if (tr) { t_w0 += (unsigned long long)clock64() - tt; tt = (unsigned long long)clock64(); }
                if (alive) alive = um_wait(b_full + 8 * bslot, (uint32_t)((li / UM_BSLOTS) & 1), p.status);
                if (tr) { t_w1 += (unsigned long long)clock64() - tt; tt = (unsigned long long)clock64(); }
                if (li >= UM_NACC && alive) alive = um_wait(acc_empty + 8 * accb, (uint32_t)((li / UM_NACC - 1) & 1), p.status);
                if (tr) t_w2 += (unsigned long long)clock64() - tt;
                if (tr) tt = (unsigned long long)clock64();
                um_fence_after();
                const uint32_t ab = a_u32 + (uint32_t)(slot * UM_A_BYTES), bs = b_u32 + (uint32_t)(bslot * L::B_BYTES);
                const uint32_t td = tmem_base + (uint32_t)(accb * 8 * NB);
                if (lane == 0) {
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    // sub-block j: K tile j >> 2, 32 bytes = 2 descriptor units along the swizzled row
                    const uint64_t ad = um_desc_sw128(ab + (uint32_t)((j >> 2) * 16384)) + (uint64_t)(2 * (j & 3));
                    const uint64_t bd = um_desc_sw128(bs + (uint32_t)((j >> 2) * (NB * 128))) + (uint64_t)(2 * (j & 3));
                    um_mma(td + (uint32_t)(j * NB), ad, bd, idesc);
                }
                if (tr) { t_i += (unsigned long long)clock64() - tt; tt = (unsigned long long)clock64(); }
                um_commit(a_empty + 8 * slot);
                um_commit(b_empty + 8 * bslot);
                um_commit(acc_full + 8 * accb);
                }
                __syncwarp();
                if (tr) t_c += (unsigned long long)clock64() - tt;
            }
            if (tr) um_trace(p.trace, 3, t_begin, t_w0, t_w1, t_w2, n_items);
            if (tr) um_trace(p.trace, 4, t_begin, t_i, t_c, 0, n_items);
        }
        __syncwarp();
    }
    um_fence_before();
    __syncthreads();
    if (warp == UM_MMA_WARP) {
        um_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)L::TMEM_COLS) : "memory");
    }
}

template <int NB>
cudaError_t um_launch(const UmParams &p, unsigned grid, cudaStream_t st) {
    using L = UmLayout<NB>;
    static bool configured[64] = {};  // per device: the shared-memory opt-in belongs to the device's copy of the function
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!configured[dev]) {
        e = cudaFuncSetAttribute(q4k_umma_kernel<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    return launch_pdl(q4k_umma_kernel<NB>, dim3(grid), dim3(UM_THREADS), (size_t)L::TOTAL, st, p);
}

}  // namespace

// Activation pass + tensor-memory decode linear.  cudaErrorNotSupported: the caller takes another path (more than 8
// rows, scratch too small for this K, or more groups than arrival counters).
cudaError_t launch_q4k_umma(const LinearArgs &a, const XqView &xq, int64_t xq_capacity_k, int sms, int *status, unsigned long long *trace,
                            float *ws, size_t ws_bytes, unsigned *counters, int64_t counters_cap, cudaStream_t st, int *launches) {
    *launches = 0;
    if (a.M < 1 || a.M > 8) return cudaErrorNotSupported;
    if (a.SBp * TILE_K > xq_capacity_k) return cudaErrorNotSupported;
    UmParams p;
    p.a = a;
    p.xq = xq;
    p.ws = ws;
    p.counters = counters;
    p.status = status;
    p.trace = trace;
    p.n_groups = (a.NT + UM_GROUP_TILES - 1) / UM_GROUP_TILES;
    p.total_items = p.n_groups * a.SBp;
    static const bool prefetch = env_flag("TTQ_UMMA_PREFETCH", true);
    p.prefetch = prefetch ? 1 : 0;
    const unsigned grid = (unsigned)(p.total_items < sms ? p.total_items : sms);
    if (p.n_groups > counters_cap) return cudaErrorNotSupported;
    if ((size_t)(grid + p.n_groups) * a.M * UM_GROUP_ROWS * sizeof(float) > ws_bytes) return cudaErrorNotSupported;
    cudaError_t e = launch_xprep(a, xq, a.M, trace, st, true);
    if (e != cudaSuccess) return e;
    ++*launches;
    e = a.M <= 4 ? um_launch<8>(p, grid, st) : um_launch<16>(p, grid, st);
    if (e == cudaSuccess) ++*launches;
    return e;
}

}  // namespace ttq
