// Decode-side kernels: y[M<=16][N] = x . W^T on the tiled quantized layout.
//
// Arithmetic: activations are converted once per call to 16-bit fixed point per 256-wide K chunk
// (xq = 256*hi + lo, both planes int8, one fp32 scale sx per chunk).  Weight quants stay integers.
// The dot product of one sub-block (32 weights for Q4_K / Q8_0, 16 for Q6_K) is an integer
// tensor-core instruction (mma.sync m16n8k32 / m16n8k16, u8|s8 x s8 -> s32) and is exact; the
// sub-block scale, the Q4_K min term and sx are applied in fp32.  One MMA covers 16 weight rows and
// 4 activation rows (8 columns = 4 x {hi, lo}).
//
// Work split: a persistent grid (up to three CTAs per SM).  The 8 warps of a CTA form 8/WK groups of
// WK warps; a group owns one row tile (16 rows) per iteration and its warps split K.  Every warp
// streams its run of tiles through a private ring of shared-memory stages filled by bulk async
// copies (cp.async.bulk + mbarrier, no multicast), so the bytes in flight per SM do not depend on
// registers; a 16-byte shared load per lane is a complete A fragment.  Partial sums of a group meet
// in shared memory behind a named barrier.
//
// Activations reach the CTA in one of three ways (template XSRC):
//   0  converted in the CTA prologue from x itself (no extra launch; every CTA repeats the work)
//   1  converted once by a separate pass into scratch, then bulk-copied into shared memory
//   2  converted once into scratch and read from there fragment by fragment (M > 4, or planes too
//      large for shared memory)
// Kernels are launched with programmatic stream serialization: a kernel starts its weight copies
// while its predecessor drains and executes griddepcontrol.wait before touching activations.
#include <cstdlib>

#include "ttq_internal.cuh"

namespace ttq {

namespace {

constexpr int GEMV_WARPS = 8;
constexpr int GEMV_THREADS = GEMV_WARPS * 32;
constexpr int PLANE_PAD = 16;  // bytes between activation planes in shared memory (bank spread)

// ---- integer tensor-core wrappers ---------------------------------------------------------------
__device__ __forceinline__ void mma_k32_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};\n"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_k32_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};\n"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_k16_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};\n"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// ---- bulk-copy ring primitives (all waits are bounded) ---------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
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
// Waits for a stage; gives up after WAIT_LIMIT polls, records the failure and lets the caller go on
// (with garbage data) so that every warp still reaches its barriers and the kernel returns.
constexpr int WAIT_LIMIT = 1 << 20;
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int *status) {
    for (int i = 0; i < WAIT_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    atomicOr(status, 1);
    return false;
}
__device__ __forceinline__ void named_barrier(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// compile-time loop: f(std::integral_constant<int, I>) for I in [0, N)
template <int V>
struct IC {
    static constexpr int value = V;
};
template <int I, int N, class F>
__device__ __forceinline__ void static_for(F &&f) {
    if constexpr (I < N) {
        f(IC<I>{});
        static_for<I + 1, N>(f);
    }
}

// ---- activation conversion -------------------------------------------------------------------
// Destination of one activation row's planes and side sums (shared memory or global scratch).
struct XqRow {
    int8_t *hi, *lo;  // [Kp]
    float *sum16;     // [Kp/16]
    float *sum32;     // [Kp/32]
    float *sx;        // [SBs]
};

__host__ __device__ constexpr int sx_stride(int64_t SBp) { return (int)((SBp + 3) & ~(int64_t)3); }

// One warp converts the 256-wide chunk `sb` of activation row `xrow` (nullptr = emit zeros):
// xq = round(x * 32639 / amax) in [-32639, 32639], stored as two int8 planes with xq = 256*hi + lo.
__device__ __forceinline__ void xprep_chunk(const void *xrow, int x_dt, int64_t K, int sb, int lane, const XqRow &dst) {
    const int64_t k0 = (int64_t)sb * TILE_K + 8 * lane;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = 0.f;
    if (xrow != nullptr) {
        const bool vec = (x_dt != TTQ_DT_F32) && (k0 + 8 <= K) &&
                         ((reinterpret_cast<uintptr_t>(xrow) + 2 * k0) & 15) == 0;
        if (vec) {
            uint4 raw = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(xrow) + k0);
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                if (x_dt == TTQ_DT_BF16) {
                    v[2 * i] = __uint_as_float(w[i] << 16);
                    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
                } else {
                    float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
                    v[2 * i] = f.x;
                    v[2 * i + 1] = f.y;
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++)
                if (k0 + i < K) v[i] = load_as_float(xrow, x_dt, k0 + i);
        }
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    // amax * inv <= 32639 * (1 + 2^-22): rounds to at most 32639, no clamp needed
    const float inv = amax > 1e-20f ? (float)XQ_MAX * __frcp_rn(amax) : 0.f;
    int q[8], s = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        q[i] = __float2int_rn(v[i] * inv);
        s += q[i];
    }
    // low plane = low byte of q (as int8); high plane = byte 1 of q + 128 (carry when the low byte is negative)
    uint32_t low[2], hiw[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const uint32_t a = __byte_perm(q[4 * i], q[4 * i + 1], 0x0040), b = __byte_perm(q[4 * i + 2], q[4 * i + 3], 0x0040);
        low[i] = __byte_perm(a, b, 0x5410);
        const uint32_t c = __byte_perm(q[4 * i] + 128, q[4 * i + 1] + 128, 0x0051),
                       d = __byte_perm(q[4 * i + 2] + 128, q[4 * i + 3] + 128, 0x0051);
        hiw[i] = __byte_perm(c, d, 0x5410);
    }
    *reinterpret_cast<uint2 *>(dst.hi + k0) = make_uint2(hiw[0], hiw[1]);
    *reinterpret_cast<uint2 *>(dst.lo + k0) = make_uint2(low[0], low[1]);
    const int s16 = s + __shfl_xor_sync(0xffffffffu, s, 1);
    const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);
    if ((lane & 1) == 0) dst.sum16[sb * 16 + (lane >> 1)] = (float)s16;
    if ((lane & 3) == 0) dst.sum32[sb * 8 + (lane >> 2)] = (float)s32;
    if (lane == 0) dst.sx[sb] = amax > 1e-20f ? amax * (1.0f / (float)XQ_MAX) : 0.f;
}

// Separate conversion pass: (Mpad x SBp) chunks, one warp each; rows >= M are written as zeros.
__global__ void __launch_bounds__(GEMV_THREADS) xprep_kernel(const void *__restrict__ x, int x_dt, int64_t M,
                                                             int64_t Mpad, int64_t K, int64_t ldx, int64_t SBp,
                                                             XqView xq) {
    grid_launch_dependents();
    grid_dependency_wait();  // the scratch planes may still be read by the preceding kernel
    const int lane = threadIdx.x & 31;
    const int64_t Kp = SBp * TILE_K;
    const int64_t unit = (int64_t)blockIdx.x * GEMV_WARPS + (threadIdx.x >> 5);
    if (unit >= Mpad * SBp) return;
    const int64_t m = unit / SBp;
    const int sb = (int)(unit % SBp);
    XqRow dst{xq.planes + (2 * m) * Kp, xq.planes + (2 * m + 1) * Kp, xq.sum16 + m * (Kp / 16),
              xq.sum32 + m * (Kp / 32), xq.sx + m * sx_stride(SBp)};
    const void *xrow = nullptr;
    if (m < M) {
        const int esz = x_dt == TTQ_DT_F32 ? 4 : 2;
        xrow = reinterpret_cast<const uint8_t *>(x) + m * ldx * esz;
    }
    xprep_chunk(xrow, x_dt, K, sb, lane, dst);
}

// ---- shared-memory access with 32-bit addresses and immediate offsets ----------------------------
template <int OFF>
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ float ldsf(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2+%3];" : "=f"(v.x), "=f"(v.y) : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ float4 lds128f(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4+%5];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ void stsf(uint32_t addr, float v) {
    asm volatile("st.shared.f32 [%0+%1], %2;" ::"r"(addr), "n"(OFF), "f"(v) : "memory");
}

// ---- the GEMV --------------------------------------------------------------------------------
struct GemvParams {
    LinearArgs a;
    XqView xq;    // activation planes in scratch (XSRC 1 and 2)
    int wk;       // warps that split K of one row tile (1, 2, 4 or 8)
    int *status;  // device word: bit 0 set when a bounded wait gave up
};

#ifndef TTQ_RING_STAGES
#define TTQ_RING_STAGES 2
#endif
constexpr int RING_STAGES = TTQ_RING_STAGES;  // stages of each warp's bulk-copy ring
constexpr int XSRC_CONVERT = 0, XSRC_COPY = 1, XSRC_GLOBAL = 2;

// Shared-memory carve-up, identical on host (size) and device (offsets).  `rows` = activation rows
// held in shared memory (0 when they stay in scratch).
struct SmemLayout {
    uint32_t bars, hdr, red, ring, sx, sum32, sum16, planes, total;
};
__host__ __device__ inline SmemLayout smem_layout(int fmt, int MG, int rows, int64_t SBp) {
    SmemLayout L;
    const int64_t Kp = SBp * TILE_K;
    uint32_t o = 0;
    L.bars = o; o += 256 + 64 * (RING_STAGES > 3 ? RING_STAGES - 3 : 0);  // [warps][stages] mbarriers + one for the planes (last 8 bytes)
    L.hdr = o; o += GEMV_WARPS * 1024;                      // per-warp unpacked sub-block scales
    L.red = o; o += GEMV_WARPS * MG * 6 * 32 * 4;           // per-warp partial sums (dot part + offset part)
    L.ring = o; o += GEMV_WARPS * RING_STAGES * tile_bytes(fmt);
    L.sx = L.sum32 = L.sum16 = L.planes = o;
    if (rows > 0) {
        L.sx = o; o += (uint32_t)(rows * sx_stride(SBp) * 4);
        L.sum32 = o; o += (uint32_t)(rows * (Kp / 32) * 4);
        L.sum16 = o; o += (uint32_t)(rows * (Kp / 16) * 4);
        L.planes = o; o += (uint32_t)(2 * rows * (Kp + PLANE_PAD));
    }
    L.total = o;
    return L;
}

// Per-lane view of the activation side, set up once per kernel.
template <int MG, bool SHARED>
struct ActView {
    uint32_t bfrag_s;            // SHARED: address of this lane's B word stream (column g, byte 4t)
    const uint8_t *bfrag_g[MG];  // !SHARED: pointers, one per activation group (column 8q+g)
    uint32_t sx_s, sum32_s, sum16_s;        // SHARED: addresses of row 0
    const float *sx_g, *sum32_g, *sum16_g;  // !SHARED
    int SBs, Kp;
    int rows;  // activation rows that exist in the side arrays

    template <int OFF>
    __device__ __forceinline__ uint32_t bword(int q, uint32_t tile_off) const {
        if constexpr (SHARED) return lds32<OFF>(bfrag_s + tile_off);
        else return __ldg(reinterpret_cast<const uint32_t *>(bfrag_g[q] + tile_off + OFF));
    }
    __device__ __forceinline__ float sx(int m, int sb) const {
        if constexpr (SHARED) return ldsf<0>(sx_s + (uint32_t)(m * SBs + sb) * 4);
        else return __ldg(sx_g + m * SBs + sb);
    }
    // four consecutive group sums of row m starting at group index gi (a multiple of 4)
    __device__ __forceinline__ float4 sum32x4(int m, int gi) const {
        if constexpr (SHARED) return lds128f<0>(sum32_s + (uint32_t)(m * (Kp / 32) + gi) * 4);
        else return __ldg(reinterpret_cast<const float4 *>(sum32_g + m * (Kp / 32) + gi));
    }
    __device__ __forceinline__ float4 sum16x4(int m, int gi) const {
        if constexpr (SHARED) return lds128f<0>(sum16_s + (uint32_t)(m * (Kp / 16) + gi) * 4);
        else return __ldg(reinterpret_cast<const float4 *>(sum16_g + m * (Kp / 16) + gi));
    }
};

__device__ __forceinline__ float byte_to_float(uint32_t w, int i) { return (float)((w >> (8 * i)) & 0xffu); }

// One tile (16 rows x 256 weights) from a shared-memory stage.
//  Main role, lane (g,t): integer dot products of rows g and g+8 with activation row 4q+t, scaled
//  by the sub-block scale, accumulated into yacc[q][0..1].
//  Header role, lane (r = lane&15, h = lane>>4): unpacks the scales of row r (half h of the
//  sub-blocks) into shared memory for the main role, and accumulates the part of the result that
//  does not depend on the quants (Q4_K: dmin*m_j * sum of activations; Q6_K: the -32 offset) into
//  oacc[m], m < MR.  Output = sum over K tiles of (yacc part) - (oacc parts of both halves).
template <int FMT, int MG, bool SHARED, int MR>
__device__ __forceinline__ void compute_tile(uint32_t stage, int sb, int lane, uint32_t hdr,
                                             const ActView<MG, SHARED> &A, float (&yacc)[MG][2], float (&oacc)[MR]) {
    const int g = lane >> 2, t = lane & 3;
    const int r = lane & 15, h = lane >> 4;
    const uint32_t hr = hdr + (uint32_t)g * 8;  // reader base: {scale(row g), scale(row g+8)} of sub-block 0
    const uint32_t sa = stage + (uint32_t)lane * 16;
    const uint32_t toff = (uint32_t)sb * TILE_K;
    float tmp[MG][2];
#pragma unroll
    for (int q = 0; q < MG; q++) tmp[q][0] = tmp[q][1] = 0.f;

    if constexpr (FMT == TTQ_FMT_Q4_K) {
        {
            const uint32_t hw = hdr + (uint32_t)((h * 4 * 8 + (r & 7)) * 2 + (r >> 3)) * 4;
            const uint4 hv = lds128<2048>(stage + (uint32_t)r * 16);
            const __half2 dd = *reinterpret_cast<const __half2 *>(&hv.x);
            const float d = __low2float(dd), dmin = __high2float(dd), d16 = d * 0.0625f;
            uint32_t scw, mw;
            if (h == 0) {
                scw = hv.y & 0x3f3f3f3fu;
                mw = hv.z & 0x3f3f3f3fu;
            } else {
                scw = (hv.w & 0x0f0f0f0fu) | ((hv.y >> 2) & 0x30303030u);
                mw = ((hv.w >> 4) & 0x0f0f0f0fu) | ((hv.z >> 2) & 0x30303030u);
            }
            __syncwarp();  // main-role reads of the previous tile's scales are done
            // odd sub-blocks are fed to the MMA as 16*q (high nibble left in place): scale by d/16
            stsf<0 * 64>(hw, d * byte_to_float(scw, 0));
            stsf<1 * 64>(hw, d16 * byte_to_float(scw, 1));
            stsf<2 * 64>(hw, d * byte_to_float(scw, 2));
            stsf<3 * 64>(hw, d16 * byte_to_float(scw, 3));
            const float m0 = byte_to_float(mw, 0), m1 = byte_to_float(mw, 1), m2 = byte_to_float(mw, 2),
                        m3 = byte_to_float(mw, 3);
#pragma unroll
            for (int m = 0; m < MR; m++) {
                const float4 s4 = A.sum32x4(m, sb * 8 + h * 4);
                const float part = fmaf(m0, s4.x, fmaf(m1, s4.y, fmaf(m2, s4.z, m3 * s4.w)));
                oacc[m] = fmaf(A.sx(m, sb) * dmin, part, oacc[m]);
            }
            __syncwarp();
        }
        static_for<0, 4>([&](auto pp_) {
            constexpr int pp = decltype(pp_)::value;
            const uint4 w = lds128<pp * 512>(sa);
            static_for<0, 2>([&](auto hn_) {
                constexpr int hn = decltype(hn_)::value;
                constexpr int j = 2 * pp + hn;
                constexpr uint32_t msk = hn ? 0xf0f0f0f0u : 0x0f0f0f0fu;
                const float2 sc = lds64f<j * 64>(hr);
#pragma unroll
                for (int q = 0; q < MG; q++) {
                    int c[4];
                    mma_k32_u8s8(c, w.x & msk, w.y & msk, w.z & msk, w.w & msk, A.template bword<j * 32>(q, toff),
                                 A.template bword<j * 32 + 16>(q, toff));
                    tmp[q][0] = fmaf(sc.x, (float)(c[0] * 256 + c[1]), tmp[q][0]);
                    tmp[q][1] = fmaf(sc.y, (float)(c[2] * 256 + c[3]), tmp[q][1]);
                }
            });
        });
    } else if constexpr (FMT == TTQ_FMT_Q8_0) {
        {
            // fp16 d[r][b]: header lane (r, h) converts blocks 4h..4h+3 of row r
            const uint32_t hw = hdr + (uint32_t)((h * 4 * 8 + (r & 7)) * 2 + (r >> 3)) * 4;
            const uint2 dv = lds64<4096>(stage + (uint32_t)r * 16 + (uint32_t)h * 8);
            const float2 f01 = __half22float2(*reinterpret_cast<const __half2 *>(&dv.x));
            const float2 f23 = __half22float2(*reinterpret_cast<const __half2 *>(&dv.y));
            __syncwarp();
            stsf<0 * 64>(hw, f01.x);
            stsf<1 * 64>(hw, f01.y);
            stsf<2 * 64>(hw, f23.x);
            stsf<3 * 64>(hw, f23.y);
            __syncwarp();
        }
        static_for<0, 8>([&](auto b_) {
            constexpr int b = decltype(b_)::value;
            const uint4 w = lds128<b * 512>(sa);
            const float2 sc = lds64f<b * 64>(hr);
#pragma unroll
            for (int q = 0; q < MG; q++) {
                int c[4];
                mma_k32_s8s8(c, w.x, w.y, w.z, w.w, A.template bword<b * 32>(q, toff), A.template bword<b * 32 + 16>(q, toff));
                tmp[q][0] = fmaf(sc.x, (float)(c[0] * 256 + c[1]), tmp[q][0]);
                tmp[q][1] = fmaf(sc.y, (float)(c[2] * 256 + c[3]), tmp[q][1]);
            }
        });
    } else {
        {
            // int8 scales[r][16], fp16 d[r]: header lane (r, h) handles sub-blocks 8h..8h+7 of row r
            const uint2 scw = lds64<3072>(stage + (uint32_t)r * 16 + (uint32_t)h * 8);
            const float d = __half2float(
                __ushort_as_half((unsigned short)(lds32<3328>(stage + (uint32_t)(r >> 1) * 4) >> (16 * (r & 1)))));
            const uint32_t hw6 = hdr + (uint32_t)((h * 8 * 8 + (r & 7)) * 2 + (r >> 3)) * 4;
            float ds[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t word = i < 4 ? scw.x : scw.y;
                ds[i] = d * (float)(int)(int8_t)((word >> (8 * (i & 3))) & 0xff);
            }
            __syncwarp();
            stsf<0 * 64>(hw6, ds[0]); stsf<1 * 64>(hw6, ds[1]); stsf<2 * 64>(hw6, ds[2]); stsf<3 * 64>(hw6, ds[3]);
            stsf<4 * 64>(hw6, ds[4]); stsf<5 * 64>(hw6, ds[5]); stsf<6 * 64>(hw6, ds[6]); stsf<7 * 64>(hw6, ds[7]);
#pragma unroll
            for (int m = 0; m < MR; m++) {
                const float4 sA = A.sum16x4(m, sb * 16 + h * 8), sB = A.sum16x4(m, sb * 16 + h * 8 + 4);
                float part = fmaf(ds[0], sA.x, fmaf(ds[1], sA.y, fmaf(ds[2], sA.z, ds[3] * sA.w)));
                part = fmaf(ds[4], sB.x, fmaf(ds[5], sB.y, fmaf(ds[6], sB.z, fmaf(ds[7], sB.w, part))));
                oacc[m] = fmaf(A.sx(m, sb) * 32.f, part, oacc[m]);  // quants are stored with a +32 offset
            }
            __syncwarp();
        }
        static_for<0, 4>([&](auto c4_) {
            constexpr int c4 = decltype(c4_)::value;
            const uint4 w = lds128<c4 * 512>(sa);
            const uint2 hq = lds64<2048 + (c4 >> 1) * 512 + (c4 & 1) * 8>(sa);
            static_for<0, 4>([&](auto s_) {
                constexpr int s = decltype(s_)::value;
                constexpr int j = 4 * c4 + s;
                const uint32_t l0 = (s & 2) ? w.z : w.x, l1 = (s & 2) ? w.w : w.y;
                uint32_t a0 = (s & 1) ? (l0 >> 4) : l0, a1 = (s & 1) ? (l1 >> 4) : l1;
                // high 2 bits of sub-block s sit at bit pair s of each byte: move them to bits 4..5
                const uint32_t h0 = s == 0 ? (hq.x << 4) : s == 1 ? (hq.x << 2) : s == 2 ? hq.x : (hq.x >> 2);
                const uint32_t h1 = s == 0 ? (hq.y << 4) : s == 1 ? (hq.y << 2) : s == 2 ? hq.y : (hq.y >> 2);
                a0 = (a0 & 0x0f0f0f0fu) | (h0 & 0x30303030u);
                a1 = (a1 & 0x0f0f0f0fu) | (h1 & 0x30303030u);
                const float2 sc = lds64f<j * 64>(hr);
#pragma unroll
                for (int q = 0; q < MG; q++) {
                    int c[4];
                    mma_k16_u8s8(c, a0, a1, A.template bword<j * 16>(q, toff));
                    tmp[q][0] = fmaf(sc.x, (float)(c[0] * 256 + c[1]), tmp[q][0]);
                    tmp[q][1] = fmaf(sc.y, (float)(c[2] * 256 + c[3]), tmp[q][1]);
                }
            });
        });
    }
#pragma unroll
    for (int q = 0; q < MG; q++) {
        const int mrow = (4 * q + t) < A.rows ? (4 * q + t) : A.rows - 1;
        const float sx = A.sx(mrow, sb);
        yacc[q][0] = fmaf(sx, tmp[q][0], yacc[q][0]);
        yacc[q][1] = fmaf(sx, tmp[q][1], yacc[q][1]);
    }
}

template <int FMT, int MG, int XSRC, int MR>
__global__ void __launch_bounds__(GEMV_THREADS, XSRC == XSRC_GLOBAL ? 2 : 3) gemv_kernel(GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr bool SHARED = XSRC != XSRC_GLOBAL;
    constexpr int TB = tile_bytes(FMT);
    constexpr int STAGES = RING_STAGES;
    constexpr int MP = 4 * MG;
    const LinearArgs &a = p.a;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int SBp = (int)a.SBp, Kp = SBp * TILE_K, SBs = sx_stride(a.SBp);
    const int M = (int)a.M;
    const SmemLayout L = smem_layout(FMT, MG, SHARED ? MR : 0, a.SBp);
    const uint32_t smem0 = smem_u32(smem);

    const uint32_t hdr_u32 = smem0 + L.hdr + warp * 1024;
    float *red_s = reinterpret_cast<float *>(smem + L.red);
    const uint32_t ring_u32 = smem0 + L.ring + warp * STAGES * TB;
    const uint32_t bar_u32 = smem0 + L.bars + warp * STAGES * 8;
    const uint32_t xbar_u32 = smem0 + L.hdr - 8;  // last slot of the barrier area, past every ring barrier

    // group / K-slice of this warp
    const int WK = p.wk, R = GEMV_WARPS / WK;
    const int grp = warp / WK, ks = warp % WK;
    const int sb_begin = (ks * SBp) / WK, sb_end = ((ks + 1) * SBp) / WK;
    const int nsb = sb_end - sb_begin;
    // row tiles of this group: rt(it) = (it * gridDim.x + blockIdx.x) * R + grp
    const int64_t rt0 = (int64_t)blockIdx.x * R + grp, rt_step = (int64_t)gridDim.x * R;
    const int n_iters = rt0 < a.NT ? (int)((a.NT - rt0 + rt_step - 1) / rt_step) : 0;
    const int total_items = n_iters * nsb;

    grid_launch_dependents();  // the next kernel may start its own weight copies as soon as it fits

    // ---- ring set-up and first copies (weights do not depend on the activations)
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) mbar_init(bar_u32 + 8 * s, 1);
        if (XSRC == XSRC_COPY && warp == 0) mbar_init(xbar_u32, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    // producer state (lane 0): next item to issue, walking (iteration, K tile) without divisions
    int p_item = 0, p_sbi = 0;
    const uint8_t *p_row = a.tiles + (rt0 * SBp + sb_begin) * (int64_t)TB;
    const int64_t p_row_step = rt_step * SBp * (int64_t)TB;
    auto issue_next = [&]() {
        const int s = p_item % STAGES;
        mbar_expect_tx(bar_u32 + 8 * s, TB);
        bulk_g2s(ring_u32 + s * TB, p_row + (int64_t)p_sbi * TB, TB, bar_u32 + 8 * s);
        p_item++;
        if (++p_sbi == nsb) {
            p_sbi = 0;
            p_row += p_row_step;
        }
    };
    if (lane == 0) {
        for (int i = 0; i < STAGES && i < total_items; i++) issue_next();
    }

    // ---- activations: everything below may depend on the preceding kernel
    grid_dependency_wait();
    ActView<MG, SHARED> A;
    A.SBs = SBs;
    A.Kp = Kp;
    const int g = lane >> 2, t = lane & 3;
    bool alive = true;  // false once a bounded wait gave up: skip further waits, keep the barriers
    if constexpr (SHARED) {
        if constexpr (XSRC == XSRC_CONVERT) {
            float *sx_s = reinterpret_cast<float *>(smem + L.sx);
            float *sum32_s = reinterpret_cast<float *>(smem + L.sum32);
            float *sum16_s = reinterpret_cast<float *>(smem + L.sum16);
            int8_t *planes_s = reinterpret_cast<int8_t *>(smem + L.planes);
            const int esz = a.x_dt == TTQ_DT_F32 ? 4 : 2;
            const int units = MR * SBp;
            for (int u = warp; u < units; u += GEMV_WARPS) {
                const int m = u / SBp, sb = u - m * SBp;
                XqRow dst{planes_s + (2 * m) * (Kp + PLANE_PAD), planes_s + (2 * m + 1) * (Kp + PLANE_PAD),
                          sum16_s + m * (Kp / 16), sum32_s + m * (Kp / 32), sx_s + m * SBs};
                xprep_chunk(reinterpret_cast<const uint8_t *>(a.x) + (int64_t)m * a.ldx * esz, a.x_dt, a.K, sb, lane, dst);
            }
            __syncthreads();
        } else {
            // planes and side arrays were produced by the conversion pass: bulk-copy them in
            __syncthreads();  // the plane barrier is initialised
            if (threadIdx.x == 0) {
                const uint32_t bytes = (uint32_t)(MR * SBs * 4 + MR * (Kp / 32) * 4 + MR * (Kp / 16) * 4 + 2 * MR * Kp);
                mbar_expect_tx(xbar_u32, bytes);
                bulk_g2s(smem0 + L.sx, p.xq.sx, MR * SBs * 4, xbar_u32);
                bulk_g2s(smem0 + L.sum32, p.xq.sum32, MR * (Kp / 32) * 4, xbar_u32);
                bulk_g2s(smem0 + L.sum16, p.xq.sum16, MR * (Kp / 16) * 4, xbar_u32);
                for (int c = 0; c < 2 * MR; c++)
                    bulk_g2s(smem0 + L.planes + c * (Kp + PLANE_PAD), p.xq.planes + (int64_t)c * Kp, Kp, xbar_u32);
            }
            alive = mbar_wait_bounded(xbar_u32, 0, p.status);
        }
        // columns beyond 2*MR do not exist: such lanes read an existing column, their outputs are never stored
        const int col = g % (2 * MR);
        A.bfrag_s = smem0 + L.planes + (uint32_t)col * (Kp + PLANE_PAD) + 4 * t;
        A.sx_s = smem0 + L.sx;
        A.sum32_s = smem0 + L.sum32;
        A.sum16_s = smem0 + L.sum16;
        A.rows = MR;
    } else {
#pragma unroll
        for (int q = 0; q < MG; q++)
            A.bfrag_g[q] = reinterpret_cast<const uint8_t *>(p.xq.planes) + (int64_t)(8 * q + g) * Kp + 4 * t;
        A.sx_g = p.xq.sx;
        A.sum32_g = p.xq.sum32;
        A.sum16_g = p.xq.sum16;
        A.rows = MP;
    }

    // ---- main loop over this warp's items
    int item = 0;
    float *red_w = red_s + warp * (MG * 6 * 32);
    for (int it = 0; it < n_iters; it++) {
        float yacc[MG][2], oacc[MR];
#pragma unroll
        for (int q = 0; q < MG; q++) yacc[q][0] = yacc[q][1] = 0.f;
#pragma unroll
        for (int m = 0; m < MR; m++) oacc[m] = 0.f;
        for (int sbi = 0; sbi < nsb; sbi++, item++) {
            const int s = item % STAGES;
            if (alive) alive = mbar_wait_bounded(bar_u32 + 8 * s, (uint32_t)((item / STAGES) & 1), p.status);
            compute_tile<FMT, MG, SHARED, MR>(ring_u32 + s * TB, sb_begin + sbi, lane, hdr_u32, A, yacc, oacc);
            __syncwarp();  // every lane is done reading the stage before it is refilled
            if (lane == 0 && alive && p_item < total_items) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                issue_next();
            }
        }
        // ---- flush the row tile of this iteration: partial sums of the group's warps meet in shared memory
        const int64_t rt = rt0 + it * rt_step;
#pragma unroll
        for (int q = 0; q < MG; q++) {
            red_w[(q * 2 + 0) * 32 + lane] = yacc[q][0];
            red_w[(q * 2 + 1) * 32 + lane] = yacc[q][1];
        }
#pragma unroll
        for (int m = 0; m < MR; m++) red_w[(MG * 2 + m) * 32 + lane] = oacc[m];
        named_barrier(1 + grp, WK * 32);
        if (ks == 0) {
            for (int o = lane; o < MR * TILE_ROWS; o += 32) {
                const int row = o & 15, m = o >> 4;
                const int64_t n = rt * TILE_ROWS + row;
                if (m < M && n < a.N) {
                    const int q = m >> 2, src_lane = (row & 7) * 4 + (m & 3), i = row >> 3;
                    float acc = 0.f;
                    for (int w = 0; w < WK; w++) {
                        const float *rw = red_s + (grp * WK + w) * (MG * 6 * 32);
                        acc += rw[(q * 2 + i) * 32 + src_lane] - rw[(MG * 2 + m) * 32 + row] -
                               rw[(MG * 2 + m) * 32 + row + 16];
                    }
                    if (a.bias != nullptr) acc += load_as_float(a.bias, a.bias_dt, n);
                    store_from_float(a.y, a.y_dt, m * a.ldy + n, acc);
                }
            }
        }
        named_barrier(1 + grp, WK * 32);  // the partial-sum area is free again
    }
}

constexpr size_t GEMV_SMEM_LIMIT = 112 * 1024;  // at least two CTAs per SM

int pick_wk(int64_t NT, int64_t SBp, int64_t resident_warps) {
    // enough (row tile, K slice) units to give every resident warp work, never more slices than K tiles
    int wk = 1;
    while (wk < GEMV_WARPS && NT * wk < resident_warps && 2 * wk <= SBp) wk *= 2;
    return wk;
}

bool env_flag(const char *name, bool dflt) {
    const char *v = getenv(name);
    if (!v || !*v) return dflt;
    return v[0] != '0';
}

// Launch with programmatic stream serialization (the kernel calls griddepcontrol.wait itself).
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

template <int FMT, int MG, int XSRC, int MR>
cudaError_t launch_one(GemvParams &p, int sms, cudaStream_t st) {
    auto kernel = gemv_kernel<FMT, MG, XSRC, MR>;
    const size_t smem = smem_layout(FMT, MG, XSRC == XSRC_GLOBAL ? 0 : MR, p.a.SBp).total;
    static bool configured = false;  // per instantiation; contexts on several devices share the setting
    static int occ_cache_smem = -1, occ_cache = 0;
    cudaError_t e;
    if (!configured) {
        if ((e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMV_SMEM_LIMIT))) return e;
        configured = true;
    }
    if (occ_cache_smem != (int)smem) {
        if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ_cache, kernel, GEMV_THREADS, smem))) return e;
        occ_cache_smem = (int)smem;
    }
    if (occ_cache < 1) return cudaErrorLaunchOutOfResources;
    const int64_t cap = (int64_t)sms * occ_cache;
    p.wk = pick_wk(p.a.NT, p.a.SBp, cap * GEMV_WARPS);
    const int R = GEMV_WARPS / p.wk;
    const int64_t cta_iters = (p.a.NT + R - 1) / R;
    const unsigned grid = (unsigned)(cta_iters < cap ? cta_iters : cap);
    return launch_pdl(kernel, dim3(grid), dim3(GEMV_THREADS), smem, st, p);
}

template <int FMT, int XSRC>
cudaError_t dispatch_shared(GemvParams &p, int sms, cudaStream_t st) {
    switch (p.a.M) {
    case 1: return launch_one<FMT, 1, XSRC, 1>(p, sms, st);
    case 2: return launch_one<FMT, 1, XSRC, 2>(p, sms, st);
    case 3: return launch_one<FMT, 1, XSRC, 3>(p, sms, st);
    default: return launch_one<FMT, 1, XSRC, 4>(p, sms, st);
    }
}

template <int FMT>
cudaError_t dispatch(GemvParams &p, int mode, int MG, int sms, cudaStream_t st) {
    if (mode == XSRC_CONVERT) return dispatch_shared<FMT, XSRC_CONVERT>(p, sms, st);
    if (mode == XSRC_COPY) return dispatch_shared<FMT, XSRC_COPY>(p, sms, st);
    if (MG == 1) return launch_one<FMT, 1, XSRC_GLOBAL, 4>(p, sms, st);
    if (MG == 2) return launch_one<FMT, 2, XSRC_GLOBAL, 8>(p, sms, st);
    return launch_one<FMT, 4, XSRC_GLOBAL, 16>(p, sms, st);
}

}  // namespace

cudaError_t gemv_configure() { return cudaSuccess; }

cudaError_t launch_gemv(int fmt, const LinearArgs &a, const XqView &xq, int64_t xq_capacity_k, int sms, int *status,
                        cudaStream_t st, int *launches) {
    // TTQ_XPREP=fused converts activations inside every CTA (no second launch); default: one separate pass
    static const bool prefer_convert = []() {
        const char *v = getenv("TTQ_XPREP");
        return v && v[0] == 'f';
    }();
    GemvParams p{a, xq, 1, status};
    *launches = 0;
    const int64_t Kp = a.SBp * TILE_K;
    const bool fits = a.M <= 4 && smem_layout(fmt, 1, (int)a.M, a.SBp).total <= GEMV_SMEM_LIMIT;
    const int MG = a.M <= 4 ? 1 : (a.M <= 8 ? 2 : 4);
    const int mode = !fits ? XSRC_GLOBAL : (prefer_convert ? XSRC_CONVERT : XSRC_COPY);
    if (mode != XSRC_CONVERT) {
        if (Kp > xq_capacity_k) return cudaErrorInvalidValue;
        const int64_t Mpad = 4 * MG, units = Mpad * a.SBp;
        cudaError_t e = launch_pdl(xprep_kernel, dim3((unsigned)((units + GEMV_WARPS - 1) / GEMV_WARPS)), dim3(GEMV_THREADS),
                                   0, st, a.x, a.x_dt, a.M, Mpad, a.K, a.ldx, a.SBp, xq);
        if (e != cudaSuccess) return e;
        ++*launches;
    }
    cudaError_t e;
    if (fmt == TTQ_FMT_Q4_K) e = dispatch<TTQ_FMT_Q4_K>(p, mode, MG, sms, st);
    else if (fmt == TTQ_FMT_Q8_0) e = dispatch<TTQ_FMT_Q8_0>(p, mode, MG, sms, st);
    else e = dispatch<TTQ_FMT_Q6_K>(p, mode, MG, sms, st);
    if (e == cudaSuccess) ++*launches;
    return e;
}

}  // namespace ttq
