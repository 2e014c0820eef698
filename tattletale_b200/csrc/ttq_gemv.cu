// Decode-side kernels: y[M<=16][N] = x . W^T on the tiled quantized layout.
//
// Arithmetic: activations are converted once per call to 16-bit fixed point per 256-wide K chunk
// (xq = 256*hi + lo, both planes int8, one fp32 scale sx per chunk).  Weight quants stay integers.
// The dot product of one sub-block (32 weights for Q4_K / Q8_0, 16 for Q6_K) is an integer
// tensor-core instruction (mma.sync m16n8k32 / m16n8k16, u8|s8 x s8 -> s32) and is exact; the
// sub-block scale, the Q4_K min term and sx are applied in fp32.  One MMA covers 16 weight rows and
// 4 activation rows (8 columns = 4 x {hi, lo}).
//
// Work split: one CTA per row tile (16 rows), its 8 warps split K; each warp streams a contiguous
// run of tiles with 16-byte loads that are already A fragments, partial sums meet in shared memory.
// For M <= 2 the activation conversion is fused into the CTA prologue (each warp converts the K
// range it will consume); for larger M a separate pass writes the planes to scratch once.
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

__device__ __forceinline__ uint4 ld_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// ---- activation conversion -------------------------------------------------------------------
// Destination of one activation row's planes and side sums (shared memory or global scratch).
struct XqRow {
    int8_t *hi, *lo;  // [Kp]
    float *sum16;     // [Kp/16]
    float *sum32;     // [Kp/32]
    float *sx;        // [SBp]
};

// One warp converts the 256-wide chunk `sb` of activation row `xrow` (nullptr = emit zeros).
__device__ __forceinline__ void xprep_chunk(const void *xrow, int x_dt, int64_t K, int64_t sb, int lane,
                                            const XqRow &dst) {
    const int64_t k0 = sb * TILE_K + 8 * lane;
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
    const float inv = amax > 0.f ? (float)XQ_MAX / amax : 0.f;
    uint32_t hiw[2] = {0, 0}, low[2] = {0, 0};
    int s = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        int q = __float2int_rn(v[i] * inv);
        q = max(-XQ_MAX, min(XQ_MAX, q));
        int h = (q + 128) >> 8;
        int l = q - (h << 8);
        s += q;
        hiw[i >> 2] |= (uint32_t)(h & 0xff) << (8 * (i & 3));
        low[i >> 2] |= (uint32_t)(l & 0xff) << (8 * (i & 3));
    }
    *reinterpret_cast<uint2 *>(dst.hi + k0) = make_uint2(hiw[0], hiw[1]);
    *reinterpret_cast<uint2 *>(dst.lo + k0) = make_uint2(low[0], low[1]);
    int s16 = s + __shfl_xor_sync(0xffffffffu, s, 1);
    int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);
    if ((lane & 1) == 0) dst.sum16[sb * 16 + (lane >> 1)] = (float)s16;
    if ((lane & 3) == 0) dst.sum32[sb * 8 + (lane >> 2)] = (float)s32;
    if (lane == 0) dst.sx[sb] = amax / (float)XQ_MAX;
}

// Separate conversion pass: grid.x covers (Mpad x SBp) chunks, one warp each.
__global__ void __launch_bounds__(GEMV_THREADS) xprep_kernel(const void *__restrict__ x, int x_dt, int64_t M,
                                                             int64_t Mpad, int64_t K, int64_t ldx, int64_t SBp,
                                                             XqView xq) {
    const int lane = threadIdx.x & 31;
    const int64_t Kp = SBp * TILE_K;
    const int64_t unit = (int64_t)blockIdx.x * GEMV_WARPS + (threadIdx.x >> 5);
    if (unit >= Mpad * SBp) return;
    const int64_t m = unit / SBp, sb = unit % SBp;
    XqRow dst{xq.planes + (2 * m) * Kp, xq.planes + (2 * m + 1) * Kp, xq.sum16 + m * (Kp / 16),
              xq.sum32 + m * (Kp / 32), xq.sx + m * SBp};
    const void *xrow = nullptr;
    if (m < M) {
        const int esz = x_dt == TTQ_DT_F32 ? 4 : 2;
        xrow = reinterpret_cast<const uint8_t *>(x) + m * ldx * esz;
    }
    xprep_chunk(xrow, x_dt, K, sb, lane, dst);
}

// ---- the GEMV --------------------------------------------------------------------------------
struct GemvParams {
    LinearArgs a;
    XqView xq;  // non-fused source
};

template <int FMT>
struct TileRegs;  // one tile's worth of per-lane registers

template <>
struct TileRegs<TTQ_FMT_Q4_K> {
    uint4 q[4];
    uint4 hdr;
    __device__ __forceinline__ void load(const uint8_t *tile, int lane) {
#pragma unroll
        for (int p = 0; p < 4; p++) q[p] = ld_stream(tile + p * 512 + lane * 16);
        hdr = ld_stream(tile + 2048 + (lane & 15) * 16);
    }
};
template <>
struct TileRegs<TTQ_FMT_Q8_0> {
    uint4 q[8];
    uint4 d0, d1;  // fp16 scales of rows g and g+8, 8 blocks each
    __device__ __forceinline__ void load(const uint8_t *tile, int lane) {
#pragma unroll
        for (int b = 0; b < 8; b++) q[b] = ld_stream(tile + b * 512 + lane * 16);
        d0 = ld_stream(tile + 4096 + (lane >> 2) * 16);
        d1 = ld_stream(tile + 4096 + ((lane >> 2) + 8) * 16);
    }
};
template <>
struct TileRegs<TTQ_FMT_Q6_K> {
    uint4 ql[4];
    uint4 qh[2];
    uint4 sc;     // 16 int8 scales of row (lane & 15)
    uint32_t dw;  // fp16 d of row (lane & 15) in the low half
    __device__ __forceinline__ void load(const uint8_t *tile, int lane) {
#pragma unroll
        for (int c = 0; c < 4; c++) ql[c] = ld_stream(tile + c * 512 + lane * 16);
#pragma unroll
        for (int e = 0; e < 2; e++) qh[e] = ld_stream(tile + 2048 + e * 512 + lane * 16);
        sc = ld_stream(tile + 3072 + (lane & 15) * 16);
        dw = *reinterpret_cast<const uint16_t *>(tile + 3328 + (lane & 15) * 2);
    }
};

// Activation fragment source for one warp: column `col` = 2*m + plane.
template <bool FUSED>
struct BSource {
    const int8_t *planes;
    int64_t stride;  // bytes between columns
    int ncols;       // valid columns (FUSED only; scratch planes are zero-padded to 8 per group)
    __device__ __forceinline__ uint32_t word(int col, int64_t k) const {
        if (FUSED) {
            if (col >= ncols) return 0u;
            return *reinterpret_cast<const uint32_t *>(planes + col * stride + k);
        }
        return __ldg(reinterpret_cast<const uint32_t *>(planes + col * stride + k));
    }
};

template <int FMT, int MG, bool FUSED>
__global__ void __launch_bounds__(GEMV_THREADS, 2) gemv_kernel(GemvParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    const LinearArgs &a = p.a;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t nt = blockIdx.x;
    const int64_t SBp = a.SBp, Kp = SBp * TILE_K;
    constexpr int TB = tile_bytes(FMT);
    constexpr int MP = 4 * MG;  // padded activation rows

    // shared memory carve-up
    float2 *hdr_s = reinterpret_cast<float2 *>(smem) + warp * 128;  // per warp: [8 or 16][16] entries, 1 KB
    float *red_s = reinterpret_cast<float *>(smem + GEMV_WARPS * 1024);   // [warps][MG*2][32]
    uint8_t *dyn = smem + GEMV_WARPS * 1024 + GEMV_WARPS * MG * 2 * 32 * 4;
    // FUSED only:
    float *sx_s = reinterpret_cast<float *>(dyn);                    // [MP][SBp]
    float *sum32_s = sx_s + MP * SBp;                                // [MP][Kp/32]
    float *sum16_s = sum32_s + MP * (Kp / 32);                       // [MP][Kp/16]
    int8_t *planes_s = reinterpret_cast<int8_t *>(sum16_s + MP * (Kp / 16));  // [2M][Kp+PAD]

    const int64_t sb_begin = (warp * SBp) / GEMV_WARPS, sb_end = ((warp + 1) * SBp) / GEMV_WARPS;
    const uint8_t *tile0 = a.tiles + (nt * SBp) * TB;

    TileRegs<FMT> cur, nxt;
    if (sb_begin < sb_end) cur.load(tile0 + sb_begin * TB, lane);

    BSource<FUSED> bsrc;
    const float *sx_p, *sum32_p, *sum16_p;
    if (FUSED) {
        const int esz = a.x_dt == TTQ_DT_F32 ? 4 : 2;
        for (int m = 0; m < MP; m++) {
            XqRow dst{planes_s + (2 * m) * (Kp + PLANE_PAD), planes_s + (2 * m + 1) * (Kp + PLANE_PAD),
                      sum16_s + m * (Kp / 16), sum32_s + m * (Kp / 32), sx_s + m * SBp};
            if (m < a.M) {
                const void *xrow = reinterpret_cast<const uint8_t *>(a.x) + m * a.ldx * esz;
                for (int64_t sb = sb_begin; sb < sb_end; sb++) xprep_chunk(xrow, a.x_dt, a.K, sb, lane, dst);
            } else {
                // padded rows: only the side sums are read (the planes are predicated off)
                for (int64_t sb = sb_begin; sb < sb_end; sb++) {
                    if (lane < 16) dst.sum16[sb * 16 + lane] = 0.f;
                    if (lane < 8) dst.sum32[sb * 8 + lane] = 0.f;
                    if (lane == 0) dst.sx[sb] = 0.f;
                }
            }
        }
        __syncwarp();
        bsrc.planes = planes_s;
        bsrc.stride = Kp + PLANE_PAD;
        bsrc.ncols = 2 * (int)a.M;
        sx_p = sx_s; sum32_p = sum32_s; sum16_p = sum16_s;
    } else {
        bsrc.planes = p.xq.planes;
        bsrc.stride = Kp;
        bsrc.ncols = 2 * MP;
        sx_p = p.xq.sx; sum32_p = p.xq.sum32; sum16_p = p.xq.sum16;
    }

    float yacc[MG][2];
#pragma unroll
    for (int q = 0; q < MG; q++) yacc[q][0] = yacc[q][1] = 0.f;

    for (int64_t sb = sb_begin; sb < sb_end; sb++) {
        if (sb + 1 < sb_end) nxt.load(tile0 + (sb + 1) * TB, lane);
        float tmp[MG][2];
#pragma unroll
        for (int q = 0; q < MG; q++) tmp[q][0] = tmp[q][1] = 0.f;
        const int64_t kbase = sb * TILE_K;

        if constexpr (FMT == TTQ_FMT_Q4_K) {
            const TileRegs<TTQ_FMT_Q4_K> &T = cur;
            // header: lane -> row (lane & 15), sub-blocks 4*(lane>>4) .. +3
            {
                const __half2 dd = *reinterpret_cast<const __half2 *>(&T.hdr.x);
                const float d = __low2float(dd), dmin = __high2float(dd);
                uint32_t scw, mw;
                if (lane < 16) {
                    scw = T.hdr.y & 0x3f3f3f3fu;
                    mw = T.hdr.z & 0x3f3f3f3fu;
                } else {
                    scw = (T.hdr.w & 0x0f0f0f0fu) | ((T.hdr.y >> 2) & 0x30303030u);
                    mw = ((T.hdr.w >> 4) & 0x0f0f0f0fu) | ((T.hdr.z >> 2) & 0x30303030u);
                }
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int j = (lane >> 4) * 4 + i;
                    float dsc = d * (float)((scw >> (8 * i)) & 0xff);
                    if (i & 1) dsc *= 0.0625f;  // odd sub-blocks are fed as 16*q (high nibble in place)
                    const float dm = dmin * (float)((mw >> (8 * i)) & 0xff);
                    hdr_s[j * 16 + (lane & 15)] = make_float2(dsc, dm);
                }
                __syncwarp();
            }
#pragma unroll
            for (int pp = 0; pp < 4; pp++) {
                const uint4 w = T.q[pp];
#pragma unroll
                for (int hn = 0; hn < 2; hn++) {
                    const int j = 2 * pp + hn;
                    const uint32_t msk = hn ? 0xf0f0f0f0u : 0x0f0f0f0fu;
                    const float2 h0 = hdr_s[j * 16 + g], h1 = hdr_s[j * 16 + g + 8];
                    const int64_t k = kbase + j * 32 + 4 * t;
#pragma unroll
                    for (int q = 0; q < MG; q++) {
                        int c[4];
                        mma_k32_u8s8(c, w.x & msk, w.y & msk, w.z & msk, w.w & msk, bsrc.word(8 * q + g, k),
                                     bsrc.word(8 * q + g, k + 16));
                        const float sm = sum32_p[(4 * q + t) * (Kp / 32) + sb * 8 + j];
                        tmp[q][0] = fmaf(h0.x, (float)(c[0] * 256 + c[1]), tmp[q][0]);
                        tmp[q][0] = fmaf(-h0.y, sm, tmp[q][0]);
                        tmp[q][1] = fmaf(h1.x, (float)(c[2] * 256 + c[3]), tmp[q][1]);
                        tmp[q][1] = fmaf(-h1.y, sm, tmp[q][1]);
                    }
                }
            }
        } else if constexpr (FMT == TTQ_FMT_Q8_0) {
            const TileRegs<TTQ_FMT_Q8_0> &T = cur;
            const uint32_t d0w[4] = {T.d0.x, T.d0.y, T.d0.z, T.d0.w};
            const uint32_t d1w[4] = {T.d1.x, T.d1.y, T.d1.z, T.d1.w};
#pragma unroll
            for (int b = 0; b < 8; b++) {
                const uint4 w = T.q[b];
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&d0w[b >> 1]));
                const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&d1w[b >> 1]));
                const float dr0 = (b & 1) ? f0.y : f0.x, dr1 = (b & 1) ? f1.y : f1.x;
                const int64_t k = kbase + b * 32 + 4 * t;
#pragma unroll
                for (int q = 0; q < MG; q++) {
                    int c[4];
                    mma_k32_s8s8(c, w.x, w.y, w.z, w.w, bsrc.word(8 * q + g, k), bsrc.word(8 * q + g, k + 16));
                    tmp[q][0] = fmaf(dr0, (float)(c[0] * 256 + c[1]), tmp[q][0]);
                    tmp[q][1] = fmaf(dr1, (float)(c[2] * 256 + c[3]), tmp[q][1]);
                }
            }
        } else {
            const TileRegs<TTQ_FMT_Q6_K> &T = cur;
            // scales: lane -> row (lane & 15), sub-blocks 8*(lane>>4) .. +7; d*sc is exact in fp32
            {
                const float d = __half2float(__ushort_as_half((unsigned short)(T.dw & 0xffff)));
                const uint32_t s0 = (lane < 16) ? T.sc.x : T.sc.z, s1 = (lane < 16) ? T.sc.y : T.sc.w;
                float *hs = reinterpret_cast<float *>(hdr_s);
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int j = (lane >> 4) * 8 + i;
                    const uint32_t word = i < 4 ? s0 : s1;
                    const int sc = (int)(int8_t)((word >> (8 * (i & 3))) & 0xff);
                    hs[j * 16 + (lane & 15)] = d * (float)sc;
                }
                __syncwarp();
            }
            const float *hs = reinterpret_cast<const float *>(hdr_s);
#pragma unroll
            for (int c4 = 0; c4 < 4; c4++) {
                const uint4 w = T.ql[c4];
                const uint4 hq = T.qh[c4 >> 1];
                const uint32_t h0 = (c4 & 1) ? hq.z : hq.x, h1 = (c4 & 1) ? hq.w : hq.y;
#pragma unroll
                for (int s = 0; s < 4; s++) {
                    const int j = 4 * c4 + s;
                    const uint32_t l0 = (s & 2) ? w.z : w.x, l1 = (s & 2) ? w.w : w.y;
                    uint32_t a0, a1;
                    if (s & 1) {
                        a0 = (l0 >> 4) & 0x0f0f0f0fu;
                        a1 = (l1 >> 4) & 0x0f0f0f0fu;
                    } else {
                        a0 = l0 & 0x0f0f0f0fu;
                        a1 = l1 & 0x0f0f0f0fu;
                    }
                    // high 2 bits of sub-block s sit at bit pair s of each byte -> move to bits 4..5
                    const int sh = 4 - 2 * s;
                    a0 |= (sh >= 0 ? (h0 << sh) : (h0 >> -sh)) & 0x30303030u;
                    a1 |= (sh >= 0 ? (h1 << sh) : (h1 >> -sh)) & 0x30303030u;
                    const float ds0 = hs[j * 16 + g], ds1 = hs[j * 16 + g + 8];
                    const int64_t k = kbase + j * 16 + 4 * t;
#pragma unroll
                    for (int q = 0; q < MG; q++) {
                        int c[4];
                        mma_k16_u8s8(c, a0, a1, bsrc.word(8 * q + g, k));
                        const float off = 32.f * sum16_p[(4 * q + t) * (Kp / 16) + sb * 16 + j];
                        tmp[q][0] = fmaf(ds0, (float)(c[0] * 256 + c[1]) - off, tmp[q][0]);
                        tmp[q][1] = fmaf(ds1, (float)(c[2] * 256 + c[3]) - off, tmp[q][1]);
                    }
                }
            }
        }
#pragma unroll
        for (int q = 0; q < MG; q++) {
            const float sx = sx_p[(4 * q + t) * SBp + sb];
            yacc[q][0] = fmaf(sx, tmp[q][0], yacc[q][0]);
            yacc[q][1] = fmaf(sx, tmp[q][1], yacc[q][1]);
        }
        cur = nxt;
    }

    // cross-warp reduction in a fixed order, then bias and store
#pragma unroll
    for (int q = 0; q < MG; q++) {
        red_s[(warp * MG * 2 + q * 2 + 0) * 32 + lane] = yacc[q][0];
        red_s[(warp * MG * 2 + q * 2 + 1) * 32 + lane] = yacc[q][1];
    }
    __syncthreads();
    {
        const int row = threadIdx.x & 15, m = threadIdx.x >> 4;
        const int64_t n = nt * TILE_ROWS + row;
        if (m < a.M && m < MP && n < a.N) {
            const int q = m >> 2, src_lane = (row & 7) * 4 + (m & 3), i = row >> 3;
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < GEMV_WARPS; w++) acc += red_s[(w * MG * 2 + q * 2 + i) * 32 + src_lane];
            if (a.bias != nullptr) acc += load_as_float(a.bias, a.bias_dt, n);
            store_from_float(a.y, a.y_dt, m * a.ldy + n, acc);
        }
    }
}

size_t gemv_smem_bytes(int MG, bool fused, int64_t M, int64_t SBp) {
    size_t s = GEMV_WARPS * 1024 + (size_t)GEMV_WARPS * MG * 2 * 32 * 4;
    if (fused) {
        const int64_t Kp = SBp * TILE_K, MP = 4 * MG;
        s += (size_t)MP * SBp * 4 + (size_t)MP * (Kp / 32) * 4 + (size_t)MP * (Kp / 16) * 4;
        s += (size_t)2 * M * (Kp + PLANE_PAD);
    }
    return s;
}

constexpr size_t FUSED_SMEM_LIMIT = 100 * 1024;

template <int FMT, int MG, bool FUSED>
cudaError_t launch_one(const GemvParams &p, size_t smem, cudaStream_t st) {
    gemv_kernel<FMT, MG, FUSED><<<(unsigned)p.a.NT, GEMV_THREADS, smem, st>>>(p);
    return cudaGetLastError();
}

template <int FMT>
cudaError_t dispatch(const GemvParams &p, int MG, bool fused, size_t smem, cudaStream_t st) {
    if (fused) return launch_one<FMT, 1, true>(p, smem, st);
    if (MG == 1) return launch_one<FMT, 1, false>(p, smem, st);
    if (MG == 2) return launch_one<FMT, 2, false>(p, smem, st);
    return launch_one<FMT, 4, false>(p, smem, st);
}

template <int FMT>
cudaError_t configure_fmt() {
    cudaError_t e = cudaFuncSetAttribute(gemv_kernel<FMT, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)FUSED_SMEM_LIMIT);
    return e;
}

}  // namespace

cudaError_t gemv_configure() {
    cudaError_t e;
    if ((e = configure_fmt<TTQ_FMT_Q8_0>()) != cudaSuccess) return e;
    if ((e = configure_fmt<TTQ_FMT_Q4_K>()) != cudaSuccess) return e;
    return configure_fmt<TTQ_FMT_Q6_K>();
}

cudaError_t launch_gemv(int fmt, const LinearArgs &a, const XqView &xq, int64_t xq_capacity_k, cudaStream_t st,
                        int *launches) {
    GemvParams p{a, xq};
    const int MG = a.M <= 4 ? 1 : (a.M <= 8 ? 2 : 4);
    const size_t fused_smem = gemv_smem_bytes(1, true, a.M, a.SBp);
    const bool fused = a.M <= 2 && fused_smem <= FUSED_SMEM_LIMIT;
    *launches = 0;
    if (!fused) {
        const int64_t Kp = a.SBp * TILE_K;
        if (Kp > xq_capacity_k) return cudaErrorInvalidValue;
        const int64_t Mpad = 4 * MG, units = Mpad * a.SBp;
        xprep_kernel<<<(unsigned)((units + GEMV_WARPS - 1) / GEMV_WARPS), GEMV_THREADS, 0, st>>>(
            a.x, a.x_dt, a.M, Mpad, a.K, a.ldx, a.SBp, xq);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        ++*launches;
    }
    const size_t smem = fused ? fused_smem : gemv_smem_bytes(MG, false, a.M, a.SBp);
    cudaError_t e;
    if (fmt == TTQ_FMT_Q4_K) e = dispatch<TTQ_FMT_Q4_K>(p, MG, fused, smem, st);
    else if (fmt == TTQ_FMT_Q8_0) e = dispatch<TTQ_FMT_Q8_0>(p, MG, fused, smem, st);
    else e = dispatch<TTQ_FMT_Q6_K>(p, MG, fused, smem, st);
    if (e == cudaSuccess) ++*launches;
    return e;
}

}  // namespace ttq
