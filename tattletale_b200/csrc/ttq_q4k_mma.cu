// Decode linear for Q4_K, 3 to 16 activation rows, in ONE kernel per call: the activation conversion runs in every
// CTA's prologue (no separate pass) and the multiply uses fp16 tensor-core instructions on exact integer operands.
//
// Arithmetic.  A 4-bit quant q of sub-block j is expanded in registers to the fp16 integer q * sc_j (sc_j = the
// 6-bit sub-block scale; q * sc_j <= 945 is exact in fp16): the nibble is OR-ed into the mantissa of 1024 and ONE
// fused multiply-add per pair of weights, (1024 + q) * sc - 1024 * sc, removes the offset exactly.  With the
// sub-block scale inside the operand one mma.sync.m16n8k16 (f16 x f16 -> f32) may mix sub-blocks freely: 16
// instructions per tile (16 weight rows x 256 weights) serve 8 activation rows, the super-block scale d is applied
// once per tile in fp32, and the min term -dmin * sum_j m_j * (sum of the activations of sub-block j) is one more
// instruction whose A operand holds the 6-bit mins and whose B operand the sub-block sums split into fp16 high
// and low parts.  Products are exact in fp32; the only rounding is the fp32 accumulation (relative L2 error
// against the fp64 checker ~3e-7).  bf16 -> fp16 is exact inside the fp16 range; a row whose largest magnitude
// falls outside [2^-8, 1024] is rescaled by a power of two (undone in the epilogue), so no input range loses
// precision.  The gated form computes silu(gate) * up in the conversion.
//
// Cost.  The legacy tensor-core path executes one mma.sync in about 45 cycles per SM sub-partition on this part,
// so the 17 instructions of a tile bound the kernel near 190 cycles per tile and SM (about half of the HBM rate)
// for any batch of up to 8 rows; the integer kernel of ttq_gemv.cu needs 8 instructions per tile and ROW and is
// the faster one up to 2 rows.
//
// Work split.  One persistent CTA per SM.  A CTA owns a contiguous run of row tiles and a slice of K
// (gridDim.y slices; the converted activations of that slice stay in shared memory).  Its tiles (2304 packed
// bytes each), taken in (row tile, K tile) order, are cut into NW equal contiguous runs, one per warp, whatever
// the matrix shape: a warp's run may start and end in the middle of a row tile.  Every warp streams its run
// through a private ring of bulk async copies (first stages issued before the dependency wait, so they overlap
// the preceding kernel's tail) and never waits for another warp: when it leaves a row tile it parks its partial
// sums in its own shared-memory slot and bumps that row tile's arrival counter; the warp that arrives last adds
// the pieces in run order and writes the outputs.  With several K slices the same protocol runs once more
// between CTAs through an fp32 workspace and global counters.  No barrier after the prologue, no spin anywhere
// except the bounded waits on the copy ring (and on peers in the tensor-parallel exchange).
#include "ttq_devutil.cuh"

namespace ttq {

namespace {

constexpr int QM_TB = 2304;  // bytes of one Q4_K tile
constexpr int QM_ZERO_BYTES = 512;
constexpr int QM_MAX_M = 16;
constexpr int QM_MAX_ROW_TILES = 128;  // row tiles one CTA may own (shared-memory arrival counters)
constexpr size_t QM_SMEM_MAX = 227 * 1024;

struct QmParams {
    LinearArgs a;
    float *ws;           // gridDim.y > 1: partial sums [slice][M][N]
    unsigned *counters;  // gridDim.y > 1: arrivals per row tile (zero between launches)
    int *status;         // device word: bit 0 a bounded copy wait gave up, bit 2 a bounded peer wait gave up
    unsigned long long *trace;
    int trace_all;       // every CTA records a timeline entry (kind 5), not only the first
    CommView comm;       // row-parallel exchange over peer memory (world <= 1: none)
};

// Shared-memory carve-up, identical on host (size) and device (offsets).  `act_bytes` = the back end's
// activation area for the CTA's K slice.
struct QmLayout {
    uint32_t bars, zero, misc, cnt, hdr, piece, ring, act, total;
};
__host__ __device__ inline QmLayout qm_layout(int nw, int stages, int hdr_bytes, int piece_bytes, uint32_t act_bytes) {
    QmLayout L;
    uint32_t o = 0;
    L.bars = o; o += nw * stages * 8;
    o = (o + 127u) & ~127u;
    L.zero = o; o += QM_ZERO_BYTES;
    L.misc = o; o += 256;                          // [16] output multipliers, [24] reduction scratch, flag word, [16] input multipliers
    L.cnt = o; o += QM_MAX_ROW_TILES * 4;          // arrivals per row tile of this CTA
    L.hdr = o; o += nw * hdr_bytes;                // per warp: unpacked sub-block scales of the current tile
    L.piece = o; o += nw * 3 * piece_bytes;        // per warp: partial sums of its first, last and current whole row tile
    L.ring = o; o += nw * stages * QM_TB;
    L.act = o; o += act_bytes;
    L.total = o;
    return L;
}

// ---- activation loads shared by both back ends -----------------------------------------------------------
// Eight consecutive 16-bit values of a row, loaded early so that several loads are in flight.
struct QmRaw {
    uint4 a, b;  // b: the `up` half of the gated form
};
__device__ __forceinline__ uint4 qm_load8(const uint16_t *p) {
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) return *reinterpret_cast<const uint4 *>(p);
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) w[i] = (uint32_t)p[2 * i] | ((uint32_t)p[2 * i + 1] << 16);
    return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void qm_unpack8(const uint4 &r, int x_dt, float (&v)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        if (x_dt == TTQ_DT_BF16) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        } else {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
}
__device__ __forceinline__ void qm_values(const QmRaw &r, int x_dt, bool gated, float (&v)[8]) {
    qm_unpack8(r.a, x_dt, v);
    if (gated) {
        // silu(gate) * up: the gated-MLP activation (kernels/activations.nim:14-38) folded into the conversion
        float u[8];
        qm_unpack8(r.b, x_dt, u);
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = v[i] / (1.f + expf(-v[i])) * u[i];
    }
}

// Visits the 8-value units of the rows in `rowmask` that belong to this thread, BATCH loads in flight.  A warp's
// 32 units are one 256-wide chunk of one row (a row has a multiple of 32 units), so `f` runs warp-converged.
template <int THREADS, int BATCH, bool GATED, class F>
__device__ __forceinline__ void qm_for_units_t(const LinearArgs &a, int M, int64_t k_begin, int units_per_row, uint32_t rowmask, F &&f) {
    const int total = M * units_per_row;
    const uint16_t *x = reinterpret_cast<const uint16_t *>(a.x);
    for (int u0 = threadIdx.x; u0 < total; u0 += BATCH * THREADS) {
        QmRaw raw[BATCH];
        int mm[BATCH], kk[BATCH];
#pragma unroll
        for (int i = 0; i < BATCH; i++) {
            const int u = u0 + i * THREADS;
            mm[i] = -1;
            if (u < total) {
                const int m = u / units_per_row, k8 = u - m * units_per_row;
                if ((rowmask >> m) & 1u) {
                    mm[i] = m;
                    kk[i] = k8;
                    const uint16_t *src = x + (int64_t)m * a.ldx + k_begin + 8 * k8;
                    raw[i].a = qm_load8(src);
                    if (GATED) raw[i].b = qm_load8(src + a.K);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < BATCH; i++)
            if (mm[i] >= 0) f(raw[i], mm[i], kk[i]);
    }
}
template <int THREADS, class F>
__device__ __forceinline__ void qm_for_units(const LinearArgs &a, int M, int64_t k_begin, int units_per_row, uint32_t rowmask, F &&f) {
    if (a.gated) qm_for_units_t<THREADS, 3, true>(a, M, k_begin, units_per_row, rowmask, f);
    else qm_for_units_t<THREADS, 6, false>(a, M, k_begin, units_per_row, rowmask, f);
}

// ===========================================================================================================
// F16 back end: fp16 tensor-core products of exact integer operands (M <= 16)
// ===========================================================================================================
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hmul2_u(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hadd2_u(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
constexpr uint32_t H2_1024 = 0x64006400u, H2_M1024 = 0xE400E400u, H2_16TH = 0x2C002C00u, H2_M64 = 0xD400D400u;

// Expands one packed register (4 bytes = positions P..P+3 of a sub-block pair for one row) into the four
// fp16x2 operands {lo nibbles of bytes 0,2 | lo of 1,3 | hi of 0,2 | hi of 1,3}, each = q * sc exactly.
__device__ __forceinline__ void qm_expand(uint32_t w, uint32_t s_lo, uint32_t o_lo, uint32_t s_hi, uint32_t o_hi, uint32_t &l02, uint32_t &l13,
                                          uint32_t &h02, uint32_t &h13, uint32_t mask_lo, uint32_t mask_hi, uint32_t k1024) {
    const uint32_t w8 = w >> 8;
    l02 = hfma2_u(and_or(w, mask_lo, k1024), s_lo, o_lo);
    h02 = hfma2_u(and_or(w, mask_hi, k1024), s_hi, o_hi);
    l13 = hfma2_u(and_or(w8, mask_lo, k1024), s_lo, o_lo);
    h13 = hfma2_u(and_or(w8, mask_hi, k1024), s_hi, o_hi);
}

template <int NCG, int NW_>
struct F16Backend {
    static constexpr int NW = NW_;
    static constexpr int THREADS = NW * 32;
    static constexpr int MIN_CTAS = 1;
    static constexpr int HDR_BYTES = 1280;           // per warp: scale operands [16][8] f16x2, min operands [16][8] f16x2, {d, dmin} [16] f32x2
    static constexpr int PIECE_BYTES = NCG * 512;    // [NCG][16 rows][8 columns] f32

    // activation area: per row the sub-block sums ({hi, lo} f16 pairs) and the fp16 values (+16: bank spread)
    __host__ __device__ static uint32_t srow(int nsb) { return (((uint32_t)nsb * 32 + 127u) & ~127u) + 16; }
    __host__ __device__ static uint32_t xrow(int nsb) { return (uint32_t)nsb * 512 + 16; }
    __host__ __device__ static uint32_t act_bytes(int M, int nsb) { return (uint32_t)M * (srow(nsb) + xrow(nsb)); }
    struct Lane {
        uint32_t bx[NCG], bs[NCG], mul[NCG];  // B-operand addresses of this lane's activation row per column group
    };
    struct Acc {
        float v[NCG][4];
        __device__ __forceinline__ void clear() {
#pragma unroll
            for (int cg = 0; cg < NCG; cg++)
#pragma unroll
                for (int i = 0; i < 4; i++) v[cg][i] = 0.f;
        }
    };

    // Converts the rows in `rowmask` (multiplied by xmul[m]) into shared memory, values in the order the weight
    // registers deliver them (each four k as 0 2 1 3).  Returns per-row range flags of the values seen by this
    // thread: bit m = a value of normal size (>= 2^-8), bit 16 + m = a value above 1024.
    __device__ static uint32_t convert(const LinearArgs &a, int M, int64_t k_begin, int nsb, uint32_t rowmask, const float *xmul, uint32_t ss,
                                       uint32_t xs) {
        uint32_t flags = 0;
        const int lane = threadIdx.x & 31;
        const uint32_t sr = srow(nsb), xr = xrow(nsb);
        qm_for_units<THREADS>(a, M, k_begin, nsb * 32, rowmask, [&](const QmRaw &raw, int m, int k8) {
            float v[8];
            qm_values(raw, a.x_dt, a.gated, v);
            const float mul = xmul[m];
            float vmax = 0.f, sum = 0.f;
            uint32_t hb[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float s = v[i] * mul;
                vmax = fmaxf(vmax, fabsf(s));
                const __half hv = __float2half_rn(s);
                hb[i] = (uint32_t)__half_as_ushort(hv);
                sum += __half2float(hv);
            }
            if (!(vmax <= 1024.f)) flags |= 1u << (16 + m);  // also NaN
            if (vmax >= 0.00390625f) flags |= 1u << m;
            sts128<0>(xs + (uint32_t)m * xr + (uint32_t)k8 * 16, hb[0] | (hb[2] << 16), hb[1] | (hb[3] << 16), hb[4] | (hb[6] << 16),
                      hb[5] | (hb[7] << 16));
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if ((lane & 3) == 0) {
                const __half hi = __float2half_rn(sum);
                const __half lo = __float2half_rn(sum - __half2float(hi));
                const uint32_t w = (uint32_t)__half_as_ushort(hi) | ((uint32_t)__half_as_ushort(lo) << 16);
                asm volatile("st.shared.u32 [%0], %1;" ::"r"(ss + (uint32_t)m * sr + (uint32_t)(k8 >> 2) * 4), "r"(w) : "memory");
            }
        });
        return flags;
    }

    // misc: [0..15] output multipliers (1 at entry), [16..39] scratch, [40] flag word (0 at entry), [48..63] input multipliers
    __device__ static void prologue(const LinearArgs &a, int M, int64_t k_begin, int nsb, uint8_t *smem, uint32_t act_off, float *misc) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const uint32_t ss = smem_u32(smem) + act_off, xs = ss + (uint32_t)M * srow(nsb);
        const uint32_t all_rows = (1u << M) - 1u;
        uint32_t flags = convert(a, M, k_begin, nsb, all_rows, misc, ss, xs);
        // bitwise OR of the range flags over the CTA (the barrier's own OR is a logical one)
        uint32_t *flag_word = reinterpret_cast<uint32_t *>(misc + 40);
        flags = __reduce_or_sync(0xffffffffu, flags);
        if (lane == 0 && flags != 0) atomicOr(flag_word, flags);
        __syncthreads();
        const uint32_t seen = *flag_word;
        const uint32_t slow = (~seen | (seen >> 16)) & all_rows;
        if (slow == 0) return;
        // rows outside the comfortable fp16 range: bring the largest magnitude into [512, 1024) with a power of two
        float *scratch = misc + 16, *xmul = misc + 48;
        for (int m = 0; m < M; m++) {
            if (!((slow >> m) & 1u)) continue;
            float amax = 0.f;
            qm_for_units<THREADS>(a, M, k_begin, nsb * 32, 1u << m, [&](const QmRaw &raw, int, int) {
                float v[8];
                qm_values(raw, a.x_dt, a.gated, v);
#pragma unroll
                for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
            });
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            if (lane == 0) scratch[warp] = amax;
            __syncthreads();
            if (threadIdx.x == 0) {
                float am = 0.f;
                for (int w = 0; w < NW; w++) am = fmaxf(am, scratch[w]);
                float mul = 1.f, inv = 1.f;
                if (am > 0.f && am < 3.0e38f) {
                    const int e = ilogbf(am);
                    mul = ldexpf(1.f, 9 - e);
                    inv = ldexpf(1.f, e - 9);
                }
                xmul[m] = mul;
                misc[m] = inv;
            }
            __syncthreads();
        }
        convert(a, M, k_begin, nsb, slow, xmul, ss, xs);
        __syncthreads();
    }

    __device__ static Lane lane_view(uint32_t smem0, const QmLayout &L, int M, int nsb, int lane) {
        const int g = lane >> 2, t = lane & 3;
        const uint32_t ss = smem0 + L.act, xs = ss + (uint32_t)M * srow(nsb);
        Lane A;
#pragma unroll
        for (int cg = 0; cg < NCG; cg++) {
            const int mrow = cg * 8 + g;
            const bool valid = mrow < M;
            A.mul[cg] = valid ? 1u : 0u;
            A.bx[cg] = valid ? xs + (uint32_t)mrow * xrow(nsb) + (uint32_t)(t >> 1) * 128 + (uint32_t)(t & 1) * 8 : smem0 + L.zero;
            A.bs[cg] = valid ? ss + (uint32_t)mrow * srow(nsb) + (uint32_t)t * 4 : smem0 + L.zero;
        }
        return A;
    }

    // Shared-memory loads are volatile and stay in program order: everything a chunk of MMAs needs is requested one
    // chunk ahead of its use, so that the load latencies hide behind the expansion and the MMAs of the chunk before.
    __device__ __forceinline__ static void tile(uint32_t stage, int sbl, int lane, uint32_t hdr, const Lane &A, Acc &acc) {
        const int g = lane >> 2, t = lane & 3;
        const int r = lane & 15, h = lane >> 4;
        const uint32_t sa = stage + (uint32_t)lane * 16;
        uint32_t xo[NCG], so[NCG];
#pragma unroll
        for (int cg = 0; cg < NCG; cg++) {
            xo[cg] = A.bx[cg] + A.mul[cg] * (uint32_t)sbl * 512u;
            so[cg] = A.bs[cg] + A.mul[cg] * (uint32_t)sbl * 32u;
        }
        // ---- loads that depend on nothing: the row header, the operands of chunk 0, the sub-block sums
        const uint4 hv = lds128<2048>(stage + (uint32_t)r * 16);
        uint4 wq[2];
        uint2 bq[2][NCG][4];  // [buffer][column group][MMA of the chunk: sub-blocks 2p0, 2p0+1, 2p0+4, 2p0+5]
        auto load_chunk = [&](auto n_, uint4 &w, uint2 (&b)[NCG][4]) {
            constexpr int n = decltype(n_)::value;
            w = lds128<n * 512>(sa);
#pragma unroll
            for (int cg = 0; cg < NCG; cg++) {
                b[cg][0] = lds64<n * 16>(xo[cg]);
                b[cg][1] = lds64<64 + n * 16>(xo[cg]);
                b[cg][2] = lds64<256 + n * 16>(xo[cg]);
                b[cg][3] = lds64<320 + n * 16>(xo[cg]);
            }
        };
        load_chunk(IC<0>{}, wq[0], bq[0]);
        uint32_t sum_lo[NCG], sum_hi[NCG];
#pragma unroll
        for (int cg = 0; cg < NCG; cg++) {
            sum_lo[cg] = lds32<0>(so[cg]);
            sum_hi[cg] = lds32<16>(so[cg]);
        }
        // ---- header role: lane (r, h) unpacks sub-blocks 4h..4h+3 of row r
        {
            uint32_t scw, mw;
            if (h == 0) {
                scw = hv.y & 0x3f3f3f3fu;
                mw = hv.z & 0x3f3f3f3fu;
            } else {
                scw = (hv.w & 0x0f0f0f0fu) | ((hv.y >> 2) & 0x30303030u);
                mw = ((hv.w >> 4) & 0x0f0f0f0fu) | ((hv.z >> 2) & 0x30303030u);
            }
            // bytes 0, 2 = even sub-blocks (low nibbles: operand scale sc), bytes 1, 3 = odd ones (high nibbles, fed as
            // 16 q: operand scale sc / 16)
            const uint32_t s_ev = hadd2_u((scw & 0x00ff00ffu) | H2_1024, H2_M1024);
            const uint32_t s_od = hfma2_u(((scw >> 8) & 0x00ff00ffu) | H2_1024, H2_16TH, H2_M64);
            const uint32_t m_ev = hadd2_u((mw & 0x00ff00ffu) | H2_1024, H2_M1024);
            const uint32_t m_od = hadd2_u(((mw >> 8) & 0x00ff00ffu) | H2_1024, H2_M1024);
            __syncwarp();  // main-role reads of the previous tile's header are done
            const uint32_t hw = hdr + (uint32_t)r * 32 + (uint32_t)h * 16;
            sts128<0>(hw, __byte_perm(s_ev, 0, 0x1010), __byte_perm(s_od, 0, 0x1010), __byte_perm(s_ev, 0, 0x3232), __byte_perm(s_od, 0, 0x3232));
            sts128<512>(hw, __byte_perm(m_ev, 0, 0x1010), __byte_perm(m_od, 0, 0x1010), __byte_perm(m_ev, 0, 0x3232), __byte_perm(m_od, 0, 0x3232));
            if (h == 0) {
                const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&hv.x));
                sts64f<1024>(hdr + (uint32_t)r * 8, dd.x, dd.y);
            }
            __syncwarp();
        }
        // ---- main role: lane (g, t) holds rows g, g+8 and the sub-block pairs p0 = t>>1 and p0 + 2
        const uint32_t hs = hdr + (uint32_t)g * 32 + (uint32_t)(t >> 1) * 8;
        const uint32_t hm = hdr + 512 + (uint32_t)g * 32 + (uint32_t)t * 4;
        uint32_t sc[2][4], of[2][4];  // [row g | g+8][pair p0 low, p0 high, p0+2 low, p0+2 high]
        const uint2 a0 = lds64<0>(hs), a1 = lds64<16>(hs), b0 = lds64<256>(hs), b1 = lds64<256 + 16>(hs);
        // the min term's operands: mins of sub-blocks t and t+4 (each twice: high and low part of the sum), {d, dmin}
        const uint32_t m0 = lds32<0>(hm), m1 = lds32<256>(hm), m2 = lds32<16>(hm), m3 = lds32<256 + 16>(hm);
        const float2 dg = lds64f<1024>(hdr + (uint32_t)g * 8), dh = lds64f<1024 + 64>(hdr + (uint32_t)g * 8);
        sc[0][0] = a0.x; sc[0][1] = a0.y; sc[0][2] = a1.x; sc[0][3] = a1.y;
        sc[1][0] = b0.x; sc[1][1] = b0.y; sc[1][2] = b1.x; sc[1][3] = b1.y;
#pragma unroll
        for (int i = 0; i < 2; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) of[i][j] = hmul2_u(sc[i][j], H2_M1024);  // -1024 sc, resp. -64 sc for the /16 operand
        // two accumulator sets per column group (low-nibble and high-nibble sub-blocks): shorter dependent chains
        float c[NCG][2][4];
#pragma unroll
        for (int cg = 0; cg < NCG; cg++)
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int i = 0; i < 4; i++) c[cg][j][i] = 0.f;
        // the three constants of the nibble expansion live in registers (opaque to the compiler's immediate folding)
        uint32_t mask_lo = 0x000f000fu, mask_hi = 0x00f000f0u, k1024 = H2_1024;
        asm volatile("" : "+r"(mask_lo), "+r"(mask_hi), "+r"(k1024));
        static_for<0, 4>([&](auto n_) {
            constexpr int n = decltype(n_)::value;
            if constexpr (n < 3) load_chunk(IC<n + 1>{}, wq[(n + 1) & 1], bq[(n + 1) & 1]);
            const uint4 w = wq[n & 1];
            uint32_t l02g, l13g, h02g, h13g, l02h, l13h, h02h, h13h;
            qm_expand(w.x, sc[0][0], of[0][0], sc[0][1], of[0][1], l02g, l13g, h02g, h13g, mask_lo, mask_hi, k1024);
            qm_expand(w.y, sc[1][0], of[1][0], sc[1][1], of[1][1], l02h, l13h, h02h, h13h, mask_lo, mask_hi, k1024);
#pragma unroll
            for (int cg = 0; cg < NCG; cg++) {
                mma_f16(c[cg][0], l02g, l02h, l13g, l13h, bq[n & 1][cg][0].x, bq[n & 1][cg][0].y);
                mma_f16(c[cg][1], h02g, h02h, h13g, h13h, bq[n & 1][cg][1].x, bq[n & 1][cg][1].y);
            }
            qm_expand(w.z, sc[0][2], of[0][2], sc[0][3], of[0][3], l02g, l13g, h02g, h13g, mask_lo, mask_hi, k1024);
            qm_expand(w.w, sc[1][2], of[1][2], sc[1][3], of[1][3], l02h, l13h, h02h, h13h, mask_lo, mask_hi, k1024);
#pragma unroll
            for (int cg = 0; cg < NCG; cg++) {
                mma_f16(c[cg][0], l02g, l02h, l13g, l13h, bq[n & 1][cg][2].x, bq[n & 1][cg][2].y);
                mma_f16(c[cg][1], h02g, h02h, h13g, h13h, bq[n & 1][cg][3].x, bq[n & 1][cg][3].y);
            }
        });
        // ---- the min term and the super-block scale
#pragma unroll
        for (int cg = 0; cg < NCG; cg++) {
            float cm[4] = {0.f, 0.f, 0.f, 0.f};
            mma_f16(cm, m0, m1, m2, m3, sum_lo[cg], sum_hi[cg]);
            acc.v[cg][0] = fmaf(dg.x, c[cg][0][0] + c[cg][1][0], fmaf(-dg.y, cm[0], acc.v[cg][0]));
            acc.v[cg][1] = fmaf(dg.x, c[cg][0][1] + c[cg][1][1], fmaf(-dg.y, cm[1], acc.v[cg][1]));
            acc.v[cg][2] = fmaf(dh.x, c[cg][0][2] + c[cg][1][2], fmaf(-dh.y, cm[2], acc.v[cg][2]));
            acc.v[cg][3] = fmaf(dh.x, c[cg][0][3] + c[cg][1][3], fmaf(-dh.y, cm[3], acc.v[cg][3]));
        }
    }

    // piece layout: [column group][row][column] f32
    __device__ __forceinline__ static void store_piece(const Acc &acc, float *slot, int lane) {
        const int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int cg = 0; cg < NCG; cg++) {
            *reinterpret_cast<float2 *>(slot + cg * 128 + g * 8 + 2 * t) = make_float2(acc.v[cg][0], acc.v[cg][1]);
            *reinterpret_cast<float2 *>(slot + cg * 128 + (g + 8) * 8 + 2 * t) = make_float2(acc.v[cg][2], acc.v[cg][3]);
        }
    }
    __device__ __forceinline__ static float piece_value(const float *slot, int mm, int row) {
        return slot[(mm >> 3) * 128 + row * 8 + (mm & 7)];
    }
};

// ===========================================================================================================
// the skeleton
// ===========================================================================================================
template <class B, int STAGES>
__global__ void __launch_bounds__(B::THREADS, B::MIN_CTAS) q4k_decode_kernel(QmParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int NW = B::NW;
    const LinearArgs &a = p.a;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int SBp = (int)a.SBp, M = (int)a.M;
    // K slice of this CTA (in tiles) and its run of row tiles
    const int ksp = (int)gridDim.y, ky = (int)blockIdx.y;
    const int csb0 = (ky * SBp) / ksp, cnsb = ((ky + 1) * SBp) / ksp - csb0;
    const int nsb_max = (SBp + ksp - 1) / ksp;
    const int64_t rt_b = ((int64_t)blockIdx.x * a.NT) / gridDim.x;
    const int nrt = (int)((((int64_t)blockIdx.x + 1) * a.NT) / gridDim.x - rt_b);
    const QmLayout L = qm_layout(NW, STAGES, B::HDR_BYTES, B::PIECE_BYTES, B::act_bytes(M, nsb_max));
    const uint32_t smem0 = smem_u32(smem);
    const uint32_t hdr_u32 = smem0 + L.hdr + warp * B::HDR_BYTES;
    const uint32_t ring_u32 = smem0 + L.ring + warp * STAGES * QM_TB;
    const uint32_t bar_u32 = smem0 + L.bars + warp * STAGES * 8;
    float *misc = reinterpret_cast<float *>(smem + L.misc);
    unsigned *cnt_s = reinterpret_cast<unsigned *>(smem + L.cnt);
    float *pieces = reinterpret_cast<float *>(smem + L.piece);
    constexpr int PF = B::PIECE_BYTES / 4;  // floats per piece

    // this warp's run of the CTA's tiles, which are numbered (row tile, K tile) row-tile-major
    const int Tc = nrt * cnsb;
    // (32-bit arithmetic: Tc <= 128 row tiles x 256 K tiles, times NW <= 24, stays below 2^31; 64-bit division is slow)
    auto run_start = [&](int w) { return (int)((unsigned)(w * Tc) / (unsigned)NW); };
    auto warp_of = [&](int tile) { return (int)((unsigned)((tile + 1) * NW - 1) / (unsigned)Tc); };  // the warp whose run holds `tile`
    const int t_begin = run_start(warp), n_items = run_start(warp + 1) - t_begin;

    unsigned long long *te = trace_open(p.trace, 2);
    if (p.trace_all && p.trace != nullptr && threadIdx.x == 0 && !(blockIdx.x == 0 && blockIdx.y == 0)) {
        const unsigned long long slot = atomicAdd(p.trace, 1ull);
        if (slot < TRACE_CAP) {
            te = p.trace + 8 + slot * 8;
            te[0] = 5;
            te[1] = global_ns();
        }
    }
    grid_launch_dependents();

    // ---- ring set-up and first copies (weights do not depend on the preceding kernel)
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) mbar_init(bar_u32 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_shared();
    }
    if (threadIdx.x < QM_ZERO_BYTES / 4) reinterpret_cast<uint32_t *>(smem + L.zero)[threadIdx.x] = 0u;
    if (threadIdx.x < 64) misc[threadIdx.x] = threadIdx.x < QM_MAX_M ? 1.f : 0.f;
    if (threadIdx.x >= 64 && threadIdx.x < 64 + QM_MAX_ROW_TILES) cnt_s[threadIdx.x - 64] = 0u;
    __syncwarp();
    int p_item = 0, p_sb = t_begin % (cnsb > 0 ? cnsb : 1);
    const uint8_t *p_ptr = a.tiles + ((rt_b + t_begin / (cnsb > 0 ? cnsb : 1)) * SBp + csb0 + p_sb) * (int64_t)QM_TB;
    auto issue_next = [&]() {
        const int s = p_item % STAGES;
        mbar_expect_tx(bar_u32 + 8 * s, QM_TB);
        bulk_g2s(ring_u32 + s * QM_TB, p_ptr, QM_TB, bar_u32 + 8 * s);
        p_item++;
        p_ptr += QM_TB;
        if (++p_sb == cnsb) {  // next row tile: skip the K tiles of other slices
            p_sb = 0;
            p_ptr += (int64_t)(SBp - cnsb) * QM_TB;
        }
    };
    // The activation rows are pulled into L2 before anything else is requested (a hint: L2 is the coherence point,
    // so lines the preceding kernel has yet to write are still read correctly after the dependency wait); when the
    // rows are cold this takes their DRAM latency off the path behind the wait.
    if (threadIdx.x < M) {
        const uint8_t *row = reinterpret_cast<const uint8_t *>(a.x) + ((size_t)threadIdx.x * a.ldx + (size_t)csb0 * TILE_K) * 2;
        const uint32_t bytes = (uint32_t)cnsb * TILE_K * 2;
        if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(row), "r"(bytes) : "memory");
            if (a.gated) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(row + (size_t)a.K * 2), "r"(bytes) : "memory");
        }
    }
    if (lane == 0) {
        for (int i = 0; i < STAGES && i < n_items; i++) issue_next();
    }

    // ---- activations: everything below may depend on the preceding kernel
    grid_dependency_wait();
    if (te) te[2] = global_ns();
    __syncthreads();  // multipliers, counters and the zero region are written
    B::prologue(a, M, (int64_t)csb0 * TILE_K, cnsb, smem, L.act, misc);
    const typename B::Lane A = B::lane_view(smem0, L, M, cnsb, lane);
    if (te) te[3] = global_ns();

    // ---- main loop over this warp's run
    bool alive = true;  // false once a bounded wait gave up: skip further waits, keep going
    int j = cnsb > 0 ? t_begin / cnsb : 0, sb = cnsb > 0 ? t_begin % cnsb : 0;  // local row tile, K tile inside the slice
    const int j_first = j;
    typename B::Acc acc;
    acc.clear();
    for (int item = 0; item < n_items; item++) {
        const int s = item % STAGES;
        if (alive) alive = mbar_wait_bounded(bar_u32 + 8 * s, (uint32_t)((item / STAGES) & 1), p.status);
        if (te && item == 0) te[4] = global_ns();
        B::tile(ring_u32 + s * QM_TB, sb, lane, hdr_u32, A, acc);
        __syncwarp();  // every lane is done reading the stage before it is refilled
        if (lane == 0 && alive && p_item < n_items) {
            fence_async_shared();
            issue_next();
        }
        if (sb == cnsb - 1 || item == n_items - 1) {
            // ---- leaving row tile j: park the partial sums, count the arrival, the last piece finishes the row tile
            const int w_first = warp_of(j * cnsb), w_last = warp_of(j * cnsb + cnsb - 1);
            // bit w - w_first of piece_mask: warp w holds a piece (warps with an empty run, fewer tiles than warps, do
            // not); same bit of head_mask: that piece sits in the warp's slot 0 (the row tile its run starts in)
            uint32_t piece_mask = 0, head_mask = 0;
            for (int w = w_first; w <= w_last; w++) {
                const int rs = run_start(w);
                if (run_start(w + 1) > rs) piece_mask |= 1u << (w - w_first);
                if (rs >= j * cnsb) head_mask |= 1u << (w - w_first);
            }
            const int n_pieces = __popc(piece_mask);
            const int slot = n_pieces == 1 ? 2 : (j == j_first ? 0 : 1);
            float *mine = pieces + (size_t)(warp * 3 + slot) * PF;
            B::store_piece(acc, mine, lane);
            acc.clear();
            bool last = true;
            if (n_pieces > 1) {
                __threadfence_block();
                __syncwarp();
                unsigned old = 0;
                if (lane == 0) old = atomicAdd(cnt_s + j, 1u);
                old = __shfl_sync(0xffffffffu, old, 0);
                last = old == (unsigned)(n_pieces - 1);
                if (last) __threadfence_block();
            } else {
                __syncwarp();
            }
            if (last) {
                const int64_t rt = rt_b + j;
                const int outs = M * TILE_ROWS;
                // value of output o = m * 16 + row: the pieces of the row tile in run order, rescaled
                auto local_sum = [&](int o) {
                    const int row = o & 15, mm = o >> 4;
                    float v = 0.f;
                    for (int w = w_first; w <= w_last; w++) {
                        if (!((piece_mask >> (w - w_first)) & 1u)) continue;
                        const int sl = n_pieces == 1 ? 2 : (((head_mask >> (w - w_first)) & 1u) ? 0 : 1);
                        v += B::piece_value(pieces + (size_t)(w * 3 + sl) * PF, mm, row);
                    }
                    return v * misc[mm];
                };
                bool final_stage = true;
                if (ksp > 1) {
                    // several K slices: park the CTA's sums, count the arrival; the last CTA to arrive adds them up
                    for (int o = lane; o < outs; o += 32) {
                        const int row = o & 15, mm = o >> 4;
                        const int64_t n = rt * TILE_ROWS + row;
                        if (n < a.N) __stcg(p.ws + ((size_t)ky * M + mm) * a.N + n, local_sum(o));
                    }
                    __threadfence();
                    __syncwarp();
                    unsigned old = 0;
                    if (lane == 0) old = atomicAdd(p.counters + rt, 1u);
                    old = __shfl_sync(0xffffffffu, old, 0);
                    final_stage = old == (unsigned)(ksp - 1);
                    if (final_stage) {
                        __threadfence();
                        if (lane == 0) p.counters[rt] = 0u;  // ready for the next launch
                    }
                }
                if (final_stage) {
                    auto full_sum = [&](int o) {
                        if (ksp == 1) return local_sum(o);
                        const int row = o & 15, mm = o >> 4;
                        const int64_t n = rt * TILE_ROWS + row;
                        float v = 0.f;
                        for (int k = 0; k < ksp; k++) v += __ldcg(p.ws + ((size_t)k * M + mm) * a.N + n);
                        return v;
                    };
                    const CommView &cm = p.comm;
                    if (cm.world <= 1) {
                        for (int o = lane; o < outs; o += 32) {
                            const int row = o & 15, mm = o >> 4;
                            const int64_t n = rt * TILE_ROWS + row;
                            if (n < a.N) {
                                float v = full_sum(o);
                                if (a.bias != nullptr) v += load_as_float(a.bias, a.bias_dt, n);
                                store_from_float(a.y, a.y_dt, mm * a.ldy + n, v);
                            }
                        }
                    } else {
                        // Row-parallel linear: the all-reduce happens here, tile by tile, over peer memory, while other
                        // warps are still streaming weights.
                        exchange_row_tile(cm, rt, M, a.N, lane, p.status, full_sum, [&](int mm, int64_t n, float v) {
                            if (a.bias != nullptr) v += load_as_float(a.bias, a.bias_dt, n);
                            store_from_float(a.y, a.y_dt, mm * a.ldy + n, v);
                        });
                    }
                }
            }
            __syncwarp();  // slot 2 may be rewritten by the next whole row tile
        }
        if (++sb == cnsb) {
            sb = 0;
            j++;
        }
    }
    if (te) {
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        te[5] = global_ns();
        te[6] = gridDim.x * gridDim.y + ((unsigned long long)blockIdx.x << 16) + ((unsigned long long)smid << 32);
        te[7] = (unsigned long long)a.N;
    }
}

struct QmPlan {
    int stages, ksplit, gx;
    size_t smem;
};

// K split across CTAs and ring depth: the fewest K slices whose activation slice fits shared memory, more only when
// that shortens the longest warp run noticeably (few row tiles per CTA).
template <class B>
bool qm_plan(const LinearArgs &a, int sms, size_t ws_bytes, int64_t counters_cap, QmPlan &best) {
    const int M = (int)a.M, SBp = (int)a.SBp;
    bool found = false;
    double best_cost = 0.0;
    static const int ksplits[] = {1, 2, 3, 4, 6, 8};
    for (int ks : ksplits) {
        if (ks > SBp || ks > sms) break;
        if (ks > 1 && ((size_t)ks * M * a.N * sizeof(float) > ws_bytes || a.NT > counters_cap)) continue;
        const int nsb_max = (SBp + ks - 1) / ks;
        // deepest ring with which B::MIN_CTAS CTAs fit one SM (1 KB per CTA is reserved by the system); else the deepest that fits at all
        int stages = 0;
        size_t smem = 0;
        const size_t share = (QM_SMEM_MAX + 1024) / B::MIN_CTAS - 1024;
        for (int pass = 0; pass < 2 && !stages; pass++)
            for (int s = 4; s >= 2 && !stages; s--) {
                smem = qm_layout(B::NW, s, B::HDR_BYTES, B::PIECE_BYTES, B::act_bytes(M, nsb_max)).total;
                if (smem <= (pass == 0 ? share : QM_SMEM_MAX)) stages = s;
            }
        if (!stages) continue;
        const bool shared_sm = smem <= share;
        const int gx_cap = (shared_sm ? sms * B::MIN_CTAS : sms) / ks;
        const int gx = (int)(a.NT < gx_cap ? a.NT : gx_cap);
        const int64_t rows = (a.NT + gx - 1) / gx;
        if (rows > QM_MAX_ROW_TILES) continue;
        const int64_t run = (rows * nsb_max + B::NW - 1) / B::NW;  // longest warp run, in tiles
        const double cost = (double)run + (ks > 1 ? 0.75 : 0.0) + 0.05 * (4 - stages) + (shared_sm ? 0.0 : 1.5);
        if (!found || cost < best_cost - 1e-9) {
            found = true;
            best_cost = cost;
            best = QmPlan{stages, ks, gx, smem};
        }
    }
    return found;
}

template <class B, int STAGES>
cudaError_t qm_launch(const QmParams &p, const QmPlan &plan, cudaStream_t st) {
    auto kernel = q4k_decode_kernel<B, STAGES>;
    static bool configured[64] = {};  // per device: the shared-memory opt-in belongs to the device's copy of the function
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!configured[dev]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)QM_SMEM_MAX);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    static const bool smem_full = env_flag("TTQ_SMEM_FULL", false);
    const size_t smem = (smem_full && B::MIN_CTAS == 1) ? QM_SMEM_MAX : plan.smem;
    return launch_pdl(kernel, dim3((unsigned)plan.gx, (unsigned)plan.ksplit), dim3(B::THREADS), smem, st, p);
}

template <class B>
cudaError_t qm_dispatch(const QmParams &p, int sms, size_t ws_bytes, int64_t counters_cap, cudaStream_t st) {
    QmPlan plan;
    if (!qm_plan<B>(p.a, sms, ws_bytes, counters_cap, plan)) return cudaErrorNotSupported;
    if (plan.stages == 4) return qm_launch<B, 4>(p, plan, st);
    return plan.stages == 3 ? qm_launch<B, 3>(p, plan, st) : qm_launch<B, 2>(p, plan, st);
}

}  // namespace

bool q4k_mma_supported(const LinearArgs &a) {
    return a.M >= 1 && a.M <= QM_MAX_M && (a.x_dt == TTQ_DT_BF16 || a.x_dt == TTQ_DT_F16) && a.K == a.SBp * TILE_K;
}

cudaError_t launch_q4k_mma(const LinearArgs &a, int sms, int *status, unsigned long long *trace, float *ws, size_t ws_bytes,
                           unsigned *counters, int64_t counters_cap, cudaStream_t st, int *launches, const CommView *comm) {
    *launches = 0;
    if (!q4k_mma_supported(a)) return cudaErrorNotSupported;
    QmParams p;
    p.a = a;
    p.ws = ws;
    p.counters = counters;
    p.status = status;
    p.trace = trace;
    static const long long trace_all_n = []() {
        const char *v = getenv("TTQ_TRACE_ALL_N");
        return v ? atoll(v) : -1ll;
    }();
    p.trace_all = trace_all_n == (long long)a.N ? 1 : 0;
    if (comm != nullptr) p.comm = *comm;
    else p.comm.world = 0;
    cudaError_t e;
    if (a.M <= 8) e = qm_dispatch<F16Backend<1, 16>>(p, sms, ws_bytes, counters_cap, st);
    else e = qm_dispatch<F16Backend<2, 20>>(p, sms, ws_bytes, counters_cap, st);
    if (e == cudaSuccess) *launches = 1;
    return e;
}

}  // namespace ttq
