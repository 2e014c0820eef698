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

#include "ttq_devutil.cuh"
#include "ttq_xprep.cuh"

namespace ttq {

namespace {

constexpr int GEMV_WARPS = 8;  // warps of the activation pass and of the small GEMV CTA; at most this many split K
constexpr int GEMV_THREADS = GEMV_WARPS * 32;
constexpr int PLANE_PAD = 16;  // bytes between activation planes in shared memory (bank spread)

// ---- integer tensor-core wrappers (D = A*B + D) ---------------------------------------------------
__device__ __forceinline__ void mma_k32_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_k32_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- activation conversion (XqRow and xprep_convert_vals: ttq_xprep.cuh) --------------------------
// Raw 8 activations of one lane (loaded early so that several chunks' loads are in flight at once).
struct RawChunk {
    uint4 raw;
    bool vec;  // raw holds 8 16-bit values; otherwise the slow path reloads element by element
};
__device__ __forceinline__ RawChunk xprep_load(const void *xrow, int x_dt, int64_t K, int sb, int lane) {
    const int64_t k0 = (int64_t)sb * TILE_K + 8 * lane;
    RawChunk rc;
    rc.raw = make_uint4(0, 0, 0, 0);
    rc.vec = xrow != nullptr && (x_dt != TTQ_DT_F32) && (k0 + 8 <= K) &&
             ((reinterpret_cast<uintptr_t>(xrow) + 2 * k0) & 15) == 0;
    if (rc.vec) rc.raw = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(xrow) + k0);
    return rc;
}

// One warp converts the 256-wide chunk `sb` of activation row `xrow` (nullptr = emit zeros):
// xq = round(x * 32639 / amax) in [-32639, 32639], stored as two int8 planes with xq = 256*hi + lo.
__device__ __forceinline__ void xprep_convert(const RawChunk &rc, const void *xrow, int x_dt, int64_t K, int sb, int lane,
                                              const XqRow &dst) {
    const int64_t k0 = (int64_t)sb * TILE_K + 8 * lane;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = 0.f;
    if (rc.vec) {
        const uint32_t w[4] = {rc.raw.x, rc.raw.y, rc.raw.z, rc.raw.w};
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
    } else if (xrow != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (k0 + i < K) v[i] = load_as_float(xrow, x_dt, k0 + i);
    }
    xprep_convert_vals(v, sb, lane, dst);
}
__device__ __forceinline__ void xprep_chunk(const void *xrow, int x_dt, int64_t K, int sb, int lane, const XqRow &dst) {
    xprep_convert(xprep_load(xrow, x_dt, K, sb, lane), xrow, x_dt, K, sb, lane, dst);
}

// Separate conversion pass: (Mpad x SBp) chunks, one warp each; rows >= M are written as zeros.
__global__ void __launch_bounds__(GEMV_THREADS) xprep_kernel(const void *__restrict__ x, int x_dt, int64_t M,
                                                             int64_t Mpad, int64_t K, int64_t ldx, int64_t SBp,
                                                             XqView xq, unsigned long long *trace, int gated) {  // gated: bit 0 = gated activation, bit 1 = interleaved planes
    unsigned long long *te = trace_open(trace, 1);
    grid_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int64_t Kp = SBp * TILE_K;
    const int64_t unit = (int64_t)blockIdx.x * GEMV_WARPS + (threadIdx.x >> 5);
    // Pull this warp's 512 bytes of x into L2 before the wait (a hint: L2 is the coherence point, so a line the
    // preceding kernel has yet to write is still read correctly afterwards); with cold activations this takes
    // their DRAM latency off the path behind the wait.
    if (unit < M * SBp && x_dt != TTQ_DT_F32) {
        const int64_t pm = unit / SBp, psb = unit % SBp;
        const uint8_t *line = reinterpret_cast<const uint8_t *>(x) + (pm * ldx + psb * TILE_K) * 2 + (lane & 3) * 128;
        if (lane < ((gated & 1) ? 8 : 4) && psb * TILE_K + (lane & 3) * 64 < K)  // only lines that start inside the row
            asm volatile("prefetch.global.L2 [%0];" ::"l"(line + (lane >> 2) * K * 2));
    }
    grid_dependency_wait();  // the scratch planes may still be read by the preceding kernel
    if (te) te[2] = global_ns();
    if (unit >= Mpad * SBp) return;
    const int64_t m = unit / SBp;
    const int sb = (int)(unit % SBp);
    XqRow dst{xq.planes + (2 * m) * Kp, xq.planes + (2 * m + 1) * Kp, xq.sum16 + m * (Kp / 16),
              xq.sum32 + m * (Kp / 32), xq.sx + m * sx_stride(SBp), (gated & 2) != 0};
    gated &= 1;
    const void *xrow = nullptr;
    if (m < M) {
        const int esz = x_dt == TTQ_DT_F32 ? 4 : 2;
        xrow = reinterpret_cast<const uint8_t *>(x) + m * ldx * esz;
    }
    if (gated && xrow != nullptr) {
        // the row holds 2K values [gate | up]: the operand is silu(gate[k]) * up[k] (the gated-MLP activation,
        // kernels/activations.nim:14-38, folded into the conversion)
        const int64_t k0 = (int64_t)sb * TILE_K + 8 * lane;
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            v[i] = 0.f;
            if (k0 + i < K) {
                const float gv = load_as_float(xrow, x_dt, k0 + i), uv = load_as_float(xrow, x_dt, K + k0 + i);
                v[i] = gv / (1.f + expf(-gv)) * uv;
            }
        }
        xprep_convert_vals(v, sb, lane, dst);
    } else {
        xprep_chunk(xrow, x_dt, K, sb, lane, dst);
    }
    if (te) {
        te[5] = global_ns();
        te[6] = gridDim.x;
    }
}

// The activation pass of many independent linears in one launch (a recorded batch of host-buffer linears): warp u of
// the grid converts chunk u - unit0 of the item whose range holds u.  The rows may live in mapped host memory: all reads
// over the host link are in flight together, and no linear of the batch has an activation pass of its own left.
__global__ void __launch_bounds__(GEMV_THREADS) xprep_batch_kernel(const XprepBatchItem *__restrict__ items, int n, int total_units) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int u = (int)blockIdx.x * GEMV_WARPS + (threadIdx.x >> 5);
    if (u >= total_units) return;
    int lo = 0, hi = n - 1;  // last item with unit0 <= u
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (items[mid].unit0 <= u) lo = mid;
        else hi = mid - 1;
    }
    const XprepBatchItem it = items[lo];
    const int local = u - it.unit0, SBp = (int)it.SBp;
    const int m = local / SBp, sb = local - m * SBp;
    const int64_t Kp = it.SBp * TILE_K;
    XqRow dst{it.xq.planes + (2 * m) * Kp, it.xq.planes + (2 * m + 1) * Kp, it.xq.sum16 + m * (Kp / 16), it.xq.sum32 + m * (Kp / 32),
              it.xq.sx + m * sx_stride(it.SBp), false};
    const int esz = it.x_dt == TTQ_DT_F32 ? 4 : 2;
    xprep_chunk(reinterpret_cast<const uint8_t *>(it.x) + (int64_t)m * it.ldx * esz, it.x_dt, it.K, sb, lane, dst);
}

// ---- the GEMV --------------------------------------------------------------------------------
struct GemvParams {
    LinearArgs a;
    XqView xq;             // activation planes in scratch
    const uint8_t *zeros;  // >= 512 zero bytes in global memory (operand of lanes outside the block diagonal)
    int wk;                // warps that split K of one row tile (1, 2, 4 or 8)
    int *status;           // device word: bit 0 set when a bounded wait gave up
    unsigned long long *trace;  // optional timeline buffer (nullptr = off): [0] = entry counter, entries of 8 words from [8]
    CommView comm;         // row-parallel exchange over peer memory (world <= 1: none)
};

constexpr int RING_STAGES = 2;  // stages of each warp's bulk-copy ring (the barrier area below is sized from it)
constexpr int XSRC_CONVERT = 0, XSRC_COPY = 1, XSRC_GLOBAL = 2;
constexpr int ZERO_BYTES = 512;

// K distance between the sub-blocks that share one MMA (groups u = 0..3), in weights = plane bytes
__host__ __device__ constexpr int group_stride(int fmt) { return fmt == TTQ_FMT_Q4_K ? 64 : (fmt == TTQ_FMT_Q8_0 ? 32 : 16); }

// Shared-memory carve-up, identical on host (size) and device (offsets).  `rows` = activation rows
// held in shared memory (0 when they stay in scratch).
struct SmemLayout {
    uint32_t bars, zero, hdr, red, ring, sx, sum32, sum16, planes, total;
};
__host__ __device__ inline SmemLayout smem_layout(int fmt, int MP, int rows, int64_t SBp, int nw) {
    SmemLayout L;
    const int64_t Kp = SBp * TILE_K;
    uint32_t o = 0;
    L.bars = o; o += nw * 8 * RING_STAGES + 64;              // [warps][stages] mbarriers, then one for the planes
    o = (o + 127u) & ~127u;
    L.zero = o; o += ZERO_BYTES;
    L.hdr = o; o += nw * 1024;                        // per-warp unpacked sub-block scales
    L.red = o; o += nw * 2 * TILE_ROWS * MP * 4;      // per-warp partial sums: dot part, offset part
    L.ring = o; o += nw * RING_STAGES * tile_bytes(fmt);
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
// Operand B of one MMA is block diagonal: column c = 2u + plane is non-zero only in K group u.  A
// lane (g, t) supplies column g in groups t>>1 (register b0) and 2 + (t>>1) (register b1), so at
// most one of its two registers is non-zero; the other one (or both) is read from a zero region.
// b0/b1 addresses of activation row m, tile sb: base + mul * (sb*256 + m*row_step), mul = 0 for zeros.
template <bool SHARED>
struct ActView {
    uint32_t b0_s, b1_s;          // SHARED: shared-memory addresses
    const uint8_t *b0_g, *b1_g;   // !SHARED: global pointers
    uint32_t mul0, mul1;          // 1 if the register is on the diagonal, else 0
    uint32_t row_step;            // bytes between the plane pairs of consecutive activation rows
    uint32_t sx_s, sum32_s, sum16_s;        // SHARED: addresses of row 0
    const float *sx_g, *sum32_g, *sum16_g;  // !SHARED
    int SBs, Kp;

    template <int OFF>
    __device__ __forceinline__ uint32_t b0(uint32_t off) const {
        if constexpr (SHARED) return lds32<OFF>(b0_s + off);
        else return __ldg(reinterpret_cast<const uint32_t *>(b0_g + off + OFF));
    }
    template <int OFF>
    __device__ __forceinline__ uint32_t b1(uint32_t off) const {
        if constexpr (SHARED) return lds32<OFF>(b1_s + off);
        else return __ldg(reinterpret_cast<const uint32_t *>(b1_g + off + OFF));
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
__device__ __forceinline__ float combine(const int (&c)[4], int i) { return (float)(c[2 * i] * 256 + c[2 * i + 1]); }

// One tile (16 rows x 256 weights) from a shared-memory stage, for MR activation rows m0..m0+MR-1.
//  Main role, lane (g,t): after the windows of a set are accumulated it owns the integer dot
//  products of sub-block t of the set for rows g and g+8; it scales them and adds them to
//  yacc[m][0..1] (the four t lanes of a row hold different sub-blocks: summed at flush time).
//  Header role, lane (r = lane&15, h = lane>>4): unpacks the scales of row r (half h of the
//  sub-blocks) into shared memory for the main role, and accumulates the part of the result that
//  does not depend on the quants (Q4_K: dmin*m_j * sum of activations; Q6_K: the -32 offset) into
//  oacc[m].  Output = sum over K tiles of (yacc parts) - (oacc parts of both halves).
template <int FMT, bool SHARED, int MR>
__device__ __forceinline__ void compute_tile(uint32_t stage, int sb, int m0, int lane, uint32_t hdr,
                                             const ActView<SHARED> &A, float (&yacc)[MR][2], float (&oacc)[MR]) {
    const int g = lane >> 2, t = lane & 3;
    const int r = lane & 15, h = lane >> 4;
    const uint32_t sa = stage + (uint32_t)lane * 16;
    const uint32_t toff = (uint32_t)sb * TILE_K + (uint32_t)m0 * A.row_step;
    const uint32_t off0 = A.mul0 * toff, off1 = A.mul1 * toff;
    const uint32_t rs0 = A.mul0 * A.row_step, rs1 = A.mul1 * A.row_step;
    float tmp[MR][2];
#pragma unroll
    for (int m = 0; m < MR; m++) tmp[m][0] = tmp[m][1] = 0.f;

    if constexpr (FMT == TTQ_FMT_Q4_K) {
        {
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
            sts128f<0>(hdr + (uint32_t)(r * 8 + 4 * h) * 4, d * byte_to_float(scw, 0), d16 * byte_to_float(scw, 1),
                       d * byte_to_float(scw, 2), d16 * byte_to_float(scw, 3));
            const float mn0 = byte_to_float(mw, 0), mn1 = byte_to_float(mw, 1), mn2 = byte_to_float(mw, 2),
                        mn3 = byte_to_float(mw, 3);
#pragma unroll
            for (int m = 0; m < MR; m++) {
                const float4 s4 = A.sum32x4(m0 + m, sb * 8 + h * 4);
                const float part = fmaf(mn0, s4.x, fmaf(mn1, s4.y, fmaf(mn2, s4.z, mn3 * s4.w)));
                oacc[m] = fmaf(A.sx(m0 + m, sb) * dmin, part, oacc[m]);
            }
            __syncwarp();
        }
        int cx[MR][4], cy[MR][4];
#pragma unroll
        for (int m = 0; m < MR; m++)
#pragma unroll
            for (int i = 0; i < 4; i++) cx[m][i] = cy[m][i] = 0;
        static_for<0, 4>([&](auto n_) {
            constexpr int n = decltype(n_)::value;
            const uint4 w = lds128<n * 512>(sa);
            const uint32_t l0 = w.x & 0x0f0f0f0fu, l1 = w.y & 0x0f0f0f0fu, l2 = w.z & 0x0f0f0f0fu, l3 = w.w & 0x0f0f0f0fu;
            const uint32_t h0 = w.x & 0xf0f0f0f0u, h1 = w.y & 0xf0f0f0f0u, h2 = w.z & 0xf0f0f0f0u, h3 = w.w & 0xf0f0f0f0u;
#pragma unroll
            for (int m = 0; m < MR; m++) {
                const uint32_t o0 = off0 + m * rs0, o1 = off1 + m * rs1;
                mma_k32_u8s8(cx[m], l0, l1, l2, l3, A.template b0<8 * n>(o0), A.template b1<8 * n>(o1));
                mma_k32_u8s8(cy[m], h0, h1, h2, h3, A.template b0<32 + 8 * n>(o0), A.template b1<32 + 8 * n>(o1));
            }
        });
        // lane (g,t): set X holds sub-block 2t, set Y sub-block 2t+1
        const uint32_t hr = hdr + (uint32_t)(g * 8 + 2 * t) * 4;
        const float2 sg = lds64f<0>(hr), sg8 = lds64f<256>(hr);
#pragma unroll
        for (int m = 0; m < MR; m++) {
            tmp[m][0] = fmaf(sg.x, combine(cx[m], 0), sg.y * combine(cy[m], 0));
            tmp[m][1] = fmaf(sg8.x, combine(cx[m], 1), sg8.y * combine(cy[m], 1));
        }
    } else if constexpr (FMT == TTQ_FMT_Q8_0) {
        {
            // fp16 d[r][b]: header lane (r, h) converts blocks 4h..4h+3 of row r
            const uint2 dv = lds64<4096>(stage + (uint32_t)r * 16 + (uint32_t)h * 8);
            const float2 f01 = __half22float2(*reinterpret_cast<const __half2 *>(&dv.x));
            const float2 f23 = __half22float2(*reinterpret_cast<const __half2 *>(&dv.y));
            __syncwarp();
            sts128f<0>(hdr + (uint32_t)(r * 8 + 4 * h) * 4, f01.x, f01.y, f23.x, f23.y);
            __syncwarp();
        }
        const uint32_t hr = hdr + (uint32_t)(g * 8 + t) * 4;
        static_for<0, 2>([&](auto s_) {
            constexpr int s = decltype(s_)::value;
            int cs[MR][4];
#pragma unroll
            for (int m = 0; m < MR; m++)
#pragma unroll
                for (int i = 0; i < 4; i++) cs[m][i] = 0;
            static_for<0, 4>([&](auto n_) {
                constexpr int n = decltype(n_)::value;
                const uint4 w = lds128<(4 * s + n) * 512>(sa);
#pragma unroll
                for (int m = 0; m < MR; m++)
                    mma_k32_s8s8(cs[m], w.x, w.y, w.z, w.w, A.template b0<128 * s + 8 * n>(off0 + m * rs0),
                                 A.template b1<128 * s + 8 * n>(off1 + m * rs1));
            });
            const float dg = ldsf<16 * s>(hr), dg8 = ldsf<256 + 16 * s>(hr);  // block 4s+t of rows g, g+8
#pragma unroll
            for (int m = 0; m < MR; m++) {
                tmp[m][0] = fmaf(dg, combine(cs[m], 0), tmp[m][0]);
                tmp[m][1] = fmaf(dg8, combine(cs[m], 1), tmp[m][1]);
            }
        });
    } else {
        {
            // int8 scales[r][16], fp16 d[r]: header lane (r, h) handles sub-blocks 8h..8h+7 of row r
            const uint2 scw = lds64<3072>(stage + (uint32_t)r * 16 + (uint32_t)h * 8);
            const float d = __half2float(
                __ushort_as_half((unsigned short)(lds32<3328>(stage + (uint32_t)(r >> 1) * 4) >> (16 * (r & 1)))));
            float ds[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t word = i < 4 ? scw.x : scw.y;
                ds[i] = d * (float)(int)(int8_t)((word >> (8 * (i & 3))) & 0xff);
            }
            __syncwarp();
            const uint32_t hw = hdr + (uint32_t)(r * 16 + 8 * h) * 4;
            sts128f<0>(hw, ds[0], ds[1], ds[2], ds[3]);
            sts128f<16>(hw, ds[4], ds[5], ds[6], ds[7]);
#pragma unroll
            for (int m = 0; m < MR; m++) {
                const float4 sA = A.sum16x4(m0 + m, sb * 16 + h * 8), sB = A.sum16x4(m0 + m, sb * 16 + h * 8 + 4);
                float part = fmaf(ds[0], sA.x, fmaf(ds[1], sA.y, fmaf(ds[2], sA.z, ds[3] * sA.w)));
                part = fmaf(ds[4], sB.x, fmaf(ds[5], sB.y, fmaf(ds[6], sB.z, fmaf(ds[7], sB.w, part))));
                oacc[m] = fmaf(A.sx(m0 + m, sb) * 32.f, part, oacc[m]);  // quants are stored with a +32 offset
            }
            __syncwarp();
        }
        const uint32_t hr = hdr + (uint32_t)(g * 16 + t) * 4;
        static_for<0, 4>([&](auto s_) {
            constexpr int s = decltype(s_)::value;
            int cs[MR][4];
#pragma unroll
            for (int m = 0; m < MR; m++)
#pragma unroll
                for (int i = 0; i < 4; i++) cs[m][i] = 0;
            static_for<0, 2>([&](auto n_) {
                constexpr int n = decltype(n_)::value;
                const uint4 ql = lds128<(2 * (s & 1) + n) * 512>(sa);
                const uint4 qh = lds128<2048 + n * 512>(sa);
                const uint32_t qlw[4] = {ql.x, ql.y, ql.z, ql.w}, qhw[4] = {qh.x, qh.y, qh.z, qh.w};
                uint32_t a[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t lo = (s >> 1) ? (qlw[i] >> 4) : qlw[i];
                    // high 2 bits of set s sit at bit pair s of each byte: move them to bits 4..5
                    const uint32_t hb = s == 0 ? (qhw[i] << 4) : s == 1 ? (qhw[i] << 2) : s == 2 ? qhw[i] : (qhw[i] >> 2);
                    a[i] = (lo & 0x0f0f0f0fu) | (hb & 0x30303030u);
                }
#pragma unroll
                for (int m = 0; m < MR; m++)
                    mma_k32_u8s8(cs[m], a[0], a[1], a[2], a[3], A.template b0<64 * s + 8 * n>(off0 + m * rs0),
                                 A.template b1<64 * s + 8 * n>(off1 + m * rs1));
            });
            const float dg = ldsf<16 * s>(hr), dg8 = ldsf<512 + 16 * s>(hr);  // sub-block 4s+t of rows g, g+8
#pragma unroll
            for (int m = 0; m < MR; m++) {
                tmp[m][0] = fmaf(dg, combine(cs[m], 0), tmp[m][0]);
                tmp[m][1] = fmaf(dg8, combine(cs[m], 1), tmp[m][1]);
            }
        });
    }
#pragma unroll
    for (int m = 0; m < MR; m++) {
        const float sx = A.sx(m0 + m, sb);
        yacc[m][0] = fmaf(sx, tmp[m][0], yacc[m][0]);
        yacc[m][1] = fmaf(sx, tmp[m][1], yacc[m][1]);
    }
}

// NPASS passes of MR activation rows each are made over every tile (NPASS > 1 only with scratch planes).
// NW warps per CTA: 8 (two or three CTAs per SM) or 16 / 24 (one CTA per SM, so that the activation
// conversion of XSRC_CONVERT is done once per SM instead of once per small CTA).
template <int FMT, int XSRC, int MR, int NPASS, int NW>
__global__ void __launch_bounds__(NW * 32, NW > 8 ? 1 : (XSRC == XSRC_GLOBAL ? 2 : 3)) gemv_kernel(GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr bool SHARED = XSRC != XSRC_GLOBAL;
    constexpr int TB = tile_bytes(FMT);
    constexpr int STAGES = RING_STAGES;
    constexpr int MP = MR * NPASS;
    const LinearArgs &a = p.a;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int SBp = (int)a.SBp, Kp = SBp * TILE_K, SBs = sx_stride(a.SBp);
    const int M = (int)a.M;
    const SmemLayout L = smem_layout(FMT, MP, SHARED ? MR : 0, a.SBp, NW);
    const uint32_t smem0 = smem_u32(smem);

    const uint32_t hdr_u32 = smem0 + L.hdr + warp * 1024;
    float *red_s = reinterpret_cast<float *>(smem + L.red);
    const uint32_t ring_u32 = smem0 + L.ring + warp * STAGES * TB;
    const uint32_t bar_u32 = smem0 + L.bars + warp * STAGES * 8;
    const uint32_t xbar_u32 = smem0 + L.bars + NW * STAGES * 8;

    // group / K-slice of this warp
    const int WK = p.wk, R = NW / WK;
    const int grp = warp / WK, ks = warp % WK;
    const int sb_begin = (ks * SBp) / WK, sb_end = ((ks + 1) * SBp) / WK;
    const int nsb = sb_end - sb_begin;
    // row tiles of this group: rt(it) = (it * gridDim.x + blockIdx.x) * R + grp
    const int64_t rt0 = (int64_t)blockIdx.x * R + grp, rt_step = (int64_t)gridDim.x * R;
    const int n_iters = rt0 < a.NT ? (int)((a.NT - rt0 + rt_step - 1) / rt_step) : 0;
    const int total_items = n_iters * nsb;

    unsigned long long *te = trace_open(p.trace, 2);
    grid_launch_dependents();  // the next kernel may start its own weight copies as soon as it fits

    // ---- ring set-up and first copies (weights do not depend on the activations)
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) mbar_init(bar_u32 + 8 * s, 1);
        if (XSRC == XSRC_COPY && warp == 0) mbar_init(xbar_u32, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (SHARED && threadIdx.x < ZERO_BYTES / 4) reinterpret_cast<uint32_t *>(smem + L.zero)[threadIdx.x] = 0u;
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
    if (te) te[2] = global_ns();
    ActView<SHARED> A;
    A.SBs = SBs;
    A.Kp = Kp;
    const int g = lane >> 2, t = lane & 3;
    // block-diagonal operand: this lane's column g belongs to K group g>>1
    const bool act0 = (g >> 1) == (t >> 1), act1 = (g >> 1) == 2 + (t >> 1);
    const uint32_t lane_off = (uint32_t)(group_stride(FMT) * (g >> 1) + 4 * (t & 1));
    A.mul0 = act0 ? 1u : 0u;
    A.mul1 = act1 ? 1u : 0u;
    bool alive = true;  // false once a bounded wait gave up: skip further waits, keep the barriers
    if constexpr (SHARED) {
        if constexpr (XSRC == XSRC_CONVERT) {
            // every CTA converts the activations itself: no second kernel on the dependency chain
            float *sx_s = reinterpret_cast<float *>(smem + L.sx);
            float *sum32_s = reinterpret_cast<float *>(smem + L.sum32);
            float *sum16_s = reinterpret_cast<float *>(smem + L.sum16);
            int8_t *planes_s = reinterpret_cast<int8_t *>(smem + L.planes);
            const int esz = a.x_dt == TTQ_DT_F32 ? 4 : 2;
            const int units = MR * SBp;
            constexpr int BATCH = NW > 8 ? 4 : 8;  // chunks whose loads one warp keeps in flight together
            for (int u0 = warp; u0 < units; u0 += BATCH * NW) {
                RawChunk rc[BATCH];
#pragma unroll
                for (int i = 0; i < BATCH; i++) {
                    const int u = u0 + i * NW;
                    if (u < units) {
                        const int m = u / SBp, sb = u - m * SBp;
                        rc[i] = xprep_load(reinterpret_cast<const uint8_t *>(a.x) + (int64_t)m * a.ldx * esz, a.x_dt, a.K, sb, lane);
                    }
                }
#pragma unroll
                for (int i = 0; i < BATCH; i++) {
                    const int u = u0 + i * NW;
                    if (u < units) {
                        const int m = u / SBp, sb = u - m * SBp;
                        XqRow dst{planes_s + (2 * m) * (Kp + PLANE_PAD), planes_s + (2 * m + 1) * (Kp + PLANE_PAD),
                                  sum16_s + m * (Kp / 16), sum32_s + m * (Kp / 32), sx_s + m * SBs};
                        xprep_convert(rc[i], reinterpret_cast<const uint8_t *>(a.x) + (int64_t)m * a.ldx * esz, a.x_dt, a.K, sb,
                                      lane, dst);
                    }
                }
            }
            __syncthreads();  // planes complete, zero region written
        } else {
            // planes and side arrays were produced by the conversion pass: bulk-copy them in
            __syncthreads();  // the plane barrier is initialised, the zero region is written
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
        const uint32_t col_base = smem0 + L.planes + (uint32_t)(g & 1) * (Kp + PLANE_PAD) + lane_off;
        // +32: keeps the broadcast zero word off the banks the diagonal lanes read
        A.b0_s = act0 ? col_base : smem0 + L.zero + 32;
        A.b1_s = act1 ? col_base : smem0 + L.zero + 32;
        A.row_step = 2u * (Kp + PLANE_PAD);
        A.sx_s = smem0 + L.sx;
        A.sum32_s = smem0 + L.sum32;
        A.sum16_s = smem0 + L.sum16;
    } else {
        const uint8_t *col_base = reinterpret_cast<const uint8_t *>(p.xq.planes) + (int64_t)(g & 1) * Kp + lane_off;
        A.b0_g = act0 ? col_base : p.zeros;
        A.b1_g = act1 ? col_base : p.zeros;
        A.row_step = 2u * Kp;
        A.sx_g = p.xq.sx;
        A.sum32_g = p.xq.sum32;
        A.sum16_g = p.xq.sum16;
    }

    if (te) te[3] = global_ns();
    // ---- main loop over this warp's items
    int item = 0;
    float *redy = red_s + warp * (2 * MP * TILE_ROWS), *redo = redy + MP * TILE_ROWS;
    for (int it = 0; it < n_iters; it++) {
        float yacc[NPASS][MR][2], oacc[NPASS][MR];
#pragma unroll
        for (int ps = 0; ps < NPASS; ps++)
#pragma unroll
            for (int m = 0; m < MR; m++) yacc[ps][m][0] = yacc[ps][m][1] = oacc[ps][m] = 0.f;
        for (int sbi = 0; sbi < nsb; sbi++, item++) {
            const int s = item % STAGES;
            if (alive) alive = mbar_wait_bounded(bar_u32 + 8 * s, (uint32_t)((item / STAGES) & 1), p.status);
            if (te && item == 0) te[4] = global_ns();
#pragma unroll
            for (int ps = 0; ps < NPASS; ps++)
                compute_tile<FMT, SHARED, MR>(ring_u32 + s * TB, sb_begin + sbi, ps * MR, lane, hdr_u32, A, yacc[ps], oacc[ps]);
            __syncwarp();  // every lane is done reading the stage before it is refilled
            if (lane == 0 && alive && p_item < total_items) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                issue_next();
            }
        }
        // ---- flush the row tile of this iteration
        // the four t lanes of a row hold different sub-blocks, the two header halves different scales
#pragma unroll
        for (int ps = 0; ps < NPASS; ps++)
#pragma unroll
            for (int m = 0; m < MR; m++) {
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    float v = yacc[ps][m][i];
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    if (t == 0) redy[(ps * MR + m) * TILE_ROWS + g + 8 * i] = v;
                }
                float o = oacc[ps][m];
                o += __shfl_xor_sync(0xffffffffu, o, 16);
                if (lane < 16) redo[(ps * MR + m) * TILE_ROWS + lane] = o;
            }
        if (WK > 1) named_barrier(1 + grp, WK * 32);
        else __syncwarp();
        if (ks == 0) {
            const int64_t rt = rt0 + it * rt_step;
            const CommView &cm = p.comm;
            if (cm.world <= 1) {
                for (int o = lane; o < MP * TILE_ROWS; o += 32) {
                    const int row = o & 15, mm = o >> 4;
                    const int64_t n = rt * TILE_ROWS + row;
                    if (mm < M && n < a.N) {
                        float acc = 0.f;
                        for (int w = 0; w < WK; w++) {
                            const float *rw = red_s + (grp * WK + w) * (2 * MP * TILE_ROWS);
                            acc += rw[o] - rw[MP * TILE_ROWS + o];
                        }
                        if (a.bias != nullptr) acc += load_as_float(a.bias, a.bias_dt, n);
                        store_from_float(a.y, a.y_dt, mm * a.ldy + n, acc);
                    }
                }
            } else {
                // Row-parallel linear: the all-reduce happens here, tile by tile, over peer memory, while other warps
                // are still streaming weights.
                exchange_row_tile(
                    cm, rt, M, a.N, lane, p.status,
                    [&](int o) {
                        float acc = 0.f;
                        for (int w = 0; w < WK; w++) {
                            const float *rw = red_s + (grp * WK + w) * (2 * MP * TILE_ROWS);
                            acc += rw[o] - rw[MP * TILE_ROWS + o];
                        }
                        return acc;
                    },
                    [&](int mm, int64_t n, float v) {
                        if (a.bias != nullptr) v += load_as_float(a.bias, a.bias_dt, n);
                        store_from_float(a.y, a.y_dt, mm * a.ldy + n, v);
                    });
            }
        }
        if (WK > 1) named_barrier(1 + grp, WK * 32);  // the partial-sum area is free again
        else __syncwarp();
    }
    if (te) {
        te[5] = global_ns();
        te[6] = gridDim.x;
        te[7] = (unsigned long long)a.N;
    }
}

constexpr size_t GEMV_SMEM_LIMIT = 112 * 1024;  // at least two CTAs per SM

// K-split factor: the one that minimises the longest CTA's work, measured in row tiles of full K
// (ties: fewer slices, less reduction).  cap = resident CTAs.
int pick_wk(int64_t NT, int64_t SBp, int64_t cap, int nw) {
    int best = 1;
    int64_t best_cost = -1;
    for (int wk = 1; wk <= GEMV_WARPS; wk *= 2) {
        if (wk > 1 && wk > SBp) break;
        const int R = nw / wk;
        const int64_t cta_iters = (NT + R - 1) / R;
        const int64_t rounds = (cta_iters + cap - 1) / cap;
        // a round costs R row tiles spread over 8 warps; compare in units of 1/8 row tile per warp
        const int64_t cost = rounds * (8 / wk);  // each round: a warp walks 1/wk of K for one row tile
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best = wk;
        }
    }
    return best;
}

constexpr size_t GEMV_SMEM_BIG = 200 * 1024;  // one CTA per SM

template <int FMT, int XSRC, int MR, int NPASS, int NW>
cudaError_t launch_one(GemvParams &p, int sms, cudaStream_t st) {
    auto kernel = gemv_kernel<FMT, XSRC, MR, NPASS, NW>;
    const size_t smem = smem_layout(FMT, MR * NPASS, XSRC == XSRC_GLOBAL ? 0 : MR, p.a.SBp, NW).total;
    // per instantiation and per device: the shared-memory opt-in belongs to the device's copy of the function
    static bool configured[64] = {};
    static int occ_cache_smem = -1, occ_cache = 0;
    cudaError_t e;
    int dev = 0;
    if ((e = cudaGetDevice(&dev))) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!configured[dev]) {
        const int lim = (int)(NW > 8 ? GEMV_SMEM_BIG : GEMV_SMEM_LIMIT);
        if ((e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, lim))) return e;
        configured[dev] = true;
    }
    if (occ_cache_smem != (int)smem) {
        if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ_cache, kernel, NW * 32, smem))) return e;
        occ_cache_smem = (int)smem;
    }
    if (occ_cache < 1) return cudaErrorLaunchOutOfResources;
    const int64_t cap = (int64_t)sms * occ_cache;
    p.wk = pick_wk(p.a.NT, p.a.SBp, cap, NW);
    const int R = NW / p.wk;
    const int64_t cta_iters = (p.a.NT + R - 1) / R;
    const unsigned grid = (unsigned)(cta_iters < cap ? cta_iters : cap);
    return launch_pdl(kernel, dim3(grid), dim3(NW * 32), smem, st, p);
}

template <int FMT, int XSRC, int NW>
cudaError_t dispatch_rows(GemvParams &p, int sms, cudaStream_t st) {
    switch (p.a.M) {
    case 1: return launch_one<FMT, XSRC, 1, 1, NW>(p, sms, st);
    case 2: return launch_one<FMT, XSRC, 2, 1, NW>(p, sms, st);
    case 3: return launch_one<FMT, XSRC, 3, 1, NW>(p, sms, st);
    default: return launch_one<FMT, XSRC, 4, 1, NW>(p, sms, st);
    }
}

// warps per CTA for the modes that keep the activations in shared memory; 0 = they do not fit
int pick_nw(int fmt, int mode, int64_t M, int64_t SBp) {
    if (mode == XSRC_CONVERT) {
        if (smem_layout(fmt, (int)M, (int)M, SBp, 24).total <= GEMV_SMEM_BIG) return 24;
        if (smem_layout(fmt, (int)M, (int)M, SBp, 16).total <= GEMV_SMEM_BIG) return 16;
    }
    if (smem_layout(fmt, (int)M, (int)M, SBp, 8).total <= GEMV_SMEM_LIMIT) return 8;
    return 0;
}

template <int FMT>
cudaError_t dispatch(GemvParams &p, int mode, int nw, int sms, cudaStream_t st) {
    if (mode == XSRC_CONVERT) {
        if (nw == 24) return dispatch_rows<FMT, XSRC_CONVERT, 24>(p, sms, st);
        if (nw == 16) return dispatch_rows<FMT, XSRC_CONVERT, 16>(p, sms, st);
        return dispatch_rows<FMT, XSRC_CONVERT, 8>(p, sms, st);
    }
    if (mode == XSRC_COPY) return dispatch_rows<FMT, XSRC_COPY, 8>(p, sms, st);
    if (p.a.M <= 4) return launch_one<FMT, XSRC_GLOBAL, 4, 1, 8>(p, sms, st);
    if (p.a.M <= 8) return launch_one<FMT, XSRC_GLOBAL, 4, 2, 8>(p, sms, st);
    return launch_one<FMT, XSRC_GLOBAL, 4, 4, 8>(p, sms, st);
}

}  // namespace

// The separate activation pass: rows [0, M) of x become int8 planes, group sums and chunk scales in `xq`; rows
// [M, Mpad) are written as zeros.
cudaError_t launch_xprep(const LinearArgs &a, const XqView &xq, int64_t Mpad, unsigned long long *trace, cudaStream_t st, bool interleaved) {
    const int64_t units = Mpad * a.SBp;
    return launch_pdl(xprep_kernel, dim3((unsigned)((units + GEMV_WARPS - 1) / GEMV_WARPS)), dim3(GEMV_THREADS), 0, st, a.x, a.x_dt, a.M,
                      Mpad, a.K, a.ldx, a.SBp, xq, trace, (a.gated ? 1 : 0) | (interleaved ? 2 : 0));
}

cudaError_t launch_xprep_batch(const XprepBatchItem *items_dev, int n, int total_units, cudaStream_t st) {
    return launch_pdl(xprep_batch_kernel, dim3((unsigned)((total_units + GEMV_WARPS - 1) / GEMV_WARPS)), dim3(GEMV_THREADS), 0, st, items_dev, n,
                      total_units);
}

// whether launch_gemv serves a linear of M rows from activation planes somebody else prepared
bool gemv_prepared_supported(int fmt, int64_t M, int64_t SBp) {
    return (fmt == TTQ_FMT_Q4_K || fmt == TTQ_FMT_Q8_0 || fmt == TTQ_FMT_Q6_K) && M >= 1 && M <= 4 && pick_nw(fmt, XSRC_COPY, M, SBp) != 0;
}

cudaError_t launch_gemv(int fmt, const LinearArgs &a, const XqView &xq, int64_t xq_capacity_k, const uint8_t *zeros,
                        int sms, int *status, unsigned long long *trace, cudaStream_t st, int *launches, const CommView *comm,
                        bool prepared) {
    GemvParams p{a, xq, zeros, 1, status, trace, {}};
    if (comm != nullptr) p.comm = *comm;
    else p.comm.world = 0;
    *launches = 0;
    const int64_t Kp = a.SBp * TILE_K;
    if (Kp > xq_capacity_k) return cudaErrorInvalidValue;
    // Activation conversion: by default one separate pass whose planes every CTA bulk-copies into shared
    // memory (measured fastest on decode chains); TTQ_XPREP=fused converts inside every CTA instead.
    static const int pref = []() {
        const char *v = getenv("TTQ_XPREP");
        if (v && v[0] == 'f') return XSRC_CONVERT;  // "fused"
        if (v && v[0] == 'g') return XSRC_GLOBAL;   // "global": separate pass, fragments read from scratch
        return XSRC_COPY;                           // "separate" (default)
    }();
    int mode = pref;
    if (a.gated && mode == XSRC_CONVERT) mode = XSRC_COPY;  // the gated activation lives in the separate pass
    if (prepared) {
        // planes written in the layout of a.M rows by the producer of the activations: only the copying mode reads that
        if (a.gated || a.M > 4 || pick_nw(fmt, XSRC_COPY, a.M, a.SBp) == 0) return cudaErrorNotSupported;
        mode = XSRC_COPY;
    }
    const int nw = (a.M <= 4 && mode != XSRC_GLOBAL) ? pick_nw(fmt, mode, a.M, a.SBp) : 0;
    if (nw == 0) mode = XSRC_GLOBAL;
    const bool shared = mode != XSRC_GLOBAL;
    cudaError_t e = cudaSuccess;
    if (mode != XSRC_CONVERT && !prepared) {
        e = launch_xprep(a, xq, shared ? a.M : (a.M <= 4 ? 4 : (a.M <= 8 ? 8 : 16)), trace, st, false);
        if (e != cudaSuccess) return e;
        ++*launches;
    }
    if (fmt == TTQ_FMT_Q4_K) e = dispatch<TTQ_FMT_Q4_K>(p, mode, nw, sms, st);
    else if (fmt == TTQ_FMT_Q8_0) e = dispatch<TTQ_FMT_Q8_0>(p, mode, nw, sms, st);
    else e = dispatch<TTQ_FMT_Q6_K>(p, mode, nw, sms, st);
    if (e == cudaSuccess) ++*launches;
    return e;
}

}  // namespace ttq

// ================================================================================================
// ttq_linear_forward_static: the same decode linear with NO allocation anywhere on its path.
//
// Who needs it: a host that may not (or cannot) call the CUDA allocator -- an inference server that
// has handed every byte of device memory to its own pool, or a plug-in running under a framework that
// forbids cudaMalloc after start-up.  ttq_init allocates scratch and staging buffers, so such a host
// cannot create a context; this entry point needs none.  The activation planes that the context
// normally keeps in allocated scratch live here in a fixed array inside the library image.  The array
// is part of the module: every GPU that loads the library reserves it until the process exits.
//
// Limits: M <= TTQ_STATIC_MAX_M rows, K <= TTQ_STATIC_MAX_K (after rounding K up to 256).
// The array is shared by all calls and keeps whatever the last call left in it; each call rewrites
// every byte it will read (padding rows are written as zeros by the conversion pass); the zero page at
// its start is never written, and the status word in it is cleared by ttq_static_status only.  Two calls that overlap on the GPU
// (different streams, or different host threads) race on the array: issue them on one stream.
// ================================================================================================
namespace ttq {
namespace {

constexpr int64_t TTQ_STATIC_MAX_M = 4;
constexpr int64_t TTQ_STATIC_MAX_K = 16384;
constexpr size_t ST_ZERO = 1024;                                             // zero page + status word at byte 768
constexpr size_t ST_PLANES = (size_t)2 * TTQ_STATIC_MAX_M * TTQ_STATIC_MAX_K;  // int8 planes
constexpr size_t ST_SUM16 = (size_t)TTQ_STATIC_MAX_M * (TTQ_STATIC_MAX_K / 16) * 4;
constexpr size_t ST_SUM32 = (size_t)TTQ_STATIC_MAX_M * (TTQ_STATIC_MAX_K / 32) * 4;
constexpr size_t ST_SX = (size_t)TTQ_STATIC_MAX_M * (TTQ_STATIC_MAX_K / 256 + 4) * 4;
constexpr size_t ST_TOTAL = ST_ZERO + ST_PLANES + ST_SUM16 + ST_SUM32 + ST_SX;
static_assert(ST_TOTAL == 157760, "the documented size of the static scratch array (ttq.h) must follow this sum");

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_static_scratch[ST_TOTAL];

struct StaticDevice {
    bool ready;
    unsigned char *base;  // device address of g_static_scratch on this device
    int sms;
};
StaticDevice g_static_dev[64];

void set_msg(char *buf, size_t len, const char *msg) {
    if (buf && len) {
        size_t i = 0;
        for (; i + 1 < len && msg[i]; i++) buf[i] = msg[i];
        buf[i] = 0;
    }
}

}  // namespace
}  // namespace ttq

extern "C" TTQ_API ttq_status ttq_linear_forward_static(const ttq_weight *w, const void *x_dev, ttq_dtype x_dt, int64_t M,
                                                        int64_t ldx, const void *bias_dev, ttq_dtype bias_dt, void *y_dev,
                                                        ttq_dtype y_dt, int64_t ldy, void *stream, char *errbuf,
                                                        size_t errbuf_len) {
    using namespace ttq;
    set_msg(errbuf, errbuf_len, "");
    if (!w || !x_dev || !y_dev) {
        set_msg(errbuf, errbuf_len, "weight, x or y pointer is NULL");
        return TTQ_ERR_INVALID_ARG;
    }
    if (M < 0 || ldx < w->K || ldy < w->N) {
        set_msg(errbuf, errbuf_len, "negative M or leading dimension smaller than the row length");
        return TTQ_ERR_SHAPE;
    }
    if (M == 0) return TTQ_OK;
    if ((x_dt != TTQ_DT_BF16 && x_dt != TTQ_DT_F16) || y_dt < TTQ_DT_BF16 || y_dt > TTQ_DT_F32 ||
        (bias_dev && (bias_dt < TTQ_DT_BF16 || bias_dt > TTQ_DT_F32))) {
        set_msg(errbuf, errbuf_len, "unsupported dtype (x: bf16|f16; y, bias: bf16|f16|f32)");
        return TTQ_ERR_INVALID_ARG;
    }
    if (w->fmt == TTQ_FMT_TQ3) {
        set_msg(errbuf, errbuf_len, "the trellis format needs the context's rotation scratch: use ttq_linear_forward");
        return TTQ_ERR_UNSUPPORTED;
    }
    if (M > TTQ_STATIC_MAX_M || w->SBp * TILE_K > TTQ_STATIC_MAX_K) {
        set_msg(errbuf, errbuf_len, "ttq_linear_forward_static is limited to M <= 4 and K <= 16384 (fixed scratch array)");
        return TTQ_ERR_LIMIT;
    }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev != w->device || dev < 0 || dev >= 64) {
        set_msg(errbuf, errbuf_len, "the weight's device must be the current CUDA device");
        return TTQ_ERR_DEVICE;
    }
    StaticDevice &sd = g_static_dev[dev];
    if (!sd.ready) {
        // one-time set-up on this device: resolve the device address of the array (no allocation)
        void *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sd.sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess || ptr == nullptr) {
            set_msg(errbuf, errbuf_len, cudaGetErrorString(e));
            return TTQ_ERR_CUDA;
        }
        sd.base = reinterpret_cast<unsigned char *>(ptr);
        sd.ready = true;
    }
    XqView xq;
    xq.planes = reinterpret_cast<int8_t *>(sd.base + ST_ZERO);
    xq.sum16 = reinterpret_cast<float *>(sd.base + ST_ZERO + ST_PLANES);
    xq.sum32 = reinterpret_cast<float *>(sd.base + ST_ZERO + ST_PLANES + ST_SUM16);
    xq.sx = reinterpret_cast<float *>(sd.base + ST_ZERO + ST_PLANES + ST_SUM16 + ST_SUM32);
    // the status word starts at zero with the module image and is cleared only by ttq_static_status, so that a
    // failure stays visible until the host has read it; everything else the kernels read is rewritten below
    int *status = reinterpret_cast<int *>(sd.base + 768);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaSuccess;
    {
        LinearArgs a;
        a.tiles = w->tiles;
        a.N = w->N; a.K = w->K; a.NT = w->NT; a.SBp = w->SBp;
        a.x = x_dev; a.x_dt = x_dt; a.M = M; a.ldx = ldx;
        a.bias = bias_dev; a.bias_dt = bias_dt;
        a.y = y_dev; a.y_dt = y_dt; a.ldy = ldy;
        int launches = 0;
        e = launch_gemv(w->fmt, a, xq, TTQ_STATIC_MAX_K, sd.base, sd.sms, status, nullptr, st, &launches);
    }
    if (e != cudaSuccess) {
        set_msg(errbuf, errbuf_len, cudaGetErrorString(e));
        return TTQ_ERR_CUDA;
    }
    return TTQ_OK;
}


// Reads (and clears) the status word of the static scratch array: the allocation-free counterpart of
// ttq_device_status.  One 4-byte copy from the array's device address into the caller's stack and one stream
// synchronisation; nothing is allocated.
extern "C" TTQ_API ttq_status ttq_static_status(void *stream, char *errbuf, size_t errbuf_len) {
    using namespace ttq;
    set_msg(errbuf, errbuf_len, "");
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        set_msg(errbuf, errbuf_len, "no current CUDA device");
        return TTQ_ERR_DEVICE;
    }
    StaticDevice &sd = g_static_dev[dev];
    if (!sd.ready) return TTQ_OK;  // ttq_linear_forward_static has not run on this device: nothing to report
    cudaStream_t st = (cudaStream_t)stream;
    int host = 0;
    cudaError_t e = cudaMemcpyAsync(&host, sd.base + 768, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e == cudaSuccess && host != 0) e = cudaMemsetAsync(sd.base + 768, 0, sizeof(int), st);
    if (e != cudaSuccess) {
        set_msg(errbuf, errbuf_len, cudaGetErrorString(e));
        return TTQ_ERR_CUDA;
    }
    if (host != 0) {
        set_msg(errbuf, errbuf_len, "a kernel launched by ttq_linear_forward_static gave up a bounded wait; results since the last check are invalid");
        return TTQ_ERR_TIMEOUT;
    }
    return TTQ_OK;
}
