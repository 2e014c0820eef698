// The fixed-point conversion of activations shared by the activation pass (ttq_gemv.cu) and by kernels that
// produce a linear's input and convert it on the way out (ttq_decode.cu).
#pragma once

#include "ttq_internal.cuh"

namespace ttq {

// Destination of one activation row's planes and side sums (shared memory or global scratch).
struct XqRow {
    int8_t *hi, *lo;  // [Kp]
    float *sum16;     // [Kp/16]
    float *sum32;     // [Kp/32]
    float *sx;        // [SBs]
    // Order of the plane bytes inside each 32-wide sub-block: false = by K; true = position 16 h + 4 n + i holds
    // K index 8 n + 4 h + i (n < 4, h < 2, i < 4), the order in which the tensor-memory decode kernel widens a packed
    // tile into its operand rows.
    bool interleaved = false;
};


// the 8 values of this lane (k0 = 256 sb + 8 lane, zero beyond K) -> planes, group sums, chunk scale
__device__ __forceinline__ void xprep_convert_vals(const float (&v)[8], int sb, int lane, const XqRow &dst) {
    const int64_t k0 = (int64_t)sb * TILE_K + 8 * lane;
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
    if (dst.interleaved) {
        // this lane holds K indices 8 n .. 8 n + 7 of its sub-block, n = lane & 3: h = 0 for the first four, 1 for the rest
        const int64_t seg = (int64_t)sb * TILE_K + 32 * (lane >> 2) + 4 * (lane & 3);
        *reinterpret_cast<uint32_t *>(dst.hi + seg) = hiw[0];
        *reinterpret_cast<uint32_t *>(dst.hi + seg + 16) = hiw[1];
        *reinterpret_cast<uint32_t *>(dst.lo + seg) = low[0];
        *reinterpret_cast<uint32_t *>(dst.lo + seg + 16) = low[1];
    } else {
        *reinterpret_cast<uint2 *>(dst.hi + k0) = make_uint2(hiw[0], hiw[1]);
        *reinterpret_cast<uint2 *>(dst.lo + k0) = make_uint2(low[0], low[1]);
    }
    const int s16 = s + __shfl_xor_sync(0xffffffffu, s, 1);
    const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);
    if ((lane & 1) == 0) dst.sum16[sb * 16 + (lane >> 1)] = (float)s16;
    if ((lane & 3) == 0) dst.sum32[sb * 8 + (lane >> 2)] = (float)s32;
    if (lane == 0) dst.sx[sb] = amax > 1e-20f ? amax * (1.0f / (float)XQ_MAX) : 0.f;
}

}  // namespace ttq
