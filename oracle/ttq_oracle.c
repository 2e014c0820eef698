/*
 * ttq_oracle.c -- CPU restatement of the quantized-linear path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker the CUDA library is compared against.  It is never linked into,
 * imported by, or executed from the product path; only the test-suite, the smoke check and the
 * CPU-baseline leg of the benchmark may load it.
 *
 * What it restates
 * ----------------
 *  - Operator semantics: y = x . W^T + b with W stored [out_features, in_features] and all leading
 *    dimensions of x flattened to M rows, as in the reference's
 *    workspace/transformers/src/layers/linear.nim:14-57 (Linear.init / Linear.forward) which
 *    forwards to ATen's linear (workspace/libtorch/src/abi/neural_nets.nim:64-81).
 *  - silu_and_mul: out = silu(x[..., :H]) * x[..., H:], the first half is the gate
 *    (workspace/transformers/src/kernels/activations.nim:14-38), used between the fused gate|up
 *    projection and the down projection (workspace/transformers/src/layers/mlp.nim:31-60).
 *  - Block formats: the reference tree holds NO quantized format, quantizer or dequantizer.  The
 *    three block layouts below (Q8_0 34 B / 32 weights, Q4_K 144 B / 256, Q6_K 210 B / 256) follow
 *    the publicly documented GGUF/ggml bit layout.  The algorithm lives in a project that is not a
 *    dependency of the reference; the independent witness used to pin this file is the PyPI package
 *    `gguf` 0.19.0 (gguf/quants.py), whose outputs are committed as fixtures under tests/golden/.
 *
 * PARITY UNPINNED against the reference: no test, golden vector or fixture of the reference pins a
 * quantized result (its only layer fixtures need a weight file that is not distributed).  What IS
 * pinned: dequantization of all three formats and the Q8_0 quantizer, bit-exact against the `gguf`
 * package; the dense operator against ATen linear (the call the reference makes).
 *
 * Numerics: dequantization returns fp32 and is exact up to the single rounding of the Q4_K subtract
 * (d*sc*q and dmin*m are exactly representable); matmuls accumulate in fp64 and round once to fp32.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define TTQ_REF_Q8_0 0
#define TTQ_REF_Q4_K 1
#define TTQ_REF_Q6_K 2

#define TTQ_REF_BF16 0
#define TTQ_REF_F16 1
#define TTQ_REF_F32 2

/* ---------------------------------------------------------------- scalar conversions */

static inline float bits_to_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* IEEE binary16 -> binary32, exact (subnormals, inf and nan included). */
float ttq_ref_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) return bits_to_f32(sign);
        /* subnormal: man * 2^-24 */
        float v = (float)man * (1.0f / 16777216.0f);
        return sign ? -v : v;
    }
    if (exp == 31) return bits_to_f32(sign | 0x7f800000u | (man << 13));
    return bits_to_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* binary32 -> binary16, round to nearest even. */
uint16_t ttq_ref_f32_to_f16(float f) {
    uint32_t x = f32_to_bits(f);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((absx > 0x7f800000u) ? 0x200u : 0u));
    }
    if (absx >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* rounds to inf (>= 65520) */
    if (absx < 0x33000001u) return sign;                           /* rounds to zero (<= 2^-25) */
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { shift = 13 + (-14 - e); base = 0; }
    else { shift = 13; base = (uint32_t)(e + 15) << 10; m &= 0x7fffffu; }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    return (uint16_t)(sign | (base + q)); /* a carry out of the mantissa bumps the exponent */
}

float ttq_ref_bf16_to_f32(uint16_t b) { return bits_to_f32((uint32_t)b << 16); }

uint16_t ttq_ref_f32_to_bf16(float f) {
    uint32_t x = f32_to_bits(f);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40u);
    uint32_t lsb = (x >> 16) & 1u;
    return (uint16_t)((x + 0x7fffu + lsb) >> 16);
}

static inline double load_act(const void *x, int dtype, int64_t i) {
    switch (dtype) {
    case TTQ_REF_BF16: return (double)ttq_ref_bf16_to_f32(((const uint16_t *)x)[i]);
    case TTQ_REF_F16: return (double)ttq_ref_f16_to_f32(((const uint16_t *)x)[i]);
    default: return (double)((const float *)x)[i];
    }
}

/* ---------------------------------------------------------------- format table */

int64_t ttq_ref_block_elems(int fmt) { return fmt == TTQ_REF_Q8_0 ? 32 : 256; }
int64_t ttq_ref_block_bytes(int fmt) {
    return fmt == TTQ_REF_Q8_0 ? 34 : (fmt == TTQ_REF_Q4_K ? 144 : 210);
}

/* ---------------------------------------------------------------- dequantizers
 * Each takes `nblocks` canonical blocks and writes nblocks * block_elems floats. */

/* Q8_0: { fp16 d; int8 qs[32] }  ->  w[i] = d * qs[i] */
static void dequant_q8_0(const uint8_t *b, float *out) {
    uint16_t dh; memcpy(&dh, b, 2);
    float d = ttq_ref_f16_to_f32(dh);
    const int8_t *qs = (const int8_t *)(b + 2);
    for (int i = 0; i < 32; i++) out[i] = d * (float)qs[i];
}

/* Q4_K 6-bit scale/min unpack: 12 bytes hold 8 scales and 8 mins.
 * j < 4: sc = s[j] & 63, m = s[j+4] & 63
 * j >= 4: sc = (s[j+4] & 15) | ((s[j-4] >> 6) << 4),  m = (s[j+4] >> 4) | ((s[j] >> 6) << 4) */
static inline void q4k_scale_min(int j, const uint8_t *s, uint8_t *sc, uint8_t *m) {
    if (j < 4) { *sc = s[j] & 63; *m = s[j + 4] & 63; }
    else {
        *sc = (uint8_t)((s[j + 4] & 0x0f) | ((s[j - 4] >> 6) << 4));
        *m = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

/* Q4_K: { fp16 d; fp16 dmin; u8 scales[12]; u8 qs[128] }.  The 256 weights are 8 sub-blocks of
 * 32; bytes qs[32p .. 32p+31] hold sub-block 2p in their low nibbles and 2p+1 in their high
 * nibbles.  w = (d * sc_j) * q - (dmin * m_j). */
static void dequant_q4_k(const uint8_t *b, float *out) {
    uint16_t dh, mh; memcpy(&dh, b, 2); memcpy(&mh, b + 2, 2);
    float d = ttq_ref_f16_to_f32(dh), dmin = ttq_ref_f16_to_f32(mh);
    const uint8_t *s = b + 4, *qs = b + 16;
    for (int p = 0; p < 4; p++) {
        uint8_t sc, m;
        q4k_scale_min(2 * p, s, &sc, &m);
        float d1 = d * (float)sc, m1 = dmin * (float)m;
        q4k_scale_min(2 * p + 1, s, &sc, &m);
        float d2 = d * (float)sc, m2 = dmin * (float)m;
        for (int l = 0; l < 32; l++) out[64 * p + l] = d1 * (float)(qs[32 * p + l] & 0x0f) - m1;
        for (int l = 0; l < 32; l++) out[64 * p + 32 + l] = d2 * (float)(qs[32 * p + l] >> 4) - m2;
    }
}

/* Q6_K: { u8 ql[128]; u8 qh[64]; i8 scales[16]; fp16 d }.  16 sub-blocks of 16 weights, 6-bit
 * quants stored as low 4 bits (ql) + high 2 bits (qh), offset by 32.  w = d * sc * (q - 32). */
static void dequant_q6_k(const uint8_t *b, float *out) {
    const uint8_t *ql = b, *qh = b + 128;
    const int8_t *sc = (const int8_t *)(b + 192);
    uint16_t dh; memcpy(&dh, b + 208, 2);
    float d = ttq_ref_f16_to_f32(dh);
    for (int half = 0; half < 2; half++) {
        for (int l = 0; l < 32; l++) {
            int is = l / 16;
            int q1 = (int)((ql[l] & 0x0f) | (((qh[l] >> 0) & 3) << 4)) - 32;
            int q2 = (int)((ql[l + 32] & 0x0f) | (((qh[l] >> 2) & 3) << 4)) - 32;
            int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            out[l] = d * (float)sc[is + 0] * (float)q1;
            out[l + 32] = d * (float)sc[is + 2] * (float)q2;
            out[l + 64] = d * (float)sc[is + 4] * (float)q3;
            out[l + 96] = d * (float)sc[is + 6] * (float)q4;
        }
        out += 128; ql += 64; qh += 32; sc += 8;
    }
}

static inline void dequant_block(int fmt, const uint8_t *b, float *out) {
    if (fmt == TTQ_REF_Q8_0) dequant_q8_0(b, out);
    else if (fmt == TTQ_REF_Q4_K) dequant_q4_k(b, out);
    else dequant_q6_k(b, out);
}

int ttq_ref_dequantize(int fmt, const uint8_t *blocks, int64_t nblocks, float *out) {
    if (fmt < 0 || fmt > 2) return 1;
    const int64_t be = ttq_ref_block_elems(fmt), bb = ttq_ref_block_bytes(fmt);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < nblocks; i++) dequant_block(fmt, blocks + i * bb, out + i * be);
    return 0;
}

/* ---------------------------------------------------------------- quantizers
 * Bit-exactness of the product is defined on dequantization of GIVEN bytes, so any valid encoder
 * serves.  Q8_0 follows the published round-to-nearest recipe (d = amax/127, q = roundf(x/d)) and is
 * pinned against the witness package; Q4_K and Q6_K use a direct min/max affine fit (no search). */

static inline float roundf_away(float v) { return roundf(v); }
static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

static void quant_q8_0(const float *x, uint8_t *b) {
    float amax = 0.0f;
    for (int i = 0; i < 32; i++) { float a = fabsf(x[i]); if (a > amax) amax = a; }
    float d = amax / 127.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    uint16_t dh = ttq_ref_f32_to_f16(d);
    memcpy(b, &dh, 2);
    int8_t *qs = (int8_t *)(b + 2);
    for (int i = 0; i < 32; i++) qs[i] = (int8_t)roundf_away(x[i] * id);
}

static void quant_q4_k(const float *x, uint8_t *b) {
    float scale[8], mn[8];
    float max_scale = 0.0f, max_min = 0.0f;
    for (int j = 0; j < 8; j++) {
        float lo = 0.0f, hi = 0.0f; /* the affine range always contains 0: min offset >= 0 */
        for (int l = 0; l < 32; l++) {
            float v = x[32 * j + l];
            if (v < lo) lo = v;
            if (v > hi) hi = v;
        }
        mn[j] = -lo;
        scale[j] = (hi - lo) / 15.0f;
        if (scale[j] > max_scale) max_scale = scale[j];
        if (mn[j] > max_min) max_min = mn[j];
    }
    uint16_t dh = ttq_ref_f32_to_f16(max_scale / 63.0f), mh = ttq_ref_f32_to_f16(max_min / 63.0f);
    float d = ttq_ref_f16_to_f32(dh), dmin = ttq_ref_f16_to_f32(mh);
    uint8_t sc[8], m[8];
    for (int j = 0; j < 8; j++) {
        sc[j] = (uint8_t)clampi(d > 0.0f ? (int)lrintf(scale[j] / d) : 0, 0, 63);
        m[j] = (uint8_t)clampi(dmin > 0.0f ? (int)lrintf(mn[j] / dmin) : 0, 0, 63);
    }
    memset(b, 0, 144);
    memcpy(b, &dh, 2); memcpy(b + 2, &mh, 2);
    uint8_t *s = b + 4, *qs = b + 16;
    for (int j = 0; j < 4; j++) {
        s[j] = (uint8_t)((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
        s[j + 4] = (uint8_t)((m[j] & 63) | ((m[j + 4] >> 4) << 6));
        s[j + 8] = (uint8_t)((sc[j + 4] & 0x0f) | ((m[j + 4] & 0x0f) << 4));
    }
    for (int j = 0; j < 8; j++) {
        float ds = d * (float)sc[j], dm = dmin * (float)m[j];
        for (int l = 0; l < 32; l++) {
            int q = ds > 0.0f ? (int)lrintf((x[32 * j + l] + dm) / ds) : 0;
            q = clampi(q, 0, 15);
            int p = j / 2;
            if (j & 1) qs[32 * p + l] |= (uint8_t)(q << 4);
            else qs[32 * p + l] |= (uint8_t)q;
        }
    }
}

static void quant_q6_k(const float *x, uint8_t *b) {
    float s[16], max_s = 0.0f;
    for (int j = 0; j < 16; j++) {
        float amax = 0.0f;
        for (int l = 0; l < 16; l++) { float a = fabsf(x[16 * j + l]); if (a > amax) amax = a; }
        s[j] = amax / 31.0f;
        if (s[j] > max_s) max_s = s[j];
    }
    uint16_t dh = ttq_ref_f32_to_f16(max_s / 127.0f);
    float d = ttq_ref_f16_to_f32(dh);
    memset(b, 0, 210);
    uint8_t *ql = b, *qh = b + 128;
    int8_t *sc = (int8_t *)(b + 192);
    memcpy(b + 208, &dh, 2);
    uint8_t q[256];
    for (int j = 0; j < 16; j++) {
        int isc = clampi(d > 0.0f ? (int)lrintf(s[j] / d) : 0, 0, 127);
        sc[j] = (int8_t)isc;
        float ds = d * (float)isc;
        for (int l = 0; l < 16; l++) {
            int v = ds > 0.0f ? (int)lrintf(x[16 * j + l] / ds) : 0;
            q[16 * j + l] = (uint8_t)(clampi(v, -32, 31) + 32);
        }
    }
    for (int half = 0; half < 2; half++) {
        const uint8_t *qq = q + 128 * half;
        for (int l = 0; l < 32; l++) {
            ql[64 * half + l] = (uint8_t)((qq[l] & 0x0f) | ((qq[l + 64] & 0x0f) << 4));
            ql[64 * half + l + 32] = (uint8_t)((qq[l + 32] & 0x0f) | ((qq[l + 96] & 0x0f) << 4));
            qh[32 * half + l] = (uint8_t)((qq[l] >> 4) | ((qq[l + 32] >> 4) << 2) |
                                          ((qq[l + 64] >> 4) << 4) | ((qq[l + 96] >> 4) << 6));
        }
    }
}

int ttq_ref_quantize(int fmt, const float *w, int64_t nelems, uint8_t *out) {
    if (fmt < 0 || fmt > 2) return 1;
    const int64_t be = ttq_ref_block_elems(fmt), bb = ttq_ref_block_bytes(fmt);
    if (nelems % be) return 2;
    const int64_t nb = nelems / be;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < nb; i++) {
        if (fmt == TTQ_REF_Q8_0) quant_q8_0(w + i * be, out + i * bb);
        else if (fmt == TTQ_REF_Q4_K) quant_q4_k(w + i * be, out + i * bb);
        else quant_q6_k(w + i * be, out + i * bb);
    }
    return 0;
}

/* ---------------------------------------------------------------- the operator
 * y[m][n] = sum_k x[m][k] * W[n][k] + bias[n]      (linear.nim:45-57; W is [N][K])
 * blocks: canonical row-major [N][K/block_elems] blocks.  x: [M][ldx] of x_dtype.  y: fp32 [M][ldy].
 * Accumulation in fp64, one rounding to fp32 at the end (the parity target). */
int ttq_ref_linear(int fmt, const uint8_t *blocks, int64_t N, int64_t K, const void *x, int x_dtype,
                   int64_t M, int64_t ldx, const float *bias, float *y, int64_t ldy) {
    if (fmt < 0 || fmt > 2) return 1;
    const int64_t be = ttq_ref_block_elems(fmt), bb = ttq_ref_block_bytes(fmt);
    if (K % be) return 2;
    const int64_t bpr = K / be;
    double *xd = (double *)malloc(sizeof(double) * (size_t)(M * K));
    if (!xd) return 3;
    for (int64_t m = 0; m < M; m++)
        for (int64_t k = 0; k < K; k++) xd[m * K + k] = load_act(x, x_dtype, m * ldx + k);
#pragma omp parallel
    {
        float *row = (float *)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static)
        for (int64_t n = 0; n < N; n++) {
            for (int64_t i = 0; i < bpr; i++) dequant_block(fmt, blocks + (n * bpr + i) * bb, row + i * be);
            for (int64_t m = 0; m < M; m++) {
                const double *xm = xd + m * K;
                double acc = 0.0;
                for (int64_t k = 0; k < K; k++) acc += xm[k] * (double)row[k];
                if (bias) acc += (double)bias[n];
                y[m * ldy + n] = (float)acc;
            }
        }
        free(row);
    }
    free(xd);
    return 0;
}

/* Same operator with fp32 accumulation, dequantizing one block at a time next to the dot product:
 * the form a CPU implementation of the fused path would take.  Used only as the timed CPU baseline
 * ("port"); it reads the packed bytes exactly once per call. */
int ttq_ref_linear_fast(int fmt, const uint8_t *blocks, int64_t N, int64_t K, const void *x, int x_dtype,
                        int64_t M, int64_t ldx, const float *bias, float *y, int64_t ldy) {
    if (fmt < 0 || fmt > 2) return 1;
    const int64_t be = ttq_ref_block_elems(fmt), bb = ttq_ref_block_bytes(fmt);
    if (K % be) return 2;
    const int64_t bpr = K / be;
    float *xf = (float *)malloc(sizeof(float) * (size_t)(M * K));
    if (!xf) return 3;
    for (int64_t m = 0; m < M; m++)
        for (int64_t k = 0; k < K; k++) xf[m * K + k] = (float)load_act(x, x_dtype, m * ldx + k);
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; n++) {
        float buf[256];
        for (int64_t m = 0; m < M; m++) y[m * ldy + n] = bias ? bias[n] : 0.0f;
        for (int64_t i = 0; i < bpr; i++) {
            dequant_block(fmt, blocks + (n * bpr + i) * bb, buf);
            for (int64_t m = 0; m < M; m++) {
                const float *xm = xf + m * K + i * be;
                float acc = 0.0f;
                for (int64_t k = 0; k < be; k++) acc += xm[k] * buf[k];
                y[m * ldy + n] += acc;
            }
        }
    }
    free(xf);
    return 0;
}

/* Dense operator on fp32 weights (the reference's literal computation), fp64 accumulation. */
int ttq_ref_linear_dense(const float *W, int64_t N, int64_t K, const void *x, int x_dtype, int64_t M,
                         int64_t ldx, const float *bias, float *y, int64_t ldy) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; n++) {
        for (int64_t m = 0; m < M; m++) {
            double acc = 0.0;
            for (int64_t k = 0; k < K; k++) acc += load_act(x, x_dtype, m * ldx + k) * (double)W[n * K + k];
            if (bias) acc += (double)bias[n];
            y[m * ldy + n] = (float)acc;
        }
    }
    return 0;
}

/* silu_and_mul (activations.nim:14-38): in [M][2H] fp32 -> out [M][H]; gate = first half. */
int ttq_ref_silu_and_mul(const float *in, int64_t M, int64_t H, float *out) {
    for (int64_t m = 0; m < M; m++)
        for (int64_t h = 0; h < H; h++) {
            double g = (double)in[m * 2 * H + h], u = (double)in[m * 2 * H + H + h];
            out[m * H + h] = (float)((g / (1.0 + exp(-g))) * u);
        }
    return 0;
}

int ttq_ref_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
