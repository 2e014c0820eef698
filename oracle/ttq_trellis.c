/*
 * ttq_trellis.c -- CPU statement of the trellis-coded 3-bit weight format (TQ3).  TEST INFRASTRUCTURE ONLY:
 * loaded by the test-suite, the smoke check and the CPU-baseline leg of the benchmark, never by the product.
 *
 * PARITY UNPINNED.  The reference tree has no quantized linear at all; its only trace of a trellis-coded
 * format is a model configuration fixture naming an "exl3" quantization
 * (tests/fixtures/configs/config-GLM-4.7-EXL3-3.84bpw.json:43-54).  No codec source, test vector or third-party
 * implementation of that format exists in the build image, so the format below is this project's own
 * definition in the same family (16x16 tiles at 3 bits per weight, Hadamard-rotated input and output);
 * checkpoints of any other tool are NOT interchangeable with it.  What the tests pin: encode -> decode
 * self-consistency, the device decode bit-exact against ttq_tq3_decode, and the device matmul against
 * ttq_tq3_linear (fp64 accumulation).
 *
 * Format (W is [N][K], N and K multiples of 128), one byte buffer of N*K*3/8 + 2N + K/8 bytes:
 *   tiles     [N/16][K/16][96 B]  one 768-bit little-endian stream per 16x16 tile
 *   out_scale [N] fp16            per output row, sign included
 *   in_sign   [K/8] bytes         bit (k & 7) of byte k >> 3: 1 = the input channel is negated
 * Weight t = 16*r + c of a tile (r: row inside the tile, c: column) is coded by the 16-bit window that starts
 * at bit 3t of the tile's stream, zero-extended past bit 767:
 *   state = (stream >> 3t) & 0xFFFF,   h = state * 2654435761 (mod 2^32),
 *   q[n][k] = (byte0(h) + byte1(h) + byte2(h) + byte3(h) - 510) * (1 / 147.8)        (about N(0,1))
 * so each weight owns the 3 low bits of its window and shares the other 13 with the 5 weights that follow
 * it: a sliding-window ("bit-shift") trellis, decodable at any position without running the chain.
 * The matrix the operator applies is
 *   W = diag(out_scale) . H_N . q . H_K . diag(in_sign)
 * with H the block-diagonal, orthonormal Sylvester-Hadamard transform on blocks of 128 (symmetric, its own
 * inverse), i.e.   y = out_scale * H_N( q . H_K(in_sign * x) ) + bias.
 *
 * Operator semantics (W [out][in], y = x . W^T + b, leading dimensions flattened to M) follow the reference's
 * Linear.forward, workspace/transformers/src/layers/linear.nim:45-57.
 *
 * Encoder: out_scale[n] = +-rms(W[n, :]) (sign and in_sign from a seeded generator), target
 * T = H_N . diag(1/out_scale) . W . diag(in_sign) . H_K, then per tile an exact Viterbi search over the
 * 2^13 contexts x 8 symbols of the trellis, run from weight 255 down to weight 0 (the window of weight 255
 * holds only its own 3 bits, so the chain starts from a known all-zero context).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

float ttq_ref_f16_to_f32(uint16_t h);
uint16_t ttq_ref_f32_to_f16(float f);
float ttq_ref_bf16_to_f32(uint16_t b);

#define TQ3_TILE_BYTES 96
#define TQ3_HAD 128
static const float TQ3_UNIT = 1.0f / 147.8f;

int64_t ttq_tq3_packed_bytes(int64_t N, int64_t K) { return N * K * 3 / 8 + 2 * N + K / 8; }

static inline float tq3_value(uint32_t state) {
    const uint32_t h = state * 2654435761u;
    const int sum = (int)(h & 0xff) + (int)((h >> 8) & 0xff) + (int)((h >> 16) & 0xff) + (int)(h >> 24);
    return (float)(sum - 510) * TQ3_UNIT;
}

static inline uint32_t tq3_window(const uint8_t *tile, int t) {
    const int bit = 3 * t, byte = bit >> 3;
    uint32_t v = 0;
    for (int i = 0; i < 3; i++)
        if (byte + i < TQ3_TILE_BYTES) v |= (uint32_t)tile[byte + i] << (8 * i);
    return (v >> (bit & 7)) & 0xffffu;
}

/* q [N][K] fp32: the decoded codes, before rotations and scales (bit-exact target of the device decode) */
int ttq_tq3_decode(const uint8_t *packed, int64_t N, int64_t K, float *out) {
    if (N % 128 || K % 128) return 1;
    const int64_t tk = K / 16;
#pragma omp parallel for schedule(static)
    for (int64_t tile = 0; tile < (N / 16) * tk; tile++) {
        const uint8_t *tb = packed + tile * TQ3_TILE_BYTES;
        const int64_t n0 = (tile / tk) * 16, k0 = (tile % tk) * 16;
        for (int t = 0; t < 256; t++) out[(n0 + t / 16) * K + k0 + t % 16] = tq3_value(tq3_window(tb, t));
    }
    return 0;
}

/* in-place orthonormal Hadamard transform on consecutive blocks of 128, stride 1 */
static void had128(double *v, int64_t n) {
    for (int64_t b = 0; b < n; b += TQ3_HAD) {
        for (int h = 1; h < TQ3_HAD; h <<= 1)
            for (int i = 0; i < TQ3_HAD; i += h << 1)
                for (int j = i; j < i + h; j++) {
                    const double a = v[b + j], c = v[b + j + h];
                    v[b + j] = a + c;
                    v[b + j + h] = a - c;
                }
        for (int i = 0; i < TQ3_HAD; i++) v[b + i] *= 0.08838834764831845; /* 1 / sqrt(128) */
    }
}

static inline double act_at(const void *x, int dtype, int64_t i) {
    if (dtype == 0) return (double)ttq_ref_bf16_to_f32(((const uint16_t *)x)[i]);
    if (dtype == 1) return (double)ttq_ref_f16_to_f32(((const uint16_t *)x)[i]);
    return (double)((const float *)x)[i];
}

/* y [M][ldy] fp32 = out_scale * H_N(q . H_K(in_sign * x)) + bias, fp64 throughout, one rounding at the end */
int ttq_tq3_linear(const uint8_t *packed, int64_t N, int64_t K, const void *x, int x_dtype, int64_t M, int64_t ldx,
                   const float *bias, float *y, int64_t ldy) {
    if (N % 128 || K % 128) return 1;
    float *q = (float *)malloc(sizeof(float) * (size_t)N * K);
    double *x1 = (double *)malloc(sizeof(double) * (size_t)M * K);
    double *y1 = (double *)malloc(sizeof(double) * (size_t)M * N);
    if (!q || !x1 || !y1) { free(q); free(x1); free(y1); return 2; }
    ttq_tq3_decode(packed, N, K, q);
    const uint16_t *oscale = (const uint16_t *)(packed + N * K * 3 / 8);
    const uint8_t *isign = packed + N * K * 3 / 8 + 2 * N;
    for (int64_t m = 0; m < M; m++) {
        for (int64_t k = 0; k < K; k++) {
            const double v = act_at(x, x_dtype, m * ldx + k);
            x1[m * K + k] = ((isign[k >> 3] >> (k & 7)) & 1) ? -v : v;
        }
        had128(x1 + m * K, K);
    }
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; n++)
        for (int64_t m = 0; m < M; m++) {
            double acc = 0.0;
            for (int64_t k = 0; k < K; k++) acc += (double)q[n * K + k] * x1[m * K + k];
            y1[m * N + n] = acc;
        }
    for (int64_t m = 0; m < M; m++) {
        had128(y1 + m * N, N);
        for (int64_t n = 0; n < N; n++)
            y[m * ldy + n] = (float)(y1[m * N + n] * (double)ttq_ref_f16_to_f32(oscale[n]) + (bias ? (double)bias[n] : 0.0));
    }
    free(q); free(x1); free(y1);
    return 0;
}

/* The dense matrix the operator applies, W [N][K] fp32 (for error measurements of the encoder). */
int ttq_tq3_effective_weight(const uint8_t *packed, int64_t N, int64_t K, float *W) {
    if (N % 128 || K % 128) return 1;
    float *q = (float *)malloc(sizeof(float) * (size_t)N * K);
    double *t = (double *)malloc(sizeof(double) * (size_t)N * K);
    double *col = (double *)malloc(sizeof(double) * (size_t)N);
    if (!q || !t || !col) { free(q); free(t); free(col); return 2; }
    ttq_tq3_decode(packed, N, K, q);
    const uint16_t *oscale = (const uint16_t *)(packed + N * K * 3 / 8);
    const uint8_t *isign = packed + N * K * 3 / 8 + 2 * N;
    for (int64_t i = 0; i < N * K; i++) t[i] = q[i];
    for (int64_t n = 0; n < N; n++) had128(t + n * K, K); /* q . H_K */
    for (int64_t k = 0; k < K; k++) {                      /* H_N . (.) */
        for (int64_t n = 0; n < N; n++) col[n] = t[n * K + k];
        had128(col, N);
        const double s = ((isign[k >> 3] >> (k & 7)) & 1) ? -1.0 : 1.0;
        for (int64_t n = 0; n < N; n++) W[n * K + k] = (float)(col[n] * (double)ttq_ref_f16_to_f32(oscale[n]) * s);
    }
    free(q); free(t); free(col);
    return 0;
}

/* exact Viterbi search of one tile: target[256] -> 96 bytes; returns the squared error */
static double encode_tile(const float *target, const float *table, uint8_t *out, float *cost, float *ncost, uint8_t *choice) {
    enum { CTX = 8192 };
    /* cost[c]: best error of weights t+1..255 given that the 13 bits above weight t's symbol are c */
    for (int c = 0; c < CTX; c++) cost[c] = c == 0 ? 0.f : INFINITY;
    for (int t = 255; t >= 0; t--) {
        for (int c = 0; c < CTX; c++) ncost[c] = INFINITY;
        uint8_t *ch = choice + (size_t)t * CTX;
        for (int c = 0; c < CTX; c++) {
            if (cost[c] == INFINITY) continue;
            for (int s = 0; s < 8; s++) {
                const uint32_t state = ((uint32_t)c << 3) | (uint32_t)s;
                const float d = table[state] - target[t];
                const float e = cost[c] + d * d;
                const int nc = (int)(state & (CTX - 1)); /* context seen by weight t-1 */
                if (e < ncost[nc]) {
                    ncost[nc] = e;
                    ch[nc] = (uint8_t)(c >> 10); /* with nc, this restores c: c = (top << 10) | (nc >> 3) */
                }
            }
        }
        float *tmp = cost; cost = ncost; ncost = tmp;
    }
    int best = 0;
    for (int c = 1; c < CTX; c++)
        if (cost[c] < cost[best]) best = c;
    const double err = cost[best];
    memset(out, 0, TQ3_TILE_BYTES);
    int nc = best;
    for (int t = 0; t < 256; t++) {
        /* nc = low 13 bits of weight t's state: its symbol is nc & 7 */
        const int sym = nc & 7, bit = 3 * t;
        for (int b = 0; b < 3; b++)
            if ((sym >> b) & 1) out[(bit + b) >> 3] |= (uint8_t)(1u << ((bit + b) & 7));
        const int top = choice[(size_t)t * CTX + nc];
        nc = (top << 10) | (nc >> 3); /* context of weight t = low 13 bits of weight t+1's state */
    }
    return err;
}

static inline uint32_t lcg(uint32_t *s) { *s = *s * 1664525u + 1013904223u; return *s >> 8; }

/* W [N][K] fp32 -> packed; returns 0, *mse_out = mean squared error of the codes against the rotated,
 * normalised target (about 0.02-0.03 for Gaussian weights at 3 bits) */
int ttq_tq3_encode(const float *W, int64_t N, int64_t K, uint32_t seed, uint8_t *packed, double *mse_out) {
    if (N % 128 || K % 128) return 1;
    uint16_t *oscale = (uint16_t *)(packed + N * K * 3 / 8);
    uint8_t *isign = packed + N * K * 3 / 8 + 2 * N;
    double *t = (double *)malloc(sizeof(double) * (size_t)N * K);
    double *col = (double *)malloc(sizeof(double) * (size_t)N);
    if (!t || !col) { free(t); free(col); return 2; }
    uint32_t rng = seed * 2654435761u + 12345u;
    memset(isign, 0, (size_t)(K / 8));
    for (int64_t k = 0; k < K; k++)
        if (lcg(&rng) & 1) isign[k >> 3] |= (uint8_t)(1u << (k & 7));
    for (int64_t n = 0; n < N; n++) {
        double ss = 0.0;
        for (int64_t k = 0; k < K; k++) ss += (double)W[n * K + k] * W[n * K + k];
        float r = (float)sqrt(ss / (double)K);
        if (!(r > 0.f)) r = 1.f;
        if (lcg(&rng) & 1) r = -r;
        oscale[n] = ttq_ref_f32_to_f16(r);
        if ((oscale[n] & 0x7fff) == 0) oscale[n] = (uint16_t)((oscale[n] & 0x8000) | 0x0001); /* never a zero scale */
        const double inv = 1.0 / (double)ttq_ref_f16_to_f32(oscale[n]);
        for (int64_t k = 0; k < K; k++) {
            const double s = ((isign[k >> 3] >> (k & 7)) & 1) ? -1.0 : 1.0;
            t[n * K + k] = (double)W[n * K + k] * inv * s;
        }
        had128(t + n * K, K);
    }
    for (int64_t k = 0; k < K; k++) {
        for (int64_t n = 0; n < N; n++) col[n] = t[n * K + k];
        had128(col, N);
        for (int64_t n = 0; n < N; n++) t[n * K + k] = col[n];
    }
    const int64_t tk = K / 16, tiles = (N / 16) * tk;
    double total = 0.0;
    float *table = (float *)malloc(sizeof(float) * 65536);
    if (!table) { free(t); free(col); return 2; }
    for (uint32_t st = 0; st < 65536; st++) table[st] = tq3_value(st);
#pragma omp parallel reduction(+ : total)
    {
        float *cost = (float *)malloc(sizeof(float) * 8192 * 2);
        uint8_t *choice = (uint8_t *)malloc((size_t)256 * 8192);
        float target[256];
#pragma omp for schedule(dynamic, 1)
        for (int64_t tile = 0; tile < tiles; tile++) {
            const int64_t n0 = (tile / tk) * 16, k0 = (tile % tk) * 16;
            for (int i = 0; i < 256; i++) target[i] = (float)t[(n0 + i / 16) * K + k0 + i % 16];
            total += encode_tile(target, table, packed + tile * TQ3_TILE_BYTES, cost, cost + 8192, choice);
        }
        free(cost); free(choice);
    }
    if (mse_out) *mse_out = total / (double)(N * K);
    free(t); free(col); free(table);
    return 0;
}
