// Trellis-coded 3-bit weights (TQ3): decode, Hadamard rotations and the decode-and-multiply kernel.
//
// Format (see include/ttq.h): W [N][K], N and K multiples of 128; one buffer of
//   tiles [N/16][K/16][96 B] | out_scale [N] fp16 | in_sign [K/8] bytes.
// Weight t = 16 r + c of a tile is coded by the 16-bit window at bit 3t of the tile's 768-bit stream
// (zero beyond the end): state -> h = state * 2654435761 -> q = (sum of the 4 bytes of h - 510) / 147.8.
// The operator is  y = out_scale * H_N( q . H_K(in_sign * x) ) + bias  with H the orthonormal Hadamard
// transform on blocks of 128.  The device keeps the buffer as it is: tiles of one 16-row band are
// contiguous along K, which is the order the kernels stream them in.
//
// Kernels
//   tq3_decode_kernel     q as fp32 [N][ld] (test hook, bit-exact) or as fp16 tile images for the plain GEMM
//   tq3_rotate_kernel     Hadamard-128 of activation rows (signs in, fp32 | fp16 out) and of result rows
//                         (scale and bias out); one warp per 128 block, four values per lane
//   tq3_mma_kernel<NA>    5 <= M <= 64: decoded weights as the B operand of mma.sync m16n8k16, every weight decoded once
//   tq3_gemv_kernel<MR>   M <= 4 rows per pass: one CTA per 16-row band, its 8 warps split K; a lane owns two
//                         rows of a tile (32 weights = 3 words of the stream), decodes each weight with one
//                         multiply and one byte-sum and accumulates in fp32
//
// The reference has no counterpart (a model configuration fixture names the format family only:
// tests/fixtures/configs/config-GLM-4.7-EXL3-3.84bpw.json:43-54).
#include "ttq_internal.cuh"

namespace ttq {
namespace {

constexpr float TQ3_UNIT = 1.0f / 147.8f;
constexpr int TQ3_TILE_BYTES = 96;

__device__ __forceinline__ int tq3_isum(uint32_t state) {
    const uint32_t h = state * 2654435761u;
    return (int)__dp4a(h, 0x01010101u, 0u) - 510;
}

// The 8 consecutive weights whose stream bits start at byte `bo` = 3 * (2 r + c / 8) of a tile (row r, columns
// c .. c + 7, c = 0 | 8): returns sum - 510 of each as an exact float.  Two aligned 32-bit loads cover the 37
// bits; the byte sum lands on the mantissa of 2^23 (the dp4a accumulator), so one subtraction replaces the
// integer-to-float conversion.
__device__ __forceinline__ void tq3_decode8(const uint8_t *tile, int bo, float (&f)[8]) {
    const int wo = bo & ~3, sh = (bo & 3) * 8;
    const uint32_t w0 = *reinterpret_cast<const uint32_t *>(tile + wo);
    const uint32_t w1 = wo + 4 < TQ3_TILE_BYTES ? *reinterpret_cast<const uint32_t *>(tile + wo + 4) : 0u;
    const uint32_t lo = __funnelshift_r(w0, w1, sh), hi = w1 >> sh;  // stream bits 8 bo .. 8 bo + 63 (zero-extended)
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t st = (3 * i + 16 <= 32 ? (lo >> (3 * i)) : __funnelshift_r(lo, hi, 3 * i)) & 0xffffu;
        f[i] = __int_as_float((int)__dp4a(st * 2654435761u, 0x01010101u, 0x4B000000u)) - 8389118.0f;  // 2^23 + 510
    }
}

__device__ __forceinline__ uint32_t tq3_window(const uint8_t *tile, int t) {
    const int bit = 3 * t, byte = bit >> 3;
    uint32_t v = 0;
#pragma unroll
    for (int i = 0; i < 3; i++)
        if (byte + i < TQ3_TILE_BYTES) v |= (uint32_t)tile[byte + i] << (8 * i);
    return (v >> (bit & 7)) & 0xffffu;
}

// IMAGES = false: out is float [N][ld];  true: out is the fp16 tile-image layout of the plain GEMM
// ([Kp/64][Np/8][1024 B], 128-byte swizzle, in-chunk K order 0 2 1 3 | 4 6 5 7), zero outside N x K.
template <bool IMAGES>
__global__ void __launch_bounds__(256) tq3_decode_kernel(const uint8_t *__restrict__ tiles, int64_t N, int64_t K, void *__restrict__ out,
                                                         int64_t ld, int64_t Np, int64_t Kp) {
    const int64_t tk = K / 16;
    if (!IMAGES) {
        const int64_t total = N * K;
        for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
            const int64_t n = e / K, k = e % K;
            const uint8_t *tb = tiles + ((n >> 4) * tk + (k >> 4)) * TQ3_TILE_BYTES;
            reinterpret_cast<float *>(out)[n * ld + k] = (float)tq3_isum(tq3_window(tb, (int)((n & 15) * 16 + (k & 15)))) * TQ3_UNIT;
        }
    } else {
        const int64_t total = Np * (Kp / 8);
        for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < total; c += (int64_t)gridDim.x * blockDim.x) {
            const int j = (int)(c & 7);
            const int64_t n = (c >> 3) % Np, it = (c >> 3) / Np;
            const int64_t k0 = (it >> 2) * 256 + 32 * j + 8 * (it & 3);  // 8 consecutive K: half a tile row
            float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (n < N && k0 < K)  // K is a multiple of 16: the 8 values are inside or outside together
                tq3_decode8(tiles + ((n >> 4) * tk + (k0 >> 4)) * TQ3_TILE_BYTES, 3 * (2 * (int)(n & 15) + (int)((k0 >> 3) & 1)), f);
            __half o[8];
#pragma unroll
            for (int q = 0; q < 8; q++) o[q] = __float2half_rn(f[(q & 4) + ((q & 1) << 1) + ((q & 2) >> 1)] * TQ3_UNIT);
            const int64_t dst = ((it * (Np >> 3) + (n >> 3)) << 10) + ((n & 7) << 7) + ((int64_t)(j ^ (int)(n & 7)) << 4);
            *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(out) + dst) = *reinterpret_cast<const uint4 *>(o);
        }
    }
}

// One warp per (row, block of 128): out = H128(in * sign) * scale + bias.
//   in:  [M][ld_in] of in_dt;  sign: bit per column or nullptr;  scale: fp16 per column or nullptr;
//   bias: per column of bias_dt or nullptr;  out: [M][ld_out] of out_dt, or (frag != 0, fp16, no scale / bias) the
//   A-operand fragments of mma.sync m16n8k16 for tq3_mma_kernel: [group of 16 rows][K tile of 16][lane 4g + t][register]
//   with register = (row >> 3 & 1) + 2 (k >> 3 & 1) holding columns 2t, 2t + 1 (+ 8) of row g (+ 8).
__global__ void __launch_bounds__(256) tq3_rotate_kernel(const void *__restrict__ in, int in_dt, int64_t M, int64_t C, int64_t ld_in,
                                                         const uint8_t *__restrict__ sign, const __half *__restrict__ scale,
                                                         const void *__restrict__ bias, int bias_dt, void *__restrict__ out, int out_dt,
                                                         int64_t ld_out, int frag) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int64_t blocks_per_row = C / 128, total = M * blocks_per_row;
    for (int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < total; w += ((int64_t)gridDim.x * blockDim.x) >> 5) {
        const int64_t m = w / blocks_per_row, c0 = (w % blocks_per_row) * 128 + 4 * lane;
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; i++) v[i] = load_as_float(in, in_dt, m * ld_in + c0 + i);
        if (sign != nullptr) {
            const uint32_t bits = (uint32_t)sign[c0 >> 3] >> (c0 & 7);
#pragma unroll
            for (int i = 0; i < 4; i++)
                if ((bits >> i) & 1) v[i] = -v[i];
        }
        // strides 1 and 2 inside the lane, 4 .. 64 across lanes
        float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
        v[0] = a + c; v[2] = a - c; v[1] = b + d; v[3] = b - d;
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float o = __shfl_xor_sync(0xffffffffu, v[i], s);
                v[i] = (lane & s) ? o - v[i] : v[i] + o;
            }
        }
        if (frag) {
            const int64_t kt = c0 >> 4;
            const int kk = (int)(c0 & 15), t0 = (kk & 7) >> 1, reg = (int)((m >> 3) & 1) + 2 * (kk >> 3);
            __half2 *dst = reinterpret_cast<__half2 *>(out) + ((((m >> 4) * (C >> 4) + kt) * 32 + 4 * (m & 7) + t0) * 4 + reg);
            dst[0] = __floats2half2_rn(v[0] * 0.08838834764831845f, v[1] * 0.08838834764831845f);
            dst[4] = __floats2half2_rn(v[2] * 0.08838834764831845f, v[3] * 0.08838834764831845f);  // next lane of the fragment
            continue;
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float r = v[i] * 0.08838834764831845f;
            if (scale != nullptr) r *= __half2float(scale[c0 + i]);
            if (bias != nullptr) r += load_as_float(bias, bias_dt, c0 + i);
            store_from_float(out, out_dt, m * ld_out + c0 + i, r);
        }
    }
}

// y1 [MR][N] (fp32) = q . x1^T for MR rows of x1 [.][K] (fp32, already rotated).
// One CTA per 16-row band, its 8 warps split K.  Per iteration a warp covers 4 tiles: lane (g, j) = (lane / 8,
// lane % 8) owns rows 2j and 2j+1 of tile g -- 32 weights = exactly three 32-bit words of the stream plus the
// 13 bits of the next word its last windows reach into.
template <int MR>
__global__ void __launch_bounds__(256) tq3_gemv_kernel(const uint8_t *__restrict__ tiles, int64_t N, int64_t K, const float *__restrict__ x1,
                                                       float *__restrict__ y1) {
    __shared__ float red[8][16][MR];
    grid_launch_dependents();
    grid_dependency_wait();  // the rotated activations come from the preceding kernel
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 3, j = lane & 7;
    const int64_t tk = K / 16, band = blockIdx.x;
    const uint8_t *band_base = tiles + band * tk * TQ3_TILE_BYTES;
    const int64_t t_begin = tk * warp / 8, t_end = tk * (warp + 1) / 8;
    float acc[MR][2];
#pragma unroll
    for (int m = 0; m < MR; m++) acc[m][0] = acc[m][1] = 0.f;
#pragma unroll 2
    for (int64_t t0 = t_begin; t0 < t_end; t0 += 4) {
        const int64_t tile = t0 + g;
        if (tile < t_end) {
            const uint32_t *tw = reinterpret_cast<const uint32_t *>(band_base + tile * TQ3_TILE_BYTES) + 3 * j;
            uint32_t w[5];
            w[0] = tw[0]; w[1] = tw[1]; w[2] = tw[2];
            w[3] = j < 7 ? tw[3] : 0u;  // the stream ends with the tile
            w[4] = 0u;
            float f[32];
#pragma unroll
            for (int i = 0; i < 32; i++) {
                const int word = (3 * i) >> 5, off = (3 * i) & 31;
                const uint32_t st = (off + 16 <= 32 ? (w[word] >> off) : __funnelshift_r(w[word], w[word + 1], off)) & 0xffffu;
                f[i] = __int_as_float((int)__dp4a(st * 2654435761u, 0x01010101u, 0x4B000000u)) - 8389118.0f;
            }
#pragma unroll
            for (int m = 0; m < MR; m++) {
                const float4 *xp = reinterpret_cast<const float4 *>(x1 + m * K + tile * 16);
                float s0 = acc[m][0], s1 = acc[m][1];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const float4 xv = __ldg(xp + q);
                    s0 = fmaf(f[4 * q], xv.x, s0); s0 = fmaf(f[4 * q + 1], xv.y, s0);
                    s0 = fmaf(f[4 * q + 2], xv.z, s0); s0 = fmaf(f[4 * q + 3], xv.w, s0);
                    s1 = fmaf(f[16 + 4 * q], xv.x, s1); s1 = fmaf(f[16 + 4 * q + 1], xv.y, s1);
                    s1 = fmaf(f[16 + 4 * q + 2], xv.z, s1); s1 = fmaf(f[16 + 4 * q + 3], xv.w, s1);
                }
                acc[m][0] = s0; acc[m][1] = s1;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MR; m++)
#pragma unroll
        for (int r = 0; r < 2; r++) {
            float s = acc[m][r];
            s += __shfl_xor_sync(0xffffffffu, s, 8);
            s += __shfl_xor_sync(0xffffffffu, s, 16);
            if (g == 0) red[warp][2 * j + r][m] = s;
        }
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * MR; i += blockDim.x) {
        const int r = i / MR, m = i % MR;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) s += red[w][r][m];
        y1[(int64_t)m * N + band * 16 + r] = s * TQ3_UNIT;
    }
}

// y1 [M][N] (fp32) = q . x1^T for M <= 16 NA rows of x1 [.][K] (fp16, already rotated) on tensor-core instructions
// (mma.sync m16n8k16, fp32 accumulate): the decoded weights are the B operand, so a lane decodes exactly the four
// weights of its fragment -- row g (first instruction) or g + 8 (second) of the tile, columns 2t, 2t+1, 2t+8,
// 2t+9 -- from the 64 stream bits that start at the row (48 bits per row; the windows of the last columns reach
// 13 bits into the next row, and past the end of the tile the stream is zero).  A decoded value is an exact
// integer in [-510, 510]: the byte sum of two weights lands on the mantissas of a {1024, 1024} fp16 pair through
// the dp4a accumulator, one HSUB2 removes 1024 + 510.  The activation rows are the A operand (16 rows per
// instruction; the rotation kernel writes them in fragment order, so a lane needs one 16-byte load per K tile).
// One CTA per 16-row band, its 8 warps split K; every weight is decoded once for all M rows.
template <int NA>
__global__ void __launch_bounds__(256) tq3_mma_kernel(const uint8_t *__restrict__ tiles, int64_t N, int64_t K, const __half *__restrict__ x1,
                                                      int M, float *__restrict__ y1) {
    __shared__ float red[8][NA * 16][16];  // [warp][activation row][weight row]
    grid_launch_dependents();
    grid_dependency_wait();  // the rotated activations come from the preceding kernel
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t tk = K / 16, band = blockIdx.x;
    const uint8_t *band_base = tiles + band * tk * TQ3_TILE_BYTES;
    const int64_t t_begin = tk * warp / 8, t_end = tk * (warp + 1) / 8;
    float c[NA][2][4];
#pragma unroll
    for (int a = 0; a < NA; a++)
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
            for (int i = 0; i < 4; i++) c[a][h][i] = 0.f;
    // row g starts at byte 6 g of the tile: word 6 g / 4 (rounded down), bit offset 0 or 16; rows g and g + 8 share it
    const int sh = (g & 1) * 16;
    const int w_lo = (6 * g) >> 2, w_hi = (6 * (g + 8)) >> 2;
    const uint32_t k1534 = 0x65FE65FEu;  // {1534, 1534} as fp16
    // activation fragments (written by the rotation kernel in fragment order): 16 bytes per lane and K tile; rows
    // beyond M hold stale data and are masked off
    const uint4 *xf[NA];
    uint32_t keep[NA][2];
#pragma unroll
    for (int a = 0; a < NA; a++) {
        xf[a] = reinterpret_cast<const uint4 *>(x1) + (int64_t)a * tk * 32 + lane;
        keep[a][0] = 16 * a + g < M ? 0xffffffffu : 0u;
        keep[a][1] = 16 * a + g + 8 < M ? 0xffffffffu : 0u;
    }
#pragma unroll 2
    for (int64_t tile = t_begin; tile < t_end; tile++) {
        const uint32_t *tw = reinterpret_cast<const uint32_t *>(band_base + tile * TQ3_TILE_BYTES);
        uint32_t b[2][2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int w0 = h == 0 ? w_lo : w_hi;
            const uint32_t q0 = __ldg(tw + w0), q1 = w0 + 1 < 24 ? __ldg(tw + w0 + 1) : 0u, q2 = w0 + 2 < 24 ? __ldg(tw + w0 + 2) : 0u;
            // the row's 64 stream bits, then shifted so that this lane's first window starts at bit 0
            uint32_t lo = __funnelshift_r(q0, q1, sh), hi = __funnelshift_r(q1, q2, sh);
            const int o = 6 * t;
            lo = __funnelshift_r(lo, hi, o);
            hi >>= o;
            const uint32_t s0 = lo & 0xffffu, s1 = (lo >> 3) & 0xffffu;
            const uint32_t s2 = __funnelshift_r(lo, hi, 24) & 0xffffu, s3 = __funnelshift_r(lo, hi, 27) & 0xffffu;
            const uint32_t p0 = __dp4a(s0 * 2654435761u, 0x01010101u, 0x64006400u), p1 = __dp4a(s1 * 2654435761u, 0x01010101u, 0u);
            const uint32_t p2 = __dp4a(s2 * 2654435761u, 0x01010101u, 0x64006400u), p3 = __dp4a(s3 * 2654435761u, 0x01010101u, 0u);
            const uint32_t v0 = p0 + (p1 << 16), v1 = p2 + (p3 << 16);
            const __half2 d0 = __hsub2(*reinterpret_cast<const __half2 *>(&v0), *reinterpret_cast<const __half2 *>(&k1534));
            const __half2 d1 = __hsub2(*reinterpret_cast<const __half2 *>(&v1), *reinterpret_cast<const __half2 *>(&k1534));
            b[h][0] = *reinterpret_cast<const uint32_t *>(&d0);
            b[h][1] = *reinterpret_cast<const uint32_t *>(&d1);
        }
#pragma unroll
        for (int a = 0; a < NA; a++) {
            const uint4 xa = __ldg(xf[a] + tile * 32);
            const uint32_t a0 = xa.x & keep[a][0], a1 = xa.y & keep[a][1], a2 = xa.z & keep[a][0], a3 = xa.w & keep[a][1];
#pragma unroll
            for (int h = 0; h < 2; h++)
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                             : "+f"(c[a][h][0]), "+f"(c[a][h][1]), "+f"(c[a][h][2]), "+f"(c[a][h][3])
                             : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b[h][0]), "r"(b[h][1]));
        }
    }
    // c[a][h]: activation rows 16 a + g (values 0, 1) and + 8 (values 2, 3), weight rows 8 h + 2 t, + 1
#pragma unroll
    for (int a = 0; a < NA; a++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            red[warp][16 * a + g][8 * h + 2 * t] = c[a][h][0];
            red[warp][16 * a + g][8 * h + 2 * t + 1] = c[a][h][1];
            red[warp][16 * a + g + 8][8 * h + 2 * t] = c[a][h][2];
            red[warp][16 * a + g + 8][8 * h + 2 * t + 1] = c[a][h][3];
        }
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * M; i += blockDim.x) {
        const int m = i >> 4, r = i & 15;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) s += red[w][m][r];
        y1[(int64_t)m * N + band * 16 + r] = s * TQ3_UNIT;
    }
}

unsigned grid_of(int64_t items, int per_block, int cap) {
    int64_t b = (items + per_block - 1) / per_block;
    if (b < 1) b = 1;
    return (unsigned)(b < cap ? b : cap);
}

}  // namespace

cudaError_t launch_tq3_decode(const uint8_t *packed, int64_t N, int64_t K, float *out, int64_t ld, cudaStream_t st) {
    tq3_decode_kernel<false><<<grid_of(N * K, 256 * 4, device_sms() * 32), 256, 0, st>>>(packed, N, K, out, ld, 0, 0);
    return cudaGetLastError();
}

cudaError_t launch_tq3_wimg(const uint8_t *packed, int64_t N, int64_t K, __half *wimg, cudaStream_t st) {
    const int64_t Np = gemm_wimg_rows(N), Kp = (K + TILE_K - 1) / TILE_K * TILE_K;
    tq3_decode_kernel<true><<<grid_of(Np * (Kp / 8), 256, device_sms() * 32), 256, 0, st>>>(packed, N, K, wimg, 0, Np, Kp);
    return cudaGetLastError();
}

cudaError_t launch_tq3_rotate(const void *in, int in_dt, int64_t M, int64_t C, int64_t ld_in, const uint8_t *sign, const __half *scale,
                              const void *bias, int bias_dt, void *out, int out_dt, int64_t ld_out, cudaStream_t st, bool fragments) {
    return launch_pdl(tq3_rotate_kernel, dim3(grid_of(M * (C / 128), 8, device_sms() * 16)), dim3(256), 0, st, in, in_dt, M, C, ld_in, sign, scale, bias,
                      bias_dt, out, out_dt, ld_out, fragments ? 1 : 0);
}

// `rows` (1..4) rows of x1 [.][K] -> y1 [.][N]
cudaError_t launch_tq3_gemv(const uint8_t *packed, int64_t N, int64_t K, const float *x1, int rows, float *y1, cudaStream_t st) {
    const unsigned grid = (unsigned)(N / 16);
    const dim3 blk(256);
    switch (rows) {
        case 1: return launch_pdl(tq3_gemv_kernel<1>, dim3(grid), blk, 0, st, packed, N, K, x1, y1);
        case 2: return launch_pdl(tq3_gemv_kernel<2>, dim3(grid), blk, 0, st, packed, N, K, x1, y1);
        case 3: return launch_pdl(tq3_gemv_kernel<3>, dim3(grid), blk, 0, st, packed, N, K, x1, y1);
        case 4: return launch_pdl(tq3_gemv_kernel<4>, dim3(grid), blk, 0, st, packed, N, K, x1, y1);
        default: return cudaErrorInvalidValue;
    }
}

// `rows` (1..64) rows of x1 [.][K] (fp16) -> y1 [.][N] on the tensor-core decode kernel
cudaError_t launch_tq3_mma(const uint8_t *packed, int64_t N, int64_t K, const __half *x1, int rows, float *y1, cudaStream_t st) {
    const unsigned grid = (unsigned)(N / 16);
    const dim3 blk(256);
    if (rows <= 16) return launch_pdl(tq3_mma_kernel<1>, dim3(grid), blk, 0, st, packed, N, K, x1, rows, y1);
    if (rows <= 32) return launch_pdl(tq3_mma_kernel<2>, dim3(grid), blk, 0, st, packed, N, K, x1, rows, y1);
    if (rows <= 64) return launch_pdl(tq3_mma_kernel<4>, dim3(grid), blk, 0, st, packed, N, K, x1, rows, y1);
    return cudaErrorInvalidValue;
}

}  // namespace ttq
