// Load-time repack (canonical GGUF-style blocks -> tiled device layout) and the inverse
// dequantization used as the bit-exactness test hook.  Both are one-pass byte-shuffling kernels,
// bound by HBM bandwidth; neither is on the per-token path.
#include "ttq_internal.cuh"

namespace ttq {

namespace {

// Canonical-side accessors for one tile (16 rows x 256 weights).
struct CanonTile {
    const uint8_t *canon;
    int64_t N, K, nt, sb;
    // Q4_K / Q6_K: block of row r.  Returns nullptr for padded rows.
    __device__ const uint8_t *block256(int r, int bb) const {
        int64_t n = nt * TILE_ROWS + r;
        if (n >= N) return nullptr;
        return canon + (n * (K / 256) + sb) * bb;
    }
    // Q8_0: block b (0..7) of row r, nullptr when padded in N or K.
    __device__ const uint8_t *block32(int r, int b) const {
        int64_t n = nt * TILE_ROWS + r;
        int64_t kb = sb * 8 + b;
        if (n >= N || kb >= K / 32) return nullptr;
        return canon + (n * (K / 32) + kb) * 34;
    }
};

// 6-bit quant (0..63) of weight kk (0..255) inside a canonical Q6_K block, split in its two parts.
__device__ __forceinline__ void q6k_parts(const uint8_t *blk, int kk, int &lo4, int &hi2) {
    int half = kk >> 7, e = kk & 127, l = e & 31, grp = e >> 5;
    uint8_t qlb = blk[half * 64 + l + ((grp & 1) ? 32 : 0)];
    lo4 = (grp >= 2) ? (qlb >> 4) : (qlb & 15);
    hi2 = (blk[128 + half * 32 + l] >> (2 * grp)) & 3;
}

// Decompose a payload offset inside a 512-byte lane-ordered chunk into A-fragment coordinates:
// lane L = 4g + t, slot sl = register a0..a3 of mma.m16n8k32, byte i.  The register covers
//   row    = g + 8 * (sl & 1)
//   group  = (t >> 1) + 2 * (sl >> 1)       one of the 4 sub-blocks that share the instruction
//   kpos   = 4 * (t & 1) + i                position inside the group's 8-weight window
__device__ __forceinline__ void frag_coords(int o512, int &row, int &group, int &kpos) {
    const int L = o512 >> 4, sl = (o512 >> 2) & 3, i = o512 & 3;
    const int g = L >> 2, t = L & 3;
    row = g + 8 * (sl & 1);
    group = (t >> 1) + 2 * (sl >> 1);
    kpos = 4 * (t & 1) + i;
}
// Inverse: byte offset inside a 512-byte chunk of (row, group, kpos).
__device__ __forceinline__ int frag_offset(int row, int group, int kpos) {
    const int g = row & 7, t = 2 * (group & 1) + (kpos >> 2), sl = (row >> 3) + 2 * (group >> 1);
    return ((g * 4 + t) << 4) + (sl << 2) + (kpos & 3);
}

template <int FMT>
__device__ uint8_t tiled_byte(const CanonTile &ct, int o) {
    int r, u, kpos;
    if (FMT == TTQ_FMT_Q4_K) {
        if (o < 2048) {
            const int n = o >> 9;  // window n: weights 8n..8n+7 of each sub-block
            frag_coords(o & 511, r, u, kpos);
            const uint8_t *blk = ct.block256(r, 144);
            return blk ? blk[16 + 32 * u + 8 * n + kpos] : 0;  // pair u: low nibble sub-block 2u, high 2u+1
        }
        int h = o - 2048;
        const uint8_t *blk = ct.block256(h >> 4, 144);
        return blk ? blk[h & 15] : 0;
    } else if (FMT == TTQ_FMT_Q8_0) {
        if (o < 4096) {
            const int c = o >> 9, s = c >> 2, n = c & 3;  // set s: blocks 4s..4s+3
            frag_coords(o & 511, r, u, kpos);
            const uint8_t *blk = ct.block32(r, 4 * s + u);
            return blk ? blk[2 + 8 * n + kpos] : 0;
        }
        int h = o - 4096;
        const uint8_t *blk = ct.block32(h >> 4, (h & 15) >> 1);
        return blk ? blk[h & 1] : 0;
    } else {
        if (o < 2048) {
            const int c = o >> 9, sp = c >> 1, n = c & 1;  // low nibbles: set sp, high nibbles: set sp+2
            frag_coords(o & 511, r, u, kpos);
            const uint8_t *blk = ct.block256(r, 210);
            if (!blk) return 0;
            int a, b2, dummy;
            q6k_parts(blk, 16 * (4 * sp + u) + 8 * n + kpos, a, dummy);
            q6k_parts(blk, 16 * (4 * (sp + 2) + u) + 8 * n + kpos, b2, dummy);
            return (uint8_t)(a | (b2 << 4));
        }
        if (o < 3072) {
            const int o2 = o - 2048, n = o2 >> 9;
            frag_coords(o2 & 511, r, u, kpos);
            const uint8_t *blk = ct.block256(r, 210);
            if (!blk) return 0;
            int v = 0;
            for (int s = 0; s < 4; s++) {
                int lo, hi;
                q6k_parts(blk, 16 * (4 * s + u) + 8 * n + kpos, lo, hi);
                v |= hi << (2 * s);
            }
            return (uint8_t)v;
        }
        if (o < 3328) {
            int h = o - 3072;
            const uint8_t *blk = ct.block256(h >> 4, 210);
            return blk ? blk[192 + (h & 15)] : 0;
        }
        int h = o - 3328;
        const uint8_t *blk = ct.block256(h >> 1, 210);
        return blk ? blk[208 + (h & 1)] : 0;
    }
}

template <int FMT>
__global__ void __launch_bounds__(128) repack_kernel(const uint8_t *__restrict__ canon,
                                                     uint8_t *__restrict__ tiled, int64_t N, int64_t K,
                                                     int64_t NT, int64_t SBp) {
    constexpr int TB = tile_bytes(FMT);
    for (int64_t tile = blockIdx.x; tile < NT * SBp; tile += gridDim.x) {
        CanonTile ct{canon, N, K, tile / SBp, tile % SBp};
        uint32_t *dst = reinterpret_cast<uint32_t *>(tiled + tile * TB);
        for (int w = threadIdx.x; w < TB / 4; w += blockDim.x) {
            uint32_t v = 0;
#pragma unroll
            for (int b = 0; b < 4; b++) v |= (uint32_t)tiled_byte<FMT>(ct, 4 * w + b) << (8 * b);
            dst[w] = v;
        }
    }
}

// ---- inverse: tiled -> fp32 [N][ld], canonical element order ----------------------------------
template <int FMT>
__device__ float dequant_elem(const uint8_t *tile, int r, int kk) {
    if (FMT == TTQ_FMT_Q4_K) {
        const int j = kk >> 5, l = kk & 31;
        const uint8_t b = tile[(l >> 3) * 512 + frag_offset(r, j >> 1, l & 7)];
        const int q = (j & 1) ? (b >> 4) : (b & 15);
        const uint8_t *hdr = tile + 2048 + r * 16;
        float d = __half2float(*reinterpret_cast<const __half *>(hdr));
        float dmin = __half2float(*reinterpret_cast<const __half *>(hdr + 2));
        int sc, m;
        q4k_scale_min(j, hdr + 4, sc, m);
        return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)m));
    } else if (FMT == TTQ_FMT_Q8_0) {
        const int b = kk >> 5, l = kk & 31;
        const int o = (4 * (b >> 2) + (l >> 3)) * 512 + frag_offset(r, b & 3, l & 7);
        float d = __half2float(*reinterpret_cast<const __half *>(tile + 4096 + r * 16 + b * 2));
        return __fmul_rn(d, (float)(int8_t)tile[o]);
    } else {
        const int j = kk >> 4, s = j >> 2, u = j & 3, l = kk & 15, n = l >> 3;
        const int fo = frag_offset(r, u, l & 7);
        const uint8_t qlb = tile[(2 * (s & 1) + n) * 512 + fo];
        const int nib = (s >> 1) ? (qlb >> 4) : (qlb & 15);
        const int hi2 = (tile[2048 + n * 512 + fo] >> (2 * s)) & 3;
        const int q = (nib | (hi2 << 4)) - 32;
        float sc = (float)(int8_t)tile[3072 + r * 16 + j];
        float d = __half2float(*reinterpret_cast<const __half *>(tile + 3328 + 2 * r));
        return __fmul_rn(__fmul_rn(d, sc), (float)q);
    }
}

template <int FMT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t *__restrict__ tiled, float *__restrict__ out,
                                                      int64_t ld, int64_t N, int64_t K, int64_t SBp) {
    constexpr int TB = tile_bytes(FMT);
    const int64_t total = N * K;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        int64_t n = e / K, k = e % K;
        const uint8_t *tile = tiled + ((n / TILE_ROWS) * SBp + (k / TILE_K)) * TB;
        out[n * ld + k] = dequant_elem<FMT>(tile, (int)(n % TILE_ROWS), (int)(k % TILE_K));
    }
}

template <typename T>
__global__ void __launch_bounds__(256) silu_and_mul_kernel(const T *__restrict__ in, T *__restrict__ out,
                                                           int64_t M, int64_t H, int64_t ld_in, int64_t ld_out) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int64_t total = M * H;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        int64_t m = e / H, h = e % H;
        float g = (float)in[m * ld_in + h], u = (float)in[m * ld_in + H + h];
        out[m * ld_out + h] = (T)((g / (1.0f + expf(-g))) * u);
    }
}

int grid_for(int64_t work_items, int per_block, int cap) {
    int64_t b = (work_items + per_block - 1) / per_block;
    if (b < 1) b = 1;
    return (int)(b < cap ? b : cap);
}

}  // namespace

cudaError_t launch_repack(int fmt, const uint8_t *canon, uint8_t *tiled, int64_t N, int64_t K, int64_t NT,
                          int64_t SBp, cudaStream_t st) {
    int grid = grid_for(NT * SBp, 1, device_sms() * 64);
    if (fmt == TTQ_FMT_Q4_K) repack_kernel<TTQ_FMT_Q4_K><<<grid, 128, 0, st>>>(canon, tiled, N, K, NT, SBp);
    else if (fmt == TTQ_FMT_Q8_0) repack_kernel<TTQ_FMT_Q8_0><<<grid, 128, 0, st>>>(canon, tiled, N, K, NT, SBp);
    else repack_kernel<TTQ_FMT_Q6_K><<<grid, 128, 0, st>>>(canon, tiled, N, K, NT, SBp);
    return cudaGetLastError();
}

cudaError_t launch_dequant(int fmt, const uint8_t *tiled, float *out, int64_t ld, int64_t N, int64_t K,
                           int64_t SBp, cudaStream_t st) {
    int grid = grid_for(N * K, 256 * 8, device_sms() * 32);
    if (fmt == TTQ_FMT_Q4_K) dequant_kernel<TTQ_FMT_Q4_K><<<grid, 256, 0, st>>>(tiled, out, ld, N, K, SBp);
    else if (fmt == TTQ_FMT_Q8_0) dequant_kernel<TTQ_FMT_Q8_0><<<grid, 256, 0, st>>>(tiled, out, ld, N, K, SBp);
    else dequant_kernel<TTQ_FMT_Q6_K><<<grid, 256, 0, st>>>(tiled, out, ld, N, K, SBp);
    return cudaGetLastError();
}

cudaError_t launch_silu_and_mul(const void *in, int dt, int64_t M, int64_t H, int64_t ld_in, void *out,
                                int64_t ld_out, cudaStream_t st) {
    int grid = grid_for(M * H, 256 * 4, device_sms() * 16);
    if (dt == TTQ_DT_BF16)
        return launch_pdl(silu_and_mul_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16 *)in, (__nv_bfloat16 *)out, M, H,
                          ld_in, ld_out);
    if (dt == TTQ_DT_F16)
        return launch_pdl(silu_and_mul_kernel<__half>, dim3(grid), dim3(256), 0, st, (const __half *)in, (__half *)out, M, H, ld_in, ld_out);
    return launch_pdl(silu_and_mul_kernel<float>, dim3(grid), dim3(256), 0, st, (const float *)in, (float *)out, M, H, ld_in, ld_out);
}

}  // namespace ttq
