// Decode-step kernels around the quantized linears: residual add + RMSNorm, RoPE + KV-cache append, and
// single-query grouped-query attention over a contiguous KV cache.  These are the steps that sit between two
// linears of a decoder layer in the reference:
//   RmsNorm.forward / forward_with_residual   workspace/transformers/src/layers/norm.nim:23-38 (the unfused add +
//                                             norm is flagged TODO at :35)
//   rotary embedding (rotate-half form)        workspace/transformers/src/layers/rope.nim:29-92
//   attention with a growing KV cache          workspace/transformers/src/layers/attn.nim:97-104,149-189
// All 16-bit tensors are bf16 or f16 (one dtype per call), arithmetic is fp32.
//
//   add_rmsnorm_kernel        one CTA per row: h += delta (optional), out = h * rsqrt(mean(h^2) + eps) * weight
//   rope_kv_kernel            one CTA per (sequence, head of the fused qkv row): rotates q and k heads, writes q to
//                             its own buffer, k and v into the cache at `pos`
//   decode_attn_kernel        one CTA per (sequence, kv head, slice of 128 cache positions): thread t scores
//                             position t against the G query heads of the group (K row read as 16 vector loads),
//                             block softmax statistics, then thread t accumulates output dimension t over the
//                             slice (V read coalesced); partial (max, sum, output) per slice
//   decode_attn_merge_kernel  one CTA per (sequence, query head): merges the slices
#include "ttq_internal.cuh"
#include "ttq_xprep.cuh"

namespace ttq {
namespace {

constexpr int ATT_D = 128;      // head dimension served by the attention kernels
constexpr int ATT_SLICE = 128;  // cache positions per CTA

__device__ __forceinline__ void unpack8(const uint4 &raw, int dt, float (&f)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        if (dt == TTQ_DT_BF16) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        } else {
            const float2 v = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            f[2 * i] = v.x;
            f[2 * i + 1] = v.y;
        }
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8], int dt) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        if (dt == TTQ_DT_BF16) {
            const __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&t);
        } else {
            const __half2 t = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&t);
        }
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ float block_sum(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float s = 0.f;
    for (int i = 0; i < nw; i++) s += red[i];
    return s;
}
// H % 8 == 0, rows 16-byte aligned (checked by the launcher).
// `xq.planes` != nullptr (H a multiple of 256, H <= 8192): the normalised row, as rounded for `out`, is also converted
// to the fixed-point planes a decode linear reads (thread t holds the 8 values lane t & 31 of chunk t >> 5 converts in
// the activation pass), so that the linear that consumes `out` can skip its own conversion pass.
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(void *__restrict__ h, const void *__restrict__ delta, const void *__restrict__ weight,
                                                          int dt, int64_t H, int64_t ld_h, int64_t ld_delta, float eps,
                                                          void *__restrict__ out, int64_t ld_out, XqView xq) {
    __shared__ float red[8];
    grid_launch_dependents();
    grid_dependency_wait();
    const int64_t m = blockIdx.x;
    uint8_t *hrow = reinterpret_cast<uint8_t *>(h) + m * ld_h * 2;
    const uint8_t *drow = delta ? reinterpret_cast<const uint8_t *>(delta) + m * ld_delta * 2 : nullptr;
    const uint8_t *wrow = reinterpret_cast<const uint8_t *>(weight);
    uint8_t *orow = reinterpret_cast<uint8_t *>(out) + m * ld_out * 2;
    const int64_t chunks = H / 8;
    constexpr int KEEP = 4;  // chunks of 8 values a thread keeps in registers between the two passes (H <= 8192)
    if (chunks <= (int64_t)KEEP * blockDim.x) {
        // all loads first (row, residual, weight), one reduction, then the output straight from registers
        uint4 hv[KEEP], dv[KEEP], wv[KEEP];
#pragma unroll
        for (int i = 0; i < KEEP; i++) {
            const int64_t c = threadIdx.x + (int64_t)i * blockDim.x;
            if (c < chunks) {
                hv[i] = *reinterpret_cast<const uint4 *>(hrow + c * 16);
                if (drow) dv[i] = *reinterpret_cast<const uint4 *>(drow + c * 16);
                wv[i] = *reinterpret_cast<const uint4 *>(wrow + c * 16);
            }
        }
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < KEEP; i++) {
            const int64_t c = threadIdx.x + (int64_t)i * blockDim.x;
            if (c < chunks) {
                float v[8];
                unpack8(hv[i], dt, v);
                if (drow) {
                    float d[8];
                    unpack8(dv[i], dt, d);
#pragma unroll
                    for (int q = 0; q < 8; q++) v[q] += d[q];
                    hv[i] = pack8(v, dt);  // the residual stream is stored (and normalised) in its 16-bit rounding
                    *reinterpret_cast<uint4 *>(hrow + c * 16) = hv[i];
                    unpack8(hv[i], dt, v);
                }
#pragma unroll
                for (int q = 0; q < 8; q++) ss = fmaf(v[q], v[q], ss);
            }
        }
        const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
#pragma unroll
        for (int i = 0; i < KEEP; i++) {
            const int64_t c = threadIdx.x + (int64_t)i * blockDim.x;
            if (c < chunks) {
                float v[8], w[8];
                unpack8(hv[i], dt, v);
                unpack8(wv[i], dt, w);
#pragma unroll
                for (int q = 0; q < 8; q++) v[q] = v[q] * inv * w[q];
                const uint4 packed = pack8(v, dt);
                *reinterpret_cast<uint4 *>(orow + c * 16) = packed;
                if (xq.planes != nullptr) {
                    // (whole warps pass here: H / 8 is a multiple of 32)
                    const int64_t SBp = H / TILE_K, Kp = H;
                    unpack8(packed, dt, v);
                    const XqRow dst{xq.planes + (2 * m) * Kp, xq.planes + (2 * m + 1) * Kp, xq.sum16 + m * (Kp / 16), xq.sum32 + m * (Kp / 32),
                                    xq.sx + m * sx_stride(SBp)};
                    xprep_convert_vals(v, (int)(c >> 5), (int)(threadIdx.x & 31), dst);
                }
            }
        }
        return;
    }
    float ss = 0.f;
    for (int64_t c = threadIdx.x; c < chunks; c += blockDim.x) {
        float v[8];
        unpack8(*reinterpret_cast<const uint4 *>(hrow + c * 16), dt, v);
        if (drow) {
            float d[8];
            unpack8(*reinterpret_cast<const uint4 *>(drow + c * 16), dt, d);
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] += d[i];
            const uint4 packed = pack8(v, dt);
            *reinterpret_cast<uint4 *>(hrow + c * 16) = packed;
            unpack8(packed, dt, v);  // the norm sees the stored (rounded) residual stream, as the unfused sequence does
        }
#pragma unroll
        for (int i = 0; i < 8; i++) ss = fmaf(v[i], v[i], ss);
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
    for (int64_t c = threadIdx.x; c < chunks; c += blockDim.x) {
        float v[8], w[8];
        unpack8(*reinterpret_cast<const uint4 *>(hrow + c * 16), dt, v);
        unpack8(*reinterpret_cast<const uint4 *>(wrow + c * 16), dt, w);
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = v[i] * inv * w[i];
        *reinterpret_cast<uint4 *>(orow + c * 16) = pack8(v, dt);
    }
}

// grid (hq + 2 hkv, B), d / 2 threads.  qkv row: [hq heads | hkv k heads | hkv v heads] of d values.
__global__ void rope_kv_kernel(const void *__restrict__ qkv, int dt, int64_t ld_qkv, int hq, int hkv, int d, const void *__restrict__ cosv,
                               const void *__restrict__ sinv, void *__restrict__ q_out, void *__restrict__ k_cache, void *__restrict__ v_cache,
                               int64_t ctx_len, int64_t pos) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int head = blockIdx.x, b = blockIdx.y, i = threadIdx.x, half = d / 2;
    const int64_t src = (int64_t)b * ld_qkv + (int64_t)head * d;
    const float x1 = load_as_float(qkv, dt, src + i), x2 = load_as_float(qkv, dt, src + half + i);
    if (head < hq + hkv) {
        // rotate-half: out = x * cos + rotate_half(x) * sin, rotate_half(x) = [-x2, x1]; fp32, rounded once
        const float c1 = load_as_float(cosv, dt, i), c2 = load_as_float(cosv, dt, half + i);
        const float s1 = load_as_float(sinv, dt, i), s2 = load_as_float(sinv, dt, half + i);
        const float o1 = x1 * c1 - x2 * s1, o2 = x2 * c2 + x1 * s2;
        if (head < hq) {
            const int64_t dst = ((int64_t)b * hq + head) * d;
            store_from_float(q_out, dt, dst + i, o1);
            store_from_float(q_out, dt, dst + half + i, o2);
        } else {
            const int64_t dst = (((int64_t)b * hkv + (head - hq)) * ctx_len + pos) * d;
            store_from_float(k_cache, dt, dst + i, o1);
            store_from_float(k_cache, dt, dst + half + i, o2);
        }
    } else {
        const int64_t dst = (((int64_t)b * hkv + (head - hq - hkv)) * ctx_len + pos) * d;
        store_from_float(v_cache, dt, dst + i, x1);
        store_from_float(v_cache, dt, dst + half + i, x2);
    }
}

// grid (slices, hkv, B), 128 threads.  part: [B][hkv][slices][G][2 + 128] floats = (max, sum, unnormalised output).
// Scores: a half-warp reads one K row per load (16 lanes x 16 bytes, two rows per warp instruction, all 16 loads of
// a warp's 32 positions in flight together), partial dots are folded over the 16 lanes.  Output: thread (pg, dg)
// accumulates dimensions 8 dg .. 8 dg + 7 over positions pg, pg + 8, ... with 16-byte V loads, the 8 position
// groups are summed through shared memory.
// Seven CTAs per SM (72 registers) on large grids: 1024 CTAs at batch 8 then fit one wave (22.9 against 25.1 us per call);
// batch 32 is unchanged.
// PREFETCH: every K and V row of the thread is requested before anything else (helps while the grid leaves SMs
// under-occupied, costs registers and therefore occupancy on large grids).
template <int G, bool PREFETCH>
__global__ void __launch_bounds__(ATT_SLICE, PREFETCH ? 1 : 7) decode_attn_kernel(const void *__restrict__ q, const void *__restrict__ k_cache,
                                                                const void *__restrict__ v_cache, int dt, int hq, int hkv, int64_t ctx_len,
                                                                int64_t n_ctx, float scale, float *__restrict__ part) {
    __shared__ float q_s[G][ATT_D];
    __shared__ float p_s[G][ATT_SLICE];
    __shared__ float o_s[8][G][ATT_D];
    grid_launch_dependents();
    grid_dependency_wait();
    const int slice = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, t = threadIdx.x;
    const int warp = t >> 5, lane = t & 31;
    const int slices = gridDim.x;
    const int64_t p0 = (int64_t)slice * ATT_SLICE;
    const int64_t n_here = n_ctx - p0 < ATT_SLICE ? n_ctx - p0 : ATT_SLICE;
    const uint8_t *kbase = reinterpret_cast<const uint8_t *>(k_cache) + ((((int64_t)b * hkv + kvh) * ctx_len + p0) * ATT_D) * 2;
    const uint8_t *vbase = reinterpret_cast<const uint8_t *>(v_cache) + ((((int64_t)b * hkv + kvh) * ctx_len + p0) * ATT_D) * 2;
    const int hw = lane >> 4, c = lane & 15;
    const int pg = t >> 4, dg = t & 15;
    // PREFETCH (small grids, about one CTA per SM: latency is everything and registers are free): every K and V row of
    // the thread is requested before anything else, the query loads and all arithmetic run under those loads.
    constexpr int NK = PREFETCH ? 16 : 8, NV = PREFETCH ? 16 : 1;
    uint4 kraw[NK], vraw[NV];
    auto load_k = [&](int first, int count, uint4 *dst) {
#pragma unroll
        for (int i = 0; i < 16; i++) {
            if (i < count) {
                const int j = 32 * warp + 2 * (first + i) + hw;
                dst[i] = j < n_here ? *reinterpret_cast<const uint4 *>(kbase + (int64_t)j * (ATT_D * 2) + 16 * c) : make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };
    if constexpr (PREFETCH) {
        load_k(0, 16, kraw);
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int j = pg + 8 * i;
            vraw[i] = j < n_here ? *reinterpret_cast<const uint4 *>(vbase + (int64_t)j * (ATT_D * 2) + 16 * dg) : make_uint4(0u, 0u, 0u, 0u);
        }
    }
    for (int i = t; i < G * ATT_D; i += ATT_SLICE)
        q_s[i / ATT_D][i % ATT_D] = load_as_float(q, dt, ((int64_t)b * hq + (int64_t)kvh * G + i / ATT_D) * ATT_D + i % ATT_D) * scale;
    __syncthreads();
    {
#pragma unroll 1
        for (int half = 0; half < (PREFETCH ? 1 : 2); half++) {
            if constexpr (!PREFETCH) load_k(8 * half, 8, kraw);
#pragma unroll
            for (int i8 = 0; i8 < NK; i8++) {
                const int it = 8 * half + i8;
                float kv[8];
                unpack8(kraw[i8], dt, kv);
                float sg[G];
#pragma unroll
                for (int g = 0; g < G; g++) {
                    float a = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; i++) a = fmaf(kv[i], q_s[g][8 * c + i], a);
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                    sg[g] = a;
                }
                if (c == 0) {
                    const int j = 32 * warp + 2 * it + hw;
#pragma unroll
                    for (int g = 0; g < G; g++) p_s[g][j] = sg[g];
                }
            }
        }
    }
    __syncthreads();
    float *my = part + ((((int64_t)b * hkv + kvh) * slices + slice) * G) * (2 + ATT_D);
    // softmax statistics of the slice: one warp per query head, four positions per lane
    for (int g = warp; g < G; g += ATT_SLICE / 32) {
        float sc[4], mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            sc[i] = lane + 32 * i < n_here ? p_s[g][lane + 32 * i] : -INFINITY;
            mx = fmaxf(mx, sc[i]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float e = lane + 32 * i < n_here ? __expf(sc[i] - mx) : 0.f;
            p_s[g][lane + 32 * i] = e;
            sum += e;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) {
            my[g * (2 + ATT_D)] = mx;
            my[g * (2 + ATT_D) + 1] = sum;
        }
    }
    __syncthreads();
    {
        float o[G][8];
#pragma unroll
        for (int g = 0; g < G; g++)
#pragma unroll
            for (int i = 0; i < 8; i++) o[g][i] = 0.f;
#pragma unroll 1
        for (int half = 0; half < 2; half++) {
        uint4 raw[8];
#pragma unroll
        for (int i8 = 0; i8 < 8; i8++) {
            const int j = pg + 8 * (8 * half + i8);
            if constexpr (PREFETCH) raw[i8] = half == 0 ? vraw[i8] : vraw[8 + i8];
            else raw[i8] = j < n_here ? *reinterpret_cast<const uint4 *>(vbase + (int64_t)j * (ATT_D * 2) + 16 * dg) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int i8 = 0; i8 < 8; i8++) {
            const int j = pg + 8 * (8 * half + i8);
            float v[8];
            unpack8(raw[i8], dt, v);
#pragma unroll
            for (int g = 0; g < G; g++) {
                const float pw = p_s[g][j];  // zero beyond n_here
#pragma unroll
                for (int i = 0; i < 8; i++) o[g][i] = fmaf(pw, v[i], o[g][i]);
            }
        }
        }
#pragma unroll
        for (int g = 0; g < G; g++)
#pragma unroll
            for (int i = 0; i < 8; i++) o_s[pg][g][8 * dg + i] = o[g][i];
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; g++) {
        float a = 0.f;
#pragma unroll
        for (int r = 0; r < 8; r++) a += o_s[r][g][t];
        my[g * (2 + ATT_D) + 2 + t] = a;
    }
}

// grid (hq, B), 128 threads.  The slices' statistics are read by one thread each and their weights exp(max_s - max)
// shared through shared memory, so that the loads of a merge are in flight together instead of one L2 round trip per
// slice (a decode step at batch 1 is a chain of such latencies).
constexpr int ATT_MERGE_SLICES = 512;  // slices whose weights fit the shared array (context 65536); beyond: recomputed
__global__ void __launch_bounds__(ATT_D) decode_attn_merge_kernel(const float *__restrict__ part, int hq, int hkv, int G, int slices,
                                                                  void *__restrict__ out, int dt) {
    __shared__ float w_s[ATT_MERGE_SLICES];
    __shared__ float red[2][ATT_D / 32];
    grid_launch_dependents();
    grid_dependency_wait();
    const int h = blockIdx.x, b = blockIdx.y, t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int kvh = h / G, g = h % G;
    const float *base = part + (((int64_t)b * hkv + kvh) * slices * G + g) * (2 + ATT_D);
    const int64_t stride = (int64_t)G * (2 + ATT_D);
    // this thread's slices: t, t + 128, ...
    float mx = -INFINITY;
    for (int s = t; s < slices; s += ATT_D) mx = fmaxf(mx, base[s * stride]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[0][warp] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(red[0][0], red[0][1]), fmaxf(red[0][2], red[0][3]));
    float den = 0.f;
    for (int s = t; s < slices; s += ATT_D) {
        const float w = __expf(base[s * stride] - mx);
        if (s < ATT_MERGE_SLICES) w_s[s] = w;
        den = fmaf(w, base[s * stride + 1], den);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
    if (lane == 0) red[1][warp] = den;
    __syncthreads();
    den = (red[1][0] + red[1][1]) + (red[1][2] + red[1][3]);
    float num = 0.f;
    int s = 0;
    for (; s + 8 <= slices && s + 8 <= ATT_MERGE_SLICES; s += 8) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = base[(s + i) * stride + 2 + t];
#pragma unroll
        for (int i = 0; i < 8; i++) num = fmaf(w_s[s + i], v[i], num);
    }
    for (; s < slices; s++) {
        const float w = s < ATT_MERGE_SLICES ? w_s[s] : __expf(base[s * stride] - mx);
        num = fmaf(w, base[s * stride + 2 + t], num);
    }
    store_from_float(out, dt, ((int64_t)b * hq + h) * ATT_D + t, num / den);
}

}  // namespace

cudaError_t launch_add_rmsnorm(void *h, const void *delta, const void *weight, int dt, int64_t M, int64_t H, int64_t ld_h, int64_t ld_delta,
                               float eps, void *out, int64_t ld_out, cudaStream_t st, const XqView *xq) {
    XqView v{nullptr, nullptr, nullptr, nullptr};
    if (xq != nullptr) {
        if (H % TILE_K || H > 8192) return cudaErrorInvalidValue;  // whole 256-wide chunks, row kept in registers
        v = *xq;
    }
    return launch_pdl(add_rmsnorm_kernel, dim3((unsigned)M), dim3(256), 0, st, h, delta, weight, dt, H, ld_h, ld_delta, eps, out, ld_out, v);
}

cudaError_t launch_rope_kv(const void *qkv, int dt, int64_t B, int64_t ld_qkv, int hq, int hkv, int d, const void *cosv, const void *sinv,
                           void *q_out, void *k_cache, void *v_cache, int64_t ctx_len, int64_t pos, cudaStream_t st) {
    return launch_pdl(rope_kv_kernel, dim3((unsigned)(hq + 2 * hkv), (unsigned)B), dim3((unsigned)(d / 2)), 0, st, qkv, dt, ld_qkv, hq, hkv, d,
                      cosv, sinv, q_out, k_cache, v_cache, ctx_len, pos);
}

int64_t decode_attention_scratch_floats(int64_t B, int hq, int64_t n_ctx) {
    const int64_t slices = (n_ctx + ATT_SLICE - 1) / ATT_SLICE;
    return B * hq * slices * (2 + ATT_D);
}

cudaError_t launch_decode_attention(const void *q, const void *k_cache, const void *v_cache, int dt, int64_t B, int hq, int hkv, int d,
                                    int64_t ctx_len, int64_t n_ctx, float *part, void *out, cudaStream_t st) {
    if (d != ATT_D || hq % hkv) return cudaErrorInvalidValue;
    const int G = hq / hkv;
    const int slices = (int)((n_ctx + ATT_SLICE - 1) / ATT_SLICE);
    const float scale = rsqrtf((float)d);
    const dim3 grid((unsigned)slices, (unsigned)hkv, (unsigned)B);
    cudaError_t e;
    const dim3 blk(ATT_SLICE);
    const bool pre = (int64_t)slices * hkv * B <= 2 * (int64_t)device_sms();  // at most two CTAs per SM: registers are free, latency is not
#define TTQ_ATT_LAUNCH(GG)                                                                                                          \
    e = pre ? launch_pdl(decode_attn_kernel<GG, true>, grid, blk, 0, st, q, k_cache, v_cache, dt, hq, hkv, ctx_len, n_ctx, scale, part) \
            : launch_pdl(decode_attn_kernel<GG, false>, grid, blk, 0, st, q, k_cache, v_cache, dt, hq, hkv, ctx_len, n_ctx, scale, part)
    switch (G) {
        case 1: TTQ_ATT_LAUNCH(1); break;
        case 2: TTQ_ATT_LAUNCH(2); break;
        case 4: TTQ_ATT_LAUNCH(4); break;
        case 8: TTQ_ATT_LAUNCH(8); break;
        default: return cudaErrorInvalidValue;
    }
#undef TTQ_ATT_LAUNCH
    if (e != cudaSuccess) return e;
    return launch_pdl(decode_attn_merge_kernel, dim3((unsigned)hq, (unsigned)B), dim3(ATT_D), 0, st, (const float *)part, hq, hkv, G, slices, out, dt);
}

}  // namespace ttq
