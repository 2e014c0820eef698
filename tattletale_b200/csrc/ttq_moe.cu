// Routing and combination kernels of the mixture-of-experts layer built on the grouped Q4_K GEMM.
//
// A layer call routes every (token, choice) pair to a row of a padded, expert-sorted row space:
// expert e owns ceil(count_e / BM) consecutive BM-row tiles, so that each row tile of the grouped GEMM
// multiplies exactly one expert's matrices.  Nothing is copied to the host: tile counts and tables stay
// on the device and the GEMM reads them there.
//
//   route_count   histogram of the expert ids
//   route_plan    prefix over the experts -> first row of each expert, expert of each row tile, tile count
//   route_scatter slot of every pair (atomic cursor per expert), source token of every slot
//   combine       y[t] = sum_j w[t][j] * o[slot(t, j)]   (fixed order over j: the result does not depend
//                 on the order in which the atomics handed out the slots)
//
// The reference has no mixture-of-experts layer; the dataflow is the gated MLP of
// workspace/transformers/src/layers/mlp.nim:56-60 applied per expert, weighted and summed.
#include "ttq_internal.cuh"

namespace ttq {
namespace {

__global__ void __launch_bounds__(256) route_count_kernel(const int *__restrict__ ids, int64_t pairs, int E, int *__restrict__ counts) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += (int64_t)gridDim.x * blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < E) atomicAdd(counts + e, 1);
    }
}

// One block.  Expert counts -> padded row ranges and the row-tile tables.  Fixed tile heights (64, 128, 256): an
// expert's rows are padded to whole tiles.  BM = 384: rows are padded to 128 and a tile holds up to three
// 128-row blocks of ONE expert, so that the expert's weight rows are expanded once for (almost always) all of
// its rows.  `mt_cap` bounds the tables (they cannot overflow when the capacity was sized as the launcher does;
// the check keeps a bad call from writing out of bounds).
__global__ void __launch_bounds__(1024) route_plan_kernel(const int *__restrict__ counts, int E, int BM, int mt_cap,
                                                          int *__restrict__ row_start, int *__restrict__ cursor,
                                                          int *__restrict__ mt_group, int *__restrict__ mt_row0,
                                                          int *__restrict__ mt_mh, int *__restrict__ n_mt) {
    extern __shared__ int plan_s[];  // tile_start [E + 1], row_begin [E + 1]
    int *tile_start = plan_s, *row_begin = plan_s + E + 1;
    const int unit = BM == 384 ? 128 : BM;
    if (threadIdx.x == 0) {
        int tiles = 0, rows = 0;
        for (int e = 0; e < E; e++) {
            tile_start[e] = tiles;
            row_begin[e] = rows;
            const int padded = (counts[e] + unit - 1) / unit * unit;
            tiles += (padded + BM - 1) / BM;
            rows += padded;
        }
        tile_start[E] = tiles;
        row_begin[E] = rows;
        n_mt[0] = tiles < mt_cap ? tiles : mt_cap;
        n_mt[1] = rows;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        row_start[e] = row_begin[e];
        cursor[e] = 0;
        const int padded = row_begin[e + 1] - row_begin[e];
        for (int t = tile_start[e]; t < tile_start[e + 1] && t < mt_cap; t++) {
            const int off = (t - tile_start[e]) * BM;
            mt_group[t] = e;
            mt_row0[t] = row_begin[e] + off;
            const int left = padded - off;
            mt_mh[t] = BM == 384 ? (left >= 384 ? 3 : left / 128) : (BM > 128 ? BM / 128 : 1);
        }
    }
}

__global__ void __launch_bounds__(256) route_scatter_kernel(const int *__restrict__ ids, int64_t pairs, int top_k, int E, int64_t Mp,
                                                            const int *__restrict__ row_start, int *__restrict__ cursor,
                                                            int *__restrict__ slot_of, int *__restrict__ row_src) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += (int64_t)gridDim.x * blockDim.x) {
        const int e = ids[i];
        int slot = -1;
        if (e >= 0 && e < E) {
            slot = row_start[e] + atomicAdd(cursor + e, 1);
            if (slot < Mp) row_src[slot] = (int)(i / top_k);
            else slot = -1;
        }
        slot_of[i] = slot;
    }
}

// 8 outputs per thread; o rows are fp16 or bf16 (16-byte aligned rows take the vector path)
__global__ void __launch_bounds__(256) combine_kernel(const void *__restrict__ o, int o_dt, int64_t ldo, const int *__restrict__ slot_of,
                                                      const float *__restrict__ w, int64_t T, int top_k, int64_t H, void *__restrict__ y,
                                                      int y_dt, int64_t ldy) {
    const int64_t per_row = (H + 7) / 8, total = T * per_row;
    for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < total; c += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = c / per_row, h0 = (c % per_row) * 8;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < top_k; j++) {
            const int slot = slot_of[t * top_k + j];
            if (slot < 0) continue;
            const float wj = w[t * top_k + j];
            const bool vec = o_dt == TTQ_DT_F16 && h0 + 8 <= H &&
                             ((reinterpret_cast<uintptr_t>(o) + (size_t)((int64_t)slot * ldo + h0) * 2) & 15) == 0;
            if (vec) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(o) + (int64_t)slot * ldo + h0);
                const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const float2 v = __half22float2(h2[q]);
                    acc[2 * q] = fmaf(wj, v.x, acc[2 * q]);
                    acc[2 * q + 1] = fmaf(wj, v.y, acc[2 * q + 1]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++)
                    if (h0 + i < H) acc[i] = fmaf(wj, load_as_float(o, o_dt, (int64_t)slot * ldo + h0 + i), acc[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (h0 + i < H) store_from_float(y, y_dt, t * ldy + h0 + i, acc[i]);
    }
}

unsigned grid_of(int64_t items, int cap) {
    int64_t b = (items + 255) / 256;
    if (b < 1) b = 1;
    return (unsigned)(b < cap ? b : cap);
}

}  // namespace

cudaError_t launch_moe_route(const MoeRouting &r, const int *topk_ids, int64_t T, int top_k, int E, int BM, int64_t Mp,
                             int64_t mt_cap, cudaStream_t st, int *launches) {
    *launches = 0;
    const int64_t pairs = T * top_k;
    cudaError_t e = cudaMemsetAsync(r.counts, 0, sizeof(int) * (size_t)E, st);
    if (e != cudaSuccess) return e;
    e = cudaMemsetAsync(r.row_src, 0xff, sizeof(int) * (size_t)Mp, st);  // every row is padding until a pair claims it
    if (e != cudaSuccess) return e;
    route_count_kernel<<<grid_of(pairs, device_sms() * 4), 256, 0, st>>>(topk_ids, pairs, E, r.counts);
    route_plan_kernel<<<1, 1024, 2 * sizeof(int) * (size_t)(E + 1), st>>>(r.counts, E, BM, (int)mt_cap, r.row_start, r.cursor, r.mt_group,
                                                                          r.mt_row0, r.mt_mh, r.n_mt);
    route_scatter_kernel<<<grid_of(pairs, device_sms() * 4), 256, 0, st>>>(topk_ids, pairs, top_k, E, Mp, r.row_start, r.cursor, r.slot_of,
                                                                  r.row_src);
    *launches = 3;
    return cudaGetLastError();
}

cudaError_t launch_moe_combine(const MoeRouting &r, const void *o, int o_dt, int64_t ldo, const float *topk_w, int64_t T,
                               int top_k, int64_t H, void *y, int y_dt, int64_t ldy, cudaStream_t st) {
    combine_kernel<<<grid_of(T * ((H + 7) / 8), device_sms() * 16), 256, 0, st>>>(o, o_dt, ldo, r.slot_of, topk_w, T, top_k, H, y, y_dt, ldy);
    return cudaGetLastError();
}

}  // namespace ttq
