// Device-side helpers shared by the decode kernels: bulk-copy rings on mbarriers (every wait bounded),
// shared-memory access with immediate offsets, the per-kernel timeline entry, a compile-time loop.
#pragma once

#include "ttq_internal.cuh"

namespace ttq {

// ---- bulk-copy ring primitives ------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Untiled bulk copy global -> this CTA's shared memory (no multicast); both addresses 16-byte aligned, bytes a
// multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for a stage; gives up after WAIT_LIMIT polls, records the failure (status bit 0) and lets the caller
// go on with garbage data, so that every warp still reaches its barriers and the kernel returns.
constexpr int WAIT_LIMIT = 1 << 20;
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int *status) {
    for (int i = 0; i < WAIT_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    report_failure(status, 1);
    return false;
}
__device__ __forceinline__ void named_barrier(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- timeline -----------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
constexpr int TRACE_CAP = TTQ_TRACE_ENTRIES;
// Timeline entry of one kernel (written by thread 0 of block 0 when tracing is on):
// [0] kind (1 = activation pass, 2 = decode linear), [1] start, [2] after the dependency wait, [3] activations
// ready, [4] first weight tile ready, [5] end of block 0, [6] grid size, [7] N
__device__ __forceinline__ unsigned long long *trace_open(unsigned long long *trace, unsigned long long kind) {
    if (trace == nullptr || blockIdx.x != 0 || blockIdx.y != 0 || threadIdx.x != 0) return nullptr;
    const unsigned long long slot = atomicAdd(trace, 1ull);
    if (slot >= TRACE_CAP) return nullptr;
    unsigned long long *e = trace + 8 + slot * 8;
    e[0] = kind;
    e[1] = global_ns();
    return e;
}

// compile-time loop: f(IC<I>) for I in [0, N)
template <int V>
struct IC {
    static constexpr int value = V;
};
template <int I, int N, class F>
__device__ __forceinline__ void static_for(F &&f) {
    if constexpr (I < N) {
        f(IC<I>{});
        static_for<I + 1, N>(f);
    }
}

// ---- shared-memory access with 32-bit addresses and immediate offsets -----------------------------
template <int OFF>
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ float ldsf(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2+%3];" : "=f"(v.x), "=f"(v.y) : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ float4 lds128f(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4+%5];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ void stsf(uint32_t addr, float v) {
    asm volatile("st.shared.f32 [%0+%1], %2;" ::"r"(addr), "n"(OFF), "f"(v) : "memory");
}
template <int OFF>
__device__ __forceinline__ void sts64f(uint32_t addr, float a, float b) {
    asm volatile("st.shared.v2.f32 [%0+%1], {%2,%3};" ::"r"(addr), "n"(OFF), "f"(a), "f"(b) : "memory");
}
template <int OFF>
__device__ __forceinline__ void sts128f(uint32_t addr, float a, float b, float c, float d) {
    asm volatile("st.shared.v4.f32 [%0+%1], {%2,%3,%4,%5};" ::"r"(addr), "n"(OFF), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
template <int OFF>
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0+%1], {%2,%3,%4,%5};" ::"r"(addr), "n"(OFF), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

}  // namespace ttq
