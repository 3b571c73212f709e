// Device-side wrappers around mbarrier and TMA (cp.async.bulk.tensor) PTX, shared by the kernels that
// stage tiles through shared memory, and the host-side tensor-map maker.
//
// Every wait is bounded: after ``limit`` polls the waiting thread records ``code`` in ``*error_word``
// (first error wins) and returns, so a kernel always ends; its result is then invalid and the host,
// which reads the word, says so.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tbtma {

#ifndef TB_WAIT_LIMIT_LOG2
#define TB_WAIT_LIMIT_LOG2 18
#endif
constexpr uint32_t WAIT_LIMIT = 1u << TB_WAIT_LIMIT_LOG2;      // try_wait rounds; each lasts up to the hardware's time limit

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// mbarrier.try_wait suspends the thread in hardware until the phase completes or a system time limit
// (microseconds) passes, so a waiter wakes as soon as the barrier flips; no sleep of our own is added.
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, unsigned int* error_word, unsigned code) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try(bar, parity)) return;
        if ((i & 255u) == 255u && *(volatile unsigned int*)error_word) break;     // another wait gave up already
    }
    atomicCAS(error_word, 0u, code);
}
// One 2-D tile: x = coordinate along the contiguous dimension (x * element size must be a multiple of
// 16 bytes), y = row.  Rows and columns outside the tensor arrive as zeros.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// Data that is read once (weights in a decode step, the cache's pages) should leave L2 first.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void tma_load_2d_hint(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(policy) : "memory");
}

// ---- clusters of two CTAs
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The shared::cluster address of the same variable in CTA ``rank`` of the cluster.
__device__ __forceinline__ uint32_t cluster_addr(const void* p, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(p)), "r"(rank));
    return a;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_addr_) {      // another CTA's shared memory
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr_) : "memory");
    return v;
}
// A value into another CTA's shared memory that counts its four bytes on a barrier of THAT CTA when it has landed:
// the receiver expects the bytes of all its senders and needs no arrival after them.
__device__ __forceinline__ void st_async_f32(uint32_t cluster_addr_, float v, uint32_t cluster_bar_addr) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %1, [%2];"
                 ::"r"(cluster_addr_), "f"(v), "r"(cluster_bar_addr) : "memory");
}
// Split cluster barrier: every thread of the cluster arrives (does not block) and, later, waits.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
// A wait that also sees what other CTAs of the cluster wrote into this CTA's shared memory (st_async_f32 counts its
// bytes on the barrier; an arrival by mbar_arrive_cluster releases at cluster scope): it acquires at cluster scope.
// Bounded like mbar_wait.
__device__ __forceinline__ void mbar_wait_cluster(uint64_t* bar, uint32_t parity, unsigned int* error_word, unsigned code) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (ok) return;
        if ((i & 255u) == 255u && *(volatile unsigned int*)error_word) break;
    }
    atomicCAS(error_word, 0u, code);
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar_addr) : "memory");
}
// A tile into this CTA's shared memory whose bytes are counted on a barrier of the pair's leader
// (``cluster_bar_addr`` from cluster_addr(bar, 0)); no multicast: each CTA loads what it needs itself.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t cluster_bar_addr, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(cluster_bar_addr), "r"(x), "r"(y) : "memory");
}

}  // namespace tbtma

// A [rows][cols] bfloat16 matrix with row stride ``stride`` elements, cut into boxes of
// box_rows x 64 elements (128 bytes), 128-byte swizzle, zero fill.  Cached by arguments.  0 on success.
int tb_make_map_bf16(CUtensorMap* out, const void* ptr, long long rows, long long cols, long long stride, int box_rows);
