// An optional probe for the decode kernels: with -DTB_TIMELINE every CTA of an instrumented kernel takes a record in
// a buffer that the host has named (tb_*_timeline) and stamps it with the global timer at a few points of its life:
// its start, the end of its wait for the kernel before it, its first tile, its last one, its end.  Read back after
// one replay of a captured decode step, the records show when each kernel's CTAs start, what they wait for and for
// how long (``python bench.py --timeline B`` prints them).  Without the flag the probe is empty functions: no code,
// no registers, no shared memory.
//
// Buffer (unsigned 64-bit): [0] = records taken so far; record r at 1 + 8 r: tag, block | sm << 32, stamps 0 .. 5.
#pragma once
#include <cuda_runtime.h>

#ifdef TB_TIMELINE
static __device__ unsigned long long* g_timeline_buffer = nullptr;      // one per translation unit, set by its own setter
constexpr unsigned long long TIMELINE_RECORDS = 200000ull;

struct TimelineProbe {
    unsigned long long* rec = nullptr;
    static __device__ __forceinline__ unsigned long long now() {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        return t;
    }
    // thread 0 of the CTA, before a barrier of the CTA; every thread calls attach() after that barrier
    __device__ __forceinline__ void begin(unsigned long long tag, unsigned long long block) {
        if (threadIdx.x == 0) {
            unsigned long long* slot = nullptr;
            if (g_timeline_buffer) {
                const unsigned long long r = atomicAdd(g_timeline_buffer, 1ull);
                if (r < TIMELINE_RECORDS) {
                    unsigned int sm;
                    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
                    slot = g_timeline_buffer + 1 + 8 * r;
                    slot[0] = tag; slot[1] = block | ((unsigned long long)sm << 32); slot[2] = now();
                    slot[3] = slot[4] = slot[5] = slot[6] = slot[7] = 0;
                }
            }
            shared_slot() = slot;
        }
    }
    __device__ __forceinline__ void attach() { rec = shared_slot(); }
    __device__ __forceinline__ void stamp(int k) const { if (rec) rec[2 + k] = now(); }
    static __device__ __forceinline__ unsigned long long*& shared_slot() {
        __shared__ unsigned long long* s;
        return s;
    }
};
#define TB_TIMELINE_SETTER(name) \
    extern "C" int name(void* buffer) { return cudaMemcpyToSymbol(g_timeline_buffer, &buffer, sizeof(buffer)) == cudaSuccess ? 1 : -1; }
#else
struct TimelineProbe {
    __device__ __forceinline__ void begin(unsigned long long, unsigned long long) {}
    __device__ __forceinline__ void attach() {}
    __device__ __forceinline__ void stamp(int) const {}
};
#define TB_TIMELINE_SETTER(name) extern "C" int name(void*) { return 0; }      // 0: the library was built without the probe
#endif
