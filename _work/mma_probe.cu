// A measurement, not part of any step: how many clocks one tcgen05.mma (cta_group::1, kind::f16,
// bfloat16 operands, M = 128, K = 16) takes against its N, issued back to back by one thread per SM into
// one accumulator.  The answer decides tile shapes elsewhere in this library (which N keeps the tensor
// pipe at full rate, and what the issuing thread itself costs per instruction).
//
// berniehans/titan has no counterpart: its kernels use CUDA cores and mma.sync.
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

using namespace tbtc;
using namespace tbtma;

__device__ unsigned int g_probe_error = 0;

__global__ void __launch_bounds__(128) mma_probe_kernel(int N, int iters, long long* clocks) {
    extern __shared__ uint8_t raw[];
    uint8_t* base = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t bar;
    __shared__ uint32_t slot;
    for (int i = threadIdx.x; i < 48 * 1024 / 4; i += blockDim.x) ((uint32_t*)base)[i] = 0x3c003c00u;   // finite operands
    if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
    if (threadIdx.x < 32) tmem_alloc(&slot, 256);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = slot;
    if (threadIdx.x == 0) {
        // K-major operands, 128-byte swizzle (the descriptors of gemm_tc.cu); D float32
        auto desc = [](uint32_t addr) {
            return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
                   ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
        };
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        const uint64_t a = desc(smem_u32(base)), b = desc(smem_u32(base + 16384));
        const long long t0 = clock64();
        for (int i = 0; i < iters; ++i) tc_mma(tmem, a + 2 * (i & 3), b + 2 * (i & 3), idesc, 1u);
        tc_commit(&bar);
        mbar_wait(&bar, 0, &g_probe_error, 1);
        const long long t1 = clock64();
        if (blockIdx.x == 0) clocks[0] = t1 - t0;
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) {
        tc_fence_after();
        tmem_dealloc(tmem, 256);
    }
}

}  // namespace

// Clocks per MMA of 128 x n x 16 (n a multiple of 16 up to 256), averaged over ``iters`` instructions,
// with every SM busy.  Returns 0 and writes the figure, or 1 with the reason in tb_last_error().
extern "C" int tb_mma_probe(int n, int iters, double* clocks_per_mma) {
    TB_REQUIRE(n >= 16 && n <= 256 && n % 16 == 0, "mma_probe: N=%d must be a multiple of 16 from 16 to 256", n);
    TB_REQUIRE(iters > 0 && iters <= (1 << 20), "mma_probe: iters=%d out of range", iters);
    long long* d = nullptr;
    TB_REQUIRE(cudaMalloc(&d, sizeof(long long)) == cudaSuccess, "mma_probe: no memory");
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(mma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 50 * 1024);
    mma_probe_kernel<<<sms, 128, 50 * 1024>>>(n, iters, d);
    const cudaError_t e = cudaDeviceSynchronize();
    long long h = 0;
    cudaMemcpy(&h, d, sizeof(h), cudaMemcpyDeviceToHost);
    cudaFree(d);
    unsigned int err = 0, zero = 0;
    cudaMemcpyFromSymbol(&err, g_probe_error, sizeof(err));
    if (err) cudaMemcpyToSymbol(g_probe_error, &zero, sizeof(zero));
    TB_REQUIRE(e == cudaSuccess && err == 0, "mma_probe: %s (wait error %u)", cudaGetErrorString(e), err);
    *clocks_per_mma = (double)h / iters;
    return 0;
}
