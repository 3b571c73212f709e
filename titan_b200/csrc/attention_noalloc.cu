// Split-KV decode attention for callers that cannot allocate: the partials live in a fixed array of
// this file instead of a buffer the caller brings.  See attention_noalloc.h for who needs this, the
// size limit and the rules on first use and on overlapping calls.
#include <mutex>

#include "attention_noalloc.h"
#include "common.cuh"

extern "C" int tb_attn_decode(const AttnArgs* args, int dtype, cudaStream_t stream);

// In host code this name is only a stand-in for the device array: its host address must never be
// handed to a kernel.  The device address is asked for once per device, below.
static __device__ __align__(256) float g_noalloc_scratch[TB_NOALLOC_SCRATCH_FLOATS];

namespace {

constexpr int MAX_DEVICES = 64;
float* g_scratch_on_device[MAX_DEVICES] = {};
std::mutex g_setup_mutex;

// The array's address on the current device, looked up on the first call for that device.
int scratch_address(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    TB_REQUIRE(e == cudaSuccess, "attn_decode_noalloc: cudaGetDevice failed: %s", cudaGetErrorString(e));
    TB_REQUIRE(dev >= 0 && dev < MAX_DEVICES, "attn_decode_noalloc: device index %d is not below %d", dev, MAX_DEVICES);
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_on_device[dev]) {
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
        TB_REQUIRE(e == cudaSuccess && ptr, "attn_decode_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                   cudaGetErrorString(e));
        g_scratch_on_device[dev] = ptr;
    }
    *out = g_scratch_on_device[dev];
    return 0;
}

}  // namespace

extern "C" int tb_attn_decode_noalloc(const AttnArgs* args, int dtype, cudaStream_t stream) {
    TB_REQUIRE(args, "attn_decode_noalloc: no arguments");
    AttnArgs a = *args;
    TB_REQUIRE(a.batch.B > 0 && a.nh > 0 && a.n_splits > 0 && a.hd > 0, "attn_decode_noalloc: sizes must be positive");
    const unsigned long long need = (unsigned long long)a.batch.B * a.nh * a.n_splits * (a.hd + 2);
    TB_REQUIRE(need <= TB_NOALLOC_SCRATCH_FLOATS,
               "attn_decode_noalloc: %d sequences x %d heads x %d splits x (%d + 2) need %llu scratch values; the built-in "
               "scratch holds %u (use tb_attn_decode with a buffer of your own, or fewer splits)",
               a.batch.B, a.nh, a.n_splits, a.hd, need, (unsigned)TB_NOALLOC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    if (scratch_address(&scratch)) return 1;
    a.scratch = scratch;                         // the caller's field is ignored
    return tb_attn_decode(&a, dtype, stream);    // the same kernels, on the built-in scratch
}
