// Shared helpers of the sm_100a kernels: element types, reductions, error reporting.
//
// Every launcher is an extern "C" function that returns 0 or a non-zero code and
// leaves a message for tb_last_error().  Launchers validate sizes on the host and
// refuse what a kernel cannot run, so that a kernel never computes a wrong result.
// berniehans/titan checks sizes before each launch in the same spirit
// (engine/engine-cuda/src/batched_gemm.rs:1413-1450, paged_attention.rs:193-257).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <utility>

#define TB_F32 0
#define TB_BF16 1

extern "C" const char* tb_last_error();
void tb_set_error(const char* fmt, ...);

#define TB_REQUIRE(cond, ...)              \
    do {                                   \
        if (!(cond)) {                     \
            tb_set_error(__VA_ARGS__);     \
            return 1;                      \
        }                                  \
    } while (0)

#define TB_CHECK_LAUNCH(name)                                                       \
    do {                                                                            \
        cudaError_t e_ = cudaGetLastError();                                        \
        if (e_ != cudaSuccess) {                                                    \
            tb_set_error("%s: launch failed: %s", name, cudaGetErrorString(e_));    \
            return 2;                                                               \
        }                                                                           \
    } while (0)

// One view of a cache group's storage for one layer; mirrors
// titan_b200.cache.groups.KVGroup.  Storage: [2][num_pages][kv_heads][page_size][head_dim].
struct TbKvView {
    void* storage;
    const int* table;      // [max_slots][table_width] page ids
    int table_width;
    int ring_rows;         // 0: position p is row p; else row p % ring_rows
    int page_size;
    int num_pages;
    int kv_heads;
    int head_dim;
};

// The ragged batch of one step; mirrors titan_b200.engine.batch.StepLayout.
struct TbBatch {
    const int* tokens;        // [T]
    const int* seq_of;        // [T] index of the token's sequence in this batch
    const int* pos_of;        // [T] absolute position of the token
    const int* slot_of_seq;   // [B]
    const int* q_start;       // [B+1] first token index of each sequence
    const int* start_pos;     // [B] tokens already in the cache before this step
    const int* kv_len;        // [B] tokens in the cache after this step
    int T;
    int B;
    int max_new;              // largest number of new tokens of a sequence
    int max_kv_len;           // largest kv_len (host bound for grids)
};

template <typename T> struct ElemOps;
template <> struct ElemOps<float> {
    static __device__ __forceinline__ float ld(const float* p) { return *p; }
    static __device__ __forceinline__ void st(float* p, float v) { *p = v; }
};
template <> struct ElemOps<__nv_bfloat16> {
    static __device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};
template <typename T> __device__ __forceinline__ float ldf(const T* p) { return ElemOps<T>::ld(p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v) { ElemOps<T>::st(p, v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  ``red`` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// Row of the cache that holds position ``pos`` of the sequence in ``slot``:
// element offset of [page][head][row][0] inside one of the K or V halves.
__device__ __forceinline__ size_t kv_row_offset(const TbKvView& c, int slot, int pos, int head) {
    const int row = c.ring_rows ? pos % c.ring_rows : pos;
    const int page = c.table[(size_t)slot * c.table_width + row / c.page_size];
    return (((size_t)page * c.kv_heads + head) * c.page_size + (row % c.page_size)) * c.head_dim;
}
__device__ __forceinline__ size_t kv_half_elems(const TbKvView& c) {
    return (size_t)c.num_pages * c.kv_heads * c.page_size * c.head_dim;
}

// ---------------------------------------------------------------- programmatic dependent launch
// Kernels of a step are launched so that a kernel may start while its predecessor in the stream is
// still finishing (its blocks are scheduled once every block of the predecessor has called
// pdl_launch_dependents or exited).  A kernel calls pdl_wait() before it reads or writes anything an
// earlier kernel wrote; what it does before that (barrier set-up, tensor-memory allocation, loads of
// weights, which no kernel writes) overlaps the predecessor's tail.  Every kernel launched this way
// calls pdl_wait() on every path, so completion stays transitive along the stream.
extern int g_tb_pdl;      // 1: on (default); tb_set_pdl(0) launches everything fully serialised

template <typename... KArgs, typename... Args>
inline cudaError_t tb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = g_tb_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
// The same launch as a grid of thread-block clusters of (1, 1, cluster_z) CTAs (cluster_z <= 8).
template <typename... KArgs, typename... Args>
inline cudaError_t tb_launch_cluster_z(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                       int cluster_z, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = (unsigned)cluster_z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = g_tb_pdl ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
