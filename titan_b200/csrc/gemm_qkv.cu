// The Q | K | V projection of a decode step with everything that follows it up to the cache, in one kernel:
//     (x . W^T) per head  ->  RMSNorm over the head (Q and K)  ->  half-split rotary  ->  Q rows out,
//     K and V rows into the paged cache.
// Weights sit on the 128-row side of the MMA (one 128-row tile = one head of 128), the step's tokens
// (at most 16) on the narrow side, as in gemm_tc.cu's swap mode.  The K dimension is cut into slices so
// that the machine is full; the slices of a head are the CTAs of one thread-block cluster.  Each leaves
// its partial sums (float32) in its own shared memory, and after a cluster barrier the CTAs share out
// the tokens: for a token, 128 threads add the slices' sums in slice order through distributed shared
// memory, so a thread holds one element of the finished head, and norm, rotation and the stores follow
// as in qk_norm_rope (elementwise.cu).  Against product -> float32 atomics -> qk_norm_rope this saves
// a kernel, the accumulation buffer's round trip and its zeroing, and the sum no longer depends on the
// order in which atomics arrive.
//
// Measured (Qwen3-8B sizes, batch 8, 8,192 keys, 36 layers): 4.49 to 4.59 ms per decode step with 2 to 8
// slices against 4.42 ms for the three separate kernels, so the engine's default stays "split": the two
// cluster barriers and the co-scheduling of a cluster's CTAs cost more than the saved launch, and a
// cluster of CTAs that each hold half an SM's shared memory starts later behind the previous kernel.
// The kernel is kept as the option qkv="fused" (deterministic sums) and is tested like the others.
//
// berniehans/titan: a quantised GEMV per projection, then qk_norm_rope_kernel and the KV append
// (engine/engine-cuda/kernels/norm_rope.cu:83-117, 226-245).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "qk_args.h"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace {

using namespace tbtc;
using namespace tbtma;

__device__ unsigned int g_qkv_error = 0;

constexpr int BM = 128, BN = 16, BK = 64, STAGES = 6, THREADS = 192;
constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
// After the main loop the ring is drained, and its first stage holds the slice's sums instead:
// [16 tokens][128] float32, then [128] for the rotation's partner and [4] sums of squares (9 KB of 16).
constexpr size_t SMEM = 1024 + (size_t)STAGES * (A_BYTES + B_BYTES) + 256;      // two CTAs per SM

struct QkvArgs {
    QkArgs q;
    int K; int k_blocks_per_split; int n_splits; int M;
};

__device__ __forceinline__ void wait(uint64_t* bar, uint32_t parity, unsigned code) { tbtma::mbar_wait(bar, parity, &g_qkv_error, code); }
// K-major tile whose rows are 128 bytes, 128-byte swizzled (the descriptors of gemm_tc.cu)
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__global__ void __launch_bounds__(THREADS)
gemm_qkv_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, QkvArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = base;
    uint8_t* smem_b = base + STAGES * A_BYTES;
    uint64_t* full = (uint64_t*)(base + STAGES * (A_BYTES + B_BYTES));
    uint64_t* empty = full + STAGES;
    uint64_t* accum = empty + STAGES;
    uint32_t* tmem_slot = (uint32_t*)(accum + 1);
    float* part = (float*)base;                          // [16][128] this slice's sums (over the drained first stage)
    float* xs = part + 16 * 128;                         // [128] a head, for the rotation's partner
    float* red = xs + 128;                               // [4] sums of squares of the four warps

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.y;                         // head: Q heads, then K heads, then V heads
    const int split = blockIdx.z;
    const int kb_total = (a.K + BK - 1) / BK;
    const int kb0 = split * a.k_blocks_per_split;
    const int n_kb = max(0, min(kb_total, kb0 + a.k_blocks_per_split) - kb0);

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        mbar_init(accum, 1);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, 32);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0 && n_kb > 0) {
            const int pre = n_kb < STAGES ? n_kb : STAGES;
            const uint64_t once = l2_evict_first_policy();               // every weight is read once per step
            for (int i = 0; i < pre; ++i) {                              // weights first: no kernel writes them
                mbar_expect_tx(full + i, A_BYTES + B_BYTES);
                tma_load_2d_hint(smem_a + i * A_BYTES, &map_w, full + i, (kb0 + i) * BK, tile * BM, once);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i) tma_load_2d(smem_b + i * B_BYTES, &map_x, full + i, (kb0 + i) * BK, 0);
            for (int i = pre; i < n_kb; ++i) {
                const int s = i % STAGES, round = i / STAGES;
                wait(empty + s, (round - 1) & 1, 1);
                mbar_expect_tx(full + s, A_BYTES + B_BYTES);
                tma_load_2d_hint(smem_a + s * A_BYTES, &map_w, full + s, (kb0 + i) * BK, tile * BM, once);
                tma_load_2d(smem_b + s * B_BYTES, &map_x, full + s, (kb0 + i) * BK, 0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n_kb > 0) {
            pdl_wait();
            for (int i = 0; i < n_kb; ++i) {
                const int s = i % STAGES, round = i / STAGES;
                wait(full + s, round & 1, 2);
                tc_fence_after();
                const uint64_t da = smem_desc(smem_u32(smem_a + s * A_BYTES)), db = smem_desc(smem_u32(smem_b + s * B_BYTES));
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) tc_mma(tmem, da + 2 * k, db + 2 * k, IDESC, (i > 0 || k > 0) ? 1u : 0u);
                tc_commit(empty + s);
            }
            tc_commit(accum);
        }
    }
    // ---- epilogue warps.  What depends on a token alone (its angle's sine and cosine, where its row lies in
    // the cache: chains of dependent loads) is fetched while the main loop runs, for the first PRE tokens
    // this CTA will finish; only then do they wait for the accumulator.
    constexpr int PRE = 4;
    const QkArgs& q = a.q;
    const int n = (warp & 3) * 32 + lane;                  // element of the head (epilogue warps)
    const bool is_q = tile < q.nh, is_k = !is_q && tile < q.nh + q.nkv;
    const int rank = (int)cluster_rank();
    float cs[PRE], sn[PRE];
    long long roff[PRE];
    auto token_facts = [&](int m, float& c, float& s_, long long& off) {
        const int pos = q.pos_of[m], seq = q.seq_of[m];
        c = 1.f; s_ = 0.f; off = -1;
        if (q.inv_freq && (is_q || is_k)) sincosf((float)pos * q.inv_freq[n & 63], &s_, &c);
        if (!is_q && !(q.cache.ring_rows && q.kv_len && pos < q.kv_len[seq] - q.cache.ring_rows)) {
            const int head = is_k ? tile - q.nh : tile - q.nh - q.nkv;
            off = (long long)((is_k ? 0 : kv_half_elems(q.cache)) + kv_row_offset(q.cache, q.slot_of_seq[seq], pos, head));
        }
    };
    if (warp >= 2) {
        pdl_wait();
#pragma unroll
        for (int j = 0; j < PRE; ++j) {
            const int m = rank + j * a.n_splits;
            cs[j] = 1.f; sn[j] = 0.f; roff[j] = -1;
            if (m < a.M) token_facts(m, cs[j], sn[j], roff[j]);
        }
        const int quarter = warp & 3;                      // a warp reads TMEM lanes 32 * (warp % 4) ..
        float v[16];
        if (n_kb > 0) {
            wait(accum, 0, 3);
            tc_fence_after();
            tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16), v);
        } else {
#pragma unroll
            for (int m = 0; m < 16; ++m) v[m] = 0.f;
        }
#pragma unroll
        for (int m = 0; m < 16; ++m) part[m * 128 + n] = v[m];
    }
    pdl_wait();
    tc_fence_before();
    cluster_sync();                                        // every slice's sums are in its shared memory

    if (warp >= 2) {
        const float* w = is_q ? q.q_w : (is_k ? q.k_w : nullptr);
        const float wn = w ? w[n] : 1.f;
        auto finish = [&](int m, float c, float s_, long long off) {
            float x = 0.f;
            for (int r = 0; r < a.n_splits; ++r) x += ld_cluster_f32(cluster_addr(part + m * 128 + n, r));   // in slice order
            if (is_q || is_k) {
                if (w) {
                    float ss = x * x;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    if (lane == 0) red[warp & 3] = ss;
                    asm volatile("bar.sync 2, 128;" ::: "memory");
                    ss = (red[0] + red[1]) + (red[2] + red[3]);
                    x = x * (1.0f / sqrtf(ss / 128.f + q.eps)) * wn;
                }
                if (q.inv_freq) {
                    xs[n] = x;
                    asm volatile("bar.sync 2, 128;" ::: "memory");
                    const float other = xs[n ^ 64];
                    x = n < 64 ? x * c - other * s_ : other * s_ + x * c;
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");           // red and xs may be written again
            }
            if (is_q) ((__nv_bfloat16*)q.q_out)[(size_t)m * q.q_stride + tile * 128 + n] = __float2bfloat16_rn(x);
            else if (off >= 0) ((__nv_bfloat16*)q.cache.storage)[off + n] = __float2bfloat16_rn(x);
        };
#pragma unroll
        for (int j = 0; j < PRE; ++j) {                    // this CTA's tokens: rank, rank + slices, ...
            const int m = rank + j * a.n_splits;
            if (m < a.M) finish(m, cs[j], sn[j], roff[j]);
        }
        for (int m = rank + PRE * a.n_splits; m < a.M; m += a.n_splits) {   // (more than PRE per CTA: few slices, many tokens)
            float c, s_;
            long long off;
            token_facts(m, c, s_, off);
            finish(m, c, s_, off);
        }
    }
    cluster_sync();                                        // nobody leaves while its sums are still being read
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 32);
    }
}

int check(int M, int N, int K, int ldx, const void* X, const void* W, const QkArgs& q, int out_dtype) {
    TB_REQUIRE(M > 0 && M <= BN, "gemm_qkv: %d tokens (at most %d)", M, BN);
    TB_REQUIRE(q.hd == 128 && (q.rot == 128 || !q.inv_freq), "gemm_qkv: heads of 128 with the rotation over the whole head");
    TB_REQUIRE(N == (q.nh + 2 * q.nkv) * 128 && q.nh > 0 && q.nkv > 0, "gemm_qkv: N=%d is not (%d + 2 * %d) heads of 128", N, q.nh, q.nkv);
    TB_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)X & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_qkv: operands must be 16-byte aligned rows");
    TB_REQUIRE(out_dtype == TB_BF16, "gemm_qkv: bfloat16 queries and cache only");
    TB_REQUIRE(q.append && q.cache.storage && q.cache.head_dim == 128 && q.cache.kv_heads == q.nkv && !q.k_out && q.q_out,
               "gemm_qkv: K and V go to the cache (single-token steps), Q to its buffer");
    TB_REQUIRE(q.T == M, "gemm_qkv: %d tokens in the arguments, %d rows", q.T, M);
    return 0;
}

}  // namespace

extern "C" int tb_gemm_qkv_check(int M, int N, int K, int ldx, const void* X, const void* W, const QkArgs* q, int out_dtype) {
    return check(M, N, K, ldx, X, W, *q, out_dtype);
}

// X [M][ldx] bfloat16 (M <= 16), W [N][K] bfloat16 with N = (nh + 2 nkv) * 128; the rest as tb_qk_norm_rope.
extern "C" int tb_gemm_qkv(const void* X, const void* W, int M, int N, int K, int ldx, const QkArgs* q, int out_dtype, cudaStream_t stream) {
    if (check(M, N, K, ldx, X, W, *q, out_dtype)) return 1;
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
    }
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_qkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
        cudaFuncSetAttribute(gemm_qkv_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        TB_REQUIRE(e == cudaSuccess, "gemm_qkv: cannot reserve %zu bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
        configured = true;
    }
    const int tiles = N / BM, kb = (K + BK - 1) / BK;
    int s = 2 * sm_count / tiles;                         // two CTAs fit an SM: fill the machine once
    const int max_s = kb / 4 > 0 ? kb / 4 : 1;            // at least four 64-wide blocks per slice
    s = s < 1 ? 1 : (s > 8 ? 8 : s);                      // a portable cluster holds 8 CTAs
    s = s > max_s ? max_s : s;
    QkvArgs a;
    a.q = *q; a.K = K; a.M = M;
    a.k_blocks_per_split = (kb + s - 1) / s;
    a.n_splits = (kb + a.k_blocks_per_split - 1) / a.k_blocks_per_split;      // no empty slice
    CUtensorMap mw, mx;
    if (tb_make_map_bf16(&mw, W, N, K, K, BM) || tb_make_map_bf16(&mx, X, M, K, ldx, BN)) return 1;
    TB_REQUIRE(tiles <= 65535, "gemm_qkv: too many heads");
    const cudaError_t e = tb_launch_cluster_z(gemm_qkv_kernel, dim3(1, tiles, a.n_splits), THREADS, SMEM, stream, a.n_splits, mw, mx, a);
    TB_REQUIRE(e == cudaSuccess, "gemm_qkv: launch failed: %s", cudaGetErrorString(e));
    TB_CHECK_LAUNCH("gemm_qkv");
    return 0;
}

// Reads and clears the error word of this file's kernel (0: none).  Synchronises the device.
extern "C" int tb_gemm_qkv_error() {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_qkv_error, sizeof(v)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_qkv_error, &zero, sizeof(zero));
    return (int)v;
}
