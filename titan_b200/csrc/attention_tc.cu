// Causal attention of prompts that start at position 0 on the tcgen05 tensor cores (head size 128).
//
// One CTA per (sequence, query head, block of 128 queries).  Per tile of 128 keys:
//     S = Q . K^T        tcgen05.mma, A = Q and B = K both K-major in shared memory, S in tensor memory
//     P = exp2(S*c - m)  four softmax warps, one thread per query row, read S with tcgen05.ld, write P
//                        (bfloat16) into shared memory in the 128-byte-swizzled K-major layout
//     O_t = P . V        tcgen05.mma, A = P (K-major), B = V as MN-major operand (V's rows are keys,
//                        its contiguous dimension is the output dimension), O_t in tensor memory
//     O = O * a + O_t    in the softmax threads' registers (one row of 128 each), so tensor memory
//                        is never rescaled
// S is double buffered: the MMA thread issues S of the next tile before it waits for P of this one.
// Warp 0 loads Q once and K, V tiles through TMA (two stages), warp 1 allocates tensor memory and
// issues the MMAs, warps 2..5 are the softmax / output warps.  The step's own [T][Q | K | V] rows
// are the only source (every sequence starts at position 0); the cache is not read.
//
// All waits are bounded (tma.cuh); tb_attn_tc_error() reads the error word.
//
// berniehans/titan: flash_attention_2_kernel, one warp per (head, query), one key per iteration,
// scalar FMA (engine/engine-cuda/kernels/flash_attention_2.cu:22-106).
#include <float.h>

#include "attention_args.h"
#include "common.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace {

using namespace tbtma;
using namespace tbtc;

__device__ unsigned int g_attn_tc_error = 0;

constexpr int HD = 128, BQ = 128, BKEY = 128;
constexpr int THREADS = 192;
constexpr uint32_t TILE_BYTES = 128 * HD * 2;          // one 128 x 128 bfloat16 tile: two boxes of 128 rows x 64 columns
constexpr uint32_t BOX_BYTES = 128 * 128;              // one box: 128 rows of 128 bytes
constexpr int KV_STAGES = 2;

struct TcAttnArgs {
    __nv_bfloat16* out; int out_stride;
    const int* q_start; int B;
    int nh; int nkv; int window; float scale_log2;
    int k_col0; int v_col0;
};

__device__ __forceinline__ void wait(uint64_t* bar, uint32_t parity, unsigned code) {
    tbtma::mbar_wait(bar, parity, &g_attn_tc_error, code);
}

// K-major operand tile (rows of 128 bytes, 128-byte swizzle): 8 rows per 1024 bytes.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand tile: 64 contiguous elements of the MN dimension per 128-byte row, rows are K;
// leading byte offset = distance between 64-element MN blocks (one box), stride byte offset = 8 rows.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(BOX_BYTES >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// kind::f16, D float32, A and B bfloat16, M = N = 128; bit 16 set: B is MN-major.
constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
constexpr uint32_t IDESC_PV = IDESC_S | (1u << 16);

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&p);
}

__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap qkv_map, TcAttnArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_smem = base;                                       // 32 KB
    uint8_t* kv_smem = base + TILE_BYTES;                         // stages x (K 32 KB + V 32 KB)
    uint8_t* p_smem = kv_smem + KV_STAGES * 2 * TILE_BYTES;       // 32 KB
    uint64_t* bars = (uint64_t*)(p_smem + TILE_BYTES);
    uint64_t* q_full = bars;
    uint64_t* kv_full = bars + 1;            // [2]
    uint64_t* kv_empty = bars + 3;           // [2]
    uint64_t* s_full = bars + 5;             // [2]
    uint64_t* p_full = bars + 7;
    uint64_t* o_full = bars + 8;
    uint64_t* o_empty = bars + 9;
    uint32_t* tmem_slot = (uint32_t*)(bars + 10);

    pdl_launch_dependents();
    pdl_wait();
    // which sequence and which block of 128 queries (blocks are numbered from the heaviest)
    int rem = blockIdx.x, seq = -1, blk = 0, tok0 = 0, n = 0;
    for (int s = 0; s < a.B; ++s) {
        const int t0 = a.q_start[s], ns = a.q_start[s + 1] - t0, nb = (ns + BQ - 1) / BQ;
        if (rem < nb) { seq = s; blk = nb - 1 - rem; tok0 = t0; n = ns; break; }
        rem -= nb;
    }
    if (seq < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y, kh = h / (a.nh / a.nkv);
    const int r0 = blk * BQ;
    const int last_key = min(n - 1, r0 + BQ - 1);
    const int first_key = a.window > 0 ? max(0, r0 - a.window + 1) : 0;
    const int kt0 = first_key / BKEY, n_tiles = last_key / BKEY - kt0 + 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) { mbar_init(kv_full + s, 1); mbar_init(kv_empty + s, 1); mbar_init(s_full + s, 1); }
        mbar_init(p_full, 4);
        mbar_init(o_full, 1);
        mbar_init(o_empty, 4);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_s = tmem;             // two S buffers: columns 0..127 and 128..255
    const uint32_t tmem_o = tmem + 256;       // O of one tile: columns 256..383

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(q_full, TILE_BYTES);
            tma_load_2d(q_smem, &qkv_map, q_full, h * HD, tok0 + r0);
            tma_load_2d(q_smem + BOX_BYTES, &qkv_map, q_full, h * HD + 64, tok0 + r0);
            for (int i = 0; i < n_tiles; ++i) {
                const int s = i & 1;
                if (i >= KV_STAGES) wait(kv_empty + s, ((i >> 1) - 1) & 1, 1);
                uint8_t* kd = kv_smem + s * 2 * TILE_BYTES;
                const int row = tok0 + (kt0 + i) * BKEY;
                mbar_expect_tx(kv_full + s, 2 * TILE_BYTES);
                tma_load_2d(kd, &qkv_map, kv_full + s, a.k_col0 + kh * HD, row);
                tma_load_2d(kd + BOX_BYTES, &qkv_map, kv_full + s, a.k_col0 + kh * HD + 64, row);
                tma_load_2d(kd + TILE_BYTES, &qkv_map, kv_full + s, a.v_col0 + kh * HD, row);
                tma_load_2d(kd + TILE_BYTES + BOX_BYTES, &qkv_map, kv_full + s, a.v_col0 + kh * HD + 64, row);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t q_addr = smem_u32(q_smem), p_addr = smem_u32(p_smem);
            auto issue_s = [&](int i) {                     // S_i = Q . K_i^T into S buffer i & 1
                const int s = i & 1;
                wait(kv_full + s, (i >> 1) & 1, 2);
                tc_fence_after();
                const uint32_t k_addr = smem_u32(kv_smem + s * 2 * TILE_BYTES);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {      // 16 dims per step: box ks / 4, 32 bytes per step inside it
                    const uint32_t off = (ks >> 2) * BOX_BYTES + (ks & 3) * 32;
                    tc_mma(tmem_s + s * 128, desc_k_major(q_addr + off), desc_k_major(k_addr + off), IDESC_S, ks > 0 ? 1u : 0u);
                }
                tc_commit(s_full + s);
            };
            wait(q_full, 0, 3);
            issue_s(0);
            for (int j = 0; j < n_tiles; ++j) {
                if (j + 1 < n_tiles) issue_s(j + 1);        // the other S buffer was read before P of tile j - 1 was signalled
                wait(p_full, j & 1, 4);
                if (j >= 1) wait(o_empty, (j - 1) & 1, 5);  // the softmax warps have read O of tile j - 1
                tc_fence_after();
                const uint32_t v_addr = smem_u32(kv_smem + (j & 1) * 2 * TILE_BYTES + TILE_BYTES);
#pragma unroll
                for (int ks = 0; ks < BKEY / 16; ++ks) {    // 16 keys per step
                    const uint64_t da = desc_k_major(p_addr + (ks >> 2) * BOX_BYTES + (ks & 3) * 32);
                    const uint64_t db = desc_mn_major(v_addr + ks * 2048);          // 16 key rows of 128 bytes
                    tc_mma(tmem_o, da, db, IDESC_PV, ks > 0 ? 1u : 0u);
                }
                tc_commit(kv_empty + (j & 1));              // K_j (read by S_j) and V_j are free
                tc_commit(o_full);
            }
        }
    } else {
        // ---------------- softmax / output warps: thread = query row = tensor-memory lane
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int qpos = r0 + row;
        const int lo = a.window > 0 ? qpos - a.window + 1 : 0;
        float acc[HD];
#pragma unroll
        for (int d = 0; d < HD; ++d) acc[d] = 0.f;
        float m_run = -1e30f, m_acc = -1e30f, l_run = 0.f;       // m_acc: the maximum that acc is scaled to
        uint8_t* p_row = p_smem + row * 128;
        for (int j = 0; j < n_tiles; ++j) {
            const int key0 = (kt0 + j) * BKEY;
            const uint32_t s_addr = tmem_s + (j & 1) * 128 + lane_addr;
            wait(s_full + (j & 1), (j >> 1) & 1, 6);
            tc_fence_after();
            // pass 1: the row's maximum over this tile
            float mx = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < BKEY; c += 32) {
                float v[32];
                tmem_ld32(s_addr + c, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int key = key0 + c + i;
                    if (key <= qpos && key >= lo) mx = fmaxf(mx, v[i]);
                }
            }
            const float m_new = fmaxf(m_run, mx * a.scale_log2);
            // O of the tile before: P.V of tile j - 1 has finished, so its O can be folded and P reused
            if (j >= 1) {
                wait(o_full, (j - 1) & 1, 7);
                tc_fence_after();
                const float f = exp2f(m_acc - m_run);           // m_run is still the maximum after tile j - 1
#pragma unroll
                for (int c = 0; c < HD; c += 32) {
                    float v[32];
                    tmem_ld32(tmem_o + lane_addr + c, v);
#pragma unroll
                    for (int i = 0; i < 32; ++i) acc[c + i] = fmaf(acc[c + i], f, v[i]);
                }
                m_acc = m_run;
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(o_empty);
            }
            // pass 2: P = exp2(S * scale - m), as bfloat16 into the swizzled K-major tile
            float sum = 0.f;
#pragma unroll 1
            for (int c = 0; c < BKEY; c += 32) {
                float v[32];
                tmem_ld32(s_addr + c, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int key = key0 + c + i;
                    const float p = (key <= qpos && key >= lo) ? exp2f(fmaf(v[i], a.scale_log2, -m_new)) : 0.f;
                    v[i] = p;
                    sum += p;
                }
#pragma unroll
                for (int i = 0; i < 32; i += 8) {            // 8 keys = one 16-byte chunk of the row
                    const int chunk = (c + i) >> 3;          // 0..15 over the 128 keys
                    uint4 pk;
                    pk.x = pack_bf16x2(v[i], v[i + 1]); pk.y = pack_bf16x2(v[i + 2], v[i + 3]);
                    pk.z = pack_bf16x2(v[i + 4], v[i + 5]); pk.w = pack_bf16x2(v[i + 6], v[i + 7]);
                    *reinterpret_cast<uint4*>(p_row + (chunk >> 3) * BOX_BYTES + (((chunk & 7) ^ (row & 7)) << 4)) = pk;
                }
            }
            l_run = l_run * exp2f(m_run - m_new) + sum;
            m_run = m_new;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor core's proxy
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        // the last tile's O
        wait(o_full, (n_tiles - 1) & 1, 8);
        tc_fence_after();
        const float f = exp2f(m_acc - m_run);
        const float inv = 1.0f / l_run;
        __nv_bfloat16* o = a.out + (size_t)(tok0 + qpos) * a.out_stride + h * HD;
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
            float v[32];
            tmem_ld32(tmem_o + lane_addr + c, v);
            if (qpos < n) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 pk;
                    pk.x = pack_bf16x2(fmaf(acc[c + i], f, v[i]) * inv, fmaf(acc[c + i + 1], f, v[i + 1]) * inv);
                    pk.y = pack_bf16x2(fmaf(acc[c + i + 2], f, v[i + 2]) * inv, fmaf(acc[c + i + 3], f, v[i + 3]) * inv);
                    pk.z = pack_bf16x2(fmaf(acc[c + i + 4], f, v[i + 4]) * inv, fmaf(acc[c + i + 5], f, v[i + 5]) * inv);
                    pk.w = pack_bf16x2(fmaf(acc[c + i + 6], f, v[i + 6]) * inv, fmaf(acc[c + i + 7], f, v[i + 7]) * inv);
                    *reinterpret_cast<uint4*>(o + c + i) = pk;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace

// 0 if the tcgen05 prompt kernel takes this problem, else 1 with the reason in tb_last_error().
extern "C" int tb_attn_prefill_tc_check(const AttnArgs* a, int dtype, int all_fresh) {
    TB_REQUIRE(dtype == TB_BF16, "attn_prefill_tc: bfloat16 only");
    TB_REQUIRE(all_fresh, "attn_prefill_tc: a sequence continues from the cache");
    TB_REQUIRE(a->hd == HD, "attn_prefill_tc: head_dim %d is not %d", a->hd, HD);
    TB_REQUIRE(a->nkv > 0 && a->nh % a->nkv == 0, "attn_prefill_tc: heads");
    TB_REQUIRE(a->kv_new && a->q_stride == a->kv_stride && a->q_stride % 8 == 0, "attn_prefill_tc: Q, K and V must be columns of one row-major buffer");
    TB_REQUIRE(((uintptr_t)a->q & 15) == 0, "attn_prefill_tc: the buffer must be 16-byte aligned");
    const long long off = ((const char*)a->kv_new - (const char*)a->q) / 2;
    TB_REQUIRE(off == (long long)a->nh * a->hd, "attn_prefill_tc: K must follow Q in the buffer");
    TB_REQUIRE(a->out_stride % 8 == 0 && ((uintptr_t)a->out & 15) == 0, "attn_prefill_tc: the output must be 16-byte aligned");
    return 0;
}

extern "C" int tb_attn_prefill_tc(const AttnArgs* args, int all_fresh, cudaStream_t stream) {
    const AttnArgs& a = *args;
    if (tb_attn_prefill_tc_check(args, TB_BF16, all_fresh)) return 1;
    TB_REQUIRE(a.batch.T > 0 && a.batch.B > 0, "attn_prefill_tc: no tokens");
    CUtensorMap map;
    if (tb_make_map_bf16(&map, a.q, a.batch.T, a.q_stride, a.q_stride, 128)) return 1;
    TcAttnArgs p;
    p.out = (__nv_bfloat16*)a.out; p.out_stride = a.out_stride; p.q_start = a.batch.q_start; p.B = a.batch.B;
    p.nh = a.nh; p.nkv = a.nkv; p.window = a.window; p.scale_log2 = a.scale * 1.4426950408889634f;
    p.k_col0 = a.nh * a.hd; p.v_col0 = (a.nh + a.nkv) * a.hd;
    constexpr size_t smem = 1024 + (size_t)(2 + KV_STAGES * 2) * TILE_BYTES + 128;
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        TB_REQUIRE(e == cudaSuccess, "attn_prefill_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    const int blocks = (a.batch.T + BQ - 1) / BQ + a.batch.B;      // upper bound on sum over sequences of ceil(n / 128)
    TB_REQUIRE(a.nh <= 65535, "attn_prefill_tc: too many heads");
    tb_launch(attn_prefill_tc_kernel, dim3(blocks, a.nh), THREADS, smem, stream, map, p);
    TB_CHECK_LAUNCH("attn_prefill_tc");
    return 0;
}

// Reads and clears the error word of this file's kernel (0: none).  Synchronises the device.
extern "C" int tb_attn_tc_error() {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_tc_error, sizeof(v)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_attn_tc_error, &zero, sizeof(zero));
    return (int)v;
}
