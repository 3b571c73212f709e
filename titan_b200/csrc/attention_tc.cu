// Causal attention of prompts that start at position 0 on the tcgen05 tensor cores (head size 128).
//
// One CTA per (sequence, query head, block of 128 queries).  Per tile of 64 keys:
//     S = Q . K^T        tcgen05.mma, A = Q and B = K both K-major in shared memory, S in tensor memory
//     P = 2^(S*c - m)    eight softmax warps read S with tcgen05.ld (a thread holds half a query row)
//                        and write P (bfloat16) into shared memory in the 128-byte-swizzled K-major layout
//     O_t = P . V        tcgen05.mma, A = P (K-major), B = V as MN-major operand (V's rows are keys,
//                        its contiguous dimension is the output dimension), O_t in tensor memory
//     O = O * a + O_t    in the softmax threads' registers (64 output dims each), so tensor memory is
//                        never rescaled
// S, P and O_t are double buffered: the MMA thread issues S of the next tile before it waits for P of
// this one, and P of tile j is written while P.V of tile j - 1 still runs; its O is folded afterwards.
// Warp 0 loads Q once and K, V tiles through TMA (four stages), warp 1 allocates tensor memory and
// issues the MMAs, warps 2..9 are the softmax / output warps (two per quarter of the rows).  The step's
// own [T][Q | K | V] rows are the only source (every sequence starts at position 0); the cache is
// not read.  Tensor memory: S 2 x 64 columns, O_t 2 x 128 columns.
//
// All waits are bounded (tma.cuh); tb_attn_tc_error() reads the error word.  Built with -DTB_TC_TIMING
// (TITAN_B200_NVCC_FLAGS), one warp of the first CTA adds up clock64() per phase of the softmax loop
// (tb_attn_tc_clocks); that build is for experiments only.
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
#ifdef TB_TC_TIMING
__device__ unsigned long long g_tc_clk[16];
#define TCLK(i) do { if (timing) { const long long now_ = clock64(); atomicAdd(&g_tc_clk[i], (unsigned long long)(now_ - tprev)); tprev = now_; } } while (0)
#else
#define TCLK(i) do {} while (0)
#endif

constexpr int HD = 128, BQ = 128, BKEY = 64;
constexpr int THREADS = 320;                           // producer, MMA issuer, eight softmax / output warps
constexpr uint32_t Q_BYTES = BQ * HD * 2;              // two boxes of 128 rows x 64 columns
constexpr uint32_t Q_BOX = BQ * 128;
constexpr uint32_t KV_TILE = BKEY * HD * 2;            // one K or V tile: two boxes of 64 rows x 64 columns
constexpr uint32_t KV_BOX = BKEY * 128;
constexpr uint32_t P_BYTES = BQ * BKEY * 2;            // one box of 128 rows x 64 keys
constexpr int KV_STAGES = 4;                           // K and V tiles in flight: the loads run well ahead of P.V

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
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(KV_BOX >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// kind::f16, D float32, A and B bfloat16, M = 128; S: N = 64 keys; P.V: N = 128 dims, bit 16: B is MN-major.
constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BKEY >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&p);
}
__device__ __forceinline__ float ex2(float x) {          // 2^x, one instruction; -inf gives 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map, TcAttnArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_smem = base;                                       // 32 KB
    uint8_t* kv_smem = base + Q_BYTES;                            // KV_STAGES x (K 16 KB + V 16 KB)
    uint8_t* p_smem = kv_smem + KV_STAGES * 2 * KV_TILE;          // 2 x 16 KB
    uint64_t* bars = (uint64_t*)(p_smem + 2 * P_BYTES);
    uint64_t* q_full = bars;
    uint64_t* kv_full = bars + 1;            // [KV_STAGES]
    uint64_t* kv_empty = bars + 5;           // [KV_STAGES]
    uint64_t* s_full = bars + 9;             // [2]
    uint64_t* p_full = bars + 11;            // [2]
    uint64_t* o_full = bars + 13;            // [2]
    uint64_t* o_empty = bars + 15;           // [2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 17);
    float* sum_sh = (float*)(bars + 18);     // [2 halves][128 rows]: the halves' sums at the end

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
        for (int s = 0; s < KV_STAGES; ++s) { mbar_init(kv_full + s, 1); mbar_init(kv_empty + s, 1); }
        for (int s = 0; s < 2; ++s) {
            mbar_init(s_full + s, 1); mbar_init(p_full + s, 8); mbar_init(o_full + s, 1); mbar_init(o_empty + s, 8);
        }
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_s = tmem;             // two S buffers of 64 columns: 0..63, 64..127
    const uint32_t tmem_o = tmem + 128;       // two O buffers of 128 columns: 128..255, 256..383

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(q_full, Q_BYTES);
            tma_load_2d(q_smem, &q_map, q_full, h * HD, tok0 + r0);
            tma_load_2d(q_smem + Q_BOX, &q_map, q_full, h * HD + 64, tok0 + r0);
            for (int i = 0; i < n_tiles; ++i) {
                const int s = i % KV_STAGES;
                if (i >= KV_STAGES) wait(kv_empty + s, (i / KV_STAGES - 1) & 1, 1);
                uint8_t* kd = kv_smem + s * 2 * KV_TILE;
                const int row = tok0 + (kt0 + i) * BKEY;
                mbar_expect_tx(kv_full + s, 2 * KV_TILE);
                tma_load_2d(kd, &kv_map, kv_full + s, a.k_col0 + kh * HD, row);
                tma_load_2d(kd + KV_BOX, &kv_map, kv_full + s, a.k_col0 + kh * HD + 64, row);
                tma_load_2d(kd + KV_TILE, &kv_map, kv_full + s, a.v_col0 + kh * HD, row);
                tma_load_2d(kd + KV_TILE + KV_BOX, &kv_map, kv_full + s, a.v_col0 + kh * HD + 64, row);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t q_addr = smem_u32(q_smem), p_addr = smem_u32(p_smem);
            auto issue_s = [&](int i) {                     // S_i = Q . K_i^T into S buffer i & 1
                const int s = i % KV_STAGES;
                wait(kv_full + s, (i / KV_STAGES) & 1, 2);
                tc_fence_after();
                const uint32_t k_addr = smem_u32(kv_smem + s * 2 * KV_TILE);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)        // 16 dims per step: box ks / 4, 32 bytes per step inside it
                    tc_mma(tmem_s + (i & 1) * BKEY, desc_k_major(q_addr + (ks >> 2) * Q_BOX + (ks & 3) * 32),
                           desc_k_major(k_addr + (ks >> 2) * KV_BOX + (ks & 3) * 32), IDESC_S, ks > 0 ? 1u : 0u);
                tc_commit(s_full + (i & 1));
            };
            wait(q_full, 0, 3);
            issue_s(0);
            for (int j = 0; j < n_tiles; ++j) {
                const int b = j & 1;
                if (j + 1 < n_tiles) issue_s(j + 1);        // its S buffer was read before P of tile j - 1 was signalled
                wait(p_full + b, (j >> 1) & 1, 4);
                if (j >= 2) wait(o_empty + b, ((j >> 1) - 1) & 1, 5);   // O of tile j - 2 has been folded
                tc_fence_after();
                const uint32_t v_addr = smem_u32(kv_smem + (j % KV_STAGES) * 2 * KV_TILE + KV_TILE);
#pragma unroll
                for (int ks = 0; ks < BKEY / 16; ++ks)      // 16 keys per step: 32 bytes of a P row, 16 rows of V
                    tc_mma(tmem_o + b * HD, desc_k_major(p_addr + b * P_BYTES + ks * 32), desc_mn_major(v_addr + ks * 2048),
                           IDESC_PV, ks > 0 ? 1u : 0u);
                tc_commit(kv_empty + j % KV_STAGES);        // K_j (read by S_j) and V_j are free
                tc_commit(o_full + b);
            }
        }
    } else {
        // ---------------- softmax / output warps.  A warp may read the 32 tensor-memory lanes (query rows)
        // 32 * (warp % 4) ..; two warps share each quarter, one takes the tile's keys 0..31 and output dims
        // 0..63, the other keys 32..63 and dims 64..127.  The two agree on the row maximum through shared
        // memory once per tile; each keeps its own partial sum until the end.  P and O are double buffered:
        // P of tile j is written while the tensor core still multiplies P of tile j - 1 by V, and O of
        // tile j - 1 is folded into the registers afterwards.
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int qpos = r0 + row;
        const int lo = a.window > 0 ? qpos - a.window + 1 : 0;
        float acc[64];
#pragma unroll
        for (int d = 0; d < 64; ++d) acc[d] = 0.f;
        float m_run = -1e30f, m_acc = -1e30f, l_run = 0.f;       // m_acc: the maximum that acc is scaled to
        auto fold = [&](int b, uint32_t parity, float m_of_tile) {          // acc = acc * 2^(m_acc - m) + O_tile
            wait(o_full + b, parity, 7);
            tc_fence_after();
            float o[64];
            tmem_ld32_nowait(tmem_o + b * HD + lane_addr + half * 64, o);
            tmem_ld32_nowait(tmem_o + b * HD + lane_addr + half * 64 + 32, o + 32);
            tmem_wait_ld<64>(o);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_empty + b);
            const float f = ex2(m_acc - m_of_tile);
#pragma unroll
            for (int i = 0; i < 64; ++i) acc[i] = fmaf(acc[i], f, o[i]);
            m_acc = m_of_tile;
        };
#ifdef TB_TC_TIMING
        const bool timing = blockIdx.x == 0 && blockIdx.y == 0 && warp == 2 && lane == 0;
        long long tprev = clock64();
#endif
        for (int j = 0; j < n_tiles; ++j) {
            const int b = j & 1;
            const int key0 = (kt0 + j) * BKEY + half * 32;
            const bool tile_visible = (kt0 + j) * BKEY + BKEY - 1 <= qpos && (kt0 + j) * BKEY >= lo;   // no mask needed in this tile
            TCLK(0);
            wait(s_full + b, (j >> 1) & 1, 6);
            tc_fence_after();
            TCLK(1);
            // Both threads of a row read all 64 scores for the row maximum (tensor-memory reads are cheap, a
            // barrier between the two warps is not); each then exponentiates its own 32.
            float v[32], w[32];
            tmem_ld32_nowait(tmem_s + b * BKEY + lane_addr + half * 32, v);
            tmem_ld32_nowait(tmem_s + b * BKEY + lane_addr + (half ^ 1) * 32, w);
            tmem_wait_ld<32>(v);
            tmem_wait_ld<32>(w);
            TCLK(2);
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};     // four chains, not one of 64 links
            if (tile_visible) {
#pragma unroll
                for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], fmaxf(v[i], w[i]));
            } else {
                const int other0 = (kt0 + j) * BKEY + (half ^ 1) * 32;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    v[i] = (key0 + i <= qpos && key0 + i >= lo) ? v[i] : -INFINITY;
                    const float o = (other0 + i <= qpos && other0 + i >= lo) ? w[i] : -INFINITY;
                    mx4[i & 3] = fmaxf(mx4[i & 3], fmaxf(v[i], o));
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            TCLK(3);
            const float m_before = m_run;
            const float m_new = fmaxf(m_run, mx * a.scale_log2);
            // P = 2^(S * scale - m) as bfloat16 into the swizzled K-major tile (masked keys hold -inf: P = 0).
            // Its buffer is free: P.V of tile j - 2 had finished when its O was folded.
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                v[i] = ex2(fmaf(v[i], a.scale_log2, -m_new));
                sum4[i & 3] += v[i];
            }
            const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            uint8_t* p_row = p_smem + b * P_BYTES + row * 128;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {                // 8 keys = one 16-byte chunk of the row
                uint4 pk;
                pk.x = pack_bf16x2(v[i], v[i + 1]); pk.y = pack_bf16x2(v[i + 2], v[i + 3]);
                pk.z = pack_bf16x2(v[i + 4], v[i + 5]); pk.w = pack_bf16x2(v[i + 6], v[i + 7]);
                *reinterpret_cast<uint4*>(p_row + (((half * 4 + (i >> 3)) ^ (row & 7)) << 4)) = pk;
            }
            l_run = l_run * ex2(m_run - m_new) + sum;
            m_run = m_new;
            TCLK(4);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor core's proxy
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + b);
            TCLK(5);
            if (j >= 1) fold(b ^ 1, ((j - 1) >> 1) & 1, m_before);
            TCLK(6);         // O of tile j - 1, scaled to the maximum it was made with
        }
        fold((n_tiles - 1) & 1, ((n_tiles - 1) >> 1) & 1, m_run);
        // the two halves' sums
        sum_sh[half * 128 + row] = l_run;
        asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter));          // the two warps of this quarter
        l_run += sum_sh[(half ^ 1) * 128 + row];
        const float inv = 1.0f / l_run;
        if (qpos < n) {
            __nv_bfloat16* dst = a.out + (size_t)(tok0 + qpos) * a.out_stride + h * HD + half * 64;
#pragma unroll
            for (int i = 0; i < 64; i += 8) {
                uint4 pk;
                pk.x = pack_bf16x2(acc[i] * inv, acc[i + 1] * inv); pk.y = pack_bf16x2(acc[i + 2] * inv, acc[i + 3] * inv);
                pk.z = pack_bf16x2(acc[i + 4] * inv, acc[i + 5] * inv); pk.w = pack_bf16x2(acc[i + 6] * inv, acc[i + 7] * inv);
                *reinterpret_cast<uint4*>(dst + i) = pk;
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
    CUtensorMap q_map, kv_map;       // the same rows, cut into boxes of 128 rows (Q) and of 64 rows (K, V)
    if (tb_make_map_bf16(&q_map, a.q, a.batch.T, a.q_stride, a.q_stride, BQ)) return 1;
    if (tb_make_map_bf16(&kv_map, a.q, a.batch.T, a.q_stride, a.q_stride, BKEY)) return 1;
    TcAttnArgs p;
    p.out = (__nv_bfloat16*)a.out; p.out_stride = a.out_stride; p.q_start = a.batch.q_start; p.B = a.batch.B;
    p.nh = a.nh; p.nkv = a.nkv; p.window = a.window; p.scale_log2 = a.scale * 1.4426950408889634f;
    p.k_col0 = a.nh * a.hd; p.v_col0 = (a.nh + a.nkv) * a.hd;
    constexpr size_t smem = 1024 + Q_BYTES + KV_STAGES * 2 * KV_TILE + 2 * P_BYTES + 256 + 2 * 128 * sizeof(float);
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        TB_REQUIRE(e == cudaSuccess, "attn_prefill_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    const int blocks = (a.batch.T + BQ - 1) / BQ + a.batch.B;      // upper bound on sum over sequences of ceil(n / 128)
    TB_REQUIRE(a.nh <= 65535, "attn_prefill_tc: too many heads");
    tb_launch(attn_prefill_tc_kernel, dim3(blocks, a.nh), THREADS, smem, stream, q_map, kv_map, p);
    TB_CHECK_LAUNCH("attn_prefill_tc");
    return 0;
}

#ifdef TB_TC_TIMING
extern "C" int tb_attn_tc_clocks(unsigned long long* out16) {
    unsigned long long zero[16] = {};
    if (cudaMemcpyFromSymbol(out16, g_tc_clk, sizeof(zero)) != cudaSuccess) return 1;
    cudaMemcpyToSymbol(g_tc_clk, zero, sizeof(zero));
    return 0;
}
#endif

// Reads and clears the error word of this file's kernel (0: none).  Synchronises the device.
extern "C" int tb_attn_tc_error() {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_tc_error, sizeof(v)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_attn_tc_error, &zero, sizeof(zero));
    return (int)v;
}
