// Causal attention of prompts and of continuation chunks on the tcgen05 tensor cores (head size 128).
//
// One CTA per (sequence, query head, block of 128 queries).  Per tile of 64 keys:
//     S = Q . K^T        tcgen05.mma, A = Q and B = K both K-major in shared memory, S in tensor memory
//     P = 2^(S*c - m)    a softmax thread reads its query row of S with tcgen05.ld and writes P (pairs of
//                        bfloat16) back over the first half of the same columns with tcgen05.st
//     O += P . V         tcgen05.mma with A = P from tensor memory, B = V as MN-major operand from shared
//                        memory (V's rows are keys, its contiguous dimension is the output dimension),
//                        O accumulated in tensor memory
// The eight softmax warps form two groups of four (a thread = a query row); group g takes the key tiles
// j with j % 2 == g as an online softmax of its own: its own running maximum and sum, and its own O in
// tensor memory.  A row's maximum is raised only when a tile exceeds it by more than
// 2^RESCALE_LOG2 (P stays below that bound, which bfloat16 and the float32 sum hold easily); only then is
// the group's O rescaled in tensor memory, which after the first tiles is rare.  At the end the groups'
// (m, l, O) are merged like the parts of a split-key decode.  So a thread reads each score once,
// nothing passes through registers per tile but the scores, and a group has a whole tile's time of
// slack before its next scores are needed.
// Warp 0 loads Q once and K and V tiles through TMA (rings of four each: K_j is free as soon as S_j is
// done and is wanted four tiles ahead, V_j only after P.V).  Warp 1 allocates tensor memory and issues
// the S MMAs of the even tiles, warp 11 those of the odd tiles, into four S buffers, up to four tiles
// ahead (a buffer is free again when the P.V of the tile it held is complete); warp 10 issues the P.V
// MMAs.  The issue is split three ways because the issuing thread is the narrow place: a tcgen05.mma
// costs it tens of cycles however small the product.  One tcgen05.commit per event: "S_j done" serves the
// softmax group and the K ring, "P.V_j done" the V ring, the S issuer and (for a rescale, and at the
// end) the group.  Warps 2..9 are the softmax groups.  The step's own [T][Q | K | V] rows are the
// only source (every sequence starts at position 0); the cache is not read.  The grid runs over heads
// fastest, so the heaviest query blocks of all heads start first and the lightest make the tail.
// Tensor memory: S (then P) 4 x 64 columns, O 2 x 128 columns (all 512).
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

constexpr int HD = 128, BQ = 128, BKEY = 64;
constexpr int THREADS = 384;                           // producer, S issuer (even tiles), eight softmax warps, P.V issuer, S issuer (odd tiles)
constexpr uint32_t Q_BYTES = BQ * HD * 2;              // two boxes of 128 rows x 64 columns
constexpr uint32_t Q_BOX = BQ * 128;
constexpr uint32_t KV_TILE = BKEY * HD * 2;            // one K or V tile: two boxes of 64 rows x 64 columns
constexpr uint32_t KV_BOX = BKEY * 128;
constexpr int KV_STAGES = 4;                           // K and V tiles in flight: the loads run well ahead of P.V

struct TcAttnArgs {
    __nv_bfloat16* out; int out_stride;
    const int* q_start; int B;
    int nh; int nkv; int window; float scale_log2;
    int k_col0; int v_col0;
    // keys and values from the cache (continuation steps): the first position of each sequence's rows, its slot,
    // the block table, and the row of the first V page in the cache's tensor map; paged = 0: from the step's rows
    int paged; const int* start_pos; const int* slot_of_seq; const int* table; int table_width; int v_row0;
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
__device__ __forceinline__ float max3(float a, float b, float c) {      // one instruction on sm_100
    float y;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
    return y;
}
__device__ __forceinline__ float ex2(float x) {          // 2^x, one instruction; -inf gives 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

constexpr float RESCALE_LOG2 = 8.0f;

// Barriers and why no waiter can fall behind.  A parity wait only tells "the phase with this parity is
// over" from the barrier's CURRENT phase, so a waiter must see phase k before phase k + 1 ends; every
// barrier below keeps that by construction (tile j uses slot j % 4; a slot's phases are tiles j, j + 4, ..).
//   k_full[s], v_full[s]   TMA bytes of K_j, V_j.  Waited by the S issuer of tile j / the P.V issuer.  The
//                          next load into the slot needs s_done / pv_done of tile j, i.e. the MMAs that
//                          the waiter issued after its wait.
//   s_done[s]              tcgen05.commit after S_j.  Waited by the softmax group of tile j (every phase)
//                          and polled by the producer for K_{j+4}; S_{j+4} needs that K tile and pv_done(j),
//                          which needs the group's P_j.
//   p_full[g]              four arrivals (the group's warps) per tile of group g.  Waited by the P.V issuer,
//                          every phase.  The group arrives for tile j only after pv_done(j - 2): without
//                          that, a group that never rescales could arrive for j and j + 2 before the
//                          issuer had looked once (an intermittent deadlock on long prompts).
//   pv_done[s]             tcgen05.commit after P.V_j.  Polled by the producer for V_{j+4}, waited by the S
//                          issuer of tile j + 4 (both every phase) and by the group of tile j + 2 before it
//                          arrives (and before a rescale, and once after its last tile); P.V_{j+4} needs
//                          all three to have moved on.

__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map, TcAttnArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_smem = base;                                       // 32 KB
    uint8_t* kv_smem = base + Q_BYTES;                            // KV_STAGES x (K 16 KB + V 16 KB)
    uint64_t* bars = (uint64_t*)(kv_smem + KV_STAGES * 2 * KV_TILE);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;             // [4] K and V have rings of their own: K_j is free as soon as S_j is
    uint64_t* v_full = bars + 5;             // [4] done, long before V_j, and is wanted four tiles ahead
    uint64_t* s_done = bars + 9;             // [4] S of tile j is in tensor-memory buffer j % 4 (and K stage j % 4 is free)
    uint64_t* pv_done = bars + 13;           // [4] P.V of tile j is complete: V stage j % 4 and S buffer j % 4 are free, O holds it
    uint64_t* p_full = bars + 17;            // [2] the group's four warps have written P
    uint32_t* tmem_slot = (uint32_t*)(bars + 19);
    float* ml_sh = (float*)(bars + 20);      // [2 groups][m, l][128 rows]

    pdl_launch_dependents();
    pdl_wait();
    // blockIdx.y: which sequence and which block of 128 queries (a sequence's blocks from the heaviest,
    // the last, down); blockIdx.x, which runs fastest in the dispatch order: the head
    int rem = blockIdx.y, seq = -1, blk = 0, tok0 = 0, n = 0;
    for (int s = 0; s < a.B; ++s) {
        const int t0 = a.q_start[s], ns = a.q_start[s + 1] - t0, nb = (ns + BQ - 1) / BQ;
        if (rem < nb) { seq = s; blk = nb - 1 - rem; tok0 = t0; n = ns; break; }
        rem -= nb;
    }
    if (seq < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.x, kh = h / (a.nh / a.nkv);
    const int r0 = blk * BQ;                                      // first row of the block among the sequence's rows of this step
    const int p0 = a.paged ? a.start_pos[seq] : 0;                // position of the sequence's first row
    const int last_key = p0 + min(n - 1, r0 + BQ - 1);
    const int first_key = a.window > 0 ? max(0, p0 + r0 - a.window + 1) : 0;
    const int kt0 = first_key / BKEY, n_tiles = last_key / BKEY - kt0 + 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(k_full + s, 1); mbar_init(v_full + s, 1); mbar_init(s_done + s, 1); mbar_init(pv_done + s, 1);
        }
        for (int s = 0; s < 2; ++s) mbar_init(p_full + s, 4);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_s = tmem;             // S of tile j: columns 64 (j % 4) ..; a group owns two of the four buffers
    const uint32_t tmem_o = tmem + 256;       // O of group g: columns 256 + 128 g ..

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(q_full, Q_BYTES);
            tma_load_2d(q_smem, &q_map, q_full, h * HD, tok0 + r0);
            tma_load_2d(q_smem + Q_BOX, &q_map, q_full, h * HD + 64, tok0 + r0);
            // K and V tiles as their rings allow, whichever is free first (bounded polling)
            const int* tab = a.paged ? a.table + (size_t)a.slot_of_seq[seq] * a.table_width : nullptr;
            const int kx = a.paged ? 0 : a.k_col0 + kh * HD, vx = a.paged ? 0 : a.v_col0 + kh * HD;
            int ki = 0, vi = 0;
            for (uint32_t spin = 0; (ki < n_tiles || vi < n_tiles) && spin < (tbtma::WAIT_LIMIT << 4); ++spin) {
                if (ki < n_tiles && (ki < KV_STAGES || tbtma::mbar_test(s_done + ki % KV_STAGES, (ki / KV_STAGES - 1) & 1))) {
                    const int s = ki % KV_STAGES;
                    const int row = a.paged ? (tab[kt0 + ki] * a.nkv + kh) * BKEY : tok0 + (kt0 + ki) * BKEY;
                    uint8_t* kd = kv_smem + s * 2 * KV_TILE;
                    mbar_expect_tx(k_full + s, KV_TILE);
                    tma_load_2d(kd, &kv_map, k_full + s, kx, row);
                    tma_load_2d(kd + KV_BOX, &kv_map, k_full + s, kx + 64, row);
                    ++ki; spin = 0;
                }
                if (vi < n_tiles && (vi < KV_STAGES || tbtma::mbar_test(pv_done + vi % KV_STAGES, (vi / KV_STAGES - 1) & 1))) {
                    const int s = vi % KV_STAGES;
                    const int row = a.paged ? a.v_row0 + (tab[kt0 + vi] * a.nkv + kh) * BKEY : tok0 + (kt0 + vi) * BKEY;
                    uint8_t* vd = kv_smem + s * 2 * KV_TILE + KV_TILE;
                    mbar_expect_tx(v_full + s, KV_TILE);
                    tma_load_2d(vd, &kv_map, v_full + s, vx, row);
                    tma_load_2d(vd + KV_BOX, &kv_map, v_full + s, vx + 64, row);
                    ++vi; spin = 0;
                }
            }
            if (ki < n_tiles || vi < n_tiles) atomicCAS(&g_attn_tc_error, 0u, 1u);
        }
    } else if (warp == 1 || warp == 11) {
        // ---- S issuers (warp 1: even tiles, warp 11: odd tiles): S_i = Q . K_i^T into S buffer i % 4, up to
        // four tiles ahead of the softmax; a tile's descriptors differ from a base by constants.
        if (lane == 0) {
            const uint64_t q_desc = desc_k_major(smem_u32(q_smem));
            wait(q_full, 0, 3);
            for (int i = warp == 1 ? 0 : 1; i < n_tiles; i += 2) {
                const int s = i % KV_STAGES;
                if (i >= 4) wait(pv_done + (i & 3), ((i >> 2) - 1) & 1, 9);       // the buffer held S, then P, of tile i - 4
                wait(k_full + s, (i / KV_STAGES) & 1, 2);
                tc_fence_after();
                const uint64_t k_desc = desc_k_major(smem_u32(kv_smem + s * 2 * KV_TILE));
                const uint32_t d = tmem_s + (i & 3) * BKEY;
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)        // 16 dims per step: box ks / 4, 32 bytes per step inside it
                    tc_mma(d, q_desc + (uint64_t)(((ks >> 2) * Q_BOX + (ks & 3) * 32) >> 4),
                           k_desc + (uint64_t)(((ks >> 2) * KV_BOX + (ks & 3) * 32) >> 4), IDESC_S, ks > 0 ? 1u : 0u);
                tc_commit(s_done + (i & 3));                // one arrival for the softmax group and for the K ring
            }
        }
    } else if (warp == 10) {
        // ---- P.V issuer: O_g += P_j . V_j for the group g = j % 2
        if (lane == 0) {
            for (int j = 0; j < n_tiles; ++j) {
                const int g = j & 1, s = j % KV_STAGES;
                wait(v_full + s, (j / KV_STAGES) & 1, 5);
                wait(p_full + g, (j >> 1) & 1, 4);          // the group has rescaled O if it had to and written P_j
                tc_fence_after();
                const uint64_t v_desc = desc_mn_major(smem_u32(kv_smem + s * 2 * KV_TILE + KV_TILE));
                const uint32_t p_tmem = tmem_s + (j & 3) * BKEY;      // P_j lies over the first half of S_j
                const uint32_t d = tmem_o + g * HD;
#pragma unroll
                for (int ks = 0; ks < BKEY / 16; ++ks)      // 16 keys per step: 8 columns of P, 16 rows of V
                    tc_mma_a_tmem(d, p_tmem + ks * 8, v_desc + (uint64_t)((ks * 2048) >> 4), IDESC_PV, (j >= 2 || ks > 0) ? 1u : 0u);
                tc_commit(pv_done + (j & 3));               // one arrival for the V ring, the S issuer and the group
            }
        }
    } else {
        const int g = (warp - 2) >> 2, quarter = warp & 3;       // a warp may touch the tensor-memory lanes 32 * (warp % 4) ..
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int qpos = p0 + r0 + row;                          // the row's position in its sequence
        const int lo = a.window > 0 ? qpos - a.window + 1 : 0;
        float m_run = -1e30f, l_run = 0.f;                       // the maximum P is taken against (may lag), the sum
        int mine = 0;                                            // tiles of this group so far
        for (int j = g; j < n_tiles; j += 2, ++mine) {
            const int key0 = (kt0 + j) * BKEY;
            const bool tile_visible = key0 + BKEY - 1 <= qpos && key0 >= lo;       // no mask needed in this tile
            wait(s_done + (j & 3), (j >> 2) & 1, 6);
            tc_fence_after();
            float v[64];
            tmem_ld32_nowait(tmem_s + (j & 3) * BKEY + lane_addr, v);
            tmem_ld32_nowait(tmem_s + (j & 3) * BKEY + lane_addr + 32, v + 32);
            tmem_wait_ld<64>(v);
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (!tile_visible) {
#pragma unroll
                for (int i = 0; i < 64; ++i) v[i] = (key0 + i <= qpos && key0 + i >= lo) ? v[i] : -INFINITY;
            }
#pragma unroll
            for (int i = 0; i < 64; i += 8) {               // four chains of three-input maxima
                mx4[0] = max3(mx4[0], v[i], v[i + 1]); mx4[1] = max3(mx4[1], v[i + 2], v[i + 3]);
                mx4[2] = max3(mx4[2], v[i + 4], v[i + 5]); mx4[3] = max3(mx4[3], v[i + 6], v[i + 7]);
            }
            const float cand = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;
            // Raise the row's maximum only when the tile exceeds it by more than the bound.
            const bool raise = cand > m_run + RESCALE_LOG2;
            const float m_new = raise ? cand : m_run;
            const float f = raise ? ex2(m_run - m_new) : 1.f;
            // Only a rescale touches O, and only then must the group's earlier P.V be complete (P itself goes
            // into this tile's own S buffer).  f = 1 for the rows of the warp that keep their maximum.
            if (mine >= 1 && __any_sync(0xffffffffu, raise)) {
                wait(pv_done + ((j - 2) & 3), ((j - 2) >> 2) & 1, 7);
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < HD; c += 32) {
                    float o[32];
                    tmem_ld32(tmem_o + g * HD + lane_addr + c, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= f;
                    tmem_st32(tmem_o + g * HD + lane_addr + c, o);
                }
            }
            // two scores per instruction where the hardware has one (packed float32 FMA and add on sm_100):
            // the softmax warps are short of issue slots, not only of special-function units
            const float2 scale2 = make_float2(a.scale_log2, a.scale_log2), shift2 = make_float2(-m_new, -m_new);
            float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int i = 0; i < 64; i += 2) {
                const float2 x = __ffma2_rn(make_float2(v[i], v[i + 1]), scale2, shift2);
                v[i] = ex2(x.x); v[i + 1] = ex2(x.y);
                sum2[(i >> 1) & 1] = __fadd2_rn(sum2[(i >> 1) & 1], make_float2(v[i], v[i + 1]));
            }
            l_run = l_run * f + ((sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y));
            m_run = m_new;
            // P as bfloat16 pairs over the first 32 columns of this tile's S buffer (this thread's lane: its
            // scores are all in registers by now): the A operand of P.V, which never touches shared memory
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) pk[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
            tmem_st32_bits(tmem_s + (j & 3) * BKEY + lane_addr, pk);
            // The P.V issuer must have seen this group's previous arrival before the next one, or the
            // barrier would run two phases ahead of it and its parity wait would never end.  P.V of that
            // tile complete implies it; by now (a whole tile later) this wait is almost always over.
            if (mine >= 1) wait(pv_done + ((j - 2) & 3), ((j - 2) >> 2) & 1, 10);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + g);
        }
        if (mine >= 1) {                                         // the group's last P.V
            const int last = g + 2 * (mine - 1);
            wait(pv_done + (last & 3), (last >> 2) & 1, 8);
            tc_fence_after();
        }
        // merge the two groups: weights 2^(m_g - M) / L
        ml_sh[(g * 2 + 0) * 128 + row] = mine ? m_run : -1e30f;
        ml_sh[(g * 2 + 1) * 128 + row] = mine ? l_run : 0.f;
        tc_fence_before();
        asm volatile("bar.sync 1, 256;" ::: "memory");           // all eight softmax warps
        tc_fence_after();
        const float m0 = ml_sh[0 * 128 + row], l0 = ml_sh[1 * 128 + row], m1 = ml_sh[2 * 128 + row], l1 = ml_sh[3 * 128 + row];
        const float M = fmaxf(m0, m1);
        const float w0 = ex2(m0 - M), w1 = n_tiles > 1 ? ex2(m1 - M) : 0.f;
        const float inv = 1.0f / (l0 * w0 + l1 * w1);
        // this thread: output dims 64 g .. 64 g + 63 of its row, from both groups' O
        float o0[64], o1[64];
        tmem_ld32_nowait(tmem_o + lane_addr + g * 64, o0);
        tmem_ld32_nowait(tmem_o + lane_addr + g * 64 + 32, o0 + 32);
        if (n_tiles > 1) {                                       // uniform over the CTA
            tmem_ld32_nowait(tmem_o + HD + lane_addr + g * 64, o1);
            tmem_ld32_nowait(tmem_o + HD + lane_addr + g * 64 + 32, o1 + 32);
        }
        tmem_wait_ld<64>(o0);
        if (n_tiles > 1) tmem_wait_ld<64>(o1);
        if (r0 + row < n) {
            const float c0 = w0 * inv, c1 = w1 * inv;
            __nv_bfloat16* dst = a.out + (size_t)(tok0 + r0 + row) * a.out_stride + h * HD + g * 64;
#pragma unroll
            for (int i = 0; i < 64; i += 8) {
                float r[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) r[e] = n_tiles > 1 ? o0[i + e] * c0 + o1[i + e] * c1 : o0[i + e] * c0;
                uint4 pk;
                pk.x = pack_bf16x2(r[0], r[1]); pk.y = pack_bf16x2(r[2], r[3]);
                pk.z = pack_bf16x2(r[4], r[5]); pk.w = pack_bf16x2(r[6], r[7]);
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
// source: TB_KV_FROM_STEP (1): keys and values are the step's own rows, so every sequence must start at position 0;
// TB_KV_FROM_CACHE (2): they are read from the cache's pages, where the step's own keys already lie (a cache
// that keeps every key: no ring).
extern "C" int tb_attn_prefill_tc_check(const AttnArgs* a, int dtype, int source) {
    TB_REQUIRE(dtype == TB_BF16, "attn_prefill_tc: bfloat16 only");
    TB_REQUIRE(source == TB_KV_FROM_STEP || source == TB_KV_FROM_CACHE, "attn_prefill_tc: a sequence continues from the cache and its keys are not all there");
    TB_REQUIRE(a->hd == HD, "attn_prefill_tc: head_dim %d is not %d", a->hd, HD);
    TB_REQUIRE(a->nkv > 0 && a->nh % a->nkv == 0, "attn_prefill_tc: heads");
    TB_REQUIRE(a->q_stride % 8 == 0 && ((uintptr_t)a->q & 15) == 0, "attn_prefill_tc: the queries must be 16-byte aligned rows");
    if (source == TB_KV_FROM_STEP) {
        TB_REQUIRE(a->kv_new && a->q_stride == a->kv_stride, "attn_prefill_tc: Q, K and V must be columns of one row-major buffer");
        const long long off = ((const char*)a->kv_new - (const char*)a->q) / 2;
        TB_REQUIRE(off == (long long)a->nh * a->hd, "attn_prefill_tc: K must follow Q in the buffer");
    } else {
        TB_REQUIRE(a->cache.storage && a->cache.page_size == BKEY && a->cache.ring_rows == 0, "attn_prefill_tc: needs a cache of %d-row pages that keeps every key", BKEY);
        TB_REQUIRE(a->cache.head_dim == a->hd && a->cache.kv_heads == a->nkv, "attn_prefill_tc: the cache view does not match the heads");
    }
    TB_REQUIRE(a->out_stride % 8 == 0 && ((uintptr_t)a->out & 15) == 0, "attn_prefill_tc: the output must be 16-byte aligned");
    return 0;
}

extern "C" int tb_attn_prefill_tc(const AttnArgs* args, int source, cudaStream_t stream) {
    const AttnArgs& a = *args;
    if (tb_attn_prefill_tc_check(args, TB_BF16, source)) return 1;
    TB_REQUIRE(a.batch.T > 0 && a.batch.B > 0, "attn_prefill_tc: no tokens");
    CUtensorMap q_map, kv_map;       // the step's rows cut into boxes of 128 rows (Q), and of 64 rows (K, V) or the cache's pages
    if (tb_make_map_bf16(&q_map, a.q, a.batch.T, a.q_stride, a.q_stride, BQ)) return 1;
    TcAttnArgs p;
    p.paged = source == TB_KV_FROM_CACHE;
    if (p.paged) {
        const long long rows = 2LL * a.cache.num_pages * a.nkv * BKEY;
        if (tb_make_map_bf16(&kv_map, a.cache.storage, rows, a.hd, a.hd, BKEY)) return 1;
    } else if (tb_make_map_bf16(&kv_map, a.q, a.batch.T, a.q_stride, a.q_stride, BKEY)) return 1;
    p.start_pos = a.batch.start_pos; p.slot_of_seq = a.batch.slot_of_seq; p.table = a.cache.table; p.table_width = a.cache.table_width;
    p.v_row0 = a.cache.num_pages * a.nkv * BKEY;
    p.out = (__nv_bfloat16*)a.out; p.out_stride = a.out_stride; p.q_start = a.batch.q_start; p.B = a.batch.B;
    p.nh = a.nh; p.nkv = a.nkv; p.window = a.window; p.scale_log2 = a.scale * 1.4426950408889634f;
    p.k_col0 = a.nh * a.hd; p.v_col0 = (a.nh + a.nkv) * a.hd;
    constexpr size_t smem = 1024 + Q_BYTES + KV_STAGES * 2 * KV_TILE + 256 + 4 * 128 * sizeof(float);
    static_assert(KV_STAGES == 4, "the second kernel's barrier layout and S buffers assume four stages");
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        TB_REQUIRE(e == cudaSuccess, "attn_prefill_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    const int blocks = (a.batch.T + BQ - 1) / BQ + a.batch.B;      // upper bound on sum over sequences of ceil(n / 128)
    TB_REQUIRE(blocks <= 65535, "attn_prefill_tc: too many query blocks (%d)", blocks);
    tb_launch(attn_prefill_tc_kernel, dim3(a.nh, blocks), THREADS, smem, stream, q_map, kv_map, p);      // heads fastest: the heaviest blocks of all heads start first
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
