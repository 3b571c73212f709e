// bfloat16 attention on tensor cores for the head sizes serving uses (64 and 128), pages of 64 rows.
//
//   tb_attn_decode_mma   one query per sequence over its cached keys.  One CTA per (sequence, kv
//                        head, chunk of keys): TMA brings whole K and V pages (64 keys) of that head
//                        into a ring of shared-memory stages; four warps each take 16 keys of the page,
//                        S = Q K^T and O += P V run as mma.sync.m16n8k16 with the kv head's whole
//                        group of query heads in the 16 rows of the tile, so every key and value is
//                        read from HBM once for the group.  Partials go through the same
//                        (max, sum, unnormalised output) format as the plain kernel and the same merge.
//
// A sequence's keys are cut into splits by its own length (tb_split_keys): the borders are multiples of
// the page size and depend on that length and on the launch's (fewest keys per split, most splits) only.
//
// Keys and values arrive 128-byte swizzled (tensor map of 64 x 64 boxes), which makes the ldmatrix
// reads conflict-free.  All waits are bounded (tma.cuh); tb_attn_mma_error() reads the error word.
//
// berniehans/titan: flash_decoding_split_kernel, one warp per (head, split), one key per iteration,
// scalar FMA (engine/engine-cuda/kernels/paged_attention.cu:200-309).
#include <float.h>

#include "attention_args.h"
#include "common.cuh"
#include "timeline.cuh"
#include "tma.cuh"

namespace {

using namespace tbtma;

__device__ unsigned int g_attn_error = 0;

constexpr int PAGE = 64;
constexpr int DEC_WARPS = 4;                 // compute warps; warp DEC_WARPS produces
constexpr int DEC_THREADS = (DEC_WARPS + 1) * 32;

struct DecArgs {
    const __nv_bfloat16* q; int q_stride;    // [B][q_stride]
    float* scratch;                          // [B][nh][n_splits][hd + 2]
    const int* table; int table_width; int ring_rows; int num_pages;
    const int* slot_of_seq; const int* kv_len;
    const int* early_len; int early_mode;    // lengths that were final before the step's first kernel (see AttnArgs); 0: none
    int nh; int nkv; int window; float scale_log2;   // scale * log2(e)
    int chunk; int n_splits;
    __nv_bfloat16* out; int out_stride;      // [B][out_stride]: written by the kernel itself when its splits form a cluster
    // FUSED: the projection's float32 sums [B][acc_stride] (Q heads, K heads, V heads; rows not yet scaled if row_sumsq is
    // given), which this kernel scales, norms, rotates and, for the new key and value, appends to the cache itself
    float* acc; int acc_stride; const float* q_w; const float* k_w; float qk_eps; TbRotary rope;
    const float* row_sumsq; int row_parts; int row_width; float row_eps;
    __nv_bfloat16* storage; long long v_half;      // the cache's K half and the distance to its V half, in elements
    int late_trigger;                              // the next kernel may start once this one's pages are read (else: at once)
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&p);
}
// Byte offset of (row, 16-byte chunk of the row's 128 bytes) in a 64-row, 128-byte-swizzled box.
__device__ __forceinline__ uint32_t swz(int row, int chunk16) { return (uint32_t)(row * 128 + ((chunk16 ^ (row & 7)) << 4)); }

// HD: head size (64 or 128).  WIDE: the group has more than 8 query heads (rows 8..15 of the tile are live).
// CL: the splits of a (sequence, kv head) are the CTAs of one thread-block cluster (up to 16).  Every CTA merges a
// share of the output rows: each split SENDS its part of every share (sums, maxima, sums of weights) into the
// shared memory of the CTA that merges it (st.async: every value counts its bytes on that CTA's barrier when it has
// landed); a CTA whose barrier has counted all splits' bytes merges from its own memory, writes the result and leaves.  No scratch memory, no merge kernel, and no barrier of
// the whole cluster at the end (one at the start, where nobody waits for it: the barriers must exist before anyone
// arrives on them).
// One head of the projection's sums through row scale, head norm and rotation: a lane holds elements lane + 32 i, so an
// element and its rotation partner (HD / 2 further on) sit in the same lane.  The formulas of qk_norm_rope_vec_kernel.
template <int HD>
__device__ __forceinline__ void load_head(const float* src, int lane, float* v) {      // through L2: reductions at L2 made these sums
#pragma unroll
    for (int i = 0; i < HD / 32; ++i) v[i] = __ldcg(src + lane + 32 * i);
}
// The norm's weight ``w`` (if ``normed``) and the rotation's sines and cosines ``sn``, ``cs`` (if ``rotated``) are in
// registers already: they depend on nothing that the kernels before this one make, so the caller fetches and
// computes them while it still waits for those kernels.
template <int HD>
__device__ __forceinline__ void fused_head(float row_scale, bool normed, const float* w, float eps, bool rotated,
                                           const float* sn, const float* cs, float* v) {
    constexpr int N = HD / 32;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) { v[i] *= row_scale; ss += v[i] * v[i]; }
    if (normed) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float scale = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] = v[i] * scale * w[i];
    }
    if (rotated) {
#pragma unroll
        for (int i = 0; i < N / 2; ++i) {
            const float sv = sn[i], cv = cs[i];
            const float x = v[i], y = v[i + N / 2];
            v[i] = x * cv - y * sv;
            v[i + N / 2] = y * cv + x * sv;
        }
    }
}

template <int HD, bool WIDE, bool CL, bool FUSED = false>
__global__ void __launch_bounds__(DEC_THREADS)
attn_decode_mma_kernel(const __grid_constant__ CUtensorMap kv_map, DecArgs a) {
    static_assert(!FUSED || CL, "the folded head norm needs the cluster's barrier to know when the sums may be cleared");
    constexpr int STAGES = HD == 128 ? 3 : 4;
    constexpr int BOXES = HD / 64;                      // 64-column boxes per tile
    constexpr uint32_t TILE_BYTES = PAGE * HD * 2;      // one K or V page of one head
    constexpr int KS = HD / 16, NT = HD / 8;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(base + STAGES * 2 * TILE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* merge_bar = empty + STAGES;                             // CL: counts the parts that the cluster's CTAs have sent here
    __nv_bfloat16* q_sh = (__nv_bfloat16*)(empty + STAGES + 2);      // FUSED: the group's queries [16][HD], made here
    float* recv = reinterpret_cast<float*>(q_sh + 16 * HD);          // CL: [split][per + 32]: every split's values for this CTA's share of the output, its maxima and sums

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x, kh = blockIdx.y, split = blockIdx.z;
    TimelineProbe probe;              // stamps: 1 wait for the kernels before passed, 2 queries ready, 3 pages done, 5 all parts here, 4 end
    probe.begin(100000 + gridDim.z, blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
    // The kernel after this one may start (and request its first weight tiles) while this one runs.  Those requests
    // would queue in front of this kernel's own pages, which at small batches are all that its time depends on, so
    // it lets the next kernel in only once its pages have been requested (the producer) and read (the compute warps).
    if (!a.late_trigger) pdl_launch_dependents();
    // Queries and the newest cache row come from the kernels just before this one.  The length does too,
    // unless the caller names a copy that was final before the step's first kernel: then the pages that hold
    // only older positions are requested before the wait, while those kernels still run.
    const bool early = a.early_mode != 0;
    if (!early) pdl_wait();
    const int len = a.early_mode == 2 ? a.early_len[a.slot_of_seq[b]] + 1 : (early ? a.early_len[b] : a.kv_len[b]);
    const int keys = tb_split_keys(len, a.chunk, a.n_splits);
    if (!CL && (long long)split * keys >= len) return;  // uniform over the CTA; the merge skips these splits (in a cluster the CTA stays, with no pages, for the barrier)
    const int group = a.nh / a.nkv;
    const int wlo = a.window > 0 ? max(0, len - a.window) : 0;       // first visible key of position len - 1
    const int lo = max(wlo, (int)min((long long)len, (long long)split * keys)), hi = (int)min((long long)len, (long long)(split + 1) * keys);
    const int page0 = lo / PAGE, n_pages = lo < hi ? (hi - 1) / PAGE - page0 + 1 : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, DEC_WARPS); }
        if (CL) {
            // every split sends this CTA its values for this CTA's share of the output and the rows' maxima and sums
            const int total = (a.nh / a.nkv) * HD, per = (total + a.n_splits - 1) / a.n_splits;
            const int mine = min(total, (split + 1) * per) - min(total, split * per);
            mbar_init(merge_bar, 1);
            mbar_fence_init();
            mbar_expect_tx(merge_bar, (uint32_t)(a.n_splits * (mine + 2 * (a.nh / a.nkv)) * sizeof(float)));
        }
        mbar_fence_init();
    }
    __syncthreads();
    // CL: no CTA may send its part before every CTA of the cluster has its barrier; the arrival is here, the wait
    // where the parts are sent, long after the cluster's barrier has completed
    if (CL) tbtma::cluster_arrive();
    probe.attach();

    if (warp == DEC_WARPS) {                            // ---------------- producer
        if (lane == 0) {
            const int slot = a.slot_of_seq[b];
            const int* tab = a.table + (size_t)slot * a.table_width;
            const int v_rows = a.num_pages * a.nkv * PAGE;          // rows of the K half
            const uint64_t once = l2_evict_first_policy();          // a step reads every page once
            // before the wait: the first pages of the ring, but never the page that holds position len - 1
            // (the last page of the split that ends at len), whose newest row is still being written
            // (FUSED: no kernel before writes the cache; the newest row is this kernel's own and is patched in shared memory)
            const int old_pages = FUSED ? n_pages : n_pages - (hi == len && n_pages > 0 ? 1 : 0);
            const int ahead = early ? (old_pages < STAGES ? old_pages : STAGES) : 0;
            for (int i = 0; i < n_pages; ++i) {
                if (early && i == ahead) {
                    pdl_wait();
                    if (a.kv_len[b] != len) atomicCAS(&g_attn_error, 0u, 7u);     // the early length was not the step's
                }
                const int s = i % STAGES, round = i / STAGES;
                if (round > 0) mbar_wait(empty + s, (round - 1) & 1, &g_attn_error, 1);
                const int pos0 = (page0 + i) * PAGE;
                const int page = tab[(a.ring_rows ? pos0 % a.ring_rows : pos0) / PAGE];
                const int row = (page * a.nkv + kh) * PAGE;
                uint8_t* kd = base + s * 2 * TILE_BYTES;
                mbar_expect_tx(full + s, 2 * TILE_BYTES);
#pragma unroll
                for (int x = 0; x < BOXES; ++x) {
                    tma_load_2d_hint(kd + x * (PAGE * 128), &kv_map, full + s, x * 64, row, once);
                    tma_load_2d_hint(kd + TILE_BYTES + x * (PAGE * 128), &kv_map, full + s, x * 64, v_rows + row, once);
                }
            }
            if (early && ahead >= n_pages) {                // everything was requested ahead: check the length all the same
                pdl_wait();
                if (a.kv_len[b] != len) atomicCAS(&g_attn_error, 0u, 7u);
            }
        }
        if (a.late_trigger) pdl_launch_dependents();
        if (!CL) return;
    }

    // ---------------- compute warps: this warp takes keys 16 * warp .. + 15 of every page
    // CL: share of the output (group x HD values) that each CTA of the cluster merges, and the row stride of ``recv``
    const int merge_per = (group * HD + a.n_splits - 1) / a.n_splits, merge_stride = merge_per + 32;
    if (warp < DEC_WARPS) {
    const int g = lane >> 2, t = lane & 3;
    uint32_t qf[KS][4];
    // FUSED: the warp that owns the newest key's row of the last page keeps the new key and value, to put them there
    const int new_row = (len - 1) % PAGE;
    const bool appends = FUSED && hi == len && n_pages > 0 && warp == (new_row >> 4);
    float kn[HD / 32], vn[HD / 32];
    // FUSED: the norms' weights, the rotation's frequencies and the place of the new cache row depend on nothing that
    // the kernels before this one make: they are requested while the wait for those kernels lasts, and the sines and
    // cosines are computed while the sums are on their way (these were round trips to memory one after the other)
    float qw[HD / 32], kw[HD / 32], fr[HD / 64], sn[HD / 64], cs[HD / 64];
    int new_page = 0;
    if (FUSED) {
        const int slot = appends ? a.slot_of_seq[b] : 0;
#pragma unroll
        for (int i = 0; i < HD / 64; ++i) fr[i] = a.rope.inv_freq ? a.rope.inv_freq[lane + 32 * i] : 0.f;
#pragma unroll
        for (int i = 0; i < HD / 32; ++i) {
            qw[i] = a.q_w ? a.q_w[lane + 32 * i] : 1.f;
            kw[i] = (appends && a.k_w) ? a.k_w[lane + 32 * i] : 1.f;
        }
        if (appends) {
            const int crow = a.ring_rows ? (len - 1) % a.ring_rows : len - 1;
            new_page = a.table[(size_t)slot * a.table_width + crow / PAGE];
        }
    }
    if (early) pdl_wait();
    if (threadIdx.x == 0) probe.stamp(1);
    if (FUSED) {
        // every load first (the sums of this warp's first query head, of the new key and value, the row's parts):
        // they do not depend on one another, and at small batches this kernel is all latency
        float* arow = a.acc + (size_t)b * a.acc_stride;
        float* ksrc = arow + (size_t)(a.nh + kh) * HD;
        float* vsrc = arow + (size_t)(a.nh + a.nkv + kh) * HD;
        float v[HD / 32];
        if (warp < group) load_head<HD>(arow + (size_t)(kh * group + warp) * HD, lane, v);
        if (appends) { load_head<HD>(ksrc, lane, kn); load_head<HD>(vsrc, lane, vn); }
        float part[16];
        if (a.row_sumsq) {
#pragma unroll
            for (int z = 0; z < 16; ++z) part[z] = z < a.row_parts ? __ldcg(a.row_sumsq + z * 32 + b) : 0.f;
        }
        const bool rotated = a.rope.inv_freq != nullptr;
        if (rotated) {
#pragma unroll
            for (int i = 0; i < HD / 64; ++i) {
                sincosf(((float)(len - 1) + a.rope.offset) * fr[i], &sn[i], &cs[i]);
                sn[i] *= a.rope.magnitude; cs[i] *= a.rope.magnitude;
            }
        }
        float rs = 1.f;
        if (a.row_sumsq) {
            float total = 0.f;
#pragma unroll
            for (int z = 0; z < 16; ++z) total += part[z];                 // in the order of the parts
            rs = 1.0f / sqrtf(total / (float)a.row_width + a.row_eps);
        }
        for (int h = warp; h < group; h += DEC_WARPS) {
            if (h != warp) load_head<HD>(arow + (size_t)(kh * group + h) * HD, lane, v);
            fused_head<HD>(rs, a.q_w != nullptr, qw, a.qk_eps, rotated, sn, cs, v);
#pragma unroll
            for (int i = 0; i < HD / 32; ++i) q_sh[h * HD + lane + 32 * i] = __float2bfloat16_rn(v[i]);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(DEC_WARPS * 32));      // the group's queries are in shared memory
        if (threadIdx.x == 0) probe.stamp(2);
        if (appends) {              // after the barrier: the other warps need not wait for the new key and value
            fused_head<HD>(rs, a.k_w != nullptr, kw, a.qk_eps, rotated, sn, cs, kn);
            __nv_bfloat16* kdst = a.storage + ((size_t)(new_page * a.nkv + kh) * PAGE + new_row) * HD;
#pragma unroll
            for (int i = 0; i < HD / 32; ++i) {
                vn[i] *= rs;
                kn[i] = __bfloat162float(__float2bfloat16_rn(kn[i]));          // as the cache holds them
                vn[i] = __bfloat162float(__float2bfloat16_rn(vn[i]));
                kdst[lane + 32 * i] = __float2bfloat16_rn(kn[i]);
                kdst[a.v_half + lane + 32 * i] = __float2bfloat16_rn(vn[i]);
                ksrc[lane + 32 * i] = 0.f;                                       // the sums are left cleared for the next step
                vsrc[lane + 32 * i] = 0.f;
            }
        }
    }
    {
        const __nv_bfloat16* q0 = FUSED ? q_sh : a.q + (size_t)b * a.q_stride + (size_t)(kh * group) * HD;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int d = ks * 16 + 2 * t;
            qf[ks][0] = g < group ? *reinterpret_cast<const uint32_t*>(q0 + g * HD + d) : 0u;
            qf[ks][2] = g < group ? *reinterpret_cast<const uint32_t*>(q0 + g * HD + d + 8) : 0u;
            qf[ks][1] = (WIDE && g + 8 < group) ? *reinterpret_cast<const uint32_t*>(q0 + (g + 8) * HD + d) : 0u;
            qf[ks][3] = (WIDE && g + 8 < group) ? *reinterpret_cast<const uint32_t*>(q0 + (g + 8) * HD + d + 8) : 0u;
        }
    }
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m0 = -1e30f, m1 = -1e30f, l0 = 0.f, l1 = 0.f;       // rows g and g + 8

    for (int i = 0; i < n_pages; ++i) {
        const int s = i % STAGES;
        mbar_wait(full + s, (i / STAGES) & 1, &g_attn_error, 2);
        const uint32_t ks_base = smem_u32(base + s * 2 * TILE_BYTES);
        const uint32_t vs_base = ks_base + TILE_BYTES;
        if (appends && i == n_pages - 1) {                  // the page as the cache held it before this step: put the new row in
            uint8_t* kt = base + s * 2 * TILE_BYTES;
#pragma unroll
            for (int j = 0; j < HD / 32; ++j) {
                const int e = lane + 32 * j;
                const uint32_t off = (uint32_t)((e >> 6) * (PAGE * 128)) + swz(new_row, (e & 63) >> 3) + (uint32_t)((e & 7) * 2);
                *reinterpret_cast<__nv_bfloat16*>(kt + off) = __float2bfloat16_rn(kn[j]);
                *reinterpret_cast<__nv_bfloat16*>(kt + TILE_BYTES + off) = __float2bfloat16_rn(vn[j]);
            }
            __syncwarp();
        }
        // S[16 x 16] = Q . K^T for this warp's 16 keys: two n-tiles of 8 keys
        float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        {
            const int mtx = lane >> 3, r = lane & 7;
            const int key = warp * 16 + (mtx >> 1) * 8 + r;              // matrices 0,1: first 8 keys; 2,3: next 8
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int dim0 = ks * 16 + (mtx & 1) * 8;
                uint32_t b0, b1, b2, b3;
                ldsm_x4(ks_base + (dim0 >> 6) * (PAGE * 128) + swz(key, (dim0 & 63) >> 3), b0, b1, b2, b3);
                mma_bf16(sc[0], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                mma_bf16(sc[1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
            }
        }
        // mask, scale, running softmax
        const int pos_base = (page0 + i) * PAGE + warp * 16 + 2 * t;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int pos = pos_base + j * 8 + c;
                const bool ok = pos >= lo && pos < hi;
                sc[j][c] = ok ? sc[j][c] * a.scale_log2 : -INFINITY;
                sc[j][c + 2] = ok ? sc[j][c + 2] * a.scale_log2 : -INFINITY;
                mx0 = fmaxf(mx0, sc[j][c]);
                mx1 = fmaxf(mx1, sc[j][c + 2]);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        const float al0 = exp2f(m0 - n0), al1 = exp2f(m1 - n1);
        m0 = n0; m1 = n1;
        float p[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            p[j][0] = exp2f(sc[j][0] - n0); p[j][1] = exp2f(sc[j][1] - n0);
            p[j][2] = WIDE ? exp2f(sc[j][2] - n1) : 0.f; p[j][3] = WIDE ? exp2f(sc[j][3] - n1) : 0.f;
        }
        l0 = l0 * al0 + p[0][0] + p[0][1] + p[1][0] + p[1][1];
        l1 = l1 * al1 + p[0][2] + p[0][3] + p[1][2] + p[1][3];
        const uint32_t pa0 = pack2(p[0][0], p[0][1]), pa1 = pack2(p[0][2], p[0][3]);
        const uint32_t pa2 = pack2(p[1][0], p[1][1]), pa3 = pack2(p[1][2], p[1][3]);
        // O[16 x HD] = alpha * O + P . V over this warp's 16 keys
        {
            const int mtx = lane >> 3, r = lane & 7;
            const int key = warp * 16 + (mtx & 1) * 8 + r;              // matrices 0,2: keys 0-7; 1,3: keys 8-15
#pragma unroll
            for (int n = 0; n < NT; n += 2) {
                const int dim0 = (n + (mtx >> 1)) * 8;
                uint32_t b0, b1, b2, b3;
                ldsm_x4_trans(vs_base + (dim0 >> 6) * (PAGE * 128) + swz(key, (dim0 & 63) >> 3), b0, b1, b2, b3);
                o[n][0] *= al0; o[n][1] *= al0; o[n][2] *= al1; o[n][3] *= al1;
                o[n + 1][0] *= al0; o[n + 1][1] *= al0; o[n + 1][2] *= al1; o[n + 1][3] *= al1;
                mma_bf16(o[n], pa0, pa1, pa2, pa3, b0, b1);
                mma_bf16(o[n + 1], pa0, pa1, pa2, pa3, b2, b3);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (a.late_trigger) pdl_launch_dependents();
    if (threadIdx.x == 0) probe.stamp(3);

    // ---------------- merge the four warps through shared memory (the stages are drained)
    asm volatile("bar.sync 1, %0;" ::"n"(DEC_WARPS * 32));      // compute warps only; the producer has left
    float* mo = reinterpret_cast<float*>(base);                 // [warp][16][HD]
    float* mm = mo + DEC_WARPS * 16 * HD;                       // [warp][16] max, then [warp][16] sum
    float* ml = mm + DEC_WARPS * 16;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        float* r0 = mo + (warp * 16 + g) * HD + n * 8 + 2 * t;
        r0[0] = o[n][0]; r0[1] = o[n][1];
        if (WIDE) { r0[8 * HD] = o[n][2]; r0[8 * HD + 1] = o[n][3]; }
    }
    if (t == 0) {
        mm[warp * 16 + g] = m0; ml[warp * 16 + g] = l0;
        mm[warp * 16 + g + 8] = WIDE ? m1 : -1e30f; ml[warp * 16 + g + 8] = WIDE ? l1 : 0.f;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(DEC_WARPS * 32));
    const float ln2 = 0.69314718055994531f;
    for (int idx = threadIdx.x; idx < group * HD; idx += DEC_WARPS * 32) {
        const int row = idx / HD, d = idx % HD;
        float M = -1e30f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, mm[w * 16 + row]);
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float f = exp2f(mm[w * 16 + row] - M);
            acc += f * mo[(w * 16 + row) * HD + d];
            L += f * ml[w * 16 + row];
        }
        if (CL && a.n_splits == 1) {      // nothing to merge with: this is the result
            a.out[(size_t)b * a.out_stride + (size_t)(kh * group + row) * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        } else if (CL) {
            // to the CTA that merges this element, into the row of this split; a row's maximum and sum of weights to all
            const int owner = idx / merge_per, e = idx - owner * merge_per;
            tbtma::st_async_f32(tbtma::cluster_addr(recv + split * merge_stride + e, owner), acc, tbtma::cluster_addr(merge_bar, owner));
            if (d < a.n_splits) {      // the row's first n threads: one CTA of the cluster each
                const uint32_t bar = tbtma::cluster_addr(merge_bar, d);
                tbtma::st_async_f32(tbtma::cluster_addr(recv + split * merge_stride + merge_per + row, d), M, bar);
                tbtma::st_async_f32(tbtma::cluster_addr(recv + split * merge_stride + merge_per + 16 + row, d), L, bar);
            }
        } else {
            float* part = a.scratch + ((size_t)(b * a.nh + kh * group + row) * a.n_splits + split) * (HD + 2);
            part[d] = acc;
            if (d == 0) { part[HD] = M * ln2; part[HD + 1] = L; }     // the merge works with natural exponents
        }
    }
    }       // compute warps
    if (CL) {
        // The splits of a (sequence, kv head) merge without a barrier of the cluster at the end: every CTA has SENT its
        // part to the CTAs that merge it (above), waits until its own barrier has counted the bytes of every split,
        // merges its share from its own shared memory and leaves.  Nobody reads this CTA's memory, and nobody writes
        // to it after the last of the bytes it waits for.
        tbtma::cluster_wait();                                      // every thread; completed long ago (see the arrival above)
        if (warp < DEC_WARPS) {
            if (a.n_splits > 1) tbtma::mbar_wait_cluster(merge_bar, 0, &g_attn_error, 8);      // every split's values have landed here
            if (threadIdx.x == 0) probe.stamp(5);
            if (FUSED && split == 0) {      // every split has sent its part, so it has read the queries' sums: clear them for the next step
                float* qsum = a.acc + (size_t)b * a.acc_stride + (size_t)(kh * group) * HD;
                for (int i = threadIdx.x; i < group * HD; i += DEC_WARPS * 32) qsum[i] = 0.f;
            }
            const int n = a.n_splits, total = group * HD;
            const int first = split * merge_per, last = n > 1 ? min(total, first + merge_per) : 0;
            for (int idx = first + (int)threadIdx.x; idx < last; idx += DEC_WARPS * 32) {
                const int row = idx / HD, d = idx % HD, e = idx - first;
                float mr[16], lr[16], vr[16];
#pragma unroll
                for (int r = 0; r < 16; ++r) {
                    const bool on = r < n;
                    mr[r] = on ? recv[r * merge_stride + merge_per + row] : -1e30f;
                    lr[r] = on ? recv[r * merge_stride + merge_per + 16 + row] : 0.f;
                    vr[r] = on ? recv[r * merge_stride + e] : 0.f;
                }
                float M = -1e30f;
#pragma unroll
                for (int r = 0; r < 16; ++r) M = fmaxf(M, mr[r]);
                float acc = 0.f, L = 0.f;
#pragma unroll
                for (int r = 0; r < 16; ++r) {              // in the order of the splits
                    const float f = r < n ? exp2f(mr[r] - M) : 0.f;
                    acc += f * vr[r];
                    L += f * lr[r];
                }
                a.out[(size_t)b * a.out_stride + (size_t)(kh * group + row) * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
            }
        }
    }
    if (threadIdx.x == 0) probe.stamp(4);
}


// ------------------------------------------------------------------ prompts and continuation chunks
// One CTA per (sequence, query head, block of 64 queries), four compute warps of 16 query rows each
// and a producer warp.  Queries are read by TMA from the step's own [T][Q | K | V] rows (64 x 64 boxes,
// 128-byte swizzle); keys and values from the same rows when every sequence starts at position 0 (the
// cache is not touched), else from the cache's pages through the block table (a key tile is one page;
// the step's own keys were appended before).  Key tiles of 64 run from the window's first key to the
// diagonal; S and P.V are mma.sync.m16n8k16 as above.  Heavy (late) query blocks are scheduled first.
struct PreArgs {
    __nv_bfloat16* out; int out_stride;
    const int* q_start; int B;
    int nh; int nkv; int window; float scale_log2;
    int k_col0; int v_col0;                  // first column of the K heads and of the V heads
    // keys and values from the cache: first position of each sequence's rows, slots, block table, first V row of the map
    int paged; const int* start_pos; const int* slot_of_seq; const int* table; int table_width; int v_row0;
};

template <int HD>
__global__ void __launch_bounds__(DEC_THREADS, 2)
attn_prefill_mma_kernel(const __grid_constant__ CUtensorMap qkv_map, const __grid_constant__ CUtensorMap kv_map, PreArgs a) {
    constexpr int STAGES = 2;
    constexpr int BOXES = HD / 64;
    constexpr uint32_t TILE_BYTES = 64 * HD * 2;
    constexpr int KS = HD / 16, NT = HD / 8;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_smem = base + STAGES * 2 * TILE_BYTES;
    uint64_t* full = (uint64_t*)(q_smem + TILE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* qbar = empty + STAGES;

    pdl_launch_dependents();
    pdl_wait();
    // which sequence and which block of it (blocks are numbered from the heaviest)
    int rem = blockIdx.y, seq = -1, blk = 0, tok0 = 0, n = 0;       // heads run fastest: the heaviest blocks of all heads start first
    for (int s = 0; s < a.B; ++s) {
        const int t0 = a.q_start[s], ns = a.q_start[s + 1] - t0, nb = (ns + 63) >> 6;
        if (rem < nb) { seq = s; blk = nb - 1 - rem; tok0 = t0; n = ns; break; }
        rem -= nb;
    }
    if (seq < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.x, kh = h / (a.nh / a.nkv);
    const int r0 = blk * 64;                                         // first row of the block among the sequence's rows
    const int p0 = a.paged ? a.start_pos[seq] : 0;                   // position of the sequence's first row
    const int last_key = p0 + min(n - 1, r0 + 63);
    const int first_key = a.window > 0 ? max(0, p0 + r0 - a.window + 1) : 0;
    const int kt0 = first_key >> 6, n_tiles = (last_key >> 6) - kt0 + 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, DEC_WARPS); }
        mbar_init(qbar, 1);
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == DEC_WARPS) {
        if (lane == 0) {
            mbar_expect_tx(qbar, TILE_BYTES);
#pragma unroll
            for (int x = 0; x < BOXES; ++x) tma_load_2d(q_smem + x * 8192, &qkv_map, qbar, h * HD + x * 64, tok0 + r0);
            const int* tab = a.paged ? a.table + (size_t)a.slot_of_seq[seq] * a.table_width : nullptr;
            const int kx = a.paged ? 0 : a.k_col0 + kh * HD, vx = a.paged ? 0 : a.v_col0 + kh * HD;
            for (int i = 0; i < n_tiles; ++i) {
                const int s = i % STAGES, round = i / STAGES;
                if (round > 0) mbar_wait(empty + s, (round - 1) & 1, &g_attn_error, 3);
                uint8_t* kd = base + s * 2 * TILE_BYTES;
                const int krow = a.paged ? (tab[kt0 + i] * a.nkv + kh) * 64 : tok0 + (kt0 + i) * 64;
                const int vrow = a.paged ? a.v_row0 + krow : krow;
                mbar_expect_tx(full + s, 2 * TILE_BYTES);
#pragma unroll
                for (int x = 0; x < BOXES; ++x) {
                    tma_load_2d(kd + x * 8192, a.paged ? &kv_map : &qkv_map, full + s, kx + x * 64, krow);
                    tma_load_2d(kd + TILE_BYTES + x * 8192, a.paged ? &kv_map : &qkv_map, full + s, vx + x * 64, vrow);
                }
            }
        }
        return;
    }

    const int g = lane >> 2, t = lane & 3, mtx = lane >> 3, r = lane & 7;
    uint32_t qf[KS][4];
    mbar_wait(qbar, 0, &g_attn_error, 4);
    {
        const uint32_t qs = smem_u32(q_smem);
        const int row = warp * 16 + (mtx & 1) * 8 + r;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int dim0 = ks * 16 + (mtx >> 1) * 8;
            ldsm_x4(qs + (dim0 >> 6) * 8192 + swz(row, (dim0 & 63) >> 3), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
        }
    }
    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -1e30f, m1 = -1e30f, l0 = 0.f, l1 = 0.f;
    const int qr0 = r0 + warp * 16 + g, qr1 = qr0 + 8;              // this thread's two rows among the sequence's rows ...
    const int qp0 = p0 + qr0, qp1 = p0 + qr1;                       // ... and their positions
    const int lo0 = a.window > 0 ? qp0 - a.window + 1 : 0, lo1 = a.window > 0 ? qp1 - a.window + 1 : 0;

    for (int i = 0; i < n_tiles; ++i) {
        const int s = i % STAGES;
        mbar_wait(full + s, (i / STAGES) & 1, &g_attn_error, 5);
        const uint32_t ks_base = smem_u32(base + s * 2 * TILE_BYTES), vs_base = ks_base + TILE_BYTES;
        float sc[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) { sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int dim0 = ks * 16 + (mtx & 1) * 8;
            const uint32_t col = (dim0 >> 6) * 8192, ch = (dim0 & 63) >> 3;
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {
                const int key = (2 * jp + (mtx >> 1)) * 8 + r;
                uint32_t b0, b1, b2, b3;
                ldsm_x4(ks_base + col + swz(key, ch), b0, b1, b2, b3);
                mma_bf16(sc[2 * jp], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                mma_bf16(sc[2 * jp + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
            }
        }
        const int key_base = (kt0 + i) * 64 + 2 * t;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int key = key_base + j * 8 + c;
                sc[j][c] = (key <= qp0 && key >= lo0) ? sc[j][c] * a.scale_log2 : -INFINITY;
                sc[j][c + 2] = (key <= qp1 && key >= lo1) ? sc[j][c + 2] * a.scale_log2 : -INFINITY;
                mx0 = fmaxf(mx0, sc[j][c]);
                mx1 = fmaxf(mx1, sc[j][c + 2]);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        const float al0 = exp2f(m0 - n0), al1 = exp2f(m1 - n1);
        m0 = n0; m1 = n1;
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            sc[j][0] = exp2f(sc[j][0] - n0); sc[j][1] = exp2f(sc[j][1] - n0);
            sc[j][2] = exp2f(sc[j][2] - n1); sc[j][3] = exp2f(sc[j][3] - n1);
            s0 += sc[j][0] + sc[j][1]; s1 += sc[j][2] + sc[j][3];
        }
        l0 = l0 * al0 + s0; l1 = l1 * al1 + s1;
#pragma unroll
        for (int i2 = 0; i2 < NT; ++i2) { o[i2][0] *= al0; o[i2][1] *= al0; o[i2][2] *= al1; o[i2][3] *= al1; }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const uint32_t pa0 = pack2(sc[2 * kk][0], sc[2 * kk][1]), pa1 = pack2(sc[2 * kk][2], sc[2 * kk][3]);
            const uint32_t pa2 = pack2(sc[2 * kk + 1][0], sc[2 * kk + 1][1]), pa3 = pack2(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
            const int key = kk * 16 + (mtx & 1) * 8 + r;
#pragma unroll
            for (int nn = 0; nn < NT; nn += 2) {
                const int dim0 = (nn + (mtx >> 1)) * 8;
                uint32_t b0, b1, b2, b3;
                ldsm_x4_trans(vs_base + (dim0 >> 6) * 8192 + swz(key, (dim0 & 63) >> 3), b0, b1, b2, b3);
                mma_bf16(o[nn], pa0, pa1, pa2, pa3, b0, b1);
                mma_bf16(o[nn + 1], pa0, pa1, pa2, pa3, b2, b3);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = 1.0f / l0, i1 = 1.0f / l1;
    __nv_bfloat16* out0 = a.out + (size_t)(tok0 + qr0) * a.out_stride + h * HD + 2 * t;
    __nv_bfloat16* out1 = a.out + (size_t)(tok0 + qr1) * a.out_stride + h * HD + 2 * t;
#pragma unroll
    for (int nn = 0; nn < NT; ++nn) {
        if (qr0 < n) *reinterpret_cast<uint32_t*>(out0 + nn * 8) = pack2(o[nn][0] * i0, o[nn][1] * i0);
        if (qr1 < n) *reinterpret_cast<uint32_t*>(out1 + nn * 8) = pack2(o[nn][2] * i1, o[nn][3] * i1);
    }
}

}  // namespace


extern "C" int tb_attn_merge(const AttnArgs* args, int dtype, cudaStream_t stream);

// Shared memory of the decode kernel: the ring, its barriers, and the group's queries (used when the head norm is folded in).
template <int HD> constexpr size_t decode_smem() {
    return 1024 + (size_t)(HD == 128 ? 3 : 4) * 2 * PAGE * HD * 2 + 2 * (HD == 128 ? 3 : 4) * sizeof(uint64_t) + 16 + 16 * HD * 2 +
           (16 * HD + 16 + 16 * 32) * sizeof(float);      // the parts received for the merge: up to 16 splits x (share + 32)
}
template <int HD, bool WIDE, bool CL, bool FUSED = false>
static int launch_decode(const CUtensorMap& map, const DecArgs& d, dim3 grid, cudaStream_t stream) {
    constexpr size_t smem = decode_smem<HD>();
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(attn_decode_mma_kernel<HD, WIDE, CL, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(attn_decode_mma_kernel<HD, WIDE, CL, FUSED>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);   // room for several CTAs per SM
        if (CL) cudaFuncSetAttribute(attn_decode_mma_kernel<HD, WIDE, CL, FUSED>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);    // clusters of up to 16
        TB_REQUIRE(e == cudaSuccess, "attn_decode_mma: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    if (CL) {
        const cudaError_t e = tb_launch_cluster_z(attn_decode_mma_kernel<HD, WIDE, CL, FUSED>, grid, DEC_THREADS, smem, stream, (int)grid.z, map, d);
        TB_REQUIRE(e == cudaSuccess, "attn_decode_mma: cluster launch failed: %s", cudaGetErrorString(e));
    } else {
        tb_launch(attn_decode_mma_kernel<HD, WIDE, CL, FUSED>, grid, DEC_THREADS, smem, stream, map, d);
    }
    return 0;
}
// The largest cluster of this kernel that the device can place: 16 where the non-portable size is allowed
// and fits (B200), else 8, else 1 (no clusters).
template <int HD, bool WIDE>
static int cluster_limit() {
    static int limit = -1;
    if (limit < 0) {
        limit = 1;
        constexpr size_t smem = decode_smem<HD>();
        auto kernel = attn_decode_mma_kernel<HD, WIDE, true>;
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        for (int size : {16, 8}) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(1, 1, size); cfg.blockDim = dim3(DEC_THREADS, 1, 1); cfg.dynamicSmemBytes = smem;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = (unsigned)size;
            cfg.attrs = attr; cfg.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) == cudaSuccess && clusters > 0) { limit = size; break; }
            cudaGetLastError();
        }
    }
    return limit;
}
// Launches the kernel; *merged says whether the splits merged among themselves (a cluster) or left their parts in scratch.
template <int HD, bool WIDE>
static int launch_decode_any(const CUtensorMap& map, const DecArgs& d, dim3 grid, bool may_cluster, bool* merged, cudaStream_t stream) {
    *merged = may_cluster && (int)grid.z <= cluster_limit<HD, WIDE>();
    if (d.acc) {
        TB_REQUIRE(*merged, "attn_decode_mma: the folded head norm needs the splits to form a cluster (%d splits)", (int)grid.z);
        return launch_decode<HD, WIDE, true, true>(map, d, grid, stream);
    }
    TB_REQUIRE(*merged || d.scratch, "attn_decode_mma: %d splits need scratch memory", (int)grid.z);
    return *merged ? launch_decode<HD, WIDE, true>(map, d, grid, stream) : launch_decode<HD, WIDE, false>(map, d, grid, stream);
}

int g_decode_cluster = 1;
int g_late_trigger = 1;
// When the kernel after decode attention may start: once this one's pages have been read (1, default) or at once (0).
// Measured after 2,048-token prompts: batch 1 2.85 -> 2.81 ms per step, batch 4 3.11 -> 3.06, batch 8 3.27 -> 3.24; no
// difference at 7,000 tokens or at batch 64.
extern "C" void tb_attn_decode_set_late_trigger(int on) { g_late_trigger = on ? 1 : 0; }
// The splits of decode attention merge inside a thread-block cluster (1, default, up to 16 splits where the device places such clusters) or through scratch memory and the merge kernel (0).
extern "C" void tb_attn_decode_set_cluster(int on) { g_decode_cluster = on ? 1 : 0; }

// 0 if the tensor-core decode kernel takes this problem, else 1 with the reason in tb_last_error().
extern "C" int tb_attn_decode_mma_check(const AttnArgs* a, int dtype) {
    TB_REQUIRE(dtype == TB_BF16, "attn_decode_mma: bfloat16 only");
    TB_REQUIRE(a->hd == 64 || a->hd == 128, "attn_decode_mma: head_dim %d is not 64 or 128", a->hd);
    TB_REQUIRE(a->cache.page_size == PAGE, "attn_decode_mma: pages of %d rows, not %d", PAGE, a->cache.page_size);
    TB_REQUIRE(a->nkv > 0 && a->nh % a->nkv == 0 && a->nh / a->nkv <= 16, "attn_decode_mma: at most 16 query heads per kv head");
    TB_REQUIRE(a->chunk > 0 && a->chunk % PAGE == 0, "attn_decode_mma: the chunk %d must be a multiple of %d", a->chunk, PAGE);
    if (a->fused_qk) {
        const QkArgs& q = *a->fused_qk;
        TB_REQUIRE(q.in && q.in_stride % 4 == 0 && ((uintptr_t)q.in & 15) == 0, "attn_decode_mma: the projection's sums must be 16-byte aligned float32 rows");
        TB_REQUIRE(q.nh == a->nh && q.nkv == a->nkv && q.hd == a->hd, "attn_decode_mma: the folded head norm's heads do not match");
        TB_REQUIRE(!q.rope.inv_freq || q.rope.rot == a->hd, "attn_decode_mma: the folded rotation must span the whole head");
        TB_REQUIRE(q.cache.storage == a->cache.storage, "attn_decode_mma: the folded append writes the cache it reads");
        TB_REQUIRE(!q.row_sumsq || (q.row_width > 0 && q.row_parts > 0 && q.row_parts <= 16 && a->batch.B <= 32), "attn_decode_mma: row sums of squares need their width, 1 to 16 parts and at most 32 rows");
        const bool wide = a->nh / a->nkv > 8;
        const int limit = a->hd == 128 ? (wide ? cluster_limit<128, true>() : cluster_limit<128, false>())
                                       : (wide ? cluster_limit<64, true>() : cluster_limit<64, false>());
        TB_REQUIRE(g_decode_cluster && a->out && a->n_splits <= limit, "attn_decode_mma: the folded head norm needs the splits to form a cluster");
    } else {
        TB_REQUIRE(a->q_stride % 2 == 0 && ((uintptr_t)a->q & 3) == 0, "attn_decode_mma: queries must be 4-byte aligned");
    }
    return 0;
}

extern "C" int tb_attn_decode_mma(const AttnArgs* args, cudaStream_t stream) {
    const AttnArgs& a = *args;
    if (tb_attn_decode_mma_check(args, TB_BF16)) return 1;
    // few enough splits form a cluster and merge among themselves; more leave parts in scratch and tb_attn_merge finishes
    const bool may_cluster = g_decode_cluster && a.out != nullptr;
    TB_REQUIRE(a.batch.B > 0 && a.cache.storage, "attn_decode_mma: needs sequences and a cache");
    TB_REQUIRE(a.n_splits > 0 && a.n_splits <= 65535 && a.nkv <= 65535, "attn_decode_mma: bad grid");
    TB_REQUIRE(a.cache.head_dim == a.hd && a.cache.kv_heads == a.nkv, "attn_decode_mma: the cache view does not match the heads");
    CUtensorMap map;
    const long long rows = 2LL * a.cache.num_pages * a.nkv * PAGE;
    if (tb_make_map_bf16(&map, a.cache.storage, rows, a.hd, a.hd, PAGE)) return 1;
    DecArgs d;
    d.q = (const __nv_bfloat16*)a.q; d.q_stride = a.q_stride; d.scratch = a.scratch;
    d.table = a.cache.table; d.table_width = a.cache.table_width; d.ring_rows = a.cache.ring_rows; d.num_pages = a.cache.num_pages;
    d.slot_of_seq = a.batch.slot_of_seq; d.kv_len = a.batch.kv_len;
    d.early_len = a.early_len; d.early_mode = a.early_len ? a.early_mode : 0;
    TB_REQUIRE(d.early_mode >= 0 && d.early_mode <= 2, "attn_decode_mma: early_mode %d (0, 1 or 2)", d.early_mode);
    d.nh = a.nh; d.nkv = a.nkv; d.window = a.window; d.scale_log2 = a.scale * 1.4426950408889634f;
    d.chunk = a.chunk; d.n_splits = a.n_splits;
    d.out = (__nv_bfloat16*)a.out; d.out_stride = a.out_stride;
    d.acc = nullptr; d.acc_stride = 0; d.q_w = d.k_w = nullptr; d.qk_eps = 0.f; d.rope = TbRotary{nullptr, 0, 0.f, 1.f};
    d.row_sumsq = nullptr; d.row_parts = 0; d.row_width = 1; d.row_eps = 0.f; d.storage = nullptr; d.v_half = 0;
    if (a.fused_qk) {
        const QkArgs& q = *a.fused_qk;
        d.acc = (float*)const_cast<void*>(q.in); d.acc_stride = q.in_stride; d.q_w = q.q_w; d.k_w = q.k_w; d.qk_eps = q.eps; d.rope = q.rope;
        d.row_sumsq = q.row_sumsq; d.row_parts = q.row_parts; d.row_width = q.row_width; d.row_eps = q.row_eps;
        d.storage = (__nv_bfloat16*)a.cache.storage; d.v_half = (long long)a.cache.num_pages * a.nkv * PAGE * a.hd;
    }
    dim3 grid(a.batch.B, a.nkv, a.n_splits);
    d.late_trigger = g_late_trigger;
    const bool wide = a.nh / a.nkv > 8;
    int rc;
    bool merged = false;
    if (a.hd == 128) rc = wide ? launch_decode_any<128, true>(map, d, grid, may_cluster, &merged, stream) : launch_decode_any<128, false>(map, d, grid, may_cluster, &merged, stream);
    else rc = wide ? launch_decode_any<64, true>(map, d, grid, may_cluster, &merged, stream) : launch_decode_any<64, false>(map, d, grid, may_cluster, &merged, stream);
    if (rc) return rc;
    TB_CHECK_LAUNCH("attn_decode_mma");
    return merged ? 0 : tb_attn_merge(args, TB_BF16, stream);
}

// Reads and clears the error word of this file's kernels (0: none).  Synchronises the device.
extern "C" int tb_attn_mma_error() {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_error, sizeof(v)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(zero));
    return (int)v;
}

template <int HD>
static int launch_prefill(const CUtensorMap& map, const CUtensorMap& kv_map, const PreArgs& p, dim3 grid, cudaStream_t stream) {
    constexpr size_t smem = 1024 + (size_t)(2 * 2 + 1) * 64 * HD * 2 + 8 * sizeof(uint64_t);
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(attn_prefill_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(attn_prefill_mma_kernel<HD>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);   // room for several CTAs per SM
        TB_REQUIRE(e == cudaSuccess, "attn_prefill_mma: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    tb_launch(attn_prefill_mma_kernel<HD>, grid, DEC_THREADS, smem, stream, map, kv_map, p);
    return 0;
}

// 0 if the tensor-core prompt kernel takes this problem, else 1 with the reason.  source: TB_KV_FROM_STEP (every
// sequence of the step starts at position 0, so all keys are among the step's own rows) or TB_KV_FROM_CACHE (keys
// and values from the pages of a cache that keeps every key, the step's own appended already).
extern "C" int tb_attn_prefill_mma_check(const AttnArgs* a, int dtype, int source) {
    TB_REQUIRE(dtype == TB_BF16, "attn_prefill_mma: bfloat16 only");
    TB_REQUIRE(source == TB_KV_FROM_STEP || source == TB_KV_FROM_CACHE, "attn_prefill_mma: a sequence continues from the cache and its keys are not all there");
    TB_REQUIRE(a->hd == 64 || a->hd == 128, "attn_prefill_mma: head_dim %d is not 64 or 128", a->hd);
    TB_REQUIRE(a->nkv > 0 && a->nh % a->nkv == 0, "attn_prefill_mma: heads");
    TB_REQUIRE(a->q_stride % 8 == 0 && ((uintptr_t)a->q & 15) == 0, "attn_prefill_mma: the queries must be 16-byte aligned rows");
    if (source == TB_KV_FROM_STEP) {
        TB_REQUIRE(a->kv_new && a->q_stride == a->kv_stride, "attn_prefill_mma: Q, K and V must be columns of one row-major buffer");
        const long long off = ((const char*)a->kv_new - (const char*)a->q) / 2;
        TB_REQUIRE(off == (long long)a->nh * a->hd, "attn_prefill_mma: K must follow Q in the buffer");
    } else {
        TB_REQUIRE(a->cache.storage && a->cache.page_size == PAGE && a->cache.ring_rows == 0, "attn_prefill_mma: needs a cache of %d-row pages that keeps every key", PAGE);
        TB_REQUIRE(a->cache.head_dim == a->hd && a->cache.kv_heads == a->nkv, "attn_prefill_mma: the cache view does not match the heads");
    }
    TB_REQUIRE(a->out_stride % 2 == 0 && ((uintptr_t)a->out & 3) == 0, "attn_prefill_mma: the output must be 4-byte aligned");
    return 0;
}

extern "C" int tb_attn_prefill_mma(const AttnArgs* args, int source, cudaStream_t stream) {
    const AttnArgs& a = *args;
    if (tb_attn_prefill_mma_check(args, TB_BF16, source)) return 1;
    TB_REQUIRE(a.batch.T > 0 && a.batch.B > 0, "attn_prefill_mma: no tokens");
    CUtensorMap map, kv_map;
    if (tb_make_map_bf16(&map, a.q, a.batch.T, a.q_stride, a.q_stride, 64)) return 1;
    kv_map = map;
    PreArgs p;
    p.paged = source == TB_KV_FROM_CACHE;
    if (p.paged && tb_make_map_bf16(&kv_map, a.cache.storage, 2LL * a.cache.num_pages * a.nkv * PAGE, a.hd, a.hd, PAGE)) return 1;
    p.start_pos = a.batch.start_pos; p.slot_of_seq = a.batch.slot_of_seq; p.table = a.cache.table; p.table_width = a.cache.table_width;
    p.v_row0 = a.cache.num_pages * a.nkv * PAGE;
    p.out = (__nv_bfloat16*)a.out; p.out_stride = a.out_stride; p.q_start = a.batch.q_start; p.B = a.batch.B;
    p.nh = a.nh; p.nkv = a.nkv; p.window = a.window; p.scale_log2 = a.scale * 1.4426950408889634f;
    p.k_col0 = a.nh * a.hd; p.v_col0 = (a.nh + a.nkv) * a.hd;
    const int blocks = (a.batch.T + 63) / 64 + a.batch.B;          // upper bound on sum over sequences of ceil(n / 64)
    TB_REQUIRE(blocks <= 65535, "attn_prefill_mma: too many query blocks (%d)", blocks);
    dim3 grid(a.nh, blocks);
    const int rc = a.hd == 128 ? launch_prefill<128>(map, kv_map, p, grid, stream) : launch_prefill<64>(map, kv_map, p, grid, stream);
    if (rc) return rc;
    TB_CHECK_LAUNCH("attn_prefill_mma");
    return 0;
}

// Names the buffer of the timeline probe (timeline.cuh); 1 if the library was built with it, 0 if not.
TB_TIMELINE_SETTER(tb_attn_mma_timeline)
