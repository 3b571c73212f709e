// Causal grouped-query attention over the paged cache, for every head size and group.
//
//   tb_attn_prefill  queries of a ragged step; keys before the step come from the cache, keys of
//                    the step itself from the step's own K | V rows (so a ring cache can be
//                    written after attention)
//   tb_attn_decode   one query per sequence over its cached keys, cut into splits by the sequence's
//                    own length (tb_split_keys), each giving (max, sum, unnormalised output)
//   tb_attn_merge    log-sum-exp merge of the chunks in chunk order
//
// One warp per (query, head): a lane scores one key per round with the whole query in shared
// memory, the warp folds 32 scores into the running softmax, then every lane accumulates its
// output dims over the 32 values.  Scores, softmax and PV are float32 with precise expf.
// A chunk's borders depend on the sequence's own length only, never on the batch.
//
// berniehans/titan: flash_attention_2_kernel (engine/engine-cuda/kernels/flash_attention_2.cu:22-106),
// paged_attention_decode_kernel, flash_decoding_split_kernel and flash_decoding_reduce_kernel
// (kernels/paged_attention.cu:6-103, 200-309, 314-369): score = q.k / sqrt(hd), keys t <= position,
// query head h reads kv head h / (nh/nkv), partials merged with exp(m_s - m_max).
#include <float.h>

#include "attention_args.h"
#include "common.cuh"

#define ATT_MAXE 8        // head_dim <= 256
#define ATT_WARPS 4


template <typename T> __device__ __forceinline__ void load8(const T* p, float* o);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* o) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* o) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        o[2 * i] = __uint_as_float(w[i] << 16);
        o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// Running softmax state of one warp: every lane holds the same m and l, and acc for dims lane + 32 j.
struct Running {
    float m, l;
    float acc[ATT_MAXE];
};

// Folds keys [lo, hi) of one sequence into ``st``.  Keys at positions >= first_new are read from the
// step's own rows (row index first_new_row + pos - first_new), earlier ones from the cache.
template <typename T>
__device__ __forceinline__ void attend_range(Running& st, const float* qs, const AttnArgs& a, int lo, int hi,
                                             int first_new, int first_new_row, int slot, int kh, int lane) {
    const int hd = a.hd;
    const T* knew = (const T*)a.kv_new;
    const T* cache = (const T*)a.cache.storage;
    const size_t vhalf = cache ? kv_half_elems(a.cache) : 0;
    for (int base = lo; base < hi; base += 32) {
        const int kpos = base + lane;
        const bool valid = kpos < hi;
        const T* kp = nullptr;
        const T* vp = nullptr;
        if (valid) {
            if (kpos >= first_new) {
                kp = knew + (size_t)(first_new_row + kpos - first_new) * a.kv_stride + kh * hd;
                vp = kp + a.nkv * hd;
            } else {
                kp = cache + kv_row_offset(a.cache, slot, kpos, kh);
                vp = kp + vhalf;
            }
        }
        float s = -FLT_MAX;
        if (valid) {
            float dot = 0.f;
            for (int e = 0; e < hd; e += 8) {
                float kv[8];
                load8<T>(kp + e, kv);
#pragma unroll
                for (int i = 0; i < 8; ++i) dot = fmaf(qs[e + i], kv[i], dot);
            }
            s = dot * a.scale;
        }
        const float m_new = fmaxf(st.m, warp_max(s));
        const float alpha = expf(st.m - m_new);           // st.m = -FLT_MAX at the start: exp(-huge) = 0
        const float p = valid ? expf(s - m_new) : 0.f;
        st.l = st.l * alpha + warp_sum(p);
        st.m = m_new;
#pragma unroll
        for (int j = 0; j < ATT_MAXE; ++j) st.acc[j] *= alpha;
        const int n_valid = min(32, hi - base);
        for (int kk = 0; kk < n_valid; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            const T* v = (const T*)__shfl_sync(0xffffffffu, (unsigned long long)vp, kk);
#pragma unroll
            for (int j = 0; j < ATT_MAXE; ++j) {
                const int d = lane + 32 * j;
                if (d < hd) st.acc[j] = fmaf(pk, ldf(v + d), st.acc[j]);
            }
        }
    }
}

template <typename T>
__device__ __forceinline__ void load_query(float* qs, const T* q, int hd, int lane) {
    for (int e = lane; e < hd; e += 32) qs[e] = ldf(q + e);
    __syncwarp();
}

// ------------------------------------------------------------------ prefill
// grid (T, ceil(nh / ATT_WARPS)); warp = one head of one query token.
template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32) attn_prefill_kernel(AttnArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float q_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x, h = blockIdx.y * ATT_WARPS + warp;
    if (h >= a.nh) return;
    const int hd = a.hd;
    float* qs = q_smem + warp * hd;
    load_query<T>(qs, (const T*)a.q + (size_t)t * a.q_stride + h * hd, hd, lane);
    const int seq = a.batch.seq_of[t], pos = a.batch.pos_of[t];
    const int slot = a.batch.slot_of_seq[seq];
    const int first_new = a.kv_new ? a.batch.start_pos[seq] : 0x7fffffff;
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    Running st;
    st.m = -FLT_MAX; st.l = 0.f;
#pragma unroll
    for (int j = 0; j < ATT_MAXE; ++j) st.acc[j] = 0.f;
    attend_range<T>(st, qs, a, lo, pos + 1, first_new, a.batch.q_start[seq], slot, h / (a.nh / a.nkv), lane);
    const float inv = 1.0f / st.l;
    T* o = (T*)a.out + (size_t)t * a.out_stride + h * hd;
#pragma unroll
    for (int j = 0; j < ATT_MAXE; ++j) {
        const int d = lane + 32 * j;
        if (d < hd) stf(o + d, st.acc[j] * inv);
    }
}

// ------------------------------------------------------------------ decode, split over the keys
// grid (B, nkv, n_splits); the warps of a block take the query heads of one kv head in turn.
// Partial of (sequence b, head h, split s) at scratch[((b * nh + h) * n_splits + s) * (hd + 2)]:
// hd unnormalised outputs, then m, then l (l = 0: the split saw no key).
template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32) attn_decode_kernel(AttnArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float q_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b = blockIdx.x, kh = blockIdx.y, split = blockIdx.z;
    const int hd = a.hd, group = a.nh / a.nkv;
    const int len = a.batch.kv_len[b];
    const int keys = tb_split_keys(len, a.chunk, a.n_splits);
    if ((long long)split * keys >= len) return;     // the merge reads ceil(len / keys) splits only
    const int pos = len - 1;
    const int slot = a.batch.slot_of_seq[b];
    const int wlo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int lo = max(wlo, split * keys), hi = min(len, (split + 1) * keys);
    float* qs = q_smem + warp * hd;
    for (int g = warp; g < group; g += ATT_WARPS) {
        const int h = kh * group + g;
        float* part = a.scratch + ((size_t)(b * a.nh + h) * a.n_splits + split) * (hd + 2);
        Running st;
        st.m = -FLT_MAX; st.l = 0.f;
#pragma unroll
        for (int j = 0; j < ATT_MAXE; ++j) st.acc[j] = 0.f;
        if (lo < hi) {
            __syncwarp();
            load_query<T>(qs, (const T*)a.q + (size_t)b * a.q_stride + h * hd, hd, lane);
            attend_range<T>(st, qs, a, lo, hi, 0x7fffffff, 0, slot, kh, lane);
        }
#pragma unroll
        for (int j = 0; j < ATT_MAXE; ++j) {
            const int d = lane + 32 * j;
            if (d < hd) part[d] = st.acc[j];
        }
        if (lane == 0) { part[hd] = st.m; part[hd + 1] = st.l; }
    }
}

// grid (B, nh), one warp: out = sum_s exp(m_s - m) acc_s / sum_s exp(m_s - m) l_s, splits in order.
// Lane s holds the weight of split s (32 splits per round), so the loads of the accumulation are
// independent of one another.
template <typename T>
__global__ void attn_merge_kernel(AttnArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x, h = blockIdx.y, lane = threadIdx.x, hd = a.hd, stride = hd + 2;
    const float* part = a.scratch + (size_t)(b * a.nh + h) * a.n_splits * stride;
    const int len = a.batch.kv_len[b], keys = tb_split_keys(len, a.chunk, a.n_splits);
    const int used = min(a.n_splits, (len + keys - 1) / keys);
    float m = -FLT_MAX;
    for (int s = lane; s < used; s += 32)
        if (part[s * stride + hd + 1] > 0.f) m = fmaxf(m, part[s * stride + hd]);
    m = warp_max(m);
    float l = 0.f, acc[ATT_MAXE];
#pragma unroll
    for (int j = 0; j < ATT_MAXE; ++j) acc[j] = 0.f;
    for (int s0 = 0; s0 < used; s0 += 32) {
        const int s = s0 + lane;
        float w = 0.f;
        if (s < used) {
            const float ls = part[s * stride + hd + 1];
            if (ls > 0.f) { w = expf(part[s * stride + hd] - m); l += w * ls; }
        }
        const int n = min(32, used - s0);
        for (int k = 0; k < n; ++k) {
            const float wk = __shfl_sync(0xffffffffu, w, k);
            const float* p = part + (size_t)(s0 + k) * stride;
#pragma unroll
            for (int j = 0; j < ATT_MAXE; ++j) {
                const int d = lane + 32 * j;
                if (d < hd) acc[j] = fmaf(wk, p[d], acc[j]);
            }
        }
    }
    l = warp_sum(l);
    const float inv = 1.0f / l;
    T* o = (T*)a.out + (size_t)b * a.out_stride + h * hd;
#pragma unroll
    for (int j = 0; j < ATT_MAXE; ++j) {
        const int d = lane + 32 * j;
        if (d < hd) stf(o + d, acc[j] * inv);
    }
}

static int check_common(const AttnArgs& a, const char* who) {
    TB_REQUIRE(a.nh > 0 && a.nkv > 0 && a.nh % a.nkv == 0, "%s: %d query heads are not a multiple of %d kv heads", who, a.nh, a.nkv);
    TB_REQUIRE(a.hd >= 8 && a.hd % 8 == 0 && a.hd <= 32 * ATT_MAXE, "%s: head_dim %d must be a multiple of 8 up to %d", who, a.hd, 32 * ATT_MAXE);
    TB_REQUIRE(a.q_stride % 8 == 0 && a.kv_stride % 8 == 0, "%s: row strides must be multiples of 8 elements", who);
    TB_REQUIRE(a.window >= 0, "%s: negative window", who);
    TB_REQUIRE(!a.cache.storage || (a.cache.head_dim == a.hd && a.cache.kv_heads == a.nkv), "%s: the cache view does not match the heads", who);
    return 0;
}

extern "C" int tb_attn_prefill(const AttnArgs* args, int dtype, cudaStream_t stream) {
    AttnArgs a = *args;
    if (check_common(a, "attn_prefill")) return 1;
    TB_REQUIRE(a.batch.T > 0, "attn_prefill: no tokens");
    TB_REQUIRE(a.kv_new || a.cache.storage, "attn_prefill: neither new keys nor a cache");
    dim3 grid(a.batch.T, (a.nh + ATT_WARPS - 1) / ATT_WARPS);
    const size_t smem = (size_t)ATT_WARPS * a.hd * sizeof(float);
    if (dtype == TB_F32) tb_launch(attn_prefill_kernel<float>, grid, ATT_WARPS * 32, smem, stream, a);
    else if (dtype == TB_BF16) tb_launch(attn_prefill_kernel<__nv_bfloat16>, grid, ATT_WARPS * 32, smem, stream, a);
    else TB_REQUIRE(false, "attn_prefill: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("attn_prefill");
    return 0;
}

extern "C" int tb_attn_merge(const AttnArgs* args, int dtype, cudaStream_t stream) {
    AttnArgs a = *args;
    dim3 mgrid(a.batch.B, a.nh);
    if (dtype == TB_F32) tb_launch(attn_merge_kernel<float>, mgrid, 32, 0, stream, a);
    else if (dtype == TB_BF16) tb_launch(attn_merge_kernel<__nv_bfloat16>, mgrid, 32, 0, stream, a);
    else TB_REQUIRE(false, "attn_merge: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("attn_merge");
    return 0;
}

extern "C" int tb_attn_decode(const AttnArgs* args, int dtype, cudaStream_t stream) {
    AttnArgs a = *args;
    if (check_common(a, "attn_decode")) return 1;
    TB_REQUIRE(a.batch.B > 0 && a.cache.storage && a.scratch, "attn_decode: needs sequences, a cache and scratch");
    TB_REQUIRE(a.chunk > 0 && a.n_splits > 0 && a.n_splits <= 65535, "attn_decode: bad split (chunk=%d splits=%d)", a.chunk, a.n_splits);
    TB_REQUIRE(a.nkv <= 65535, "attn_decode: too many kv heads");
    dim3 grid(a.batch.B, a.nkv, a.n_splits), mgrid(a.batch.B, a.nh);
    const size_t smem = (size_t)ATT_WARPS * a.hd * sizeof(float);
    if (dtype == TB_F32) {
        tb_launch(attn_decode_kernel<float>, grid, ATT_WARPS * 32, smem, stream, a);
        tb_launch(attn_merge_kernel<float>, mgrid, 32, 0, stream, a);
    } else if (dtype == TB_BF16) {
        tb_launch(attn_decode_kernel<__nv_bfloat16>, grid, ATT_WARPS * 32, smem, stream, a);
        tb_launch(attn_merge_kernel<__nv_bfloat16>, mgrid, 32, 0, stream, a);
    } else TB_REQUIRE(false, "attn_decode: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("attn_decode");
    return 0;
}
