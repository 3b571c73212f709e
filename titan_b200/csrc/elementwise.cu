// Row kernels: embedding gather, RMSNorm, per-head Q/K norm + rotary (+ cache append),
// cache append of a prompt's keys and values, and the device-side step bookkeeping.
//
// Counterparts in berniehans/titan: get_rows_* (engine/engine-cuda/kernels/gemm_quant.cu:2365-2508),
// norm_rope_swiglu_kernel and fused_qk_norm_rope_kernel (kernels/norm_rope.cu:3-134, 136-300),
// paged_append_kv_kernel (kernels/paged_kv.cu:13-45), gpu_advance_token_step_kernel
// (kernels/gemm_quant.cu:2570-2587).  Sums of squares, the norm scale and the rotation
// angle are float32 with precise sqrtf / sincosf (the reference uses fast-math, norm_rope.cu:101-113).
#include "common.cuh"
#include "qk_args.h"

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int H, int V) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int tok = tokens[t];
    tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);   // ids are validated on the host; never read outside
    const T* row = table + (size_t)tok * H;
    float* o = out + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = ldf(row + i);
}

extern "C" int tb_embed(const void* table, int dtype, const int* tokens, float* out, int T, int H, int V,
                        cudaStream_t stream) {
    TB_REQUIRE(T > 0 && H > 0 && V > 0, "embed: sizes must be positive (T=%d H=%d V=%d)", T, H, V);
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == TB_F32)
        tb_launch(embed_kernel<float>, T, threads, 0, stream, (const float*)table, tokens, out, H, V);
    else if (dtype == TB_BF16)
        tb_launch(embed_kernel<__nv_bfloat16>, T, threads, 0, stream, (const __nv_bfloat16*)table, tokens, out, H, V);
    else
        TB_REQUIRE(false, "embed: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("embed");
    return 0;
}

// x *= factor (float32, in place): an embedding multiplier or a logit scale of the model's description.
__global__ void scale_f32_kernel(float* __restrict__ x, long long n, float factor) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) x[i] *= factor;
}

extern "C" int tb_scale_f32(float* x, long long n, float factor, cudaStream_t stream) {
    TB_REQUIRE(x && n > 0, "scale_f32: nothing to scale");
    const int threads = 256;
    const long long blocks = (n + threads - 1) / threads;
    tb_launch(scale_f32_kernel, (int)(blocks < 4096 ? blocks : 4096), threads, 0, stream, x, n, factor);
    TB_CHECK_LAUNCH("scale_f32");
    return 0;
}

// ------------------------------------------------------------------ RMSNorm
// y[r] = x[rows ? rows[r] : r] * 1/sqrt(mean(x^2) + eps) * w      (x float32, y in the compute dtype)
template <typename T> __device__ __forceinline__ void store4(T* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&lo);
    u.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
}

// VEC: H is a multiple of 4 and a row fits the block's registers (H <= 16 * blockDim): the row is read
// once, as float4, and kept in registers between the sum of squares and the scaling.
template <typename T, bool VEC>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                               const int* __restrict__ rows, int H, float eps) {
    pdl_launch_dependents();
    __shared__ float red[33];
    const int r = blockIdx.x;
    T* yr = y + (size_t)r * H;
    if (VEC) {
        float4 v[4], ww[4];
        const int n4 = H >> 2;
        // the norm's weight depends on nothing that the kernel before makes: requested while the wait for it lasts
        // (it used to be a round trip of its own after the row's sum)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            ww[j] = i < n4 ? reinterpret_cast<const float4*>(w)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        pdl_wait();
        const float* xr = x + (size_t)(rows ? rows[r] : r) * H;
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            v[j] = i < n4 ? reinterpret_cast<const float4*>(xr)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
        ss = block_sum(ss, red);
        const float scale = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < n4)
                store4<T>(yr + 4 * i, v[j].x * scale * ww[j].x, v[j].y * scale * ww[j].y, v[j].z * scale * ww[j].z, v[j].w * scale * ww[j].w);
        }
    } else {
        pdl_wait();
        const float* xr = x + (size_t)(rows ? rows[r] : r) * H;
        float ss = 0.f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = xr[i];
            ss += v * v;
        }
        ss = block_sum(ss, red);
        const float scale = 1.0f / sqrtf(ss / (float)H + eps);
        for (int i = threadIdx.x; i < H; i += blockDim.x) stf(yr + i, xr[i] * scale * w[i]);
    }
}

template <typename T>
static void launch_rmsnorm(const float* x, const float* w, T* y, const int* rows, int n_rows, int H, float eps, cudaStream_t stream) {
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : (H >= 256 ? 64 : 32));
    const bool vec = (H % 4 == 0) && H <= 16 * threads && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)y % 16 == 0);
    if (vec) tb_launch(rmsnorm_kernel<T, true>, n_rows, threads, 0, stream, x, w, y, rows, H, eps);
    else tb_launch(rmsnorm_kernel<T, false>, n_rows, threads, 0, stream, x, w, y, rows, H, eps);
}

extern "C" int tb_rmsnorm(const float* x, const float* w, void* y, int dtype, const int* rows, int n_rows,
                          int H, float eps, cudaStream_t stream) {
    TB_REQUIRE(n_rows > 0 && H > 0, "rmsnorm: sizes must be positive (rows=%d H=%d)", n_rows, H);
    if (dtype == TB_F32) launch_rmsnorm<float>(x, w, (float*)y, rows, n_rows, H, eps, stream);
    else if (dtype == TB_BF16) launch_rmsnorm<__nv_bfloat16>(x, w, (__nv_bfloat16*)y, rows, n_rows, H, eps, stream);
    else TB_REQUIRE(false, "rmsnorm: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("rmsnorm");
    return 0;
}

// The scale of a row whose norm was folded into the projection: its partial sums of squares, one per K slice of
// that product, added in slice order (read through L2: they were written by the kernel just before).
__device__ __forceinline__ float folded_row_scale(const QkArgs& a, int t) {
    if (!a.row_sumsq) return 1.f;
    float total = 0.f;
    for (int z = 0; z < a.row_parts; ++z) total += __ldcg(a.row_sumsq + z * 32 + t);
    return 1.0f / sqrtf(total / (float)a.row_width + a.row_eps);
}

// ------------------------------------------------------------------ Q/K head norm + rotary (+ append)
// One warp per (token, head).  Heads 0..nh-1 are Q, nh..nh+nkv-1 are K, and, when the cache is
// written here, nh+nkv.. are V (copied unchanged).  Per head: RMSNorm over head_dim with a shared
// weight (skipped when the weight pointer is null), then the half-split rotation of the first
// ``rot`` dims: for k < rot/2, angle = (pos + offset) * inv_freq[k], (y_k, y_{k+rot/2}) rotated and
// scaled by ``magnitude`` (offset 0 and magnitude 1 for plain rotary; TbRotary in qk_args.h)
// (kernels/norm_rope.cu:226-245 and :83-117 in berniehans/titan).
#define QK_MAXE 8   // head_dim <= 32 * QK_MAXE

template <typename TIn, typename TOut>
__global__ void qk_norm_rope_kernel(QkArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float head_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int t = blockIdx.x;
    const int head = blockIdx.y * nwarp + warp;
    const int n_heads = a.nh + a.nkv + (a.append ? a.nkv : 0);
    // cosine and sine of this token's angles, once per block: [rot/2] each, behind the warps' rows
    float* cs = head_smem + nwarp * a.hd;
    float* sn = cs + (a.rope.rot >> 1);
    if (a.rope.inv_freq) {
        const float p = (float)a.pos_of[t] + a.rope.offset;
        for (int k = threadIdx.x; k < (a.rope.rot >> 1); k += blockDim.x) {
            float sv, cv;
            sincosf(p * a.rope.inv_freq[k], &sv, &cv);
            sn[k] = sv * a.rope.magnitude; cs[k] = cv * a.rope.magnitude;
        }
    }
    __syncthreads();
    if (head >= n_heads) return;
    float* y = head_smem + warp * a.hd;
    const int hd = a.hd;
    const bool is_q = head < a.nh, is_k = !is_q && head < a.nh + a.nkv;
    const int col = is_q ? head * hd : (is_k ? a.nh * hd + (head - a.nh) * hd
                                             : (a.nh + a.nkv) * hd + (head - a.nh - a.nkv) * hd);
    const TIn* x = (const TIn*)a.in + (size_t)t * a.in_stride + col;
    const float row_scale = folded_row_scale(a, t);
    float v[QK_MAXE];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < QK_MAXE; ++j) {
        const int e = lane + 32 * j;
        v[j] = e < hd ? ldf(x + e) * row_scale : 0.f;
        ss += v[j] * v[j];
        if (a.zero_in && e < hd) const_cast<TIn*>(x)[e] = TIn(0.f);
    }
    const int pos = a.pos_of[t];
    const int seq = a.seq_of[t];
    const int slot = a.slot_of_seq[seq];
    const bool to_cache = a.append && !(a.cache.ring_rows && a.kv_len && pos < a.kv_len[seq] - a.cache.ring_rows);
    if (!is_q && !is_k) {   // V: straight copy into the cache
        if (!to_cache) return;
        TOut* dst = (TOut*)a.cache.storage + kv_half_elems(a.cache) + kv_row_offset(a.cache, slot, pos, head - a.nh - a.nkv);
#pragma unroll
        for (int j = 0; j < QK_MAXE; ++j) {
            const int e = lane + 32 * j;
            if (e < hd) stf(dst + e, v[j]);
        }
        return;
    }
    const float* w = is_q ? a.q_w : a.k_w;
    float scale = 1.f;
    if (w) {
        ss = warp_sum(ss);
        scale = 1.0f / sqrtf(ss / (float)hd + a.eps);
    }
#pragma unroll
    for (int j = 0; j < QK_MAXE; ++j) {
        const int e = lane + 32 * j;
        if (e < hd) y[e] = w ? v[j] * scale * w[e] : v[j];
    }
    __syncwarp();
    const int half = a.rope.rot >> 1;
    TOut* out = is_q ? (TOut*)a.q_out + (size_t)t * a.q_stride + head * hd
                     : (a.k_out ? (TOut*)a.k_out + (size_t)t * a.k_stride + (head - a.nh) * hd : nullptr);
    TOut* cdst = (is_k && to_cache)
                     ? (TOut*)a.cache.storage + kv_row_offset(a.cache, slot, pos, head - a.nh) : nullptr;
#pragma unroll
    for (int j = 0; j < QK_MAXE; ++j) {
        const int e = lane + 32 * j;
        if (e >= hd) continue;
        float r = y[e];
        if (a.rope.inv_freq && e < a.rope.rot) {
            const bool first = e < half;
            const int k = first ? e : e - half;
            const float s = sn[k], c = cs[k];
            r = first ? y[e] * c - y[e + half] * s : y[e - half] * s + y[e] * c;
        }
        if (out) stf(out + e, r);
        if (cdst) stf(cdst + e, r);
    }
}

// Fast path for head sizes 64, 128 and 256 with the rotation over the whole head (or none): a lane
// holds a few consecutive elements of the head's first half and their rotation partners from the second
// half, so the head never goes through shared memory.  Arguments and results are those of
// qk_norm_rope_kernel.
template <typename T, int VE> __device__ __forceinline__ void load_vec(const T* p, float* o) {
    constexpr int BYTES = VE * (int)sizeof(T);
    T tmp[VE];
    if constexpr (BYTES == 32) {
        const uint4 a = reinterpret_cast<const uint4*>(p)[0], b = reinterpret_cast<const uint4*>(p)[1];
        memcpy(tmp, &a, 16);
        memcpy(reinterpret_cast<char*>(tmp) + 16, &b, 16);
    } else if constexpr (BYTES == 16) {
        const uint4 a = *reinterpret_cast<const uint4*>(p);
        memcpy(tmp, &a, 16);
    } else if constexpr (BYTES == 8) {
        const uint2 a = *reinterpret_cast<const uint2*>(p);
        memcpy(tmp, &a, 8);
    } else {
        const uint32_t a = *reinterpret_cast<const uint32_t*>(p);
        memcpy(tmp, &a, 4);
    }
#pragma unroll
    for (int i = 0; i < VE; ++i) o[i] = ldf(tmp + i);
}
template <typename T, int VE> __device__ __forceinline__ void store_vec(T* p, const float* v) {
    constexpr int BYTES = VE * (int)sizeof(T);
    T tmp[VE];
#pragma unroll
    for (int i = 0; i < VE; ++i) stf(tmp + i, v[i]);
    if constexpr (BYTES == 32) {
        uint4 a, b;
        memcpy(&a, tmp, 16);
        memcpy(&b, reinterpret_cast<char*>(tmp) + 16, 16);
        reinterpret_cast<uint4*>(p)[0] = a;
        reinterpret_cast<uint4*>(p)[1] = b;
    } else if constexpr (BYTES == 16) {
        uint4 a;
        memcpy(&a, tmp, 16);
        *reinterpret_cast<uint4*>(p) = a;
    } else if constexpr (BYTES == 8) {
        uint2 a;
        memcpy(&a, tmp, 8);
        *reinterpret_cast<uint2*>(p) = a;
    } else {
        uint32_t a;
        memcpy(&a, tmp, 4);
        *reinterpret_cast<uint32_t*>(p) = a;
    }
}

// A block takes TOK tokens.  First it puts what depends on the token alone into shared memory: the
// rotation's cosines and sines and the place of the token's row in the cache (position, slot, block
// table: a chain of dependent loads that is paid once per token, not once per head).  Then every warp
// walks over heads (blockIdx.y * warps + warp, in steps of gridDim.y * warps), the same head for all TOK
// tokens, whose TOK loads are in flight together.  A decode step launches one token and few heads per
// block (many small blocks); a prompt launches four tokens and half of the heads per block.
template <typename TIn, typename TOut, int HD, int LPH, int TOK>
__global__ void qk_norm_rope_vec_kernel(QkArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float head_smem[];
    constexpr int HALF = HD / 2;
    __shared__ long long row_off[TOK];              // element offset of the token's cache row for kv head 0; < 0: not written
    __shared__ float row_scale[TOK];                // what the token's input row is multiplied by first (a folded norm's scale)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int t0 = blockIdx.x * TOK;
    const int n_tok = a.T - t0 < TOK ? a.T - t0 : TOK;
    const int n_heads = a.nh + a.nkv + (a.append ? a.nkv : 0);
    float* cs = head_smem;                           // [TOK][HALF] cosines, then [TOK][HALF] sines
    float* sn = cs + TOK * HALF;
    if (threadIdx.x < n_tok) {
        const int t = t0 + threadIdx.x;
        const int pos = a.pos_of[t], seq = a.seq_of[t];
        const bool to_cache = a.append && !(a.cache.ring_rows && a.kv_len && pos < a.kv_len[seq] - a.cache.ring_rows);
        row_off[threadIdx.x] = to_cache ? (long long)kv_row_offset(a.cache, a.slot_of_seq[seq], pos, 0) : -1;
        row_scale[threadIdx.x] = folded_row_scale(a, t);
    }
    if (a.rope.inv_freq) {
        for (int i = threadIdx.x; i < n_tok * HALF; i += blockDim.x) {
            const int j = i / HALF, k = i - j * HALF;
            float sv, cv;
            sincosf(((float)a.pos_of[t0 + j] + a.rope.offset) * a.rope.inv_freq[k], &sv, &cv);
            sn[i] = sv * a.rope.magnitude; cs[i] = cv * a.rope.magnitude;
        }
    }
    __syncthreads();
    const size_t head_stride = (size_t)a.cache.page_size * a.cache.head_dim;      // between kv heads of a page
    // LPH lanes hold a head, so a warp works on 32 / LPH heads at once.  A lane holds HV = HD / LPH / 2
    // consecutive elements of the head's first half and the HV elements HD / 2 further on: an element and
    // its rotation partner sit in the same lane, and both use the same angle.  Every lane runs every
    // shuffle of the norm's sum: what a lane's head needs (norm, rotation, where it goes) is data, not
    // control flow.
    constexpr int HPW = 32 / LPH, HV = HD / LPH / 2;
    const int sub = lane / LPH, l = lane % LPH;
    for (int group = blockIdx.y * nwarp + warp; group * HPW < n_heads; group += gridDim.y * nwarp) {
        const int head = group * HPW + sub;
        const bool live = head < n_heads;
        const bool is_q = head < a.nh, is_k = !is_q && head < a.nh + a.nkv;
        const int col = head * HD + l * HV;          // Q heads, then K heads, then V heads, all HD wide
        float lo[TOK][HV], hi[TOK][HV];
#pragma unroll
        for (int j = 0; j < TOK; ++j) {              // all loads first
            if (live && j < n_tok) {
                const TIn* src = (const TIn*)a.in + (size_t)(t0 + j) * a.in_stride + col;
                load_vec<TIn, HV>(src, lo[j]);
                load_vec<TIn, HV>(src + HALF, hi[j]);
            } else {
#pragma unroll
                for (int i = 0; i < HV; ++i) lo[j][i] = hi[j][i] = 0.f;
            }
        }
        const float* w = is_q ? a.q_w : (is_k ? a.k_w : nullptr);
        float wlo[HV], whi[HV];
#pragma unroll
        for (int i = 0; i < HV; ++i) {
            wlo[i] = w ? w[l * HV + i] : 1.f;
            whi[i] = w ? w[HALF + l * HV + i] : 1.f;
        }
        const bool rotate = a.rope.inv_freq && (is_q || is_k);
        // No early exit from this loop: its TOK bodies are independent, and the compiler interleaves
        // them; a token beyond the end computes on zeros and stores nothing.
#pragma unroll
        for (int j = 0; j < TOK; ++j) {
            const bool tok_live = live && j < n_tok;
            const int t = t0 + j;
            if (a.zero_in && tok_live) {
                float z[HV];
#pragma unroll
                for (int i = 0; i < HV; ++i) z[i] = 0.f;
                TIn* src = (TIn*)const_cast<void*>(a.in) + (size_t)t * a.in_stride + col;
                store_vec<TIn, HV>(src, z);
                store_vec<TIn, HV>(src + HALF, z);
            }
            const float rs = row_scale[j < n_tok ? j : 0];
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < HV; ++i) {
                lo[j][i] *= rs; hi[j][i] *= rs;
                ss += lo[j][i] * lo[j][i] + hi[j][i] * hi[j][i];
            }
#pragma unroll
            for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float scale = w ? 1.0f / sqrtf(ss / (float)HD + a.eps) : 1.f;
#pragma unroll
            for (int i = 0; i < HV; ++i) {
                const float x = lo[j][i] * scale * wlo[i], y = hi[j][i] * scale * whi[i];
                const float c = rotate ? cs[j * HALF + l * HV + i] : 1.f, sv = rotate ? sn[j * HALF + l * HV + i] : 0.f;
                lo[j][i] = x * c - y * sv;
                hi[j][i] = y * c + x * sv;
            }
            if (!tok_live) continue;
            const long long off = row_off[j];
            TOut* dst = nullptr;
            if (is_q) {
                dst = (TOut*)a.q_out + (size_t)t * a.q_stride + col;
            } else if (is_k) {
                if (a.k_out) {
                    TOut* kd = (TOut*)a.k_out + (size_t)t * a.k_stride + col - a.nh * HD;
                    store_vec<TOut, HV>(kd, lo[j]);
                    store_vec<TOut, HV>(kd + HALF, hi[j]);
                }
                if (off >= 0) dst = (TOut*)a.cache.storage + (size_t)off + (size_t)(head - a.nh) * head_stride + l * HV;
            } else if (off >= 0) {
                dst = (TOut*)a.cache.storage + kv_half_elems(a.cache) + (size_t)off + (size_t)(head - a.nh - a.nkv) * head_stride + l * HV;
            }
            if (dst) {
                store_vec<TOut, HV>(dst, lo[j]);
                store_vec<TOut, HV>(dst + HALF, hi[j]);
            }
        }
    }
}

template <typename TIn, typename TOut, int TOK>
static void launch_qk_vec_tok(const QkArgs& a, int warps, int head_groups, cudaStream_t stream) {
    dim3 grid((a.T + TOK - 1) / TOK, head_groups);
    const size_t smem = (size_t)TOK * a.hd * sizeof(float);
    // sixteen lanes per head where a lane's share still is one or two 16-byte accesses
    if (a.hd == 64) tb_launch(qk_norm_rope_vec_kernel<TIn, TOut, 64, 16, TOK>, grid, warps * 32, smem, stream, a);
    else if (a.hd == 128) tb_launch(qk_norm_rope_vec_kernel<TIn, TOut, 128, 16, TOK>, grid, warps * 32, smem, stream, a);
    else tb_launch(qk_norm_rope_vec_kernel<TIn, TOut, 256, 32, TOK>, grid, warps * 32, smem, stream, a);
}
template <typename TIn, typename TOut>
static void launch_qk_vec(const QkArgs& a, dim3 grid, int threads, cudaStream_t stream) {
    (void)threads;
    if (a.T >= 512) launch_qk_vec_tok<TIn, TOut, 4>(a, 4, 2, stream);         // prompts: half of the heads of four tokens per block
    else launch_qk_vec_tok<TIn, TOut, 1>(a, 4, (grid.y + 1) / 2, stream);    // decode steps and short prompts: eight heads of one token per block (T x heads / 8 blocks)
}

extern "C" int tb_qk_norm_rope(const QkArgs* args, int in_dtype, int out_dtype, cudaStream_t stream) {
    QkArgs a = *args;
    TB_REQUIRE(a.T > 0 && a.nh > 0 && a.nkv >= 0, "qk_norm_rope: sizes must be positive");
    TB_REQUIRE(a.hd > 0 && a.hd <= 32 * QK_MAXE, "qk_norm_rope: head_dim %d is not in 1..%d", a.hd, 32 * QK_MAXE);
    TB_REQUIRE(a.rope.rot >= 0 && a.rope.rot <= a.hd && a.rope.rot % 2 == 0, "qk_norm_rope: rotary_dim %d must be even and <= head_dim %d", a.rope.rot, a.hd);
    TB_REQUIRE(!a.zero_in || (a.append && a.in != a.q_out && a.k_out == nullptr),
               "qk_norm_rope: zeroing the input needs every head to be read (append) and outputs elsewhere");
    TB_REQUIRE(!a.row_sumsq || (a.row_width > 0 && a.row_parts > 0 && a.T <= 32), "qk_norm_rope: row sums of squares need the rows' width, their number of parts and at most 32 rows");
    TB_REQUIRE(!a.append || (a.cache.storage && a.cache.head_dim == a.hd && a.cache.kv_heads == a.nkv),
               "qk_norm_rope: the cache view does not match the heads");
    const int warps = 4;
    const int n_heads = a.nh + a.nkv + (a.append ? a.nkv : 0);
    dim3 grid(a.T, (n_heads + warps - 1) / warps);
    const size_t smem = ((size_t)warps * a.hd + a.rope.rot) * sizeof(float);
    const int in_bytes = in_dtype == TB_F32 ? 4 : 2, out_bytes = out_dtype == TB_F32 ? 4 : 2;
    const int hv = a.hd == 256 ? 4 : a.hd / 32;        // consecutive elements per lane and half of the fast path
    auto aligned = [&](const void* p, long long stride_elems, int esz) {
        const int unit = hv * esz < 16 ? hv * esz : 16;   // read and written in pieces of at most 16 bytes
        return p == nullptr || (((uintptr_t)p % (size_t)unit) == 0 && (stride_elems * esz) % unit == 0);
    };
    const bool vec = (a.hd == 64 || a.hd == 128 || a.hd == 256) && (a.rope.rot == a.hd || !a.rope.inv_freq) &&
                     aligned(a.in, a.in_stride, in_bytes) && aligned(a.q_out, a.q_stride, out_bytes) &&
                     aligned(a.k_out, a.k_stride, out_bytes) && aligned(a.cache.storage, a.hd, out_bytes);
    if (in_dtype == TB_F32 && out_dtype == TB_F32) {
        if (vec) launch_qk_vec<float, float>(a, grid, warps * 32, stream);
        else tb_launch(qk_norm_rope_kernel<float, float>, grid, warps * 32, smem, stream, a);
    } else if (in_dtype == TB_BF16 && out_dtype == TB_BF16) {
        if (vec) launch_qk_vec<__nv_bfloat16, __nv_bfloat16>(a, grid, warps * 32, stream);
        else tb_launch(qk_norm_rope_kernel<__nv_bfloat16, __nv_bfloat16>, grid, warps * 32, smem, stream, a);
    } else if (in_dtype == TB_F32 && out_dtype == TB_BF16) {
        if (vec) launch_qk_vec<float, __nv_bfloat16>(a, grid, warps * 32, stream);
        else tb_launch(qk_norm_rope_kernel<float, __nv_bfloat16>, grid, warps * 32, smem, stream, a);
    } else {
        TB_REQUIRE(false, "qk_norm_rope: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
    }
    TB_CHECK_LAUNCH("qk_norm_rope");
    return 0;
}

// ------------------------------------------------------------------ append a prompt's K and V
// Copies rows of the step's own K | V (``kv`` [T][stride], K heads then V heads) into the cache.
// In a ring, a token whose row a later token of the same step also maps to is skipped.
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ kv, int stride, TbKvView c, const int* pos_of,
                                 const int* seq_of, const int* slot_of_seq, const int* kv_len) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, h2 = blockIdx.y;            // h2 < 2 * kv_heads
    const int seq = seq_of[t], pos = pos_of[t];
    if (c.ring_rows && pos < kv_len[seq] - c.ring_rows) return;
    const int is_v = h2 >= c.kv_heads, head = is_v ? h2 - c.kv_heads : h2;
    const T* src = kv + (size_t)t * stride + (size_t)h2 * c.head_dim;
    T* dst = (T*)c.storage + (is_v ? kv_half_elems(c) : 0) + kv_row_offset(c, slot_of_seq[seq], pos, head);
    constexpr int PER = 16 / sizeof(T);            // elements per 16-byte chunk
    if (c.head_dim % PER == 0 && ((uintptr_t)src % 16 == 0) && ((uintptr_t)dst % 16 == 0)) {
        for (int e = threadIdx.x; e < c.head_dim / PER; e += blockDim.x)
            reinterpret_cast<uint4*>(dst)[e] = reinterpret_cast<const uint4*>(src)[e];
    } else {
        for (int e = threadIdx.x; e < c.head_dim; e += blockDim.x) dst[e] = src[e];
    }
}

extern "C" int tb_kv_append(const void* kv, int stride, int dtype, const TbKvView* cache, const TbBatch* b,
                            cudaStream_t stream) {
    TbKvView c = *cache;
    TB_REQUIRE(b->T > 0 && c.storage, "kv_append: nothing to append or no cache");
    dim3 grid(b->T, 2 * c.kv_heads);
    const int threads = 32;
    if (dtype == TB_F32)
        tb_launch(kv_append_kernel<float>, grid, threads, 0, stream, (const float*)kv, stride, c, b->pos_of, b->seq_of, b->slot_of_seq, b->kv_len);
    else if (dtype == TB_BF16)
        tb_launch(kv_append_kernel<__nv_bfloat16>, grid, threads, 0, stream, (const __nv_bfloat16*)kv, stride, c, b->pos_of, b->seq_of, b->slot_of_seq, b->kv_len);
    else
        TB_REQUIRE(false, "kv_append: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("kv_append");
    return 0;
}

// ------------------------------------------------------------------ device-side step bookkeeping
// A captured decode step must not depend on host values that change from step to step.  Before the
// blocks run, this kernel derives the step's layout from the per-slot state: the token to feed
// (the slot's last sampled token, or one the host has put into ``tokens``), its position, and the
// cache length after the step.  berniehans/titan keeps pos_dev and token_id_dev for the same reason
// (engine/engine-core/src/forward_driver.rs:2444-2452, kernels/gemm_quant.cu:2570-2587).
__global__ void decode_prepare_kernel(const int* __restrict__ slot_of_seq, const int* __restrict__ seq_len,
                                      const int* __restrict__ last_token, int feed_last, int* tokens, int* pos_of,
                                      int* start_pos, int* kv_len, int B) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    const int slot = slot_of_seq[b], len = seq_len[slot];
    if (feed_last) tokens[b] = last_token[slot];
    pos_of[b] = len;
    start_pos[b] = len;
    kv_len[b] = len + 1;
}

extern "C" int tb_decode_prepare(const int* slot_of_seq, const int* seq_len, const int* last_token, int feed_last,
                                 int* tokens, int* pos_of, int* start_pos, int* kv_len, int B, cudaStream_t stream) {
    TB_REQUIRE(B > 0, "decode_prepare: no sequences");
    tb_launch(decode_prepare_kernel, (B + 127) / 128, 128, 0, stream, slot_of_seq, seq_len, last_token, feed_last, tokens,
              pos_of, start_pos, kv_len, B);
    TB_CHECK_LAUNCH("decode_prepare");
    return 0;
}

// seq_len[slot_of_seq[b]] = kv_len[b]: the device copy of the lengths after a step.
__global__ void commit_lengths_kernel(const int* __restrict__ slot_of_seq, const int* __restrict__ kv_len,
                                      int* seq_len, int B) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B) seq_len[slot_of_seq[b]] = kv_len[b];
}

extern "C" int tb_commit_lengths(const int* slot_of_seq, const int* kv_len, int* seq_len, int B, cudaStream_t stream) {
    TB_REQUIRE(B > 0, "commit_lengths: no sequences");
    tb_launch(commit_lengths_kernel, (B + 127) / 128, 128, 0, stream, slot_of_seq, kv_len, seq_len, B);
    TB_CHECK_LAUNCH("commit_lengths");
    return 0;
}
