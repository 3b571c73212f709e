// Token sampling on the device: several blocks per row find the maximum and its lowest index (the
// answer when greedy), then one block per row does the rest.
//
// Order of operations, after berniehans/titan's host sampler (engine/engine-core/src/sampler.rs:109-240):
// repetition penalty over the tokens seen so far (positive logit / pen, else * pen, :132-145);
// temperature <= 1e-4 -> argmax (:148-158); else logits / T (:161-164), keep the top_k largest
// (:167-177), softmax with max subtraction (:184-200), keep the shortest descending prefix whose
// mass reaches top_p (:203-226), draw (:229-239).  Its device argmax is gpu_sample_greedy_kernel
// (engine/engine-cuda/kernels/gemm_quant.cu:2510-2568), which skips a vocabulary tail that is no
// multiple of 4 and breaks ties by thread order; here the whole vocabulary is read and the lowest
// index wins, in argmax and at the top_k / top_p borders.
//
// Differences, stated: top_k = 0 keeps the whole vocabulary (the reference keeps 1024); the
// draw walks the kept tokens in vocabulary order (same distribution, no sort); the uniform number
// is a hash of (seed, sequence id, step), so a sequence draws the same tokens in any batch.
// Masses are summed as 2^-40 fixed point in integers, so every sum is exact and order-free.
#include <float.h>
#include <limits.h>

#include "common.cuh"

struct SampleArgs {
    const float* logits; int ld; int V; int B;
    const int* slot_of_row;                      // [B]
    const float* temperature; const int* top_k; const float* top_p; const float* penalty;   // per slot
    const long long* seed; const long long* sequence_id; int* sample_step; int* last_token; // per slot
    unsigned* seen; int seen_words;              // per slot bitmap of context tokens, or null
    int* out;                                    // [B]
    float* part_best; int* part_idx; int parts;  // [B][parts] scratch: the maximum as found by several blocks per row (parts 0: one block scans the row)
};

typedef unsigned long long u64;

__device__ __forceinline__ unsigned order_key(float x) {      // larger float -> larger key; NaN -> 0
    if (x != x) return 0u;
    const unsigned u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__host__ __device__ inline u64 mix64(u64 z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// 24-bit uniform integer from (seed, sequence, step).
__host__ __device__ inline unsigned uniform24(u64 seed, u64 sequence, u64 step) {
    u64 z = seed * 0x9E3779B97F4A7C15ull + sequence * 0xBF58476D1CE4E5B9ull + step * 0x94D049BB133111EBull +
            0x2545F4914F6CDD1Dull;
    z = mix64(mix64(z));
    return (unsigned)(z >> 40);
}

struct Row {
    const float* logits; const unsigned* seen; float pen; float inv_t; int V;
    __device__ __forceinline__ float value(int i) const {
        float l = logits[i];
        if (seen && pen > 1.0f && ((seen[i >> 5] >> (i & 31)) & 1u)) l = l > 0.f ? l / pen : l * pen;
        l *= inv_t;
        return l != l ? -INFINITY : l;
    }
};

// Kept set: key above the threshold, or equal to it with index <= cut.
struct Keep {
    unsigned thr; int cut;
    __device__ __forceinline__ bool has(unsigned key, int i) const { return key > thr || (key == thr && i <= cut); }
};

// Exclusive scan over the block (blockDim.x <= 1024); returns this thread's prefix, total in *total.
__device__ u64 block_exclusive_scan(u64 v, u64* smem /* 33 */, u64* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    u64 inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) smem[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        u64 w = lane < nwarp ? smem[lane] : 0, winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const u64 n = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += n;
        }
        smem[lane] = winc - w;
        if (lane == 31) smem[32] = winc;
    }
    __syncthreads();
    *total = smem[32];
    return smem[warp] + inc - v;
}

#define SAMPLE_THREADS 1024
#define FIX_ONE 1099511627776.0f     // 2^40

struct Shared {
    u64 hist[256];
    u64 scan[33];
    u64 bcast[4];
    float fred[33];
    int ired[33];
    int result;
};

// Largest key ``thr`` such that the weight of {key >= thr} reaches ``target``; ``above`` = weight of
// {key > thr}, ``ties`` = weight of {key == thr}.  weight(i, key, x) is 0 for tokens outside the set.
template <typename WFn>
__device__ void radix_select(const Row& r, WFn weight, u64 target, Shared& sh, unsigned& thr, u64& above, u64& ties) {
    unsigned prefix = 0, mask = 0;
    u64 acc_above = 0, sel = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int b = threadIdx.x; b < 256; b += blockDim.x) sh.hist[b] = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < r.V; i += blockDim.x) {
            const float x = r.value(i);
            const unsigned key = order_key(x);
            if ((key & mask) != prefix) continue;
            const u64 w = weight(i, key, x);
            if (w) atomicAdd(&sh.hist[(key >> shift) & 255u], w);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            u64 a = acc_above;
            int b = 255;
            for (; b > 0; --b) {
                if (a + sh.hist[b] >= target) break;
                a += sh.hist[b];
            }
            sh.bcast[0] = a; sh.bcast[1] = (u64)b; sh.bcast[2] = sh.hist[b];
        }
        __syncthreads();
        acc_above = sh.bcast[0];
        prefix |= (unsigned)sh.bcast[1] << shift;
        mask |= 255u << shift;
        sel = sh.bcast[2];
        __syncthreads();
    }
    thr = prefix; above = acc_above; ties = sel;
}

// Index of the ``need``-th (1-based) token in vocabulary order for which pred(i) holds.
template <typename PFn>
__device__ int nth_in_order(int V, PFn pred, u64 need, Shared& sh) {
    const int per = (V + blockDim.x - 1) / blockDim.x;
    const int lo = min(V, (int)threadIdx.x * per), hi = min(V, lo + per);
    u64 cnt = 0;
    for (int i = lo; i < hi; ++i) cnt += pred(i) ? 1 : 0;
    u64 total;
    const u64 before = block_exclusive_scan(cnt, sh.scan, &total);
    if (threadIdx.x == 0) sh.result = INT_MAX;
    __syncthreads();
    if (cnt && before < need && need <= before + cnt) {
        u64 seen = before;
        for (int i = lo; i < hi; ++i)
            if (pred(i) && ++seen == need) { sh.result = i; break; }
    }
    __syncthreads();
    return sh.result;
}

// (value, index) pairs: the larger value wins, the lower index among equals; INT_MAX marks "none yet".
__device__ __forceinline__ bool better(float ob, int oi, float best, int best_i) {
    return oi != INT_MAX && (best_i == INT_MAX || ob > best || (ob == best && oi < best_i));
}

// Maximum of value(i) over [lo, hi) and its lowest index, per thread (eight loads in flight).
__device__ __forceinline__ void scan_max(const Row& r, int lo, int hi, int tid, int nthreads, float& best, int& best_i) {
    for (int i0 = lo + tid; i0 < hi; i0 += 8 * nthreads) {
        float xs[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * nthreads;
            xs[u] = i < hi ? r.value(i) : -INFINITY;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * nthreads;
            if (i < hi && (best_i == INT_MAX || xs[u] > best)) { best = xs[u]; best_i = i; }
        }
    }
}

__device__ __forceinline__ Row row_of(const SampleArgs& a, int row, int slot, bool greedy, float temperature) {
    Row r;
    r.logits = a.logits + (size_t)row * a.ld;
    r.seen = a.seen ? a.seen + (size_t)slot * a.seen_words : nullptr;
    r.pen = a.penalty[slot];
    r.inv_t = greedy ? 1.0f : 1.0f / temperature;
    r.V = a.V;
    return r;
}

// Block (row, part): the maximum of the part's slice of the row, for sample_kernel to finish.
#define MAX_THREADS 256
__global__ void __launch_bounds__(MAX_THREADS) sample_max_kernel(SampleArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float fred[MAX_THREADS / 32];
    __shared__ int ired[MAX_THREADS / 32];
    const int row = blockIdx.x, part = blockIdx.y, slot = a.slot_of_row[row], tid = threadIdx.x;
    const float temperature = a.temperature[slot];
    const Row r = row_of(a, row, slot, temperature <= 1e-4f, temperature);
    const int per = (a.V + a.parts - 1) / a.parts;
    const int lo = min(a.V, part * per), hi = min(a.V, lo + per);
    float best = -INFINITY; int best_i = INT_MAX;
    scan_max(r, lo, hi, tid, blockDim.x, best, best_i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (better(ob, oi, best, best_i)) { best = ob; best_i = oi; }
    }
    if ((tid & 31) == 0) { fred[tid >> 5] = best; ired[tid >> 5] = best_i; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < MAX_THREADS / 32; ++w)
            if (better(fred[w], ired[w], best, best_i)) { best = fred[w]; best_i = ired[w]; }
        a.part_best[(size_t)row * a.parts + part] = best;
        a.part_idx[(size_t)row * a.parts + part] = best_i;
    }
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(SampleArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ Shared sh;
    const int row = blockIdx.x, slot = a.slot_of_row[row], V = a.V, tid = threadIdx.x;
    const float temperature = a.temperature[slot];
    const bool greedy = temperature <= 1e-4f;
    const Row r = row_of(a, row, slot, greedy, temperature);

    // ---- maximum and its lowest index (this is the answer when greedy): from the parts that
    // sample_max_kernel left, or by scanning the row here
    float best = -INFINITY; int best_i = INT_MAX;
    if (a.parts > 0) {
        for (int p = tid; p < a.parts; p += blockDim.x) {
            const float ob = a.part_best[(size_t)row * a.parts + p];
            const int oi = a.part_idx[(size_t)row * a.parts + p];
            if (better(ob, oi, best, best_i)) { best = ob; best_i = oi; }
        }
    } else {
        scan_max(r, 0, V, tid, blockDim.x, best, best_i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (better(ob, oi, best, best_i)) { best = ob; best_i = oi; }
    }
    if ((tid & 31) == 0) { sh.fred[tid >> 5] = best; sh.ired[tid >> 5] = best_i; }
    __syncthreads();
    if (tid < 32) {
        const int nwarp = (blockDim.x + 31) >> 5;
        best = tid < nwarp ? sh.fred[tid] : -INFINITY;
        best_i = tid < nwarp ? sh.ired[tid] : INT_MAX;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (better(ob, oi, best, best_i)) { best = ob; best_i = oi; }
        }
        if (tid == 0) { sh.fred[32] = best; sh.ired[32] = best_i; }
    }
    __syncthreads();
    const float x_max = sh.fred[32];
    int token = sh.ired[32];
    if (token == INT_MAX) token = 0;

    if (!greedy) {
        Keep k1; k1.thr = 0u; k1.cut = INT_MAX;                       // after top_k
        const int top_k = a.top_k[slot];
        if (top_k > 0 && top_k < V) {
            unsigned thr; u64 above, ties;
            radix_select(r, [](int, unsigned, float) -> u64 { return 1; }, (u64)top_k, sh, thr, above, ties);
            k1.thr = thr;
            const u64 need = (u64)top_k - above;
            if (need < ties)
                k1.cut = nth_in_order(V, [&](int i) { return order_key(r.value(i)) == thr; }, need, sh);
        }
        auto mass = [&](int i, unsigned key, float x) -> u64 {
            return k1.has(key, i) ? __float2ull_rd(expf(x - x_max) * FIX_ONE) : 0ull;
        };
        Keep k2 = k1;                                                  // after top_p
        const float top_p = a.top_p[slot];
        if (top_p < 1.0f) {
            u64 part = 0, total;
            for (int i = tid; i < V; i += blockDim.x) { const float x = r.value(i); part += mass(i, order_key(x), x); }
            block_exclusive_scan(part, sh.scan, &total);
            u64 target = (u64)ceil((double)top_p * (double)total);
            target = target < 1 ? 1 : (target > total ? total : target);
            unsigned thr; u64 above, ties;
            radix_select(r, mass, target, sh, thr, above, ties);
            if (total > 0) {
                // every tie has the same mass q; keep the first ceil((target - above) / q) of them
                const float xt = [&]() { unsigned u = (thr & 0x80000000u) ? (thr & 0x7fffffffu) : ~thr; return __uint_as_float(u); }();
                const u64 q = __float2ull_rd(expf(xt - x_max) * FIX_ONE);
                const u64 n_ties = q ? ties / q : 0;
                const u64 need = q ? (target - above + q - 1) / q : 0;
                k2.thr = thr;
                k2.cut = k1.cut;
                if (q && need < n_ties)
                    k2.cut = nth_in_order(V, [&](int i) { const unsigned key = order_key(r.value(i)); return key == thr && k1.has(key, i); }, need, sh);
            }
        }
        // ---- draw in vocabulary order
        auto kept_mass = [&](int i) -> u64 {
            const float x = r.value(i);
            const unsigned key = order_key(x);
            return (k1.has(key, i) && k2.has(key, i)) ? __float2ull_rd(expf(x - x_max) * FIX_ONE) : 0ull;
        };
        const int per = (V + blockDim.x - 1) / blockDim.x;
        const int lo = min(V, tid * per), hi = min(V, lo + per);
        u64 part = 0, total;
        for (int i = lo; i < hi; ++i) part += kept_mass(i);
        const u64 before = block_exclusive_scan(part, sh.scan, &total);
        const unsigned u24 = uniform24((u64)a.seed[slot], (u64)a.sequence_id[slot], (u64)a.sample_step[slot]);
        // target in [0, total): floor(u * total) with u = u24 / 2^24, from the 128-bit product
        const u64 target = (__umul64hi(total, (u64)u24) << 40) | ((total * (u64)u24) >> 24);
        if (tid == 0) sh.result = token;
        __syncthreads();
        if (total > 0 && part && before <= target && target < before + part) {
            u64 run = before;
            for (int i = lo; i < hi; ++i) {
                run += kept_mass(i);
                if (run > target) { sh.result = i; break; }
            }
        }
        __syncthreads();
        token = sh.result;
    }
    if (tid == 0) {
        a.out[row] = token;
        a.last_token[slot] = token;
        a.sample_step[slot] += 1;
        if (r.seen) atomicOr(a.seen + (size_t)slot * a.seen_words + (token >> 5), 1u << (token & 31));
    }
}

extern "C" int tb_sample(const SampleArgs* args, cudaStream_t stream) {
    SampleArgs a = *args;
    TB_REQUIRE(a.B > 0 && a.V > 0 && a.ld >= a.V, "sample: bad sizes (B=%d V=%d ld=%d)", a.B, a.V, a.ld);
    TB_REQUIRE(!a.seen || a.seen_words * 32 >= a.V, "sample: the seen-bitmap is shorter than the vocabulary");
    TB_REQUIRE(a.parts >= 0 && (a.parts == 0 || (a.part_best && a.part_idx)), "sample: parts without their scratch");
    if (a.parts > 0) tb_launch(sample_max_kernel, dim3(a.B, a.parts), MAX_THREADS, 0, stream, a);
    tb_launch(sample_kernel, a.B, SAMPLE_THREADS, 0, stream, a);
    TB_CHECK_LAUNCH("sample");
    return 0;
}

// Marks the tokens of a step as seen (context of the repetition penalty).
__global__ void mark_seen_kernel(const int* tokens, const int* seq_of, const int* slot_of_seq, unsigned* seen,
                                 int seen_words, int T) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const int tok = tokens[t];
    if (tok >= 0 && tok < seen_words * 32)
        atomicOr(seen + (size_t)slot_of_seq[seq_of[t]] * seen_words + (tok >> 5), 1u << (tok & 31));
}

extern "C" int tb_mark_seen(const int* tokens, const int* seq_of, const int* slot_of_seq, unsigned* seen,
                            int seen_words, int T, cudaStream_t stream) {
    TB_REQUIRE(T > 0 && seen, "mark_seen: nothing to mark");
    tb_launch(mark_seen_kernel, (T + 255) / 256, 256, 0, stream, tokens, seq_of, slot_of_seq, seen, seen_words, T);
    TB_CHECK_LAUNCH("mark_seen");
    return 0;
}

// Host copy of the device's uniform number, for tests and for the plain sampler's parity.
extern "C" unsigned tb_uniform24(long long seed, long long sequence, long long step) {
    return uniform24((u64)seed, (u64)sequence, (u64)step);
}
