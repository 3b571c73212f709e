// Token sampling on the device.  Several blocks per row find the maximum and its lowest index (the
// answer when greedy).  A row that is not greedy is then shared by a team of CTAs (a thread-block cluster of
// up to 8; one CTA for small vocabularies), each on a contiguous slice of the vocabulary: top_k and top_p
// thresholds by radix selection (three passes of 12, 12 and 8 key bits; bins summed over the team through
// distributed shared memory), the kept tokens of a top_k up to 1,024 gathered into a list that one CTA
// finishes on, the draw by an ordered search that narrows slice, warp run, position.  At a vocabulary of
// 151,936 a decode step pays 20 to 70 us for a sampled row instead of 10 us for a greedy one.
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

__device__ __forceinline__ unsigned order_key(float x) {      // larger float -> larger key; NaN -> 0; -0 and +0 share a key
    if (x != x) return 0u;
    const unsigned u = x == 0.f ? 0u : __float_as_uint(x);
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
    __device__ __forceinline__ float value(int i) const { return adjust(i, logits[i]); }
    __device__ __forceinline__ float adjust(int i, float l) const {
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
#define DIGIT_BINS 4096              // a selection pass sorts by 12 bits of the key (12 + 12 + 8)
#define LIST_MAX 1024                // top_k up to this many: the kept tokens are gathered, later passes walk the list
#define TEAM_MAX 8                   // CTAs that share a row (a thread-block cluster)

struct Shared {
    unsigned hist_lo[DIGIT_BINS], hist_hi[DIGIT_BINS];     // this CTA's bins: a 64-bit sum per bin as two words (see bin_add)
    unsigned all_lo[DIGIT_BINS], all_hi[DIGIT_BINS];       // the team's bins
    u64 scan[33];
    u64 bcast[4];
    u64 team_sum;
    float fred[33];
    int ired[33];
    int result;
    int count;
    int team_found;
    int list_idx[LIST_MAX];
    float list_x[LIST_MAX];
};

// The CTAs that work on one row: the CTAs of a thread-block cluster (each takes a contiguous slice of the
// vocabulary, in rank order), or one CTA alone.  Every CTA of a team runs the same sequence of sync() calls:
// what decides a branch around one is either a sampling parameter of the row or a value that all CTAs
// computed from the same team-wide sums.
struct Team {
    int size, rank;
    __device__ __forceinline__ void sync() const {
        if (size > 1) asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        else __syncthreads();
    }
};
// The word at the same place of CTA r's shared memory.
__device__ __forceinline__ unsigned peer_u32(const void* mine, int r) {
    unsigned addr, v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"((unsigned)__cvta_generic_to_shared(mine)), "r"(r));
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ u64 peer_u64(const void* mine, int r) {
    unsigned addr; u64 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"((unsigned)__cvta_generic_to_shared(mine)), "r"(r));
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(addr) : "memory");
    return v;
}

// Adds to a bin's 64-bit sum with 32-bit shared-memory atomics (the hardware has those; a 64-bit add in
// shared memory is a compare-and-swap loop): the low word wraps and its carry goes to the high word.
__device__ __forceinline__ void bin_add(Shared& sh, int b, u64 w) {
    const unsigned lo = (unsigned)w, hi = (unsigned)(w >> 32);
    const unsigned old = atomicAdd(&sh.hist_lo[b], lo);
    const unsigned carry = (old + lo < old) ? 1u : 0u;
    if (hi + carry) atomicAdd(&sh.hist_hi[b], hi + carry);
}

// What a pass walks: a slice [lo, hi) of the row (values made on the fly; lo is a multiple of 4), or the
// tokens that top_k kept.  A position j of the source is the token index(j).
struct RowSlice {
    Row r; int lo, hi;
    __device__ __forceinline__ int size() const { return hi - lo; }
    __device__ __forceinline__ int index(int j) const { return lo + j; }
    __device__ __forceinline__ float value(int j) const { return r.value(lo + j); }
};
struct KeptList {                    // in vocabulary order
    const int* idx; const float* x; int n;
    __device__ __forceinline__ int size() const { return n; }
    __device__ __forceinline__ int index(int j) const { return idx[j]; }
    __device__ __forceinline__ float value(int j) const { return x[j]; }
};

// Calls body(j, value(j)) for every position of the source, eight loads in flight per thread.
template <typename Src, typename Body>
__device__ __forceinline__ void for_each(const Src& src, Body body) {
    const int n = src.size(), step = blockDim.x;
    for (int j0 = threadIdx.x; j0 < n; j0 += 8 * step) {
        float xs[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = j0 + u * step;
            xs[u] = j < n ? src.value(j) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = j0 + u * step;
            if (j < n) body(j, xs[u]);
        }
    }
}
// The same over a slice of a row, with 16-byte loads where the row starts on a 16-byte boundary.
template <typename Body>
__device__ __forceinline__ void for_each(const RowSlice& src, Body body) {
    const Row& r = src.r;
    const int step = blockDim.x, n = src.size();
    int done = 0;
    if ((((size_t)r.logits) & 15) == 0) {
        const int n4 = n >> 2;
        const float4* p = reinterpret_cast<const float4*>(r.logits + src.lo);
        for (int q0 = threadIdx.x; q0 < n4; q0 += 4 * step) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int q = q0 + u * step;
                v[u] = q < n4 ? p[q] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int q = q0 + u * step, j = 4 * q, i = src.lo + j;
                if (q < n4) {
                    body(j, r.adjust(i, v[u].x)); body(j + 1, r.adjust(i + 1, v[u].y));
                    body(j + 2, r.adjust(i + 2, v[u].z)); body(j + 3, r.adjust(i + 3, v[u].w));
                }
            }
        }
        done = n4 << 2;
    }
    for (int j = done + threadIdx.x; j < n; j += step) body(j, src.value(j));
}

// Largest key ``thr`` such that the team-wide weight of {key >= thr} reaches the target; ``above`` =
// weight of {key > thr}, ``ties`` = weight of {key == thr}.  weight(i, key, x) is 0 for tokens outside the
// set.  The target is target_of(total weight), known after the first pass.  Three passes over the source
// (12, 12 and 8 bits of the key); each CTA fills its own bins, a team then sums them through distributed
// shared memory (every CTA gets every sum), and the bin that holds the target is found by all threads.
template <bool COUNT, typename Src, typename WFn, typename TFn>
__device__ void radix_select(const Team& team, const Src& src, WFn weight, TFn target_of, Shared& sh, unsigned& thr,
                             u64& above, u64& ties, u64& total, u64& target) {
    unsigned prefix = 0, mask = 0;
    u64 acc_above = 0, sel = 0;
    total = 0; target = 0;
    for (int pass = 0; pass < 3; ++pass) {
        const int shift = pass == 0 ? 20 : (pass == 1 ? 8 : 0);
        const int bins = pass == 2 ? 256 : DIGIT_BINS;
        for (int b = threadIdx.x; b < bins; b += blockDim.x) { sh.hist_lo[b] = 0; sh.hist_hi[b] = 0; }
        __syncthreads();
        for_each(src, [&](int j, float x) {
            const unsigned key = order_key(x);
            if ((key & mask) != prefix) return;
            const u64 w = weight(src.index(j), key, x);
            const int b = (int)((key >> shift) & (unsigned)(bins - 1));
            if (COUNT) { if (w) atomicAdd(&sh.hist_lo[b], (unsigned)w); }      // weights of 0 or 1: no carry, no answer awaited
            else if (w) bin_add(sh, b, w);
        });
        __syncthreads();
        const unsigned* lo_w = sh.hist_lo;
        const unsigned* hi_w = sh.hist_hi;
        if (team.size > 1) {
            team.sync();                                   // every CTA's bins are complete
            for (int b = threadIdx.x; b < bins; b += blockDim.x) {
                u64 sum = 0;
                for (int r = 0; r < team.size; ++r)
                    sum += COUNT ? (u64)peer_u32(&sh.hist_lo[b], r)
                                 : (((u64)peer_u32(&sh.hist_hi[b], r) << 32) + peer_u32(&sh.hist_lo[b], r));
                sh.all_lo[b] = (unsigned)sum; sh.all_hi[b] = (unsigned)(sum >> 32);
            }
            team.sync();                                   // and have been read by every CTA
            lo_w = sh.all_lo; hi_w = sh.all_hi;
        }
        auto sum_of = [&](int b) -> u64 { return ((u64)hi_w[b] << 32) + lo_w[b]; };
        // bins in descending order, a run of them per thread
        const int per = (bins + blockDim.x - 1) / blockDim.x;
        const int lo = min(bins, (int)threadIdx.x * per), hi = min(bins, lo + per);
        u64 mine = 0;
        for (int rb = lo; rb < hi; ++rb) mine += sum_of(bins - 1 - rb);
        u64 all;
        const u64 before = block_exclusive_scan(mine, sh.scan, &all);
        if (pass == 0) { total = all; target = target_of(all); }
        if (threadIdx.x == 0) {         // no bin reaches the target: the lowest bin, as a walk from the top ends
            sh.bcast[0] = acc_above + all - sum_of(0); sh.bcast[1] = 0; sh.bcast[2] = sum_of(0);
        }
        __syncthreads();
        u64 a = acc_above + before;
        for (int rb = lo; rb < hi; ++rb) {
            const int b = bins - 1 - rb;
            const u64 h = sum_of(b);
            if (b > 0 && a < target && a + h >= target) { sh.bcast[0] = a; sh.bcast[1] = (u64)b; sh.bcast[2] = h; }
            a += h;
        }
        __syncthreads();
        acc_above = sh.bcast[0];
        prefix |= (unsigned)sh.bcast[1] << shift;
        mask |= (unsigned)(bins - 1) << shift;
        sel = sh.bcast[2];
        __syncthreads();
    }
    thr = prefix; above = acc_above; ties = sel;
}

// Position j of the source, in its order, at which the running sum of f first exceeds the target
// (INT_MAX if it never does), by this CTA alone.  The target is target_of(sum of f over the source).
// The source is cut into one run per warp, the run that holds the target into runs again, until a
// thread holds one position: every level reads coalesced, and all levels together read little more
// than the source once.
template <typename Src, typename F, typename TFn>
__device__ int locate_here(const Src& src, F f, TFn target_of, Shared& sh, u64& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    int lo = 0, hi = src.size();
    u64 target = 0;
    bool have = false;
    while (hi - lo > (int)blockDim.x) {
        const int per = (((hi - lo + nwarp - 1) / nwarp) + 31) & ~31;
        const int clo = min(hi, lo + warp * per), chi = min(hi, clo + per);
        u64 s = 0;
        for (int j0 = clo + lane; j0 < chi; j0 += 128) {
            float xs[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) xs[u] = j0 + 32 * u < chi ? src.value(j0 + 32 * u) : 0.f;
#pragma unroll
            for (int u = 0; u < 4; ++u) if (j0 + 32 * u < chi) s += f(j0 + 32 * u, xs[u]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        __syncthreads();
        if (lane == 0) sh.scan[warp] = s;
        __syncthreads();
        if (!have) {
            u64 all = 0;
            for (int w = 0; w < nwarp; ++w) all += sh.scan[w];
            total = all; target = target_of(all); have = true;
        }
        u64 a = 0;
        int c = -1;
        for (int w = 0; w < nwarp; ++w) {
            const u64 sw = sh.scan[w];
            if (c < 0) { if (a + sw > target) c = w; else a += sw; }
        }
        __syncthreads();
        if (c < 0) return INT_MAX;
        target -= a;
        lo = min(hi, lo + c * per);
        hi = min(hi, lo + per);
    }
    const int j = lo + (int)threadIdx.x;
    const u64 v = j < hi ? f(j, src.value(j)) : 0ull;
    u64 all;
    const u64 before = block_exclusive_scan(v, sh.scan, &all);
    if (!have) { total = all; target = target_of(all); }
    if (threadIdx.x == 0) sh.result = INT_MAX;
    __syncthreads();
    if (v && before <= target && target < before + v) sh.result = j;
    __syncthreads();
    const int found = sh.result;
    __syncthreads();
    return found;
}

// The token, in vocabulary order over the whole team's sources, at which the running sum of f first
// exceeds target_of(team-wide sum of f); INT_MAX if none.  A team first sums each CTA's slice, every CTA
// reads all the sums, and the CTA whose slice holds the target searches it.
template <typename Src, typename F, typename TFn>
__device__ int locate(const Team& team, const Src& src, F f, TFn target_of, Shared& sh, u64& total) {
    if (team.size == 1) {
        const int j = locate_here(src, f, target_of, sh, total);
        return j == INT_MAX ? INT_MAX : src.index(j);
    }
    u64 s = 0;
    for_each(src, [&](int j, float x) { s += f(j, x); });
    u64 mine;
    block_exclusive_scan(s, sh.scan, &mine);
    if (threadIdx.x == 0) sh.team_sum = mine;
    team.sync();
    u64 sums[TEAM_MAX], all = 0;
#pragma unroll
    for (int r = 0; r < TEAM_MAX; ++r) { sums[r] = r < team.size ? peer_u64(&sh.team_sum, r) : 0ull; all += sums[r]; }
    total = all;
    const u64 target = target_of(all);
    u64 a = 0;
    int c = -1;
#pragma unroll
    for (int r = 0; r < TEAM_MAX; ++r)
        if (r < team.size && c < 0) { if (a + sums[r] > target) c = r; else a += sums[r]; }
    if (team.rank == c) {
        u64 unused;
        const int j = locate_here(src, f, [&](u64) -> u64 { return target - a; }, sh, unused);
        if (threadIdx.x == 0) sh.team_found = j == INT_MAX ? INT_MAX : src.index(j);
    }
    team.sync();
    const int found = c < 0 ? INT_MAX : (int)peer_u32(&sh.team_found, c);
    team.sync();                                           // before team_sum and team_found are written again
    return found;
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

// top_p over the tokens that ``k1`` keeps, then the draw in vocabulary order; INT_MAX if nothing has mass.
template <typename Src>
__device__ int top_p_and_draw(const Team& team, const Src& src, Keep k1, float x_max, float top_p, unsigned u24, Shared& sh) {
    auto mass = [&](int i, unsigned key, float x) -> u64 {
        return k1.has(key, i) ? __float2ull_rd(expf(x - x_max) * FIX_ONE) : 0ull;
    };
    Keep k2 = k1;                                                  // after top_p
    if (top_p < 1.0f) {
        unsigned thr; u64 above, ties, total, target;
        radix_select<false>(team, src, mass, [&](u64 all) -> u64 {
            const u64 t = (u64)ceil((double)top_p * (double)all);
            return t < 1 ? (all < 1 ? all : 1) : (t > all ? all : t);
        }, sh, thr, above, ties, total, target);
        if (total > 0) {
            // every tie has the same mass q; keep the first ceil((target - above) / q) of them
            const unsigned bits = (thr & 0x80000000u) ? (thr & 0x7fffffffu) : ~thr;
            const u64 q = __float2ull_rd(expf(__uint_as_float(bits) - x_max) * FIX_ONE);
            const u64 n_ties = q ? ties / q : 0;
            const u64 need = q ? (target - above + q - 1) / q : 0;
            k2.thr = thr;
            k2.cut = INT_MAX;              // (k1 still applies beside k2: its cut is about ties at ITS threshold)
            if (q && need < n_ties) {
                u64 counted;
                k2.cut = locate(team, src, [&](int j, float x) -> u64 {
                    const unsigned key = order_key(x);
                    return (key == thr && k1.has(key, src.index(j))) ? 1 : 0;
                }, [&](u64) -> u64 { return need - 1; }, sh, counted);
            }
        }
    }
    // the draw: the first token, in vocabulary order, at which the running kept mass exceeds
    // floor(u * total), u = u24 / 2^24 (from the 128-bit product)
    u64 total;
    return locate(team, src, [&](int j, float x) -> u64 {
        const unsigned key = order_key(x);
        const int i = src.index(j);
        return (k1.has(key, i) && k2.has(key, i)) ? __float2ull_rd(expf(x - x_max) * FIX_ONE) : 0ull;
    }, [&](u64 all) -> u64 { return (__umul64hi(all, (u64)u24) << 40) | ((all * (u64)u24) >> 24); }, sh, total);
}

// Grid (rows, 1, team): the CTAs of a row are a thread-block cluster (1, 1, team).
__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(SampleArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char sample_shared[];
    Shared& sh = *reinterpret_cast<Shared*>(sample_shared);
    const Team team{(int)gridDim.z, (int)blockIdx.z};
    const int row = blockIdx.x, slot = a.slot_of_row[row], V = a.V, tid = threadIdx.x;
    const float temperature = a.temperature[slot];
    const bool greedy = temperature <= 1e-4f;
    const Row r = row_of(a, row, slot, greedy, temperature);

    // ---- maximum and its lowest index (this is the answer when greedy): from the parts that
    // sample_max_kernel left, or by scanning the row here (every CTA of a team finds the same)
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
        const int top_k = a.top_k[slot];
        const float top_p = a.top_p[slot];
        const unsigned u24 = uniform24((u64)a.seed[slot], (u64)a.sequence_id[slot], (u64)a.sample_step[slot]);
        const int per = (((V + team.size - 1) / team.size) + 3) & ~3;
        RowSlice mine; mine.r = r; mine.lo = min(V, team.rank * per); mine.hi = min(V, mine.lo + per);
        Keep k1; k1.thr = 0u; k1.cut = INT_MAX;                       // after top_k
        if (top_k > 0 && top_k < V) {
            unsigned thr; u64 above, ties, total, target;
            radix_select<true>(team, mine, [](int, unsigned, float) -> u64 { return 1; },
                               [&](u64) -> u64 { return (u64)top_k; }, sh, thr, above, ties, total, target);
            k1.thr = thr;
            const u64 need = (u64)top_k - above;
            if (need < ties) {
                u64 n_ties;
                k1.cut = locate(team, mine, [&](int, float x) -> u64 { return order_key(x) == thr ? 1 : 0; },
                                [&](u64) -> u64 { return need - 1; }, sh, n_ties);
            }
        }
        int drawn;
        if (top_k > 0 && top_k < V && top_k <= LIST_MAX) {
            // gather the kept tokens of this slice, put them in vocabulary order (a token's place is the
            // number of kept tokens with a lower index); the team's first CTA then appends the other
            // slices' lists in rank order and finishes on the list alone
            if (tid == 0) sh.count = 0;
            __syncthreads();
            for_each(mine, [&](int j, float x) {
                const int i = mine.index(j);
                if (k1.has(order_key(x), i)) {
                    const int at = atomicAdd(&sh.count, 1);
                    if (at < LIST_MAX) { sh.list_idx[at] = i; sh.list_x[at] = x; }
                }
            });
            __syncthreads();
            int n = min(sh.count, LIST_MAX);
            const int my_i = tid < n ? sh.list_idx[tid] : INT_MAX;
            const float my_x = tid < n ? sh.list_x[tid] : 0.f;
            int place = 0;
            for (int u = 0; u < n; ++u) place += sh.list_idx[u] < my_i ? 1 : 0;
            __syncthreads();
            if (tid < n) { sh.list_idx[place] = my_i; sh.list_x[place] = my_x; }
            __syncthreads();
            if (team.size > 1) {
                team.sync();                                       // every slice's list is in place
                if (team.rank == 0) {
                    for (int rk = 1; rk < team.size; ++rk) {
                        const int theirs = min((int)peer_u32(&sh.count, rk), LIST_MAX);
                        for (int u = tid; u < theirs && n + u < LIST_MAX; u += blockDim.x) {
                            sh.list_idx[n + u] = (int)peer_u32(&sh.list_idx[u], rk);
                            sh.list_x[n + u] = __uint_as_float(peer_u32(&sh.list_x[u], rk));
                        }
                        n = min(LIST_MAX, n + theirs);
                    }
                    __syncthreads();
                }
                team.sync();                                       // the lists have been read: the others may leave
                if (team.rank != 0) return;
            }
            Keep all; all.thr = 0u; all.cut = INT_MAX;
            drawn = top_p_and_draw(Team{1, 0}, KeptList{sh.list_idx, sh.list_x, n}, all, x_max, top_p, u24, sh);
        } else {
            drawn = top_p_and_draw(team, mine, k1, x_max, top_p, u24, sh);
        }
        if (drawn != INT_MAX) token = drawn;
    }
    if (team.rank == 0 && tid == 0) {
        a.out[row] = token;
        a.last_token[slot] = token;
        a.sample_step[slot] += 1;
        if (r.seen) atomicOr(a.seen + (size_t)slot * a.seen_words + (token >> 5), 1u << (token & 31));
    }
}

// CTAs per row for rows that are not greedy: 0 = by the size of the vocabulary, else 1, 2, 4 or 8.
static int g_sample_team = 0;
extern "C" void tb_sample_set_team(int team) { g_sample_team = team; }

extern "C" int tb_sample(const SampleArgs* args, cudaStream_t stream) {
    SampleArgs a = *args;
    TB_REQUIRE(a.B > 0 && a.V > 0 && a.ld >= a.V, "sample: bad sizes (B=%d V=%d ld=%d)", a.B, a.V, a.ld);
    TB_REQUIRE(!a.seen || a.seen_words * 32 >= a.V, "sample: the seen-bitmap is shorter than the vocabulary");
    TB_REQUIRE(a.parts >= 0 && (a.parts == 0 || (a.part_best && a.part_idx)), "sample: parts without their scratch");
    // by default a slice of at least 8,192 tokens per CTA, and about as many CTAs as the device runs at once
    int team = g_sample_team;
    if (!team) {
        team = a.V >= 65536 ? 8 : (a.V >= 16384 ? 4 : 1);
        static int sm_count = 0;
        if (!sm_count) {
            int dev = 0;
            cudaGetDevice(&dev);
            if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
        }
        while (team > 1 && a.B * team > 2 * sm_count) team >>= 1;
    }
    TB_REQUIRE(team == 1 || team == 2 || team == 4 || team == 8, "sample: a team of %d CTAs (1, 2, 4 or 8)", team);
    static bool prepared = false;
    if (!prepared) {
        TB_REQUIRE(cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Shared)) == cudaSuccess,
                   "sample: %d bytes of shared memory refused", (int)sizeof(Shared));
        prepared = true;
    }
    if (a.parts > 0) tb_launch(sample_max_kernel, dim3(a.B, a.parts), MAX_THREADS, 0, stream, a);
    tb_launch_cluster_z(sample_kernel, dim3(a.B, 1, team), SAMPLE_THREADS, sizeof(Shared), stream, team, a);
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
