// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05) of sm_100a:
//     out = epilogue(X[M,K] . W[N,K]^T),  float32 accumulation in tensor memory.
//
// Tiles of D = A . B^T are 128 x BN, A and B both K-major:
//   plain mode  A = X (rows = tokens), B = W (rows = outputs):  D[m][n]     (prompts, M >= 128)
//   swap mode   A = W,                 B = X:                   D[n][m]     (decode: a few tokens)
// so that in decode the 128-row side of the instruction is filled by weight rows and the batch is the
// narrow side (BN = 16..128).
//
// Plain mode is persistent.  From 129 rows and 256 columns on it runs on PAIRS of CTAs (gemm_tc_pair_kernel, a
// cluster of two, tcgen05.mma.cta_group::2 with M = 256: see the comment above that kernel); smaller
// outputs run on single CTAs (gemm_tc_persistent_kernel: one CTA per SM walks over 128 x 256 tiles).
// In both the accumulator is double buffered in tensor memory, so the epilogue of a tile overlaps the
// MMAs of the next, and the tiles of a last, partly filled round can be cut along K for the ADD
// epilogue (struct Segments).  Swap mode (gemm_tc_kernel) is one tile per CTA with two CTAs per SM (the
// ring is six to three stages deep, by the tile's width); it
// can cut K into slices (grid.z), each CTA adding its partial sum into a float32 output with atomics, to
// fill the machine once when N / 128 is small; its weights are loaded with the L2 evict-first hint.
//
// Data path: TMA (cp.async.bulk.tensor.2d, 128-byte swizzle, zero fill outside the tensor) into a
// ring of shared-memory stages -> tcgen05.mma.kind::f16 issued by one thread, four K=16 steps per
// 64-wide stage -> accumulator in TMEM -> tcgen05.ld by four epilogue warps.
// Warp 0 produces, warp 1 allocates TMEM and issues MMAs, warps 2..5 run the epilogue.
// No TMA multicast anywhere.  Kernels are launched with programmatic dependent launch: the
// producer requests the first ring of WEIGHT tiles before it waits for the kernel before (no kernel
// writes weights), so a decode step's weight stream does not stop between kernels.
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT polls the thread records an error code
// in a device word (read with tb_gemm_tc_error) and goes on, so the kernel always ends and frees
// its tensor memory; the result is then invalid and the host says so.
//
// berniehans/titan's counterpart is gemm_q4k_batched_kernel (engine/engine-cuda/kernels/
// gemm_quant.cu:3365-3499), a scalar-FMA warp-per-column kernel with the residual in its
// epilogue (:3489-3493); it has no tensor-core path.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "gemm.h"
#include "tcgen05.cuh"
#include "timeline.cuh"
#include "tma.cuh"

namespace {

constexpr int BM = 128;          // rows of A per tile = M of the instruction
constexpr int BK = 64;           // bf16 elements per stage row = 128 bytes = one swizzle span
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;

__device__ unsigned int g_tc_error = 0;

// ---------------------------------------------------------------- PTX wrappers
using tbtma::smem_u32;
using tbtma::mbar_init;
using tbtma::mbar_expect_tx;
using tbtma::tma_load_2d;
using tbtma::tma_load_2d_hint;
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, unsigned code) {
    tbtma::mbar_wait(bar, parity, &g_tc_error, code);
}
using namespace tbtc;

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzled:
// start address >> 4 in bits 0-13, leading byte offset (unused for swizzled K-major) 1 in 16-29,
// stride byte offset 1024 >> 4 (eight rows) in 32-45, version 1 in 46-47, swizzle mode 2 (128 B) in 61-63.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor, kind::f16: D float32 (1 << 4), A and B bfloat16 (1 << 7, 1 << 10), both
// K-major (bits 15, 16 clear), N >> 3 in bits 17-22, M >> 4 in bits 24-28.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// silu(g) * u with the fast exponential and division: the result is rounded to bfloat16 anyway, and the
// epilogue warps run one per scheduler, so every instruction here is on the critical path of a tile.
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&p);
}

struct TcArgs {
    void* out;
    int rows_a;      // valid rows of A (M in plain mode, N in swap mode)
    int rows_b;      // valid rows of B
    int K;
    int ldo;         // row stride of out in elements
    int k_blocks_per_split;
    int atomic;      // ADD epilogue through atomics (several K slices)
    int tiles_m;     // persistent kernel: tiles along A's rows and along B's rows
    int tiles_n;
    int tail_split;  // persistent kernel, ADD epilogue: K parts of the tiles of the last, partly filled round (1: whole)
    // swap mode with the RMS norm of the input folded in (NORMED): the activations are float32 rows xf [rows_b][ldxf]
    // and the norm's weight norm_w [K]; the kernel multiplies by the weight on the way into shared memory and by
    // 1/sqrt(mean(x^2) + eps) in its epilogue, or (K cut into slices: no CTA sees a whole row) leaves its rows'
    // partial sums of squares at sumsq_out [slice][32] for the consumer of the sums to add up, in slice order, and apply
    const float* xf; int ldxf; const float* norm_w; float* sumsq_out; float norm_eps;
};

// TMA ring depth.  Decode tiles (BN <= 64) take as many stages as still let two CTAs share an SM: the
// ring is filled before the wait on the previous kernel, so its depth is what bridges kernel boundaries.
template <int BN> constexpr int stages_for() { return BN >= 256 ? 4 : (BN >= 128 ? 5 : (BN >= 64 ? 4 : (BN >= 32 ? 5 : 6))); }
// Swap mode with 65..128 rows of activations: three stages, so that two CTAs share an SM here too and the
// 192 tiles of the gate-and-up product are resident at once (measured at 96 rows: 59.8 -> 44.0 us).  The
// bfloat16 store (a short prompt's Q|K|V: 48 tiles, no K slices) keeps the deeper ring of one CTA per SM.
template <int BN, int EPI, bool SWAP> constexpr int stages_of() {
    return (SWAP && BN == 128 && EPI != TB_EPI_STORE) ? 3 : stages_for<BN>();
}
template <int BN> constexpr int tmem_cols_for() { return BN < 32 ? 32 : BN; }
constexpr int EPI_TILE_FLOATS = 32 * 33;      // one warp's 32 x 32 transposition tile, padded against bank conflicts
template <int BN, bool SWAP, int STAGES = stages_for<BN>()> constexpr size_t smem_for() {
    return 1024 /*alignment slack*/ + (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + (SWAP ? 1024 : 256) /*barriers; sums of the folded norm*/ +
           (SWAP ? 0 : 4 * EPI_TILE_FLOATS * sizeof(float));
}

// Plain mode: the epilogue of one 32-column chunk held by one thread (row = token m, columns = outputs col0 + j).
template <int EPI, int NV>
__device__ __forceinline__ void epilogue_chunk(const float* v, const TcArgs& a, int row, int col0, int lane) {
    {
        const int m = row;
        if (m >= a.rows_a) return;
        if (EPI == TB_EPI_SWIGLU) {
            __nv_bfloat16* o = (__nv_bfloat16*)a.out + (size_t)m * a.ldo + col0 / 2;
            if (col0 + NV <= a.rows_b && NV == 32) {      // 16 outputs: two 16-byte stores
#pragma unroll
                for (int j = 0; j < NV; j += 16) {
                    uint4 pk;
                    pk.x = pack_bf16(silu_mul(v[j], v[j + 1]), silu_mul(v[j + 2], v[j + 3]));
                    pk.y = pack_bf16(silu_mul(v[j + 4], v[j + 5]), silu_mul(v[j + 6], v[j + 7]));
                    pk.z = pack_bf16(silu_mul(v[j + 8], v[j + 9]), silu_mul(v[j + 10], v[j + 11]));
                    pk.w = pack_bf16(silu_mul(v[j + 12], v[j + 13]), silu_mul(v[j + 14], v[j + 15]));
                    *reinterpret_cast<uint4*>(o + j / 2) = pk;
                }
            } else {
#pragma unroll
                for (int j = 0; j < NV; j += 2)
                    if (col0 + j + 1 < a.rows_b) o[j / 2] = __float2bfloat16_rn(silu_mul(v[j], v[j + 1]));
            }
        } else if (EPI == TB_EPI_STORE) {
            __nv_bfloat16* o = (__nv_bfloat16*)a.out + (size_t)m * a.ldo + col0;
            if (col0 + NV <= a.rows_b) {            // whole chunk inside: 16-byte stores (ldo and col0 are multiples of 8)
#pragma unroll
                for (int j = 0; j < NV; j += 8) {
                    uint4 pk;
                    pk.x = pack_bf16(v[j], v[j + 1]); pk.y = pack_bf16(v[j + 2], v[j + 3]);
                    pk.z = pack_bf16(v[j + 4], v[j + 5]); pk.w = pack_bf16(v[j + 6], v[j + 7]);
                    *reinterpret_cast<uint4*>(o + j) = pk;
                }
            } else {
#pragma unroll
                for (int j = 0; j < NV; ++j)
                    if (col0 + j < a.rows_b) o[j] = __float2bfloat16_rn(v[j]);
            }
        } else {
            float* o = (float*)a.out + (size_t)m * a.ldo + col0;
            if (col0 + NV <= a.rows_b && !a.atomic && (a.ldo & 3) == 0) {
                float4 old[NV / 4];
                if (EPI == TB_EPI_ADD) {            // all loads first: they are independent of the stores below
#pragma unroll
                    for (int j = 0; j < NV; j += 4) old[j / 4] = *reinterpret_cast<const float4*>(o + j);
                }
#pragma unroll
                for (int j = 0; j < NV; j += 4) {
                    float4 r = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    if (EPI == TB_EPI_ADD) { r.x += old[j / 4].x; r.y += old[j / 4].y; r.z += old[j / 4].z; r.w += old[j / 4].w; }
                    *reinterpret_cast<float4*>(o + j) = r;
                }
            } else {
#pragma unroll
                for (int j = 0; j < NV; ++j) {
                    if (col0 + j >= a.rows_b) continue;
                    if (EPI == TB_EPI_F32) o[j] = v[j];
                    else if (a.atomic) atomicAdd(o + j, v[j]);
                    else o[j] += v[j];
                }
            }
        }
    }
}

// Plain mode: one warp's 32 rows x 32 output columns.  ``val`` holds this lane's row; the tile is turned
// in shared memory so that afterwards a lane holds a column and the warp reads and writes whole rows of
// the output (128 bytes of float32, 64 of bfloat16), eight rows in flight at a time.
template <int EPI>
__device__ __forceinline__ void epilogue_rows(const float* val, float* tile, const TcArgs& a, int row0, int col0,
                                              int n_cols, int lane, bool atomic = false) {
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 32; ++j) tile[lane * 33 + j] = val[j];
    __syncwarp();
    if (EPI == TB_EPI_ADD && atomic) {
        // The residual sum as reductions at L2 (red.global.add.v4.f32), for whole tiles as for the K parts of a tail
        // tile: nothing is read back, so the epilogue does not wait for a round trip per 32 rows (the o-projection of
        // a 2,048-token prompt: 69 -> 58 us); an element that one CTA alone adds to gets the same sum as by load and store.
        // Four rows per instruction, a lane adds four neighbouring columns with one vector reduction.
        const int sub = lane >> 3, c = (lane & 7) * 4;
        float* base = (float*)a.out + (size_t)row0 * a.ldo + col0 + c;
#pragma unroll
        for (int r4 = 0; r4 < 32; r4 += 4) {
            const int r = r4 + sub;
            if (row0 + r >= a.rows_a) continue;
            const float* t = tile + r * 33 + c;
            float* dst = base + (size_t)r * a.ldo;
            if (col0 + c + 3 < n_cols) {
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(t[0]), "f"(t[1]), "f"(t[2]), "f"(t[3]) : "memory");
            } else {
                for (int j = 0; j < 4; ++j)
                    if (col0 + c + j < n_cols) atomicAdd(dst + j, t[j]);
            }
        }
        return;
    }
    const int col = col0 + lane;
    if (col >= n_cols) return;
    float* o = (float*)a.out + (size_t)row0 * a.ldo + col;
    if (EPI == TB_EPI_ADD) {
        // all 32 rows of the residual are requested before the first is needed: one round trip, not four
        float old[32];
#pragma unroll
        for (int r = 0; r < 32; ++r) old[r] = (row0 + r < a.rows_a) ? o[(size_t)r * a.ldo] : 0.f;
#pragma unroll
        for (int r = 0; r < 32; ++r)
            if (row0 + r < a.rows_a) o[(size_t)r * a.ldo] = old[r] + tile[r * 33 + lane];
    } else {
#pragma unroll
        for (int r = 0; r < 32; ++r) {
            if (row0 + r >= a.rows_a) continue;
            const float v = tile[r * 33 + lane];
            if (EPI == TB_EPI_F32) o[(size_t)r * a.ldo] = v;
            else ((__nv_bfloat16*)a.out)[(size_t)(row0 + r) * a.ldo + col] = __float2bfloat16_rn(v);
        }
    }
}

// Swap mode: the tile as the epilogue warps have left it in shared memory, ``part`` [token][row of the tile = output
// column], goes out along the output's rows: a thread takes four neighbouring columns of a token (sixteen for SwiGLU:
// eight outputs), so a warp writes 512 contiguous bytes with one instruction where a thread that holds one column of
// every token needs an instruction per token (64 rows: 3.2 us of scalar reductions per CTA, 5 us of 2-byte stores).
template <int BN, int EPI>
__device__ __forceinline__ void swap_tile_out(const float* part, const TcArgs& a, int tile_a, int t) {
    if (EPI == TB_EPI_SWIGLU) {
        for (int item = t; item < BN * 8; item += 128) {
            const int m = item >> 3, n0 = tile_a * BM + (item & 7) * 16;
            if (m >= a.rows_b || n0 >= a.rows_a) continue;
            const float4* p = reinterpret_cast<const float4*>(part + m * BM + (item & 7) * 16);
            const float4 f0 = p[0], f1 = p[1], f2 = p[2], f3 = p[3];
            __nv_bfloat16* o = (__nv_bfloat16*)a.out + (size_t)m * a.ldo + n0 / 2;
            if (n0 + 16 <= a.rows_a) {
                uint4 pk;
                pk.x = pack_bf16(silu_mul(f0.x, f0.y), silu_mul(f0.z, f0.w)); pk.y = pack_bf16(silu_mul(f1.x, f1.y), silu_mul(f1.z, f1.w));
                pk.z = pack_bf16(silu_mul(f2.x, f2.y), silu_mul(f2.z, f2.w)); pk.w = pack_bf16(silu_mul(f3.x, f3.y), silu_mul(f3.z, f3.w));
                *reinterpret_cast<uint4*>(o) = pk;
            } else {
                const float v[16] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w, f2.x, f2.y, f2.z, f2.w, f3.x, f3.y, f3.z, f3.w};
                for (int j = 0; j < 16; j += 2)
                    if (n0 + j + 1 < a.rows_a) o[j / 2] = __float2bfloat16_rn(silu_mul(v[j], v[j + 1]));
            }
        }
    } else {
        for (int item = t; item < BN * 32; item += 128) {
            const int m = item >> 5, n0 = tile_a * BM + (item & 31) * 4;
            if (m >= a.rows_b || n0 >= a.rows_a) continue;
            const float4 f = *reinterpret_cast<const float4*>(part + m * BM + (item & 31) * 4);
            const bool whole = n0 + 4 <= a.rows_a;
            if (EPI == TB_EPI_STORE) {
                __nv_bfloat16* o = (__nv_bfloat16*)a.out + (size_t)m * a.ldo + n0;
                if (whole) {
                    *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16(f.x, f.y), pack_bf16(f.z, f.w));
                } else {
                    const float v[4] = {f.x, f.y, f.z, f.w};
                    for (int j = 0; j < 4; ++j) if (n0 + j < a.rows_a) o[j] = __float2bfloat16_rn(v[j]);
                }
            } else {
                float* o = (float*)a.out + (size_t)m * a.ldo + n0;
                if (whole && EPI == TB_EPI_F32) {
                    *reinterpret_cast<float4*>(o) = f;
                } else if (whole && a.atomic) {
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o), "f"(f.x), "f"(f.y), "f"(f.z), "f"(f.w) : "memory");
                } else if (whole) {
                    float4 old = *reinterpret_cast<const float4*>(o);
                    old.x += f.x; old.y += f.y; old.z += f.z; old.w += f.w;
                    *reinterpret_cast<float4*>(o) = old;
                } else {
                    const float v[4] = {f.x, f.y, f.z, f.w};
                    for (int j = 0; j < 4; ++j) {
                        if (n0 + j >= a.rows_a) continue;
                        if (EPI == TB_EPI_F32) o[j] = v[j];
                        else if (a.atomic) atomicAdd(o + j, v[j]);
                        else o[j] += v[j];
                    }
                }
            }
        }
    }
}

// ORDERED (swap mode, ADD epilogue): the K slices of a tile are the CTAs of one thread-block cluster.  Each leaves its
// partial tile in its own shared memory; after a cluster barrier every CTA adds up a share of the tile's elements
// from all slices, in slice order, through distributed shared memory, and adds the sum to the output.  An element is
// then written once, by one CTA, from a sum whose order is fixed: the same inputs give the same bits on every run,
// which float32 reductions that meet at L2 in the order they arrive do not.
template <int BN, int EPI, bool SWAP, bool NORMED = false, bool ORDERED = false>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcArgs a) {
    static_assert(!NORMED || (SWAP && BN <= 32), "the folded norm is for decode tiles (swap mode, at most 32 rows of activations)");
    static_assert(SWAP, "this kernel takes the decode products (weights on the 128-row side); prompts have the persistent and the pair kernel");
    static_assert(!ORDERED || EPI == TB_EPI_ADD, "slices in a fixed order: the ADD epilogue");
    constexpr int STAGES = stages_of<BN, EPI, SWAP>();
    constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    constexpr uint32_t TMEM_COLS = tmem_cols_for<BN>();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);     // swizzled tiles want 1024-byte alignment
    uint8_t* smem_a = base;
    uint8_t* smem_b = base + STAGES * A_BYTES;
    uint64_t* full = (uint64_t*)(base + STAGES * (A_BYTES + B_BYTES));
    uint64_t* empty = full + STAGES;
    uint64_t* accum = empty + STAGES;
    uint32_t* tmem_slot = (uint32_t*)(accum + 1);
    float* norm_sh = (float*)(tmem_slot + 2);               // NORMED: [4 warps][BN] sums of squares, then [BN] scales

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_a = blockIdx.y;                          // tile index along A's rows
    const int tile_b = blockIdx.x;                          // tile index along B's rows
    const int kb_total = (a.K + BK - 1) / BK;
    const int kb0 = blockIdx.z * a.k_blocks_per_split;
    const int kb1 = min(kb_total, kb0 + a.k_blocks_per_split);
    const int n_kb = kb1 - kb0;

    TimelineProbe probe;              // stamps: 1 wait for the kernel before passed, 2 first stage full, 3 last MMA done, 4 end, 5 last tile requested
    probe.begin(gridDim.y * 100 + gridDim.z, blockIdx.y + gridDim.y * blockIdx.z);
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        // NORMED: a stage is full when the weights have landed (TMA) and a warp has written the activations
        for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, NORMED ? 2 : 1); mbar_init(empty + s, 1); }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (NORMED) {       // rows of the activation tiles that no token fills stay zero (TMA would have filled them so)
        for (int i = threadIdx.x; i < (int)(STAGES * B_BYTES / 16); i += THREADS) reinterpret_cast<uint4*>(smem_b)[i] = make_uint4(0, 0, 0, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    constexpr uint32_t TX_BYTES = NORMED ? A_BYTES : A_BYTES + B_BYTES;
    probe.attach();

    if (n_kb > 0) {
        if (warp == 0) {
            if (lane == 0) {
                // The weight operand (A in swap mode, B in plain mode) is written by no kernel, so its
                // tiles for the first stages are requested before the wait on the previous kernel.
                const int pre = n_kb < STAGES ? n_kb : STAGES;
                const uint64_t once = tbtma::l2_evict_first_policy();     // swap mode: every weight is read once
                for (int i = 0; i < pre; ++i) {
                    mbar_expect_tx(full + i, TX_BYTES);
                    if (SWAP) tma_load_2d_hint(smem_a + i * A_BYTES, &map_a, full + i, (kb0 + i) * BK, tile_a * BM, once);
                    else tma_load_2d(smem_b + i * B_BYTES, &map_b, full + i, (kb0 + i) * BK, tile_b * BN);
                }
                pdl_wait();
                probe.stamp(1);
                for (int i = 0; i < pre; ++i) {
                    if (NORMED) continue;
                    if (SWAP) tma_load_2d(smem_b + i * B_BYTES, &map_b, full + i, (kb0 + i) * BK, tile_b * BN);
                    else tma_load_2d(smem_a + i * A_BYTES, &map_a, full + i, (kb0 + i) * BK, tile_a * BM);
                }
                for (int i = pre; i < n_kb; ++i) {
                    const int s = i % STAGES, round = i / STAGES;
                    mbar_wait(empty + s, (round - 1) & 1, 1);
                    mbar_expect_tx(full + s, TX_BYTES);
                    if (SWAP) tma_load_2d_hint(smem_a + s * A_BYTES, &map_a, full + s, (kb0 + i) * BK, tile_a * BM, once);
                    else tma_load_2d(smem_a + s * A_BYTES, &map_a, full + s, (kb0 + i) * BK, tile_a * BM);
                    if (!NORMED) tma_load_2d(smem_b + s * B_BYTES, &map_b, full + s, (kb0 + i) * BK, tile_b * BN);
                }
                probe.stamp(5);
            }
        } else if (warp == 1) {
            if (lane == 0) {
                pdl_wait();                                   // polling starts once the previous kernel is through
                constexpr uint32_t idesc = instr_desc(BM, BN);
                for (int i = 0; i < n_kb; ++i) {
                    const int s = i % STAGES, round = i / STAGES;
                    mbar_wait(full + s, round & 1, 2);
                    if (i == 0) probe.stamp(2);
                    tc_fence_after();
                    const uint64_t da = smem_desc(smem_u32(smem_a + s * A_BYTES));
                    const uint64_t db = smem_desc(smem_u32(smem_b + s * B_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)     // 32 bytes per K step: +2 in the descriptor's address field
                        tc_mma(tmem, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    tc_commit(empty + s);                     // the stage is free once these MMAs have read it
                }
                tc_commit(accum);
            }
        } else {
            // NORMED: the norm's weight for this warp's first activation tile depends on nothing that the kernel before
            // makes: it is requested while the wait for that kernel lasts
            float wv[8];
            if (NORMED && warp - 2 < n_kb) {
                const int k0 = (kb0 + warp - 2) * BK + (lane & 7) * 8;
                if (k0 < a.K) {
                    const float4 w0 = *reinterpret_cast<const float4*>(a.norm_w + k0), w1 = *reinterpret_cast<const float4*>(a.norm_w + k0 + 4);
                    wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w; wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
                }
            }
            pdl_wait();
            if (NORMED) {
                // The four epilogue warps make the activation tiles meanwhile, a stage each in turn (four stages in
                // flight): float32 rows of the residual stream times the norm's weight, rounded to bfloat16, into the
                // K-major 128-byte-swizzled layout that TMA would have written; and the rows' sums of squares.
                const int w4 = warp - 2;
                constexpr int UNITS = BN * 8 / 32;            // (row, 16-byte chunk) units per lane
                float ss[UNITS];
#pragma unroll
                for (int u = 0; u < UNITS; ++u) ss[u] = 0.f;
                for (int i = w4; i < n_kb; i += 4) {
                    const int s = i % STAGES, round = i / STAGES;
                    float xv[UNITS][8];
                    const int chunk = lane & 7, k0 = (kb0 + i) * BK + chunk * 8;
                    const bool k_ok = k0 < a.K;               // K is a multiple of 8: a chunk is inside or outside
                    if (k_ok && i != w4) {
                        const float4 w0 = *reinterpret_cast<const float4*>(a.norm_w + k0), w1 = *reinterpret_cast<const float4*>(a.norm_w + k0 + 4);
                        wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w; wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
                    }
#pragma unroll
                    for (int u = 0; u < UNITS; ++u) {         // all loads first
                        const int row = (lane >> 3) + 4 * u;
                        if (k_ok && row < a.rows_b) {
                            // Through L2 only: the rows were changed (float32 reductions at L2) by the product before, and
                            // this SM's L1 may still hold them as an earlier product's CTAs read them while this grid was
                            // already launched and waiting (programmatic dependent launch keeps three grids in flight).
                            const float* xp = a.xf + (size_t)row * a.ldxf + k0;
                            const float4 x0 = __ldcg(reinterpret_cast<const float4*>(xp)), x1 = __ldcg(reinterpret_cast<const float4*>(xp + 4));
                            xv[u][0] = x0.x; xv[u][1] = x0.y; xv[u][2] = x0.z; xv[u][3] = x0.w; xv[u][4] = x1.x; xv[u][5] = x1.y; xv[u][6] = x1.z; xv[u][7] = x1.w;
                        }
                    }
                    if (round > 0) mbar_wait(empty + s, (round - 1) & 1, 5);
#pragma unroll
                    for (int u = 0; u < UNITS; ++u) {
                        const int row = (lane >> 3) + 4 * u;
                        if (row >= a.rows_b) continue;
                        uint4 pk = make_uint4(0, 0, 0, 0);
                        if (k_ok) {
#pragma unroll
                            for (int e = 0; e < 8; ++e) ss[u] = fmaf(xv[u][e], xv[u][e], ss[u]);
                            pk.x = pack_bf16(xv[u][0] * wv[0], xv[u][1] * wv[1]); pk.y = pack_bf16(xv[u][2] * wv[2], xv[u][3] * wv[3]);
                            pk.z = pack_bf16(xv[u][4] * wv[4], xv[u][5] * wv[5]); pk.w = pack_bf16(xv[u][6] * wv[6], xv[u][7] * wv[7]);
                        }
                        *reinterpret_cast<uint4*>(smem_b + s * B_BYTES + row * 128 + ((chunk ^ (row & 7)) << 4)) = pk;
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // the tensor core reads these writes
                    __syncwarp();
                    if (lane == 0) tbtma::mbar_arrive(full + s);
                }
                // a row's sum: over the eight lanes that share it, then over the four warps
#pragma unroll
                for (int u = 0; u < UNITS; ++u) {
                    float v = ss[u];
                    v += __shfl_xor_sync(0xffffffffu, v, 1); v += __shfl_xor_sync(0xffffffffu, v, 2); v += __shfl_xor_sync(0xffffffffu, v, 4);
                    if ((lane & 7) == 0) norm_sh[w4 * BN + (lane >> 3) + 4 * u] = v;
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");
                if (warp == 2 && lane < BN) {
                    const float total = norm_sh[lane] + norm_sh[BN + lane] + norm_sh[2 * BN + lane] + norm_sh[3 * BN + lane];
                    if (a.sumsq_out) {                        // K slices: the consumer of the sums scales (a store, not an atomic: a fixed order of addition)
                        if (tile_a == 0 && lane < a.rows_b) a.sumsq_out[blockIdx.z * 32 + lane] = total;
                        norm_sh[4 * BN + lane] = 1.f;
                    } else {
                        norm_sh[4 * BN + lane] = 1.0f / sqrtf(total / (float)a.K + a.norm_eps);
                    }
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");
            }
            mbar_wait(accum, 0, 3);
            if (threadIdx.x == 64) probe.stamp(3);
            tc_fence_after();
            const int quarter = warp & 3;                     // a warp reads TMEM lanes 32 * (warp % 4) ..
            const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16);
            if (BN >= 32) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    float v[32];
                    tmem_ld32(taddr + c, v);
                    if (NORMED) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] *= norm_sh[4 * BN + c + j];
                    }
                    // the ring has drained: its first bytes hold the tile, [token][row of the tile]
#pragma unroll
                    for (int j = 0; j < 32; ++j) reinterpret_cast<float*>(smem_a)[(c + j) * BM + quarter * 32 + lane] = v[j];
                }
            } else {
                float v[16];
                tmem_ld16(taddr, v);
                if (NORMED) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] *= norm_sh[4 * BN + j];
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) reinterpret_cast<float*>(smem_a)[j * BM + quarter * 32 + lane] = v[j];
            }
            if (!ORDERED) {
                asm volatile("bar.sync 2, 128;" ::: "memory");         // the four epilogue warps: the tile is whole
                swap_tile_out<BN, EPI>(reinterpret_cast<const float*>(smem_a), a, tile_a, (int)threadIdx.x - 64);
            }
        }
    }
    pdl_wait();                                               // on every path (cheap once it has been passed)
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
    if (threadIdx.x == 0) probe.stamp(4);
    if (ORDERED) {
        // every thread of every CTA of the cluster: parts written -> summed -> may leave
        __syncwarp();
        tbtma::cluster_sync();
        const int n = (int)gridDim.z, total = a.rows_b * BM;          // tokens x rows of the tile (swap mode has one tile of tokens)
        const int per = (total + n - 1) / n, first = (int)tbtma::cluster_rank() * per, last = min(total, first + per);
        const float* part = reinterpret_cast<const float*>(smem_a);
        for (int idx = first + (int)threadIdx.x; idx < last; idx += THREADS) {
            float v[16];
#pragma unroll
            for (int r = 0; r < 16; ++r) v[r] = r < n ? tbtma::ld_cluster_f32(tbtma::cluster_addr(part + idx, r)) : 0.f;     // all loads first
            float sum = 0.f;
#pragma unroll
            for (int r = 0; r < 16; ++r) sum += v[r];                  // in the order of the slices
            const int m = idx / BM, row = tile_a * BM + idx % BM;
            if (row < a.rows_a) atomicAdd((float*)a.out + (size_t)m * a.ldo + row, sum);      // the element's only writer in this launch
        }
        __syncwarp();
        tbtma::cluster_sync();
    }
}

// ---------------------------------------------------------------- prompts: persistent, plain mode
// One CTA per SM walks over the output tiles (tile t = blockIdx.x + i * gridDim.x; consecutive tiles
// share a panel of W, so concurrent CTAs read the same weights from L2).  The accumulator is double
// buffered in tensor memory (2 x BN columns): while the four epilogue warps drain tile i, the MMA
// thread already accumulates tile i + 1 into the other buffer, and the TMA ring never drains between
// tiles.  Roles and barriers: producer -> full[s] -> MMA -> empty[s] -> producer;
// MMA -> acc_full[b] -> epilogue -> acc_empty[b] -> MMA.
// The work of one CTA of the persistent kernel as a list of segments (tile, first k-block, k-blocks).
// CTA c takes tiles c, c + grid, ... whole, as long as a round of tiles fills the grid.  The tiles of a
// last, partly filled round can be cut along K into ``tail_split`` parts (ADD epilogue only, where a
// partial sum can simply be added to the output through atomics), and the parts are dealt out the same
// way, so that the round takes ceil(tiles * parts / grid) / parts of a tile's time instead of all of it.
// Part p of every tail tile comes before part p + 1 of any, which keeps the CTAs that share an operand
// panel at nearby k-blocks (L2 reuse).
struct Segments {
    int n_kb, total, head, tail_units, parts, kb_per_part;
    int next_tile, next_unit, stride;
    __device__ Segments(const TcArgs& a, int n_kb_, int worker, int workers) : n_kb(n_kb_) {
        total = a.tiles_m * a.tiles_n;
        stride = workers;
        parts = 1; kb_per_part = n_kb;
        head = total;
        if (a.tail_split > 1) {
            kb_per_part = (n_kb + a.tail_split - 1) / a.tail_split;
            parts = (n_kb + kb_per_part - 1) / kb_per_part;
            head = total / stride * stride;
        }
        tail_units = (total - head) * parts;
        next_tile = worker; next_unit = worker;
    }
    __device__ bool next(int& tile, int& kb0, int& count) {
        if (next_tile < head) {
            tile = next_tile; kb0 = 0; count = n_kb; next_tile += stride;
            return true;
        }
        if (next_unit >= tail_units) return false;
        const int tail_tiles = total - head, part = next_unit / tail_tiles;
        tile = head + next_unit - part * tail_tiles;
        kb0 = part * kb_per_part;
        count = n_kb - kb0 < kb_per_part ? n_kb - kb0 : kb_per_part;
        next_unit += stride;
        return true;
    }
};
// The same walk one k-block at a time (for the TMA producer).
struct KBlocks {
    Segments seg; int tile, kb, left, tiles_m;
    __device__ KBlocks(const TcArgs& a, int n_kb, int worker, int workers)
        : seg(a, n_kb, worker, workers), tile(0), kb(0), left(0), tiles_m(a.tiles_m) {}
    __device__ bool next(int& tile_a, int& tile_b, int& k) {
        if (left == 0) {
            int kb0, count;
            if (!seg.next(tile, kb0, count)) return false;
            kb = kb0; left = count;
        }
        tile_a = tile % tiles_m; tile_b = tile / tiles_m; k = kb;
        ++kb; --left;
        return true;
    }
};

template <int BN, int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcArgs a) {
    constexpr int STAGES = stages_for<BN>();
    constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    constexpr uint32_t TMEM_COLS = 2 * BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = base;
    uint8_t* smem_b = base + STAGES * A_BYTES;
    uint64_t* full = (uint64_t*)(base + STAGES * (A_BYTES + B_BYTES));
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;          // [2]
    uint64_t* acc_empty = acc_full + 2;           // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    float* epi_tiles = (float*)(base + STAGES * (A_BYTES + B_BYTES) + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kb = (a.K + BK - 1) / BK;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            KBlocks w_blocks(a, n_kb, blockIdx.x, gridDim.x), blocks(a, n_kb, blockIdx.x, gridDim.x);       // two walks over the same k-blocks
            int ta, tb, k, pre = 0;
            for (; pre < STAGES && w_blocks.next(ta, tb, k); ++pre) {     // weights first: no kernel writes them
                mbar_expect_tx(full + pre, A_BYTES + B_BYTES);
                tma_load_2d(smem_b + pre * B_BYTES, &map_b, full + pre, k * BK, tb * BN);
            }
            pdl_wait();                                       // the activations come from the kernel before
            for (int it = 0; it < pre; ++it) {
                blocks.next(ta, tb, k);
                tma_load_2d(smem_a + it * A_BYTES, &map_a, full + it, k * BK, ta * BM);
            }
            for (int it = pre; blocks.next(ta, tb, k); ++it) {
                const int s = it % STAGES, round = it / STAGES;
                mbar_wait(empty + s, (round - 1) & 1, 1);
                mbar_expect_tx(full + s, A_BYTES + B_BYTES);
                tma_load_2d(smem_a + s * A_BYTES, &map_a, full + s, k * BK, ta * BM);
                tma_load_2d(smem_b + s * B_BYTES, &map_b, full + s, k * BK, tb * BN);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            pdl_wait();
            constexpr uint32_t idesc = instr_desc(BM, BN);
            Segments segs(a, n_kb, blockIdx.x, gridDim.x);
            int it = 0, tile, kb0, count;
            for (int j = 0; segs.next(tile, kb0, count); ++j) {
                const int buf = j & 1;
                if (j >= 2) mbar_wait(acc_empty + buf, ((j >> 1) - 1) & 1, 4);     // the epilogue has drained this buffer
                tc_fence_after();
                const uint32_t acc = tmem + buf * BN;
                for (int i = 0; i < count; ++i, ++it) {
                    const int s = it % STAGES, round = it / STAGES;
                    mbar_wait(full + s, round & 1, 2);
                    tc_fence_after();
                    const uint64_t da = smem_desc(smem_u32(smem_a + s * A_BYTES));
                    const uint64_t db = smem_desc(smem_u32(smem_b + s * B_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        tc_mma(acc, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    tc_commit(empty + s);
                }
                tc_commit(acc_full + buf);
            }
        }
    } else {
        pdl_wait();
        const int quarter = warp & 3;
        float* tile = epi_tiles + quarter * EPI_TILE_FLOATS;
        Segments segs(a, n_kb, blockIdx.x, gridDim.x);
        int t, kb0, count;
        for (int j = 0; segs.next(t, kb0, count); ++j) {
            const int tile_a = t % a.tiles_m, tile_b = t / a.tiles_m;
            (void)count;
            const int buf = j & 1;
            mbar_wait(acc_full + buf, (j >> 1) & 1, 3);
            tc_fence_after();
            const int row = tile_a * BM + quarter * 32 + lane;
            const uint32_t taddr = tmem + buf * BN + ((uint32_t)(quarter * 32) << 16);
            if (EPI == TB_EPI_ADD) {
                const int row0 = tile_a * BM + quarter * 32;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    float v[32];
                    tmem_ld32(taddr + c, v);
                    epilogue_rows<EPI>(v, tile, a, row0, tile_b * BN + c, a.rows_b, lane, true);
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    float v[32];
                    tmem_ld32(taddr + c, v);
                    epilogue_chunk<EPI, 32>(v, a, row, tile_b * BN + c, lane);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tbtma::mbar_arrive(acc_empty + buf);
        }
    }
    pdl_wait();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// ---------------------------------------------------------------- prompts: pairs of CTAs (cta_group::2)
// A cluster of two CTAs on neighbouring SMs works on one 256 x 256 tile: each CTA loads 128 rows of X and
// 128 rows of W per k-block (32 KB instead of the 48 KB a lone CTA needs for 128 x 256, so six stages
// fit and every byte in shared memory feeds twice the MMA work), the leader (rank 0) issues
// tcgen05.mma.cta_group::2 with M = 256, which reads both CTAs' shared memory, and each CTA's tensor
// memory receives its 128 rows of the tile (two buffers of 256 columns: all 512).  Barriers:
//   full[s]     leader only; both CTAs' TMA loads count their bytes on it (no multicast anywhere)
//   empty[s]    in both CTAs; the leader's tcgen05.commit arrives on both when the MMAs have read stage s
//   acc_full[b] in both CTAs, same way;  acc_empty[b]: leader only, the eight epilogue warps of the pair arrive
// The walk over tiles, the tail split and the epilogues are those of the one-CTA kernel.
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_N = 256;
constexpr uint32_t PAIR_A_BYTES = BM * BK * 2, PAIR_B_BYTES = 128 * BK * 2;
constexpr size_t PAIR_SMEM = 1024 + (size_t)PAIR_STAGES * (PAIR_A_BYTES + PAIR_B_BYTES) + 256 + 4 * EPI_TILE_FLOATS * sizeof(float);

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcArgs a) {
    constexpr int STAGES = PAIR_STAGES;
    constexpr uint32_t A_BYTES = PAIR_A_BYTES, B_BYTES = PAIR_B_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = base;
    uint8_t* smem_b = base + STAGES * A_BYTES;
    uint64_t* full = (uint64_t*)(base + STAGES * (A_BYTES + B_BYTES));
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;          // [2]
    uint64_t* acc_empty = acc_full + 2;           // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    float* epi_tiles = (float*)(base + STAGES * (A_BYTES + B_BYTES) + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = tbtma::cluster_rank();
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int n_kb = (a.K + BK - 1) / BK;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, 512);
    tc_fence_before();
    tbtma::cluster_sync();                         // both CTAs' barriers exist before either signals the other's
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            KBlocks w_blocks(a, n_kb, pair, pairs), blocks(a, n_kb, pair, pairs);
            int ta, tb, k, pre = 0;
            for (; pre < STAGES && w_blocks.next(ta, tb, k); ++pre) {     // weights first: no kernel writes them
                if (rank == 0) mbar_expect_tx(full + pre, 2 * (A_BYTES + B_BYTES));
                tbtma::tma_load_2d_pair(smem_b + pre * B_BYTES, &map_b, tbtma::cluster_addr(full + pre, 0), k * BK, tb * PAIR_N + rank * 128);
            }
            pdl_wait();
            for (int it = 0; it < pre; ++it) {
                blocks.next(ta, tb, k);
                tbtma::tma_load_2d_pair(smem_a + it * A_BYTES, &map_a, tbtma::cluster_addr(full + it, 0), k * BK, ta * 2 * BM + rank * BM);
            }
            for (int it = pre; blocks.next(ta, tb, k); ++it) {
                const int s = it % STAGES, round = it / STAGES;
                mbar_wait(empty + s, (round - 1) & 1, 1);
                if (rank == 0) mbar_expect_tx(full + s, 2 * (A_BYTES + B_BYTES));
                const uint32_t bar = tbtma::cluster_addr(full + s, 0);
                tbtma::tma_load_2d_pair(smem_a + s * A_BYTES, &map_a, bar, k * BK, ta * 2 * BM + rank * BM);
                tbtma::tma_load_2d_pair(smem_b + s * B_BYTES, &map_b, bar, k * BK, tb * PAIR_N + rank * 128);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            pdl_wait();
            constexpr uint32_t idesc = instr_desc(2 * BM, PAIR_N);
            Segments segs(a, n_kb, pair, pairs);
            int it = 0, tile, kb0, count;
            for (int j = 0; segs.next(tile, kb0, count); ++j) {
                const int buf = j & 1;
                if (j >= 2) mbar_wait(acc_empty + buf, ((j >> 1) - 1) & 1, 4);     // both CTAs' epilogues have drained this buffer
                tc_fence_after();
                const uint32_t acc = tmem + buf * PAIR_N;
                for (int i = 0; i < count; ++i, ++it) {
                    const int s = it % STAGES, round = it / STAGES;
                    mbar_wait(full + s, round & 1, 2);
                    tc_fence_after();
                    const uint64_t da = smem_desc(smem_u32(smem_a + s * A_BYTES));
                    const uint64_t db = smem_desc(smem_u32(smem_b + s * B_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        tc_mma_pair(acc, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    tc_commit_pair(empty + s, 3);
                }
                tc_commit_pair(acc_full + buf, 3);
            }
        }
    } else {
        pdl_wait();
        const int quarter = warp & 3;
        float* tile = epi_tiles + quarter * EPI_TILE_FLOATS;
        Segments segs(a, n_kb, pair, pairs);
        int t, kb0, count;
        for (int j = 0; segs.next(t, kb0, count); ++j) {
            const int tile_a = t % a.tiles_m, tile_b = t / a.tiles_m;
            (void)count;
            const int buf = j & 1;
            mbar_wait(acc_full + buf, (j >> 1) & 1, 3);
            tc_fence_after();
            const int row0 = tile_a * 2 * BM + (int)rank * BM + quarter * 32;
            const uint32_t taddr = tmem + buf * PAIR_N + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < PAIR_N; c += 32) {
                float v[32];
                tmem_ld32(taddr + c, v);
                if (EPI == TB_EPI_ADD) epilogue_rows<EPI>(v, tile, a, row0, tile_b * PAIR_N + c, a.rows_b, lane, true);
                else epilogue_chunk<EPI, 32>(v, a, row0 + lane, tile_b * PAIR_N + c, lane);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tbtma::mbar_arrive_cluster(tbtma::cluster_addr(acc_empty + buf, 0));
        }
    }
    pdl_wait();
    tc_fence_before();
    tbtma::cluster_sync();                         // nobody leaves while the other still reads its shared memory or signals it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem, 512);
    }
}

// ---------------------------------------------------------------- host side
template <int BN, int EPI, bool SWAP>
int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const TcArgs& a, dim3 grid, cudaStream_t stream) {
    static bool configured = false;
    constexpr size_t smem = smem_for<BN, SWAP, stages_of<BN, EPI, SWAP>()>();
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI, SWAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI, SWAP>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);   // room for several CTAs per SM
        TB_REQUIRE(e == cudaSuccess, "gemm_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    tb_launch(gemm_tc_kernel<BN, EPI, SWAP>, grid, THREADS, smem, stream, ma, mb, a);
    return 0;
}

template <int BN, int EPI>
int launch_tc_normed(const CUtensorMap& ma, const TcArgs& a, dim3 grid, cudaStream_t stream) {
    static bool configured = false;
    constexpr size_t smem = smem_for<BN, true, stages_of<BN, EPI, true>()>();
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI, true, true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        TB_REQUIRE(e == cudaSuccess, "gemm_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    tb_launch(gemm_tc_kernel<BN, EPI, true, true>, grid, THREADS, smem, stream, ma, ma, a);
    return 0;
}

// Swap mode, ADD epilogue, the K slices of a tile as one cluster (grid.z CTAs) that adds them up in slice order.
template <int BN, bool NORMED>
int launch_tc_ordered(const CUtensorMap& ma, const CUtensorMap& mb, const TcArgs& a, dim3 grid, cudaStream_t stream) {
    static bool configured = false;
    constexpr size_t smem = smem_for<BN, true, stages_of<BN, TB_EPI_ADD, true>()>();
    auto kernel = gemm_tc_kernel<BN, TB_EPI_ADD, true, NORMED, true>;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);      // clusters of up to 16
        TB_REQUIRE(e == cudaSuccess, "gemm_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    const cudaError_t e = tb_launch_cluster_z(kernel, grid, THREADS, smem, stream, (int)grid.z, ma, mb, a);
    TB_REQUIRE(e == cudaSuccess, "gemm_tc: the launch of clusters of %d K slices failed: %s", (int)grid.z, cudaGetErrorString(e));
    return 0;
}
// How many clusters of ``size`` CTAs of this kernel the device holds at once (0: it places none).  Clusters are placed
// as wholes inside one part of the chip, so this is less than the CTAs it holds divided by the size.
template <int BN, bool NORMED>
int ordered_clusters(int size) {
    static int cached[17];
    static bool known[17] = {false};
    if (size < 1 || size > 16) return 0;
    if (!known[size]) {
        constexpr size_t smem = smem_for<BN, true, stages_of<BN, TB_EPI_ADD, true>()>();
        auto kernel = gemm_tc_kernel<BN, TB_EPI_ADD, true, NORMED, true>;
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, 1, size); cfg.blockDim = dim3(THREADS, 1, 1); cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = (unsigned)size;
        cfg.attrs = attr; cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) { clusters = 0; cudaGetLastError(); }
        cached[size] = clusters; known[size] = true;
    }
    return cached[size];
}
int ordered_clusters_for(int bn, bool normed, int size) {
    if (normed) return bn == 16 ? ordered_clusters<16, true>(size) : ordered_clusters<32, true>(size);
    switch (bn) {
        case 16: return ordered_clusters<16, false>(size);
        case 32: return ordered_clusters<32, false>(size);
        case 64: return ordered_clusters<64, false>(size);
    }
    return ordered_clusters<128, false>(size);
}
// The most K slices, at most ``wanted``, with which the clusters of all ``tiles`` tiles are held at once (a cluster
// that waits for a second round costs more than the slices gain); 1: no slices.
int ordered_fit(int bn, bool normed, int tiles, int wanted) {
    for (int size = wanted > 16 ? 16 : wanted; size > 1; --size)
        if (ordered_clusters_for(bn, normed, size) >= tiles) return size;
    return 1;
}

template <int BN, int EPI>
int launch_persistent_epi(const CUtensorMap& ma, const CUtensorMap& mb, const TcArgs& a, dim3 grid, cudaStream_t stream) {
    static bool configured = false;
    constexpr size_t smem = smem_for<BN, false>();
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, EPI>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);   // room for several CTAs per SM
        TB_REQUIRE(e == cudaSuccess, "gemm_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    tb_launch(gemm_tc_persistent_kernel<BN, EPI>, grid, THREADS, smem, stream, ma, mb, a);
    return 0;
}

template <int BN>
int launch_persistent(int epi, const CUtensorMap& ma, const CUtensorMap& mb, const TcArgs& a, dim3 grid, cudaStream_t stream) {
    switch (epi) {
        case TB_EPI_STORE: return launch_persistent_epi<BN, TB_EPI_STORE>(ma, mb, a, grid, stream);
        case TB_EPI_F32: return launch_persistent_epi<BN, TB_EPI_F32>(ma, mb, a, grid, stream);
        case TB_EPI_ADD: return launch_persistent_epi<BN, TB_EPI_ADD>(ma, mb, a, grid, stream);
        case TB_EPI_SWIGLU: return launch_persistent_epi<BN, TB_EPI_SWIGLU>(ma, mb, a, grid, stream);
    }
    tb_set_error("gemm_tc: unknown epilogue %d", epi);
    return 1;
}

// Clusters of two that the device can hold at once (0 if the query fails: then the one-CTA kernel runs).
template <int EPI>
int pair_clusters() {
    static int n = -1;
    if (n < 0) {
        n = 0;
        if (cudaFuncSetAttribute(gemm_tc_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PAIR_SMEM) == cudaSuccess) {
            cudaFuncSetAttribute(gemm_tc_pair_kernel<EPI>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(2, 1, 1); cfg.blockDim = dim3(THREADS, 1, 1); cfg.dynamicSmemBytes = PAIR_SMEM;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, gemm_tc_pair_kernel<EPI>, &cfg) == cudaSuccess && clusters > 0) n = clusters;
            else cudaGetLastError();
        } else {
            cudaGetLastError();
        }
    }
    return n;
}
template <int EPI>
int launch_pair_epi(const CUtensorMap& ma, const CUtensorMap& mb, const TcArgs& a, int pairs, cudaStream_t stream) {
    tb_launch(gemm_tc_pair_kernel<EPI>, dim3(2 * pairs, 1, 1), THREADS, PAIR_SMEM, stream, ma, mb, a);
    return 0;
}
int pair_clusters_for(int epi) {
    switch (epi) {
        case TB_EPI_STORE: return pair_clusters<TB_EPI_STORE>();
        case TB_EPI_F32: return pair_clusters<TB_EPI_F32>();
        case TB_EPI_ADD: return pair_clusters<TB_EPI_ADD>();
        case TB_EPI_SWIGLU: return pair_clusters<TB_EPI_SWIGLU>();
    }
    return 0;
}
int launch_pair(int epi, const CUtensorMap& ma, const CUtensorMap& mb, const TcArgs& a, int pairs, cudaStream_t stream) {
    switch (epi) {
        case TB_EPI_STORE: return launch_pair_epi<TB_EPI_STORE>(ma, mb, a, pairs, stream);
        case TB_EPI_F32: return launch_pair_epi<TB_EPI_F32>(ma, mb, a, pairs, stream);
        case TB_EPI_ADD: return launch_pair_epi<TB_EPI_ADD>(ma, mb, a, pairs, stream);
        case TB_EPI_SWIGLU: return launch_pair_epi<TB_EPI_SWIGLU>(ma, mb, a, pairs, stream);
    }
    tb_set_error("gemm_tc: unknown epilogue %d", epi);
    return 1;
}

template <int BN, bool SWAP>
int launch_epi(int epi, const CUtensorMap& ma, const CUtensorMap& mb, const TcArgs& a, dim3 grid, cudaStream_t stream) {
    switch (epi) {
        case TB_EPI_STORE: return launch_tc<BN, TB_EPI_STORE, SWAP>(ma, mb, a, grid, stream);
        case TB_EPI_F32: return launch_tc<BN, TB_EPI_F32, SWAP>(ma, mb, a, grid, stream);
        case TB_EPI_ADD: return launch_tc<BN, TB_EPI_ADD, SWAP>(ma, mb, a, grid, stream);
        case TB_EPI_SWIGLU: return launch_tc<BN, TB_EPI_SWIGLU, SWAP>(ma, mb, a, grid, stream);
    }
    tb_set_error("gemm_tc: unknown epilogue %d", epi);
    return 1;
}

}  // namespace

// Reads and clears the error word of the tensor-core kernels (0: none; 1, 2, 3: a wait of the
// producer, the MMA issuer or the epilogue ran out).  Synchronises the device.
int g_plain_tile = 0;
int g_swap_below = 128;
extern "C" void tb_gemm_tc_set_swap_below(int m) { g_swap_below = m; }
// Prompt products: 0 chooses the tile shape, 1 forces CTA pairs (256 x 256), 2 single CTAs with 128 x 256, 3 with 128 x 128.
extern "C" void tb_gemm_tc_set_plain_tile(int which) { g_plain_tile = which; }

int g_pair = 1;
// Prompt products on pairs of CTAs (cta_group::2; 1, default) or on single CTAs (0).
extern "C" void tb_gemm_tc_set_pair(int on) { g_pair = on ? 1 : 0; }

// How many CTA pairs the device holds at once for this epilogue's kernel (0: the pair kernel cannot run).
extern "C" int tb_gemm_tc_pair_clusters(int epi) { return pair_clusters_for(epi); }

int g_tail_split = 1;
// Prompt products with the ADD epilogue: cut the tiles of a last, partly filled round along K (1, default) or not (0).
extern "C" void tb_gemm_tc_set_tail_split(int on) { g_tail_split = on ? 1 : 0; }

extern "C" int tb_gemm_tc_error() {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(v)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(zero));
    return (int)v;
}

// 0 if tb_gemm_tc can run these sizes, else 1 with the reason in tb_last_error().
extern "C" int tb_gemm_tc_check(int M, int N, int K, int ldx, int ldo, int epi, const void* X, const void* W, const void* out) {
    TB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tc: sizes must be positive");
    TB_REQUIRE(K % 8 == 0 && ldx % 8 == 0, "gemm_tc: K=%d and the row stride %d of X must be multiples of 8 (16-byte TMA rows)", K, ldx);
    TB_REQUIRE(((uintptr_t)X & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_tc: operands must be 16-byte aligned");
    TB_REQUIRE(epi != TB_EPI_SWIGLU || N % 2 == 0, "gemm_tc: the SwiGLU epilogue needs an even N");
    TB_REQUIRE(epi < 0 || ((uintptr_t)out & 15) == 0, "gemm_tc: the output must be 16-byte aligned");
    const int unit = (epi == TB_EPI_STORE || epi == TB_EPI_SWIGLU) ? 8 : 4;
    TB_REQUIRE(ldo % unit == 0, "gemm_tc: the row stride %d of the output must be a multiple of %d", ldo, unit);
    return 0;
}

// 0 if tb_gemm_tc_normed takes this product: a decode step's rows (at most 32), the SwiGLU epilogue or float32 sums.
extern "C" int tb_gemm_tc_normed_check(int M, int N, int K, int ldxf, int ldo, int epi, const void* xf, const void* norm_w,
                                       const void* W, const void* out, const void* sumsq_out) {
    TB_REQUIRE(M > 0 && M <= 32 && M < g_swap_below, "gemm_tc_normed: %d rows (a decode step's: at most 32)", M);
    TB_REQUIRE(epi == TB_EPI_ADD || epi == TB_EPI_SWIGLU, "gemm_tc_normed: the epilogue must be ADD (sums for a consumer that scales) or SWIGLU");
    TB_REQUIRE((epi == TB_EPI_ADD) == (sumsq_out != nullptr), "gemm_tc_normed: sums of squares go out with the ADD epilogue and only with it");
    TB_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && ldxf % 4 == 0, "gemm_tc_normed: K=%d must be a multiple of 8 and the row stride %d of x a multiple of 4", K, ldxf);
    TB_REQUIRE(((uintptr_t)xf & 15) == 0 && ((uintptr_t)norm_w & 15) == 0 && ((uintptr_t)W & 15) == 0 && ((uintptr_t)out & 15) == 0,
               "gemm_tc_normed: operands must be 16-byte aligned");
    TB_REQUIRE(epi != TB_EPI_SWIGLU || N % 2 == 0, "gemm_tc_normed: the SwiGLU epilogue needs an even N");
    TB_REQUIRE(ldo % (epi == TB_EPI_SWIGLU ? 8 : 4) == 0, "gemm_tc_normed: the row stride %d of the output", ldo);
    return 0;
}

// K slices of tb_gemm_tc_normed with the ADD epilogue for these sizes: as many as fill the machine once, four blocks each at least.
static int normed_slices(int N, int K, int epi, int M = 1, bool ordered = false) {
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
    }
    const int kb = (K + BK - 1) / BK, tiles = (N + BM - 1) / BM;
    int s = 1;
    if (epi == TB_EPI_ADD) {
        s = 2 * sm_count / tiles;
        const int max_s = kb / 4 > 0 ? kb / 4 : 1;
        s = s < 1 ? 1 : (s > max_s ? max_s : s);
        s = s > 16 ? 16 : s;
        if (ordered) s = ordered_fit(M <= 16 ? 16 : 32, true, tiles, s);
    }
    const int per = (kb + s - 1) / s;
    return (kb + per - 1) / per;
}
// M, ordered: the rows of the step and whether the slices add up in a fixed order (a cluster per tile: fewer slices fit).
extern "C" int tb_gemm_tc_normed_slices(int N, int K, int epi, int M, int ordered) { return normed_slices(N, K, epi, M, ordered != 0); }

// out (epilogue) = rmsnorm(xf; norm_w, eps)[M,K] . W[N,K]^T for a decode step's rows, the norm folded into the product:
// the kernel reads the float32 rows, multiplies by the norm's weight on the way into shared memory and by
// 1/sqrt(mean(x^2) + eps) in its epilogue (SWIGLU), or (ADD: K is cut into slices) adds the products of the
// unscaled rows into ``out`` and leaves the rows' sums of squares, one row of 32 per K slice
// (tb_gemm_tc_normed_slices of them), at ``sumsq_out`` [slices][32], for the consumer to add up and scale.
// ordered: the K slices add up in slice order inside a thread-block cluster (the same bits on every run) instead of through
// float32 reductions that meet at L2 in the order they arrive.
extern "C" int tb_gemm_tc_normed(const float* xf, int ldxf, const float* norm_w, float eps, const void* W, void* out,
                                 int M, int N, int K, int ldo, int epi, float* sumsq_out, int ordered, cudaStream_t stream) {
    if (tb_gemm_tc_normed_check(M, N, K, ldxf, ldo, epi, xf, norm_w, W, out, sumsq_out)) return 1;
    const int kb = (K + BK - 1) / BK;
    const int tiles = (N + BM - 1) / BM;
    TB_REQUIRE(tiles <= 65535, "gemm_tc_normed: N=%d is too large for one launch", N);
    const int s = normed_slices(N, K, epi, M, ordered != 0);
    TcArgs a;
    a.out = out; a.rows_a = N; a.rows_b = M; a.K = K; a.ldo = ldo; a.tiles_m = a.tiles_n = 0; a.tail_split = 1;
    a.k_blocks_per_split = (kb + s - 1) / s;
    a.atomic = s > 1;
    a.xf = xf; a.ldxf = ldxf; a.norm_w = norm_w; a.sumsq_out = sumsq_out; a.norm_eps = eps;
    CUtensorMap ma;
    if (tb_make_map_bf16(&ma, W, N, K, K, BM)) return 1;
    dim3 grid(1, tiles, s);
    int rc;
    if (ordered && epi == TB_EPI_ADD && s > 1) {
        TB_REQUIRE(ordered_clusters_for(M <= 16 ? 16 : 32, true, s) > 0, "gemm_tc_normed: this device places no cluster of %d K slices", s);
        a.atomic = 0;
        rc = M <= 16 ? launch_tc_ordered<16, true>(ma, ma, a, grid, stream) : launch_tc_ordered<32, true>(ma, ma, a, grid, stream);
    } else if (M <= 16) rc = epi == TB_EPI_ADD ? launch_tc_normed<16, TB_EPI_ADD>(ma, a, grid, stream) : launch_tc_normed<16, TB_EPI_SWIGLU>(ma, a, grid, stream);
    else rc = epi == TB_EPI_ADD ? launch_tc_normed<32, TB_EPI_ADD>(ma, a, grid, stream) : launch_tc_normed<32, TB_EPI_SWIGLU>(ma, a, grid, stream);
    if (rc) return rc;
    TB_CHECK_LAUNCH("gemm_tc_normed");
    return 0;
}

// splits: K slices (swap mode, ADD epilogue only); 0 = choose; -1 = choose, and add the parts of a sum in a fixed order
// (swap mode: the slices of a tile form a thread-block cluster; prompt products: no tile is cut along K), so that
// the same inputs give the same bits on every run.
extern "C" int tb_gemm_tc(const void* X, const void* W, void* out, int M, int N, int K, int ldx, int ldo, int epi,
                          int splits, cudaStream_t stream) {
    if (tb_gemm_tc_check(M, N, K, ldx, ldo, epi, X, W, out)) return 1;
    const bool ordered = splits < 0;
    if (ordered) splits = 0;
    const bool swap = M < g_swap_below;
    const int kb = (K + BK - 1) / BK;
    CUtensorMap ma, mb;
    TcArgs a;
    a.out = out; a.K = K; a.ldo = ldo; a.k_blocks_per_split = kb; a.atomic = 0; a.tiles_m = a.tiles_n = 0; a.tail_split = 1;
    a.xf = nullptr; a.ldxf = 0; a.norm_w = nullptr; a.sumsq_out = nullptr; a.norm_eps = 0.f;
    int rc = 0;
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
    }
    // parts along K for the tiles of a last, partly filled round of ``workers``: the fewest that make
    // the round shortest (an epilogue per part is charged; a part keeps at least four k-blocks)
    auto tail_parts = [&](int total, int workers) {
        const int tail = total % workers;
        int best = 1;
        if (epi != TB_EPI_ADD || !g_tail_split || ordered || !tail) return best;      // total < workers: every tile is in the last round
        double best_cost = 1.0;
        for (int p = 2; p <= 8 && kb / p >= 4; ++p) {
            const double cost = (double)((tail * p + workers - 1) / workers) / p + 0.02 * p;
            if (cost < best_cost - 1e-9) { best = p; best_cost = cost; }
        }
        return best;
    };
    int pairs_max = (!swap && g_pair && M > 128 && N >= 256) ? pair_clusters_for(epi) : 0;
    int single_bn = N >= 256 ? 256 : 128;
    if (!swap && M < 1024) {
        // Which tile shape is fastest for this output (from 1,024 rows on: pairs).  Measured at M = 128 .. 1024: where rows are few, a CTA
        // is bound by the tiles it loads, and a tile of a pair's CTA (128 rows of X, 128 of W for 128 x 256
        // outputs) costs 1, a lone 128 x 256 tile 1.1 and a 128 x 128 tile 0.85; what decides is how many
        // rounds of tiles the shape needs and how many rows its padding wastes.  The ADD epilogue cuts a
        // last round into K parts, so its rounds count as fractions.
        const bool parts = epi == TB_EPI_ADD && g_tail_split && !ordered;
        auto rounds = [&](long long tiles, int workers) {
            const double r = parts ? (double)tiles / workers : (double)((tiles + workers - 1) / workers);
            return r < 0.125 ? 0.125 : r;
        };
        const long long m128 = (M + 127) / 128, m256 = (M + 255) / 256;
        const double t_pair = pairs_max > 0 ? rounds(m256 * ((N + 255) / 256), pairs_max) * 1.0 : 1e30;
        const double t_256 = N >= 256 ? rounds(m128 * ((N + 255) / 256), sm_count) * 1.1 : 1e30;
        const double t_128 = rounds(m128 * ((N + 127) / 128), sm_count) * 0.85;
        if (t_128 < t_pair && t_128 < t_256) { pairs_max = 0; single_bn = 128; }
        else if (t_256 < t_pair) pairs_max = 0;
    }
    if (!swap && g_plain_tile == 1 && M > 128 && N >= 256) pairs_max = pair_clusters_for(epi);
    if (!swap && g_plain_tile == 2) { pairs_max = 0; single_bn = N >= 256 ? 256 : 128; }
    if (!swap && g_plain_tile == 3) { pairs_max = 0; single_bn = 128; }
    if (pairs_max > 0) {
        a.rows_a = M; a.rows_b = N;
        a.tiles_m = (M + 2 * BM - 1) / (2 * BM); a.tiles_n = (N + PAIR_N - 1) / PAIR_N;
        if (tb_make_map_bf16(&ma, X, M, K, ldx, BM) || tb_make_map_bf16(&mb, W, N, K, K, 128)) return 1;
        TB_REQUIRE((long long)a.tiles_m * a.tiles_n < (1LL << 30), "gemm_tc: too many tiles");
        const int total = a.tiles_m * a.tiles_n;
        a.tail_split = tail_parts(total, pairs_max);
        const int units = total < pairs_max ? total * a.tail_split : total;      // fewer tiles than pairs: the parts fill the grid
        const int pairs = units < pairs_max ? units : pairs_max;
        rc = launch_pair(epi, ma, mb, a, pairs, stream);
    } else if (!swap) {
        const int bn = single_bn;
        a.rows_a = M; a.rows_b = N;
        a.tiles_m = (M + BM - 1) / BM; a.tiles_n = (N + bn - 1) / bn;
        if (tb_make_map_bf16(&ma, X, M, K, ldx, BM) || tb_make_map_bf16(&mb, W, N, K, K, bn)) return 1;
        TB_REQUIRE((long long)a.tiles_m * a.tiles_n < (1LL << 30), "gemm_tc: too many tiles");
        const int total = a.tiles_m * a.tiles_n;
        a.tail_split = tail_parts(total, sm_count);
        const int units = total < sm_count ? total * a.tail_split : total;
        dim3 grid(units < sm_count ? units : sm_count, 1, 1);
        rc = bn == 256 ? launch_persistent<256>(epi, ma, mb, a, grid, stream) : launch_persistent<128>(epi, ma, mb, a, grid, stream);
    } else {
        const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
        a.rows_a = N; a.rows_b = M;
        const int tiles = (N + BM - 1) / BM;
        int s = 1;
        if (epi == TB_EPI_ADD) {
            // as many K slices as fill the machine once
            const int room = 2 * sm_count;                        // two CTAs fit an SM at every width
            s = splits > 0 ? splits : room / tiles;
            const int max_s = kb / 4 > 0 ? kb / 4 : 1;              // at least four 64-wide blocks per slice
            s = s < 1 ? 1 : (s > max_s ? max_s : s);
            if (ordered) s = ordered_fit(bn, false, tiles, s);
        }
        a.k_blocks_per_split = (kb + s - 1) / s;
        s = (kb + a.k_blocks_per_split - 1) / a.k_blocks_per_split;  // no empty slice
        a.atomic = s > 1 && !ordered;
        if (tb_make_map_bf16(&ma, W, N, K, K, BM) || tb_make_map_bf16(&mb, X, M, K, ldx, bn)) return 1;
        dim3 grid(1, tiles, s);
        TB_REQUIRE(tiles <= 65535, "gemm_tc: N=%d is too large for one launch", N);
        if (ordered && epi == TB_EPI_ADD && s > 1) {
            switch (bn) {
                case 16: rc = launch_tc_ordered<16, false>(ma, mb, a, grid, stream); break;
                case 32: rc = launch_tc_ordered<32, false>(ma, mb, a, grid, stream); break;
                case 64: rc = launch_tc_ordered<64, false>(ma, mb, a, grid, stream); break;
                default: rc = launch_tc_ordered<128, false>(ma, mb, a, grid, stream); break;
            }
        } else
        switch (bn) {
            case 16: rc = launch_epi<16, true>(epi, ma, mb, a, grid, stream); break;
            case 32: rc = launch_epi<32, true>(epi, ma, mb, a, grid, stream); break;
            case 64: rc = launch_epi<64, true>(epi, ma, mb, a, grid, stream); break;
            default: rc = launch_epi<128, true>(epi, ma, mb, a, grid, stream); break;
        }
    }
    if (rc) return rc;
    TB_CHECK_LAUNCH("gemm_tc");
    return 0;
}

// Names the buffer of the timeline probe (timeline.cuh); 1 if the library was built with it, 0 if not.
TB_TIMELINE_SETTER(tb_gemm_tc_timeline)
