// Plain matrix product on the CUDA cores: out = X[M,K] . W[N,K]^T with float32 accumulation.
//
// This is the true 32-bit path (T = float: FFMA only, no tensor-core or reduced-precision mode)
// and the plain twin of the tensor-core kernel for bfloat16 operands; it takes every M, N, K.
// berniehans/titan's counterpart is its warp-per-column kernels
// (engine/engine-cuda/kernels/gemm_quant.cu:2331-2363 gemm_f32_kernel, :3365-3499 batched), which
// fuse the residual into the epilogue (:3489-3493) and SwiGLU into gate/up (:2589).
//
// Epilogues:
//   TB_EPI_STORE   out[m][n] = acc                      (compute dtype)
//   TB_EPI_F32     out[m][n] = acc                      (float32: logits)
//   TB_EPI_ADD     out[m][n] += acc                     (float32 residual stream, in place)
//   TB_EPI_SWIGLU  out[m][j] = silu(acc[2j]) * acc[2j+1] (rows of W interleaved gate, up; N even)
#include "common.cuh"
#include "gemm.h"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ X, const T* __restrict__ W, void* __restrict__ out,
                 int M, int N, int K, int ldx, int ldo) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;     // thread tile: rows ty*4.., cols tx*4..
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k of each operand: 1024 elements, 4 per thread
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            const int r = idx / BK, kk = idx % BK;
            const int k = k0 + kk;
            xs[kk][r] = (m0 + r < M && k < K) ? ldf(X + (size_t)(m0 + r) * ldx + k) : 0.f;
            ws[kk][r] = (n0 + r < N && k < K) ? ldf(W + (size_t)(n0 + r) * K + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
        if (EPI == TB_EPI_SWIGLU) {
#pragma unroll
            for (int j = 0; j < TN; j += 2) {
                const int n = n0 + tx * TN + j;
                if (n + 1 < N) {
                    const float g = acc[i][j], u = acc[i][j + 1];
                    stf((T*)out + (size_t)m * ldo + n / 2, g / (1.0f + expf(-g)) * u);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const int n = n0 + tx * TN + j;
                if (n >= N) continue;
                if (EPI == TB_EPI_STORE) stf((T*)out + (size_t)m * ldo + n, acc[i][j]);
                if (EPI == TB_EPI_F32) ((float*)out)[(size_t)m * ldo + n] = acc[i][j];
                if (EPI == TB_EPI_ADD) ((float*)out)[(size_t)m * ldo + n] += acc[i][j];
            }
        }
    }
}

template <typename T>
int launch(const void* X, const void* W, void* out, int M, int N, int K, int ldx, int ldo, int epi,
           cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    const T* x = (const T*)X;
    const T* w = (const T*)W;
    switch (epi) {
        case TB_EPI_STORE: tb_launch(gemm_simt_kernel<T, TB_EPI_STORE>, grid, 256, 0, stream, x, w, out, M, N, K, ldx, ldo); break;
        case TB_EPI_F32: tb_launch(gemm_simt_kernel<T, TB_EPI_F32>, grid, 256, 0, stream, x, w, out, M, N, K, ldx, ldo); break;
        case TB_EPI_ADD: tb_launch(gemm_simt_kernel<T, TB_EPI_ADD>, grid, 256, 0, stream, x, w, out, M, N, K, ldx, ldo); break;
        case TB_EPI_SWIGLU: tb_launch(gemm_simt_kernel<T, TB_EPI_SWIGLU>, grid, 256, 0, stream, x, w, out, M, N, K, ldx, ldo); break;
        default: tb_set_error("gemm: unknown epilogue %d", epi); return 1;
    }
    return 0;
}

}  // namespace

// ldx: row stride of X in elements; ldo: row stride of out in elements.
extern "C" int tb_gemm_simt(const void* X, const void* W, void* out, int dtype, int M, int N, int K, int ldx,
                            int ldo, int epi, cudaStream_t stream) {
    TB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: sizes must be positive (M=%d N=%d K=%d)", M, N, K);
    TB_REQUIRE(ldx >= K, "gemm: row stride %d of X is shorter than K=%d", ldx, K);
    TB_REQUIRE(epi != TB_EPI_SWIGLU || N % 2 == 0, "gemm: the SwiGLU epilogue needs an even N, found %d", N);
    TB_REQUIRE((M + BM - 1) / BM <= 65535, "gemm: M=%d is too large for one launch", M);
    int rc;
    if (dtype == TB_F32) rc = launch<float>(X, W, out, M, N, K, ldx, ldo, epi, stream);
    else if (dtype == TB_BF16) rc = launch<__nv_bfloat16>(X, W, out, M, N, K, ldx, ldo, epi, stream);
    else { tb_set_error("gemm: unknown dtype %d", dtype); return 1; }
    if (rc) return rc;
    TB_CHECK_LAUNCH("gemm_simt");
    return 0;
}
