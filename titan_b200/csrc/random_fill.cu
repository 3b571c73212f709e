// Random weights made on the device: element i of a tensor is a pure function of (key, i), where the key is
// derived on the host from (seed, tensor name).  The same function is written once more in numpy
// (titan_b200/weights/random_init.py) and the two give the same bits: every step below is integer
// arithmetic or a single IEEE-754 double operation (add, multiply, divide, square root: correctly rounded
// on both sides), written with the _rn intrinsics so that the compiler fuses no multiply with an add, and
// there is no call of a library logarithm or cosine, whose last bit differs between libraries.
//
//   z      = mix64(key + (i + 1) * 0x9E3779B97F4A7C15)              (the finaliser of splitmix64)
//   u1     = ((z >> 40) + 1) / 2^24 in (0, 1],   k2 = (z >> 16) & 0xFFFFFF
//   normal = sqrt(-2 ln u1) * cos(2 pi k2 / 2^24)                    (Box-Muller)
//   ln u1  = (e - 24) ln 2 + 2 atanh((m - 1) / (m + 1)),  u1 = m 2^(e - 24), m in [1, 2): eleven terms
//   cos    : the quadrant from the top two bits of k2, then Taylor polynomials of degree 18 and 19 on [0, pi/2)
//   value  = float(normal) * std + mean in float32, then rounded to the tensor's dtype
//
// berniehans/titan has no random weights; its only generator is the fixed pattern of
// tools/build_synthetic_gguf.py:129-203.
#include "common.cuh"

namespace {

__host__ __device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ double standard_normal(unsigned long long z) {
    const unsigned int n = (unsigned int)(z >> 40) + 1u;          // 1 .. 2^24
    const unsigned int k2 = (unsigned int)(z >> 16) & 0xFFFFFFu;
    const int e = 31 - __clz(n);                                  // n = m 2^e, m in [1, 2)
    const double m = __dmul_rn((double)n, __longlong_as_double((long long)(1023 - e) << 52));    // exact
    const double t = __ddiv_rn(__dadd_rn(m, -1.0), __dadd_rn(m, 1.0));
    const double t2 = __dmul_rn(t, t);
    double s = 1.0 / 21.0;                                        // sum_{j=0..10} t^(2j) / (2j + 1), by Horner
#pragma unroll
    for (int j = 9; j >= 0; --j) s = __dadd_rn(__dmul_rn(s, t2), __ddiv_rn(1.0, (double)(2 * j + 1)));
    const double ln_m = __dmul_rn(__dmul_rn(2.0, t), s);
    const double ln_u = __dadd_rn(__dmul_rn((double)(e - 24), 0.6931471805599453094), ln_m);
    const double r = __dsqrt_rn(__dmul_rn(-2.0, ln_u));
    const unsigned int quadrant = k2 >> 22;
    const double phi = __dmul_rn(__dmul_rn((double)(k2 & 0x3FFFFFu), 1.0 / 4194304.0), 1.5707963267948966192);
    const double p2 = __dmul_rn(phi, phi);
    double c = 0.0, sn = 0.0;                                     // cos = sum (-1)^j p^(2j) / (2j)!, sin = p sum (-1)^j p^(2j) / (2j+1)!
    double fc = 6402373705728000.0, fs = 121645100408832000.0;    // 18!, 19!
#pragma unroll
    for (int j = 9; j >= 0; --j) {
        const double sign = (j & 1) ? -1.0 : 1.0;
        c = __dadd_rn(__dmul_rn(c, p2), __ddiv_rn(sign, fc));
        sn = __dadd_rn(__dmul_rn(sn, p2), __ddiv_rn(sign, fs));
        if (j > 0) { fc = __ddiv_rn(fc, (double)((2 * j) * (2 * j - 1))); fs = __ddiv_rn(fs, (double)((2 * j + 1) * (2 * j))); }
    }
    sn = __dmul_rn(sn, phi);
    const double trig = quadrant == 0 ? c : (quadrant == 1 ? -sn : (quadrant == 2 ? -c : sn));
    return __dmul_rn(r, trig);
}

template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, long long n, unsigned long long key, float std, float mean) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const unsigned long long z = mix64(key + (unsigned long long)(i + 1) * 0x9E3779B97F4A7C15ull);
        const float v = __fadd_rn(__fmul_rn((float)standard_normal(z), std), mean);
        stf(out + i, v);
    }
}

__global__ void fill_int_kernel(int* __restrict__ out, long long n, unsigned long long key, int bound_bits) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const unsigned long long z = mix64(key + (unsigned long long)(i + 1) * 0x9E3779B97F4A7C15ull);
        out[i] = (int)(z >> (64 - bound_bits));
    }
}

}  // namespace

// out[i] = value(key, i) * std + mean for i < n.  dtype: TB_F32 or TB_BF16, or -1 for int32 values in [0, 2^15).
extern "C" int tb_fill_random(void* out, int dtype, long long n, unsigned long long key, float std, float mean, cudaStream_t stream) {
    TB_REQUIRE(out && n > 0, "fill_random: nothing to fill");
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (dtype == TB_F32) fill_normal_kernel<float><<<blocks, threads, 0, stream>>>((float*)out, n, key, std, mean);
    else if (dtype == TB_BF16) fill_normal_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((__nv_bfloat16*)out, n, key, std, mean);
    else if (dtype == -1) fill_int_kernel<<<blocks, threads, 0, stream>>>((int*)out, n, key, 15);
    else TB_REQUIRE(false, "fill_random: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("fill_random");
    return 0;
}
