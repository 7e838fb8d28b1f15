// Seeded random weights on the device: normal deviates that are a pure function of (key, element index), with the
// same bits as the host's generator (hyperion_b200/weights/philox_normal.py).
//
// Counter c = index / 2 goes through Philox4x32-10 (Salmon et al., SC11; the reference's sampler uses the same
// generator, helios/crates/helios-hal/src/sampler_reference.rs:67-84); its first two words are the uniforms of a
// Box-Muller transform, whose cosine branch is element 2c and whose sine branch is element 2c + 1. The logarithm and
// the cosine and sine are series in 64-bit floating point whose coefficients the caller supplies (the host
// evaluates the same series with the same numbers). Every operation is an explicitly rounded IEEE 754 one
// (__dadd_rn, __dmul_rn, __ddiv_rn, __dsqrt_rn): the compiler may not fuse a product with a sum, so the result does
// not depend on the compiler or on the machine. The reference has no random-weight mode
// (scripts/gen-sharded-fixture.py:32-50 saves a library's default initialisation).
#include "common.cuh"

namespace {
constexpr int LN_TERMS = 9, TRIG_TERMS = 12;

struct NormalConstants {
    double ln[LN_TERMS];     // 1 / (2k + 1)
    double cos[TRIG_TERMS];  // (-1)^k / (2k)!
    double sin[TRIG_TERMS];  // (-1)^k / (2k + 1)!
    double ln2, half_pi, sqrt_half;
};

__device__ __forceinline__ void philox4x32_10(unsigned c0, unsigned c1, unsigned k0, unsigned k1, unsigned& w0, unsigned& w1) {
    unsigned c2 = 0, c3 = 0;
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        const unsigned long long p0 = 0xD2511F53ull * c0, p1 = 0xCD9E8D57ull * c2;
        const unsigned n0 = (unsigned)(p1 >> 32) ^ c1 ^ k0, n1 = (unsigned)p1, n2 = (unsigned)(p0 >> 32) ^ c3 ^ k1, n3 = (unsigned)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    w0 = c0;
    w1 = c1;
}

template <int N>
__device__ __forceinline__ double series(double x2, const double (&c)[N]) {
    double acc = c[N - 1];
#pragma unroll
    for (int k = N - 2; k >= 0; --k) acc = __dadd_rn(__dmul_rn(acc, x2), c[k]);
    return acc;
}

// The standard normal pair of counter `pair`.
__device__ __forceinline__ void normal_pair(unsigned long long pair, unsigned k0, unsigned k1, const NormalConstants& k, double& z0, double& z1) {
    unsigned w0, w1;
    philox4x32_10((unsigned)pair, (unsigned)(pair >> 32), k0, k1, w0, w1);
    const double u1 = __dmul_rn(__dadd_rn((double)w0, 0.5), 0x1p-32);  // in (0, 1): exact
    int e;
    double m = frexp(u1, &e);  // exact
    if (m < k.sqrt_half) { m = __dmul_rn(m, 2.0); e -= 1; }
    const double s = __ddiv_rn(__dadd_rn(m, -1.0), __dadd_rn(m, 1.0));
    const double log_u1 = __dadd_rn(__dmul_rn((double)e, k.ln2), __dmul_rn(__dmul_rn(2.0, s), series(__dmul_rn(s, s), k.ln)));
    const double radius = __dsqrt_rn(__dmul_rn(-2.0, log_u1));
    const int quadrant = (int)(w1 >> 30);
    const double r = __dmul_rn((double)(w1 & 0x3FFFFFFFu), 0x1p-30);
    const double phi = __dmul_rn(r, k.half_pi), phi2 = __dmul_rn(phi, phi);
    const double c = series(phi2, k.cos), sn = __dmul_rn(phi, series(phi2, k.sin));
    const double cos_t = quadrant == 0 ? c : (quadrant == 1 ? -sn : (quadrant == 2 ? -c : sn));
    const double sin_t = quadrant == 0 ? sn : (quadrant == 1 ? c : (quadrant == 2 ? -sn : -c));
    z0 = __dmul_rn(radius, cos_t);
    z1 = __dmul_rn(radius, sin_t);
}

template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, long long count, unsigned k0, unsigned k1, double std, double mean,
                                     const NormalConstants k) {
    const long long pairs = (count + 1) / 2;
    for (long long pair = (long long)blockIdx.x * blockDim.x + threadIdx.x; pair < pairs; pair += (long long)gridDim.x * blockDim.x) {
        double z0, z1;
        normal_pair((unsigned long long)pair, k0, k1, k, z0, z1);
        // one rounding from double to float, then the storage type's own
        out[2 * pair] = from_float<T>(__double2float_rn(__dadd_rn(__dmul_rn(z0, std), mean)));
        if (2 * pair + 1 < count) out[2 * pair + 1] = from_float<T>(__double2float_rn(__dadd_rn(__dmul_rn(z1, std), mean)));
    }
}
}  // namespace

// out[i] = mean + std * z_i for i < count, z standard normal from (key_lo, key_hi, i); out is float or bfloat16.
// `constants` points at the host's copy of the series coefficients (NormalConstants), passed on to the kernel by value.
HB_EXPORT int hb_random_normal(void* out, int out_is_bf16, long long count, unsigned key_lo, unsigned key_hi, double std, double mean,
                               const void* constants, cudaStream_t stream) {
    if (count <= 0) return 0;
    if (!constants || !out) return HB_BAD_ARGUMENT;
    const NormalConstants k = *reinterpret_cast<const NormalConstants*>(constants);
    const long long pairs = (count + 1) / 2;
    const int threads = 256;
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
        return HB_BAD_ARGUMENT;
    const long long wanted = (pairs + threads - 1) / threads, most = (long long)sms * 16;  // the kernel strides over what is left
    const int blocks = (int)(wanted < most ? wanted : most);
    if (out_is_bf16) random_normal_kernel<<<blocks, threads, 0, stream>>>((__nv_bfloat16*)out, count, key_lo, key_hi, std, mean, k);
    else random_normal_kernel<<<blocks, threads, 0, stream>>>((float*)out, count, key_lo, key_hi, std, mean, k);
    return launch_status();
}
