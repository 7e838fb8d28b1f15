// The 32-bit matrix product of the true float path: C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]), all
// float, plain FFMA (no tensor cores, hence no reduced-precision matrix mode). Every output element
// is one sequential chain of fused multiply-adds over k = 0..K-1, so its value depends on neither M,
// nor the tile it falls in, nor what else is in the batch. The reference has no device float path;
// its float arithmetic is the f64 `linear` of helios/crates/helios-hal/src/reference.rs:24-41.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256) sgemm_kernel(const float* __restrict__ a, const float* __restrict__ w,
                                                    const float* __restrict__ bias, float* __restrict__ c, int m, int n,
                                                    int k, int lda, int ldc) {
    __shared__ float as[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
    const int ty = tid / 16, tx = tid % 16;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    // each thread loads 4 consecutive k of one row of each tile: 64 rows x 16 k = 256 threads x 4
    const int lrow = tid / 4, lk = (tid % 4) * 4;
    for (int k0 = 0; k0 < k; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int kk = k0 + lk + e;
            const int ar = row0 + lrow, wr = col0 + lrow;
            as[lk + e][lrow] = (ar < m && kk < k) ? a[(size_t)ar * lda + kk] : 0.f;
            ws[lk + e][lrow] = (wr < n && kk < k) ? w[(size_t)wr * k + kk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float av[TM], wv[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = as[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) wv[j] = ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = row0 + ty * TM + i;
        if (r >= m) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int col = col0 + tx * TN + j;
            if (col < n) c[(size_t)r * ldc + col] = acc[i][j] + (bias ? bias[col] : 0.f);
        }
    }
}
}  // namespace

// A rows are `lda` floats apart, C rows `ldc`; W is dense [n, k]. Zero padding of the k tail adds
// exact zeros to the chain and does not change the result.
HB_EXPORT int hb_sgemm_f32(const float* a, const float* w, const float* bias, float* c, int m, int n, int k, int lda,
                           int ldc, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0) return HB_BAD_ARGUMENT;
    dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
    if (grid.y > 65535) return HB_UNSUPPORTED_SIZE;
    sgemm_kernel<<<grid, 256, 0, stream>>>(a, w, bias, c, m, n, k, lda, ldc);
    return launch_status();
}
