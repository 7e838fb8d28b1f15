// Causal grouped-query attention over the paged cache for any head size up to 256, any number of
// heads and groups, and an optional window: the kernel of the 32-bit path (and of float tests of the
// bfloat16 kernels). One block serves one token and up to 8 query heads of one key/value head.
// Keys are walked in tiles of 64 absolute positions (tile t covers positions 64t..64t+63), with a
// running maximum and sum in float, so a token's result does not depend on how its request was cut
// into steps or on the rest of the batch. The formula is the reference's: q head h reads kv head
// h / group, scores (q.k) * scale for key position <= query position, softmax, weighted sum of values
// (helios/crates/helios-hal/src/reference.rs:118-156; kernels/elementwise.cu:64-118).
#include "common.cuh"

namespace {
constexpr int TILE = 64, THREADS = 128, GMAX = 8, DMAX = 256;

template <typename T>
__global__ void __launch_bounds__(THREADS) attention_generic_kernel(
    const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride, const T* __restrict__ cache,
    const int* __restrict__ block_table, int table_width, const int* __restrict__ token_row,
    const int* __restrict__ positions, int heads, int kv_heads, int head_dim, int page_size, int pages, float scale,
    int window, int* status) {
    __shared__ float qs[GMAX][DMAX];
    __shared__ float score[GMAX][TILE];
    __shared__ float m_run[GMAX], l_run[GMAX], alpha[GMAX];
    __shared__ int tile_page[TILE];

    const int t = blockIdx.x, kvh = blockIdx.y;
    const int group = heads / kv_heads;
    const int g0 = blockIdx.z * GMAX;
    const int g = min(GMAX, group - g0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pos = positions[t];
    const int row = token_row[t];
    const int* table = block_table + (size_t)row * table_width;

    for (int e = tid; e < g * head_dim; e += THREADS) {
        const int hh = e / head_dim, d = e - hh * head_dim;
        qs[hh][d] = to_float(q[(size_t)t * q_stride + (size_t)(kvh * group + g0 + hh) * head_dim + d]);
    }
    if (tid < GMAX) { m_run[tid] = -INFINITY; l_run[tid] = 0.f; }
    float acc[GMAX][DMAX / THREADS];
#pragma unroll
    for (int hh = 0; hh < GMAX; ++hh)
#pragma unroll
        for (int c = 0; c < DMAX / THREADS; ++c) acc[hh][c] = 0.f;

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const size_t head_stride = (size_t)page_size * head_dim;
    const size_t page_stride = 2 * (size_t)kv_heads * head_stride;
    bool bad_page = false;
    __syncthreads();

    for (int base = (lo / TILE) * TILE; base <= pos; base += TILE) {
        // pages of the tile's keys
        if (tid < TILE) {
            const int j = base + tid;
            int page = -1;
            if (j >= lo && j <= pos) {
                const int block = j / page_size;
                page = block < table_width ? table[block] : -1;
                if (page < 0 || page >= pages) { bad_page = true; page = -1; }
            }
            tile_page[tid] = page;
        }
        __syncthreads();
        // scores: one warp per key, lanes across the head dimension
        for (int jj = warp; jj < TILE; jj += THREADS / 32) {
            const int j = base + jj;
            const int page = tile_page[jj];
            float part[GMAX];
#pragma unroll
            for (int hh = 0; hh < GMAX; ++hh) part[hh] = 0.f;
            if (page >= 0) {
                const T* kp = cache + (size_t)page * page_stride + (size_t)kvh * head_stride + (size_t)(j % page_size) * head_dim;
                for (int d = lane; d < head_dim; d += 32) {
                    const float kv = to_float(kp[d]);
#pragma unroll
                    for (int hh = 0; hh < GMAX; ++hh)
                        if (hh < g) part[hh] = fmaf(qs[hh][d], kv, part[hh]);
                }
            }
#pragma unroll
            for (int hh = 0; hh < GMAX; ++hh) {
                if (hh < g) {
                    const float s = warp_sum(part[hh]);
                    if (lane == 0) score[hh][jj] = page >= 0 ? s * scale : -INFINITY;
                }
            }
        }
        __syncthreads();
        // new running maximum and the rescale factor, one thread per head
        if (tid < g) {
            float m = m_run[tid];
            for (int jj = 0; jj < TILE; ++jj) m = fmaxf(m, score[tid][jj]);
            alpha[tid] = (m == -INFINITY) ? 1.f : expf(m_run[tid] - m);
            m_run[tid] = m;
        }
        __syncthreads();
        for (int e = tid; e < g * TILE; e += THREADS) {
            const int hh = e / TILE, jj = e - hh * TILE;
            const float m = m_run[hh];
            score[hh][jj] = (m == -INFINITY) ? 0.f : expf(score[hh][jj] - m);
        }
        __syncthreads();
        if (tid < g) {
            float l = l_run[tid] * alpha[tid];
            for (int jj = 0; jj < TILE; ++jj) l += score[tid][jj];
            l_run[tid] = l;
        }
        // weighted values: thread d walks the tile's keys in order
#pragma unroll
        for (int c = 0; c < DMAX / THREADS; ++c) {
            const int d = tid + c * THREADS;
            if (d < head_dim) {
#pragma unroll
                for (int hh = 0; hh < GMAX; ++hh)
                    if (hh < g) acc[hh][c] *= alpha[hh];
                for (int jj = 0; jj < TILE; ++jj) {
                    const int page = tile_page[jj];
                    if (page < 0) continue;
                    const int j = base + jj;
                    const float vv = to_float(cache[(size_t)page * page_stride + (size_t)(kv_heads + kvh) * head_stride +
                                                    (size_t)(j % page_size) * head_dim + d]);
#pragma unroll
                    for (int hh = 0; hh < GMAX; ++hh)
                        if (hh < g) acc[hh][c] = fmaf(score[hh][jj], vv, acc[hh][c]);
                }
            }
        }
        __syncthreads();
    }
    if (bad_page) atomicOr(status, HB_STATUS_BAD_PAGE);
#pragma unroll
    for (int c = 0; c < DMAX / THREADS; ++c) {
        const int d = tid + c * THREADS;
        if (d < head_dim) {
#pragma unroll
            for (int hh = 0; hh < GMAX; ++hh)
                if (hh < g) {
                    const float l = l_run[hh];
                    out[(size_t)t * out_stride + (size_t)(kvh * group + g0 + hh) * head_dim + d] =
                        from_float<T>(l > 0.f ? acc[hh][c] / l : 0.f);
                }
        }
    }
}
}  // namespace

HB_EXPORT int hb_attention_generic(const void* q, int q_stride, void* out, int out_stride, int is_bf16, const void* cache,
                                   const int* block_table, int table_width, const int* token_row, const int* positions,
                                   int tokens, int heads, int kv_heads, int head_dim, int page_size, int pages, float scale,
                                   int window, int* status, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (head_dim <= 0 || head_dim > DMAX || kv_heads <= 0 || heads % kv_heads || page_size <= 0) return HB_UNSUPPORTED_SIZE;
    const int group = heads / kv_heads;
    dim3 grid(tokens, kv_heads, (group + GMAX - 1) / GMAX);
    if (grid.y > 65535 || grid.z > 65535) return HB_UNSUPPORTED_SIZE;
    if (is_bf16)
        attention_generic_kernel<<<grid, THREADS, 0, stream>>>((const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride,
                                                               (const __nv_bfloat16*)cache, block_table, table_width, token_row,
                                                               positions, heads, kv_heads, head_dim, page_size, pages, scale, window, status);
    else
        attention_generic_kernel<<<grid, THREADS, 0, stream>>>((const float*)q, q_stride, (float*)out, out_stride, (const float*)cache,
                                                               block_table, table_width, token_row, positions, heads, kv_heads,
                                                               head_dim, page_size, pages, scale, window, status);
    return launch_status();
}
