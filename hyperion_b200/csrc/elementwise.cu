// Row-wise kernels of the decoder: embedding lookup, residual add fused with RMSNorm, SwiGLU,
// rotate-half position encoding, and the write of new keys and values into cache pages.
// Each is instantiated for float (the 32-bit path) and for bfloat16 storage; arithmetic is float in
// both. What they compute corresponds to the reference's embedding_gather_bf16, add_rmsnorm_bf16,
// swiglu_rows_bf16, rope_bf16 and kv_append_rows_paged_bf16
// (helios/crates/helios-hal/kernels/elementwise.cu:13,29,42,844; kernels/rmsnorm.cu:66), except
// that the residual stream stays in float and a value is rounded once, when it is stored.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embedding_kernel(const TW* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                 int hidden, int vocab, int* status) {
    const int t = blockIdx.x;
    const int id = ids[t];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, HB_STATUS_BAD_TOKEN);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)t * hidden + i] = 0.f;
        return;
    }
    const TW* row = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)t * hidden + i] = to_float(row[i]);
}

// bfloat16 rows whose width is a multiple of 8: one 16-byte load and two 16-byte stores per thread.
__global__ void embedding_bf16x8_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                        int hidden, int vocab, int* status) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0) atomicOr(status, HB_STATUS_BAD_TOKEN);
    const __nv_bfloat16* row = table + (size_t)(ok ? id : 0) * hidden;
    for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (ok) {
            const uint4 v = *reinterpret_cast<const uint4*>(row + i);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
            const float2 f0 = __bfloat1622float2(h[0]), f1 = __bfloat1622float2(h[1]), f2 = __bfloat1622float2(h[2]), f3 = __bfloat1622float2(h[3]);
            a = make_float4(f0.x, f0.y, f1.x, f1.y);
            b = make_float4(f2.x, f2.y, f3.x, f3.y);
        }
        *reinterpret_cast<float4*>(out + (size_t)t * hidden + i) = a;
        *reinterpret_cast<float4*>(out + (size_t)t * hidden + i + 4) = b;
    }
}

HB_EXPORT int hb_embedding(const void* table, int table_is_bf16, const int* ids, float* out, int tokens, int hidden,
                           int vocab, int* status, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (table_is_bf16 && hidden % 8 == 0 && (((uintptr_t)table | (uintptr_t)out) & 15) == 0) {
        const int threads = min(512, ((hidden / 8 + 31) / 32) * 32);
        embedding_bf16x8_kernel<<<tokens, threads, 0, stream>>>((const __nv_bfloat16*)table, ids, out, hidden, vocab, status);
        return launch_status();
    }
    if (table_is_bf16)
        embedding_kernel<<<tokens, 256, 0, stream>>>((const __nv_bfloat16*)table, ids, out, hidden, vocab, status);
    else
        embedding_kernel<<<tokens, 256, 0, stream>>>((const float*)table, ids, out, hidden, vocab, status);
    return launch_status();
}

// Tokens that were sampled by the step before and never left the device: ids[pairs[2i]] = source[pairs[2i+1]].
__global__ void place_tokens_kernel(int* __restrict__ ids, const int* __restrict__ source, const int* __restrict__ pairs, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) ids[pairs[2 * i]] = source[pairs[2 * i + 1]];
}

// The caller has checked the pairs against the sizes of ids and source.
HB_EXPORT int hb_place_tokens(int* ids, const int* source, const int* pairs, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    place_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(ids, source, pairs, n);
    return launch_status();
}

// ---------------------------------------------------------------- residual add + RMSNorm
// Output row r normalises source row s = rows ? rows[r] : r of h (+ delta). With `write_h` the sum
// is stored back into h[s] (the residual stream); it is skipped when rows are gathered for the
// final norm, whose sum nobody reads again. The sum of squares is taken in a fixed order.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta, const float* __restrict__ weight,
                                   TO* __restrict__ out, const int* __restrict__ rows, int hidden, float eps, int write_h) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* hrow = h + (size_t)s * hidden;
    const TD* drow = delta ? delta + (size_t)s * hidden : nullptr;
    float sum = 0.f;
    let_next_kernel_start();
    wait_for_previous_kernels();
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = hrow[i];
        if (drow) {
            v += to_float(drow[i]);
            if (write_h) hrow[i] = v;
        }
        sum = fmaf(v, v, sum);
    }
    const float total = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    TO* orow = out + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = hrow[i];
        if (drow && !write_h) v += to_float(drow[i]);
        orow[i] = from_float<TO>(v * inv * weight[i]);
    }
}

// The same with a row's values held in registers between the two passes (rows of up to 8 values per thread): one trip
// to memory instead of two, which is what counts when a decode step has only a handful of rows.
template <typename TD, typename TO>
__global__ void add_rmsnorm_cached_kernel(float* __restrict__ h, const TD* __restrict__ delta, const float* __restrict__ weight,
                                          TO* __restrict__ out, const int* __restrict__ rows, int hidden, float eps, int write_h) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* hrow = h + (size_t)s * hidden;
    const TD* drow = delta ? delta + (size_t)s * hidden : nullptr;
    float v[8], w[8];
    float sum = 0.f;
    let_next_kernel_start();
#pragma unroll
    for (int j = 0; j < 8; ++j) {  // the norm's weight is nobody's output: it is fetched while the kernel before still runs
        const int i = threadIdx.x + j * blockDim.x;
        w[j] = i < hidden ? weight[i] : 0.f;
    }
    wait_for_previous_kernels();
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        v[j] = 0.f;
        if (i < hidden) {
            v[j] = hrow[i];
            if (drow) v[j] += to_float(drow[i]);
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {  // the same order of additions per thread as the uncached kernel
        const int i = threadIdx.x + j * blockDim.x;
        if (i < hidden) {
            if (drow && write_h) hrow[i] = v[j];
            sum = fmaf(v[j], v[j], sum);
        }
    }
    const float total = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    TO* orow = out + (size_t)r * hidden;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < hidden) orow[i] = from_float<TO>(v[j] * inv * w[j]);
    }
}

// The serving path's shape of it (bfloat16 delta and output, rows of a multiple of 8 values): 8 values per thread and
// group with 16- and 32-byte accesses, each row read once. G groups per thread cover rows of up to 8 * G * 512 values.
// With `partials` ([splits, tokens, hidden] floats: the split-K sums of the product that made the delta) the delta is
// their sum in split order plus the bias, rounded to bfloat16 as the product's own reduction would store it.
// split-K pieces a thread asks for at once (products of a decode step are split 5 to 10 times); fewer where a thread holds
// several groups of a wide row
__host__ __device__ constexpr int pieces_ahead(int groups_per_thread) { return groups_per_thread == 1 ? 12 : (groups_per_thread == 2 ? 8 : 4); }
struct SplitDelta {
    const float* partials;
    size_t split_stride;  // tokens * hidden
    int splits;
    const float* bias_f;
    const __nv_bfloat16* bias_h;
};

template <int G>
__global__ void __launch_bounds__(512) add_rmsnorm_bf16x8_kernel(float* __restrict__ h, const __nv_bfloat16* __restrict__ delta, const SplitDelta split,
                                          const float* __restrict__ weight, __nv_bfloat16* __restrict__ out, const int* __restrict__ rows,
                                          int hidden, float eps, int write_h) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* hrow = h + (size_t)s * hidden;
    const __nv_bfloat16* drow = delta + (size_t)s * hidden;
    float v[G][8], w[G][8];
    let_next_kernel_start();
#pragma unroll
    for (int g = 0; g < G; ++g) {  // the norm's weight is nobody's output: it is fetched while the kernel before still runs
        const int i = (threadIdx.x + g * blockDim.x) * 8;
        if (i < hidden) {
            const float4 a = *reinterpret_cast<const float4*>(weight + i), b = *reinterpret_cast<const float4*>(weight + i + 4);
            w[g][0] = a.x; w[g][1] = a.y; w[g][2] = a.z; w[g][3] = a.w; w[g][4] = b.x; w[g][5] = b.y; w[g][6] = b.z; w[g][7] = b.w;
        }
    }
    wait_for_previous_kernels();
    float sum = 0.f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const int i = (threadIdx.x + g * blockDim.x) * 8;
        if (i < hidden) {
            const float4 a = *reinterpret_cast<const float4*>(hrow + i), b = *reinterpret_cast<const float4*>(hrow + i + 4);
            uint4 d4;
            if (split.partials) {
                float d[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                const float* first = split.partials + (size_t)s * hidden + i;
                // Every piece is asked for before the first is added: a thread that loads four pieces, adds them and only
                // then loads the next four waits for memory once per group, and a step of a handful of rows is nothing but
                // such waits. The order of the additions stays the order of the splits.
                constexpr int PIECES_AHEAD = pieces_ahead(G);
                float4 p0[PIECES_AHEAD], p1[PIECES_AHEAD];
#pragma unroll
                for (int k = 0; k < PIECES_AHEAD; ++k) {
                    if (k < split.splits) {
                        p0[k] = *reinterpret_cast<const float4*>(first + k * split.split_stride);
                        p1[k] = *reinterpret_cast<const float4*>(first + k * split.split_stride + 4);
                    }
                }
#pragma unroll
                for (int k = 0; k < PIECES_AHEAD; ++k) {
                    if (k < split.splits) {
                        d[0] += p0[k].x; d[1] += p0[k].y; d[2] += p0[k].z; d[3] += p0[k].w;
                        d[4] += p1[k].x; d[5] += p1[k].y; d[6] += p1[k].z; d[7] += p1[k].w;
                    }
                }
                for (int k = PIECES_AHEAD; k < split.splits; ++k) {
                    const float4 q0 = *reinterpret_cast<const float4*>(first + k * split.split_stride);
                    const float4 q1 = *reinterpret_cast<const float4*>(first + k * split.split_stride + 4);
                    d[0] += q0.x; d[1] += q0.y; d[2] += q0.z; d[3] += q0.w; d[4] += q1.x; d[5] += q1.y; d[6] += q1.z; d[7] += q1.w;
                }
                __nv_bfloat162* packed = reinterpret_cast<__nv_bfloat162*>(&d4);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float b0 = split.bias_f ? split.bias_f[i + 2 * e] : (split.bias_h ? __bfloat162float(split.bias_h[i + 2 * e]) : 0.f);
                    const float b1 = split.bias_f ? split.bias_f[i + 2 * e + 1] : (split.bias_h ? __bfloat162float(split.bias_h[i + 2 * e + 1]) : 0.f);
                    packed[e] = __floats2bfloat162_rn(d[2 * e] + b0, d[2 * e + 1] + b1);
                }
            } else {
                d4 = *reinterpret_cast<const uint4*>(drow + i);
            }
            const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&d4);
            const float2 d0 = __bfloat1622float2(d2[0]), d1 = __bfloat1622float2(d2[1]), d2f = __bfloat1622float2(d2[2]), d3 = __bfloat1622float2(d2[3]);
            v[g][0] = a.x + d0.x; v[g][1] = a.y + d0.y; v[g][2] = a.z + d1.x; v[g][3] = a.w + d1.y;
            v[g][4] = b.x + d2f.x; v[g][5] = b.y + d2f.y; v[g][6] = b.z + d3.x; v[g][7] = b.w + d3.y;
            if (write_h) {
                *reinterpret_cast<float4*>(hrow + i) = make_float4(v[g][0], v[g][1], v[g][2], v[g][3]);
                *reinterpret_cast<float4*>(hrow + i + 4) = make_float4(v[g][4], v[g][5], v[g][6], v[g][7]);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) sum = fmaf(v[g][e], v[g][e], sum);
        }
    }
    const float total = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    __nv_bfloat16* orow = out + (size_t)r * hidden;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const int i = (threadIdx.x + g * blockDim.x) * 8;
        if (i < hidden) {
            uint4 o4;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
            for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(v[g][2 * e] * inv * w[g][2 * e], v[g][2 * e + 1] * inv * w[g][2 * e + 1]);
            *reinterpret_cast<uint4*>(orow + i) = o4;
        }
    }
}

static bool bf16x8_norm_takes(const void* h, const void* delta, const void* weight, const void* out, int hidden) {
    return hidden % 8 == 0 && hidden <= 16384 && (((uintptr_t)h | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out) & 15) == 0;
}

static int launch_bf16x8_norm(float* h, const __nv_bfloat16* delta, const SplitDelta& split, const float* weight, __nv_bfloat16* out, const int* rows,
                              int n_rows, int hidden, float eps, int write_h, cudaStream_t stream) {
    const int groups = hidden / 8;
    const int per_thread = groups > 1024 ? 4 : (groups > 512 ? 2 : 1);  // blocks of at most 512 threads: the kernel holds a row's pieces in registers
    const int width = ((groups + per_thread - 1) / per_thread + 31) / 32 * 32;
    if (per_thread == 1)
        return launch_after_previous(add_rmsnorm_bf16x8_kernel<1>, n_rows, width, 0, stream, h, delta, split, weight, out, rows, hidden, eps, write_h);
    if (per_thread == 2)
        return launch_after_previous(add_rmsnorm_bf16x8_kernel<2>, n_rows, width, 0, stream, h, delta, split, weight, out, rows, hidden, eps, write_h);
    return launch_after_previous(add_rmsnorm_bf16x8_kernel<4>, n_rows, width, 0, stream, h, delta, split, weight, out, rows, hidden, eps, write_h);
}

// The same with the delta still in pieces: partials [splits, tokens, hidden] floats (+ a bias) are added up in split order
// and rounded to bfloat16 before they join the residual stream. Refuses (HB_UNSUPPORTED_SIZE) what the 8-wide kernel cannot take.
HB_EXPORT int hb_add_rmsnorm_splits(float* h, const float* partials, int splits, int tokens, const float* bias_f, const void* bias_h,
                                    const float* weight, void* out, const int* rows, int n_rows, int hidden, float eps, int write_h,
                                    cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (!partials || splits < 1 || tokens < 1) return HB_BAD_ARGUMENT;
    if (!bf16x8_norm_takes(h, partials, weight, out, hidden)) return HB_UNSUPPORTED_SIZE;
    const SplitDelta split{partials, (size_t)tokens * hidden, splits, bias_f, (const __nv_bfloat16*)bias_h};
    return launch_bf16x8_norm(h, nullptr, split, weight, (__nv_bfloat16*)out, rows, n_rows, hidden, eps, write_h, stream);
}

HB_EXPORT int hb_add_rmsnorm(float* h, const void* delta, int delta_is_bf16, const float* weight, void* out,
                             int out_is_bf16, const int* rows, int n_rows, int hidden, float eps, int write_h,
                             cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (delta && delta_is_bf16 && out_is_bf16 && bf16x8_norm_takes(h, delta, weight, out, hidden))
        return launch_bf16x8_norm(h, (const __nv_bfloat16*)delta, SplitDelta{nullptr, 0, 0, nullptr, nullptr}, weight, (__nv_bfloat16*)out, rows, n_rows,
                                  hidden, eps, write_h, stream);
    const int threads = hidden >= 4096 ? 1024 : (hidden >= 1024 ? 512 : 256);
    int status = 0;
    const bool cached = hidden <= 8 * threads;  // both kernels add a thread's squares in the same order, so they agree bit for bit
#define HB_NORM(TD, TO)                                                                                                                    \
    if (cached) status = launch_after_previous(add_rmsnorm_cached_kernel<TD, TO>, n_rows, threads, 0, stream, h, (const TD*)delta, weight, (TO*)out, rows, hidden, eps, write_h); \
    else status = launch_after_previous(add_rmsnorm_kernel<TD, TO>, n_rows, threads, 0, stream, h, (const TD*)delta, weight, (TO*)out, rows, hidden, eps, write_h)
    if (delta_is_bf16) {
        if (out_is_bf16) { HB_NORM(__nv_bfloat16, __nv_bfloat16); } else { HB_NORM(__nv_bfloat16, float); }
    } else {
        if (out_is_bf16) { HB_NORM(float, __nv_bfloat16); } else { HB_NORM(float, float); }
    }
#undef HB_NORM
    return status;
}

// ---------------------------------------------------------------- SwiGLU
// in: [tokens, 2*inter]: gate and up columns alternate in blocks of `block` columns (block gate columns, then the block up
// columns that belong to them; block = inter is the plain arrangement, all gate columns first);
// out[t, i] = silu(gate_i) * up_i, silu(g) = g / (1 + exp(-g)) in float.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, int block) {
    const int t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= inter) return;
    const size_t at = (size_t)t * 2 * inter + (size_t)(i / block) * 2 * block + i % block;
    const float g = to_float(gate_up[at]);
    const float u = to_float(gate_up[at + block]);
    out[(size_t)t * inter + i] = from_float<T>(g / (1.0f + expf(-g)) * u);
}

// bfloat16 rows whose width and block are multiples of 8: 16-byte loads and stores, 8 elements per thread.
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out, int inter, int block) {
    const int t = blockIdx.y;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    let_next_kernel_start();
    wait_for_previous_kernels();
    if (i >= inter) return;
    const size_t at = (size_t)t * 2 * inter + (size_t)(i / block) * 2 * block + i % block;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gate_up + at);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gate_up + at + block);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
        o2[e] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * inter + i) = o4;
}

// block: columns per run of gate (and of up) columns; it divides inter (inter itself: all gate columns first).
HB_EXPORT int hb_swiglu(const void* gate_up, void* out, int is_bf16, int tokens, int inter, int block, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (tokens > 65535) return HB_UNSUPPORTED_SIZE;
    if (block <= 0 || inter % block) return HB_BAD_ARGUMENT;
    if (is_bf16 && inter % 8 == 0 && block % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0) {
        dim3 grid8((inter / 8 + 255) / 256, tokens);
        return launch_after_previous(swiglu_bf16x8_kernel, grid8, 256, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, block);
    }
    dim3 grid((inter + 255) / 256, tokens);
    if (is_bf16)
        swiglu_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, block);
    else
        swiglu_kernel<<<grid, 256, 0, stream>>>((const float*)gate_up, (float*)out, inter, block);
    return launch_status();
}

// ---------------------------------------------------------------- rotate-half position encoding
// Rotates `heads` consecutive heads of `head_dim` columns at the start of every row of `x` (row
// stride `stride` elements), in place: y[i] = x[i] c - x[i+d/2] s, y[i+d/2] = x[i+d/2] c + x[i] s
// with (c, s) = table[position][i]. The table holds cos and sin of position * base^(-2i/d).
template <typename T>
__global__ void rope_kernel(T* __restrict__ x, const int* __restrict__ positions, const float2* __restrict__ table,
                            int stride, int heads, int head_dim, int max_positions, int* status) {
    const int t = blockIdx.x;
    const int half = head_dim >> 1;
    const int pos = positions[t];
    if (pos < 0 || pos >= max_positions) {
        if (threadIdx.x == 0) atomicOr(status, HB_STATUS_BAD_POSITION);
        return;
    }
    T* row = x + (size_t)t * stride;
    const float2* cs = table + (size_t)pos * half;
    for (int e = threadIdx.x; e < heads * half; e += blockDim.x) {
        const int head = e / half, i = e - head * half;
        const float2 c = cs[i];
        T* p = row + head * head_dim + i;
        const float x1 = to_float(p[0]), x2 = to_float(p[half]);
        p[0] = from_float<T>(x1 * c.x - x2 * c.y);
        p[half] = from_float<T>(x2 * c.x + x1 * c.y);
    }
}

HB_EXPORT int hb_rope(void* x, int is_bf16, const int* positions, const float* table, int tokens, int stride, int heads,
                      int head_dim, int max_positions, int* status, cudaStream_t stream) {
    if (tokens <= 0 || heads <= 0) return 0;
    if (head_dim & 1) return HB_UNSUPPORTED_SIZE;
    if (is_bf16)
        rope_kernel<<<tokens, 256, 0, stream>>>((__nv_bfloat16*)x, positions, (const float2*)table, stride, heads, head_dim, max_positions, status);
    else
        rope_kernel<<<tokens, 256, 0, stream>>>((float*)x, positions, (const float2*)table, stride, heads, head_dim, max_positions, status);
    return launch_status();
}

// ---------------------------------------------------------------- key/value write into pages
// One cache layer is [pages, 2, kv_heads, page_size, head_dim]. Token t of row r = token_row[t] at
// position p goes to page block_table[r][p / page_size], slot p % page_size. A missing page sets
// the status word and the token is skipped.
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ src, int stride, int k_offset, int v_offset, T* __restrict__ cache,
                                const int* __restrict__ block_table, int table_width, const int* __restrict__ token_row,
                                const int* __restrict__ positions, int kv_heads, int head_dim, int page_size, int pages,
                                int* status) {
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int block = pos / page_size;
    const int page = (block < table_width && pos >= 0) ? block_table[(size_t)token_row[t] * table_width + block] : -1;
    if (page < 0 || page >= pages) {
        if (threadIdx.x == 0) atomicOr(status, HB_STATUS_BAD_PAGE);
        return;
    }
    const int slot = pos - block * page_size;
    const int width = kv_heads * head_dim;
    const T* row = src + (size_t)t * stride;
    const size_t page_base = (size_t)page * 2 * kv_heads * page_size * head_dim;
    for (int e = threadIdx.x; e < 2 * width; e += blockDim.x) {
        const int which = e / width, c = e - which * width;
        const int head = c / head_dim, d = c - head * head_dim;
        const T v = row[(which ? v_offset : k_offset) + c];
        cache[page_base + (((size_t)which * kv_heads + head) * page_size + slot) * head_dim + d] = v;
    }
}

// ---------------------------------------------------------------- rotation fused with the cache write
// One pass over a token's [q | k | v] row: the query heads are rotated in place, the key heads are
// rotated on their way into the cache (the row's own copy of k is left as it was: nothing reads it
// again), the value heads are copied.  Same arithmetic as rope_kernel followed by kv_store_kernel.
template <typename T>
__global__ void rope_kv_store_kernel(T* __restrict__ x, int stride, int q_heads, int kv_heads, int head_dim,
                                     const int* __restrict__ positions, const float2* __restrict__ table, int max_positions,
                                     T* __restrict__ cache, const int* __restrict__ block_table, int table_width,
                                     const int* __restrict__ token_row, int page_size, int pages, int* status) {
    const int t = blockIdx.x;
    const int half = head_dim >> 1;
    const int pos = positions[t];
    if (pos < 0 || pos >= max_positions) {
        if (threadIdx.x == 0) atomicOr(status, HB_STATUS_BAD_POSITION);
        return;
    }
    const int block = pos / page_size;
    const int page = block < table_width ? block_table[(size_t)token_row[t] * table_width + block] : -1;
    const bool page_ok = page >= 0 && page < pages;
    if (!page_ok && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, HB_STATUS_BAD_PAGE);
    const int slot = pos - block * page_size;
    T* row = x + (size_t)t * stride;
    const float2* cs = table + (size_t)pos * half;
    const size_t page_base = (size_t)(page_ok ? page : 0) * 2 * kv_heads * page_size * head_dim;
    const int rotated = (q_heads + kv_heads) * half;
    // blockIdx.y cuts a token's work into slices of blockDim.x element pairs, so that a decode step of a few tokens
    // still spreads over many blocks
    for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < rotated + kv_heads * half; e += gridDim.y * blockDim.x) {
        if (e < rotated) {
            const int head = e / half, i = e - head * half;
            const float2 c = cs[i];
            T* p = row + head * head_dim + i;
            const float x1 = to_float(p[0]), x2 = to_float(p[half]);
            const T y1 = from_float<T>(x1 * c.x - x2 * c.y), y2 = from_float<T>(x2 * c.x + x1 * c.y);
            if (head < q_heads) {
                p[0] = y1; p[half] = y2;
            } else if (page_ok) {
                T* dst = cache + page_base + (((size_t)(head - q_heads)) * page_size + slot) * head_dim + i;
                dst[0] = y1; dst[half] = y2;
            }
        } else if (page_ok) {  // values: two elements per thread
            const int f = e - rotated, head = f / half, i = (f - head * half) * 2;
            const T* p = row + (q_heads + kv_heads + head) * head_dim + i;
            T* dst = cache + page_base + (((size_t)(kv_heads + head)) * page_size + slot) * head_dim + i;
            dst[0] = p[0]; dst[1] = p[1];
        }
    }
}

// bfloat16 with head sizes that are multiples of 16: every thread rotates 8 consecutive pairs (two 16-byte loads, two
// 16-byte stores) or copies 8 values; same arithmetic per element as the scalar kernel.
__global__ void rope_kv_store_bf16x8_kernel(__nv_bfloat16* __restrict__ x, int stride, int q_heads, int kv_heads, int head_dim,
                                            const int* __restrict__ positions, const float2* __restrict__ table, int max_positions,
                                            __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table, int table_width,
                                            const int* __restrict__ token_row, int page_size, int pages, int* status) {
    const int t = blockIdx.x;
    const int half = head_dim >> 1, chunks = half >> 3;  // 8-pair chunks per head
    let_next_kernel_start();
    const int pos = positions[t];  // positions and tables come with the step's one copy from the host, not from a kernel
    const bool pos_ok = pos >= 0 && pos < max_positions;
    const int block = pos_ok ? pos / page_size : 0;
    const int page = pos_ok && block < table_width ? block_table[(size_t)token_row[t] * table_width + block] : -1;
    wait_for_previous_kernels();
    if (!pos_ok) {
        if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, HB_STATUS_BAD_POSITION);
        return;
    }
    const bool page_ok = page >= 0 && page < pages;
    if (!page_ok && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, HB_STATUS_BAD_PAGE);
    const int slot = pos - block * page_size;
    __nv_bfloat16* row = x + (size_t)t * stride;
    const float2* cs = table + (size_t)pos * half;
    const size_t page_base = (size_t)(page_ok ? page : 0) * 2 * kv_heads * page_size * head_dim;
    const int rotated = (q_heads + kv_heads) * chunks;
    const int total = rotated + kv_heads * 2 * chunks;  // values: head_dim / 8 chunks per head
    for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < total; e += gridDim.y * blockDim.x) {
        if (e < rotated) {
            const int head = e / chunks, i = (e - head * chunks) * 8;
            __nv_bfloat16* p = row + head * head_dim + i;
            const uint4 lo4 = *reinterpret_cast<const uint4*>(p), hi4 = *reinterpret_cast<const uint4*>(p + half);
            const __nv_bfloat16* lo = reinterpret_cast<const __nv_bfloat16*>(&lo4);
            const __nv_bfloat16* hi = reinterpret_cast<const __nv_bfloat16*>(&hi4);
            uint4 out_lo, out_hi;
            __nv_bfloat16* y1 = reinterpret_cast<__nv_bfloat16*>(&out_lo);
            __nv_bfloat16* y2 = reinterpret_cast<__nv_bfloat16*>(&out_hi);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float2 c = cs[i + j];
                const float x1 = __bfloat162float(lo[j]), x2 = __bfloat162float(hi[j]);
                y1[j] = __float2bfloat16_rn(x1 * c.x - x2 * c.y);
                y2[j] = __float2bfloat16_rn(x2 * c.x + x1 * c.y);
            }
            if (head < q_heads) {
                *reinterpret_cast<uint4*>(p) = out_lo;
                *reinterpret_cast<uint4*>(p + half) = out_hi;
            } else if (page_ok) {
                __nv_bfloat16* dst = cache + page_base + (((size_t)(head - q_heads)) * page_size + slot) * head_dim + i;
                *reinterpret_cast<uint4*>(dst) = out_lo;
                *reinterpret_cast<uint4*>(dst + half) = out_hi;
            }
        } else if (page_ok) {
            const int f = e - rotated, head = f / (2 * chunks), i = (f - head * 2 * chunks) * 8;
            const uint4 v = *reinterpret_cast<const uint4*>(row + (q_heads + kv_heads + head) * head_dim + i);
            *reinterpret_cast<uint4*>(cache + page_base + (((size_t)(kv_heads + head)) * page_size + slot) * head_dim + i) = v;
        }
    }
}

HB_EXPORT int hb_rope_kv_store(void* x, int is_bf16, int tokens, int stride, int q_heads, int kv_heads, int head_dim,
                               const int* positions, const float* table, int max_positions, void* cache, const int* block_table,
                               int table_width, const int* token_row, int page_size, int pages, int* status, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (head_dim & 1) return HB_UNSUPPORTED_SIZE;
    if (is_bf16 && head_dim % 16 == 0 && stride % 8 == 0 && (((uintptr_t)x | (uintptr_t)cache) & 15) == 0) {
        const int items = (q_heads + 2 * kv_heads) * (head_dim / 16);
        const int threads = items >= 256 ? 256 : 128;
        const dim3 grid8(tokens, tokens >= 512 ? 1 : min(8, (items + threads - 1) / threads));
        return launch_after_previous(rope_kv_store_bf16x8_kernel, grid8, threads, 0, stream, (__nv_bfloat16*)x, stride, q_heads, kv_heads, head_dim,
                                     positions, (const float2*)table, max_positions, (__nv_bfloat16*)cache, block_table, table_width, token_row,
                                     page_size, pages, status);
    }
    const int pairs = (q_heads + 2 * kv_heads) * (head_dim / 2);
    const int slices = tokens >= 512 ? 1 : min(16, (pairs + 255) / 256);
    const dim3 grid(tokens, slices);
    if (is_bf16)
        rope_kv_store_kernel<<<grid, 256, 0, stream>>>((__nv_bfloat16*)x, stride, q_heads, kv_heads, head_dim, positions, (const float2*)table,
                                                       max_positions, (__nv_bfloat16*)cache, block_table, table_width, token_row, page_size, pages, status);
    else
        rope_kv_store_kernel<<<grid, 256, 0, stream>>>((float*)x, stride, q_heads, kv_heads, head_dim, positions, (const float2*)table,
                                                       max_positions, (float*)cache, block_table, table_width, token_row, page_size, pages, status);
    return launch_status();
}

HB_EXPORT int hb_kv_store(const void* src, int is_bf16, int tokens, int stride, int k_offset, int v_offset, void* cache,
                          const int* block_table, int table_width, const int* token_row, const int* positions,
                          int kv_heads, int head_dim, int page_size, int pages, int* status, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (is_bf16)
        kv_store_kernel<<<tokens, 256, 0, stream>>>((const __nv_bfloat16*)src, stride, k_offset, v_offset, (__nv_bfloat16*)cache,
                                                    block_table, table_width, token_row, positions, kv_heads, head_dim, page_size, pages, status);
    else
        kv_store_kernel<<<tokens, 256, 0, stream>>>((const float*)src, stride, k_offset, v_offset, (float*)cache, block_table,
                                                    table_width, token_row, positions, kv_heads, head_dim, page_size, pages, status);
    return launch_status();
}
