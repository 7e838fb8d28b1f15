// Token choice on the device: argmax (temperature 0) and sampling with repetition penalty,
// temperature, top-k, top-p and a counter-based random draw, one block per row of float logits.
//
// The options and their order are the reference's sampler (penalty, then temperature, then the top-k
// set ordered by value descending with ties to the lower index, then the nucleus over that set, then a
// Philox4x32-10 draw keyed by the request's seed with the number of tokens sampled so far as the
// counter: helios/crates/helios-hal/src/sampler_reference.rs:4-26; argmax takes the lowest index on
// ties and never a NaN: helios/crates/helios-hal/kernels/elementwise.cu:948-1004).  The method differs:
// instead of sorting candidates, the k-th largest value and the nucleus boundary are found by
// bisection over the ordered bit patterns of the adjusted logits, each probe one pass over the row
// with sums taken in a fixed order, so a row's token depends only on its own logits and options.
#include "common.cuh"

namespace {
constexpr int THREADS = 1024;

struct RowOptions {
    float temperature, top_p, penalty;
    int top_k;
    unsigned seed_lo, seed_hi, counter;
    int slot;
};

// Philox4x32 with 10 rounds (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC11).
__device__ __forceinline__ unsigned philox_first_word(unsigned c0, unsigned k0, unsigned k1) {
    unsigned c[4] = {c0, 0u, 0u, 0u};
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        const unsigned long long p0 = 0xD2511F53ull * c[0], p1 = 0xCD9E8D57ull * c[2];
        const unsigned n0 = (unsigned)(p1 >> 32) ^ c[1] ^ k0, n1 = (unsigned)p1;
        const unsigned n2 = (unsigned)(p0 >> 32) ^ c[3] ^ k1, n3 = (unsigned)p0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    return c[0];
}

// A float's bits mapped so that unsigned comparison orders like the floats; NaN maps below everything.
__device__ __forceinline__ unsigned ordered_key(float v) {
    if (v != v) return 0u;
    const unsigned bits = __float_as_uint(v);
    return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

__device__ __forceinline__ float adjusted(const float* logits, const unsigned* seen, int i, float penalty, float divisor) {
    float z = logits[i];
    if (seen && penalty != 1.0f && ((seen[i >> 5] >> (i & 31)) & 1u)) z = z > 0.f ? z / penalty : z * penalty;
    return z / divisor;
}

__device__ __forceinline__ int block_sum_int(int v, int* scratch) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    int total = 0;
    for (int w = 0; w < THREADS / 32; ++w) total += scratch[w];
    return total;
}

__global__ void __launch_bounds__(THREADS) sample_kernel(const float* __restrict__ logits, int row_stride, int vocab,
                                                         const int* __restrict__ options_raw, unsigned* __restrict__ seen_all,
                                                         int seen_words, int* __restrict__ tokens) {
    __shared__ float fscratch[32];
    __shared__ int iscratch[32];
    __shared__ float best_value[32];
    __shared__ int best_index[32];
    __shared__ int winner;
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* z_row = logits + (size_t)row * row_stride;
    RowOptions o;
    {
        const int* r = options_raw + row * 8;
        o.temperature = __int_as_float(r[0]); o.top_p = __int_as_float(r[1]); o.penalty = __int_as_float(r[2]);
        o.top_k = r[3]; o.seed_lo = (unsigned)r[4]; o.seed_hi = (unsigned)r[5]; o.counter = (unsigned)r[6]; o.slot = r[7];
    }
    unsigned* seen = (seen_all && o.slot >= 0) ? seen_all + (size_t)o.slot * seen_words : nullptr;
    const bool greedy = !(o.temperature > 0.f);
    const float divisor = greedy ? 1.0f : o.temperature;
    const float penalty = greedy ? 1.0f : o.penalty;

    // ---- maximum with the lowest index on ties; NaN never wins
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < vocab; i += THREADS) {
        const float z = adjusted(z_row, seen, i, penalty, divisor);
        if (z > bv || (bi == 0x7fffffff && z == z)) { bv = z; bi = i; }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, offset);
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    if ((tid & 31) == 0) { best_value[tid >> 5] = bv; best_index[tid >> 5] = bi; }
    __syncthreads();
    bv = best_value[0]; bi = best_index[0];
    for (int w = 1; w < THREADS / 32; ++w) {
        const float ov = best_value[w];
        const int oi = best_index[w];
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    if (bi == 0x7fffffff) bi = 0;  // a row of NaN only
    if (greedy) {
        if (tid == 0) {
            tokens[row] = bi;
            if (seen) atomicOr(&seen[bi >> 5], 1u << (bi & 31));
        }
        return;
    }
    const float zmax = bv;

    // ---- top-k: the k-th largest key by bisection, then how many ties at it are kept (lowest indices)
    unsigned key_floor = 0u;      // keys above this are kept whole
    int tie_limit = 0x7fffffff;   // among keys equal to key_floor, indices up to this are kept
    bool limited = false;
    const int k = (o.top_k > 0 && o.top_k < vocab) ? o.top_k : 0;
    if (k) {
        unsigned lo = 0u, hi = 0xffffffffu;  // largest K with count(key >= K) >= k
        while (lo < hi) {
            const unsigned mid = lo + (unsigned)(((unsigned long long)hi - lo + 1ull) >> 1);
            int count = 0;
            for (int i = tid; i < vocab; i += THREADS) count += ordered_key(adjusted(z_row, seen, i, penalty, divisor)) >= mid;
            if (block_sum_int(count, iscratch) >= k) lo = mid; else hi = mid - 1u;
        }
        key_floor = lo;
        int above = 0;
        for (int i = tid; i < vocab; i += THREADS) above += ordered_key(adjusted(z_row, seen, i, penalty, divisor)) > key_floor;
        const int ties_kept = k - block_sum_int(above, iscratch);
        int a = 0, b = vocab - 1;  // smallest c with count(key == floor, i <= c) >= ties_kept
        while (a < b) {
            const int mid = (a + b) >> 1;
            int count = 0;
            for (int i = tid; i <= mid; i += THREADS) count += ordered_key(adjusted(z_row, seen, i, penalty, divisor)) == key_floor;
            if (block_sum_int(count, iscratch) >= ties_kept) b = mid; else a = mid + 1;
        }
        tie_limit = a;
        limited = true;
    }
#define HB_KEPT(key, i) (!limited || (key) > key_floor || ((key) == key_floor && (i) <= tie_limit))

    // ---- mass of the kept set
    float part = 0.f;
    for (int i = tid; i < vocab; i += THREADS) {
        const float z = adjusted(z_row, seen, i, penalty, divisor);
        const unsigned key = ordered_key(z);
        if (key != 0u && HB_KEPT(key, i)) part += expf(z - zmax);
    }
    float mass = block_sum(part, fscratch);

    // ---- top-p: the smallest prefix (by value descending, ties to the lower index) whose mass reaches top_p * mass
    if (o.top_p < 1.0f) {
        const float need = o.top_p * mass;
        unsigned lo = 0u, hi = 0xffffffffu;  // largest K with mass(kept, key >= K) >= need
        while (lo < hi) {
            const unsigned mid = lo + (unsigned)(((unsigned long long)hi - lo + 1ull) >> 1);
            float p = 0.f;
            for (int i = tid; i < vocab; i += THREADS) {
                const float z = adjusted(z_row, seen, i, penalty, divisor);
                const unsigned key = ordered_key(z);
                if (key != 0u && key >= mid && HB_KEPT(key, i)) p += expf(z - zmax);
            }
            if (block_sum(p, fscratch) >= need) lo = mid; else hi = mid - 1u;
        }
        const unsigned nucleus_floor = lo;
        float p = 0.f;
        int ties = 0;
        float tie_weight = 0.f;
        for (int i = tid; i < vocab; i += THREADS) {
            const float z = adjusted(z_row, seen, i, penalty, divisor);
            const unsigned key = ordered_key(z);
            if (key == 0u || !HB_KEPT(key, i)) continue;
            if (key > nucleus_floor) p += expf(z - zmax);
            else if (key == nucleus_floor) { ties += 1; tie_weight = expf(z - zmax); }
        }
        const float above = block_sum(p, fscratch);
        const int n_ties = block_sum_int(ties, iscratch);
        const float w = block_max(tie_weight, fscratch);
        int ties_kept = w > 0.f ? (int)ceilf((need - above) / w) : n_ties;
        ties_kept = max(1, min(n_ties, ties_kept));
        int a = 0, b = vocab - 1;
        while (a < b) {
            const int mid = (a + b) >> 1;
            int count = 0;
            for (int i = tid; i <= mid; i += THREADS) {
                const unsigned key = ordered_key(adjusted(z_row, seen, i, penalty, divisor));
                count += key == nucleus_floor && HB_KEPT(key, i);
            }
            if (block_sum_int(count, iscratch) >= ties_kept) b = mid; else a = mid + 1;
        }
        key_floor = nucleus_floor;
        tie_limit = a;
        limited = true;
        mass = above + (float)ties_kept * w;
    }

    // ---- the draw: walk the kept tokens in index order until the running mass passes u * mass
    const float u = (float)(philox_first_word(o.counter, o.seed_lo, o.seed_hi) >> 8) * (1.0f / 16777216.0f);
    const int chunk = (vocab + THREADS - 1) / THREADS;
    const int begin = min(vocab, tid * chunk), end = min(vocab, begin + chunk);
    float mine = 0.f;
    int last_kept = -1;
    for (int i = begin; i < end; ++i) {
        const float z = adjusted(z_row, seen, i, penalty, divisor);
        const unsigned key = ordered_key(z);
        if (key != 0u && HB_KEPT(key, i)) { mine += expf(z - zmax); last_kept = i; }
    }
    // exclusive prefix over threads: inclusive scan inside the warp, then the warps in order
    float inclusive = mine;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
        const float other = __shfl_up_sync(0xffffffffu, inclusive, offset);
        if ((tid & 31) >= offset) inclusive += other;
    }
    __syncthreads();
    if ((tid & 31) == 31) fscratch[tid >> 5] = inclusive;
    if (tid == 0) winner = 0x7fffffff;
    __syncthreads();
    float base = 0.f;
    for (int w = 0; w < (tid >> 5); ++w) base += fscratch[w];
    float total = 0.f;
    for (int w = 0; w < THREADS / 32; ++w) total += fscratch[w];
    const float target = u * total;
    const float before = base + inclusive - mine;
    if (mine > 0.f && before + mine > target) atomicMin(&winner, tid);
    __syncthreads();
    int fallback = last_kept;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) fallback = max(fallback, __shfl_xor_sync(0xffffffffu, fallback, offset));
    __syncthreads();
    if ((tid & 31) == 0) iscratch[tid >> 5] = fallback;
    __syncthreads();
    if (tid == (winner == 0x7fffffff ? 0 : winner)) {
        int token = -1;
        if (winner != 0x7fffffff) {
            float running = before;
            for (int i = begin; i < end; ++i) {
                const float z = adjusted(z_row, seen, i, penalty, divisor);
                const unsigned key = ordered_key(z);
                if (key != 0u && HB_KEPT(key, i)) {
                    running += expf(z - zmax);
                    token = i;
                    if (running > target) break;
                }
            }
        } else {
            for (int w = 0; w < THREADS / 32; ++w) token = max(token, iscratch[w]);
            if (token < 0) token = bi;
        }
        tokens[row] = token;
        if (seen) atomicOr(&seen[token >> 5], 1u << (token & 31));
    }
#undef HB_KEPT
}


// Argmax of every row in two launches (for steps in which every row is greedy): `chunks` blocks per row find the best
// of their slice, then one warp per row picks among them; lowest index on ties, NaN never wins.
__global__ void argmax_partial_kernel(const float* __restrict__ logits, int row_stride, int vocab, int chunks, float* __restrict__ best_value,
                                      int* __restrict__ best_index) {
    __shared__ float sv[8];
    __shared__ int si[8];
    const int row = blockIdx.x, chunk = blockIdx.y;
    const int per = (vocab + chunks - 1) / chunks;
    const int begin = chunk * per, end = min(vocab, begin + per);
    const float* z = logits + (size_t)row * row_stride;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    let_next_kernel_start();
    wait_for_previous_kernels();
    // the body in 16-byte loads where the row allows it; a thread keeps the lowest index among equal values because
    // it walks its indices upwards and takes a later value only when it is larger
    const bool wide = ((((uintptr_t)z) & 15) == 0) && (begin % 4 == 0);
    const int body_end = wide ? begin + ((end - begin) / 4) * 4 : begin;
    for (int i = begin + threadIdx.x * 4; i < body_end; i += blockDim.x * 4) {
        const float4 v4 = *reinterpret_cast<const float4*>(z + i);
        const float v[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
            if (v[e] > bv || (bi == 0x7fffffff && v[e] == v[e])) { bv = v[e]; bi = i + e; }
    }
    for (int i = body_end + threadIdx.x; i < end; i += blockDim.x) {
        const float v = z[i];
        if (v > bv || (bi == 0x7fffffff && v == v) || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, offset);
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (si[w] != 0x7fffffff && (bi == 0x7fffffff || sv[w] > bv || (sv[w] == bv && si[w] < bi))) { bv = sv[w]; bi = si[w]; }
        best_value[row * chunks + chunk] = bv;
        best_index[row * chunks + chunk] = bi;
    }
}

__global__ void argmax_final_kernel(const float* __restrict__ best_value, const int* __restrict__ best_index, int chunks,
                                    const int* __restrict__ options_raw, unsigned* __restrict__ seen_all, int seen_words, int* __restrict__ tokens) {
    const int row = blockIdx.x;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    wait_for_previous_kernels();
    for (int c = threadIdx.x; c < chunks; c += 32) {
        const float ov = best_value[row * chunks + c];
        const int oi = best_index[row * chunks + c];
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, offset);
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    if (threadIdx.x == 0) {
        if (bi == 0x7fffffff) bi = 0;
        tokens[row] = bi;
        const int slot = options_raw[row * 8 + 7];
        if (seen_all && slot >= 0) atomicOr(&seen_all[(size_t)slot * seen_words + (bi >> 5)], 1u << (bi & 31));
    }
}
}  // namespace

// workspace: 2 * rows * chunks words (values then indices).
HB_EXPORT int hb_argmax(const float* logits, int row_stride, int rows, int vocab, int chunks, void* workspace, const int* options,
                        unsigned* seen, int seen_words, int* tokens, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || chunks < 1 || chunks > 1024 || !workspace) return HB_BAD_ARGUMENT;
    float* values = reinterpret_cast<float*>(workspace);
    int* indices = reinterpret_cast<int*>(workspace) + (size_t)rows * chunks;
    int code = launch_after_previous(argmax_partial_kernel, dim3(rows, chunks), 256, 0, stream, logits, row_stride, vocab, chunks, values, indices);
    if (code) return code;
    return launch_after_previous(argmax_final_kernel, rows, 32, 0, stream, (const float*)values, (const int*)indices, chunks, options, seen, seen_words, tokens);
}

namespace {
}  // namespace

// options: 8 int32 words per row: temperature, top_p, repetition penalty (float bits), top_k, seed low,
// seed high, draw counter, state slot (-1: no record of generated tokens). seen: [slots, seen_words]
// bitmaps of the tokens each request generated, updated with the token chosen.
HB_EXPORT int hb_sample(const float* logits, int row_stride, int rows, int vocab, const int* options, unsigned* seen,
                        int seen_words, int* tokens, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return HB_BAD_ARGUMENT;
    sample_kernel<<<rows, THREADS, 0, stream>>>(logits, row_stride, vocab, options, seen, seen_words, tokens);
    return launch_status();
}
