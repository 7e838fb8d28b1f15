// Token choice on the device: argmax (temperature 0) and sampling with repetition penalty,
// temperature, top-k, top-p and a counter-based random draw, one block per row of float logits.
//
// The options and their order are the reference's sampler (penalty, then temperature, then the top-k
// set ordered by value descending with ties to the lower index, then the nucleus over that set, then a
// Philox4x32-10 draw keyed by the request's seed with the number of tokens sampled so far as the
// counter: helios/crates/helios-hal/src/sampler_reference.rs:4-26; argmax takes the lowest index on
// ties and never a NaN: helios/crates/helios-hal/kernels/elementwise.cu:948-1004).  The method differs:
// instead of sorting candidates, the k-th largest value and the nucleus boundary are found by a
// radix search over the ordered bit patterns of the adjusted logits (histograms of eleven bits at a
// time, masses as fixed-point integers), so a row's token depends only on its own logits and options.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

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

// ---------------------------------------------------------------------------------------------------------------------
// Selection by radix instead of bisection: the k-th largest key, and the key at which the mass of the larger keys
// reaches top_p of the whole, are found eleven bits at a time from histograms in shared memory (three passes over the
// row instead of thirty-two). Counts are integers; masses are summed as 40-bit fixed point (exp(z - max) * 2^40 as an
// integer), so a histogram's sums do not depend on the order in which threads add to it and a row's token depends
// only on its own logits and options.
//
// A row of a large vocabulary is shared by the TEAM blocks of a thread-block cluster: each takes a slice of the row,
// builds its own histograms, and reads the others' through distributed shared memory; every block then takes the same
// decisions from the same sums, so nothing has to be sent back.
constexpr int BINS = 2048;
constexpr int LIST = 1024;  // a top-k set of up to this many tokens is copied out of the row; everything after works on the copy
constexpr int TEAM = 8;
constexpr int TEAM_FROM_VOCAB = 8192;  // smaller rows are one block's work

struct Scratch {
    unsigned hist_lo[BINS];          // weight per bin (count or fixed-point mass), low word and high word: two 32-bit adds
    unsigned hist_hi[BINS];          // with a carry were measured a third faster here than one 64-bit add to shared memory
    int count[BINS];                 // elements per bin (kept for the last level of a mass search only)
    unsigned long long warp_total[THREADS / 32];
    float fscratch[32];
    int iscratch[32];
    int raw_index[LIST];
    float raw_z[LIST];
    int list_index[LIST];
    float list_z[LIST];
    int chosen_bin;
    unsigned long long chosen_above;
    int n_list;
    int winner;
    // what a block shows its team
    float team_float;
    int team_int;
    int team_winner;
    int team_fallback;
};

// The blocks that share a row. With one block nothing of the cluster is touched.
struct Team {
    int size, rank;
    __device__ __forceinline__ void sync() const {
        if (size > 1) cg::this_cluster().sync(); else __syncthreads();
    }
    template <class T>
    __device__ __forceinline__ T* peer(T* mine, int r) const {
        return size > 1 ? cg::this_cluster().map_shared_rank(mine, r) : mine;
    }
    __device__ __forceinline__ int sum(int block_total, Scratch& s) const {
        if (size == 1) return block_total;
        if (threadIdx.x == 0) s.team_int = block_total;
        sync();
        int total = 0;
        for (int r = 0; r < size; ++r) total += *peer(&s.team_int, r);
        sync();
        return total;
    }
};

// Which tokens are still in the race: keys above the floor, and of the keys at the floor the lowest indices.
struct Limits {
    bool limited;
    unsigned key_floor;
    int tie_limit;
    __device__ __forceinline__ bool kept(unsigned key, int i) const {
        return !limited || key > key_floor || (key == key_floor && i <= tie_limit);
    }
};

// This block's slice [first, last) of the row as it lies in memory: element j is token j, its logit adjusted by
// penalty and temperature.
struct RowView {
    const float* z_row;
    const unsigned* seen;
    float penalty, divisor;
    int first, last;
    __device__ __forceinline__ void get(int j, float& z, int& i) const { i = j; z = adjusted(z_row, seen, j, penalty, divisor); }
};

// A short list of (token, adjusted logit) in shared memory, ordered by token.
struct ListView {
    const float* z_list;
    const int* index_list;
    int first, last;
    __device__ __forceinline__ void get(int j, float& z, int& i) const { i = index_list[j]; z = z_list[j]; }
};

__device__ __forceinline__ unsigned long long fixed_weight(float z, float zmax) {
    return __float2ull_rn(expf(z - zmax) * 1099511627776.0f);  // 2^40; z <= zmax, so at most 2^40
}

// Inclusive scan over the block's threads in thread order; total = the sum over all threads.
__device__ __forceinline__ unsigned long long block_scan(unsigned long long v, Scratch& s, unsigned long long& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
        const unsigned long long other = __shfl_up_sync(0xffffffffu, v, offset);
        if (lane >= offset) v += other;
    }
    __syncthreads();
    if (lane == 31) s.warp_total[warp] = v;
    __syncthreads();
    unsigned long long base = 0;
    total = 0;
    for (int w = 0; w < THREADS / 32; ++w) {
        const unsigned long long t = s.warp_total[w];
        if (w < warp) base += t;
        total += t;
    }
    return v + base;
}

// Bin b's weight in block r of the team.
__device__ __forceinline__ unsigned long long bin_weight(const Team& team, Scratch& s, int r, int b) {
    return ((unsigned long long)team.peer(s.hist_hi, r)[b] << 32) + team.peer(s.hist_lo, r)[b];
}

struct Selected {
    unsigned key;                 // the largest key K with weight(kept, key >= K) >= need
    unsigned long long need;      // what had to be reached
    unsigned long long above;     // weight(kept, key > K)
    unsigned long long at;        // weight(kept, key == K)
    int n_at;                     // how many kept elements have key K
};

// MASS: weights are fixed-point masses, NaN is left out, need = fraction * total (at least 1 unit).
// else: weights are 1 (NaN counts, with the lowest key), need = count_needed.
// first_level_ready: the histogram of the first level stands already (the caller built it on an earlier pass).
// levels: 3 for the exact key; 1 stops after the first eleven bits (key = those bits, at = the weight of their bin)
// and leaves the histogram standing.
template <bool MASS, class View>
__device__ Selected radix_select(const View& view, const Team& team, const Limits& lim, float zmax, float fraction, int count_needed, Scratch& s,
                                 bool first_level_ready = false, int levels = 3) {
    const int tid = threadIdx.x;
    unsigned prefix = 0u;
    unsigned long long above = 0, need = MASS ? 0ull : (unsigned long long)count_needed;
    int decided_from = 32;  // bits [decided_from, 32) of the key are fixed
    int bin = 0;
    for (int level = 0; level < levels; ++level) {
        const int width = level == 2 ? 10 : 11;
        const int shift = decided_from - width;
        const int bins = 1 << width;
        const bool ready = level == 0 && first_level_ready;
        if (!ready)
            for (int b = tid; b < BINS; b += THREADS) { s.hist_lo[b] = 0u; s.hist_hi[b] = 0u; s.count[b] = 0; }
        if (tid == 0) s.chosen_bin = -1;
        __syncthreads();
        for (int j = view.first + tid; j < view.last && !ready; j += THREADS) {
            float z; int i;
            view.get(j, z, i);
            const unsigned key = ordered_key(z);
            if (MASS && key == 0u) continue;
            if (!lim.kept(key, i)) continue;
            if (level > 0 && (key >> decided_from) != (prefix >> decided_from)) continue;
            const unsigned b = (key >> shift) & (unsigned)(bins - 1);
            const unsigned long long w = MASS ? fixed_weight(z, zmax) : 1ull;
            if (w) {
                // the low word wraps exactly floor(sum / 2^32) times whatever the order of the adds; each wrap is seen by
                // the add that caused it and carried into the high word
                const unsigned w_lo = (unsigned)w, w_hi = (unsigned)(w >> 32);
                const unsigned old = atomicAdd(&s.hist_lo[b], w_lo);
                const unsigned up = w_hi + ((unsigned)(old + w_lo) < old ? 1u : 0u);
                if (up) atomicAdd(&s.hist_hi[b], up);
            }
            if (MASS && level == 2) atomicAdd(&s.count[b], 1);  // how many share the last level's key; counts are the weights otherwise
        }
        team.sync();  // every block's histogram is complete
        // thread t looks at bins (bins - 1 - 2t) and (bins - 2 - 2t): the scan runs from the largest keys down
        unsigned long long h0 = 0, h1 = 0;
        if (2 * tid < bins) {
            for (int r = 0; r < team.size; ++r) {
                h0 += bin_weight(team, s, r, bins - 1 - 2 * tid);
                h1 += bin_weight(team, s, r, bins - 2 - 2 * tid);
            }
        }
        unsigned long long total;
        const unsigned long long inclusive = block_scan(h0 + h1, s, total);
        if (level == 0 && MASS) {
            need = (unsigned long long)((double)fraction * (double)total);
            if (need < 1ull) need = 1ull;
            if (need > total) need = total;
        }
        const unsigned long long want = need - above;  // what this level's bins must still bring
        const unsigned long long before = inclusive - (h0 + h1);
        if (2 * tid < bins && before < want && want <= inclusive) {
            if (before + h0 >= want) { s.chosen_bin = bins - 1 - 2 * tid; s.chosen_above = before; }
            else { s.chosen_bin = bins - 2 - 2 * tid; s.chosen_above = before + h0; }
        }
        __syncthreads();
        if (s.chosen_bin < 0) {
            // the bins do not reach what is wanted (nothing kept at all): the lowest bin that holds anything, else bin 0
            if (tid == 0) {
                int lowest = 0;
                unsigned long long sum = 0;
                for (int b = bins - 1; b >= 0; --b) {
                    unsigned long long h = 0;
                    for (int r = 0; r < team.size; ++r) h += bin_weight(team, s, r, b);
                    if (h > 0ull) { lowest = b; }
                }
                for (int b = bins - 1; b > lowest; --b)
                    for (int r = 0; r < team.size; ++r) sum += bin_weight(team, s, r, b);
                s.chosen_above = sum;
                s.chosen_bin = lowest;
            }
            __syncthreads();
        }
        bin = s.chosen_bin;
        above += s.chosen_above;
        prefix |= (unsigned)bin << shift;
        decided_from = shift;
        if (level + 1 < levels) team.sync();  // nobody reads these histograms any more: the next level may clear them
    }
    Selected r;
    r.key = prefix; r.need = need; r.above = above; r.at = 0ull; r.n_at = 0;
    for (int t = 0; t < team.size; ++t) {
        r.at += bin_weight(team, s, t, bin);
        r.n_at += team.peer(s.count, t)[bin];
    }
    if (!MASS) r.n_at = (int)r.at;
    team.sync();  // the histograms may be cleared by whoever comes next
    return r;
}

// Smallest index c such that `wanted` kept elements with this key have an index <= c (bisection over the index; only
// needed when ties at the floor are cut, which equal logits alone bring about).
template <class View>
__device__ int tie_index(const View& view, const Team& team, const Limits& lim, unsigned key_at, int wanted, int vocab, Scratch& s) {
    int a = 0, b = vocab - 1;
    while (a < b) {
        const int mid = (a + b) >> 1;
        int count = 0;
        for (int j = view.first + threadIdx.x; j < view.last; j += THREADS) {
            float z; int i;
            view.get(j, z, i);
            const unsigned key = ordered_key(z);
            count += i <= mid && key == key_at && lim.kept(key, i);
        }
        if (team.sum(block_sum_int(count, s.iscratch), s) >= wanted) b = mid; else a = mid + 1;
    }
    return a;
}

// Copies the tokens `lim` keeps out of the row: every block its own, the first block then takes them all and orders
// them by token into the list. Returns their number; only the first block may go on with the list (the others are
// done once this returns). No more than LIST tokens may be kept.
__device__ int copy_out(const RowView& slice, const Team& team, const Limits& lim, Scratch& s) {
    const int tid = threadIdx.x;
    if (tid == 0) s.n_list = 0;
    __syncthreads();
    for (int i = slice.first + tid; i < slice.last; i += THREADS) {
        const float z = adjusted(slice.z_row, slice.seen, i, slice.penalty, slice.divisor);
        if (lim.kept(ordered_key(z), i)) {
            const int at = atomicAdd(&s.n_list, 1);
            if (at < LIST) { s.raw_index[at] = i; s.raw_z[at] = z; }
        }
    }
    team.sync();
    int n = min(s.n_list, LIST);
    if (team.rank == 0) {
        for (int r = 1; r < team.size; ++r) {
            const int theirs = min(*team.peer(&s.n_list, r), LIST - n);
            const int* their_index = team.peer(s.raw_index, r);
            const float* their_z = team.peer(s.raw_z, r);
            for (int e = tid; e < theirs; e += THREADS) { s.raw_index[n + e] = their_index[e]; s.raw_z[n + e] = their_z[e]; }
            n += theirs;
        }
    }
    team.sync();  // the first block has everything
    if (team.rank != 0) return 0;
    for (int a = tid; a < n; a += THREADS) {
        const int mine = s.raw_index[a];
        int rank = 0;
        for (int m = 0; m < n; ++m) rank += s.raw_index[m] < mine;
        s.list_index[rank] = mine;
        s.list_z[rank] = s.raw_z[a];
    }
    __syncthreads();
    return n;
}

// The nucleus over what `lim` keeps, then the draw among what is left. `fallback_token` is taken when nothing has mass.
// Every block of the team calls this; the block that holds the chosen token writes it. No block returns while another
// may still read its shared memory.
template <class View>
__device__ void nucleus_and_draw(const View& view, const Team& team, Limits lim, const RowOptions& o, float zmax, int vocab, int fallback_token,
                                 unsigned* seen, int* token_out, Scratch& s) {
    const int tid = threadIdx.x;
    // ---- top-p: the smallest prefix (by value descending, ties to the lower index) whose mass reaches top_p * mass
    if (o.top_p < 1.0f) {
        const Selected sel = radix_select<true>(view, team, lim, zmax, o.top_p, 0, s);
        if (sel.n_at > 0) {
            const unsigned long long w = sel.at / (unsigned long long)sel.n_at;  // equal keys have equal weights
            long long ties_kept = sel.n_at;
            if (w > 0ull && sel.need > sel.above) ties_kept = (long long)((sel.need - sel.above + w - 1ull) / w);
            ties_kept = max(1ll, min((long long)sel.n_at, ties_kept));
            int tie_limit = (lim.limited && lim.key_floor == sel.key) ? lim.tie_limit : 0x7fffffff;
            if (ties_kept < sel.n_at) tie_limit = tie_index(view, team, lim, sel.key, (int)ties_kept, vocab, s);
            lim.limited = true;
            lim.key_floor = sel.key;
            lim.tie_limit = tie_limit;
        }
    }

    // ---- the draw: walk the kept tokens in index order until the running mass passes u * mass
    const float u = (float)(philox_first_word(o.counter, o.seed_lo, o.seed_hi) >> 8) * (1.0f / 16777216.0f);
    const int chunk = (view.last - view.first + THREADS - 1) / THREADS;
    const int begin = min(view.last, view.first + tid * chunk), end = min(view.last, begin + chunk);
    float mine = 0.f;
    int last_kept = -1;
    for (int j = begin; j < end; ++j) {
        float z; int i;
        view.get(j, z, i);
        const unsigned key = ordered_key(z);
        if (key != 0u && lim.kept(key, i)) { mine += expf(z - zmax); last_kept = i; }
    }
    // exclusive prefix over threads: inclusive scan inside the warp, then the warps in order, then the blocks in order
    float inclusive = mine;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
        const float other = __shfl_up_sync(0xffffffffu, inclusive, offset);
        if ((tid & 31) >= offset) inclusive += other;
    }
    int fallback = last_kept;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) fallback = max(fallback, __shfl_xor_sync(0xffffffffu, fallback, offset));
    __syncthreads();
    if ((tid & 31) == 31) s.fscratch[tid >> 5] = inclusive;
    if ((tid & 31) == 0) s.iscratch[tid >> 5] = fallback;
    if (tid == 0) s.winner = 0x7fffffff;
    __syncthreads();
    float base = 0.f, block_total = 0.f;
    for (int w = 0; w < THREADS / 32; ++w) {
        if (w < (tid >> 5)) base += s.fscratch[w];
        block_total += s.fscratch[w];
        fallback = max(fallback, s.iscratch[w]);
    }
    if (tid == 0) { s.team_float = block_total; s.team_fallback = fallback; }
    team.sync();
    float blocks_before = 0.f, total = 0.f;
    for (int r = 0; r < team.size; ++r) {
        const float theirs = *team.peer(&s.team_float, r);
        if (r < team.rank) blocks_before += theirs;
        total += theirs;
        fallback = max(fallback, *team.peer(&s.team_fallback, r));
    }
    const float target = u * total;
    const float before = blocks_before + base + inclusive - mine;
    if (mine > 0.f && before + mine > target) atomicMin(&s.winner, tid);
    __syncthreads();
    if (tid == 0) s.team_winner = s.winner == 0x7fffffff ? 0x7fffffff : team.rank * THREADS + s.winner;
    team.sync();
    int winner = 0x7fffffff;
    for (int r = 0; r < team.size; ++r) winner = min(winner, *team.peer(&s.team_winner, r));
    team.sync();  // nothing of another block's shared memory is read after this
    if (winner == 0x7fffffff) {
        if (team.rank == 0 && tid == 0) {
            const int token = fallback >= 0 ? fallback : fallback_token;
            *token_out = token;
            if (seen) atomicOr(&seen[token >> 5], 1u << (token & 31));
        }
        return;
    }
    if (winner / THREADS == team.rank && winner % THREADS == tid) {
        int token = -1;
        float running = before;
        for (int j = begin; j < end; ++j) {
            float z; int i;
            view.get(j, z, i);
            const unsigned key = ordered_key(z);
            if (key != 0u && lim.kept(key, i)) {
                running += expf(z - zmax);
                token = i;
                if (running > target) break;
            }
        }
        *token_out = token;
        if (seen) atomicOr(&seen[token >> 5], 1u << (token & 31));
    }
}

__global__ void __launch_bounds__(THREADS) sample_kernel(const float* __restrict__ logits, int row_stride, int vocab,
                                                         const int* __restrict__ options_raw, unsigned* __restrict__ seen_all,
                                                         int seen_words, int* __restrict__ tokens, int team_size) {
    __shared__ Scratch s;
    Team team;
    team.size = team_size;
    team.rank = team_size > 1 ? (int)cg::this_cluster().block_rank() : 0;
    const int row = blockIdx.x / team_size, tid = threadIdx.x;
    const float* z_row = logits + (size_t)row * row_stride;
    RowOptions o;
    {
        const int* r = options_raw + row * 8;
        o.temperature = __int_as_float(r[0]); o.top_p = __int_as_float(r[1]); o.penalty = __int_as_float(r[2]);
        o.top_k = r[3]; o.seed_lo = (unsigned)r[4]; o.seed_hi = (unsigned)r[5]; o.counter = (unsigned)r[6]; o.slot = r[7];
    }
    unsigned* seen = (seen_all && o.slot >= 0) ? seen_all + (size_t)o.slot * seen_words : nullptr;
    const bool greedy = !(o.temperature > 0.f);
    const int per_block = (vocab + team.size - 1) / team.size;
    RowView slice;
    slice.z_row = z_row; slice.seen = seen;
    slice.first = min(vocab, team.rank * per_block); slice.last = min(vocab, slice.first + per_block);
    slice.divisor = greedy ? 1.0f : o.temperature;
    slice.penalty = greedy ? 1.0f : o.penalty;

    // ---- maximum with the lowest index on ties; NaN never wins. With top-k the same pass counts the keys' first
    // eleven bits, which need no maximum.
    const int k = (!greedy && o.top_k > 0 && o.top_k < vocab) ? o.top_k : 0;
    if (k) {
        for (int b = tid; b < BINS; b += THREADS) { s.hist_lo[b] = 0u; s.hist_hi[b] = 0u; s.count[b] = 0; }
        __syncthreads();
    }
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = slice.first + tid; i < slice.last; i += THREADS) {
        const float z = adjusted(z_row, seen, i, slice.penalty, slice.divisor);
        if (z > bv || (bi == 0x7fffffff && z == z)) { bv = z; bi = i; }
        if (k) atomicAdd(&s.hist_lo[ordered_key(z) >> 21], 1u);
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, offset);
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    if ((tid & 31) == 0) { s.fscratch[tid >> 5] = bv; s.iscratch[tid >> 5] = bi; }
    __syncthreads();
    bv = s.fscratch[0]; bi = s.iscratch[0];
    for (int w = 1; w < THREADS / 32; ++w) {
        const float ov = s.fscratch[w];
        const int oi = s.iscratch[w];
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    if (tid == 0) { s.team_float = bv; s.team_int = bi; }
    team.sync();  // also: the scratch is used again below
    bv = -INFINITY; bi = 0x7fffffff;
    for (int r = 0; r < team.size; ++r) {
        const float ov = *team.peer(&s.team_float, r);
        const int oi = *team.peer(&s.team_int, r);
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    team.sync();
    if (bi == 0x7fffffff) bi = 0;  // a row of NaN only
    if (greedy) {
        if (team.rank == 0 && tid == 0) {
            tokens[row] = bi;
            if (seen) atomicOr(&seen[bi >> 5], 1u << (bi & 31));
        }
        return;
    }
    const float zmax = bv;

    // ---- top-k: the k-th largest key, then how many ties at it are kept (lowest indices)
    Limits lim;
    lim.limited = false; lim.key_floor = 0u; lim.tie_limit = 0x7fffffff;
    if (k) {
        // Where the k-th largest key's first eleven bits are known and few enough tokens share them or stand above, those
        // are copied out and the rest of the search runs on the copy.
        const Selected coarse = radix_select<false>(slice, team, lim, zmax, 0.f, k, s, true, 1);
        if (coarse.above + coarse.at <= (unsigned long long)LIST) {
            Limits from_bin;
            from_bin.limited = true; from_bin.key_floor = coarse.key; from_bin.tie_limit = 0x7fffffff;  // coarse.key: the bin's lowest key
            const int n = copy_out(slice, team, from_bin, s);
            if (team.rank != 0) return;
            ListView list;
            list.z_list = s.list_z; list.index_list = s.list_index; list.first = 0; list.last = n;
            Team alone;
            alone.size = 1; alone.rank = 0;
            const Selected sel = radix_select<false>(list, alone, lim, zmax, 0.f, k, s);
            const int ties_kept = max(1, min(sel.n_at, k - (int)sel.above));
            Limits all_ties;
            all_ties.limited = true; all_ties.key_floor = sel.key; all_ties.tie_limit = 0x7fffffff;
            const int tie_limit = ties_kept < sel.n_at ? tie_index(list, alone, all_ties, sel.key, ties_kept, vocab, s) : 0x7fffffff;
            lim.limited = true; lim.key_floor = sel.key; lim.tie_limit = tie_limit;
            nucleus_and_draw(list, alone, lim, o, zmax, vocab, bi, seen, tokens + row, s);
            return;
        }
        const Selected sel = radix_select<false>(slice, team, lim, zmax, 0.f, k, s, true);
        const int ties_kept = max(1, min(sel.n_at, k - (int)sel.above));
        Limits all_ties;
        all_ties.limited = true; all_ties.key_floor = sel.key; all_ties.tie_limit = 0x7fffffff;
        const int tie_limit = ties_kept < sel.n_at ? tie_index(slice, team, all_ties, sel.key, ties_kept, vocab, s) : 0x7fffffff;
        lim.limited = true; lim.key_floor = sel.key; lim.tie_limit = tie_limit;
        if (k <= LIST) {
            const int n = copy_out(slice, team, lim, s);
            if (team.rank != 0) return;
            ListView list;
            list.z_list = s.list_z; list.index_list = s.list_index; list.first = 0; list.last = n;
            Limits none;
            none.limited = false; none.key_floor = 0u; none.tie_limit = 0x7fffffff;
            Team alone;
            alone.size = 1; alone.rank = 0;
            nucleus_and_draw(list, alone, none, o, zmax, vocab, bi, seen, tokens + row, s);
            return;
        }
    }
    nucleus_and_draw(slice, team, lim, o, zmax, vocab, bi, seen, tokens + row, s);
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
    const int team = vocab >= TEAM_FROM_VOCAB ? TEAM : 1;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(rows * team);
    config.blockDim = dim3(THREADS);
    config.stream = stream;
    cudaLaunchAttribute cluster[1];
    cluster[0].id = cudaLaunchAttributeClusterDimension;
    cluster[0].val.clusterDim.x = team;
    cluster[0].val.clusterDim.y = 1;
    cluster[0].val.clusterDim.z = 1;
    config.attrs = cluster;
    config.numAttrs = team > 1 ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&config, sample_kernel, logits, row_stride, vocab, options, seen, seen_words, tokens, team);
    return e == cudaSuccess ? launch_status() : (int)e;
}
