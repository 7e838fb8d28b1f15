// Paged bfloat16 attention with TMA-fed key/value tiles and a dedicated producer warp, for head sizes
// that are multiples of 64 (HB_HEAD_DIM = 64, 128, 192, 256) and pages of 8 to 64 tokens.
//
// Same two launch shapes and the same arithmetic as attention_bf16.cu (64-key tiles, Q K^T and P V with
// mma.sync m16n8k16, float running maximum and sum in the exp2 domain), but the key/value tiles do not
// pass through the math warps' registers and address arithmetic: one lane of a producer warp issues one
// cp.async.bulk.tensor per page and 64-column half (128-byte swizzle, no multicast) into a ring of
// stages, signalled by mbarriers with a byte count; four consumer warps wait, compute and hand the stage
// back.  The cache layer [pages, 2, kv_heads, page_size, D] is addressed as a matrix of
// pages * 2 * kv_heads * page_size rows of D columns, so a page of one head is a box of page_size rows.
// Pages a tile does not need (beyond the query's position, or released by a window) are not fetched; the
// ring is zeroed once so that what they leave in shared memory is finite.
//
// Every mbarrier wait is bounded; a wait that runs out sets HB_STATUS_WAIT_EXPIRED and the block leaves.
// Counterparts in the reference: attention_mma_paged_*_bf16 and attention_split_rows_*_bf16 +
// attention_combine_rows_bf16 (helios/crates/helios-hal/kernels/elementwise.cu:576-729,749,875-937).
#include <cuda.h>

#include "common.cuh"

#ifndef HB_HEAD_DIM
#define HB_HEAD_DIM 128
#endif

namespace {
typedef __nv_bfloat16 bf16;
constexpr int D = HB_HEAD_DIM;
static_assert(D % 64 == 0 && D >= 64 && D <= 256, "the TMA attention takes head sizes that are multiples of 64 up to 256");
constexpr int BN = 64;                        // keys per tile
constexpr int HALVES = D / 64;                // 64-column (128-byte) panels of a tile
constexpr int PANEL = BN * 64;                // elements of one panel: 64 keys x 64 columns, 8 KB
constexpr int TILE_ELEMS = HALVES * PANEL;    // one K (or V) tile
constexpr int STAGE_BYTES = 2 * TILE_ELEMS * 2;
constexpr int LDQ = D + 8;                    // padded row of the query tile
constexpr int CONSUMERS = 4;
constexpr int FRESH_TOKENS = 4;                // a row that takes the token shape brings at most this many tokens (the planner's TOKEN_SHAPE_MAX)
constexpr int THREADS = 32 * (CONSUMERS + 1);
constexpr unsigned WAIT_LIMIT = 1u << 24;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* failed) {
    const unsigned addr = smem_u32(bar);
    for (unsigned spin = 0; spin < WAIT_LIMIT; ++spin) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if ((spin & 1023) == 1023 && *failed) return false;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, unsigned long long* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// Element (key, 16-byte chunk cc of the row) of a K or V tile written by TMA with the 128-byte swizzle:
// panel cc / 8, row `key` of 128 bytes, chunk (cc % 8) xor (key % 8).
__device__ __forceinline__ const bf16* swizzled(const bf16* tile, int key, int cc) {
    return tile + (cc >> 3) * PANEL + key * 64 + (((cc & 7) ^ (key & 7)) << 3);
}

struct RowState {
    float m[2], l[2];
    float o[D / 8][4];
    __device__ __forceinline__ void init() {
        m[0] = m[1] = -INFINITY; l[0] = l[1] = 0.f;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    }
};

// One warp: 16 query rows (padded tile `qs`) against NT * 8 keys starting at key `key0` of the swizzled K / V tiles.
template <int NT>
__device__ __forceinline__ void process_keys(RowState& st, const bf16* qs, const bf16* ks, const bf16* vs, int key0, int base,
                                             const int (&hi)[2], const int (&lo)[2], float scale_log2) {
    const int lane = threadIdx.x & 31, m = lane >> 3;
    float s[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
        unsigned a[4];
        ldmatrix_x4(a, qs + (lane & 15) * LDQ + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int n = 0; n < NT; n += 2) {
            unsigned b[4];
            ldmatrix_x4(b, swizzled(ks, key0 + n * 8 + (lane & 7) + (m >> 1) * 8, kk * 2 + (m & 1)));
            mma_bf16(s[n], a, b[0], b[1]);
            mma_bf16(s[n + 1], a, b[2], b[3]);
        }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            const int pos = base + key0 + n * 8 + (lane & 3) * 2 + (e & 1);
            const float v = (pos <= hi[r] && pos >= lo[r]) ? s[n][e] * scale_log2 : -INFINITY;
            s[n][e] = v;
            mx[r] = fmaxf(mx[r], v);
        }
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(st.m[r], mx[r]);
        alpha[r] = (m_new == -INFINITY) ? 1.f : exp2f(st.m[r] - m_new);
        st.m[r] = m_new;
        mx[r] = (m_new == -INFINITY) ? 0.f : m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float p = exp2f(s[n][e] - mx[e >> 1]);
            s[n][e] = p;
            sum[e >> 1] += p;
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
        st.l[r] = st.l[r] * alpha[r] + sum[r];
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        st.o[i][0] *= alpha[0]; st.o[i][1] *= alpha[0]; st.o[i][2] *= alpha[1]; st.o[i][3] *= alpha[1];
    }
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        unsigned a[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                         pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
        for (int n = 0; n < D / 8; n += 2) {
            unsigned b[4];
            ldmatrix_x4_trans(b, swizzled(vs, key0 + kk * 16 + (lane & 7) + (m & 1) * 8, n + (m >> 1)));
            mma_bf16(st.o[n], a, b[0], b[1]);
            mma_bf16(st.o[n + 1], a, b[2], b[3]);
        }
    }
}

struct AttnArgs {
    const bf16* q; int q_stride;
    bf16* out; int out_stride;
    const int* block_table; int table_width;
    const int* token_row;
    const int* positions;
    int heads, kv_heads, page_size, pages, window;
    float scale_log2;
    int* status;
};

__host__ __device__ constexpr int stages_for(bool tokens) { return D <= 64 ? 4 : (tokens && D <= 128 ? 3 : 2); }

// work: TOKENS ? flat token indices : triples (first token, count, batch row).
template <bool TOKENS>
__global__ void __launch_bounds__(THREADS) attention_tma_kernel(const __grid_constant__ CUtensorMap kv_map, const AttnArgs a,
                                                                const int* __restrict__ work, int gc, int head_chunks, int splits,
                                                                float* __restrict__ ws_o, float* __restrict__ ws_ml) {
    constexpr int ROWS = TOKENS ? 16 : 64;
    constexpr int STAGES = stages_for(TOKENS);
    extern __shared__ unsigned char smem_raw[];
    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    bf16* qs = reinterpret_cast<bf16*>(ring + (size_t)STAGES * STAGE_BYTES);
    unsigned long long* full = reinterpret_cast<unsigned long long*>(qs + ROWS * LDQ);
    unsigned long long* empty = full + STAGES;
    volatile int* failed = reinterpret_cast<volatile int*>(empty + STAGES);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    let_next_kernel_start();
    int tok0, ntok, brow, split = 0;
    if (TOKENS) {
        tok0 = work[blockIdx.x]; ntok = 1; brow = a.token_row[tok0]; split = blockIdx.z;
    } else {
        tok0 = work[3 * blockIdx.x]; ntok = work[3 * blockIdx.x + 1]; brow = work[3 * blockIdx.x + 2];
    }
    const int kvh = blockIdx.y / head_chunks, chunk = blockIdx.y - kvh * head_chunks;
    const int group = a.heads / a.kv_heads;
    const int first_head = kvh * group + chunk * gc;
    const int heads_here = min(gc, group - chunk * gc);
    const int* table = a.block_table + (size_t)brow * a.table_width;
    const int pos_first = a.positions[tok0], pos_last = pos_first + ntok - 1;
    const int need_lo = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
    const int start = (need_lo / BN) * BN;
    const int n_tiles = (pos_last - start) / BN + 1;
    int first = 0, last = n_tiles;
    if (TOKENS) {
        const int per_split = (n_tiles + splits - 1) / splits;
        first = split * per_split;
        last = min(n_tiles, first + per_split);
    }

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], CONSUMERS); }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Pages that are not fetched (before a window's start, beyond the last position) leave whatever the stage held
    // before under masked keys; that is earlier key/value data, which is finite, unless the stage was never written.
    // So a stage is zeroed when its first tile is one of the two that can be fetched in part.
    for (int s = 0; s < STAGES && first + s < last; ++s) {
        const int tile = first + s;
        if (tile != n_tiles - 1 && !(tile == 0 && need_lo > start)) continue;
        uint4* stage = reinterpret_cast<uint4*>(ring + (size_t)s * STAGE_BYTES);
        for (int e = tid; e < STAGE_BYTES / 16; e += THREADS) stage[e] = make_uint4(0, 0, 0, 0);
    }
    // The token shape lets its producer start before the kernels ahead in the stream have finished: keys and values of
    // earlier steps are in the cache already, only the newest positions (and the queries) come from the kernel before.
    // Its consumers wait, fetch the queries and meet at a barrier of their own; the tile shape waits as a whole.
    if (TOKENS) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
    }
    if (!TOKENS || warp != CONSUMERS) {
        wait_for_previous_kernels();  // the queries and the newest keys and values come from the kernel before
        // queries: virtual row v = token * gc + head
        const int loaders = TOKENS ? 32 * CONSUMERS : THREADS;
        for (int e = tid; e < ROWS * (D / 8); e += loaders) {
            const int v = e / (D / 8), c = e - v * (D / 8);
            const int tok = v / gc, hh = v - tok * gc;
            uint4 value = make_uint4(0, 0, 0, 0);
            if (tok < ntok && hh < heads_here)
                value = *reinterpret_cast<const uint4*>(a.q + (size_t)(tok0 + tok) * a.q_stride + (size_t)(first_head + hh) * D + c * 8);
            *reinterpret_cast<uint4*>(qs + v * LDQ + c * 8) = value;
        }
    }
    if (TOKENS) {
        if (warp != CONSUMERS) asm volatile("bar.sync 1, %0;" ::"n"(32 * CONSUMERS) : "memory");
    } else {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
    }

    if (warp == CONSUMERS) {
        // a token of this shape sees at most FRESH_TOKENS positions written by the kernel before (its own and those of
        // the same row's tokens before it): tiles that end below them may be fetched at once
        bool waited = !TOKENS;
        const int fresh_from = pos_first - (FRESH_TOKENS - 1);
        // ------------------------------------------------------------------ producer
        // The whole warp takes part: lane p looks up page p of the tile, lane 0 arms the barrier with the byte count,
        // then every lane issues one copy (page, K or V, 64-column panel), so the copies of a tile start together.
        const int shift = 31 - __clz(a.page_size);
        const int pages_per_tile = BN >> shift;
        const int ops = pages_per_tile * 2 * HALVES;
        const unsigned page_bytes = 2u * a.page_size * D * 2u;
        if (lane == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&kv_map) : "memory");
        // A block that walks many tiles reads the page numbers of several tiles from the table at once (one per lane): a
        // read per tile puts a round trip to memory before every tile's copies, and a long walk is bound by them (batch 64,
        // one split: 4.66 -> 4.60 ms per step). A block with a handful of tiles has them in flight before the kernel ahead
        // has finished either way, and was measured a little slower with the wider read.
        const int tiles_per_look = 32 / pages_per_tile;
        const bool looks_ahead = last - first > 8;
        int looked_from = first, looked_id = -1;
        auto look_up = [&](int from) {
            looked_from = from;
            const int block = (start + from * BN + lane * a.page_size) >> shift;
            looked_id = block < a.table_width ? __ldg(table + block) : -1;
        };
        if (looks_ahead) look_up(first);
        for (int it = first; it < last; ++it) {
            const int s = (it - first) % STAGES, round = (it - first) / STAGES;
            if (looks_ahead && it - looked_from >= tiles_per_look) look_up(it);
            int ok = 1;
            if (lane == 0) ok = mbar_wait(&empty[s], (round & 1) ^ 1, failed) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                if (!waited) wait_for_previous_kernels();  // no write to global memory before that
                if (lane == 0) { *failed = 1; atomicOr(a.status, HB_STATUS_WAIT_EXPIRED | (TOKENS ? HB_STATUS_IN_ATTENTION_TMA_TOKENS : HB_STATUS_IN_ATTENTION_TMA_TILES)); }
                break;
            }
            const int base = start + it * BN;
            if (!waited && base + BN - 1 >= fresh_from) {
                wait_for_previous_kernels();
                waited = true;
            }
            int my_page = -1;
            const int k0 = base + lane * a.page_size;
            const int looked = looks_ahead ? __shfl_sync(0xffffffffu, looked_id, ((it - looked_from) * pages_per_tile + lane) & 31) : -1;
            if (lane < pages_per_tile && k0 <= pos_last && k0 + a.page_size - 1 >= need_lo) {
                const int block = k0 >> shift;
                const int id = looks_ahead ? looked : (block < a.table_width ? __ldg(table + block) : -1);
                if (id >= 0 && id < a.pages) my_page = id;
                else {
                    if (!waited) wait_for_previous_kernels();
                    atomicOr(a.status, HB_STATUS_BAD_PAGE);
                }
            }
            const unsigned valid = __popc(__ballot_sync(0xffffffffu, my_page >= 0));
            if (lane == 0) {
                if (valid) mbar_expect_tx(&full[s], valid * page_bytes); else mbar_arrive(&full[s]);
            }
            __syncwarp();
            bf16* stage = reinterpret_cast<bf16*>(ring + (size_t)s * STAGE_BYTES);
            for (int op0 = 0; op0 < ops; op0 += 32) {
                const int op = op0 + lane;
                const int p = min(op, ops - 1) / (2 * HALVES), rest = op % (2 * HALVES);
                const int which = rest / HALVES, h = rest - which * HALVES;
                const int page = __shfl_sync(0xffffffffu, my_page, p);
                if (op < ops && page >= 0)
                    tma_load_2d(stage + which * TILE_ELEMS + h * PANEL + p * a.page_size * 64, &kv_map, &full[s], h * 64,
                                ((page * 2 + which) * a.kv_heads + kvh) * a.page_size);
            }
        }
        return;
    }
    // ---------------------------------------------------------------------- consumers
    int hi[2], lo[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int v = (TOKENS ? 0 : warp * 16) + (lane >> 2) + r * 8;
        const int tok = v / gc, hh = v - tok * gc;
        const bool valid = tok < ntok && hh < heads_here;
        hi[r] = valid ? pos_first + tok : -1;
        lo[r] = (valid && a.window > 0) ? max(0, hi[r] - a.window + 1) : 0;
    }
    const int warp_first_tok = TOKENS ? 0 : (warp * 16) / gc;
    const int warp_hi = pos_first + (TOKENS ? 0 : min(ntok - 1, (warp * 16 + 15) / gc));
    const int warp_lo = a.window > 0 ? max(0, pos_first + warp_first_tok - a.window + 1) : 0;
    const bool warp_has_rows = warp_first_tok < ntok;
    RowState st;
    st.init();
    bool ok = true;
    for (int it = first; it < last; ++it) {
        const int s = (it - first) % STAGES, round = (it - first) / STAGES;
        if (!mbar_wait(&full[s], round & 1, failed)) { *failed = 1; atomicOr(a.status, HB_STATUS_WAIT_EXPIRED | (TOKENS ? HB_STATUS_IN_ATTENTION_TMA_TOKENS : HB_STATUS_IN_ATTENTION_TMA_TILES)); ok = false; break; }
        const bf16* ks = reinterpret_cast<const bf16*>(ring + (size_t)s * STAGE_BYTES);
        const int base = start + it * BN;
        if (TOKENS) {
            if (base + warp * 16 <= pos_last) process_keys<2>(st, qs, ks, ks + TILE_ELEMS, warp * 16, base, hi, lo, a.scale_log2);
        } else if (!TOKENS) {
            if (warp_has_rows && base <= warp_hi && base + BN - 1 >= warp_lo)
                process_keys<BN / 8>(st, qs + warp * 16 * LDQ, ks, ks + TILE_ELEMS, 0, base, hi, lo, a.scale_log2);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }
    if (!TOKENS) {
        if (!ok) return;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int v = warp * 16 + (lane >> 2) + r * 8;
            const int tok = v / gc, hh = v - tok * gc;
            if (tok >= ntok || hh >= heads_here) continue;
            const float inv = st.l[r] > 0.f ? 1.f / st.l[r] : 0.f;
            bf16* dst = a.out + (size_t)(tok0 + tok) * a.out_stride + (size_t)(first_head + hh) * D + (lane & 3) * 2;
#pragma unroll
            for (int n = 0; n < D / 8; ++n)
                *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = __floats2bfloat162_rn(st.o[n][2 * r] * inv, st.o[n][2 * r + 1] * inv);
        }
        return;
    }
    // token shape: merge the four consumer warps (each saw a quarter of every tile) through the ring, which no copy
    // targets any more once every consumer has passed its last tile
    asm volatile("bar.sync 1, %0;" ::"n"(32 * CONSUMERS) : "memory");
    float* wo = reinterpret_cast<float*>(ring);   // [4][16][D]
    float* wm = wo + CONSUMERS * 16 * D;          // [4][16]
    float* wl = wm + CONSUMERS * 16;              // [4][16]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = (lane >> 2) + r * 8;
        if ((lane & 3) == 0) { wm[warp * 16 + row] = st.m[r]; wl[warp * 16 + row] = st.l[r]; }
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            float* dst = wo + ((size_t)warp * 16 + row) * D + n * 8 + (lane & 3) * 2;
            dst[0] = st.o[n][2 * r]; dst[1] = st.o[n][2 * r + 1];
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(32 * CONSUMERS) : "memory");
    if (*failed) return;
    for (int e = tid; e < heads_here * D; e += 32 * CONSUMERS) {
        const int row = e / D, c = e - row * D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < CONSUMERS; ++w) m = fmaxf(m, wm[w * 16 + row]);
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < CONSUMERS; ++w) {
            const float f = (wm[w * 16 + row] == -INFINITY) ? 0.f : exp2f(wm[w * 16 + row] - m);
            l += f * wl[w * 16 + row];
            o += f * wo[((size_t)w * 16 + row) * D + c];
        }
        const int head = first_head + row;
        if (splits == 1) {
            a.out[(size_t)tok0 * a.out_stride + (size_t)head * D + c] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
        } else {
            const size_t slot = ((size_t)blockIdx.x * a.heads + head) * splits + split;
            ws_o[slot * D + c] = o;
            if (c == 0) { ws_ml[slot * 2] = m; ws_ml[slot * 2 + 1] = l; }
        }
    }
}

// Every piece is asked for before the first is used: a thread that fetches a piece, folds it in and only then fetches the
// next waits for memory once per piece, and at a handful of rows the kernel is nothing but such waits. The order of the
// sums stays the order of the splits.
constexpr int MERGE_AHEAD = 16;
__global__ void attention_merge_kernel(const int* __restrict__ items, const float* __restrict__ ws_o, const float* __restrict__ ws_ml,
                                       bf16* __restrict__ out, int out_stride, int heads, int splits) {
    const int item = blockIdx.x, head = blockIdx.y, t = items[item];
    let_next_kernel_start();
    wait_for_previous_kernels();
    const size_t slot0 = ((size_t)item * heads + head) * splits;
    const float2* ml = reinterpret_cast<const float2*>(ws_ml) + slot0;  // (maximum, sum) of each piece
    float2 piece[MERGE_AHEAD];
#pragma unroll
    for (int s = 0; s < MERGE_AHEAD; ++s)
        if (s < splits) piece[s] = ml[s];
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float value[MERGE_AHEAD];
#pragma unroll
        for (int s = 0; s < MERGE_AHEAD; ++s)
            if (s < splits) value[s] = ws_o[(slot0 + s) * D + c];
        float m = -INFINITY;
#pragma unroll
        for (int s = 0; s < MERGE_AHEAD; ++s)
            if (s < splits) m = fmaxf(m, piece[s].x);
        for (int s = MERGE_AHEAD; s < splits; ++s) m = fmaxf(m, ml[s].x);
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int s = 0; s < MERGE_AHEAD; ++s) {
            if (s < splits) {
                const float f = (piece[s].x == -INFINITY) ? 0.f : exp2f(piece[s].x - m);
                l += f * piece[s].y;
                o += f * value[s];
            }
        }
        for (int s = MERGE_AHEAD; s < splits; ++s) {
            const float2 p = ml[s];
            const float f = (p.x == -INFINITY) ? 0.f : exp2f(p.x - m);
            l += f * p.y;
            o += f * ws_o[(slot0 + s) * D + c];
        }
        out[(size_t)t * out_stride + (size_t)head * D + c] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* found = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &found, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(found);
    }
    return fn;
}

template <bool TOKENS>
constexpr size_t smem_bytes() {
    return 1024 + (size_t)stages_for(TOKENS) * STAGE_BYTES + (size_t)(TOKENS ? 16 : 64) * LDQ * sizeof(bf16) + 2 * stages_for(TOKENS) * 8 + 16;
}

// The cache layer as a matrix [pages * 2 * kv_heads * page_size, D] fetched in boxes of page_size rows x 64 columns.
int prepare(CUtensorMap* map, AttnArgs& a, const void* q, int q_stride, void* out, int out_stride, const void* cache, const int* block_table,
            int table_width, const int* token_row, const int* positions, int heads, int kv_heads, int head_dim, int page_size, int pages,
            float scale, int window, int* status) {
    if (head_dim != D) return HB_UNSUPPORTED_SIZE;
    if (kv_heads <= 0 || heads % kv_heads || q_stride % 8 || out_stride % 2) return HB_BAD_ARGUMENT;
    if (page_size < 8 || page_size > 64 || (page_size & (page_size - 1))) return HB_UNSUPPORTED_SIZE;
    if (((uintptr_t)q | (uintptr_t)cache) & 15) return HB_BAD_ARGUMENT;
    EncodeTiled encode = encode_tiled();
    if (!encode) return HB_BAD_ARGUMENT;
    const cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)pages * 2 * kv_heads * page_size};
    const cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
    const cuuint32_t elem[2] = {1, 1};
    if (encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return HB_BAD_ARGUMENT;
    a = AttnArgs{(const bf16*)q, q_stride, (bf16*)out, out_stride, block_table, table_width, token_row, positions,
                 heads, kv_heads, page_size, pages, window, scale * 1.4426950408889634f, status};
    return 0;
}
}  // namespace

HB_EXPORT int hb_attention_tma_tiles(const void* q, int q_stride, void* out, int out_stride, const void* cache, const int* block_table,
                                     int table_width, const int* token_row, const int* positions, const int* tiles, int n_tiles, int heads,
                                     int kv_heads, int head_dim, int page_size, int pages, float scale, int window, int* status,
                                     cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    CUtensorMap map;
    AttnArgs a;
    if (int code = prepare(&map, a, q, q_stride, out, out_stride, cache, block_table, table_width, token_row, positions, heads, kv_heads,
                           head_dim, page_size, pages, scale, window, status)) return code;
    const int group = heads / kv_heads, gc = group < 64 ? group : 64, head_chunks = (group + gc - 1) / gc;
    if ((long long)kv_heads * head_chunks > 65535) return HB_UNSUPPORTED_SIZE;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<false>());
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return launch_after_previous(attention_tma_kernel<false>, dim3(n_tiles, kv_heads * head_chunks), THREADS, smem_bytes<false>(), stream, map, a, tiles,
                                 gc, head_chunks, 1, nullptr, nullptr);
}

HB_EXPORT int hb_attention_tma_tokens(const void* q, int q_stride, void* out, int out_stride, const void* cache, const int* block_table,
                                      int table_width, const int* token_row, const int* positions, const int* items, int n_items, int splits,
                                      float* workspace, int heads, int kv_heads, int head_dim, int page_size, int pages, float scale,
                                      int window, int* status, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    CUtensorMap map;
    AttnArgs a;
    if (int code = prepare(&map, a, q, q_stride, out, out_stride, cache, block_table, table_width, token_row, positions, heads, kv_heads,
                           head_dim, page_size, pages, scale, window, status)) return code;
    const int group = heads / kv_heads, head_chunks = (group + 15) / 16;
    if (splits < 1 || splits > 65535 || (long long)kv_heads * head_chunks > 65535 || (splits > 1 && !workspace)) return HB_BAD_ARGUMENT;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<true>());
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    float* ws_o = workspace;
    float* ws_ml = workspace ? workspace + (size_t)n_items * heads * splits * D : nullptr;
    int code = launch_after_previous(attention_tma_kernel<true>, dim3(n_items, kv_heads * head_chunks, splits), THREADS, smem_bytes<true>(), stream, map, a,
                                     items, 16, head_chunks, splits, ws_o, ws_ml);
    if (code || splits == 1) return code;
    return launch_after_previous(attention_merge_kernel, dim3(n_items, heads), D < 128 ? 64 : 128, 0, stream, items, (const float*)ws_o,
                                 (const float*)ws_ml, (bf16*)out, out_stride, heads, splits);
}
