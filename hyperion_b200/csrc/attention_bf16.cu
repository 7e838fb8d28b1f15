// Causal grouped-query attention over the paged bfloat16 cache on tensor cores, compiled for one head
// size (HB_HEAD_DIM, a multiple of 16 up to 256).
//
// Two launch shapes share one inner loop (flash-attention style: 64-key tiles staged in shared memory
// with cp.async, Q K^T and P V with mma.sync.m16n8k16 bf16 -> f32, running maximum and sum in float in
// the exp2 domain, P rounded to bfloat16 for P V):
//   * tiles: one block per (tile of up to 64 "virtual rows" = tokens x heads of one key/value group,
//     key/value head); each of its 4 warps owns 16 rows and walks all keys.  Prompt portions.
//   * tokens: one block per (token, key/value head, split of the keys); the 4 warps share the token's
//     heads (<= 16 rows) and divide every key tile between them; partial results of the splits are
//     merged by a second kernel in split order.  Decoded tokens and very short portions.
// The reference's counterparts are attention_mma_paged_*_bf16 for prompt chunks and
// attention_split_rows_*_bf16 + attention_combine_rows_bf16 for decode rows
// (helios/crates/helios-hal/kernels/elementwise.cu:576-729,749,875-937); mask: key position <= query
// position (:660-663), optionally > position - window.
#include "common.cuh"

#ifndef HB_HEAD_DIM
#define HB_HEAD_DIM 128
#endif

namespace {
constexpr int D = HB_HEAD_DIM;
constexpr int BN = 64;             // keys per tile
constexpr int BM = 64;             // virtual rows per block in the tile shape
constexpr int THREADS = 128;
constexpr int LDS = D + 8;         // padded row of a shared-memory tile, in elements (odd count of 16-byte chunks)
constexpr int CHUNKS = D / 8;      // 16-byte chunks per row
constexpr int LOADS = BN * CHUNKS / THREADS;  // chunks per thread per tile
constexpr int TOKEN_STAGES = (D <= 128) ? 3 : 2;  // key/value tiles in the ring of the token shape (two blocks of it fit an SM)
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16 up to 256");
static_assert((BN * CHUNKS) % THREADS == 0, "tile loads must divide evenly");

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// Running state of 16 rows in one warp: thread (lane) holds rows lane/4 and lane/4 + 8.
struct RowState {
    float m[2], l[2];
    float o[D / 8][4];
    __device__ __forceinline__ void init() {
        m[0] = m[1] = -INFINITY; l[0] = l[1] = 0.f;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    }
};

// One warp: 16 query rows (shared tile `qs`, row 0 = the warp's first row) against NT*8 keys that start
// at row `key0` of the shared K and V tiles.  hi[r] / lo[r]: last and first visible key position of the
// thread's rows (hi < lo: nothing visible); `base`: position of the tile's key 0.
template <int NT>
__device__ __forceinline__ void process_keys(RowState& st, const bf16* qs, const bf16* ks, const bf16* vs, int key0, int base,
                                             const int (&hi)[2], const int (&lo)[2], float scale_log2) {
    const int lane = threadIdx.x & 31;
    float s[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
        unsigned a[4];
        ldmatrix_x4(a, qs + (lane & 15) * LDS + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int n = 0; n < NT; n += 2) {
            unsigned b[4];
            const int m = lane >> 3;
            ldmatrix_x4(b, ks + (key0 + n * 8 + (lane & 7) + (m >> 1) * 8) * LDS + kk * 16 + (m & 1) * 8);
            mma_bf16(s[n], a, b[0], b[1]);
            mma_bf16(s[n + 1], a, b[2], b[3]);
        }
    }
    // mask, scale into the exp2 domain, new row maxima
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
        mx[r] = (m_new == -INFINITY) ? 0.f : m_new;  // subtracting 0 keeps exp2(-inf) = 0 without NaN
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
    // O += P V, 16 keys per step
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        unsigned a[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                         pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
        for (int n = 0; n < D / 8; n += 2) {
            unsigned b[4];
            const int m = lane >> 3;
            ldmatrix_x4_trans(b, vs + (key0 + kk * 16 + (lane & 7) + (m & 1) * 8) * LDS + n * 8 + (m >> 1) * 8);
            mma_bf16(st.o[n], a, b[0], b[1]);
            mma_bf16(st.o[n + 1], a, b[2], b[3]);
        }
    }
}

// Stage keys [base, base + 64) of one key/value head into the shared K and V tiles. Keys outside
// [need_lo, need_hi] or without a page are zero-filled; a missing page inside the range sets the status.
__device__ __forceinline__ void load_kv_tile(bf16* ks, bf16* vs, const bf16* cache, const int* table, int table_width, int base,
                                             int need_lo, int need_hi, int kvh, int kv_heads, int page_size, int pages, int* status) {
    // page_size is a power of two (the launcher refuses anything else).  All table entries are fetched first and the
    // copies issued afterwards, so the table reads of a tile overlap instead of each standing in front of its copy.
    const int shift = 31 - __clz(page_size);
    const size_t head_stride = (size_t)page_size * D;
    const size_t page_stride = 2 * (size_t)kv_heads * head_stride;
    int page[LOADS];
#pragma unroll
    for (int i = 0; i < LOADS; ++i) {
        const int pos = base + (i * THREADS + (int)threadIdx.x) / CHUNKS;
        const int block = pos >> shift;
        page[i] = (pos >= need_lo && pos <= need_hi) ? (block < table_width ? max(__ldg(table + block), -2) : -2) : -3;
    }
#pragma unroll
    for (int i = 0; i < LOADS; ++i) {
        const int chunk = i * THREADS + threadIdx.x;
        const int key = chunk / CHUNKS, c = chunk - key * CHUNKS;
        const int pos = base + key;
        const bool wanted = page[i] != -3;
        const bool valid = page[i] >= 0 && page[i] < pages;
        if (wanted && !valid) atomicOr(status, HB_STATUS_BAD_PAGE);
        const bf16* src = valid ? cache + (size_t)page[i] * page_stride + (size_t)kvh * head_stride +
                                      (size_t)(pos & (page_size - 1)) * D + c * 8
                                : cache;
        cp_async16(ks + key * LDS + c * 8, src, valid);
        cp_async16(vs + key * LDS + c * 8, valid ? src + (size_t)kv_heads * head_stride : src, valid);
    }
}

struct AttnArgs {
    const bf16* q; int q_stride;       // queries [tokens, >= heads * D], row stride in elements
    bf16* out; int out_stride;         // [tokens, heads * D]
    const bf16* cache;                 // one cache layer [pages, 2, kv_heads, page_size, D]
    const int* block_table; int table_width;
    const int* token_row;              // batch row of every token
    const int* positions;              // position of every token
    int heads, kv_heads, page_size, pages, window;
    float scale_log2;                  // scale * log2(e)
    int* status;
};

// ---------------------------------------------------------------------------------- tile shape
// tiles[3*i] = first token (flat index), tiles[3*i+1] = token count, tiles[3*i+2] = batch row.
__global__ void __launch_bounds__(THREADS) attention_tiles_kernel(AttnArgs a, const int* __restrict__ tiles, int gc, int head_chunks) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* kv = qs + BM * LDS;  // [2 buffers][K | V][BN][LDS]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tok0 = tiles[3 * blockIdx.x], ntok = tiles[3 * blockIdx.x + 1], brow = tiles[3 * blockIdx.x + 2];
    const int kvh = blockIdx.y / head_chunks, chunk = blockIdx.y - kvh * head_chunks;
    const int group = a.heads / a.kv_heads;
    const int first_head = kvh * group + chunk * gc;
    const int heads_here = min(gc, group - chunk * gc);
    const int* table = a.block_table + (size_t)brow * a.table_width;
    const int pos_first = a.positions[tok0], pos_last = pos_first + ntok - 1;

    // queries of the tile: virtual row v = token * gc + head
    for (int e = tid; e < BM * CHUNKS; e += THREADS) {
        const int v = e / CHUNKS, c = e - v * CHUNKS;
        const int tok = v / gc, hh = v - tok * gc;
        const bool valid = tok < ntok && hh < heads_here;
        const bf16* src = valid ? a.q + (size_t)(tok0 + tok) * a.q_stride + (size_t)(first_head + hh) * D + c * 8 : a.q;
        cp_async16(qs + v * LDS + c * 8, src, valid);
    }
    int hi[2], lo[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int v = warp * 16 + (lane >> 2) + r * 8;
        const int tok = v / gc, hh = v - tok * gc;
        const bool valid = tok < ntok && hh < heads_here;
        hi[r] = valid ? pos_first + tok : -1;
        lo[r] = (valid && a.window > 0) ? max(0, hi[r] - a.window + 1) : 0;
    }
    const int warp_hi = pos_first + min(ntok - 1, (warp * 16 + 15) / gc);
    const int warp_first_tok = (warp * 16) / gc;
    const int warp_lo = a.window > 0 ? max(0, pos_first + warp_first_tok - a.window + 1) : 0;
    const bool warp_has_rows = warp_first_tok < ntok;

    const int need_lo = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
    const int start = (need_lo / BN) * BN;
    const int n_tiles = (pos_last - start) / BN + 1;
    RowState st;
    st.init();
    load_kv_tile(kv, kv + BN * LDS, a.cache, table, a.table_width, start, need_lo, pos_last, kvh, a.kv_heads, a.page_size, a.pages, a.status);
    cp_async_commit();
    for (int it = 0; it < n_tiles; ++it) {
        bf16* ks = kv + (it & 1) * 2 * BN * LDS;
        if (it + 1 < n_tiles) {
            bf16* nk = kv + ((it + 1) & 1) * 2 * BN * LDS;
            load_kv_tile(nk, nk + BN * LDS, a.cache, table, a.table_width, start + (it + 1) * BN, need_lo, pos_last, kvh, a.kv_heads,
                         a.page_size, a.pages, a.status);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int base = start + it * BN;
        if (warp_has_rows && base <= warp_hi && base + BN - 1 >= warp_lo)
            process_keys<BN / 8>(st, qs + warp * 16 * LDS, ks, ks + BN * LDS, 0, base, hi, lo, a.scale_log2);
        __syncthreads();
    }
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
}

// ---------------------------------------------------------------------------------- token shape
// items[i] = flat index of a token; grid (items, kv_heads * head_chunks, splits). With one split the
// result is final; otherwise (m, l) and the unnormalised sums go to the workspace.
__global__ void __launch_bounds__(THREADS) attention_tokens_kernel(AttnArgs a, const int* __restrict__ items, int head_chunks,
                                                                   int splits, float* __restrict__ ws_o, float* __restrict__ ws_ml) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);  // 16 rows
    bf16* kv = qs + 16 * LDS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int item = blockIdx.x, t = items[item], split = blockIdx.z;
    const int kvh = blockIdx.y / head_chunks, chunk = blockIdx.y - kvh * head_chunks;
    const int group = a.heads / a.kv_heads;
    const int first_head = kvh * group + chunk * 16;
    const int heads_here = min(16, group - chunk * 16);
    const int pos = a.positions[t];
    const int* table = a.block_table + (size_t)a.token_row[t] * a.table_width;
    const int need_lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int start = (need_lo / BN) * BN;
    const int n_tiles = (pos - start) / BN + 1;
    const int per_split = (n_tiles + splits - 1) / splits;
    const int first = split * per_split, last = min(n_tiles, first + per_split);

    for (int e = tid; e < 16 * CHUNKS; e += THREADS) {
        const int v = e / CHUNKS, c = e - v * CHUNKS;
        const bool valid = v < heads_here;
        cp_async16(qs + v * LDS + c * 8, valid ? a.q + (size_t)t * a.q_stride + (size_t)(first_head + v) * D + c * 8 : a.q, valid);
    }
    int hi[2], lo[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        hi[r] = ((lane >> 2) + r * 8 < heads_here) ? pos : -1;
        lo[r] = need_lo;
    }
    RowState st;
    st.init();
    // A ring of TOKEN_STAGES key/value tiles: TOKEN_STAGES - 1 tiles are in flight while one is consumed, which is
    // what keeps a block streaming from HBM (one tile in flight leaves it waiting a memory latency per tile).
    // A group is committed every iteration, empty or not, so that wait_group counts tiles.
#pragma unroll
    for (int s = 0; s < TOKEN_STAGES - 1; ++s) {
        if (first + s < last) {
            bf16* nk = kv + s * 2 * BN * LDS;
            load_kv_tile(nk, nk + BN * LDS, a.cache, table, a.table_width, start + (first + s) * BN, need_lo, pos, kvh, a.kv_heads, a.page_size,
                         a.pages, a.status);
        }
        cp_async_commit();
    }
    for (int it = first; it < last; ++it) {
        const int ahead = it + TOKEN_STAGES - 1;
        if (ahead < last) {
            bf16* nk = kv + ((ahead - first) % TOKEN_STAGES) * 2 * BN * LDS;
            load_kv_tile(nk, nk + BN * LDS, a.cache, table, a.table_width, start + ahead * BN, need_lo, pos, kvh, a.kv_heads, a.page_size,
                         a.pages, a.status);
        }
        cp_async_commit();
        cp_async_wait<TOKEN_STAGES - 1>();
        __syncthreads();
        bf16* ks = kv + ((it - first) % TOKEN_STAGES) * 2 * BN * LDS;
        const int base = start + it * BN;
        if (base + warp * 16 <= pos) process_keys<2>(st, qs, ks, ks + BN * LDS, warp * 16, base, hi, lo, a.scale_log2);
        __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();
    // merge the four warps (each saw a quarter of every tile) through shared memory
    float* wo = reinterpret_cast<float*>(kv);          // [4][16][D]
    float* wm = wo + 4 * 16 * D;                       // [4][16]
    float* wl = wm + 4 * 16;                           // [4][16]
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
    __syncthreads();
    for (int e = tid; e < heads_here * D; e += THREADS) {
        const int row = e / D, c = e - row * D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, wm[w * 16 + row]);
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = (wm[w * 16 + row] == -INFINITY) ? 0.f : exp2f(wm[w * 16 + row] - m);
            l += f * wl[w * 16 + row];
            o += f * wo[((size_t)w * 16 + row) * D + c];
        }
        const int head = first_head + row;
        if (splits == 1) {
            a.out[(size_t)t * a.out_stride + (size_t)head * D + c] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
        } else {
            const size_t slot = ((size_t)item * a.heads + head) * splits + split;
            ws_o[slot * D + c] = o;
            if (c == 0) { ws_ml[slot * 2] = m; ws_ml[slot * 2 + 1] = l; }
        }
    }
}

__global__ void attention_merge_kernel(const int* __restrict__ items, const float* __restrict__ ws_o, const float* __restrict__ ws_ml,
                                       bf16* __restrict__ out, int out_stride, int heads, int splits) {
    const int item = blockIdx.x, head = blockIdx.y, t = items[item];
    const size_t slot0 = ((size_t)item * heads + head) * splits;
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, ws_ml[(slot0 + s) * 2]);
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float l = 0.f, o = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ms = ws_ml[(slot0 + s) * 2];
            const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
            l += f * ws_ml[(slot0 + s) * 2 + 1];
            o += f * ws_o[(slot0 + s) * D + c];
        }
        out[(size_t)t * out_stride + (size_t)head * D + c] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
}

constexpr size_t TILES_SMEM = (size_t)(BM + 4 * BN) * LDS * sizeof(bf16);
constexpr size_t TOKENS_KV_SMEM = (size_t)TOKEN_STAGES * 2 * BN * LDS * sizeof(bf16);
constexpr size_t TOKENS_MERGE_SMEM = (size_t)(4 * 16 * D + 2 * 4 * 16) * sizeof(float);
constexpr size_t TOKENS_SMEM = 16 * LDS * sizeof(bf16) + (TOKENS_KV_SMEM > TOKENS_MERGE_SMEM ? TOKENS_KV_SMEM : TOKENS_MERGE_SMEM);

int fill_args(AttnArgs& a, const void* q, int q_stride, void* out, int out_stride, const void* cache, const int* block_table,
              int table_width, const int* token_row, const int* positions, int heads, int kv_heads, int head_dim, int page_size,
              int pages, float scale, int window, int* status) {
    if (head_dim != D) return HB_UNSUPPORTED_SIZE;
    if (kv_heads <= 0 || heads % kv_heads || page_size <= 0 || q_stride % 8 || out_stride % 2) return HB_BAD_ARGUMENT;
    if (page_size & (page_size - 1)) return HB_UNSUPPORTED_SIZE;  // pages hold a power of two of tokens
    if (((uintptr_t)q | (uintptr_t)cache) & 15) return HB_BAD_ARGUMENT;
    a = AttnArgs{(const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)cache, block_table, table_width, token_row, positions,
                 heads, kv_heads, page_size, pages, window, scale * 1.4426950408889634f, status};
    return 0;
}
}  // namespace

HB_EXPORT int hb_attention_head_dim() { return D; }

// Tokens per tile for a group size: the planner on the host cuts rows into tiles of this many tokens.
HB_EXPORT int hb_attention_tile_tokens(int heads, int kv_heads) {
    const int group = heads / kv_heads;
    return BM / (group < BM ? group : BM);
}

HB_EXPORT int hb_attention_tiles(const void* q, int q_stride, void* out, int out_stride, const void* cache, const int* block_table,
                                 int table_width, const int* token_row, const int* positions, const int* tiles, int n_tiles, int heads,
                                 int kv_heads, int head_dim, int page_size, int pages, float scale, int window, int* status,
                                 cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    AttnArgs a;
    if (int code = fill_args(a, q, q_stride, out, out_stride, cache, block_table, table_width, token_row, positions, heads, kv_heads,
                             head_dim, page_size, pages, scale, window, status)) return code;
    const int group = heads / kv_heads, gc = group < BM ? group : BM, head_chunks = (group + gc - 1) / gc;
    if ((long long)kv_heads * head_chunks > 65535) return HB_UNSUPPORTED_SIZE;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tiles_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TILES_SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    attention_tiles_kernel<<<dim3(n_tiles, kv_heads * head_chunks), THREADS, TILES_SMEM, stream>>>(a, tiles, gc, head_chunks);
    return launch_status();
}

// Workspace floats needed by hb_attention_tokens for n_items tokens and `splits` splits.
HB_EXPORT long long hb_attention_tokens_workspace(int n_items, int heads, int splits) {
    return splits <= 1 ? 0 : (long long)n_items * heads * splits * (D + 2);
}

HB_EXPORT int hb_attention_tokens(const void* q, int q_stride, void* out, int out_stride, const void* cache, const int* block_table,
                                  int table_width, const int* token_row, const int* positions, const int* items, int n_items, int splits,
                                  float* workspace, int heads, int kv_heads, int head_dim, int page_size, int pages, float scale,
                                  int window, int* status, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    AttnArgs a;
    if (int code = fill_args(a, q, q_stride, out, out_stride, cache, block_table, table_width, token_row, positions, heads, kv_heads,
                             head_dim, page_size, pages, scale, window, status)) return code;
    const int group = heads / kv_heads, head_chunks = (group + 15) / 16;
    if (splits < 1 || splits > 65535 || (long long)kv_heads * head_chunks > 65535 || (splits > 1 && !workspace)) return HB_BAD_ARGUMENT;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tokens_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TOKENS_SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    float* ws_o = workspace;
    float* ws_ml = workspace ? workspace + (size_t)n_items * heads * splits * D : nullptr;
    attention_tokens_kernel<<<dim3(n_items, kv_heads * head_chunks, splits), THREADS, TOKENS_SMEM, stream>>>(a, items, head_chunks, splits, ws_o, ws_ml);
    int code = launch_status();
    if (code || splits == 1) return code;
    attention_merge_kernel<<<dim3(n_items, heads), D < 64 ? 32 : (D < 128 ? 64 : 128), 0, stream>>>(items, ws_o, ws_ml, (bf16*)out, out_stride, heads, splits);
    return launch_status();
}
