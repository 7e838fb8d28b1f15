// Prompt attention on the 5th-generation tensor cores: causal grouped-query attention of a tile of 128
// "virtual rows" (tokens x heads of one key/value group) over the paged bfloat16 cache, with S = Q K^T and
// O += P V issued as tcgen05.mma and S and O living in tensor memory.  Head sizes 64 and 128 (HB_HEAD_DIM),
// pages of 8 to 64 tokens.
//
// Roles in a block of 192 threads:
//   warp 0      producer: one cp.async.bulk.tensor per page and 64-column panel into a ring of key/value stages
//               (the same layout and barriers as attention_tma.cu);
//   warp 1      owns tensor memory and issues the products: S_j = Q K_j^T (M 128, N 64, K = head size) into one of
//               two S buffers, and O += P_j V_j (M 128, N = head size, K 64) with V as an MN-major operand.  S_{j+1}
//               is issued before P_j is waited for, so the tensor cores work while the softmax warps do;
//   warps 2-5   softmax: thread r owns row r (tensor-memory lane r).  It reads S_j with tcgen05.ld, masks and scales
//               into the exp2 domain, keeps a running maximum and sum in float, writes P_j as bfloat16 into shared
//               memory in the swizzled K-major layout the product wants (after the previous product has finished
//               with that buffer), and rescales O in tensor memory only when
//               the maximum has grown by more than 2^8 (until then the stale maximum is kept, which changes no
//               result: the final division uses the same maximum for numerator and denominator).
// Every mbarrier wait is bounded; a wait that runs out sets HB_STATUS_WAIT_EXPIRED, all roles leave their loops, the block
// takes no further item, tensor memory is freed and the block returns.
//
// Counterpart in the reference: attention_mma_paged_*_bf16 (mma.sync m16n8k16, 64 x 64 tiles;
// helios/crates/helios-hal/kernels/elementwise.cu:576-729,749); mask: key position <= query position (:660-663).
#include <cuda.h>

#include "common.cuh"

#ifndef HB_HEAD_DIM
#define HB_HEAD_DIM 128
#endif

namespace {
typedef __nv_bfloat16 bf16;
constexpr int D = HB_HEAD_DIM;
static_assert(D == 64 || D == 128, "the tcgen05 attention takes head sizes 64 and 128");
constexpr int BM = 128;                       // virtual rows per block = tensor-memory lanes
constexpr int BN = 64;                        // keys per tile
constexpr int HALVES = D / 64;
constexpr int PANEL = BN * 64;                // elements of a 64-key x 64-column panel (8 KB)
constexpr int QPANEL = BM * 64;               // elements of a 128-row x 64-column panel of Q (16 KB)
constexpr int TILE_ELEMS = HALVES * PANEL;
constexpr int TILE_BYTES = TILE_ELEMS * 2;      // one K or one V tile
constexpr int STAGES = 2;                     // K tiles and V tiles have rings of their own: a K slot is free as soon as S is done,
                                              // so K is fetched two tiles ahead; with one P buffer two blocks fit an SM (2 x 112 KB)
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 256;                // S0 [0,64) S1 [64,128) O [128,128+D)
constexpr int O_COL = 128;
constexpr unsigned WAIT_LIMIT = 1u << 24;
constexpr float RESCALE_THRESHOLD = 8.0f;     // in the exp2 domain

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
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// The lane that issues the products is one thread, and a lone thread runs a few cycles per instruction: descriptor
// arithmetic between two products is time the tensor cores stand idle. So descriptors are kept as 32-bit low words that
// are only added to (the high word is the same for K-major and MN-major tiles with the 128-byte swizzle and 8-row groups
// 1,024 bytes apart), and the products of a tile are issued from one statement.
constexpr unsigned DESC_HIGH = (unsigned)(1024 >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ unsigned low_k_major(const void* tile) { return ((smem_u32(tile) & 0x3FFFFu) >> 4) | (1u << 16); }
__device__ __forceinline__ unsigned low_mn_major(const void* tile, unsigned panel_bytes) { return ((smem_u32(tile) & 0x3FFFFu) >> 4) | ((panel_bytes >> 4) << 16); }

// S = Q K^T over one 64-column panel of the head (4 products of 16 columns); `first` = 0 starts a new S.
__device__ __forceinline__ void umma_s_panel(unsigned tmem_d, unsigned q_low, unsigned k_low, unsigned idesc, unsigned first) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\t.reg .b32 al, bl;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 q, 0, 0;\n\t"
        "mov.b64 da, {%1, %5};\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t"
        "add.u32 al, %1, 2;\n\t"
        "add.u32 bl, %2, 2;\n\t"
        "mov.b64 da, {al, %5};\n\t"
        "mov.b64 db, {bl, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, q;\n\t"
        "add.u32 al, %1, 4;\n\t"
        "add.u32 bl, %2, 4;\n\t"
        "mov.b64 da, {al, %5};\n\t"
        "mov.b64 db, {bl, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, q;\n\t"
        "add.u32 al, %1, 6;\n\t"
        "add.u32 bl, %2, 6;\n\t"
        "mov.b64 da, {al, %5};\n\t"
        "mov.b64 db, {bl, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, q;\n\t}"
        ::"r"(tmem_d), "r"(q_low), "r"(k_low), "r"(idesc), "r"(first), "r"(DESC_HIGH) : "memory");
}
// O += P V over the 64 keys of a tile: 4 products of 16 keys, P from tensor memory (8 columns per 16 keys), V MN-major
// (16 keys = two 8-key groups = 2,048 bytes = 128 units of the descriptor's address field).
__device__ __forceinline__ void umma_pv_tile(unsigned tmem_o, unsigned tmem_p, unsigned v_low, unsigned idesc, unsigned first) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .b64 db;\n\t.reg .b32 bl, pa;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 q, 0, 0;\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t"
        "add.u32 bl, %2, 128;\n\t"
        "add.u32 pa, %1, 8;\n\t"
        "mov.b64 db, {bl, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [pa], db, %3, q;\n\t"
        "add.u32 bl, %2, 256;\n\t"
        "add.u32 pa, %1, 16;\n\t"
        "mov.b64 db, {bl, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [pa], db, %3, q;\n\t"
        "add.u32 bl, %2, 384;\n\t"
        "add.u32 pa, %1, 24;\n\t"
        "mov.b64 db, {bl, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [pa], db, %3, q;\n\t}"
        ::"r"(tmem_o), "r"(tmem_p), "r"(v_low), "r"(idesc), "r"(first), "r"(DESC_HIGH) : "memory");
}
__device__ __forceinline__ void umma_commit_at(unsigned bar_addr) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
}
// float accumulator, bfloat16 operands, A K-major, M 128, N n; B MN-major when b_mn.
__device__ __forceinline__ unsigned idesc_for(int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((unsigned)(n >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
}
__device__ __forceinline__ void tmem_ld16(unsigned taddr, float (&v)[16]) {
    unsigned r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// 64 consecutive float columns of this thread's lane in one instruction.
__device__ __forceinline__ void tmem_ld64(unsigned taddr, float (&v)[64]) {
    unsigned r[64];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
        "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]),
          "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]),
          "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]),
          "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
// 2^x by the hardware approximation (inputs are <= 8 here; -inf gives 0).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_st16(unsigned taddr, const float (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
                   "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
                   "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                   "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
                 : "memory");
}

__device__ __forceinline__ void tmem_st16_words(unsigned taddr, const unsigned* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
                   "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
                 : "memory");
}

struct AttnArgs {
    const bf16* q; int q_stride;
    bf16* out; int out_stride;
    const int* block_table; int table_width;
    const int* positions;
    int heads, kv_heads, page_size, pages, window;
    float scale_log2;
    int* status;
};

// tiles[3*i] = first token (flat index), tiles[3*i+1] = token count, tiles[3*i+2] = batch row; virtual row v of a tile is
// token v / gc, head v % gc of the block's key/value group (gc = min(group, 128) heads per block).
//
// The blocks are persistent: a work item is (tile, key/value head and head chunk), item i being tile n_tiles - 1 - i / ys
// (within a prompt the later tiles walk more keys, so the long items come first), and every block takes the next item
// from a counter in global memory when it has finished one. A prompt's first tile walks one tile of keys and its last
// tile all of them; with one block per item the longest item alone set the kernel's time (32 key tiles in a row for a
// 2,048-token prompt), now the items spread evenly over the blocks. `work` = {next item, blocks that have finished}:
// the block that finishes last sets both back to zero for the next launch in the stream.
__global__ void __launch_bounds__(THREADS) attention_tc_kernel(const __grid_constant__ CUtensorMap kv_map, const AttnArgs a,
                                                               const int* __restrict__ tiles, int n_work_tiles, int ys, int gc, int head_chunks,
                                                               int* __restrict__ work) {
    // The swizzled tiles need a 1024-byte aligned base; where dynamic shared memory starts is not promised, so the
    // launch asks for 1 KB more and the base is rounded up.
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    let_next_kernel_start();
    unsigned char* k_ring = base;                                                   // STAGES K tiles
    unsigned char* v_ring = base + (size_t)STAGES * TILE_BYTES;                     // STAGES V tiles
    bf16* qs = reinterpret_cast<bf16*>(base + (size_t)2 * STAGES * TILE_BYTES);     // HALVES panels of 128 rows x 64
    unsigned long long* k_full = reinterpret_cast<unsigned long long*>(qs + HALVES * QPANEL);
    unsigned long long* k_empty = k_full + STAGES;
    unsigned long long* v_full = k_empty + STAGES;
    unsigned long long* v_empty = v_full + STAGES;
    unsigned long long* s_full = v_empty + STAGES;    // [2]
    unsigned long long* p_full = s_full + 2;          // [1]
    unsigned long long* o_done = p_full + 1;          // [1]
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(o_done + 1);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* item_slot = failed + 1;             // [2]: the item of this round and of the next

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int total_items = n_work_tiles * ys;
    const int group = a.heads / a.kv_heads;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        for (int b = 0; b < 2; ++b) mbar_init(&s_full[b], 1);
        mbar_init(p_full, 4);
        mbar_init(o_done, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Pages that a tile does not fetch (beyond the last position, before a window's start) leave under masked keys what
    // the stage held before: earlier keys and values, which are finite. The rings start as zeros so that this holds for
    // the first tiles too.
    for (int e = tid; e < 2 * STAGES * TILE_BYTES / 16; e += THREADS) reinterpret_cast<uint4*>(base)[e] = make_uint4(0, 0, 0, 0);
    wait_for_previous_kernels();  // the queries and the newest keys and values come from the kernel before; so does the counter's reset
    if (tid == 0) item_slot[0] = atomicAdd(&work[0], 1);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = *tmem_slot;
    const int shift = 31 - __clz(a.page_size);
    const unsigned idesc_s = idesc_for(BN, false), idesc_o = idesc_for(D, true);
    if (warp == 0 && lane == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&kv_map) : "memory");

    // g0: key tiles of the items before this one. Rings and barriers run on across items: stage g % STAGES, phase by g.
    int g0 = 0;
    for (int round = 0;; ++round) {
        const int item = item_slot[round & 1];
        if (item >= total_items || *failed) break;  // the same for every thread: both were written before the barrier behind us
        const int tile = n_work_tiles - 1 - item / ys, y = item % ys;
        const int tok0 = tiles[3 * tile], ntok = tiles[3 * tile + 1], brow = tiles[3 * tile + 2];
        const int kvh = y / head_chunks, chunk = y - kvh * head_chunks;
        const int first_head = kvh * group + chunk * gc;
        const int heads_here = min(gc, group - chunk * gc);
        const int* table = a.block_table + (size_t)brow * a.table_width;
        const int pos_first = a.positions[tok0], pos_last = pos_first + ntok - 1;
        const int need_lo = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
        const int start = (need_lo / BN) * BN;
        const int n_tiles = (pos_last - start) / BN + 1;

        // queries into the swizzled K-major panels: element (row v, column c) -> panel c / 64, row v, chunk ((c % 64) / 8) ^ (v % 8)
        // (every product of the item before has finished: its rows were read out of tensor memory before the barrier behind us)
        for (int e = tid; e < BM * (D / 8); e += THREADS) {
            const int v = e / (D / 8), cc = e - v * (D / 8);
            const int tok = v / gc, hh = v - tok * gc;
            uint4 value = make_uint4(0, 0, 0, 0);
            if (tok < ntok && hh < heads_here)
                value = *reinterpret_cast<const uint4*>(a.q + (size_t)(tok0 + tok) * a.q_stride + (size_t)(first_head + hh) * D + cc * 8);
            *reinterpret_cast<uint4*>(qs + (cc >> 3) * QPANEL + v * 64 + (((cc & 7) ^ (v & 7)) << 3)) = value;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        tc_fence_before();
        __syncthreads();
        tc_fence_after();

        if (warp == 0) {
            // ------------------------------------------------------------------ producer (whole warp)
            const int pages_per_tile = BN >> shift;
            const int ops = pages_per_tile * HALVES;
            const unsigned page_bytes = (unsigned)a.page_size * D * 2u;  // of one page of K, or of V
            bool alive = true;
            for (int it = 0; it < n_tiles && alive; ++it) {
                const int g = g0 + it, s = g % STAGES, turn = g / STAGES;
                const int tile_base = start + it * BN;
                int my_page = -1;
                const int k0 = tile_base + lane * a.page_size;
                if (lane < pages_per_tile && k0 <= pos_last && k0 + a.page_size - 1 >= need_lo) {
                    const int block = k0 >> shift;
                    const int id = block < a.table_width ? __ldg(table + block) : -1;
                    if (id >= 0 && id < a.pages) my_page = id;
                    else atomicOr(a.status, HB_STATUS_BAD_PAGE);
                }
                const unsigned valid = __popc(__ballot_sync(0xffffffffu, my_page >= 0));
                for (int which = 0; which < 2 && alive; ++which) {  // the K tile, then the V tile
                    unsigned long long* full = which ? &v_full[s] : &k_full[s];
                    int ok = 1;
                    if (lane == 0) ok = mbar_wait(which ? &v_empty[s] : &k_empty[s], (turn & 1) ^ 1, failed) ? 1 : 0;
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) { if (lane == 0) *failed = 1; alive = false; break; }
                    if (lane == 0) {
                        if (valid) mbar_expect_tx(full, valid * page_bytes); else mbar_arrive(full);
                    }
                    __syncwarp();
                    bf16* stage = reinterpret_cast<bf16*>((which ? v_ring : k_ring) + (size_t)s * TILE_BYTES);
                    for (int op0 = 0; op0 < ops; op0 += 32) {
                        const int op = op0 + lane;
                        const int p = min(op, ops - 1) / HALVES, h = op % HALVES;
                        const int page = __shfl_sync(0xffffffffu, my_page, p);
                        if (op < ops && page >= 0)
                            tma_load_2d(stage + h * PANEL + p * a.page_size * 64, &kv_map, full, h * 64,
                                        ((page * 2 + which) * a.kv_heads + kvh) * a.page_size);
                    }
                }
            }
            // the next item, taken while the others still work on this one (they read this round's slot long ago: nobody
            // passes the barrier at the end of the round before every thread is there)
            if (lane == 0) item_slot[(round + 1) & 1] = *failed ? total_items : atomicAdd(&work[0], 1);
        } else if (warp == 1) {
            // ------------------------------------------------------------------ tensor-core issuer (one lane)
            if (lane == 0) {
                bool ok = true;
                const unsigned q_low = low_k_major(qs), k_low0 = low_k_major(k_ring), v_low0 = low_mn_major(v_ring, PANEL * 2);
                const unsigned k_empty0 = smem_u32(&k_empty[0]), v_empty0 = smem_u32(&v_empty[0]), s_full0 = smem_u32(&s_full[0]), o_done_at = smem_u32(o_done);
                auto issue_s = [&](int g) {
                    const unsigned stage = (unsigned)(g % STAGES), k_low = k_low0 + stage * (TILE_BYTES >> 4);
                    umma_s_panel(tmem + (g & 1) * BN, q_low, k_low, idesc_s, 0u);
                    if (HALVES == 2) umma_s_panel(tmem + (g & 1) * BN, q_low + (QPANEL * 2 >> 4), k_low + (PANEL * 2 >> 4), idesc_s, 1u);
                    umma_commit_at(k_empty0 + 8u * stage);  // the K slot is free once this product has read it
                    umma_commit_at(s_full0 + 8u * (unsigned)(g & 1));
                };
                if (!mbar_wait(&k_full[g0 % STAGES], (g0 / STAGES) & 1, failed)) { *failed = 1; ok = false; }
                if (ok) { tc_fence_after(); issue_s(g0); }
                for (int j = 0; j < n_tiles && ok; ++j) {
                    const int g = g0 + j;
                    if (j + 1 < n_tiles) {
                        if (!mbar_wait(&k_full[(g + 1) % STAGES], ((g + 1) / STAGES) & 1, failed)) { *failed = 1; ok = false; break; }
                        // S(g + 1) lands in the columns that P(g - 1) was read from: the product that read it must be over
                        // (for the item's first tile it is: the item before ended with every product done)
                        if (j > 0 && !mbar_wait(o_done, (g - 1) & 1, failed)) { *failed = 1; ok = false; break; }
                        tc_fence_after();
                        issue_s(g + 1);
                    }
                    if (!mbar_wait(p_full, g & 1, failed)) { *failed = 1; ok = false; break; }
                    if (!mbar_wait(&v_full[g % STAGES], (g / STAGES) & 1, failed)) { *failed = 1; ok = false; break; }
                    tc_fence_after();
                    // P(g) lies in tensor memory over the first half of S(g)'s columns: 16 keys = 8 columns per product
                    const unsigned stage = (unsigned)(g % STAGES);
                    umma_pv_tile(tmem + O_COL, tmem + (g & 1) * BN, v_low0 + stage * (TILE_BYTES >> 4), idesc_o, j > 0 ? 1u : 0u);
                    umma_commit_at(v_empty0 + 8u * stage);
                    umma_commit_at(o_done_at);
                }
            }
        } else {
            // ------------------------------------------------------------------ softmax: thread = row = tensor-memory lane
            const int quarter = warp & 3;
            const int r = quarter * 32 + lane;
            const unsigned lane_addr = tmem + ((unsigned)(quarter * 32) << 16);
            const int tok = r / gc, hh = r - tok * gc;
            const bool row_valid = tok < ntok && hh < heads_here;
            const int hi = row_valid ? pos_first + tok : -1;
            const int lo = (row_valid && a.window > 0) ? max(0, hi - a.window + 1) : 0;
            float m = -INFINITY, l = 0.f;
            bool ok = true;
            for (int j = 0; j < n_tiles; ++j) {
                const int g = g0 + j, b = g & 1;
                if (!mbar_wait(&s_full[b], (g >> 1) & 1, failed)) { *failed = 1; ok = false; break; }
                tc_fence_after();
                float s[BN];
                tmem_ld64(lane_addr + b * BN, s);
                const int tile_base = start + j * BN;
                float tmax = -INFINITY;
                if (tile_base + BN - 1 <= hi && tile_base >= lo) {  // every key of the tile is visible to this row
#pragma unroll
                    for (int i = 0; i < BN; ++i) {
                        s[i] *= a.scale_log2;
                        tmax = fmaxf(tmax, s[i]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < BN; ++i) {
                        const int pos = tile_base + i;
                        s[i] = (pos <= hi && pos >= lo) ? s[i] * a.scale_log2 : -INFINITY;
                        tmax = fmaxf(tmax, s[i]);
                    }
                }
                const float m_new = fmaxf(m, tmax);
                float alpha = 1.f;
                if (m == -INFINITY) {
                    m = m_new;  // nothing visible so far: the row of O holds zeros (or is overwritten by the first product), no rescale
                } else if (m_new - m > RESCALE_THRESHOLD) {
                    alpha = exp2f(m - m_new);
                    m = m_new;
                }
                const float m_use = (m == -INFINITY) ? 0.f : m;
                float sum = 0.f;
                uint4 packed[BN / 8];
#pragma unroll
                for (int c = 0; c < BN / 8; ++c) {
                    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&packed[c]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float p0 = fast_exp2(s[c * 8 + 2 * e] - m_use), p1 = fast_exp2(s[c * 8 + 2 * e + 1] - m_use);
                        sum += p0 + p1;
                        h2[e] = __floats2bfloat162_rn(p0, p1);
                    }
                }
                l = l * alpha + sum;
                // P(g) goes into this thread's lane over the columns S(g) came from (the thread holds its S row in registers;
                // the tensor core writes those columns again only with S(g + 2), issued after the product that reads P(g))
                const unsigned* words = reinterpret_cast<const unsigned*>(packed);
                tmem_st16_words(lane_addr + b * BN, words);
                tmem_st16_words(lane_addr + b * BN + 16, words + 16);
                // Every thread sees every phase of o_done go by, tile by tile: a wait by parity tells "phase g - 1 is over" only
                // to a thread that knows phase g - 2 is (a thread two phases behind would read the parity of a later phase as
                // "not yet" and wait for ever). Here phase g - 2 was waited for one tile ago (or, at an item's second tile, at
                // the end of the item before) and the product of tile g cannot start before this thread hands P(g) over, so
                // the barrier is in phase g - 1 or g. The product of tile g - 1 was issued a whole tile ago; the wait is
                // almost always over at the first look.
                if (j > 0 && !mbar_wait(o_done, (g - 1) & 1, failed)) { *failed = 1; ok = false; break; }
                if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                    // O may be rescaled only between two products: the one before is done
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < D; c += 16) {
                        float o[16];
                        tmem_ld16(lane_addr + O_COL + c, o);
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] *= alpha;
                        tmem_st16(lane_addr + O_COL + c, o);
                    }
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full);
            }
            // every phase but the item's last was seen in the loop
            if (ok) ok = mbar_wait(o_done, (g0 + n_tiles - 1) & 1, failed);
            if (!ok) *failed = 1;
            tc_fence_after();
            if (ok) {
                const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
                for (int c = 0; c < D; c += 16) {
                    float o[16];
                    tmem_ld16(lane_addr + O_COL + c, o);
                    if (row_valid) {
                        uint4 w[2];
                        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(w);
#pragma unroll
                        for (int i = 0; i < 8; ++i) h2[i] = __floats2bfloat162_rn(o[2 * i] * inv, o[2 * i + 1] * inv);
                        uint4* dst = reinterpret_cast<uint4*>(a.out + (size_t)(tok0 + tok) * a.out_stride + (size_t)(first_head + hh) * D + c);
                        dst[0] = w[0];
                        dst[1] = w[1];
                    }
                }
            }
        }
        g0 += n_tiles;
        // the end of the round: every product of this item is over (the softmax threads saw the last one finish and have
        // read their rows), the next item's number is in its slot
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
    }
    if (tid == 0) {
        if (*failed) atomicOr(a.status, HB_STATUS_WAIT_EXPIRED | HB_STATUS_IN_ATTENTION_TCGEN05);
        __threadfence();
        if (atomicAdd(&work[1], 1) == (int)gridDim.x - 1) {  // the last block to finish: every block has taken its last number
            work[0] = 0;
            work[1] = 0;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
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

constexpr size_t SMEM_USED = 1024 + (size_t)2 * STAGES * TILE_BYTES + (size_t)HALVES * QPANEL * sizeof(bf16) + (4 * STAGES + 4) * 8 + 32;
// A block holds half of the SM's tensor memory, so two blocks are all an SM can serve. The launch asks for at least
// 80 KB of shared memory so that no third block becomes resident only to wait for tensor memory: such a block of a
// kernel launched early (as a programmatic dependent) would hold what a block of the kernel before it still needs.
constexpr size_t SMEM_BYTES = SMEM_USED > 80 * 1024 ? SMEM_USED : 80 * 1024;
}  // namespace

// Rows of a tile (tokens x heads of a group) this kernel wants: the host planner cuts rows into tiles of
// 128 / min(group, 128) tokens.
HB_EXPORT int hb_attention_tc_tile_rows() { return BM; }

HB_EXPORT int hb_attention_tc_tiles(const void* q, int q_stride, void* out, int out_stride, const void* cache, const int* block_table,
                                    int table_width, const int* token_row, const int* positions, const int* tiles, int n_tiles, int heads,
                                    int kv_heads, int head_dim, int page_size, int pages, float scale, int window, int* status,
                                    int* work, cudaStream_t stream) {
    (void)token_row;
    if (!work) return HB_BAD_ARGUMENT;
    if (n_tiles <= 0) return 0;
    if (head_dim != D) return HB_UNSUPPORTED_SIZE;
    if (kv_heads <= 0 || heads % kv_heads || q_stride % 8 || out_stride % 8) return HB_BAD_ARGUMENT;
    if (page_size < 8 || page_size > 64 || (page_size & (page_size - 1))) return HB_UNSUPPORTED_SIZE;
    if (((uintptr_t)q | (uintptr_t)cache | (uintptr_t)out) & 15) return HB_BAD_ARGUMENT;
    EncodeTiled encode = encode_tiled();
    if (!encode) return HB_BAD_ARGUMENT;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)pages * 2 * kv_heads * page_size};
    const cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
    const cuuint32_t elem[2] = {1, 1};
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return HB_BAD_ARGUMENT;
    AttnArgs a{(const bf16*)q, q_stride, (bf16*)out, out_stride, block_table, table_width, positions,
               heads, kv_heads, page_size, pages, window, scale * 1.4426950408889634f, status};
    const int group = heads / kv_heads, gc = group < BM ? group : BM, head_chunks = (group + gc - 1) / gc;
    if ((long long)kv_heads * head_chunks > 65535) return HB_UNSUPPORTED_SIZE;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    // two blocks fit an SM (tensor memory, shared memory): that many persistent blocks, or one per item if there are fewer
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
        return HB_BAD_ARGUMENT;
    const long long items = (long long)n_tiles * kv_heads * head_chunks;
    if (items > 0x7fffffffLL) return HB_UNSUPPORTED_SIZE;
    const int blocks = (int)(items < 2LL * sms ? items : 2LL * sms);
    return launch_after_previous(attention_tc_kernel, dim3(blocks), THREADS, SMEM_BYTES, stream, map, a, tiles, n_tiles, kv_heads * head_chunks, gc,
                                 head_chunks, work);
}
