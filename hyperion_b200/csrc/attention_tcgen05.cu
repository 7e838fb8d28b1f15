// Prompt attention on the 5th-generation tensor cores: causal grouped-query attention of a tile of 256
// "virtual rows" (tokens x heads of one key/value group) over the paged bfloat16 cache, with S = Q K^T and
// O += P V issued as tcgen05.mma and S, P and O living in tensor memory.  Head sizes 64 and 128 (HB_HEAD_DIM),
// pages of 8 to 64 tokens.
//
// One block per SM holds all of the SM's tensor memory and works on two halves of 128 rows (H and L) that walk the
// same key tiles of 128 keys.  While the softmax threads of one half work on their S, the tensor core runs the other
// half's products, so neither stands still for long:
//   warp 0      producer: one cp.async.bulk.tensor per page and 64-column panel into rings of key and of value tiles, and
//               the item's queries as one 3-D box per panel (columns x heads of the group x tokens of the tile), which
//               lands the rows token x head in the swizzled K-major layout the products read;
//   warp 1      issues the products, per key tile and half: O_x += P_x V (M 128, N = head size, K 128, P read from
//               tensor memory, V an MN-major operand) as soon as the half's softmax threads have handed P over, then
//               at once S_x = Q_x K_next^T (M 128, N 128, K = head size) into the columns P_x was read from (products
//               of one thread run in the order they were issued);
//   warps 2-5   softmax of half H, warps 6-9 of half L: thread r owns row r (tensor-memory lane r).  It reads its S row
//               with tcgen05.ld, masks, keeps a running maximum and sum in float, writes P as bfloat16 over the first
//               half of S's columns, and rescales O only when the maximum has grown by more than 2^8 (until then the
//               stale maximum is kept, which changes no result: the final division uses the same maximum for
//               numerator and denominator).
// A product of 64 keys cannot feed the tensor core: it is bound by reading Q out of shared memory (measured: 54 clocks
// for M 128, N 64, K 16 against 64 for N 128, which does twice the arithmetic), and the hand-overs between the roles
// cost the same per tile whatever its width; hence tiles of 128 keys.
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
constexpr int BM = 128;                       // rows of one half = tensor-memory lanes
constexpr int ROWS = 2 * BM;                  // virtual rows of a tile
constexpr int BN = 128;                       // keys per tile
constexpr int PANELS = D / 64;
constexpr int KV_PANEL = BN * 64;             // elements of a 128-key x 64-column panel (16 KB)
constexpr int Q_PANEL = ROWS * 64;            // elements of a 256-row x 64-column panel of Q (32 KB)
constexpr int TILE_BYTES = PANELS * KV_PANEL * 2;  // one K or one V tile
constexpr int STAGES = 2;                     // K tiles and V tiles have rings of their own: a K slot is free as soon as both S are done
constexpr int THREADS = 320;
constexpr int TMEM_COLS = 512;                // S_H [0,128) S_L [128,256) O_H [256,256+D) O_L [384,384+D); P_x over S_x's first 64 columns
constexpr int O_COL = 256;
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
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, unsigned long long* bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// The lane that issues the products is one thread, and a lone thread runs a few cycles per instruction: descriptor
// arithmetic between two products is time the tensor cores stand idle. So descriptors are kept as 32-bit low words that
// are only added to (the high word is the same for K-major and MN-major tiles with the 128-byte swizzle and 8-row groups
// 1,024 bytes apart), and four products are issued from one statement.
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
// O += P V over 64 keys: 4 products of 16 keys, P from tensor memory (8 columns per 16 keys), V MN-major
// (16 keys = two 8-key groups = 2,048 bytes = 128 units of the descriptor's address field).
__device__ __forceinline__ void umma_pv_64(unsigned tmem_o, unsigned tmem_p, unsigned v_low, unsigned idesc, unsigned first) {
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
__device__ __forceinline__ void tmem_ld64(unsigned taddr, float* v) {
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
__device__ __forceinline__ unsigned pack_bf16x2(float lo, float hi) {
    unsigned w;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(hi), "f"(lo));
    return w;
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
    int wide_stores;  // rows of the output start on 32-byte boundaries
};

// tiles[3*i] = first token (flat index), tiles[3*i+1] = token count, tiles[3*i+2] = batch row; virtual row v of a tile is
// token v / gc, head v % gc of the block's key/value group (gc = min(group, 256) heads per block); rows 0-127 are half
// H, rows 128-255 half L. A tile of at most 128 rows runs half H alone.
//
// The blocks are persistent: a work item is (tile, key/value head and head chunk), item i being tile n_tiles - 1 - i / ys
// (within a prompt the later tiles walk more keys, so the long items come first), and every block takes the next item
// from a counter in global memory when it has finished one. A prompt's first tile walks one tile of keys and its last
// tile all of them; with one block per item the longest item alone would set the kernel's time, now the items spread
// evenly over the blocks. `work` = {items handed out beyond every block's first, blocks that have finished}: the block
// that finishes last sets both back to zero for the next launch in the stream.
__global__ void __launch_bounds__(THREADS, 1) attention_tc_kernel(const __grid_constant__ CUtensorMap kv_map, const __grid_constant__ CUtensorMap q_map,
                                                                  const AttnArgs a,
                                                                  const int* __restrict__ tiles, int n_work_tiles, int ys, int gc, int head_chunks,
                                                                  int* __restrict__ work) {
    // The swizzled tiles need a 1024-byte aligned base; where dynamic shared memory starts is not promised, so the
    // launch asks for 1 KB more and the base is rounded up.
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    let_next_kernel_start();
    unsigned char* k_ring = base;                                                   // STAGES K tiles
    unsigned char* v_ring = base + (size_t)STAGES * TILE_BYTES;                     // STAGES V tiles
    bf16* qs = reinterpret_cast<bf16*>(base + (size_t)2 * STAGES * TILE_BYTES);     // PANELS panels of 256 rows x 64
    unsigned long long* k_full = reinterpret_cast<unsigned long long*>(qs + PANELS * Q_PANEL);
    unsigned long long* k_empty = k_full + STAGES;
    unsigned long long* v_full = k_empty + STAGES;
    unsigned long long* v_empty = v_full + STAGES;
    unsigned long long* s_full = v_empty + STAGES;    // [2]: per half
    unsigned long long* p_full = s_full + 2;          // [2]
    unsigned long long* o_done = p_full + 2;          // [2]
    unsigned long long* q_full = o_done + 2;          // [1]: the item's queries have landed
    unsigned long long* q_empty = q_full + 1;         // [1]: the item's last S has been computed
    unsigned long long* round_done = q_empty + 1;     // [1]: the eight softmax warps have finished the item
    unsigned long long* q_seen = round_done + 1;      // [1]: the eight softmax warps have seen the item's queries land
    const int total_items = n_work_tiles * ys;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(q_seen + 1);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // [4][5]: the items in flight, each with what every thread wants to know of it (item, first token, token count, batch
    // row, first position), fetched by the producer while the item before is still being worked on
    volatile int* item_slot = failed + 1;
    auto note_item = [&](int slot, int item) {  // one thread
        volatile int* info = item_slot + 5 * slot;
        info[0] = item;
        if (item < total_items) {
            const int tile = n_work_tiles - 1 - item / ys;
            const int tok0 = tiles[3 * tile];
            info[1] = tok0;
            info[2] = tiles[3 * tile + 1];
            info[3] = tiles[3 * tile + 2];
            info[4] = a.positions[tok0];
        }
    };
    // A block's first item is the one of its own number (the grid has no more blocks than there are items); the counter
    // hands out the items after those.
    auto take_item = [&](int slot) { note_item(slot, *failed ? total_items : (int)gridDim.x + atomicAdd(&work[0], 1)); };

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = a.heads / a.kv_heads;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        for (int x = 0; x < 2; ++x) { mbar_init(&s_full[x], 1); mbar_init(&p_full[x], 4); mbar_init(&o_done[x], 1); }
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        mbar_init(round_done, 8);
        mbar_init(q_seen, 8);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Pages that a tile does not fetch (beyond the last position, before a window's start) leave under masked keys what
    // the stage held before: earlier keys and values, which are finite. The rings start as zeros so that this holds for
    // the first tiles too. The rows of Q that no copy writes (beyond tokens x heads of a tile) are never stored; they start
    // as zeros all the same.
    for (int e = tid; e < (2 * STAGES * TILE_BYTES + PANELS * Q_PANEL * 2) / 16; e += THREADS) reinterpret_cast<uint4*>(base)[e] = make_uint4(0, 0, 0, 0);
    // what the first item is needs nothing of the kernel before: the tiles and positions were copied in at the step's start
    if (tid == 0) note_item(0, (int)blockIdx.x);
    wait_for_previous_kernels();  // the queries and the newest keys and values come from the kernel before; so does the counter's reset
    // All of the SM's tensor memory, and only now: a block of a kernel further back in the stream that has yet to start
    // on this SM can no longer want any.
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = *tmem_slot;
    const int shift = 31 - __clz(a.page_size);
    const unsigned idesc_s = idesc_for(BN, false), idesc_o = idesc_for(D, true);
    if (warp == 0 && lane == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&kv_map) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&q_map) : "memory");
    }
    const int tokens_per_tile = ROWS / gc;

    // The roles run through the items each at its own pace, held together by the barriers of the data alone: the producer
    // fetches the next item's keys while the last tiles of this one are worked on, its queries as soon as this item's last
    // S has been issued, and the first S of the next item follows the last product of this one without a pause.
    // g0: key tiles of the items before this one; the rings of K and V run on across items (stage g % STAGES, phase by g).
    // h0[x]: key tiles half x has seen; its three barriers change phase once per tile of an item the half takes part in.
    struct Item { int tok0, ntok, kvh, first_head, heads_here, pos_first, pos_last, need_lo, start, n_tiles, halves; const int* table; };
    auto read_item = [&](int round, Item& it) -> bool {  // false: no item left
        volatile int* info = item_slot + 5 * (round & 3);
        const int item = info[0];
        if (item >= total_items) return false;
        const int y = item % ys;
        it.tok0 = info[1];
        it.ntok = info[2];
        it.table = a.block_table + (size_t)info[3] * a.table_width;
        it.kvh = y / head_chunks;
        const int chunk = y - it.kvh * head_chunks;
        it.first_head = it.kvh * group + chunk * gc;
        it.heads_here = min(gc, group - chunk * gc);
        it.pos_first = info[4];
        it.pos_last = it.pos_first + it.ntok - 1;
        it.need_lo = a.window > 0 ? max(0, it.pos_first - a.window + 1) : 0;
        it.start = (it.need_lo / BN) * BN;
        it.n_tiles = (it.pos_last - it.start) / BN + 1;
        it.halves = it.ntok * gc > BM ? 2 : 1;
        return true;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ producer (whole warp)
        const int pages_per_tile = BN >> shift;
        const int ops = pages_per_tile * PANELS;
        const unsigned page_bytes = (unsigned)a.page_size * D * 2u;  // of one page of K, or of V
        bool alive = true;
        int g0 = 0;
        for (int round = 0; alive; ++round) {
            Item it;
            __syncwarp();  // lane 0 wrote the item's slot
            if (!read_item(round, it)) {
                // the others learn from the slot that nothing is left; this phase of q_full, like every other, may only
                // complete once every waiter has seen the one before
                if (lane == 0) {
                    if (mbar_wait(q_empty, (round & 1) ^ 1, failed) && mbar_wait(q_seen, (round & 1) ^ 1, failed)) mbar_arrive(q_full);
                    else *failed = 1;
                }
                break;
            }
            // The item's queries: a box of (64 columns, gc heads, tokens of a tile) per panel lands as rows token x head of
            // 128 bytes, swizzled like every K-major operand. Tokens beyond the tile's own (another request's, or none) and
            // heads beyond the group's come along or are filled with zeros; their rows are never stored. The buffer is free
            // once the last S of the item before has been computed. And every thread that waits for q_full has to have seen
            // the phase before go by: an item of one key tile has its only S issued before the softmax threads need look
            // at their barrier, and a phase that completes twice behind a waiter's back looks to it like one that has not.
            if (lane == 0) {
                if (!mbar_wait(q_empty, (round & 1) ^ 1, failed) || !mbar_wait(q_seen, (round & 1) ^ 1, failed)) { *failed = 1; alive = false; }
                if (alive) {
                    mbar_expect_tx(q_full, (unsigned)(PANELS * 128 * gc * tokens_per_tile));
                    for (int h = 0; h < PANELS; ++h) tma_load_3d(qs + h * Q_PANEL, &q_map, q_full, h * 64, it.first_head, it.tok0);
                }
            }
            alive = __shfl_sync(0xffffffffu, alive ? 1 : 0, 0) != 0;
            for (int t = 0; t < it.n_tiles && alive; ++t) {
                const int g = g0 + t, s = g % STAGES, turn = g / STAGES;
                const int tile_base = it.start + t * BN;
                int my_page = -1;
                const int k0 = tile_base + lane * a.page_size;
                if (lane < pages_per_tile && k0 <= it.pos_last && k0 + a.page_size - 1 >= it.need_lo) {
                    const int block = k0 >> shift;
                    const int id = block < a.table_width ? __ldg(it.table + block) : -1;
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
                        const int p = min(op, ops - 1) / PANELS, h = op % PANELS;
                        const int page = __shfl_sync(0xffffffffu, my_page, p);
                        if (op < ops && page >= 0)
                            tma_load_2d(stage + h * KV_PANEL + p * a.page_size * 64, &kv_map, full, h * 64,
                                        ((page * 2 + which) * a.kv_heads + it.kvh) * a.page_size);
                    }
                }
            }
            g0 += it.n_tiles;
            // the next item and what the others want to know of it; its slot was last read four items ago
            if (lane == 0 && alive) take_item((round + 1) & 3);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ tensor-core issuer (one lane)
        if (lane == 0) {
            bool ok = true;
            const unsigned q_low0 = low_k_major(qs), k_low0 = low_k_major(k_ring), v_low0 = low_mn_major(v_ring, KV_PANEL * 2);
            const unsigned k_empty0 = smem_u32(&k_empty[0]), v_empty0 = smem_u32(&v_empty[0]), s_full0 = smem_u32(&s_full[0]), o_done0 = smem_u32(&o_done[0]);
            const unsigned q_empty_at = smem_u32(q_empty);
            auto issue_s = [&](int x, int g) {  // S_x = Q_x K(g)^T
                const unsigned k_low = k_low0 + (unsigned)(g % STAGES) * (TILE_BYTES >> 4), q_low = q_low0 + (unsigned)x * (BM * 128 >> 4);
                umma_s_panel(tmem + x * BN, q_low, k_low, idesc_s, 0u);
                if (PANELS == 2) umma_s_panel(tmem + x * BN, q_low + (Q_PANEL * 2 >> 4), k_low + (KV_PANEL * 2 >> 4), idesc_s, 1u);
                umma_commit_at(s_full0 + 8u * (unsigned)x);
            };
            auto issue_pv = [&](int x, int g, unsigned accumulate) {  // O_x (+)= P_x V(g); P_x lies over the first 64 columns of S_x
                const unsigned v_low = v_low0 + (unsigned)(g % STAGES) * (TILE_BYTES >> 4);
                umma_pv_64(tmem + O_COL + x * BM, tmem + x * BN, v_low, idesc_o, accumulate);
                umma_pv_64(tmem + O_COL + x * BM, tmem + x * BN + 32, v_low + 512, idesc_o, 1u);
                umma_commit_at(o_done0 + 8u * (unsigned)x);
            };
            int g0 = 0, h0[2] = {0, 0};
            for (int round = 0; ok; ++round) {
                Item it;
                if (!mbar_wait(q_full, round & 1, failed)) { *failed = 1; break; }
                if (!read_item(round, it)) break;
                const int halves = it.halves, n_tiles = it.n_tiles;
                if (!mbar_wait(&k_full[g0 % STAGES], (g0 / STAGES) & 1, failed)) { *failed = 1; break; }
                tc_fence_after();
                // S_x of the first tile lands in the columns the last product of the item before read its P from: products
                // of one thread run in the order of their issue
                for (int x = 0; x < halves; ++x) issue_s(x, g0);
                umma_commit_at(k_empty0 + 8u * (unsigned)(g0 % STAGES));  // the K slot is free once both products have read it
                if (n_tiles == 1) umma_commit_at(q_empty_at);            // and so are the queries after the item's last S
                for (int j = 0; j < n_tiles && ok; ++j) {
                    const int g = g0 + j;
                    const bool more = j + 1 < n_tiles;
                    for (int x = 0; x < halves && ok; ++x) {
                        if (!mbar_wait(&p_full[x], (h0[x] + j) & 1, failed)) { *failed = 1; ok = false; break; }
                        if (x == 0 && !mbar_wait(&v_full[g % STAGES], (g / STAGES) & 1, failed)) { *failed = 1; ok = false; break; }
                        tc_fence_after();
                        issue_pv(x, g, j > 0 ? 1u : 0u);
                        if (x == halves - 1) umma_commit_at(v_empty0 + 8u * (unsigned)(g % STAGES));
                        if (more) {
                            if (x == 0) {
                                if (!mbar_wait(&k_full[(g + 1) % STAGES], ((g + 1) / STAGES) & 1, failed)) { *failed = 1; ok = false; break; }
                                tc_fence_after();
                            }
                            // S_x(g + 1) lands in the columns the product just issued reads P_x(g) from: products of one
                            // thread run in the order of their issue, so the columns are read before they are written
                            issue_s(x, g + 1);
                            if (x == halves - 1) {
                                umma_commit_at(k_empty0 + 8u * (unsigned)((g + 1) % STAGES));
                                if (j + 2 == n_tiles) umma_commit_at(q_empty_at);
                            }
                        }
                    }
                }
                g0 += n_tiles;
                h0[0] += n_tiles;
                if (halves == 2) h0[1] += n_tiles;
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax: thread = row = tensor-memory lane of its half
        const int x = (warp - 2) >> 2;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const int v = x * BM + r;
        const unsigned lane_addr = tmem + ((unsigned)(quarter * 32) << 16);
        const unsigned s_addr = lane_addr + x * BN, o_addr = lane_addr + O_COL + x * BM;
        const float scale = a.scale_log2;
        int hx = 0;  // key tiles this half has seen
        bool ok = true;
        for (int round = 0; ok; ++round) {
            Item it;
            if (!mbar_wait(q_full, round & 1, failed)) { *failed = 1; break; }  // every thread sees every phase of it go by
            __syncwarp();
            if (lane == 0) mbar_arrive(q_seen);
            if (!read_item(round, it)) break;
            if (x < it.halves) {
                const int n_tiles = it.n_tiles;
                const int tok = v / gc, hh = v - tok * gc;
                const bool row_valid = tok < it.ntok && hh < it.heads_here;
                // A row beyond the tile's end (or beyond the heads of the chunk) is computed like the tile's last token and never
                // stored: it takes the same way through the code as its neighbours, so no warp has to walk two ways.
                const int hi = row_valid ? it.pos_first + tok : it.pos_last;
                const int lo = a.window > 0 ? max(0, hi - a.window + 1) : 0;
                float m = -INFINITY, l = 0.f;
                for (int j = 0; j < n_tiles; ++j) {
                    const int h = hx + j;
                    if (!mbar_wait(&s_full[x], h & 1, failed)) { *failed = 1; ok = false; break; }
                    tc_fence_after();
                    float s[BN];
                    tmem_ld64(s_addr, s);
                    tmem_ld64(s_addr + 64, s + 64);
                    const int tile_base = it.start + j * BN;
                    // one way for the whole warp: the masked walk only where some row of the warp needs it
                    const int last_visible = hi - tile_base, first_visible = lo - tile_base;  // among the tile's keys 0 .. BN - 1
                    if (!__all_sync(0xffffffffu, last_visible >= BN - 1 && first_visible <= 0)) {
#pragma unroll
                        for (int i = 0; i < BN; ++i) s[i] = (i <= last_visible && i >= first_visible) ? s[i] : -INFINITY;
                    }
                    float part[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                    for (int i = 0; i < BN; ++i) part[i & 3] = fmaxf(part[i & 3], s[i]);
                    const float tmax = fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3])) * scale;  // the scale is positive: the largest score stays the largest
                    const float m_new = fmaxf(m, tmax);
                    float alpha = 1.f;
                    if (m == -INFINITY) {
                        m = m_new;  // nothing visible so far: the row of O holds zeros (or is overwritten by the first product), no rescale
                    } else if (m_new - m > RESCALE_THRESHOLD) {
                        alpha = exp2f(m - m_new);
                        m = m_new;
                    }
                    const float minus_m = (m == -INFINITY) ? 0.f : -m;
                    float sum[4] = {0.f, 0.f, 0.f, 0.f};
                    unsigned words[BN / 2];
#pragma unroll
                    for (int i = 0; i < BN / 2; ++i) {
                        const float p0 = fast_exp2(fmaf(s[2 * i], scale, minus_m)), p1 = fast_exp2(fmaf(s[2 * i + 1], scale, minus_m));
                        sum[i & 3] += p0 + p1;
                        words[i] = pack_bf16x2(p0, p1);
                    }
                    l = l * alpha + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
                    // P goes into this thread's lane over the columns its S came from (the thread holds its S row in registers;
                    // the tensor core writes those columns again only with the next S, issued after the product that reads P)
#pragma unroll
                    for (int c = 0; c < BN / 2; c += 16) tmem_st16_words(s_addr + c, words + c);
                    // Every thread sees every phase of o_done go by, tile by tile: a wait by parity tells "phase h - 1 is over" only
                    // to a thread that knows phase h - 2 is (a thread two phases behind would read the parity of a later phase as
                    // "not yet" and wait for ever). Here phase h - 2 was waited for one tile ago (or, at an item's second tile, at
                    // the end of the item before) and the product of tile h cannot start before this thread hands P over, so
                    // the barrier is in phase h - 1 or h. The product of tile h - 1 was issued a whole tile ago; the wait is
                    // almost always over at the first look.
                    if (j > 0 && !mbar_wait(&o_done[x], (h - 1) & 1, failed)) { *failed = 1; ok = false; break; }
                    if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                        // O may be rescaled only between two products: the one before is done
                        tc_fence_after();
#pragma unroll
                        for (int c = 0; c < D; c += 16) {
                            float o[16];
                            tmem_ld16(o_addr + c, o);
#pragma unroll
                            for (int i = 0; i < 16; ++i) o[i] *= alpha;
                            tmem_st16(o_addr + c, o);
                        }
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&p_full[x]);
                }
                // every phase but the item's last was seen in the loop
                if (ok) ok = mbar_wait(&o_done[x], (hx + n_tiles - 1) & 1, failed);
                if (!ok) *failed = 1;
                tc_fence_after();
                if (ok) {
                    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
                    for (int c = 0; c < D; c += 16) {
                        float o[16];
                        tmem_ld16(o_addr + c, o);
                        if (row_valid) {
                            uint4 w[2];
                            unsigned* packed = reinterpret_cast<unsigned*>(w);
#pragma unroll
                            for (int i = 0; i < 8; ++i) packed[i] = pack_bf16x2(o[2 * i] * inv, o[2 * i + 1] * inv);
                            uint4* dst = reinterpret_cast<uint4*>(a.out + (size_t)(it.tok0 + tok) * a.out_stride + (size_t)(it.first_head + hh) * D + c);
                            if (a.wide_stores) {  // one 32-byte store per 16 columns: half as many requests to the memory pipe
                                asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(packed[0]), "r"(packed[1]), "r"(packed[2]),
                                             "r"(packed[3]), "r"(packed[4]), "r"(packed[5]), "r"(packed[6]), "r"(packed[7]) : "memory");
                            } else {
                                dst[0] = w[0];
                                dst[1] = w[1];
                            }
                        }
                    }
                    // the rows are out of tensor memory before this thread hands over the next item's first P, and only then is O written anew
                    tc_fence_before();
                }
                hx += n_tiles;
            }
            // The softmax warps end an item together, so that none of them (those of a half that had nothing to do least of
            // all) falls an item behind the others: the slot of an item is written anew three items later.
            __syncwarp();
            if (lane == 0) mbar_arrive(round_done);
            if (ok && !mbar_wait(round_done, round & 1, failed)) { *failed = 1; ok = false; }
        }
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

// More than half of an SM's shared memory, so that one block is all an SM takes: the block holds all of its tensor memory.
constexpr size_t SMEM_USED = 1024 + (size_t)2 * STAGES * TILE_BYTES + (size_t)PANELS * Q_PANEL * sizeof(bf16) + (4 * STAGES + 10) * 8 + 96;
constexpr size_t SMEM_BYTES = SMEM_USED > 120 * 1024 ? SMEM_USED : 120 * 1024;
}  // namespace

// Rows of a tile (tokens x heads of a group) this kernel wants: the host planner cuts rows into tiles of
// 256 / min(group, 256) tokens.
HB_EXPORT int hb_attention_tc_tile_rows() { return ROWS; }

HB_EXPORT int hb_attention_tc_tiles(const void* q, int q_stride, void* out, int out_stride, const void* cache, const int* block_table,
                                    int table_width, const int* token_row, const int* positions, const int* tiles, int n_tiles, int n_tokens,
                                    int heads, int kv_heads, int head_dim, int page_size, int pages, float scale, int window, int* status,
                                    int* work, cudaStream_t stream) {
    (void)token_row;
    if (!work) return HB_BAD_ARGUMENT;
    if (n_tiles <= 0) return 0;
    if (n_tokens <= 0) return HB_BAD_ARGUMENT;
    if (head_dim != D) return HB_UNSUPPORTED_SIZE;
    if (kv_heads <= 0 || heads % kv_heads || q_stride % 8 || out_stride % 8) return HB_BAD_ARGUMENT;
    if (!(scale > 0.f)) return HB_BAD_ARGUMENT;  // the row maximum is taken before the scores are scaled
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
    // the queries as (column, head, token): a tile's box is 64 columns of gc heads of its tokens
    const int group = heads / kv_heads, gc = group < ROWS ? group : ROWS, head_chunks = (group + gc - 1) / gc;
    CUtensorMap q_map;
    const cuuint64_t q_dims[3] = {(cuuint64_t)D, (cuuint64_t)heads, (cuuint64_t)n_tokens};
    const cuuint64_t q_strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)q_stride * 2};
    const cuuint32_t q_box[3] = {64, (cuuint32_t)gc, (cuuint32_t)(ROWS / gc)};
    const cuuint32_t q_elem[3] = {1, 1, 1};
    if (encode(&q_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), q_dims, q_strides, q_box, q_elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return HB_BAD_ARGUMENT;
    AttnArgs a{(const bf16*)q, q_stride, (bf16*)out, out_stride, block_table, table_width, positions,
               heads, kv_heads, page_size, pages, window, scale * 1.4426950408889634f, status,
               (((uintptr_t)out & 31) == 0 && out_stride % 16 == 0) ? 1 : 0};
    if ((long long)kv_heads * head_chunks > 65535) return HB_UNSUPPORTED_SIZE;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    // one persistent block per SM (it holds the SM's tensor memory), or one per item if there are fewer
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
        return HB_BAD_ARGUMENT;
    const long long items = (long long)n_tiles * kv_heads * head_chunks;
    if (items > 0x7fffffffLL) return HB_UNSUPPORTED_SIZE;
    const int blocks = (int)(items < (long long)sms ? items : (long long)sms);
    return launch_after_previous(attention_tc_kernel, dim3(blocks), THREADS, SMEM_BYTES, stream, map, q_map, a, tiles, n_tiles, kv_heads * head_chunks, gc,
                                 head_chunks, work);
}
