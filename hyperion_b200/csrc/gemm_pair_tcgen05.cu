// Prompt-sized bfloat16 matrix products with two SMs on one tile: C = A * W^T with A [M, K] and W [N, K], both
// K-contiguous, on 256 x BN tiles computed by a pair of blocks (a cluster of two) with tcgen05.mma.cta_group::2.
//
// Why pairs: one block on a 128 x 256 tile reads 48 KB of operands from shared memory per 64-deep step and TMA writes
// as much, 768 cycles at 128 B per cycle against 512 cycles of products, so shared memory bounds it. In a pair each
// block keeps its own 128 rows of A and only half of the W tile (BN / 2 rows); the tensor cores of both SMs read both
// halves, so a block moves 32 KB per step and the products bound the loop.
//
// Roles in each block of 320 threads (the pair's first block, rank 0, leads):
//   warp 0, one lane   producer: fetches this block's 128 x 64 tile of A and its BN / 2 x 64 half of the W tile with TMA
//                      (cp.async.bulk.tensor, 128-byte swizzle; a plain load, nothing is multicast) into a ring of
//                      stages; the bytes of both blocks count on the leader's `full` barrier of the stage;
//   warp 1             owns tensor memory (tcgen05.alloc.cta_group::2, by both blocks); in the leader one lane issues
//                      tcgen05.mma.cta_group::2 (kind::f16, M 256, N BN, K 16) four times per stage and frees the stage
//                      in both blocks with one tcgen05.commit (multicast to the two `empty` barriers);
//   warps 2-9          epilogue: each block drains its own 128 rows of the accumulator (tcgen05.ld) under the next tile's
//                      products (two accumulators alternate in tensor memory) and tells the leader when it has; a warp
//                      reads the 32 lanes of its quarter (warp % 4) and half of the columns.
// Pairs are persistent: pair c walks tiles c, c + pairs, ... (rows fastest). Epilogues: bfloat16 or float with a bias,
// and SwiGLU over a tile whose first half are gate columns and second half the matching up columns.
//
// Every wait on an mbarrier is bounded; when one runs out the block records it in the status word, its roles leave
// their loops, and it still meets its partner at the cluster barrier before tensor memory is freed.
//
// The reference leaves these products to cuBLAS (helios/crates/helios-hal/src/cuda/cublas.rs:158-188) and applies bias
// and SwiGLU in separate kernels (helios/crates/helios-hal/kernels/elementwise.cu:29,134).
#include "gemm_tcgen05.cuh"

namespace {
constexpr int PAIR_THREADS = 320;  // producer warp, tensor-core warp, eight epilogue warps (two per quarter of the accumulator's lanes)
constexpr int PAIR_ROWS = 2 * BM;  // rows of a tile
constexpr int ACC_STRIDE = 256;    // tensor-memory columns between the two accumulators
constexpr int TMEM_COLS = 512;
constexpr int A_BYTES = BM * BK * 2;
constexpr int SMEM_ROOM = 227 * 1024 - 1024 - 512;

__host__ __device__ constexpr int b_bytes(int bn) { return (bn / 2) * BK * 2; }
__host__ __device__ constexpr int stage_bytes(int bn) { return A_BYTES + b_bytes(bn); }
__host__ __device__ constexpr int stages_for(int bn) { return SMEM_ROOM / stage_bytes(bn) > 8 ? 8 : SMEM_ROOM / stage_bytes(bn); }

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address, in the cluster's shared window, of the leader's copy of a barrier of this block.
__device__ __forceinline__ unsigned in_leader(const void* local) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote) : "r"(smem_u32(local)));
    return remote;
}
__device__ __forceinline__ void arrive_in_leader(unsigned remote_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
// This block's tile into its own shared memory; the bytes count on the leader's barrier.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, unsigned leader_bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(leader_bar), "r"(x), "r"(y) : "memory");
}
// Arrives on the barrier at this offset in both blocks of the pair once the products issued so far have finished.
__device__ __forceinline__ void umma_commit_both(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((unsigned short)3) : "memory");
}
// Four products over one 64-deep stage: K advances by 16 elements = 32 bytes = 2 units of the descriptor's address field.
__device__ __forceinline__ void umma_pair_stage(unsigned tmem_d, unsigned a_low, unsigned b_low, unsigned idesc, unsigned accumulate_first) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\t.reg .b32 al, bl;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 q, 0, 0;\n\t"
        "mov.b64 da, {%1, %5};\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, p;\n\t"
        "add.u32 al, %1, 2;\n\t"
        "add.u32 bl, %2, 2;\n\t"
        "mov.b64 da, {al, %5};\n\t"
        "mov.b64 db, {bl, %5};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, q;\n\t"
        "add.u32 al, %1, 4;\n\t"
        "add.u32 bl, %2, 4;\n\t"
        "mov.b64 da, {al, %5};\n\t"
        "mov.b64 db, {bl, %5};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, q;\n\t"
        "add.u32 al, %1, 6;\n\t"
        "add.u32 bl, %2, 6;\n\t"
        "mov.b64 da, {al, %5};\n\t"
        "mov.b64 db, {bl, %5};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, q;\n\t}"
        ::"r"(tmem_d), "r"(a_low), "r"(b_low), "r"(idesc), "r"(accumulate_first), "r"(DESC_HIGH) : "memory");
}
__device__ __forceinline__ void umma_commit_both_at(unsigned bar_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar_addr), "h"((unsigned short)3) : "memory");
}

// Instruction descriptor of kind::f16: float accumulator, bfloat16 operands, both K-major, M = 256 over the pair, N = bn.
__device__ __forceinline__ unsigned pair_idesc(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(bn >> 3) << 17) | ((unsigned)(PAIR_ROWS >> 4) << 24);
}

// 32 consecutive float columns of this thread's accumulator lane.
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// One thread's share of a finished tile: accumulator lane -> output row r, the tile's columns [begin, end) (SwiGLU: the
// tile's first half are gate columns, the second half the matching up columns, the output has half the width, and
// [begin, end) counts output columns). Whole groups of 32 columns inside the matrix, without a bias, take the short way.
template <int EPI>
__device__ __forceinline__ void store_row(const GemmParams& p, unsigned lane_addr, int r, int col0, int tile_n, int bn, int begin, int end) {
    const bool plain = !p.bias_f && !p.bias_h && (p.ldc & 7) == 0;
    const int width = (EPI == EPI_SWIGLU) ? p.n / 2 : p.n;               // of the output
    const int out0 = (EPI == EPI_SWIGLU) ? tile_n * (bn / 2) : col0;      // the tile's first output column
#pragma unroll 1
    for (int c = begin; c < end; c += 32) {
        const int out_col = out0 + c;
        const int count = min(32, min(end - c, width - out_col));  // columns of this group that exist
        float v[32];
        if (count <= 0) break;
        tmem_ld32(lane_addr + c, v);
        if constexpr (EPI == EPI_SWIGLU) {
            float u[32];
            tmem_ld32(lane_addr + bn / 2 + c, u);
#pragma unroll
            for (int j = 0; j < 32; ++j) {  // the projections are rounded before the activation, as separate kernels would store them
                const float g = __bfloat162float(__float2bfloat16_rn(v[j])), uu = __bfloat162float(__float2bfloat16_rn(u[j]));
                v[j] = g / (1.0f + expf(-g)) * uu;
            }
        }
        if (r >= p.m) continue;
        if constexpr (EPI == EPI_F32) {
            float* dst = reinterpret_cast<float*>(p.c) + (size_t)r * p.ldc + out_col;
            for (int j = 0; j < count; ++j) dst[j] = v[j] + bias_at(p, out_col + j);
        } else {
            bf16* dst = reinterpret_cast<bf16*>(p.c) + (size_t)r * p.ldc + out_col;
            if (count == 32 && (plain || EPI == EPI_SWIGLU) && (p.ldc & 7) == 0) {
                uint4 w[4];
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(w);
#pragma unroll
                for (int j = 0; j < 16; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
#pragma unroll
                for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(dst)[j] = w[j];
            } else {
                for (int j = 0; j < count; ++j) dst[j] = __float2bfloat16_rn(EPI == EPI_SWIGLU ? v[j] : v[j] + bias_at(p, out_col + j));
            }
        }
    }
}

template <int EPI>
__global__ void __launch_bounds__(PAIR_THREADS) gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                                                            const GemmParams p, int tiles_m, int tiles_n, int bn, int stages) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int stage_size = stage_bytes(bn);
    unsigned long long* full = reinterpret_cast<unsigned long long*>(tiles + (size_t)stages * stage_size);  // used in the leader only
    unsigned long long* empty = full + stages;
    unsigned long long* acc_full = empty + stages;  // [2]
    unsigned long long* acc_empty = acc_full + 2;   // [2], used in the leader only: 16 warps arrive, 8 of each block
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty + 2);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    let_next_kernel_start();
    const int total = tiles_m * tiles_n;
    const int k_blocks = (p.k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 16); }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // both blocks' barriers exist before either signals the other's
    tc_fence_after();
    const unsigned tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {  // producer
            const int row_in_tile = (int)rank * BM, col_in_tile = (int)rank * (bn / 2);
            // The first ring of weight tiles is fetched before the kernels ahead in the stream have finished (no kernel
            // writes weights); the activations, which they produce, follow after the wait.
            const int t0 = pair;
            const int ahead = t0 < total ? min(k_blocks, stages) : 0;
            for (int i = 0; i < ahead; ++i) {
                if (leader) mbar_expect_tx(&full[i], 2u * (unsigned)stage_size);
                tma_load_2d_pair(tiles + (size_t)i * stage_size + A_BYTES, &map_w, in_leader(&full[i]), i * BK, (t0 / tiles_m) * bn + col_in_tile);
            }
            wait_for_previous_kernels();
            for (int i = 0; i < ahead; ++i)
                tma_load_2d_pair(tiles + (size_t)i * stage_size, &map_x, in_leader(&full[i]), i * BK, (t0 % tiles_m) * PAIR_ROWS + row_in_tile);
            // the ring goes on across tiles: stage s and the parity of its barriers step with a counter
            int s = ahead % stages;
            unsigned turn = (unsigned)(ahead / stages) & 1u;
            const unsigned full0 = in_leader(&full[0]);
            bool ok = true;
            for (int t = t0; t < total && ok; t += pairs) {
                const int row0 = (t % tiles_m) * PAIR_ROWS + row_in_tile, col0 = (t / tiles_m) * bn + col_in_tile;
                for (int kb = (t == t0 ? ahead : 0); kb < k_blocks; ++kb) {
                    if (!mbar_ready(smem_u32(&empty[s]), turn ^ 1u) && !mbar_wait(&empty[s], turn ^ 1u, failed)) { *failed = 1; ok = false; break; }
                    unsigned char* a_tile = tiles + (size_t)s * stage_size;
                    const unsigned bar = full0 + 8u * (unsigned)s;
                    if (leader) mbar_expect_tx(&full[s], 2u * (unsigned)stage_size);
                    tma_load_2d_pair(a_tile, &map_x, bar, kb * BK, row0);
                    tma_load_2d_pair(a_tile + A_BYTES, &map_w, bar, kb * BK, col0);
                    if (++s == stages) { s = 0; turn ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {  // tensor-core issuer of the pair
            const unsigned idesc = pair_idesc(bn);
            const unsigned a_low0 = desc_low(tiles), b_low0 = desc_low(tiles + A_BYTES), step = (unsigned)stage_size >> 4;
            const unsigned full0 = smem_u32(&full[0]), empty0 = smem_u32(&empty[0]);
            int s = 0;
            unsigned turn = 0, a_low = a_low0, b_low = b_low0;
            bool ok = true;
            for (int t = pair, i = 0; t < total && ok; t += pairs, ++i) {
                const int buf = i & 1;
                if (!mbar_wait(&acc_empty[buf], ((i >> 1) & 1) ^ 1, failed)) { *failed = 1; ok = false; break; }  // both epilogues have drained it
                tc_fence_after();
                const unsigned acc = tmem + buf * ACC_STRIDE;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_ready(full0 + 8u * (unsigned)s, turn) && !mbar_wait(&full[s], turn, failed)) { *failed = 1; ok = false; break; }
                    umma_pair_stage(acc, a_low, b_low, idesc, kb > 0 ? 1u : 0u);
                    umma_commit_both_at(empty0 + 8u * (unsigned)s);  // the stage is free in both blocks once these products have read it
                    a_low += step;
                    b_low += step;
                    if (++s == stages) { s = 0; turn ^= 1u; a_low = a_low0; b_low = b_low0; }
                }
                if (ok) umma_commit_both(&acc_full[buf]);
            }
        }
    } else {  // epilogue: warps 2..9; warp w reads lane quarter w % 4 and the half (w - 2) / 4 of this block's columns
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int cols = (EPI == EPI_SWIGLU) ? bn / 2 : bn;              // columns of the tile as the epilogue counts them
        const int split = ((cols / 2 + 31) / 32) * 32;                   // whole groups of 32 to the first half
        const int begin = half ? split : 0, end = half ? cols : split;
        wait_for_previous_kernels();  // before this thread writes anything
        bool ok = true;
        for (int t = pair, i = 0; t < total && ok; t += pairs, ++i) {
            const int buf = i & 1;
            if (!mbar_wait(&acc_full[buf], (i >> 1) & 1, failed)) { *failed = 1; ok = false; break; }
            tc_fence_after();
            const int tile_m = t % tiles_m, tile_n = t / tiles_m;
            store_row<EPI>(p, tmem + buf * ACC_STRIDE + ((unsigned)(quarter * 32) << 16), tile_m * PAIR_ROWS + (int)rank * BM + quarter * 32 + lane,
                           tile_n * bn, tile_n, bn, begin, end);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) arrive_in_leader(in_leader(&acc_empty[buf]));  // this warp's share of the accumulator may be written again
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *failed) atomicOr(p.status, HB_STATUS_WAIT_EXPIRED | HB_STATUS_IN_GEMM_TILES);
    cluster_sync();  // neither block leaves while the other may still read its shared memory or signal its barriers
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// The tile width (a multiple of 16 from 128 to 256) that wastes the least: pairs take ceil(tiles / pairs) rounds of
// tiles of bn columns each, and columns beyond n are computed for nothing.
int choose_pair_width(int m, int n, int pairs) {
    int best = 256;
    long long best_cost = -1;
    for (int bn = 256; bn >= 128; bn -= 16) {
        const long long tiles = (long long)((m + PAIR_ROWS - 1) / PAIR_ROWS) * ((n + bn - 1) / bn);
        const long long cost = ((tiles + pairs - 1) / pairs) * bn;
        if (best_cost < 0 || cost < best_cost) { best = bn; best_cost = cost; }
    }
    return best;
}

template <int EPI>
int launch_pairs(const CUtensorMap& map_x, const CUtensorMap& map_w, const GemmParams& p, int tiles_m, int tiles_n, int bn, int pairs,
                 cudaStream_t stream) {
    const int stages = stages_for(bn);
    const size_t smem = 1024 + (size_t)stages * stage_bytes(bn) + 512;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * pairs);
    config.blockDim = dim3(PAIR_THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 2;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = overlap_launches() ? 1 : 0;
    config.attrs = attributes;
    config.numAttrs = 2;
    return (int)cudaLaunchKernelEx(&config, gemm_pair_kernel<EPI>, map_x, map_w, p, tiles_m, tiles_n, bn, stages);
}

// How many pairs of blocks the device runs at a time (a pair needs two SMs of one processing cluster).
template <int EPI>
int resident_pairs() {
    static int pairs = 0;
    if (!pairs) {
        cudaFuncSetAttribute(gemm_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(2 * sm_count());
        config.blockDim = dim3(PAIR_THREADS);
        config.dynamicSmemBytes = 1024 + (size_t)stages_for(256) * stage_bytes(256) + 512;
        cudaLaunchAttribute attribute[1];
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = 2;
        attribute[0].val.clusterDim.y = 1;
        attribute[0].val.clusterDim.z = 1;
        config.attrs = attribute;
        config.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, gemm_pair_kernel<EPI>, &config) != cudaSuccess || clusters <= 0) clusters = sm_count() / 2;
        pairs = clusters;
    }
    return pairs;
}
}  // namespace

// C = A W^T (+ bias) on pairs of SMs.  a [m, k] (row stride lda), w [n, k] (row stride ldw), bfloat16, k-contiguous.
//   epilogue 0: c bfloat16 [m, n]; 1: c float [m, n]; 2: SwiGLU, c bfloat16 [m, n / 2] where every 256 rows of w
//   are 128 gate rows followed by their 128 up rows (n a multiple of 256).
HB_EXPORT int hb_gemm_pair_bf16(const void* a, int lda, const void* w, int ldw, void* c, int ldc, const float* bias_f, const void* bias_h,
                                int m, int n, int k, int epilogue, int* status, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0) return HB_BAD_ARGUMENT;
    if (epilogue == EPI_SWIGLU && n % 256) return HB_UNSUPPORTED_SIZE;
    if (epilogue != EPI_BF16 && epilogue != EPI_F32 && epilogue != EPI_SWIGLU) return HB_BAD_ARGUMENT;
    GemmParams p{c, bias_f, (const bf16*)bias_h, nullptr, m, n, k, ldc, (k + BK - 1) / BK, status};
    const int resident = epilogue == EPI_BF16 ? resident_pairs<EPI_BF16>() : (epilogue == EPI_F32 ? resident_pairs<EPI_F32>() : resident_pairs<EPI_SWIGLU>());
    const int bn = epilogue == EPI_SWIGLU ? 256 : choose_pair_width(m, n, resident);
    CUtensorMap map_x, map_w;
    if (int code = make_map(&map_x, a, m, k, lda, BM)) return code;
    if (int code = make_map(&map_w, w, n, k, ldw, bn / 2)) return code;
    const int tiles_m = (m + PAIR_ROWS - 1) / PAIR_ROWS, tiles_n = (n + bn - 1) / bn;
    if ((long long)tiles_m * tiles_n > 0x7fffffffLL) return HB_UNSUPPORTED_SIZE;
    const int pairs = min(tiles_m * tiles_n, resident);
    if (epilogue == EPI_BF16) return launch_pairs<EPI_BF16>(map_x, map_w, p, tiles_m, tiles_n, bn, pairs, stream);
    if (epilogue == EPI_F32) return launch_pairs<EPI_F32>(map_x, map_w, p, tiles_m, tiles_n, bn, pairs, stream);
    return launch_pairs<EPI_SWIGLU>(map_x, map_w, p, tiles_m, tiles_n, bn, pairs, stream);
}
