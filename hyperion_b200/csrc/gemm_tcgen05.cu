// bfloat16 matrix products on the 5th-generation tensor cores: C = A * W^T with A [M, K] and W [N, K],
// both K-contiguous, accumulated in float in tensor memory.
//
// Two kernels share the roles of their warps.  Warp 0 (one lane) is the producer: it fetches 128 x 64 and BN x 64
// operand tiles with TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast) into a ring of shared-memory
// stages.  Warp 1 owns tensor memory (tcgen05.alloc / dealloc) and one of its lanes issues tcgen05.mma
// (kind::f16, M = 128, N = BN, K = 16) four times per stage, releasing the stage with tcgen05.commit.  Warps 2-5
// are the epilogue: each reads its quarter of the accumulator's 128 lanes with tcgen05.ld and writes the result.
//
// * The tile shape (prompt-sized M): one persistent block per SM walks 128 x BN tiles; the ring runs on across
//   tiles and two accumulators alternate in tensor memory, so a tile's epilogue runs under the next tile's products.
//   Epilogues: bfloat16 (+ bias), float (+ bias), SwiGLU over a tile whose first half are gate columns and second
//   half the matching up columns.
// * The swapped shape (decode, M = 1..64): the weight matrix supplies the 128 rows and the batch the BN columns, the
//   tile is stored transposed, and K may be split over several blocks (float partials, summed by a second kernel or
//   by their reader) so that the weights stream from HBM once at full width.
//
// Every wait on an mbarrier is bounded: when a wait runs out, the kernel records it in the status
// word, all roles leave their loops, tensor memory is freed and the block returns.
//
// The reference leaves these products to cuBLAS (helios/crates/helios-hal/src/cuda/cublas.rs:158-188,
// cuda/cublaslt.rs:203-212) and applies bias and SwiGLU in separate kernels
// (helios/crates/helios-hal/kernels/elementwise.cu:29,134).
#include "gemm_tcgen05.cuh"

namespace {
template <int BN>
struct Layout {
    static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    // The ring's depth is chosen at launch: DEEP stages when one block per SM streams alone, SHALLOW ones (about half of
    // the shared memory) when the grid has more blocks than SMs, so that two blocks share an SM and one block's start and
    // epilogue pass under the other's stream (measured: gate+up at 8 rows 47.8 -> 44.8 us, at 64 rows 52.8 -> 47.1 us).
    static constexpr int DEEP = 8;
    static constexpr int SHALLOW = (110 * 1024) / STAGE_BYTES;
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    static constexpr size_t smem(int stages) { return 1024 + (size_t)stages * STAGE_BYTES + 256; }
};

// ---------------------------------------------------------------- the swapped shape (at most 64 rows of activations)
// map_a: the weights, which supply the tile's 128 rows (TMEM lanes); map_b: the activations, which supply its BN columns.
// One block per tile and split of K.
template <int BN, int EPI>
__global__ void __launch_bounds__(THREADS) gemm_swapped_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                                               const GemmParams p, const int stages) {
    using L = Layout<BN>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned long long* full = reinterpret_cast<unsigned long long*>(tiles + (size_t)stages * L::STAGE_BYTES);
    unsigned long long* empty = full + stages;
    unsigned long long* acc_full = empty + stages;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_full + 1);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    let_next_kernel_start();
    // blockIdx.x runs fastest over the tiles of map_a's rows, so blocks that are resident together share map_b's tile in L2
    const int row0 = blockIdx.x * BM;  // first row of map_a's operand
    const int col0 = blockIdx.y * BN;  // first row of map_b's operand
    const int k_blocks_total = (p.k + BK - 1) / BK;
    const int kb_begin = blockIdx.z * p.k_blocks_per_split;
    const int kb_end = min(k_blocks_total, kb_begin + p.k_blocks_per_split);
    const int n_kb = max(0, kb_end - kb_begin);

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(L::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {  // producer
            // The first ring of weight tiles is fetched before the kernels ahead in the stream have finished
            // (no kernel writes weights); the activations, which they produce, follow after the wait.
            const int ahead = min(n_kb, stages);
            for (int i = 0; i < ahead; ++i) {
                unsigned char* a_tile = tiles + (size_t)i * L::STAGE_BYTES;
                mbar_expect_tx(&full[i], L::STAGE_BYTES);
                tma_load_2d(a_tile, &map_a, &full[i], (kb_begin + i) * BK, row0);
            }
            wait_for_previous_kernels();
            for (int i = 0; i < ahead; ++i) {
                unsigned char* a_tile = tiles + (size_t)i * L::STAGE_BYTES;
                tma_load_2d(a_tile + L::A_BYTES, &map_b, &full[i], (kb_begin + i) * BK, col0);
            }
            int s = ahead % stages;
            unsigned turn = (unsigned)(ahead / stages) & 1u;
            for (int i = ahead; i < n_kb; ++i) {
                if (!mbar_ready(smem_u32(&empty[s]), turn ^ 1u) && !mbar_wait(&empty[s], turn ^ 1u, failed)) { *failed = 1; break; }
                unsigned char* a_tile = tiles + (size_t)s * L::STAGE_BYTES;
                mbar_expect_tx(&full[s], L::STAGE_BYTES);
                tma_load_2d(a_tile, &map_a, &full[s], (kb_begin + i) * BK, row0);
                tma_load_2d(a_tile + L::A_BYTES, &map_b, &full[s], (kb_begin + i) * BK, col0);
                if (++s == stages) { s = 0; turn ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {  // tensor-core issuer: descriptors as low words that are only added to, the ring by a counter
            const unsigned idesc = umma_idesc(BN);
            const unsigned a_low0 = desc_low(tiles), b_low0 = desc_low(tiles + L::A_BYTES), step = (unsigned)L::STAGE_BYTES >> 4;
            const unsigned full0 = smem_u32(&full[0]), empty0 = smem_u32(&empty[0]);
            int s = 0;
            unsigned turn = 0, a_low = a_low0, b_low = b_low0;
            bool ok = true;
            for (int i = 0; i < n_kb; ++i) {
                if (!mbar_ready(full0 + 8u * (unsigned)s, turn) && !mbar_wait(&full[s], turn, failed)) { *failed = 1; ok = false; break; }
                umma_stage(tmem, a_low, b_low, idesc, i > 0 ? 1u : 0u);
                umma_commit_at(empty0 + 8u * (unsigned)s);  // the stage is free once these products have read it
                a_low += step;
                b_low += step;
                if (++s == stages) { s = 0; turn ^= 1u; a_low = a_low0; b_low = b_low0; }
            }
            if (ok) umma_commit(acc_full);
        }
    } else {  // epilogue: warps 2..5 read TMEM lane quarters 2, 3, 0, 1
        const int quarter = warp & 3;
        const int r = row0 + quarter * 32 + lane;  // row of map_a's operand this thread holds
        wait_for_previous_kernels();  // before this thread writes anything
        bool ok = n_kb > 0 ? mbar_wait(acc_full, 0, failed) : true;
        if (!ok) *failed = 1;
        tc_fence_after();
        if (ok) {
            const unsigned lane_addr = tmem + ((unsigned)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                float v[16];
                if (n_kb > 0) {
                    tmem_ld16(lane_addr + c, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0.f;
                }
                // lanes are output columns (weight rows r), TMEM columns are output rows (batch): store transposed
                if (r < p.n) {
                    const float b = (EPI == EPI_PARTIAL) ? 0.f : bias_at(p, r);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int mrow = col0 + c + j;
                        if (mrow >= p.m) break;
                        if constexpr (EPI == EPI_BF16) reinterpret_cast<bf16*>(p.c)[(size_t)mrow * p.ldc + r] = __float2bfloat16_rn(v[j] + b);
                        else if constexpr (EPI == EPI_F32) reinterpret_cast<float*>(p.c)[(size_t)mrow * p.ldc + r] = v[j] + b;
                        else p.partial[((size_t)blockIdx.z * p.m + mrow) * p.n + r] = v[j];
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *failed) atomicOr(p.status, HB_STATUS_WAIT_EXPIRED | HB_STATUS_IN_GEMM_SWAPPED);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(L::TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------- the tile shape, one persistent block per SM
// Every block walks tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... of the 128 x BN grid over the output (rows
// fastest, so blocks that run side by side share a weight tile in L2). The operand ring runs on across tiles, and the
// accumulator alternates between two regions of tensor memory: while the epilogue warps drain one tile, the tensor core
// already works on the next. BN is chosen per problem so that the last round of tiles leaves few SMs idle.
template <int BN>
struct TileLayout {
    static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int ROOM = 227 * 1024 - 1024 - 256;
    static constexpr int STAGES = ROOM / STAGE_BYTES > 6 ? 6 : ROOM / STAGE_BYTES;
    static constexpr int ACC_STRIDE = 256;  // columns between the two accumulators
    static constexpr int TMEM_COLS = 512;
    static constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + 256;
};

// One thread's row of a finished tile: accumulator lane -> output row r, columns col0 .. col0 + BN - 1 (SwiGLU: the tile's
// first half are gate columns, the second half the matching up columns, and the output has half the width).
template <int BN, int EPI>
__device__ __forceinline__ void store_tile_row(const GemmParams& p, unsigned lane_addr, int r, int col0, int tile_n) {
    constexpr int COLS = (EPI == EPI_SWIGLU) ? BN / 2 : BN;
#pragma unroll 1
    for (int c = 0; c < COLS; c += 16) {
        float v[16];
        tmem_ld16(lane_addr + c, v);
        if constexpr (EPI == EPI_SWIGLU) {
            float u[16];
            tmem_ld16(lane_addr + BN / 2 + c, u);
            const int out_col = tile_n * (BN / 2) + c;
            if (r < p.m && out_col < p.n / 2) {
                bf16* dst = reinterpret_cast<bf16*>(p.c) + (size_t)r * p.ldc + out_col;
#pragma unroll
                for (int j = 0; j < 16; ++j) {  // the projections are rounded before the activation, as separate kernels would store them
                    const float g = __bfloat162float(__float2bfloat16_rn(v[j])), uu = __bfloat162float(__float2bfloat16_rn(u[j]));
                    v[j] = g / (1.0f + expf(-g)) * uu;
                }
                if (out_col + 16 <= p.n / 2 && (p.ldc & 7) == 0) {
                    uint4 w[2];
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(w);
#pragma unroll
                    for (int j = 0; j < 8; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                    reinterpret_cast<uint4*>(dst)[0] = w[0];
                    reinterpret_cast<uint4*>(dst)[1] = w[1];
                } else {
                    for (int j = 0; j < 16; ++j)
                        if (out_col + j < p.n / 2) dst[j] = __float2bfloat16_rn(v[j]);
                }
            }
        } else {
            const int col = col0 + c;
            if (r < p.m && col < p.n) {
                if constexpr (EPI == EPI_BF16) {
                    bf16* dst = reinterpret_cast<bf16*>(p.c) + (size_t)r * p.ldc + col;
                    if (col + 16 <= p.n && (p.ldc & 7) == 0) {
                        uint4 w[2];
                        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(w);
#pragma unroll
                        for (int j = 0; j < 8; ++j) h[j] = __floats2bfloat162_rn(v[2 * j] + bias_at(p, col + 2 * j), v[2 * j + 1] + bias_at(p, col + 2 * j + 1));
                        reinterpret_cast<uint4*>(dst)[0] = w[0];
                        reinterpret_cast<uint4*>(dst)[1] = w[1];
                    } else {
                        for (int j = 0; j < 16 && col + j < p.n; ++j) dst[j] = __float2bfloat16_rn(v[j] + bias_at(p, col + j));
                    }
                } else {
                    float* dst = reinterpret_cast<float*>(p.c) + (size_t)r * p.ldc + col;
                    for (int j = 0; j < 16 && col + j < p.n; ++j) dst[j] = v[j] + bias_at(p, col + j);
                }
            }
        }
    }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(THREADS) gemm_tiles_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                                                             const GemmParams p, int tiles_m, int tiles_n) {
    using L = TileLayout<BN>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned long long* full = reinterpret_cast<unsigned long long*>(tiles + (size_t)L::STAGES * L::STAGE_BYTES);
    unsigned long long* empty = full + L::STAGES;
    unsigned long long* acc_full = empty + L::STAGES;  // [2]
    unsigned long long* acc_empty = acc_full + 2;      // [2]
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty + 2);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    let_next_kernel_start();
    const int total = tiles_m * tiles_n;
    const int k_blocks = (p.k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < L::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(L::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {  // producer
            // The first ring of weight tiles is fetched before the kernels ahead in the stream have finished (no kernel
            // writes weights); the activations, which they produce, follow after the wait.
            const int t0 = blockIdx.x;
            const int ahead = min(k_blocks, L::STAGES);
            for (int i = 0; i < ahead; ++i) {
                mbar_expect_tx(&full[i], L::STAGE_BYTES);
                tma_load_2d(tiles + (size_t)i * L::STAGE_BYTES + L::A_BYTES, &map_w, &full[i], i * BK, (t0 / tiles_m) * BN);
            }
            wait_for_previous_kernels();
            for (int i = 0; i < ahead; ++i) tma_load_2d(tiles + (size_t)i * L::STAGE_BYTES, &map_x, &full[i], i * BK, (t0 % tiles_m) * BM);
            int s = ahead % L::STAGES;
            unsigned turn = (unsigned)(ahead / L::STAGES) & 1u;
            bool ok = true;
            for (int t = t0; t < total && ok; t += gridDim.x) {
                const int row0 = (t % tiles_m) * BM, col0 = (t / tiles_m) * BN;
                for (int kb = (t == t0 ? ahead : 0); kb < k_blocks; ++kb) {
                    if (!mbar_ready(smem_u32(&empty[s]), turn ^ 1u) && !mbar_wait(&empty[s], turn ^ 1u, failed)) { *failed = 1; ok = false; break; }
                    unsigned char* a_tile = tiles + (size_t)s * L::STAGE_BYTES;
                    mbar_expect_tx(&full[s], L::STAGE_BYTES);
                    tma_load_2d(a_tile, &map_x, &full[s], kb * BK, row0);
                    tma_load_2d(a_tile + L::A_BYTES, &map_w, &full[s], kb * BK, col0);
                    if (++s == L::STAGES) { s = 0; turn ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {  // tensor-core issuer: descriptors as low words that are only added to, the ring by a counter
            const unsigned idesc = umma_idesc(BN);
            const unsigned a_low0 = desc_low(tiles), b_low0 = desc_low(tiles + L::A_BYTES), step = (unsigned)L::STAGE_BYTES >> 4;
            const unsigned full0 = smem_u32(&full[0]), empty0 = smem_u32(&empty[0]);
            int s = 0;
            unsigned turn = 0, a_low = a_low0, b_low = b_low0;
            bool ok = true;
            for (int t = blockIdx.x, i = 0; t < total && ok; t += gridDim.x, ++i) {
                const int buf = i & 1;
                if (!mbar_wait(&acc_empty[buf], ((i >> 1) & 1) ^ 1, failed)) { *failed = 1; ok = false; break; }  // the epilogue has drained it
                tc_fence_after();
                const unsigned acc = tmem + buf * L::ACC_STRIDE;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_ready(full0 + 8u * (unsigned)s, turn) && !mbar_wait(&full[s], turn, failed)) { *failed = 1; ok = false; break; }
                    umma_stage(acc, a_low, b_low, idesc, kb > 0 ? 1u : 0u);
                    umma_commit_at(empty0 + 8u * (unsigned)s);  // the stage is free once these products have read it
                    a_low += step;
                    b_low += step;
                    if (++s == L::STAGES) { s = 0; turn ^= 1u; a_low = a_low0; b_low = b_low0; }
                }
                if (ok) umma_commit(&acc_full[buf]);
            }
        }
    } else {  // epilogue: warps 2..5 read TMEM lane quarters 2, 3, 0, 1
        const int quarter = warp & 3;
        wait_for_previous_kernels();  // before this thread writes anything
        bool ok = true;
        for (int t = blockIdx.x, i = 0; t < total && ok; t += gridDim.x, ++i) {
            const int buf = i & 1;
            if (!mbar_wait(&acc_full[buf], (i >> 1) & 1, failed)) { *failed = 1; ok = false; break; }
            tc_fence_after();
            const int tile_m = t % tiles_m, tile_n = t / tiles_m;
            store_tile_row<BN, EPI>(p, tmem + buf * L::ACC_STRIDE + ((unsigned)(quarter * 32) << 16), tile_m * BM + quarter * 32 + lane, tile_n * BN, tile_n);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {  // this warp's quarter of the accumulator may be written again
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *failed) atomicOr(p.status, HB_STATUS_WAIT_EXPIRED | HB_STATUS_IN_GEMM_TILES);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(L::TMEM_COLS) : "memory");
    }
}

// Sum the split-K partials in split order, add the bias, store as bfloat16 or float.
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, int m, int n, void* c, int ldc, int out_is_f32,
                                     const float* bias_f, const bf16* bias_h) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    let_next_kernel_start();
    wait_for_previous_kernels();
    if (i >= (size_t)m * n) return;
    const int row = (int)(i / n), col = (int)(i - (size_t)row * n);
    float sum = 0.f;
    for (int s = 0; s < splits; ++s) sum += partial[(size_t)s * m * n + i];
    sum += bias_f ? bias_f[col] : (bias_h ? __bfloat162float(bias_h[col]) : 0.f);
    if (out_is_f32) reinterpret_cast<float*>(c)[(size_t)row * ldc + col] = sum;
    else reinterpret_cast<bf16*>(c)[(size_t)row * ldc + col] = __float2bfloat16_rn(sum);
}

// The same, four columns per thread (n and ldc multiples of 4, aligned bases), and every piece asked for before the first
// is added: a thread that adds piece after piece waits for memory once per piece, and the kernels of a decode step are
// nothing but such waits. The order of the additions stays the order of the splits.
constexpr int REDUCE_AHEAD = 16;
__global__ void splitk_reduce4_kernel(const float* __restrict__ partial, int splits, int m, int n, void* c, int ldc, int out_is_f32,
                                      const float* bias_f, const bf16* bias_h) {
    const size_t quad = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    let_next_kernel_start();
    const size_t i = quad * 4, total = (size_t)m * n;
    const int row = (int)(i / n), col = (int)(i - (size_t)row * n);
    float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < total) {  // the bias is nobody's output: fetched while the kernel before still runs
        if (bias_f) b = *reinterpret_cast<const float4*>(bias_f + col);
        else if (bias_h) b = make_float4(__bfloat162float(bias_h[col]), __bfloat162float(bias_h[col + 1]), __bfloat162float(bias_h[col + 2]),
                                         __bfloat162float(bias_h[col + 3]));
    }
    wait_for_previous_kernels();
    if (i >= total) return;
    float4 p[REDUCE_AHEAD];
#pragma unroll
    for (int s = 0; s < REDUCE_AHEAD; ++s)
        if (s < splits) p[s] = *reinterpret_cast<const float4*>(partial + (size_t)s * total + i);
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < REDUCE_AHEAD; ++s)
        if (s < splits) { sum.x += p[s].x; sum.y += p[s].y; sum.z += p[s].z; sum.w += p[s].w; }
    for (int s = REDUCE_AHEAD; s < splits; ++s) {
        const float4 q = *reinterpret_cast<const float4*>(partial + (size_t)s * total + i);
        sum.x += q.x; sum.y += q.y; sum.z += q.z; sum.w += q.w;
    }
    sum.x += b.x; sum.y += b.y; sum.z += b.z; sum.w += b.w;
    if (out_is_f32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(c) + (size_t)row * ldc + col) = sum;
    } else {
        uint2 packed;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&packed);
        h2[0] = __floats2bfloat162_rn(sum.x, sum.y);
        h2[1] = __floats2bfloat162_rn(sum.z, sum.w);
        *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(c) + (size_t)row * ldc + col) = packed;
    }
}

static int launch_splitk_reduce(const float* workspace, int splits, int m, int n, void* c, int ldc, int out_is_f32, const float* bias_f,
                                const bf16* bias_h, cudaStream_t stream) {
    const size_t total = (size_t)m * n;
    const size_t out_bytes = out_is_f32 ? 4 : 2;
    const bool by_four = n % 4 == 0 && ldc % 4 == 0 && ((uintptr_t)workspace & 15) == 0 && ((uintptr_t)c & (4 * out_bytes - 1)) == 0 &&
                         (!bias_f || ((uintptr_t)bias_f & 15) == 0);
    if (by_four)
        return launch_after_previous(splitk_reduce4_kernel, (unsigned)((total / 4 + 127) / 128), 128, 0, stream, workspace, splits, m, n, c, ldc,
                                     out_is_f32, bias_f, bias_h);
    return launch_after_previous(splitk_reduce_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, workspace, splits, m, n, c, ldc, out_is_f32,
                                 bias_f, bias_h);
}

template <int BN, int EPI>
int launch(const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmParams& p, dim3 grid, cudaStream_t stream) {
    using L = Layout<BN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_swapped_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::smem(L::DEEP));
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    // more blocks than one and a half per SM: two of them share an SM, each with the shallow ring
    const long long blocks = (long long)grid.x * grid.y * grid.z;
    const int stages = 2 * blocks >= 3LL * sm_count() ? L::SHALLOW : L::DEEP;
    return launch_after_previous(gemm_swapped_kernel<BN, EPI>, grid, THREADS, L::smem(stages), stream, map_a, map_b, p, stages);
}

template <int BN, int EPI>
int launch_tiles(const CUtensorMap& map_x, const CUtensorMap& map_w, const GemmParams& p, int tiles_m, int tiles_n, int blocks, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tiles_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TileLayout<BN>::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return launch_after_previous(gemm_tiles_kernel<BN, EPI>, dim3(blocks), THREADS, TileLayout<BN>::SMEM, stream, map_x, map_w, p, tiles_m, tiles_n);
}

template <int BN>
int launch_tiles_for(int epilogue, const CUtensorMap& map_x, const CUtensorMap& map_w, const GemmParams& p, int tiles_m, int tiles_n, int blocks,
                     cudaStream_t stream) {
    if (epilogue == EPI_BF16) return launch_tiles<BN, EPI_BF16>(map_x, map_w, p, tiles_m, tiles_n, blocks, stream);
    if (epilogue == EPI_F32) return launch_tiles<BN, EPI_F32>(map_x, map_w, p, tiles_m, tiles_n, blocks, stream);
    return HB_BAD_ARGUMENT;
}

// The tile width that leaves the fewest SMs idle: blocks take ceil(tiles / SMs) rounds of tiles of BN columns each.
int choose_tile_width(int m, int n, int sms) {
    const int widths[5] = {256, 224, 192, 160, 128};
    int best = 256;
    long long best_cost = -1;
    for (int bn : widths) {
        const long long tiles = (long long)((m + BM - 1) / BM) * ((n + bn - 1) / bn);
        const long long cost = ((tiles + sms - 1) / sms) * bn;
        if (best_cost < 0 || cost < best_cost) { best = bn; best_cost = cost; }
    }
    return best;
}

template <int BN>
int launch_swap(int epi, const CUtensorMap& map_w, const CUtensorMap& map_x, const GemmParams& p, dim3 grid, cudaStream_t stream) {
    if (epi == EPI_BF16) return launch<BN, EPI_BF16>(map_w, map_x, p, grid, stream);
    if (epi == EPI_F32) return launch<BN, EPI_F32>(map_w, map_x, p, grid, stream);
    return launch<BN, EPI_PARTIAL>(map_w, map_x, p, grid, stream);
}
}  // namespace

// Workspace floats hb_gemm_bf16 needs for `splits` > 1.
HB_EXPORT long long hb_gemm_bf16_workspace(int m, int n, int splits) { return splits > 1 ? (long long)splits * m * n : 0; }

// C = A W^T (+ bias).  a [m, k] (row stride lda), w [n, k] (row stride ldw), bfloat16, k-contiguous.
//   epilogue 0: c bfloat16 [m, n]; 1: c float [m, n]; 2: SwiGLU, c bfloat16 [m, n / 2] where every 256 rows of w
//   are 128 gate rows followed by their 128 up rows (n a multiple of 256).
//   batch_tile 0: the activations supply the 128-row side (m large).  batch_tile 16 / 32 / 64: the weights supply it
//   and up to batch_tile rows of a form the other side (m <= batch_tile); then `splits` may divide k, with a float
//   workspace of hb_gemm_bf16_workspace(m, n, splits) elements; with leave_partials the sums stay there, [splits, m, n].
HB_EXPORT int hb_gemm_bf16(const void* a, int lda, const void* w, int ldw, void* c, int ldc, const float* bias_f, const void* bias_h,
                           int m, int n, int k, int epilogue, int batch_tile, int splits, float* workspace, int leave_partials,
                           int* status, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0 || splits < 1) return HB_BAD_ARGUMENT;
    GemmParams p{c, bias_f, (const bf16*)bias_h, workspace, m, n, k, ldc, 0, status};
    const int k_blocks = (k + BK - 1) / BK;
    CUtensorMap map_x, map_w;
    if (batch_tile == 0) {
        if (splits != 1) return HB_BAD_ARGUMENT;
        if (epilogue == EPI_SWIGLU && n % 256) return HB_UNSUPPORTED_SIZE;
        p.k_blocks_per_split = k_blocks;
        const int sms = sm_count();
        const int bn = epilogue == EPI_SWIGLU ? 256 : choose_tile_width(m, n, sms);
        if (int code = make_map(&map_x, a, m, k, lda, BM)) return code;
        if (int code = make_map(&map_w, w, n, k, ldw, bn)) return code;
        const int tiles_m = (m + BM - 1) / BM, tiles_n = (n + bn - 1) / bn;
        if ((long long)tiles_m * tiles_n > 0x7fffffffLL) return HB_UNSUPPORTED_SIZE;
        const int blocks = min(tiles_m * tiles_n, sms);
        if (epilogue == EPI_SWIGLU) return launch_tiles<256, EPI_SWIGLU>(map_x, map_w, p, tiles_m, tiles_n, blocks, stream);
        switch (bn) {
            case 256: return launch_tiles_for<256>(epilogue, map_x, map_w, p, tiles_m, tiles_n, blocks, stream);
            case 224: return launch_tiles_for<224>(epilogue, map_x, map_w, p, tiles_m, tiles_n, blocks, stream);
            case 192: return launch_tiles_for<192>(epilogue, map_x, map_w, p, tiles_m, tiles_n, blocks, stream);
            case 160: return launch_tiles_for<160>(epilogue, map_x, map_w, p, tiles_m, tiles_n, blocks, stream);
            default: return launch_tiles_for<128>(epilogue, map_x, map_w, p, tiles_m, tiles_n, blocks, stream);
        }
    }
    if ((batch_tile != 16 && batch_tile != 32 && batch_tile != 64) || m > batch_tile || epilogue == EPI_SWIGLU) return HB_BAD_ARGUMENT;
    if (splits > k_blocks) splits = k_blocks;
    if (splits > 1 && !workspace) return HB_BAD_ARGUMENT;
    p.k_blocks_per_split = (k_blocks + splits - 1) / splits;
    if (int code = make_map(&map_w, w, n, k, ldw, BM)) return code;
    if (int code = make_map(&map_x, a, m, k, lda, batch_tile)) return code;
    dim3 grid((n + BM - 1) / BM, 1, splits);
    const int epi = splits > 1 ? (int)EPI_PARTIAL : epilogue;
    int code = batch_tile == 16 ? launch_swap<16>(epi, map_w, map_x, p, grid, stream)
             : batch_tile == 32 ? launch_swap<32>(epi, map_w, map_x, p, grid, stream)
                                : launch_swap<64>(epi, map_w, map_x, p, grid, stream);
    if (code || splits == 1 || leave_partials) return code;  // the caller adds the partial sums up itself (hb_splitk_reduce, or a kernel that reads them)
    return launch_splitk_reduce((const float*)workspace, splits, m, n, c, ldc, (int)(epilogue == EPI_F32), bias_f, (const bf16*)bias_h, stream);
}

// Adds up split-K partials [splits, m, n] in split order, adds the bias and stores bfloat16 or float: the second half of
// hb_gemm_bf16 with splits > 1, for callers that asked it to leave the partials.
HB_EXPORT int hb_splitk_reduce(const float* workspace, int splits, int m, int n, void* c, int ldc, int out_is_f32, const float* bias_f,
                               const void* bias_h, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (splits < 1 || !workspace) return HB_BAD_ARGUMENT;
    return launch_splitk_reduce(workspace, splits, m, n, c, ldc, out_is_f32, bias_f, (const bf16*)bias_h, stream);
}
