// What the tcgen05 matrix-product kernels of this folder share: the problem description, mbarrier, TMA and tcgen05
// helpers in inline PTX, operand descriptors, and the host-side tensor maps.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int THREADS = 192;
constexpr unsigned WAIT_LIMIT = 1u << 24;

enum Epilogue : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2, EPI_PARTIAL = 3 };

struct GemmParams {
    void* c;              // output
    const float* bias_f;  // bias as float (or null)
    const bf16* bias_h;   // bias as bfloat16 (or null)
    float* partial;       // split-K partials [splits, rows_out, cols_out] float
    int m, n, k;          // problem: A [m, k], W [n, k]; output [m, n] (SwiGLU: [m, n / 2])
    int ldc;              // row stride of the output in elements
    int k_blocks_per_split;
    int* status;
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false when the limit ran out or another role failed.
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

// Shared-memory operand descriptor: K-major tile of 128-byte rows, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long umma_desc(const void* tile) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(tile) & 0x3FFFFu) >> 4);  // start address
    d |= 1ull << 16;                                               // leading offset: unused for swizzled K-major tiles
    d |= (unsigned long long)(1024 >> 4) << 32;                    // stride between 8-row groups
    d |= 1ull << 46;                                               // descriptor version of sm_100
    d |= 2ull << 61;                                               // 128-byte swizzle
    return d;
}

// Instruction descriptor of kind::f16: float accumulator, bfloat16 operands, both K-major, M = 128, N = bn.
__device__ __forceinline__ unsigned umma_idesc(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(bn >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// The lane that issues the products is one thread, and a lone thread runs a few cycles per instruction: whatever it
// executes between two products is time the tensor cores may stand idle (with a loop that recomputed descriptors and ring
// indices per stage the products came 150 cycles apart whatever their size; a 256 x 256 x 16 product takes 128). So the
// loop keeps the operand descriptors as 32-bit low words that it only adds to (the high word is the same for every
// K-major tile with the 128-byte swizzle), steps through the ring with a counter instead of a division, and issues the
// four products of a stage from one statement.
__device__ __forceinline__ unsigned desc_low(const void* tile) { return ((smem_u32(tile) & 0x3FFFFu) >> 4) | (1u << 16); }
constexpr unsigned DESC_HIGH = (unsigned)(1024 >> 4) | (1u << 14) | (2u << 29);  // 8-row groups 1024 bytes apart, sm_100 descriptor, 128-byte swizzle

// One look at a barrier; the bounded wait only if the phase is not over yet.
__device__ __forceinline__ bool mbar_ready(unsigned bar_addr, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar_addr), "r"(parity) : "memory");
    return done != 0;
}
// Four products of one block (cta_group::1) over one 64-deep stage: K advances by 16 elements = 32 bytes = 2 units of the
// descriptor's address field.
__device__ __forceinline__ void umma_stage(unsigned tmem_d, unsigned a_low, unsigned b_low, unsigned idesc, unsigned accumulate_first) {
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
        ::"r"(tmem_d), "r"(a_low), "r"(b_low), "r"(idesc), "r"(accumulate_first), "r"(DESC_HIGH) : "memory");
}
__device__ __forceinline__ void umma_commit_at(unsigned bar_addr) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
}

// 16 consecutive float columns of this thread's accumulator lane.
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

__device__ __forceinline__ float bias_at(const GemmParams& p, int i) {
    return p.bias_f ? p.bias_f[i] : (p.bias_h ? __bfloat162float(p.bias_h[i]) : 0.f);
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

// A [rows, k] bfloat16 matrix with row stride ld, fetched in boxes of box_rows x 64 elements with the 128-byte swizzle;
// rows and columns beyond the matrix read as zero.
int make_map(CUtensorMap* map, const void* base, int rows, int k, int ld, int box_rows) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return HB_BAD_ARGUMENT;
    if (((uintptr_t)base & 15) || (ld % 8) || box_rows > 256) return HB_UNSUPPORTED_SIZE;
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : HB_BAD_ARGUMENT;
}

int sm_count() {
    static int count = 0;
    if (!count) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
            count = 148;
    }
    return count;
}

}  // namespace
