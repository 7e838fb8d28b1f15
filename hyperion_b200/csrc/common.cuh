// Shared device helpers of the sm_100a kernels: element conversion, block reductions with a fixed
// order (so a row's result never depends on what else is in the launch), and the launcher's error
// convention: every exported launcher returns the cudaError_t of its launch as an int, 0 = success,
// and negative values for arguments it refuses.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define HB_EXPORT extern "C" __attribute__((visibility("default")))

// Refusals a launcher reports without touching the device.
enum : int {
    HB_BAD_ARGUMENT = -1,
    HB_UNSUPPORTED_SIZE = -2,
};

// Bits a kernel may set in the engine's status word instead of faulting.
enum : int {
    HB_STATUS_BAD_PAGE = 1,      // a block-table entry that had to be valid was negative or too large
    HB_STATUS_BAD_TOKEN = 2,     // a token id outside the vocabulary
    HB_STATUS_BAD_POSITION = 4,  // a position beyond the position table
    HB_STATUS_WAIT_EXPIRED = 8,  // a bounded wait on a barrier ran out; one of the bits below says in which kernel
    HB_STATUS_IN_GEMM_TILES = 0x100,
    HB_STATUS_IN_GEMM_SWAPPED = 0x200,
    HB_STATUS_IN_ATTENTION_TMA_TILES = 0x400,
    HB_STATUS_IN_ATTENTION_TMA_TOKENS = 0x800,
    HB_STATUS_IN_ATTENTION_TCGEN05 = 0x1000,
};

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Sum over a warp by a butterfly of fixed shape: every lane ends with the same value and the order
// of additions depends on nothing but the lane count.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

// Sum over a block (blockDim.x a multiple of 32, at most 1024). `scratch` holds 32 floats. The
// partial sums of the warps are added in warp order by every thread, so the result is the same in
// every thread and for every launch shape.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < warps; ++w) total += scratch[w];
    return total;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float best = scratch[0];
    for (int w = 1; w < warps; ++w) best = fmaxf(best, scratch[w]);
    return best;
}

static inline int launch_status() { return (int)cudaGetLastError(); }

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched through launch_after_previous() may start while the kernel before it in the
// stream is still running. It must call wait_for_previous_kernels() before it reads anything an
// earlier kernel wrote and before it writes global memory at all; what stands before that call
// (barrier set-up, tensor-memory allocation, loads of weights, which no kernel writes) overlaps
// the earlier kernel's tail. let_next_kernel_start() allows the kernel after this one to be
// scheduled as soon as every block of this one has called it; that kernel still waits in its own
// wait_for_previous_kernels() until this one has finished and its writes are visible. Both calls
// do nothing in a kernel that was launched the ordinary way. HYPERION_B200_PDL=0 turns the
// overlap off (every launch is then serialised as usual).
__device__ __forceinline__ void wait_for_previous_kernels() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void let_next_kernel_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool overlap_launches() {
    static const bool enabled = [] {
        const char* value = getenv("HYPERION_B200_PDL");
        return !(value && value[0] == '0');
    }();
    return enabled;
}

template <typename... Params, typename... Args>
static inline int launch_after_previous(void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared_bytes, cudaStream_t stream,
                                        Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = overlap_launches() ? 1 : 0;
    config.attrs = attribute;
    config.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}
