// The non-allocating variant of the split-key decode attention: see attention_tokens_static.h.
// The kernels are those of attention_bf16.cu, compiled into this library a second time; only the
// workspace differs: a file-scope device array instead of memory the caller allocates.
#ifndef HB_HEAD_DIM
#define HB_HEAD_DIM 128
#endif
#include "attention_bf16.cu"
#include "attention_tokens_static.h"

// In host code this name is only a stand-in for the symbol; its device address comes from
// cudaGetSymbolAddress below and is what the kernels receive.
static __device__ __align__(256) float hb_static_scratch[HB_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* scratch_address[MAX_DEVICES] = {};
}  // namespace

HB_EXPORT long long hb_attention_tokens_static_capacity(void) { return HB_STATIC_SCRATCH_FLOATS; }

HB_EXPORT int hb_attention_tokens_static(const void* q, int q_stride, void* out, int out_stride, const void* cache,
                                         const int* block_table, int table_width, const int* token_row, const int* positions,
                                         const int* items, int n_items, int splits, int heads, int kv_heads, int head_dim,
                                         int page_size, int pages, float scale, int window, int* status, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (splits < 1 || heads <= 0) return HB_BAD_ARGUMENT;
    const long long need = hb_attention_tokens_workspace(n_items, heads, splits);
    if (need > (long long)HB_STATIC_SCRATCH_FLOATS) return HB_SCRATCH_TOO_SMALL;
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) return HB_SETUP_FAILED;
    if (scratch_address[device] == nullptr) {
        // once per device, with that device current
        float* address = nullptr;
        if (cudaGetSymbolAddress((void**)&address, hb_static_scratch) != cudaSuccess || address == nullptr) {
            (void)cudaGetLastError();
            return HB_SETUP_FAILED;
        }
        if (cudaFuncSetAttribute(attention_tokens_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TOKENS_SMEM) != cudaSuccess) {
            (void)cudaGetLastError();
            return HB_SETUP_FAILED;
        }
        scratch_address[device] = address;
    }
    return hb_attention_tokens(q, q_stride, out, out_stride, cache, block_table, table_width, token_row, positions, items, n_items,
                               splits, scratch_address[device], heads, kv_heads, head_dim, page_size, pages, scale, window, status,
                               stream);
}
