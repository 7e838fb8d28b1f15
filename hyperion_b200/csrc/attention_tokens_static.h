// hb_attention_tokens_static: the split-key decode attention for callers that must not allocate.
//
// This entry point has no counterpart in the reference; it exists for users of this library.
//
// Who needs it.  hb_attention_tokens (attention_bf16.cu) splits the keys of a decoded token over several
// blocks and needs a float workspace for the partial results, which its caller allocates.  Some callers
// cannot do that at the moment of the call: code that runs inside a stream capture or a real-time loop
// where cudaMalloc (which synchronises the device and may fail) is forbidden, plug-ins that are handed
// input and output buffers by a host application and own no allocator, and processes whose memory budget
// was fixed at start-up.  For them the library itself carries the workspace, as a file-scope device array
// of fixed size.
//
// What it costs.  The array is HB_STATIC_SCRATCH_FLOATS floats (16 MiB).  Every GPU on which this
// library is loaded holds it from load until the process exits, whether or not the entry point is called.
//
// Contract.
//  * Same arguments and same result as hb_attention_tokens, without the workspace pointer.
//  * It refuses (returns HB_SCRATCH_TOO_SMALL = -3, launching nothing) when
//    n_items * heads * splits * (head_dim + 2) exceeds HB_STATIC_SCRATCH_FLOATS; use fewer splits or fewer
//    tokens per call, or the allocating entry point.
//  * It calls no cudaMalloc, cudaFree or other allocating routine.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
//    device current) and sets the kernel's shared-memory attribute; make that first call outside any
//    stream capture.  A failed look-up returns HB_SETUP_FAILED = -4.
//  * All calls on a device share the one array, which keeps the previous call's contents.  Nothing in it
//    has to start at zero: every slot the merge kernel reads is written by the split kernel of the same
//    call first.  Two calls that overlap on the GPU (different streams, or the same call replayed
//    concurrently) race on it; serialise them.
#pragma once
#include <cuda_runtime.h>

#define HB_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)
#define HB_SCRATCH_TOO_SMALL (-3)
#define HB_SETUP_FAILED (-4)

extern "C" int hb_attention_tokens_static(const void* q, int q_stride, void* out, int out_stride, const void* cache,
                                          const int* block_table, int table_width, const int* token_row, const int* positions,
                                          const int* items, int n_items, int splits, int heads, int kv_heads, int head_dim,
                                          int page_size, int pages, float scale, int window, int* status, cudaStream_t stream);

// The capacity in floats, for callers that want to size their calls.
extern "C" long long hb_attention_tokens_static_capacity(void);
