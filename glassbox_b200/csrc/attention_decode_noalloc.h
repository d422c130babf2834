// Decode attention for callers that cannot allocate device memory.
//
// This entry point is an addition of this library; the reference project has no counterpart.
//
// Who needs it: a host program that links this library through its C symbols and has no tensor
// allocator of its own (nothing of PyTorch in the process), a serving loop whose device memory was
// partitioned once at start-up and where a later cudaMalloc is forbidden (it synchronises the
// whole device and fails outright while a stream is being captured), or code that runs under a
// memory budget fixed in advance. The split-key decode attention normally needs three scratch
// buffers from its caller (partial outputs, partial softmax statistics, arrival counters); here
// they live in one array inside the library, so the caller passes inputs and outputs only.
//
// Limits and rules
//  * The scratch array is GB_NOALLOC_SCRATCH_BYTES (8 MiB) per GPU; every GPU that loads the
//    library holds it until the process ends. A call needs
//        rows * heads * 4 * splits * (head_dim + 2) * 4  +  rows * kv_heads * 4   bytes
//    (rounded up to 256-byte sections); a call that needs more is refused with an error, nothing runs.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress) with
//    that device current. Make that first call before any stream capture.
//  * Every call uses the same array and finds in it what the previous call left: the part that must
//    start at zero (the counters) is cleared on the caller's stream at each call. Two calls whose
//    kernels may overlap on the GPU (different streams, no dependency) race on the array: do not.
//  * Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
//
// Arguments are those of gb_attention_decode_mma without the scratch pointers; the result is the
// same. Returns 0 on success; otherwise non-zero, and gb_last_error() describes the refusal.
#pragma once

#include <cuda_runtime.h>

#define GB_NOALLOC_SCRATCH_BYTES (8u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int gb_attention_decode_noalloc(const void* q, long long q_stride, void* out, long long out_stride, const void* kcache,
                                const void* vcache, const int* block_tables, int max_pages, const int* row_seq,
                                const int* positions, int n, int nh, int nkv, int hd, int page_size,
                                long long num_pages, float scale, int window, int splits, int* status,
                                cudaStream_t stream);

// Bytes of the library's scratch array that a call of this shape would use (for callers that want
// to check before they call).
long long gb_attention_decode_noalloc_bytes(int n, int nh, int nkv, int hd, int splits);

#ifdef __cplusplus
}
#endif
