// Pull the cache pages that a decode-attention kernel is about to read into L2, ahead of time.
//
// A decode step reads every live request's keys and values once per layer, and the attention kernel
// of a small batch is bound by the latency of those reads, not by bandwidth. While the feed-forward
// kernels of layer l run (they use little of the memory system), this kernel, launched on a second
// stream, walks the block tables and issues prefetch.global.L2 for the pages of layer l+1, so that
// its attention kernel finds them in L2. It writes nothing and needs no result.
#include "common.cuh"

__global__ void __launch_bounds__(256) kv_prefetch_kernel(const unsigned char* __restrict__ kcache,
                                                          const unsigned char* __restrict__ vcache,
                                                          const int* __restrict__ block_tables, int max_pages,
                                                          const int* __restrict__ row_seq,
                                                          const int* __restrict__ positions, int nkv, int page_size,
                                                          long long num_pages, long long tile_bytes, int window) {
    const int row = blockIdx.y;
    const int pos = positions[row];
    if (pos < 0 || pos / page_size >= max_pages) return;   // padding, or a position the block table does not reach
    const int* table = block_tables + (size_t)row_seq[row] * max_pages;
    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int page_lo = first / page_size, page_hi = pos / page_size;
    const int lines = (int)(tile_bytes / 128);            // 128-byte lines per (page, kv head) tile
    const long long total = (long long)(page_hi - page_lo + 1) * nkv * lines;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int line = (int)(i % lines);
        const long long tile = i / lines;
        const int kvh = (int)(tile % nkv);
        const long long page = table[page_lo + (int)(tile / nkv)];
        if (page < 0 || page >= num_pages) continue;
        const long long off = (page * nkv + kvh) * tile_bytes + (long long)line * 128;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(kcache + off));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(vcache + off));
    }
}

// tile_bytes = page_size * head_dim * element size (a multiple of 128).
GB_EXPORT int gb_kv_prefetch(const void* kcache, const void* vcache, const int* block_tables, int max_pages,
                             const int* row_seq, const int* positions, int n, int nkv, int page_size, long long num_pages,
                             long long tile_bytes, int window, int blocks_per_row, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && nkv > 0 && page_size > 0 && max_pages > 0 && blocks_per_row > 0, "gb_kv_prefetch: bad sizes");
    GB_REQUIRE(tile_bytes > 0 && tile_bytes % 128 == 0, "gb_kv_prefetch: a (page, kv head) tile must be a multiple of 128 bytes");
    if (n == 0) return 0;
    dim3 grid(blocks_per_row, n);
    kv_prefetch_kernel<<<grid, 256, 0, stream>>>((const unsigned char*)kcache, (const unsigned char*)vcache, block_tables,
                                                  max_pages, row_seq, positions, nkv, page_size, num_pages, tile_bytes,
                                                  window);
    return gb_check_launch("gb_kv_prefetch");
}

// A kernel that does nothing: a node of its own on a second stream (see GqaAttention.prefetch, which launches it where
// a real prefetch does not pay).
__global__ void stream_marker_kernel() {}

GB_EXPORT int gb_stream_marker(cudaStream_t stream) {
    stream_marker_kernel<<<1, 32, 0, stream>>>();
    return gb_check_launch("gb_stream_marker");
}
