// Paged grouped-query decode attention in bfloat16 on the tensor cores, with no shared-memory
// staging and no block-wide barrier in the key loop.
//
// One block = one (row, kv head, split of the keys); its four warps take interleaved blocks of BK
// keys. The query heads that share the kv head (up to 16) are the 16 rows of the mma tile, so each
// key and value is read once for the whole group. Keys and values go straight from HBM into the
// register layout of mma.sync m16n8k16:
//   * scores S = Q K^T: the key handled by a lane group is the tile's column; a thread's 8 bytes of
//     a key are 4 consecutive channels, and the instruction's k index is a fixed permutation of the
//     channels applied to Q and K alike;
//   * output O = P V: the probabilities are reused in registers as the A operand; the instruction's
//     column n of channel tile j stands for channel (HD/8)*n + j, so a thread needs HD/8 consecutive
//     channels of its four value rows (one 16-byte load at HD 64) and ends up owning 2*HD/8
//     consecutive output channels.
// Softmax statistics and accumulators are float32. Every warp writes its partial result (maximum,
// sum, unnormalised output) and the block that finishes last merges all of them.
// Semantics as crates/glassbox-core/src/model.rs:278-317 (keys max(0, p-window+1) .. p).
// The cache must hold finite numbers everywhere (it is zero-filled when allocated): rows of a page
// beyond a request's length are loaded and then masked, not skipped.
//
// Scratch: part_acc float32 [rows, heads, 4*splits, HD], part_ml float32 [rows, heads, 4*splits, 2],
// counters int32 [rows * kv heads], zero on entry and left zero.
#include "attention_decode_mma_body.cuh"

template <int HD, int BK>
__global__ void __launch_bounds__(128) attention_decode_mma_kernel(const DecodeAttnArgs a) {
    __shared__ DecodeAttnSmem sm;
    GbPdlSync sync;
    attention_decode_mma_body<HD, BK>(a, (int)blockIdx.x, (int)blockIdx.y, (int)blockIdx.z, sm, sync);
}

template <int HD, int BK>
static int launch_mma(const void* q, long long q_stride, void* out, long long out_stride, const void* kcache,
                      const void* vcache, const int* block_tables, int max_pages, const int* row_seq,
                      const int* positions, int n, int nh, int nkv, int page_size, long long num_pages, float scale,
                      int window, int splits, float* part_acc, float* part_ml, int* counters, int* status, int pdl,
                      cudaStream_t stream) {
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, nkv, n);
    cfg.blockDim = dim3(128);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    DecodeAttnArgs a = {};
    a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride; a.out = (__nv_bfloat16*)out; a.out_stride = out_stride;
    a.kcache = (const __nv_bfloat16*)kcache; a.vcache = (const __nv_bfloat16*)vcache; a.block_tables = block_tables;
    a.max_pages = max_pages; a.row_seq = row_seq; a.positions = positions; a.nh = nh; a.nkv = nkv; a.page_size = page_size;
    a.page_shift = page_shift; a.num_pages = num_pages; a.scale = scale; a.window = window; a.splits = splits;
    a.part_acc = part_acc; a.part_ml = part_ml; a.counters = counters; a.status = status; a.n = n; a.hd = HD; a.block_keys = BK;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_decode_mma_kernel<HD, BK>, a);
    if (e != cudaSuccess) {
        gb_set_error("gb_attention_decode_mma: launch failed: %s", cudaGetErrorString(e));
        return 2;
    }
    return gb_check_launch("gb_attention_decode_mma");
}

// 1 if (head size, group size) is one this kernel is built for.
GB_EXPORT int gb_attention_decode_mma_supported(int nh, int nkv, int hd) {
    if (nkv <= 0 || nh % nkv) return 0;
    return (hd == 16 || hd == 32 || hd == 64 || hd == 128) && nh / nkv <= 16;
}

// As gb_attention_decode_mma, with the choice of launching under programmatic stream serialisation
// (pdl != 0): the kernel then starts while its predecessor in the stream still runs, reads only step
// metadata until the predecessor has finished, and releases its own successor at once. block_keys
// (0 = default) picks the variant that takes 16 keys per warp iteration where one is built (head
// size 64): fewer registers, more blocks per SM, which pays when the batch alone fills the GPU.
GB_EXPORT int gb_attention_decode_mma_pdl(const void* q, long long q_stride, void* out, long long out_stride,
                                          const void* kcache, const void* vcache, const int* block_tables,
                                          int max_pages, const int* row_seq, const int* positions, int n, int nh,
                                          int nkv, int hd, int page_size, long long num_pages, float scale, int window,
                                          int splits, float* part_acc, float* part_ml, int* counters, int* status,
                                          int pdl, int block_keys, cudaStream_t stream) {
    GB_REQUIRE(gb_attention_decode_mma_supported(nh, nkv, hd),
               "gb_attention_decode_mma: head size %d with %d heads per kv head is not built (16/32/64/128, <= 16)", hd,
               nkv > 0 ? nh / nkv : 0);
    GB_REQUIRE(page_size >= 16 && (page_size & (page_size - 1)) == 0,
               "gb_attention_decode_mma: page size %d must be a power of two >= 16", page_size);
    GB_REQUIRE((long long)num_pages * nkv * page_size < (1ll << 31), "gb_attention_decode_mma: the cache has too many rows");
    GB_REQUIRE(max_pages > 0 && splits >= 1 && part_acc && part_ml && counters,
               "gb_attention_decode_mma: bad page geometry, split count or scratch");
    GB_REQUIRE(n <= 65535 && splits <= MMA_MAX_MERGE / 4, "gb_attention_decode_mma: too many rows or splits for one launch");
    GB_REQUIRE(q_stride % 4 == 0 && (uintptr_t)q % 8 == 0, "gb_attention_decode_mma: q must be 8-byte aligned");
    if (n == 0) return 0;
#define GB_MMA(HH, BB)                                                                                             \
    return launch_mma<HH, BB>(q, q_stride, out, out_stride, kcache, vcache, block_tables, max_pages, row_seq, positions, \
                              n, nh, nkv, page_size, num_pages, scale, window, splits, part_acc, part_ml, counters,       \
                              status, pdl, stream);
    if (hd == 16) { GB_MMA(16, 32) }
    if (hd == 32) { GB_MMA(32, 32) }
    if (hd == 64) {
        if (block_keys == 16) { GB_MMA(64, 16) }   // fewer registers, three blocks per SM: better for large batches
        GB_MMA(64, 32)
    }
    GB_MMA(128, 16)
#undef GB_MMA
}

GB_EXPORT int gb_attention_decode_mma(const void* q, long long q_stride, void* out, long long out_stride,
                                      const void* kcache, const void* vcache, const int* block_tables, int max_pages,
                                      const int* row_seq, const int* positions, int n, int nh, int nkv, int hd,
                                      int page_size, long long num_pages, float scale, int window, int splits,
                                      float* part_acc, float* part_ml, int* counters, int* status,
                                      cudaStream_t stream) {
    return gb_attention_decode_mma_pdl(q, q_stride, out, out_stride, kcache, vcache, block_tables, max_pages, row_seq,
                                       positions, n, nh, nkv, hd, page_size, num_pages, scale, window, splits, part_acc,
                                       part_ml, counters, status, 0, 0, stream);
}
