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

template <int HD, int BK, int NW, bool CLUSTER>
__global__ void __launch_bounds__(NW * 32) attention_decode_mma_kernel(const DecodeAttnArgs a) {
    __shared__ DecodeAttnSmem sm;
    extern __shared__ __align__(16) float cluster_part[];   // CLUSTER: the first block's copy receives every warp's partial result
    GbPdlSync sync;
    attention_decode_mma_body<HD, BK, GbPdlSync, NW, CLUSTER>(a, (int)blockIdx.x, (int)blockIdx.y, (int)blockIdx.z, sm, sync, cluster_part);
}

// The merge runs inside a thread-block cluster in the variant for large batches (16 keys per iteration: small
// blocks, several per SM), when the splits of a (row, kv head) fit one cluster (at most 8 blocks) and their partial
// results fit the first block's shared memory. Measured at 9/3 heads, context 4096: batch 32 24.8 -> 23.2 us,
// batch 64 43.0 -> 41.0 us. The small-batch variants keep the merge through global memory: their blocks fill an SM
// each, clusters of 6 then no longer all find room in one wave (batch 8: 12.5 -> 19.5 us), and at batch 1 the
// cluster's barrier is no faster than the counter (11.2 -> 12.0 us).
constexpr int MMA_CLUSTER_SMEM_MAX = 96 * 1024;

template <int HD, int BK, int NW>
static int launch_mma(const void* q, long long q_stride, void* out, long long out_stride, const void* kcache,
                      const void* vcache, const int* block_tables, int max_pages, const int* row_seq,
                      const int* positions, int n, int nh, int nkv, int page_size, long long num_pages, float scale,
                      int window, int splits, float* part_acc, float* part_ml, int* counters, int* status, int pdl,
                      cudaStream_t stream) {
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    DecodeAttnArgs a = {};
    a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride; a.out = (__nv_bfloat16*)out; a.out_stride = out_stride;
    a.kcache = (const __nv_bfloat16*)kcache; a.vcache = (const __nv_bfloat16*)vcache; a.block_tables = block_tables;
    a.max_pages = max_pages; a.row_seq = row_seq; a.positions = positions; a.nh = nh; a.nkv = nkv; a.page_size = page_size;
    a.page_shift = page_shift; a.num_pages = num_pages; a.scale = scale; a.window = window; a.splits = splits;
    a.part_acc = part_acc; a.part_ml = part_ml; a.counters = counters; a.status = status; a.n = n; a.hd = HD; a.block_keys = BK;
    a.late_release = 1;   // (135M decode step at batch 1: 0.646 -> 0.630 ms; no difference at batch 64)
    const int group = nh / nkv;
    const int cluster_bytes = decode_attn_cluster_floats<HD>(group, splits, NW) * (int)sizeof(float);
    const bool in_cluster = BK == 16 && NW == 4 && splits <= 8 && cluster_bytes <= MMA_CLUSTER_SMEM_MAX && group * splits * NW <= MMA_MAX_MERGE;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, nkv, n);
    cfg.blockDim = dim3(NW * 32);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cudaError_t e;
    if (in_cluster) {
        static int configured = 0;
        if (cluster_bytes > configured) {
            e = cudaFuncSetAttribute(attention_decode_mma_kernel<HD, BK, NW, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, MMA_CLUSTER_SMEM_MAX);
            GB_REQUIRE(e == cudaSuccess, "gb_attention_decode_mma: %d bytes of shared memory refused: %s", MMA_CLUSTER_SMEM_MAX, cudaGetErrorString(e));
            configured = MMA_CLUSTER_SMEM_MAX;
        }
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = splits;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
        cfg.dynamicSmemBytes = cluster_bytes;
        cfg.attrs = attr;
        cfg.numAttrs = na;
        e = cudaLaunchKernelEx(&cfg, attention_decode_mma_kernel<HD, BK, NW, true>, a);
    } else {
        cfg.attrs = attr;
        cfg.numAttrs = na;
        e = cudaLaunchKernelEx(&cfg, attention_decode_mma_kernel<HD, BK, NW, false>, a);
    }
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
                                          int pdl, int block_keys, int warps, cudaStream_t stream) {
    GB_REQUIRE(gb_attention_decode_mma_supported(nh, nkv, hd),
               "gb_attention_decode_mma: head size %d with %d heads per kv head is not built (16/32/64/128, <= 16)", hd,
               nkv > 0 ? nh / nkv : 0);
    GB_REQUIRE(page_size >= 16 && (page_size & (page_size - 1)) == 0,
               "gb_attention_decode_mma: page size %d must be a power of two >= 16", page_size);
    GB_REQUIRE((long long)num_pages * nkv * page_size < (1ll << 31), "gb_attention_decode_mma: the cache has too many rows");
    GB_REQUIRE(max_pages > 0 && splits >= 1 && part_acc && part_ml && counters,
               "gb_attention_decode_mma: bad page geometry, split count or scratch");
    GB_REQUIRE(warps == 4 || (warps == 8 && hd == 64), "gb_attention_decode_mma: %d warps per block are not built for this variant (4; 8 at head size 64)", warps);
    GB_REQUIRE(n <= 65535 && splits <= MMA_MAX_MERGE / warps, "gb_attention_decode_mma: too many rows or splits for one launch");
    GB_REQUIRE(q_stride % 4 == 0 && (uintptr_t)q % 8 == 0, "gb_attention_decode_mma: q must be 8-byte aligned");
    if (n == 0) return 0;
#define GB_MMA(HH, BB) GB_MMAW(HH, BB, 4)
#define GB_MMAW(HH, BB, WW)                                                                                        \
    return launch_mma<HH, BB, WW>(q, q_stride, out, out_stride, kcache, vcache, block_tables, max_pages, row_seq, positions, \
                              n, nh, nkv, page_size, num_pages, scale, window, splits, part_acc, part_ml, counters,       \
                              status, pdl, stream);
    if (hd == 16) { GB_MMA(16, 32) }
    if (hd == 32) { GB_MMA(32, 32) }
    if (hd == 64) {
        if (block_keys == 16 && warps == 8) { GB_MMAW(64, 16, 8) }   // a small batch: one block per SM that leaves room beside it
        if (block_keys == 16) { GB_MMA(64, 16) }   // fewer registers, three blocks per SM: better for large batches
        if (warps == 8) { GB_MMAW(64, 32, 8) }     // a small batch: one block per SM, twice the warps
        GB_MMA(64, 32)
    }
    GB_MMA(128, 16)
#undef GB_MMA
#undef GB_MMAW
}

GB_EXPORT int gb_attention_decode_mma(const void* q, long long q_stride, void* out, long long out_stride,
                                      const void* kcache, const void* vcache, const int* block_tables, int max_pages,
                                      const int* row_seq, const int* positions, int n, int nh, int nkv, int hd,
                                      int page_size, long long num_pages, float scale, int window, int splits,
                                      float* part_acc, float* part_ml, int* counters, int* status,
                                      cudaStream_t stream) {
    return gb_attention_decode_mma_pdl(q, q_stride, out, out_stride, kcache, vcache, block_tables, max_pages, row_seq,
                                       positions, n, nh, nkv, hd, page_size, num_pages, scale, window, splits, part_acc,
                                       part_ml, counters, status, 0, 0, 4, stream);
}
