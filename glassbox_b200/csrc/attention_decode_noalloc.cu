// See attention_decode_noalloc.h. The kernel is the tensor-core decode attention of
// attention_decode_mma.cu, launched through its usual launcher; only the scratch differs: it is a
// file-scope device array of this translation unit.
#include "attention_decode_noalloc.h"

#include "common.cuh"

// In host code this name is only a stand-in for the device array: its device address has to be
// asked for (cudaGetSymbolAddress) before a kernel can be given it.
static __device__ __align__(256) unsigned char gb_noalloc_scratch[GB_NOALLOC_SCRATCH_BYTES];

extern "C" int gb_attention_decode_mma(const void* q, long long q_stride, void* out, long long out_stride,
                                       const void* kcache, const void* vcache, const int* block_tables, int max_pages,
                                       const int* row_seq, const int* positions, int n, int nh, int nkv, int hd,
                                       int page_size, long long num_pages, float scale, int window, int splits,
                                       float* part_acc, float* part_ml, int* counters, int* status,
                                       cudaStream_t stream);

static constexpr int MAX_DEVICES = 64;
static unsigned char* g_scratch_ptr[MAX_DEVICES] = {};

static long long align256(long long x) { return (x + 255) / 256 * 256; }

struct Sections {
    long long acc, ml, counters, total;
};

static Sections sections(int n, int nh, int nkv, int hd, int splits) {
    Sections s;
    s.acc = align256((long long)n * nh * 4 * splits * hd * (long long)sizeof(float));
    s.ml = align256((long long)n * nh * 4 * splits * 2 * (long long)sizeof(float));
    s.counters = align256((long long)n * nkv * (long long)sizeof(int));
    s.total = s.acc + s.ml + s.counters;
    return s;
}

GB_EXPORT long long gb_attention_decode_noalloc_bytes(int n, int nh, int nkv, int hd, int splits) {
    if (n < 0 || nh <= 0 || nkv <= 0 || hd <= 0 || splits <= 0) return -1;
    return sections(n, nh, nkv, hd, splits).total;
}

GB_EXPORT int gb_attention_decode_noalloc(const void* q, long long q_stride, void* out, long long out_stride,
                                          const void* kcache, const void* vcache, const int* block_tables,
                                          int max_pages, const int* row_seq, const int* positions, int n, int nh,
                                          int nkv, int hd, int page_size, long long num_pages, float scale, int window,
                                          int splits, int* status, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && nh > 0 && nkv > 0 && hd > 0 && splits > 0, "gb_attention_decode_noalloc: bad sizes");
    if (n == 0) return 0;
    const Sections s = sections(n, nh, nkv, hd, splits);
    GB_REQUIRE(s.total <= (long long)GB_NOALLOC_SCRATCH_BYTES,
               "gb_attention_decode_noalloc: this call needs %lld bytes of scratch, the built-in array holds %u "
               "(rows %d, heads %d, splits %d, head size %d): use fewer splits or rows, or the entry point that takes "
               "scratch from the caller",
               s.total, GB_NOALLOC_SCRATCH_BYTES, n, nh, splits, hd);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    GB_REQUIRE(e == cudaSuccess && dev >= 0 && dev < MAX_DEVICES, "gb_attention_decode_noalloc: no usable current device (%s)",
               cudaGetErrorString(e));
    if (g_scratch_ptr[dev] == nullptr) {   // set-up, once per device, with that device current
        unsigned char* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, gb_noalloc_scratch);
        GB_REQUIRE(e == cudaSuccess && p != nullptr, "gb_attention_decode_noalloc: cudaGetSymbolAddress failed: %s",
                   cudaGetErrorString(e));
        g_scratch_ptr[dev] = p;
    }
    unsigned char* base = g_scratch_ptr[dev];
    float* part_acc = reinterpret_cast<float*>(base);
    float* part_ml = reinterpret_cast<float*>(base + s.acc);
    int* counters = reinterpret_cast<int*>(base + s.acc + s.ml);
    // the counters must be zero when the kernel starts; whatever an earlier call left is cleared
    e = cudaMemsetAsync(counters, 0, (size_t)s.counters, stream);
    GB_REQUIRE(e == cudaSuccess, "gb_attention_decode_noalloc: clearing the counters failed: %s", cudaGetErrorString(e));
    return gb_attention_decode_mma(q, q_stride, out, out_stride, kcache, vcache, block_tables, max_pages, row_seq,
                                   positions, n, nh, nkv, hd, page_size, num_pages, scale, window, splits, part_acc,
                                   part_ml, counters, status, stream);
}
