// Causal grouped-query attention over the paged cache, one warp per (row, head).
//
// This kernel takes any batch row: a token of a prompt portion or a single decoded token. A row
// at position p of its request sees keys max(0, p-window+1) .. p of that request, read through
// the request's block table; there is no mask tensor (crates/glassbox-core/src/model.rs:278-317).
// Scores, the running maximum, the running sum and the output are float32 (online softmax).
// Keys are taken 32 at a time starting from the first visible key, so the reduction order of a
// row depends only on its position and window, not on the batch or on which pages hold the keys.
// It is the float32 path's attention and the reference kernel beside the tensor-core ones.
#include "common.cuh"

#include <float.h>

constexpr int ATT_WARPS = 4;
constexpr int ATT_MAX_HD = 256;

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32) attention_rows_kernel(
    const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
    const T* __restrict__ kcache, const T* __restrict__ vcache, const int* __restrict__ block_tables,
    int max_pages, const int* __restrict__ row_seq, const int* __restrict__ positions, int n, int nh, int nkv,
    int hd, int page_size, long long num_pages, float scale, int window, int* __restrict__ status) {
    __shared__ float qs[ATT_WARPS][ATT_MAX_HD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long task = (long long)blockIdx.x * ATT_WARPS + warp;
    if (task >= (long long)n * nh) return;
    const int row = (int)(task / nh), head = (int)(task % nh);
    const int kvh = head / (nh / nkv);
    int pos = positions[row];
    if (pos >= 0 && pos / page_size >= max_pages) {   // a position the block table does not reach: reported, the row reads nothing
        if (lane == 0) atomicOr(status, GB_STATUS_BAD_POSITION);
        pos = -1;
    }
    const int* table = block_tables + (size_t)row_seq[row] * max_pages;

    const T* qrow = q + (size_t)row * q_stride + head * hd;
    for (int i = lane; i < hd; i += 32) qs[warp][i] = gb_to_float(qrow[i]);
    __syncwarp();

    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    float m = -FLT_MAX, l = 0.f;
    float acc[ATT_MAX_HD / 32];
#pragma unroll
    for (int j = 0; j < ATT_MAX_HD / 32; ++j) acc[j] = 0.f;

    for (int base = first; base <= pos; base += 32) {
        const int key = base + lane;
        float s = -FLT_MAX;
        long long vrow = -1;  // element offset of this lane's key row in the cache
        if (key <= pos) {
            long long page = table[key / page_size];
            if (page < 0 || page >= num_pages) {
                atomicOr(status, GB_STATUS_BAD_SLOT);
            } else {
                vrow = ((page * nkv + kvh) * page_size + key % page_size) * hd;
                const T* kp = kcache + vrow;
                float d = 0.f;
                for (int i = 0; i < hd; ++i) d = fmaf(qs[warp][i], gb_to_float(kp[i]), d);
                s = d * scale;
            }
        }
        float m_new = fmaxf(m, gb_warp_max(s));
        float p = (vrow >= 0) ? expf(s - m_new) : 0.f;
        float corr = expf(m - m_new);
        l = l * corr + gb_warp_sum(p);
#pragma unroll
        for (int j = 0; j < ATT_MAX_HD / 32; ++j) acc[j] *= corr;
        m = m_new;
        const int count = min(32, pos - base + 1);
        for (int t = 0; t < count; ++t) {
            float pt = __shfl_sync(0xffffffffu, p, t);
            long long vr = __shfl_sync(0xffffffffu, vrow, t);
            if (vr < 0) continue;
            const T* vp = vcache + vr;
#pragma unroll
            for (int j = 0; j < ATT_MAX_HD / 32; ++j) {
                int i = lane + 32 * j;
                if (i < hd) acc[j] = fmaf(pt, gb_to_float(vp[i]), acc[j]);
            }
        }
    }
    T* orow = out + (size_t)row * out_stride + head * hd;
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int j = 0; j < ATT_MAX_HD / 32; ++j) {
        int i = lane + 32 * j;
        if (i < hd) orow[i] = gb_from_float<T>(acc[j] * inv);
    }
}

GB_EXPORT int gb_attention_rows(const void* q, long long q_stride, void* out, long long out_stride, int dtype,
                                const void* kcache, const void* vcache, const int* block_tables, int max_pages,
                                const int* row_seq, const int* positions, int n, int nh, int nkv, int hd,
                                int page_size, long long num_pages, float scale, int window, int* status,
                                cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "gb_attention_rows: heads %d must be a multiple of kv heads %d",
               nh, nkv);
    GB_REQUIRE(hd > 0 && hd <= ATT_MAX_HD, "gb_attention_rows: head size %d is outside 1..%d", hd, ATT_MAX_HD);
    GB_REQUIRE(page_size > 0 && max_pages > 0, "gb_attention_rows: bad page geometry");
    if (n == 0) return 0;
    long long tasks = (long long)n * nh;
    int blocks = gb_ceil_div(tasks, ATT_WARPS);
    if (dtype == GB_F32)
        attention_rows_kernel<float><<<blocks, ATT_WARPS * 32, 0, stream>>>(
            (const float*)q, q_stride, (float*)out, out_stride, (const float*)kcache, (const float*)vcache,
            block_tables, max_pages, row_seq, positions, n, nh, nkv, hd, page_size, num_pages, scale, window, status);
    else if (dtype == GB_BF16)
        attention_rows_kernel<__nv_bfloat16><<<blocks, ATT_WARPS * 32, 0, stream>>>(
            (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)kcache,
            (const __nv_bfloat16*)vcache, block_tables, max_pages, row_seq, positions, n, nh, nkv, hd, page_size,
            num_pages, scale, window, status);
    else
        GB_REQUIRE(false, "gb_attention_rows: unsupported dtype %d", dtype);
    return gb_check_launch("gb_attention_rows");
}
