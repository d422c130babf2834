// Paged grouped-query attention for rows that bring few queries per request (decoding): the keys
// of each (row, kv head) are split over several blocks so that a small batch still fills the GPU,
// and the block that finishes last merges the partial results (no second launch, no waiting).
//
// One block = one (row, kv head or sub-group of its query heads, split). It streams its range of
// keys 64 at a time through shared memory (cp.async, double buffered, one 16-byte chunk per
// thread per copy), so every key and value is read from HBM once for all query heads of the group.
// Scores, running maximum, running sum and the output are float32 (online softmax). The merge of
// the splits is the usual rescaling by exp(m_i - m).
// Semantics are those of crates/glassbox-core/src/model.rs:278-317: a row at position p sees keys
// max(0, p-window+1) .. p of its own request through the block table.
//
// Scratch: `part_acc` float32 [rows, heads, splits, head_dim], `part_ml` float32 [rows, heads,
// splits, 2] and `counters` int32 [rows * gridDim.y], the latter zero before the first launch (the
// kernel leaves it zero again).
#include "common.cuh"

#include <cuda_pipeline.h>

// Keys per tile (DK) is 64, 32 or 16, chosen so that the tiles fit in shared memory whatever the
// head size; a block has 2*DK threads (one per key and half of the channels), i.e. DK/16 warps.
constexpr float NEG_BIG = -1.0e30f;

template <typename T> struct Chunk;  // 16 bytes of T widened to floats
template <> struct Chunk<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
};
template <> struct Chunk<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        uint4 t = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

// exp: the float32 instantiation is the true 32-bit path and uses the accurate function.
template <typename T> __device__ __forceinline__ float exp_for(float x);
template <> __device__ __forceinline__ float exp_for<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ float exp_for<__nv_bfloat16>(float x) { return __expf(x); }

template <typename T> __device__ __forceinline__ float2 load_pair(const T* p);
template <> __device__ __forceinline__ float2 load_pair<float>(const float* p) {
    return *reinterpret_cast<const float2*>(p);
}
template <> __device__ __forceinline__ float2 load_pair<__nv_bfloat16>(const __nv_bfloat16* p) {
    uint32_t w = *reinterpret_cast<const uint32_t*>(p);
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

template <typename T, int GT, int DK>
__global__ void __launch_bounds__(2 * DK) attention_decode_kernel(
    const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
    const T* __restrict__ kcache, const T* __restrict__ vcache, const int* __restrict__ block_tables, int max_pages,
    const int* __restrict__ row_seq, const int* __restrict__ positions, int nh, int nkv, int hd, int page_size,
    long long num_pages, float scale, int window, int splits, float* __restrict__ part_acc,
    float* __restrict__ part_ml, int* __restrict__ counters, int* __restrict__ status) {
    constexpr int VEC = Chunk<T>::N;
    constexpr int DTHREADS = 2 * DK, NW = DK / 16;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int split = blockIdx.x, row = blockIdx.z;
    const int G = nh / nkv;
    const int subgroups = (G + GT - 1) / GT;
    const int kvh = blockIdx.y / subgroups, sg = blockIdx.y % subgroups;
    const int head0 = kvh * G + sg * GT;
    const int gcount = min(GT, G - sg * GT);
    const int half_dim = hd / 2;
    const int qpad = half_dim + 4;  // per-half row of q, padded against bank conflicts

    // shared memory carve-up
    T* Ks = reinterpret_cast<T*>(smem_raw);                    // [2][DK][hd]
    T* Vs = Ks + 2 * DK * hd;                                  // [2][DK][hd]
    float* qs = reinterpret_cast<float*>(Vs + 2 * DK * hd);    // [GT][2][qpad]
    float* ps = qs + GT * 2 * qpad;                            // [GT][DK]
    float* red = ps + GT * DK;                                 // [2][4][GT] (NW <= 4 rows used)
    long long* rowoff = reinterpret_cast<long long*>(red + 2 * 4 * GT);  // [2][DK]
    __shared__ int is_last;

    int pos = positions[row];
    if (pos >= 0 && pos / page_size >= max_pages) {   // a position the block table does not reach: reported, and the
        if (tid == 0) atomicOr(status, GB_STATUS_BAD_POSITION);   // row is treated as padding (nothing is read)
        pos = -1;
    }
    T* orow = out + (size_t)row * out_stride;
    if (pos < 0) {  // padding row
        if (split == 0)
            for (int i = tid; i < gcount * hd; i += DTHREADS) orow[head0 * hd + i] = gb_from_float<T>(0.f);
        return;
    }
    const int* table = block_tables + (size_t)row_seq[row] * max_pages;
    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int total = pos + 1 - first;
    const int chunk = ((total + splits - 1) / splits + DK - 1) / DK * DK;
    const int k_begin = first + split * chunk;
    const int k_end = min(pos + 1, k_begin + chunk);
    const int ntiles = k_end > k_begin ? (k_end - k_begin + DK - 1) / DK : 0;

    const T* qrow = q + (size_t)row * q_stride + head0 * hd;
    for (int i = tid; i < gcount * hd; i += DTHREADS) {
        int g = i / hd, d = i % hd;
        qs[(g * 2 + d / half_dim) * qpad + d % half_dim] = gb_to_float(qrow[i]);
    }

    const int cpr = hd / VEC;  // 16-byte chunks per key row
    auto load_tile = [&](int tile, int buf) {
        if (tid < DK) {
            int key = k_begin + tile * DK + tid;
            long long off = -1;
            if (key < k_end) {
                long long page = table[key / page_size];
                if (page < 0 || page >= num_pages) atomicOr(status, GB_STATUS_BAD_SLOT);
                else off = ((page * nkv + kvh) * page_size + key % page_size) * hd;
            }
            rowoff[buf * DK + tid] = off;
        }
        __syncthreads();
        T* kd = Ks + buf * DK * hd;
        T* vd = Vs + buf * DK * hd;
        for (int c = tid; c < DK * cpr; c += DTHREADS) {
            int kk = c / cpr, col = (c % cpr) * VEC;
            long long off = rowoff[buf * DK + kk];
            if (off >= 0) {
                __pipeline_memcpy_async(kd + kk * hd + col, kcache + off + col, 16);
                __pipeline_memcpy_async(vd + kk * hd + col, vcache + off + col, 16);
            }
        }
        __pipeline_commit();
    };

    float m_run[GT], l_run[GT];
    float acc[GT][8];  // this lane's output channels: 2*lane + 64*j + {0,1}, j < 4 (head_dim <= 256)
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        m_run[g] = NEG_BIG;
        l_run[g] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[g][j] = 0.f;
    }

    if (ntiles > 0) load_tile(0, 0);
    for (int tile = 0; tile < ntiles; ++tile) {
        const int buf = tile & 1;
        if (tile + 1 < ntiles) {
            load_tile(tile + 1, buf ^ 1);
            __pipeline_wait_prior(1);
        } else {
            __pipeline_wait_prior(0);
        }
        __syncthreads();
        const T* kt = Ks + buf * DK * hd;
        const T* vt = Vs + buf * DK * hd;

        // scores: thread = (key, half of the head's channels)
        const int kk = tid >> 1, half = tid & 1;
        const bool valid = rowoff[buf * DK + kk] >= 0;
        float dot[GT];
#pragma unroll
        for (int g = 0; g < GT; ++g) dot[g] = 0.f;
        if (valid) {
            const int nch = half_dim / VEC;
            const T* krow = kt + kk * hd + half * half_dim;
            for (int c = 0; c < nch; ++c) {
                const int cc = (c + kk) % nch;  // rotate so that neighbouring keys hit different banks
                float kv[VEC];
                Chunk<T>::load(krow + cc * VEC, kv);
#pragma unroll
                for (int g = 0; g < GT; ++g) {
                    if (g < gcount) {
                        const float* qv = qs + (g * 2 + half) * qpad + cc * VEC;
#pragma unroll
                        for (int e = 0; e < VEC; ++e) dot[g] = fmaf(qv[e], kv[e], dot[g]);
                    }
                }
            }
        }
        float s[GT];
#pragma unroll
        for (int g = 0; g < GT; ++g) {
            float d = dot[g] + __shfl_xor_sync(0xffffffffu, dot[g], 1);
            s[g] = valid ? d * scale : NEG_BIG;
            float wm = gb_warp_max(s[g]);
            if (lane == 0) red[warp * GT + g] = wm;
        }
        __syncthreads();
        float corr[GT];
#pragma unroll
        for (int g = 0; g < GT; ++g) {
            float mt = red[g];
#pragma unroll
            for (int w = 1; w < NW; ++w) mt = fmaxf(mt, red[w * GT + g]);
            float m_new = fmaxf(m_run[g], mt);
            float p = valid ? exp_for<T>(s[g] - m_new) : 0.f;
            corr[g] = exp_for<T>(m_run[g] - m_new);
            m_run[g] = m_new;
            if (half == 0) ps[g * DK + kk] = p;
            float ws = gb_warp_sum(half == 0 ? p : 0.f);
            if (lane == 0) red[(4 + warp) * GT + g] = ws;
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < GT; ++g) {
            float st = red[4 * GT + g];
#pragma unroll
            for (int w = 1; w < NW; ++w) st += red[(4 + w) * GT + g];
            l_run[g] = l_run[g] * corr[g] + st;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[g][j] *= corr[g];
        }
        // values: warp w takes keys [16w, 16w+16), lane takes channel pairs
        for (int t = 0; t < 16; ++t) {
            const int key = warp * 16 + t;
            if (rowoff[buf * DK + key] < 0) continue;
            const T* vrow = vt + key * hd;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int d = 2 * lane + 64 * j;
                if (d < hd) {
                    float2 v = load_pair<T>(vrow + d);
#pragma unroll
                    for (int g = 0; g < GT; ++g) {
                        float p = ps[g * DK + key];
                        acc[g][2 * j] = fmaf(p, v.x, acc[g][2 * j]);
                        acc[g][2 * j + 1] = fmaf(p, v.y, acc[g][2 * j + 1]);
                    }
                }
            }
        }
        __syncthreads();
    }

    // add up the warps' partial outputs (they covered different keys)
    float* accs = reinterpret_cast<float*>(smem_raw);  // [NW][GT][hd], reuses the tile memory
#pragma unroll
    for (int g = 0; g < GT; ++g)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int d = 2 * lane + 64 * j;
            if (d < hd) {
                accs[(warp * GT + g) * hd + d] = acc[g][2 * j];
                accs[(warp * GT + g) * hd + d + 1] = acc[g][2 * j + 1];
            }
        }
    __syncthreads();
    for (int i = tid; i < gcount * hd; i += DTHREADS) {
        const int g = i / hd, d = i % hd;
        float v = accs[g * hd + d];
#pragma unroll
        for (int w = 1; w < NW; ++w) v += accs[(w * GT + g) * hd + d];
        // m_run / l_run are identical in every thread, but indexed by a compile-time g: select
        float l = 0.f;
#pragma unroll
        for (int gg = 0; gg < GT; ++gg) if (gg == g) l = l_run[gg];
        if (splits == 1) {
            orow[(head0 + g) * hd + d] = gb_from_float<T>(l > 0.f ? v / l : 0.f);
        } else {
            part_acc[(((size_t)row * nh + head0 + g) * splits + split) * hd + d] = v;
        }
    }
    if (splits == 1) return;
    if (tid < gcount) {
        float m = 0.f, l = 0.f;
#pragma unroll
        for (int gg = 0; gg < GT; ++gg) if (gg == tid) { m = m_run[gg]; l = l_run[gg]; }
        float* ml = part_ml + (((size_t)row * nh + head0 + tid) * splits + split) * 2;
        ml[0] = m;
        ml[1] = l;
    }
    // the block that arrives last merges the splits
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int* counter = counters + (size_t)row * gridDim.y + blockIdx.y;
        int prev = atomicAdd(counter, 1);
        is_last = (prev == splits - 1);
        if (is_last) *counter = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int i = tid; i < gcount * hd; i += DTHREADS) {
        const int g = i / hd, d = i % hd;
        const float* ml = part_ml + ((size_t)row * nh + head0 + g) * splits * 2;
        const float* pa = part_acc + ((size_t)row * nh + head0 + g) * splits * hd;
        float m = NEG_BIG;
        for (int sidx = 0; sidx < splits; ++sidx) m = fmaxf(m, __ldcg(ml + 2 * sidx));
        float l = 0.f, v = 0.f;
        for (int sidx = 0; sidx < splits; ++sidx) {
            float w = exp_for<T>(__ldcg(ml + 2 * sidx) - m);
            l = fmaf(__ldcg(ml + 2 * sidx + 1), w, l);
            v = fmaf(__ldcg(pa + (size_t)sidx * hd + d), w, v);
        }
        orow[(head0 + g) * hd + d] = gb_from_float<T>(l > 0.f ? v / l : 0.f);
    }
}

static size_t decode_smem_bytes(int hd, int elem, int gt, int dk) {
    size_t tiles = (size_t)4 * dk * hd * elem;
    size_t rest = (size_t)(gt * 2 * (hd / 2 + 4) + gt * dk + 2 * 4 * gt) * sizeof(float) + 2 * dk * sizeof(long long);
    size_t merge = (size_t)(dk / 16) * gt * hd * sizeof(float);
    size_t total = tiles + rest;
    return total > merge ? total : merge;
}

template <typename T, int GT, int DK>
static int launch_decode_dk(const void* q, long long q_stride, void* out, long long out_stride, const void* kcache,
                         const void* vcache, const int* block_tables, int max_pages, const int* row_seq,
                         const int* positions, int n, int nh, int nkv, int hd, int page_size, long long num_pages,
                         float scale, int window, int splits, float* part_acc, float* part_ml, int* counters,
                         int* status, cudaStream_t stream) {
    const int G = nh / nkv;
    const int subgroups = (G + GT - 1) / GT;
    size_t smem = decode_smem_bytes(hd, sizeof(T), GT, DK);
    auto kernel = attention_decode_kernel<T, GT, DK>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        GB_REQUIRE(e == cudaSuccess, "gb_attention_decode: %zu bytes of shared memory refused: %s", smem,
                   cudaGetErrorString(e));
    }
    dim3 grid(splits, nkv * subgroups, n);
    kernel<<<grid, 2 * DK, smem, stream>>>((const T*)q, q_stride, (T*)out, out_stride, (const T*)kcache,
                                             (const T*)vcache, block_tables, max_pages, row_seq, positions, nh, nkv, hd,
                                             page_size, num_pages, scale, window, splits, part_acc, part_ml, counters,
                                             status);
    return gb_check_launch("gb_attention_decode");
}

template <typename T, int GT>
static int launch_decode(const void* q, long long q_stride, void* out, long long out_stride, const void* kcache,
                         const void* vcache, const int* block_tables, int max_pages, const int* row_seq,
                         const int* positions, int n, int nh, int nkv, int hd, int page_size, long long num_pages,
                         float scale, int window, int splits, float* part_acc, float* part_ml, int* counters,
                         int* status, cudaStream_t stream) {
    const size_t row_bytes = (size_t)hd * sizeof(T);
#define GB_DK(DKK)                                                                                                  \
    return launch_decode_dk<T, GT, DKK>(q, q_stride, out, out_stride, kcache, vcache, block_tables, max_pages, row_seq, \
                                        positions, n, nh, nkv, hd, page_size, num_pages, scale, window, splits,       \
                                        part_acc, part_ml, counters, status, stream);
    if (row_bytes <= 256) { GB_DK(64) }
    if (row_bytes <= 512) { GB_DK(32) }
    GB_DK(16)
#undef GB_DK
}

// Number of int32 counters the kernel needs for `n` rows.
GB_EXPORT int gb_attention_decode_counters(int n, int nh, int nkv) {
    const int G = nh / nkv;
    const int gt = G <= 4 ? G : 4;
    return n * nkv * ((G + gt - 1) / gt);
}

GB_EXPORT int gb_attention_decode(const void* q, long long q_stride, void* out, long long out_stride, int dtype,
                                  const void* kcache, const void* vcache, const int* block_tables, int max_pages,
                                  const int* row_seq, const int* positions, int n, int nh, int nkv, int hd,
                                  int page_size, long long num_pages, float scale, int window, int splits,
                                  float* part_acc, float* part_ml, int* counters, int* status,
                                  cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "gb_attention_decode: heads %d must be a multiple of kv heads %d",
               nh, nkv);
    GB_REQUIRE(hd >= 16 && hd <= 256 && hd % 16 == 0, "gb_attention_decode: head size %d must be a multiple of 16 in 16..256", hd);
    GB_REQUIRE(page_size > 0 && max_pages > 0 && splits >= 1, "gb_attention_decode: bad page geometry or split count");
    GB_REQUIRE(splits == 1 || (part_acc && part_ml && counters), "gb_attention_decode: splits need scratch buffers");
    GB_REQUIRE(n <= 65535 && splits <= 65535, "gb_attention_decode: too many rows or splits for one launch");
    if (n == 0) return 0;
    const int G = nh / nkv;
    const int gt = G <= 4 ? G : 4;
#define GB_DECODE(TT, GG)                                                                                       \
    return launch_decode<TT, GG>(q, q_stride, out, out_stride, kcache, vcache, block_tables, max_pages, row_seq, \
                                 positions, n, nh, nkv, hd, page_size, num_pages, scale, window, splits,        \
                                 part_acc, part_ml, counters, status, stream);
    if (dtype == GB_BF16) {
        if (gt == 1) { GB_DECODE(__nv_bfloat16, 1) }
        if (gt == 2) { GB_DECODE(__nv_bfloat16, 2) }
        if (gt == 3) { GB_DECODE(__nv_bfloat16, 3) }
        GB_DECODE(__nv_bfloat16, 4)
    } else if (dtype == GB_F32) {
        if (gt == 1) { GB_DECODE(float, 1) }
        if (gt == 2) { GB_DECODE(float, 2) }
        if (gt == 3) { GB_DECODE(float, 3) }
        GB_DECODE(float, 4)
    }
#undef GB_DECODE
    GB_REQUIRE(false, "gb_attention_decode: unsupported dtype %d", dtype);
}
