// Causal grouped-query flash attention for prompt portions, over the paged cache, in bfloat16 on
// the tensor cores (mma.sync m16n8k16, float32 softmax statistics and accumulators).
//
// One block = 64 consecutive query rows of one request for one query head, eight warps in two groups:
// within a group the four warps own 16 rows each; the groups take alternate tiles of 64 keys (what
// bounds a causal kernel is its longest block, the one with the most key tiles, so the tiles of one
// block are worked on by two groups at once) and their results are merged at the end. Keys and values are read from the cache pages through the request's block table (the
// rows of this very step were stored there before this kernel runs, so a portion attends to the
// pages earlier portions left and to itself alike), 64 keys at a time, staged in shared memory with
// cp.async (three buffers: loads run two tiles ahead; 16-byte chunks XOR-swizzled by row so that
// ldmatrix is conflict free).
// A query at position p sees keys max(0, p-window+1) .. p (crates/glassbox-core/src/model.rs:278-317);
// tiles of keys that no row of the block can see are never loaded.
// Row-wise online softmax: m and l per row, O rescaled when m grows; P is rounded to bfloat16 for
// the P V product, as usual for this scheme.
#include "common.cuh"

#include <cuda_pipeline.h>

constexpr int PF_BM = 64, PF_BN = 64;
constexpr int PF_STAGES = 3;   // key/value tiles in flight: loads run two tiles ahead of the arithmetic
constexpr int PF_MAX_PAGES = 1024;
constexpr float PF_NEG_BIG = -1.0e30f;

__device__ __forceinline__ void pf_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t pf_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD>
__global__ void __launch_bounds__(256) attention_prefill_kernel(
    const __nv_bfloat16* __restrict__ q, long long q_stride, __nv_bfloat16* __restrict__ out, long long out_stride,
    const __nv_bfloat16* __restrict__ kcache, const __nv_bfloat16* __restrict__ vcache,
    const int* __restrict__ block_tables, int max_pages, const int* __restrict__ seq_first_row,
    const int* __restrict__ seq_start_pos, int nh, int nkv, int page_size, int page_shift, long long num_pages,
    float scale, int window, int* __restrict__ status) {
    constexpr int KS = HD / 16, NT = HD / 8, CPR = HD / 8;   // k16 steps, n8 tiles, 16-byte chunks per row
    extern __shared__ __align__(128) unsigned char pf_smem[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(pf_smem);   // [64][HD]
    __shared__ int pages_s[PF_MAX_PAGES];

    const int group = threadIdx.x >> 7;                    // which half of the key tiles
    const int tid = threadIdx.x & 127, lane = tid & 31, warp = tid >> 5;   // within the group
    __nv_bfloat16* Ks = Qs + PF_BM * HD + group * (2 * PF_STAGES * PF_BN * HD);   // [PF_STAGES][64][HD], per group
    __nv_bfloat16* Vs = Ks + PF_STAGES * PF_BN * HD;                               // [PF_STAGES][64][HD]
    auto group_sync = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory"); };
    const int g = lane >> 2, t = lane & 3;
    const int qt = gridDim.x - 1 - blockIdx.x;   // later tiles see more keys: start the longest blocks first
    const int head = blockIdx.y, seq = blockIdx.z;
    const int row0 = seq_first_row[seq];
    const int nrows = seq_first_row[seq + 1] - row0;
    if (qt * PF_BM >= nrows) return;
    int start_pos = seq_start_pos[seq];
    if (start_pos >= 0 && ((start_pos + nrows - 1) >> page_shift) >= max_pages) {   // rows beyond the block table:
        if (threadIdx.x == 0) atomicOr(status, GB_STATUS_BAD_POSITION);             // reported, treated as padding
        start_pos = -1;
    }
    if (start_pos < 0) {                          // a padding sequence of a fixed-shape batch (uniform for the block):
        for (int i = threadIdx.x; i < nrows * (HD / 2); i += blockDim.x)   // its rows read as zeros downstream
            *reinterpret_cast<uint32_t*>(out + (size_t)(row0 + i / (HD / 2)) * out_stride + (size_t)head * HD + (i % (HD / 2)) * 2) = 0u;
        return;
    }
    const int kvh = head / (nh / nkv);
    const int q_lo = qt * PF_BM;
    const int pos_lo = start_pos + q_lo, pos_hi = start_pos + min(nrows, q_lo + PF_BM) - 1;
    const int key_lo = (window > 0 && pos_lo + 1 > window) ? pos_lo + 1 - window : 0;
    const int kt_begin = key_lo / PF_BN, kt_end = pos_hi / PF_BN;   // inclusive
    const int* table = block_tables + (size_t)seq * max_pages;

    // page ids of the key range
    const int page_lo = (kt_begin * PF_BN) >> page_shift;
    const int n_pages = (pos_hi >> page_shift) - page_lo + 1;
    const bool staged = n_pages <= PF_MAX_PAGES;
    int bad = 0;
    if (staged) {
        for (int i = threadIdx.x; i < n_pages; i += 256) {
            int page = table[page_lo + i];
            if (page < 0 || page >= num_pages) {
                if (((page_lo + i + 1) << page_shift) > key_lo) bad = 1;   // pages behind the window may be gone
                page = -1;
            }
            pages_s[i] = page;
        }
    }
    __syncthreads();

    auto swz = [](int row, int chunk) { return row * HD + ((chunk ^ (row & 7)) << 3); };   // element offset

    auto load_kv = [&](int kt, int buf) {
        __nv_bfloat16* kd = Ks + buf * PF_BN * HD;
        __nv_bfloat16* vd = Vs + buf * PF_BN * HD;
        for (int c = tid; c < PF_BN * CPR; c += 128) {
            const int kk = c / CPR, ch = c % CPR;
            const int key = kt * PF_BN + kk;
            long long page = -1;
            if (key <= pos_hi) {
                const int pi = key >> page_shift;
                if (staged) {
                    page = pages_s[pi - page_lo];
                } else {
                    page = table[pi];
                    if (page < 0 || page >= num_pages) {
                        if (((pi + 1) << page_shift) > key_lo) bad = 1;
                        page = -1;
                    }
                }
            }
            const int dst = swz(kk, ch);
            if (page >= 0) {
                const long long off = ((page * nkv + kvh) * page_size + (key & (page_size - 1))) * HD + ch * 8;
                __pipeline_memcpy_async(kd + dst, kcache + off, 16);
                __pipeline_memcpy_async(vd + dst, vcache + off, 16);
            } else {   // nothing to read: zeros, so that masked probabilities never meet garbage
                *reinterpret_cast<uint4*>(kd + dst) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vd + dst) = make_uint4(0, 0, 0, 0);
            }
        }
    };

    // this group's tiles are kt_first, kt_first + 2, ...; the first two are requested at once
    const int kt_first = kt_begin + group;
    if (kt_first <= kt_end) load_kv(kt_first, 0);
    __pipeline_commit();
    if (kt_first + 2 <= kt_end) load_kv(kt_first + 2, 1);
    __pipeline_commit();   // (possibly empty groups: the waits below count groups)
    // Q tile: plain loads by all 256 threads, visible to both groups after the barrier
    for (int c = threadIdx.x; c < PF_BM * CPR; c += 256) {
        const int r = c / CPR, ch = c % CPR;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (q_lo + r < nrows)
            v = *reinterpret_cast<const uint4*>(q + (size_t)(row0 + q_lo + r) * q_stride + (size_t)head * HD + ch * 8);
        *reinterpret_cast<uint4*>(Qs + swz(r, ch)) = v;
    }
    __syncthreads();

    const uint32_t qs_addr = (uint32_t)__cvta_generic_to_shared(Qs);
    const uint32_t ks_addr = (uint32_t)__cvta_generic_to_shared(Ks);
    const uint32_t vs_addr = (uint32_t)__cvta_generic_to_shared(Vs);

    uint32_t qf[KS][4];
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    float m_run[2] = {PF_NEG_BIG, PF_NEG_BIG}, l_run[2] = {0.f, 0.f};
    const float sl2 = scale * 1.4426950408889634f;   // scores are kept raw; exp(x*scale) = exp2(x*sl2)

    // positions of this thread's two rows (g and g+8 of the warp's 16)
    const int rpos[2] = {pos_lo + warp * 16 + g, pos_lo + warp * 16 + g + 8};
    const int warp_pos_hi = pos_lo + warp * 16 + 15;
    const int warp_pos_lo = pos_lo + warp * 16;
    const int warp_key_lo = (window > 0 && warp_pos_lo + 1 > window) ? warp_pos_lo + 1 - window : 0;

    // A fragments of Q: matrices (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
#pragma unroll
    for (int s = 0; s < KS; ++s) {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int ch = 2 * s + (lane >> 4);
        ldmatrix_x4(qf[s], qs_addr + (uint32_t)swz(r, ch) * 2);
    }

    for (int kt = kt_first; kt <= kt_end; kt += 2) {
        const int li = (kt - kt_first) >> 1;   // index among this group's tiles
        const int buf = li % PF_STAGES;
        // the tile two ahead goes into the buffer of the tile before this one; the whole group passed
        // the barrier at the end of that iteration, so it is free
        if (kt + 4 <= kt_end) load_kv(kt + 4, (li + 2) % PF_STAGES);
        __pipeline_commit();
        __pipeline_wait_prior(2);   // all but the two newest groups: tile kt has landed
        group_sync();
        const int key0 = kt * PF_BN;
        // a warp whose rows all lie before this tile, or whose window lies after it, has nothing to do
        if (key0 <= warp_pos_hi && key0 + PF_BN > warp_key_lo) {
            const uint32_t kb = ks_addr + (uint32_t)buf * PF_BN * HD * 2;
            const uint32_t vb = vs_addr + (uint32_t)buf * PF_BN * HD * 2;
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
                for (int jp = 0; jp < 4; ++jp) {   // pairs of key tiles
                    uint32_t b[4];
                    const int r = 16 * jp + (lane & 7) + (lane >> 4) * 8;      // key row
                    const int ch = 2 * ks + ((lane >> 3) & 1);                  // channel chunk
                    ldmatrix_x4(b, kb + (uint32_t)swz(r, ch) * 2);
                    pf_mma(s[2 * jp], qf[ks], b[0], b[1]);
                    pf_mma(s[2 * jp + 1], qf[ks], b[2], b[3]);
                }
            }
            // mask and row maxima
            const bool need_mask = key0 + PF_BN - 1 > warp_pos_lo || (window > 0 && key0 < warp_pos_hi + 1 - window + 0) ||
                                   key0 + PF_BN - 1 > pos_hi;
            float mx[2] = {PF_NEG_BIG, PF_NEG_BIG};
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (need_mask) {
                        const int key = key0 + 8 * j + 2 * t + (e & 1);
                        const int p = rpos[e >> 1];
                        const bool ok = key <= p && (window <= 0 || key > p - window);
                        if (!ok) s[j][e] = PF_NEG_BIG;
                    }
                    mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
                }
            float corr[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m_run[h], mx[h]);
                corr[h] = exp2f((m_run[h] - m_new) * sl2);
                m_run[h] = m_new;
                l_run[h] *= corr[h];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    // a masked score is exactly PF_NEG_BIG; if the row has seen no key yet its maximum is
                    // PF_NEG_BIG too, so test the mask, not the difference
                    const float p = s[j][e] <= PF_NEG_BIG ? 0.f : exp2f((s[j][e] - m_run[e >> 1]) * sl2);
                    s[j][e] = p;
                    l_run[e >> 1] += p;
                }
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                o[j][0] *= corr[0]; o[j][1] *= corr[0];
                o[j][2] *= corr[1]; o[j][3] *= corr[1];
            }
            // O += P V
#pragma unroll
            for (int b16 = 0; b16 < 4; ++b16) {   // 16 keys at a time
                uint32_t a[4];
                a[0] = pf_pack(s[2 * b16][0], s[2 * b16][1]);
                a[1] = pf_pack(s[2 * b16][2], s[2 * b16][3]);
                a[2] = pf_pack(s[2 * b16 + 1][0], s[2 * b16 + 1][1]);
                a[3] = pf_pack(s[2 * b16 + 1][2], s[2 * b16 + 1][3]);
#pragma unroll
                for (int jp = 0; jp < NT / 2; ++jp) {   // pairs of channel tiles
                    uint32_t b[4];
                    const int r = 16 * b16 + (lane & 7) + ((lane >> 3) & 1) * 8;   // key row
                    const int ch = 2 * jp + (lane >> 4);                            // channel chunk
                    ldmatrix_x4_trans(b, vb + (uint32_t)swz(r, ch) * 2);
                    pf_mma(o[2 * jp], a, b[0], b[1]);
                    pf_mma(o[2 * jp + 1], a, b[2], b[3]);
                }
            }
        }
        group_sync();
    }
    if (bad) atomicOr(status, GB_STATUS_BAD_SLOT);

    // merge the two groups: group 1 parks its state in shared memory (the tiles are no longer needed),
    // group 0 combines it with its own
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    __syncthreads();
    float* park = reinterpret_cast<float*>(Qs + PF_BM * HD);   // [128 threads][NT*4 + 4]
    if (group == 1) {
        float* mine = park + tid * (NT * 4 + 4);
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) mine[j * 4 + e] = o[j][e];
        mine[NT * 4] = m_run[0]; mine[NT * 4 + 1] = m_run[1];
        mine[NT * 4 + 2] = l_run[0]; mine[NT * 4 + 3] = l_run[1];
    }
    __syncthreads();
    if (group == 1) return;
    {
        const float* other = park + tid * (NT * 4 + 4);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float m1 = other[NT * 4 + h], l1 = other[NT * 4 + 2 + h];
            const float m = fmaxf(m_run[h], m1);
            const float a0 = exp2f((m_run[h] - m) * sl2), a1 = exp2f((m1 - m) * sl2);
            l_run[h] = l_run[h] * a0 + l1 * a1;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                o[j][2 * h] = o[j][2 * h] * a0 + other[j * 4 + 2 * h] * a1;
                o[j][2 * h + 1] = o[j][2 * h + 1] * a0 + other[j * 4 + 2 * h + 1] * a1;
            }
        }
    }

    // normalise and store
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = q_lo + warp * 16 + g + 8 * h;
        if (r < nrows) {
            const float inv = l_run[h] > 0.f ? 1.0f / l_run[h] : 0.f;
            __nv_bfloat16* dst = out + (size_t)(row0 + r) * out_stride + (size_t)head * HD;
#pragma unroll
            for (int j = 0; j < NT; ++j)
                *reinterpret_cast<uint32_t*>(dst + 8 * j + 2 * t) = pf_pack(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
        }
    }
}

template <int HD>
static int launch_prefill(const void* q, long long q_stride, void* out, long long out_stride, const void* kcache,
                          const void* vcache, const int* block_tables, int max_pages, const int* seq_first_row,
                          const int* seq_start_pos, int num_seqs, int max_rows_per_seq, int nh, int nkv, int page_size,
                          long long num_pages, float scale, int window, int* status, cudaStream_t stream) {
    constexpr int smem = (PF_BM * HD + 2 * 2 * PF_STAGES * PF_BN * HD) * 2;   // Q, and K/V stages of both groups
    auto kernel = attention_prefill_kernel<HD>;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        GB_REQUIRE(e == cudaSuccess, "gb_attention_prefill: %d bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    dim3 grid(gb_ceil_div(max_rows_per_seq, PF_BM), nh, num_seqs);
    kernel<<<grid, 256, smem, stream>>>((const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride,
                                        (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, block_tables,
                                        max_pages, seq_first_row, seq_start_pos, nh, nkv, page_size, page_shift,
                                        num_pages, scale, window, status);
    return gb_check_launch("gb_attention_prefill");
}

GB_EXPORT int gb_attention_prefill_supported(int nh, int nkv, int hd, int page_size) {
    if (nkv <= 0 || nh % nkv) return 0;
    return (hd == 64 || hd == 128) && page_size >= 8 && (page_size & (page_size - 1)) == 0;
}

// Rows of each request are consecutive: request s owns rows seq_first_row[s] .. seq_first_row[s+1]-1,
// at positions seq_start_pos[s] + local index. q and out are bfloat16 with 16-byte aligned rows.
GB_EXPORT int gb_attention_prefill(const void* q, long long q_stride, void* out, long long out_stride,
                                   const void* kcache, const void* vcache, const int* block_tables, int max_pages,
                                   const int* seq_first_row, const int* seq_start_pos, int num_seqs,
                                   int max_rows_per_seq, int nh, int nkv, int hd, int page_size, long long num_pages,
                                   float scale, int window, int* status, cudaStream_t stream) {
    GB_REQUIRE(gb_attention_prefill_supported(nh, nkv, hd, page_size),
               "gb_attention_prefill: head size %d (64 or 128) / page size %d (a power of two) is not built", hd, page_size);
    GB_REQUIRE(q_stride % 8 == 0 && (uintptr_t)q % 16 == 0, "gb_attention_prefill: q rows must be 16-byte aligned");
    GB_REQUIRE(out_stride % 2 == 0 && (uintptr_t)out % 4 == 0, "gb_attention_prefill: out rows must be 4-byte aligned");
    GB_REQUIRE(num_seqs >= 0 && num_seqs <= 65535 && nh <= 65535 && max_pages > 0, "gb_attention_prefill: bad batch shape");
    if (num_seqs == 0 || max_rows_per_seq <= 0) return 0;
    if (hd == 64)
        return launch_prefill<64>(q, q_stride, out, out_stride, kcache, vcache, block_tables, max_pages, seq_first_row,
                                  seq_start_pos, num_seqs, max_rows_per_seq, nh, nkv, page_size, num_pages, scale,
                                  window, status, stream);
    return launch_prefill<128>(q, q_stride, out, out_stride, kcache, vcache, block_tables, max_pages, seq_first_row,
                               seq_start_pos, num_seqs, max_rows_per_seq, nh, nkv, page_size, num_pages, scale, window,
                               status, stream);
}
