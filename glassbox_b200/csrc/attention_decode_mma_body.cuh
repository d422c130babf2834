// The body of the tensor-core decode attention (see attention_decode_mma.cu for the method) as a device function of
// a *virtual* block (split, kv head, row), so that the same code serves the stand-alone kernel, whose blocks are the
// virtual blocks, and the persistent decode-program kernel (decode_program.cu), whose resident blocks walk over them.
#pragma once

#include <cooperative_groups.h>

#include "common.cuh"

struct DecodeAttnArgs {
    const __nv_bfloat16* q;
    long long q_stride;
    __nv_bfloat16* out;
    long long out_stride;
    const __nv_bfloat16* kcache;
    const __nv_bfloat16* vcache;
    const int* block_tables;
    int max_pages;
    const int* row_seq;
    const int* positions;
    int nh, nkv, page_size, page_shift;
    long long num_pages;
    float scale;
    int window, splits;
    float* part_acc;
    float* part_ml;
    int* counters;
    int* status;
    int n;           // rows (used by the persistent kernel to count its virtual blocks)
    int hd, block_keys;
    int late_release;   // let the next kernel in the stream go only after this one's own wait (else at its start)
};

constexpr float MMA_NEG_BIG = -1.0e30f;
constexpr int MMA_MAX_MERGE = 2048;   // weights of (heads x sub-splits) merged per pass
constexpr int MMA_MAX_PAGES = 1024;   // page ids of one block's key range kept in shared memory

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Keys and values are read once: they leave no line behind in L1 (which keeps the small things that are read again:
// page ids, the products' activations). An ordinary load, not a read-only one: in a persistent kernel another block
// of the same launch has written this step's keys and values.
__device__ __forceinline__ uint4 kv_load16(const void* p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

template <int WORDS> struct RowLoad;  // WORDS 32-bit words of a value row, widest loads possible
template <> struct RowLoad<1> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, uint32_t (&w)[1]) {
        w[0] = *reinterpret_cast<const uint32_t*>(p);
    }
};
template <> struct RowLoad<2> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, uint32_t (&w)[2]) {
        uint2 v = *reinterpret_cast<const uint2*>(p);
        w[0] = v.x; w[1] = v.y;
    }
};
template <> struct RowLoad<4> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, uint32_t (&w)[4]) {
        uint4 v = kv_load16(p);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    }
};
template <> struct RowLoad<8> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, uint32_t (&w)[8]) {
        uint4 a = *reinterpret_cast<const uint4*>(p), b = *reinterpret_cast<const uint4*>(p + 8);
        w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
    }
};

// `sync` says how to wait for the work before (GbPdlSync in the stand-alone kernel, a barrier's wait in a persistent
// one). Queries, which another block of the same launch may have written, are read past L1.
// Shared memory of the body, provided by the caller.
struct __align__(16) DecodeAttnSmem {   // (a multiple of 16 bytes, so that arrays of it keep what follows aligned)
    int pages[MMA_MAX_PAGES];
    float weights[MMA_MAX_MERGE];
    int is_last;
};

// NW warps (NW * 32 threads) work on one virtual block: 4, or 8 where few blocks would otherwise leave the chip's
// memory system idle (a small batch): each warp then has half as many blocks of keys to walk through.
// Floats of shared memory that the merge inside a thread-block cluster needs in the cluster's first block: one
// (output row, maximum, sum) per head of the group and per warp of every split.
template <int HD>
__host__ __device__ constexpr int decode_attn_cluster_floats(int group, int splits, int warps) { return group * splits * warps * (HD + 2); }

// CLUSTER: the blocks of one (row, kv head), one per split, are one thread-block cluster (the caller launches them
// so). Their warps then put their partial results straight into the shared memory of the cluster's first block
// (`cluster_part`, decode_attn_cluster_floats<HD>() floats, the same offset in every block), meet at the cluster's
// barrier, and the first block merges from its own shared memory: no trip through global memory, no counter, no
// second pass over what other blocks wrote. Otherwise the partial results go through `part_acc` / `part_ml` and the
// block that arrives last at `counters` merges them.
template <int HD, int BK, class Sync, int NW = 4, bool CLUSTER = false>
__device__ __forceinline__ void attention_decode_mma_body(const DecodeAttnArgs& a, const int split, const int kvh, const int row,
                                                          DecodeAttnSmem& sm, Sync& sync, float* cluster_part = nullptr) {
    constexpr int NTHREADS = NW * 32;
    const __nv_bfloat16* __restrict__ q = a.q;
    const long long q_stride = a.q_stride, out_stride = a.out_stride;
    __nv_bfloat16* __restrict__ out = a.out;
    const __nv_bfloat16* __restrict__ kcache = a.kcache;
    const __nv_bfloat16* __restrict__ vcache = a.vcache;
    const int* __restrict__ block_tables = a.block_tables;
    const int max_pages = a.max_pages;
    const int* __restrict__ row_seq = a.row_seq;
    const int* __restrict__ positions = a.positions;
    const int nh = a.nh, nkv = a.nkv, page_size = a.page_size, page_shift = a.page_shift;
    const long long num_pages = a.num_pages;
    const float scale = a.scale;
    const int window = a.window, splits = a.splits;
    float* __restrict__ part_acc = a.part_acc;
    float* __restrict__ part_ml = a.part_ml;
    int* __restrict__ counters = a.counters;
    int* __restrict__ status = a.status;
    constexpr int KS = HD / 16;   // k16 steps over the channels (scores)
    constexpr int NT = HD / 8;    // n8 tiles over the channels (output)
    constexpr int KT = BK / 8;    // n8 tiles over the keys of a block (scores)
    constexpr int KB = BK / 16;   // k16 steps over the keys of a block (output)
    constexpr int VW = NT / 2;    // 32-bit words of a value row per thread
    const int tid = sync.thread(), lane = tid & 31, warp = tid >> 5;   // NW * 32 threads work on one virtual block
    const int g = lane >> 2, t = lane & 3;
    const int G = nh / nkv;
    const int head0 = kvh * G;
    const int S4 = splits * NW;   // partial results per head: one per warp of every split
    int& is_last = sm.is_last;

    // This kernel's own prologue (positions, block table: step metadata that no kernel writes) runs before it waits
    // for its predecessor, which wrote the queries and this step's keys and values. The next kernel in the stream is
    // let go only after that wait: released earlier, kernels pile up on the SMs, resident and waiting, in the way of
    // the one that works.
    if (!a.late_release) sync.start();
    int pos = positions[row];
    if (pos >= 0 && (pos >> page_shift) >= max_pages) {   // a position the block table does not reach: reported, and the
        if (tid == 0) atomicOr(status, GB_STATUS_BAD_POSITION);   // row is treated as padding (nothing is read)
        pos = -1;
    }
    __nv_bfloat16* orow = out + (size_t)row * out_stride;
    if (pos < 0) {  // padding row
        sync.wait();
        if (a.late_release) sync.start();
        if (sync.gave_up()) return;
        if (split == 0)
            for (int i = tid; i < G * HD; i += NTHREADS) orow[head0 * HD + i] = __float2bfloat16_rn(0.f);
        return;
    }
    if constexpr (CLUSTER)   // every block of the cluster says that it runs (its shared memory exists); waited for before the first store into another block's
        asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    const int* table = block_tables + (size_t)row_seq[row] * max_pages;
    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int first_aligned = first / BK * BK;   // blocks of keys start at multiples of BK; keys before `first` are masked
    const int total = pos + 1 - first_aligned;
    const int chunk = ((total + splits - 1) / splits + BK - 1) / BK * BK;
    const int k_begin = first_aligned + split * chunk;
    const int k_end = min(pos + 1, k_begin + chunk);
    const int nblocks = k_end > k_begin ? (k_end - k_begin + BK - 1) / BK : 0;

    float m_run[2] = {MMA_NEG_BIG, MMA_NEG_BIG}, l_run[2] = {0.f, 0.f};
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

    // Page ids of this block's key range are staged in shared memory once (bad ids are reported and
    // replaced by page 0, whose rows are then masked like any key outside the range), and blocks of
    // keys start at multiples of BK, so a half-block of 16 keys lies in one page (pages hold a power
    // of two >= 16 keys) and its addresses are a few integer operations. Loads never branch. They
    // run one block of keys ahead of the arithmetic (two register sets), so that a warp always has
    // loads in flight.
    int* pages_s = sm.pages;
    const int page_mask = page_size - 1;
    const int page_lo = k_begin >> page_shift;
    const int n_pages = nblocks > 0 ? ((k_end - 1) >> page_shift) - page_lo + 1 : 0;
    const bool staged = n_pages <= MMA_MAX_PAGES;
    int bad = 0;
    if (staged) {
        for (int i = tid; i < n_pages; i += NTHREADS) {
            int page = table[page_lo + i];
            if (page < 0 || page >= num_pages) {
                // a page wholly before the first visible key may have been given back (window): its
                // keys are masked; any other missing page is an error
                if (((page_lo + i + 1) << page_shift) > first) bad = 1;
                page = 0;
            }
            pages_s[i] = page;
        }
        sync.group_barrier();
    }
    sync.wait();   // the writes of the work before (q, this step's K/V) are visible from here
    if (a.late_release) sync.start();
    if (sync.gave_up()) return;
    // Q as the A operand: rows g and g+8 are query heads head0+g and head0+g+8 (zero beyond G).
    uint32_t qf[KS][4];
    {
        const __nv_bfloat16* q0 = q + (size_t)row * q_stride + (size_t)(head0 + g) * HD;
        const __nv_bfloat16* q1 = q0 + 8 * HD;
#pragma unroll
        for (int s = 0; s < KS; ++s) {
            uint2 a = make_uint2(0, 0), b = make_uint2(0, 0);   // (shadow the argument block inside this scope)
            // the four channels that stand for this thread's k indices of step s: any assignment works as long as the
            // keys use the same one; with an even number of steps a thread's channels of two steps are 8 in a row, so
            // that a key's share is one 16-byte load
            const int ch = KS % 2 == 0 ? 32 * (s >> 1) + 8 * t + 4 * (s & 1) : 16 * s + 4 * t;
            if (g < G) a = __ldcg(reinterpret_cast<const uint2*>(q0 + ch));
            if (g + 8 < G) b = __ldcg(reinterpret_cast<const uint2*>(q1 + ch));
            qf[s][0] = a.x; qf[s][1] = b.x; qf[s][2] = a.y; qf[s][3] = b.y;
        }
    }

    // row index (in units of cache rows) of the first key of the 16-key half-block starting at `key`
    auto half_block_row = [&](int key) -> int {
        const int pi = min(key >> page_shift, page_lo + n_pages - 1);
        int page;
        if (staged) {
            page = pages_s[pi - page_lo];
        } else {
            page = table[pi];
            if (page < 0 || page >= num_pages) {
                if (((pi + 1) << page_shift) > first) bad = 1;
                page = 0;
            }
        }
        return (page * nkv + kvh) * page_size + (key & page_mask);
    };

    struct Block {
        uint2 kf[KT][KS];
        uint32_t vf[KB][4][VW];
    };
    auto load_block = [&](int blk, Block& B) {
        const int base = k_begin + blk * BK;
        int hb[KB];
#pragma unroll
        for (int b = 0; b < KB; ++b) hb[b] = half_block_row(base + 16 * b);
#pragma unroll
        for (int j = 0; j < KT; ++j) {
            if constexpr (KS % 2 == 0) {
                const __nv_bfloat16* kp = kcache + (long long)(hb[j >> 1] + 8 * (j & 1) + g) * HD + 8 * t;
#pragma unroll
                for (int s2 = 0; s2 < KS / 2; ++s2) {
                    const uint4 v = kv_load16(kp + 32 * s2);
                    B.kf[j][2 * s2] = make_uint2(v.x, v.y);
                    B.kf[j][2 * s2 + 1] = make_uint2(v.z, v.w);
                }
            } else {
                const __nv_bfloat16* kp = kcache + (long long)(hb[j >> 1] + 8 * (j & 1) + g) * HD + 4 * t;
#pragma unroll
                for (int s = 0; s < KS; ++s) B.kf[j][s] = *reinterpret_cast<const uint2*>(kp + 16 * s);
            }
        }
#pragma unroll
        for (int b = 0; b < KB; ++b)
#pragma unroll
            for (int r = 0; r < 4; ++r)
                RowLoad<VW>::load(vcache + (long long)(hb[b] + 2 * t + (r & 1) + (r >> 1) * 8) * HD + NT * g, B.vf[b][r]);
    };
    auto compute_block = [&](int blk, Block& B) {
        const int base = k_begin + blk * BK;
        // ---- scores
        float s[KT][4];
#pragma unroll
        for (int j = 0; j < KT; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
                mma16816(s[j], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], B.kf[j][ks].x, B.kf[j][ks].y);
        }
        float mx[2] = {MMA_NEG_BIG, MMA_NEG_BIG};
#pragma unroll
        for (int j = 0; j < KT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = base + 8 * j + 2 * t + (e & 1);
                s[j][e] = (key < k_end && key >= first) ? s[j][e] * scale : MMA_NEG_BIG;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
            }
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            corr[h] = __expf(m_run[h] - m_new);
            m_run[h] = m_new;
            l_run[h] *= corr[h];
        }
#pragma unroll
        for (int j = 0; j < KT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = base + 8 * j + 2 * t + (e & 1);
                const float p = (key < k_end && key >= first) ? __expf(s[j][e] - m_run[e >> 1]) : 0.f;
                s[j][e] = p;
                l_run[e >> 1] += p;   // this thread's share; summed over the lane group at the end
            }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            acc[j][0] *= corr[0]; acc[j][1] *= corr[0];
            acc[j][2] *= corr[1]; acc[j][3] *= corr[1];
        }
        // ---- output: P (registers) times V
#pragma unroll
        for (int b = 0; b < KB; ++b) {
            const uint32_t a0 = pack_bf16(s[2 * b][0], s[2 * b][1]), a1 = pack_bf16(s[2 * b][2], s[2 * b][3]);
            const uint32_t a2 = pack_bf16(s[2 * b + 1][0], s[2 * b + 1][1]), a3 = pack_bf16(s[2 * b + 1][2], s[2 * b + 1][3]);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;   // high or low halves of the two rows' words
                const uint32_t b0 = __byte_perm(B.vf[b][0][j >> 1], B.vf[b][1][j >> 1], sel);
                const uint32_t b1 = __byte_perm(B.vf[b][2][j >> 1], B.vf[b][3][j >> 1], sel);
                mma16816(acc[j], a0, a1, a2, a3, b0, b1);
            }
        }
    };

    Block A, B;
    if (warp < nblocks) load_block(warp, A);
    for (int blk = warp; blk < nblocks; blk += 2 * NW) {
        if (blk + NW < nblocks) load_block(blk + NW, B);
        compute_block(blk, A);
        if (blk + 2 * NW < nblocks) load_block(blk + 2 * NW, A);
        if (blk + NW < nblocks) compute_block(blk + NW, B);
    }

    if (bad) atomicOr(status, GB_STATUS_BAD_SLOT);
    // ---- this warp's partial result
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    const int sub = split * NW + warp;
    float* weights = sm.weights;
    if constexpr (CLUSTER) {
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        // [head of the group][sub-split][HD channels, maximum, sum] in the first block's shared memory
        float* first = cluster.map_shared_rank(cluster_part, 0);
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int hi = g + 8 * h;
            if (hi < G) {
                float* pa = first + ((size_t)hi * S4 + sub) * (HD + 2);
                if (t == 0) {
                    pa[HD] = m_run[h];
                    pa[HD + 1] = l_run[h];
                }
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    pa[NT * (2 * t) + j] = acc[j][2 * h];
                    pa[NT * (2 * t + 1) + j] = acc[j][2 * h + 1];
                }
            }
        }
        cluster.sync();                       // (release / acquire: the first block sees what the others stored)
        if (cluster.block_rank() != 0) return;
        // one warp per head turns the (maximum, sum) pairs into normalised weights; then every thread adds up its channel
        for (int hi = warp; hi < G; hi += NW) {
            const float* ph = cluster_part + (size_t)hi * S4 * (HD + 2);
            float m = MMA_NEG_BIG;
            for (int sidx = lane; sidx < S4; sidx += 32) m = fmaxf(m, ph[sidx * (HD + 2) + HD]);
            m = gb_warp_max(m);
            float l = 0.f;
            for (int sidx = lane; sidx < S4; sidx += 32) {
                const float w = __expf(ph[sidx * (HD + 2) + HD] - m);
                weights[hi * S4 + sidx] = w;
                l = fmaf(ph[sidx * (HD + 2) + HD + 1], w, l);
            }
            l = gb_warp_sum(l);
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            __syncwarp();
            for (int sidx = lane; sidx < S4; sidx += 32) weights[hi * S4 + sidx] *= inv;
        }
        sync.group_barrier();
        for (int i = tid; i < G * HD; i += NTHREADS) {
            const int hi = i / HD, d = i % HD;
            const float* pa = cluster_part + (size_t)hi * S4 * (HD + 2) + d;
            const float* w = weights + hi * S4;
            float v = 0.f;
#pragma unroll 8
            for (int sidx = 0; sidx < S4; ++sidx) v = fmaf(pa[(size_t)sidx * (HD + 2)], w[sidx], v);
            orow[(head0 + hi) * HD + d] = __float2bfloat16_rn(v);
        }
        return;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int hi = g + 8 * h;
        if (hi < G) {
            const size_t slot = ((size_t)row * nh + head0 + hi) * S4 + sub;
            if (t == 0) {
                part_ml[slot * 2] = m_run[h];
                part_ml[slot * 2 + 1] = l_run[h];
            }
            float* pa = part_acc + slot * HD;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                pa[NT * (2 * t) + j] = acc[j][2 * h];
                pa[NT * (2 * t + 1) + j] = acc[j][2 * h + 1];
            }
        }
    }
    // ---- the block that arrives last merges every warp of every split
    __threadfence();
    sync.group_barrier();
    if (tid == 0) {
        int* counter = counters + (size_t)row * nkv + kvh;
        const int prev = atomicAdd(counter, 1);
        is_last = (prev == splits - 1);
        if (is_last) *counter = 0;
    }
    sync.group_barrier();
    if (!is_last) return;
    __threadfence();
    // Merge: one warp per head turns the (maximum, sum) pairs of all sub-splits into normalised
    // weights in shared memory; then every thread adds up its channel over the sub-splits with
    // independent loads.
    if (G * HD <= NTHREADS && S4 <= 64) {
        // The usual case (every output channel of the group has a thread of its own, at most 64 partial results per
        // head): a thread asks for its channel of every partial result at once, before the weights exist, and a lane
        // reads its (maximum, sum) pairs once; the merge is then two trips to L2 that overlap instead of four in a row.
        constexpr int MAXP = 64;
        const int hi_o = tid / HD, d_o = tid % HD;
        float pv[MAXP];
        if (tid < G * HD) {
            const float* pa = part_acc + ((size_t)row * nh + head0 + hi_o) * S4 * HD + d_o;
#pragma unroll
            for (int sidx = 0; sidx < MAXP; ++sidx) pv[sidx] = sidx < S4 ? __ldcg(pa + (size_t)sidx * HD) : 0.f;
        }
        for (int hi = warp; hi < G; hi += NW) {
            const float2* ml = reinterpret_cast<const float2*>(part_ml + ((size_t)row * nh + head0 + hi) * S4 * 2);
            const float2 p0 = lane < S4 ? __ldcg(ml + lane) : make_float2(MMA_NEG_BIG, 0.f);
            const float2 p1 = lane + 32 < S4 ? __ldcg(ml + lane + 32) : make_float2(MMA_NEG_BIG, 0.f);
            const float m = gb_warp_max(fmaxf(p0.x, p1.x));
            const float w0 = __expf(p0.x - m), w1 = __expf(p1.x - m);
            const float l = gb_warp_sum(fmaf(p0.y, w0, p1.y * w1));
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            if (lane < S4) weights[hi * S4 + lane] = w0 * inv;
            if (lane + 32 < S4) weights[hi * S4 + lane + 32] = w1 * inv;
        }
        sync.group_barrier();
        if (tid < G * HD) {
            const float* w = weights + hi_o * S4;
            float v = 0.f;
#pragma unroll
            for (int sidx = 0; sidx < MAXP; ++sidx)
                if (sidx < S4) v = fmaf(pv[sidx], w[sidx], v);
            orow[(head0 + hi_o) * HD + d_o] = __float2bfloat16_rn(v);
        }
        return;
    }
    const int per_pass = MMA_MAX_MERGE / S4;                 // heads whose weights fit at once
    for (int h0 = 0; h0 < G; h0 += per_pass) {
        const int hcount = min(per_pass, G - h0);
        for (int hi = warp; hi < hcount; hi += NW) {
            const float* ml = part_ml + ((size_t)row * nh + head0 + h0 + hi) * S4 * 2;
            float m = MMA_NEG_BIG;
            for (int sidx = lane; sidx < S4; sidx += 32) m = fmaxf(m, __ldcg(ml + 2 * sidx));
            m = gb_warp_max(m);
            float l = 0.f;
            for (int sidx = lane; sidx < S4; sidx += 32) {
                const float w = __expf(__ldcg(ml + 2 * sidx) - m);
                weights[hi * S4 + sidx] = w;
                l = fmaf(__ldcg(ml + 2 * sidx + 1), w, l);
            }
            l = gb_warp_sum(l);
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            __syncwarp();
            for (int sidx = lane; sidx < S4; sidx += 32) weights[hi * S4 + sidx] *= inv;
        }
        sync.group_barrier();
        for (int i = tid; i < hcount * HD; i += NTHREADS) {
            const int hi = i / HD, d = i % HD;
            const float* pa = part_acc + ((size_t)row * nh + head0 + h0 + hi) * S4 * HD + d;
            const float* w = weights + hi * S4;
            float v = 0.f;
#pragma unroll 8
            for (int sidx = 0; sidx < S4; ++sidx) v = fmaf(__ldcg(pa + (size_t)sidx * HD), w[sidx], v);
            orow[(head0 + h0 + hi) * HD + d] = __float2bfloat16_rn(v);
        }
        sync.group_barrier();
    }
}

