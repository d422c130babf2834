// Causal grouped-query flash attention for prompt portions on the 5th-generation tensor cores
// (sm_100a): both products of the scheme, S = Q K^T and O += P V, are tcgen05.mma instructions with
// their accumulators in tensor memory; queries, keys and values come into shared memory by TMA, the
// keys and values page by page straight from the paged cache through the request's block table.
//
// One block = 128 consecutive query rows of one request for one query head, over tiles of 128 keys:
//   warp 0, 10  producers of keys (and the query tile, once) and of values. For every key tile the lanes
//               read the page ids from the block table (one tile ahead) and each issues the TMA load of
//               one page (a page is `page_size` rows of one kv head: one box of the 2-D view
//               [pages * kv_heads * page_size, head_dim] of a cache layer) into a ring of four stages;
//               keys and values have rings of their own, since a key stage is free again much earlier.
//   warp 1      lane 0 issues the tensor-core work, whichever is ready. S_j = Q K_j^T (M 128, N 128, K
//               head_dim; both operands K-major in 128-byte-swizzled rows) goes to one of two TMEM
//               buffers, up to two tiles ahead of the softmax warps. When P_j is in tensor memory,
//               O_g += P_j V_j (M 128, N head_dim, K 128; V is the MN-major operand: its rows are keys)
//               accumulates in one of two further TMEM regions, g = j & 1.
//   warps 2-9   softmax, in two groups of four warps; group g takes the key tiles of parity g with an
//               accumulator, running maximum and row sum of its own, and the two partial results are merged
//               at the end, so one group's exponentials overlap the other's waits. Within a group a thread
//               owns one query row (a row is one TMEM lane, so no shuffles): it reads its 128 scores with
//               one tcgen05.ld, takes the maximum, and writes P_j = exp2((S_j - m) c) rounded to bfloat16
//               back into tensor memory (tcgen05.st), from where the tensor core takes it as the A operand
//               of the second product: P never passes through shared memory, whose bandwidth the operand
//               reads of the two products and the TMA writes already share. The running maximum m is
//               only raised, and O_g and the row sum rescaled (tcgen05.ld / st of the O rows by the whole
//               warp), when a new maximum exceeds it by more than 2^8 in the exponent: until then P stays
//               below 256, which bfloat16 and the float32 sums hold without loss, and the final O / l is
//               the same.
// A query at position p sees keys max(0, p-window+1) .. p (crates/glassbox-core/src/model.rs:278-317);
// the mask is applied only in tiles that cross a boundary, and key tiles no row can see are skipped.
// Pages that are missing (beyond what is reserved, or given back behind a window) can only hold
// masked keys; page 0 is read in their place, so that P = 0 never meets anything but finite numbers
// (the cache is zero-initialised and only ever holds finite values).
//
// Every wait is bounded: a wait that exceeds its limit sets GB_STATUS_WAIT_TIMEOUT in the status
// word and the block winds down (waits, again bounded, for its own TMA copies, frees its TMEM,
// returns) instead of hanging the GPU. TMA loads use no multicast.
#include "tcgen05.cuh"

constexpr int AT_BM = 128, AT_BN = 128;
constexpr float AT_NEG_BIG = -1.0e30f;

constexpr int AT_STAGES = 4;   // key tiles, and value tiles, in flight
constexpr int AT_WARPS = 11;   // key producer, MMA issuer, eight softmax warps, value producer

struct __align__(8) AtShared {
    uint64_t q_full;                 // TMA -> MMA: the query tile has landed
    uint64_t k_full[AT_STAGES];      // TMA -> MMA: a stage's keys have landed
    uint64_t k_empty[AT_STAGES];     // MMA -> TMA: S = Q K^T has read the stage
    uint64_t v_full[AT_STAGES];      // TMA -> MMA: a stage's values have landed
    uint64_t v_empty[AT_STAGES];     // MMA -> TMA: O += P V has read the stage
    uint64_t s_full[2];              // MMA -> softmax: S_j is complete in buffer j & 1
    uint64_t s_free[2];              // softmax -> MMA: S_j has been read out of buffer j & 1
    uint64_t p_ready[2];             // softmax -> MMA: P_j is in TMEM buffer j & 1 (and O is rescaled)
    uint64_t pv_done[2];             // MMA -> softmax: O += P_j V_j is complete (P buffer j & 1 is free, O is current)
    uint64_t x_ready;                // softmax <-> softmax: both groups have posted their final maximum and sum
    float row_stat[2][2][AT_BM];     // [group][maximum, sum][row]
    uint32_t tmem_base;
    int abort_flag;
    int issued[2];                   // key / value tiles whose TMA loads were issued
    int consumed[2];                 // key / value tiles whose full barrier the MMA thread has passed
    int q_issued, q_consumed;
};

template <int HD> struct AtGeometry {
    static constexpr int Q_BYTES = AT_BM * HD * 2, KV_BYTES = AT_BN * HD * 2;
    static constexpr int K_OFF = Q_BYTES, V_OFF = K_OFF + AT_STAGES * KV_BYTES;
    static constexpr int SH_OFF = V_OFF + AT_STAGES * KV_BYTES;
    static constexpr int SMEM = SH_OFF + 2560;
    // tensor memory: two S buffers of 128 columns, two accumulators O_g of HD columns, two P buffers of 64
    // columns (128 bfloat16 keys, two per 32-bit column)
    static constexpr int O_COL = 2 * AT_BN, P_COL = O_COL + 2 * HD;
    static constexpr int TMEM_COLS = 512;
    static_assert(P_COL + 2 * (AT_BN / 2) <= TMEM_COLS, "tensor memory layout");
};

// MN-major B operand (V: rows are keys, the head's channels contiguous) in 128-byte-swizzled rows:
// groups of eight keys are 1024 bytes apart (stride byte offset); the leading byte offset is the distance
// between 64-channel column blocks (one block for head size 64).
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Two non-negative floats to a bfloat16 pair, rounding half up, with integer instructions only: the
// conversion instruction shares its pipe with ex2, which is what bounds this kernel. (Half up differs
// from half to even only on exact ties, one value in 65536.)
__device__ __forceinline__ uint32_t at_pack(float lo, float hi) {
    const uint32_t a = __float_as_uint(lo) + 0x8000u, b = __float_as_uint(hi) + 0x8000u;
    return __byte_perm(a, b, 0x7632);
}

__device__ __forceinline__ float at_max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ float at_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int HD>
__global__ void __launch_bounds__(AT_WARPS * 32) attention_prefill_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, long long out_stride,
    const int* __restrict__ block_tables, int max_pages, const int* __restrict__ seq_first_row,
    const int* __restrict__ seq_start_pos, int nh, int nkv, int page_size, int page_shift, long long num_pages,
    float scale, int window, int* __restrict__ status) {
    using G = AtGeometry<HD>;
    static_assert(HD == 64, "this kernel is built for head size 64");
    extern __shared__ __align__(1024) unsigned char at_smem[];
    unsigned char* Qs = at_smem;
    unsigned char* Ks = at_smem + G::K_OFF;
    unsigned char* Vs = at_smem + G::V_OFF;
    AtShared& sh = *reinterpret_cast<AtShared*>(at_smem + G::SH_OFF);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int qt = gridDim.x - 1 - blockIdx.x;   // later tiles see more keys: start the longest blocks first
    const int head = blockIdx.y, seq = blockIdx.z;
    const int row0 = seq_first_row[seq];
    const int nrows = seq_first_row[seq + 1] - row0;
    if (qt * AT_BM >= nrows) return;              // uniform for the block, before anything is allocated
    if (smem_u32(at_smem) & 1023u) {              // swizzled tiles want 1024-byte alignment: refuse rather than compute nonsense
        if (tid == 0) atomicOr(status, GB_STATUS_WAIT_TIMEOUT);
        return;
    }
    const int start_pos = seq_start_pos[seq];
    if (start_pos < 0) {                          // a padding sequence of a fixed-shape batch (uniform for the block):
        for (int i = tid; i < nrows * (HD / 8); i += blockDim.x)   // its rows read as zeros downstream
            *reinterpret_cast<uint4*>(out + (size_t)(row0 + i / (HD / 8)) * out_stride + (size_t)head * HD + (i % (HD / 8)) * 8) =
                make_uint4(0, 0, 0, 0);
        return;
    }
    const int kvh = head / (nh / nkv);
    const int q_lo = qt * AT_BM;
    const int pos_lo = start_pos + q_lo, pos_hi = start_pos + min(nrows, q_lo + AT_BM) - 1;
    const int key_lo = (window > 0 && pos_lo + 1 > window) ? pos_lo + 1 - window : 0;
    const int kt_begin = key_lo / AT_BN, kt_end = pos_hi / AT_BN;   // inclusive
    const int ntiles = kt_end - kt_begin + 1;
    const int* table = block_tables + (size_t)seq * max_pages;

    if (tid == 0) {
        mbar_init(&sh.q_full, 1);
        for (int b = 0; b < AT_STAGES; ++b) {
            mbar_init(&sh.k_full[b], 1);
            mbar_init(&sh.k_empty[b], 1);
            mbar_init(&sh.v_full[b], 1);
            mbar_init(&sh.v_empty[b], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sh.s_full[b], 1);
            mbar_init(&sh.s_free[b], 4);    // one arrival per warp of the group
            mbar_init(&sh.p_ready[b], 4);
            mbar_init(&sh.pv_done[b], 1);
        }
        mbar_init(&sh.x_ready, 8);
        sh.abort_flag = 0;
        sh.issued[0] = sh.issued[1] = sh.consumed[0] = sh.consumed[1] = sh.q_issued = sh.q_consumed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_base)), "r"(G::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    volatile int* abort_flag = &sh.abort_flag;
    // the set-up above overlapped the tail of the kernel before; from here on its results are read
    gb_pdl_launch_dependents();
    gb_pdl_wait();

    if (warp == 0 || warp == AT_WARPS - 1) {
        // ------------------------------------------------------------------------- producers
        // warp 0 loads the query tile and the keys, the last warp the values: keys are needed (and their
        // stages free again) earlier than values, so the two rings run at their own pace
        const int what = warp == 0 ? 0 : 1;
        if (what == 0 && lane == 0) {
            mbar_expect_tx(&sh.q_full, G::Q_BYTES);
            tma_load_2d(Qs, &map_q, &sh.q_full, head * HD, row0 + q_lo);
            sh.q_issued = 1;
        }
        const int ppt = AT_BN >> page_shift;   // pages per key tile (1 .. 16)
        int bad = 0;
        auto page_of = [&](int kt) -> long long {   // this lane's page of key tile kt
            long long page = 0;
            if (lane < ppt) {
                const int pi = ((kt * AT_BN) >> page_shift) + lane;
                page = pi < max_pages ? table[pi] : -1;
                if (page < 0 || page >= num_pages) {
                    // only a page that holds a key some row can see is missed
                    const int first = pi << page_shift, last = first + page_size - 1;
                    if (first <= pos_hi && last >= key_lo) bad = 1;
                    page = 0;
                }
            }
            return page;
        };
        uint64_t* full = what == 0 ? sh.k_full : sh.v_full;
        uint64_t* empty = what == 0 ? sh.k_empty : sh.v_empty;
        unsigned char* ring = what == 0 ? Ks : Vs;
        const CUtensorMap* map = what == 0 ? &map_k : &map_v;
        long long page = page_of(kt_begin);
        for (int j = 0; j < ntiles; ++j) {
            const int s = j % AT_STAGES;
            const long long next_page = j + 1 < ntiles ? page_of(kt_begin + j + 1) : 0;   // in flight during the wait
            int ok = 1;
            if (lane == 0 && j >= AT_STAGES)
                ok = mbar_wait(&empty[s], ((j / AT_STAGES) - 1) & 1, abort_flag, status) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane == 0) mbar_expect_tx(&full[s], G::KV_BYTES);
            __syncwarp();
            if (lane < ppt) {
                const int row = (int)((page * nkv + kvh) * page_size);
                tma_load_2d(ring + s * G::KV_BYTES + lane * page_size * HD * 2, map, &full[s], 0, row);
            }
            __syncwarp();
            if (lane == 0) sh.issued[what] = j + 1;
            page = next_page;
        }
        if (bad && what == 0) atomicOr(status, GB_STATUS_BAD_SLOT);
    } else if (warp == 1) {
        // ------------------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc_qk = umma_idesc(AT_BM, AT_BN);
            const uint32_t idesc_pv = umma_idesc(AT_BM, HD) | (1u << 16);   // B is MN-major
            const uint32_t q_addr = smem_u32(Qs), k_addr = smem_u32(Ks), v_addr = smem_u32(Vs);
            bool ok = mbar_wait(&sh.q_full, 0, abort_flag, status);
            if (ok) sh.q_consumed = 1;
            // Whatever is ready is issued: S_j as soon as its keys have landed and its group has read S_{j-2} out of
            // the buffer (so S runs up to two tiles ahead and neither softmax group waits for the other), O += P_j V_j
            // as soon as P_j is written and its values have landed. The loop polls without blocking; the limit
            // counts from the last instruction issued.
            int next_qk = 0, next_pv = 0;
            long long t_last = clock64();
            while (ok && next_pv < ntiles) {
                bool progressed = false;
                if (next_qk < ntiles) {
                    const int j = next_qk, st = j % AT_STAGES;
                    if (mbar_test(&sh.k_full[st], (j / AT_STAGES) & 1) &&
                        (j < 2 || mbar_test(&sh.s_free[j & 1], ((j >> 1) - 1) & 1))) {
                        sh.consumed[0] = j + 1;
                        tc_fence_after();
                        const uint32_t kb = k_addr + (uint32_t)(st * G::KV_BYTES);
#pragma unroll
                        for (int k = 0; k < HD / 16; ++k)
                            umma_bf16(tmem + (uint32_t)((j & 1) * AT_BN), umma_desc(q_addr + k * 32), umma_desc(kb + k * 32),
                                      idesc_qk, k ? 1u : 0u);
                        umma_commit(&sh.s_full[j & 1]);
                        umma_commit(&sh.k_empty[st]);
                        ++next_qk;
                        progressed = true;
                    }
                }
                if (next_pv < next_qk) {
                    const int j = next_pv, st = j % AT_STAGES;
                    if (mbar_test(&sh.p_ready[j & 1], (j >> 1) & 1) && mbar_test(&sh.v_full[st], (j / AT_STAGES) & 1)) {
                        sh.consumed[1] = j + 1;
                        tc_fence_after();
                        const uint32_t vb = v_addr + (uint32_t)(st * G::KV_BYTES);
                        const uint32_t pt = tmem + (uint32_t)(G::P_COL + (j & 1) * (AT_BN / 2));
#pragma unroll
                        for (int kk = 0; kk < AT_BN / 16; ++kk)   // 16 keys per instruction: 8 columns of P
                            umma_bf16_ts(tmem + (uint32_t)(G::O_COL + (j & 1) * HD), pt + (uint32_t)(kk * 8),
                                         umma_desc_mn(vb + kk * 16 * 128, AT_BN * 128), idesc_pv, (j >= 2 || kk) ? 1u : 0u);
                        umma_commit(&sh.pv_done[j & 1]);
                        umma_commit(&sh.v_empty[st]);
                        ++next_pv;
                        progressed = true;
                    }
                }
                if (progressed) {
                    t_last = clock64();
                } else if (*abort_flag) {
                    ok = false;
                } else if (clock64() - t_last > TC_WAIT_CYCLES) {
                    *abort_flag = 1;
                    atomicOr(status, GB_STATUS_WAIT_TIMEOUT);
                    ok = false;
                }
            }
        }
    } else {
        // ------------------------------------------------------------------------- softmax
        // Two groups of four warps. Group g takes the key tiles j = g, g + 2, ...: it reads S_j from TMEM buffer
        // g, writes P_j into shared-memory buffer g and owns the accumulator O_g with its own running maximum
        // and row sum, so the groups never wait for each other: while one is busy with exponentials, the other
        // waits for its scores or its accumulator. The two partial results are merged at the end. Warp w reads
        // the TMEM lanes of quarter w % 4 (a hardware rule): each quarter of the rows has one warp per group.
        const int q = warp & 3;                        // the quarter of TMEM lanes this warp may read
        const int g = (warp - 2) >> 2;                 // the group: parity of its key tiles
        const int r = q * 32 + lane;                   // this thread's query row within the tile
        const int pos = pos_lo + r;
        const float sl2 = scale * 1.4426950408889634f; // exp(x * scale) = exp2(x * sl2)
        const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16);
        const uint32_t o_col = (uint32_t)(G::O_COL + g * HD);
        const int my_tiles = (ntiles - g + 1) >> 1;
        float m_run = AT_NEG_BIG, l_run = 0.f;
        bool ok = true;
        auto visible = [&](int key) { return key <= pos && (window <= 0 || key > pos - window); };
        for (int i = 0; i < my_tiles; ++i) {
            const int key0 = (kt_begin + 2 * i + g) * AT_BN;
            if (!mbar_wait_warp(&sh.s_full[g], i & 1, abort_flag, status)) { ok = false; break; }
            tc_fence_after();
            uint32_t sv[AT_BN];
            tmem_load128(lane_base + (uint32_t)(g * AT_BN), sv);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.s_free[g]);   // the buffer may take the group's next S
            // the mask matters only where the tile crosses the diagonal, the window's edge or the last key
            const bool need_mask = key0 + AT_BN - 1 > pos_lo || (window > 0 && key0 < pos_lo + AT_BM - window);
            if (need_mask) {
#pragma unroll
                for (int k = 0; k < AT_BN; ++k)
                    if (!visible(key0 + k)) sv[k] = __float_as_uint(AT_NEG_BIG);
            }
            // four independent chains of three-input maxima, to keep dependent latencies short
            float mx4[4] = {AT_NEG_BIG, AT_NEG_BIG, AT_NEG_BIG, AT_NEG_BIG};
#pragma unroll
            for (int k = 0; k < AT_BN; k += 8) {
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    mx4[u] = at_max3(mx4[u], __uint_as_float(sv[k + 2 * u]), __uint_as_float(sv[k + 2 * u + 1]));
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // O_g += P V of the group's previous tile must be complete before P is overwritten or O_g rescaled
            if (i > 0 && !mbar_wait_warp(&sh.pv_done[g], (i - 1) & 1, abort_flag, status)) { ok = false; break; }
            // raise the running maximum only when it is exceeded by more than 2^8 in the exponent
            const bool raise = (mx - m_run) * sl2 > 8.0f;
            if (i == 0) {
                if (raise) m_run = mx;               // nothing is accumulated yet
            } else if (__any_sync(0xffffffffu, raise)) {
                tc_fence_after();
                const float corr = raise ? at_exp2((m_run - mx) * sl2) : 1.0f;
                if (raise) m_run = mx;
                l_run *= corr;
#pragma unroll
                for (int c = 0; c < HD; c += 32) {
                    uint32_t ov[32];
                    tmem_load32(lane_base + o_col + (uint32_t)c, ov);
#pragma unroll
                    for (int k = 0; k < 32; ++k) ov[k] = __float_as_uint(__uint_as_float(ov[k]) * corr);
                    tmem_store32(lane_base + o_col + (uint32_t)c, ov);
                }
            }
            // P = exp2(S * sl2 - m * sl2), two keys at a time with the packed float32 instructions. A masked key holds
            // -1e30 and comes out as exactly 0; a row that has seen no key yet (its maximum is still -1e30) must not
            // cancel that, so its offset is 0.
            const float msl = m_run <= AT_NEG_BIG ? 0.f : m_run * sl2;
            const float2 scale2 = make_float2(sl2, sl2), off2 = make_float2(-msl, -msl);
            float2 l2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
            uint32_t pw[AT_BN / 2];   // P_j of this row: two keys per 32-bit column of the A operand in TMEM
#pragma unroll
            for (int c = 0; c < AT_BN; c += 2) {
                const float2 y = __ffma2_rn(make_float2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), scale2, off2);
                const float2 p = make_float2(at_exp2(y.x), at_exp2(y.y));
                l2[(c >> 1) & 3] = __fadd2_rn(l2[(c >> 1) & 3], p);
                pw[c >> 1] = at_pack(p.x, p.y);
            }
            const float2 lsum = __fadd2_rn(__fadd2_rn(l2[0], l2[1]), __fadd2_rn(l2[2], l2[3]));
            l_run += lsum.x + lsum.y;
            tmem_store64(lane_base + (uint32_t)(G::P_COL + g * (AT_BN / 2)), pw);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.p_ready[g]);
        }
        // merge: the groups post their maximum and sum per row, then each writes half of the channels
        if (ok) {
            sh.row_stat[g][0][r] = m_run;
            sh.row_stat[g][1][r] = l_run;
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.x_ready);
            ok = mbar_wait_warp(&sh.x_ready, 0, abort_flag, status);
        }
        const int tiles_of[2] = {(ntiles + 1) >> 1, ntiles >> 1};
        for (int gg = 0; gg < 2 && ok; ++gg)   // both accumulators must be final
            if (tiles_of[gg] > 0) ok = mbar_wait_warp(&sh.pv_done[gg], (tiles_of[gg] - 1) & 1, abort_flag, status);
        if (ok) {
            tc_fence_after();
            const float m0 = sh.row_stat[0][0][r], l0 = sh.row_stat[0][1][r];
            const float m1 = sh.row_stat[1][0][r], l1 = sh.row_stat[1][1][r];
            const float m = fmaxf(m0, m1);
            // a group without tiles has never written its accumulator: it is not read
            const float a0 = tiles_of[0] > 0 ? at_exp2((m0 - m) * sl2) : 0.f;
            const float a1 = tiles_of[1] > 0 ? at_exp2((m1 - m) * sl2) : 0.f;
            const float l = l0 * a0 + l1 * a1;
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            constexpr int OC = HD / 2;                 // this thread's channels: g * OC ..
            static_assert(OC == 32, "one 32-column access per accumulator");
            float o[OC];
            {
                uint32_t ov[32];
                tmem_load32(lane_base + (uint32_t)(G::O_COL + g * OC), ov);
#pragma unroll
                for (int k = 0; k < OC; ++k) o[k] = __uint_as_float(ov[k]) * a0;
            }
            if (tiles_of[1] > 0) {                      // uniform for the block
                uint32_t ov[32];
                tmem_load32(lane_base + (uint32_t)(G::O_COL + HD + g * OC), ov);
#pragma unroll
                for (int k = 0; k < OC; ++k) o[k] = fmaf(__uint_as_float(ov[k]), a1, o[k]);
            }
            if (q_lo + r < nrows) {
                __nv_bfloat16* dst = out + (size_t)(row0 + q_lo + r) * out_stride + (size_t)head * HD + g * OC;
#pragma unroll
                for (int k = 0; k < OC; k += 8) {
                    uint4 w;
                    w.x = pack2(__float_as_uint(o[k] * inv), __float_as_uint(o[k + 1] * inv));
                    w.y = pack2(__float_as_uint(o[k + 2] * inv), __float_as_uint(o[k + 3] * inv));
                    w.z = pack2(__float_as_uint(o[k + 4] * inv), __float_as_uint(o[k + 5] * inv));
                    w.w = pack2(__float_as_uint(o[k + 6] * inv), __float_as_uint(o[k + 7] * inv));
                    *reinterpret_cast<uint4*>(dst + k) = w;
                }
            }
        }
    }

    // ------------------------------------------------------------------------------- wind down
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        if (lane == 0 && sh.abort_flag) {
            // copies that were issued but never consumed may still be in flight: wait for them (bounded)
            if (sh.q_issued && !sh.q_consumed) {
                const long long t0 = clock64();
                while (!mbar_try_wait(&sh.q_full, 0) && clock64() - t0 < TC_WAIT_CYCLES) {}
            }
            for (int what = 0; what < 2; ++what)
                for (int it = sh.consumed[what]; it < sh.issued[what]; ++it) {
                    uint64_t* bar = what == 0 ? &sh.k_full[it % AT_STAGES] : &sh.v_full[it % AT_STAGES];
                    const long long t0 = clock64();
                    while (!mbar_try_wait(bar, (it / AT_STAGES) & 1) && clock64() - t0 < TC_WAIT_CYCLES) {}
                }
        }
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(G::TMEM_COLS) : "memory");
    }
}

GB_EXPORT int gb_attention_prefill_tc_supported(int nh, int nkv, int hd, int page_size) {
    if (nkv <= 0 || nh % nkv) return 0;
    return hd == 64 && page_size >= 8 && page_size <= AT_BN && (page_size & (page_size - 1)) == 0;
}

// Rows of each request are consecutive: request s owns rows seq_first_row[s] .. seq_first_row[s+1]-1, at
// positions seq_start_pos[s] + local index. q [n_rows, >= nh*hd] and out are bfloat16 with 16-byte aligned
// rows; kcache and vcache are one layer of the paged cache, [num_pages, nkv, page_size, hd] contiguous.
GB_EXPORT int gb_attention_prefill_tc(const void* q, long long q_stride, int n_rows, void* out, long long out_stride,
                                      const void* kcache, const void* vcache, const int* block_tables, int max_pages,
                                      const int* seq_first_row, const int* seq_start_pos, int num_seqs,
                                      int max_rows_per_seq, int nh, int nkv, int hd, int page_size, long long num_pages,
                                      float scale, int window, int* status, cudaStream_t stream) {
    GB_REQUIRE(gb_attention_prefill_tc_supported(nh, nkv, hd, page_size),
               "gb_attention_prefill_tc: head size %d (64) / page size %d (a power of two, 8..128) is not built", hd, page_size);
    GB_REQUIRE(q_stride % 8 == 0 && (uintptr_t)q % 16 == 0 && q_stride >= (long long)nh * hd,
               "gb_attention_prefill_tc: q rows must be 16-byte aligned");
    GB_REQUIRE(out_stride % 8 == 0 && (uintptr_t)out % 16 == 0, "gb_attention_prefill_tc: out rows must be 16-byte aligned");
    GB_REQUIRE((uintptr_t)kcache % 16 == 0 && (uintptr_t)vcache % 16 == 0, "gb_attention_prefill_tc: the cache must be 16-byte aligned");
    GB_REQUIRE(num_seqs >= 0 && num_seqs <= 65535 && nh <= 65535 && max_pages > 0 && status != nullptr && n_rows >= 0,
               "gb_attention_prefill_tc: bad batch shape");
    GB_REQUIRE(num_pages * nkv * page_size < (1ll << 31), "gb_attention_prefill_tc: the cache layer has too many rows for a 32-bit TMA coordinate");
    if (num_seqs == 0 || max_rows_per_seq <= 0 || n_rows == 0) return 0;
    using G = AtGeometry<64>;
    CUtensorMap mq, mk, mv;
    if (tc_make_map_2d(&mq, q, n_rows, (long long)nh * hd, q_stride, AT_BM, 64, "gb_attention_prefill_tc")) return 1;
    if (tc_make_map_2d(&mk, kcache, num_pages * nkv * page_size, hd, hd, page_size, 64, "gb_attention_prefill_tc")) return 1;
    if (tc_make_map_2d(&mv, vcache, num_pages * nkv * page_size, hd, hd, page_size, 64, "gb_attention_prefill_tc")) return 1;
    auto kernel = attention_prefill_tc_kernel<64>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM);
        GB_REQUIRE(e == cudaSuccess, "gb_attention_prefill_tc: %d bytes of shared memory refused: %s", G::SMEM, cudaGetErrorString(e));
        configured = true;
    }
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    dim3 grid(gb_ceil_div(max_rows_per_seq, AT_BM), nh, num_seqs);
    cudaError_t e = gb_launch(GB_PDL_ATTENTION, kernel, grid, dim3(AT_WARPS * 32), G::SMEM, stream, mq, mk, mv, (__nv_bfloat16*)out, out_stride,
                              block_tables, max_pages, seq_first_row, seq_start_pos, nh, nkv, page_size, page_shift, num_pages,
                              scale, window, status);
    GB_REQUIRE(e == cudaSuccess, "gb_attention_prefill_tc: launch failed: %s", cudaGetErrorString(e));
    return gb_check_launch("gb_attention_prefill_tc");
}
