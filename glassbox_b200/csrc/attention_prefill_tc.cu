// Causal grouped-query flash attention for prompt portions on the 5th-generation tensor cores
// (sm_100a): both products of the scheme, S = Q K^T and O += P V, are tcgen05.mma instructions with
// their accumulators in tensor memory; queries, keys and values come into shared memory by TMA, the
// keys and values page by page straight from the paged cache through the request's block table.
//
// One block = 128 consecutive query rows of one request for one query head, over tiles of 128 keys:
//   warp 0      producer. Lane 0 loads the query tile once; for every key tile the lanes read the page
//               ids from the block table (one tile ahead) and each issues the TMA loads of one page of
//               keys and one of values (a page is `page_size` rows of one kv head: one box of the 2-D
//               view [pages * kv_heads * page_size, head_dim] of a cache layer) into a ring of stages.
//   warp 1      lane 0 issues the tensor-core work. S_j = Q K_j^T (M 128, N 128, K head_dim; both
//               operands K-major in 128-byte-swizzled rows) goes to one of two TMEM buffers, so that
//               S_{j+1} is computed while the softmax warps work on S_j. When P_j is in shared memory,
//               O += P_j V_j (M 128, N head_dim, K 128; V is the MN-major operand: its rows are keys)
//               accumulates in a third TMEM region.
//   warps 2-5   softmax, one query row per thread (a row is one TMEM lane, so no shuffles): the thread
//               reads its 128 scores with one tcgen05.ld, takes the maximum, and writes
//               P_j = exp2((S_j - m) c) rounded to bfloat16 into shared memory (two buffers) in the
//               A-operand layout. The running maximum m is only raised, and O and the row sum rescaled
//               (tcgen05.ld / st of the O rows by the whole warp), when a new maximum exceeds it by
//               more than 2^8 in the exponent: until then P stays below 256, which bfloat16 and the
//               float32 sums hold without loss, and the final O / l is the same. After the last tile the
//               thread reads its O row, divides by the row sum and stores it.
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

constexpr int AT_STAGES = 3;   // key/value tiles in flight

struct __align__(8) AtShared {
    uint64_t q_full;                 // TMA -> MMA: the query tile has landed
    uint64_t kv_full[AT_STAGES];     // TMA -> MMA: a stage's keys and values have landed
    uint64_t kv_empty[AT_STAGES];    // MMA -> TMA: the tensor core has read the stage
    uint64_t s_full[2];              // MMA -> softmax: S_j is complete in buffer j & 1
    uint64_t s_free[2];              // softmax -> MMA: S_j has been read out of buffer j & 1
    uint64_t p_ready[2];             // softmax -> MMA: P_j is in shared-memory buffer j & 1 (and O is rescaled)
    uint64_t pv_done[2];             // MMA -> softmax: O += P_j V_j is complete (P buffer j & 1 is free, O is current)
    uint32_t tmem_base;
    int abort_flag;
    int issued;             // key tiles whose TMA loads were issued
    int consumed;           // key tiles whose kv_full barrier the MMA thread has passed
    int q_issued, q_consumed;
};

template <int HD> struct AtGeometry {
    static constexpr int Q_BYTES = AT_BM * HD * 2, KV_BYTES = AT_BN * HD * 2, P_BYTES = AT_BM * AT_BN * 2;
    static constexpr int K_OFF = Q_BYTES, V_OFF = K_OFF + AT_STAGES * KV_BYTES, P_OFF = V_OFF + AT_STAGES * KV_BYTES;
    static constexpr int SH_OFF = P_OFF + 2 * P_BYTES;
    static constexpr int SMEM = SH_OFF + 256;
    static constexpr int O_COL = 2 * AT_BN;   // two S buffers of 128 columns, then O
    static constexpr int TMEM_COLS = 512;
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

__device__ __forceinline__ float at_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int HD>
__global__ void __launch_bounds__(192) attention_prefill_tc_kernel(
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
    unsigned char* Ps = at_smem + G::P_OFF;
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
            mbar_init(&sh.kv_full[b], 1);
            mbar_init(&sh.kv_empty[b], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sh.s_full[b], 1);
            mbar_init(&sh.s_free[b], 4);    // one arrival per softmax warp
            mbar_init(&sh.p_ready[b], 4);
            mbar_init(&sh.pv_done[b], 1);
        }
        sh.abort_flag = 0;
        sh.issued = sh.consumed = sh.q_issued = sh.q_consumed = 0;
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

    if (warp == 0) {
        // ------------------------------------------------------------------------- producer
        if (lane == 0) {
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
        long long page = page_of(kt_begin);
        for (int j = 0; j < ntiles; ++j) {
            const int s = j % AT_STAGES;
            const long long next_page = j + 1 < ntiles ? page_of(kt_begin + j + 1) : 0;   // in flight during the wait
            int ok = 1;
            if (lane == 0 && j >= AT_STAGES)
                ok = mbar_wait(&sh.kv_empty[s], ((j / AT_STAGES) - 1) & 1, abort_flag, status) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane == 0) mbar_expect_tx(&sh.kv_full[s], 2 * G::KV_BYTES);
            __syncwarp();
            if (lane < ppt) {
                const int row = (int)((page * nkv + kvh) * page_size);
                const int dst = s * G::KV_BYTES + lane * page_size * HD * 2;
                tma_load_2d(Ks + dst, &map_k, &sh.kv_full[s], 0, row);
                tma_load_2d(Vs + dst, &map_v, &sh.kv_full[s], 0, row);
            }
            __syncwarp();
            if (lane == 0) sh.issued = j + 1;
            page = next_page;
        }
        if (bad) atomicOr(status, GB_STATUS_BAD_SLOT);
    } else if (warp == 1) {
        // ------------------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc_qk = umma_idesc(AT_BM, AT_BN);
            const uint32_t idesc_pv = umma_idesc(AT_BM, HD) | (1u << 16);   // B is MN-major
            const uint32_t q_addr = smem_u32(Qs), k_addr = smem_u32(Ks), v_addr = smem_u32(Vs), p_addr = smem_u32(Ps);
            bool ok = mbar_wait(&sh.q_full, 0, abort_flag, status);
            if (ok) sh.q_consumed = 1;
            // S_j: wait for its keys and for the buffer, issue, tell the softmax warps
            auto issue_qk = [&](int j) {
                const int s = j % AT_STAGES;
                if (!mbar_wait(&sh.kv_full[s], (j / AT_STAGES) & 1, abort_flag, status)) return false;
                sh.consumed = j + 1;
                if (j >= 2 && !mbar_wait(&sh.s_free[j & 1], ((j >> 1) - 1) & 1, abort_flag, status)) return false;
                tc_fence_after();
                const uint32_t kb = k_addr + (uint32_t)(s * G::KV_BYTES);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    umma_bf16(tmem + (uint32_t)((j & 1) * AT_BN), umma_desc(q_addr + k * 32), umma_desc(kb + k * 32), idesc_qk,
                              k ? 1u : 0u);
                umma_commit(&sh.s_full[j & 1]);
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int j = 0; j < ntiles && ok; ++j) {
                if (j + 1 < ntiles && !issue_qk(j + 1)) { ok = false; break; }
                if (!mbar_wait(&sh.p_ready[j & 1], (j >> 1) & 1, abort_flag, status)) { ok = false; break; }
                tc_fence_after();
                const int s = j % AT_STAGES;
                const uint32_t vb = v_addr + (uint32_t)(s * G::KV_BYTES);
                const uint32_t pb = p_addr + (uint32_t)((j & 1) * G::P_BYTES);
#pragma unroll
                for (int kk = 0; kk < AT_BN / 16; ++kk)   // 16 keys per instruction
                    umma_bf16(tmem + (uint32_t)G::O_COL, umma_desc(pb + (kk >> 2) * (AT_BM * 128) + (kk & 3) * 32),
                              umma_desc_mn(vb + kk * 16 * 128, AT_BN * 128), idesc_pv, (j | kk) ? 1u : 0u);
                umma_commit(&sh.pv_done[j & 1]);
                umma_commit(&sh.kv_empty[s]);
            }
        }
    } else {
        // ------------------------------------------------------------------------- softmax
        const int q = warp & 3;                        // the quarter of TMEM lanes this warp may read
        const int r = q * 32 + lane;                   // this thread's query row within the tile
        const int pos = pos_lo + r;
        const float sl2 = scale * 1.4426950408889634f; // exp(x * scale) = exp2(x * sl2)
        const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16);
        float m_run = AT_NEG_BIG, l_run = 0.f;
        bool ok = true;
        auto visible = [&](int key) { return key <= pos && (window <= 0 || key > pos - window); };
        for (int j = 0; j < ntiles; ++j) {
            const int b = j & 1, key0 = (kt_begin + j) * AT_BN;
            if (!mbar_wait_warp(&sh.s_full[b], (j >> 1) & 1, abort_flag, status)) { ok = false; break; }
            tc_fence_after();
            uint32_t sv[AT_BN];
            tmem_load128(lane_base + (uint32_t)(b * AT_BN), sv);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.s_free[b]);   // the buffer may take S_{j+2}
            // the mask matters only where the tile crosses the diagonal, the window's edge or the last key
            const bool need_mask = key0 + AT_BN - 1 > pos_lo || (window > 0 && key0 < pos_lo + AT_BM - window);
            // four independent chains each for the maximum and the sum: one warp per scheduler has nothing
            // else to hide the latency of a dependent chain behind
            float mx4[4] = {AT_NEG_BIG, AT_NEG_BIG, AT_NEG_BIG, AT_NEG_BIG};
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < AT_BN; ++i) {
                    if (!visible(key0 + i)) sv[i] = __float_as_uint(AT_NEG_BIG);
                    mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
                }
            } else {
#pragma unroll
                for (int i = 0; i < AT_BN; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // raise the running maximum only when it is exceeded by more than 2^8 in the exponent
            const bool raise = (mx - m_run) * sl2 > 8.0f;
            if (j == 0) {
                if (raise) m_run = mx;               // nothing is accumulated yet
            } else if (__any_sync(0xffffffffu, raise)) {
                // O += P_{j-1} V_{j-1} must be complete before the rows are rescaled
                if (!mbar_wait_warp(&sh.pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, status)) { ok = false; break; }
                tc_fence_after();
                const float corr = raise ? at_exp2((m_run - mx) * sl2) : 1.0f;
                if (raise) m_run = mx;
                l_run *= corr;
#pragma unroll
                for (int c = 0; c < HD; c += 32) {
                    uint32_t ov[32];
                    tmem_load32(lane_base + (uint32_t)(G::O_COL + c), ov);
#pragma unroll
                    for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
                    tmem_store32(lane_base + (uint32_t)(G::O_COL + c), ov);
                }
            }
            // P buffer b was read by O += P_{j-2} V_{j-2}
            if (j >= 2 && !mbar_wait_warp(&sh.pv_done[b], ((j >> 1) - 1) & 1, abort_flag, status)) { ok = false; break; }
            const float msl = m_run * sl2;
            float l4[4] = {0.f, 0.f, 0.f, 0.f};
            unsigned char* prow = Ps + b * G::P_BYTES + r * 128;
#pragma unroll
            for (int c = 0; c < AT_BN; c += 8) {
                float p[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    // a masked key contributes nothing, whatever the running maximum is
                    const float x = __uint_as_float(sv[c + i]);
                    p[i] = (need_mask && x <= AT_NEG_BIG) ? 0.f : at_exp2(fmaf(x, sl2, -msl));
                    l4[i & 3] += p[i];
                }
                uint4 w;
                w.x = pack2(__float_as_uint(p[0]), __float_as_uint(p[1]));
                w.y = pack2(__float_as_uint(p[2]), __float_as_uint(p[3]));
                w.z = pack2(__float_as_uint(p[4]), __float_as_uint(p[5]));
                w.w = pack2(__float_as_uint(p[6]), __float_as_uint(p[7]));
                // keys c .. c+7 of row r: chunk (c % 64) / 8 of the 64-key block c / 64
                const int chunk = (c & 63) >> 3;
                *reinterpret_cast<uint4*>(prow + (c >> 6) * (AT_BM * 128) + ((chunk ^ (r & 7)) << 4)) = w;
            }
            l_run += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            // the stores above must be visible to the tensor core (the asynchronous proxy) before it is told
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.p_ready[b]);
        }
        if (ok) ok = mbar_wait_warp(&sh.pv_done[(ntiles - 1) & 1], ((ntiles - 1) >> 1) & 1, abort_flag, status);
        if (ok) {
            tc_fence_after();
            uint32_t ov[HD];
            tmem_load64(lane_base + (uint32_t)G::O_COL, ov);
            if (q_lo + r < nrows) {
                const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
                __nv_bfloat16* dst = out + (size_t)(row0 + q_lo + r) * out_stride + (size_t)head * HD;
#pragma unroll
                for (int i = 0; i < HD; i += 8) {
                    uint4 w;
                    w.x = pack2(__float_as_uint(__uint_as_float(ov[i]) * inv), __float_as_uint(__uint_as_float(ov[i + 1]) * inv));
                    w.y = pack2(__float_as_uint(__uint_as_float(ov[i + 2]) * inv), __float_as_uint(__uint_as_float(ov[i + 3]) * inv));
                    w.z = pack2(__float_as_uint(__uint_as_float(ov[i + 4]) * inv), __float_as_uint(__uint_as_float(ov[i + 5]) * inv));
                    w.w = pack2(__float_as_uint(__uint_as_float(ov[i + 6]) * inv), __float_as_uint(__uint_as_float(ov[i + 7]) * inv));
                    *reinterpret_cast<uint4*>(dst + i) = w;
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
            for (int it = sh.consumed; it < sh.issued; ++it) {
                const long long t0 = clock64();
                while (!mbar_try_wait(&sh.kv_full[it % AT_STAGES], (it / AT_STAGES) & 1) && clock64() - t0 < TC_WAIT_CYCLES) {}
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
    kernel<<<grid, 192, G::SMEM, stream>>>(mq, mk, mv, (__nv_bfloat16*)out, out_stride, block_tables, max_pages,
                                           seq_first_row, seq_start_pos, nh, nkv, page_size, page_shift, num_pages, scale,
                                           window, status);
    return gb_check_launch("gb_attention_prefill_tc");
}
