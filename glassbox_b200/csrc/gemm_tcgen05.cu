// C[M, N] (+)= A[M, K] * W[N, K]^T in bfloat16 on the 5th-generation tensor cores (sm_100a):
// operands staged in shared memory by TMA, tcgen05.mma issued by one thread, the float32
// accumulator in tensor memory (TMEM), read back with tcgen05.ld for the epilogue.
//
// A persistent block (one per SM) computes 128 x BN tiles of C one after another (BN = 64, 128 or 256).
//   warp 0, one lane: producer. For each 64-wide k-block it waits until the stage is free, arms the
//       stage's "full" mbarrier with the bytes to come and issues two TMA loads (A box 128 x 64,
//       W box BN x 64, 128-byte swizzle; rows or columns outside the matrices are zero-filled by
//       the TMA unit, so M, N and K need not be multiples of the tile).
//   warp 1, one lane: issues 4 tcgen05.mma (M 128, N BN, K 16) per k-block from shared-memory matrix
//       descriptors, then tcgen05.commit to the stage's "empty" mbarrier (the stage is free once the
//       tensor core has read it) and, after the last k-block, to the "accumulator ready" mbarrier.
//   warps 2-5: epilogue. Each reads its quarter of the TMEM lanes (rows of the tile), 32 columns at a
//       time, and stores bfloat16 / float32, adds into float32 (the residual stream) or applies the
//       gated activation. Two accumulators alternate, so the epilogue of a tile overlaps the main loop
//       of the next.
// Both operands are K-major ([rows, K] with K contiguous), exactly as activations and [out, in]
// weights are stored (crates/glassbox-core/src/kernels.rs:381), so nothing is transposed.
//
// Every wait is bounded: a wait that exceeds its limit sets GB_STATUS_WAIT_TIMEOUT in the status
// word and the block winds down (waits, again bounded, for its own TMA copies, frees its TMEM,
// returns) instead of hanging the GPU. TMA loads use no multicast.
#include "tcgen05.cuh"

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;        // 64 bfloat16 = 128 bytes = one swizzle row

enum { TC_STORE_BF16 = 0, TC_STORE_F32 = 1, TC_ADD_F32 = 2, TC_ROPE_QKV = 3 };

// What the epilogue of a stacked QKV product needs to rotate the heads and write the cache: the
// (cos, sin) table [max_pos, hd/2], each row's position (negative: a padding row) and cache slot
// (page * page_size + offset), one layer of the paged cache [pages, nkv, page_size, hd].
struct TcQkv {
    const float2* rope;       // nullptr: no rotation
    const int* positions;
    const int* slots;
    __nv_bfloat16* kcache;
    __nv_bfloat16* vcache;
    int nh, nkv, hd, page_size, max_pos, write_kv;
    long long num_slots;
};

// An RMSNorm split between two products. The product that adds into the residual stream (the producer)
// knows every new residual value x as it writes it: it also stores bfloat16(x * gain) and, per row and
// column tile, the sum of x^2 over the tile's columns. The product that reads the normalised rows (the consumer)
// takes the bfloat16 matrix as its A operand and multiplies each row of its float32 sums by
// 1 / sqrt(sum x^2 / K + eps): a row's scale factors out of the product, so the result is that of
// normalising first (crates/glassbox-core/src/kernels.rs:36-52) with the one bfloat16 rounding of the
// activations in another place. The partial sums are added in column order: the same sums give the same bits.
struct TcNorm {
    const float* gain;        // producer: the gain of the norm that reads the residual next (nullptr: emit nothing)
    __nv_bfloat16* pre;       // producer: [M, N] bfloat16, x * gain
    long long ldp;
    float* ss_out;            // producer: [M, column tiles] partial sums of squares
    const float* ss_in;       // consumer: [M, ss_parts] (nullptr: rows are used as they are)
    int ss_parts;
    float eps;
};

constexpr int TC_MAX_STAGES = 8;

struct __align__(8) TcShared {
    uint64_t full[TC_MAX_STAGES];    // TMA -> MMA: a stage's operands have landed
    uint64_t empty[TC_MAX_STAGES];   // MMA -> TMA: the tensor core has read the stage
    uint64_t tfull[2];               // MMA -> epilogue: an accumulator is complete
    uint64_t tempty[2];              // epilogue -> MMA: an accumulator has been read out
    uint32_t tmem_base;
    int abort_flag;
    int issued;      // k-blocks whose TMA loads were issued
    int consumed;    // k-blocks whose full barrier the MMA thread has passed
};

template <int BN, bool GATED> struct TcGeometry {
    static constexpr int BNO = GATED ? BN / 2 : BN;                 // output columns per tile
    static constexpr int A_BYTES = TC_BM * TC_BK * 2, W_BYTES = BN * TC_BK * 2, STAGE_BYTES = A_BYTES + W_BYTES;
    static constexpr int STAGES = (192 * 1024 / STAGE_BYTES) < TC_MAX_STAGES ? (192 * 1024 / STAGE_BYTES) : TC_MAX_STAGES;
    static constexpr int EPI_BYTES = 4 * 32 * 33 * 4;               // per-warp transposition tiles
    static constexpr int SMEM = STAGES * STAGE_BYTES + EPI_BYTES + 1024;
};

// A persistent block walks over output tiles (tile = blockIdx.x, + gridDim.x, ...). Six warps:
//   warp 0 (one lane)  producer: TMA loads of A and W k-blocks into the stage ring, across tiles;
//   warp 1 (one lane)  MMA issuer: per tile, tcgen05.mma over the k-blocks into one of two TMEM
//                      accumulators, so that the next tile's main loop runs while the epilogue
//                      warps read the previous accumulator out;
//   warps 2-5          epilogue: warp w reads TMEM lanes 32*(w%4).. (rows of the tile), 32 columns at
//                      a time, and stores bfloat16 / float32, adds into float32 (the residual
//                      stream), or, GATED, stores silu(gate)*up: the tile's accumulator then holds the
//                      gate columns in its first half and the matching up columns (weight rows
//                      gate_rows further down, loaded by a second TMA box) in its second half
//                      (crates/glassbox-core/src/model.rs:335-340).
template <int BN, bool GATED>
__global__ void __launch_bounds__(192) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                                                           const __grid_constant__ CUtensorMap map_w, void* __restrict__ C,
                                                           int mode, int M, int N, int K, long long ldc, int gate_rows,
                                                           int* __restrict__ status, const TcQkv qkv, const TcNorm norm) {
    using G = TcGeometry<BN, GATED>;
    constexpr int STAGES = G::STAGES, BNO = G::BNO;
    extern __shared__ unsigned char smem_dyn[];
    // 128-byte-swizzled tiles want 1024-byte alignment
    unsigned char* tiles = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    float* epi = reinterpret_cast<float*>(tiles + STAGES * G::STAGE_BYTES);
    __shared__ TcShared sh;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kblocks = (K + TC_BK - 1) / TC_BK;
    const int tiles_m = (M + TC_BM - 1) / TC_BM, tiles_n = (N + BNO - 1) / BNO;
    const int ntiles = tiles_m * tiles_n;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&sh.full[s], 1);
            mbar_init(&sh.empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sh.tfull[b], 1);
            mbar_init(&sh.tempty[b], 4);   // one arrival per epilogue warp
        }
        sh.abort_flag = 0;
        sh.issued = 0;
        sh.consumed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    }
    if (warp == 0) {   // one warp allocates the two accumulators in tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_base)), "r"(2 * BN) : "memory");
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

    if (warp == 0) {
        if (lane == 0 && kblocks > 0) {
            // --------------------------------------------------------------------- producer
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * BNO;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(&sh.empty[s], ((it / STAGES) - 1) & 1, abort_flag, status)) { ok = false; break; }
                    unsigned char* a_dst = tiles + s * G::STAGE_BYTES;
                    mbar_expect_tx(&sh.full[s], G::STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, &sh.full[s], kb * TC_BK, m0);
                    if (GATED) {
                        tma_load_2d(a_dst + G::A_BYTES, &map_w, &sh.full[s], kb * TC_BK, n0);
                        tma_load_2d(a_dst + G::A_BYTES + G::W_BYTES / 2, &map_w, &sh.full[s], kb * TC_BK, gate_rows + n0);
                    } else {
                        tma_load_2d(a_dst + G::A_BYTES, &map_w, &sh.full[s], kb * TC_BK, n0);
                    }
                    sh.issued = it + 1;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && kblocks > 0) {
            // --------------------------------------------------------------------- MMA issuer
            const uint32_t idesc = umma_idesc(TC_BM, BN);
            int it = 0, tcount = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++tcount) {
                const int acc = tcount & 1;
                if (tcount >= 2 && !mbar_wait(&sh.tempty[acc], ((tcount >> 1) - 1) & 1, abort_flag, status)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem + (uint32_t)(acc * BN);
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&sh.full[s], (it / STAGES) & 1, abort_flag, status)) { ok = false; break; }
                    sh.consumed = it + 1;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + s * G::STAGE_BYTES);
                    const uint32_t w_addr = a_addr + G::A_BYTES;
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)   // 16 bfloat16 = 32 bytes further along K inside the swizzled row
                        umma_bf16(d_tmem, umma_desc(a_addr + k * 32), umma_desc(w_addr + k * 32), idesc, (kb | k) ? 1u : 0u);
                    umma_commit(&sh.empty[s]);       // arrives when the MMAs above have read the stage
                }
                if (ok) umma_commit(&sh.tfull[acc]);   // arrives when the tile's MMAs have finished
            }
        }
    } else {
        // ------------------------------------------------------------------------- epilogue
        const int q = warp & 3;                       // the quarter of TMEM lanes this warp may read
        float* stage = epi + q * (32 * 33);
        int tcount = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++tcount) {
            const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * BNO;
            const int acc = tcount & 1;
            const int row = m0 + q * 32 + lane;
            // consumer half of a split RMSNorm: this thread's row is scaled by 1 / rms of the residual row (read
            // while the tile's products still run)
            float inv_rms = 1.0f;
            if (norm.ss_in != nullptr && row < M) {
                float ss = 0.f;
                const float* sp = norm.ss_in + (size_t)row * norm.ss_parts;
                for (int p0 = 0; p0 < norm.ss_parts; p0 += 8) {   // eight loads in flight; added in the order of p
                    float part[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) part[u] = p0 + u < norm.ss_parts ? sp[p0 + u] : 0.f;
#pragma unroll
                    for (int u = 0; u < 8; ++u) ss += part[u];
                }
                inv_rms = 1.0f / sqrtf(ss / (float)K + norm.eps);
            }
            if (kblocks > 0) {
                if (!mbar_wait_warp(&sh.tfull[acc], (tcount >> 1) & 1, abort_flag, status)) { ok = false; break; }
                tc_fence_after();
            }
            const uint32_t t_base = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
            if (!GATED && mode == TC_ROPE_QKV) {
                // Stacked QKV (crates/glassbox-core/src/model.rs:266-276): a tile holds whole heads (BN is a multiple
                // of the head size). Query and key heads are rotated, channel i with channel i + hd/2, from the
                // float32 sums; queries go to C, rotated keys and the values to the row's cache slot.
                const int hd = qkv.hd, half = hd >> 1;
                const int pos = row < M ? qkv.positions[row] : -1;
                const long long slot = (row < M && pos >= 0) ? qkv.slots[row] : -1;
                const bool bad_pos = qkv.rope != nullptr && pos >= qkv.max_pos;
                const bool bad_slot = qkv.write_kv && pos >= 0 && (slot < 0 || slot >= qkv.num_slots);
                if (bad_pos) atomicOr(status, GB_STATUS_BAD_POSITION);
                if (bad_slot) atomicOr(status, GB_STATUS_BAD_SLOT);
                const int heads_total = qkv.nh + 2 * qkv.nkv;
#pragma unroll 1
                for (int c = 0; c < half; c += 32) {
                    // (cos, sin) of channels c .. c+31 at this row's position: read once, used by every head of the tile
                    float4 cs[16];
                    const bool have_cs = qkv.rope != nullptr && !bad_pos && pos >= 0;
                    if (have_cs) {
                        const float4* src = reinterpret_cast<const float4*>(qkv.rope + (size_t)pos * half + c);
#pragma unroll
                        for (int j = 0; j < 16; ++j) cs[j] = src[j];
                    }
#pragma unroll 1
                    for (int h0 = 0; h0 < BN; h0 += hd) {
                        const int head = (n0 + h0) / hd;
                        if (head >= heads_total) break;               // columns beyond the matrix (uniform for the block)
                        const bool is_q = head < qkv.nh, is_k = !is_q && head < qkv.nh + qkv.nkv;
                        __nv_bfloat16* dst = nullptr;                  // this row's head: hd contiguous bfloat16
                        if (pos >= 0) {
                            if (is_q) {
                                dst = reinterpret_cast<__nv_bfloat16*>(C) + (size_t)row * ldc + (size_t)head * hd;
                            } else if (qkv.write_kv && !bad_slot) {
                                const int kvh = is_k ? head - qkv.nh : head - qkv.nh - qkv.nkv;
                                dst = (is_k ? qkv.kcache : qkv.vcache) +
                                      (((slot / qkv.page_size) * qkv.nkv + kvh) * qkv.page_size + slot % qkv.page_size) * hd;
                            }
                        }
                        uint32_t x0[32], x1[32];   // the warp-collective loads run for every row; the stores only for live ones
                        tmem_load32(t_base + (uint32_t)(h0 + c), x0);
                        tmem_load32(t_base + (uint32_t)(h0 + half + c), x1);
                        if (norm.ss_in != nullptr) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                x0[j] = __float_as_uint(__uint_as_float(x0[j]) * inv_rms);
                                x1[j] = __float_as_uint(__uint_as_float(x1[j]) * inv_rms);
                            }
                        }
                        if ((is_q || is_k) && have_cs) {
#pragma unroll
                            for (int j = 0; j < 32; j += 2) {
                                const float4 t = cs[j >> 1];   // (cos, sin) of channels c+j and c+j+1
                                const float a0 = __uint_as_float(x0[j]), b0 = __uint_as_float(x1[j]);
                                const float a1 = __uint_as_float(x0[j + 1]), b1 = __uint_as_float(x1[j + 1]);
                                x0[j] = __float_as_uint(a0 * t.x - b0 * t.y);
                                x1[j] = __float_as_uint(b0 * t.x + a0 * t.y);
                                x0[j + 1] = __float_as_uint(a1 * t.z - b1 * t.w);
                                x1[j + 1] = __float_as_uint(b1 * t.z + a1 * t.w);
                            }
                        }
                        if (dst != nullptr) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint4 v0, v1;
                                v0.x = pack2(x0[j], x0[j + 1]); v0.y = pack2(x0[j + 2], x0[j + 3]);
                                v0.z = pack2(x0[j + 4], x0[j + 5]); v0.w = pack2(x0[j + 6], x0[j + 7]);
                                v1.x = pack2(x1[j], x1[j + 1]); v1.y = pack2(x1[j + 2], x1[j + 3]);
                                v1.z = pack2(x1[j + 4], x1[j + 5]); v1.w = pack2(x1[j + 6], x1[j + 7]);
                                *reinterpret_cast<uint4*>(dst + c + j) = v0;
                                *reinterpret_cast<uint4*>(dst + half + c + j) = v1;
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh.tempty[acc]);
                continue;
            }
            float ssq = 0.f;   // producer half of a split RMSNorm: this thread's row's sum of squares over the tile's columns
#pragma unroll 1
            for (int c0 = 0; c0 < BNO; c0 += 32) {
                uint32_t r[32];
                if (kblocks > 0) {
                    tmem_load32(t_base + (uint32_t)c0, r);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = 0u;
                }
                const int col0 = n0 + c0;
                if (norm.ss_in != nullptr) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * inv_rms);
                }
                if (GATED) {
                    uint32_t u[32];
                    if (kblocks > 0) {
                        tmem_load32(t_base + (uint32_t)(BN / 2 + c0), u);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) u[j] = 0u;
                    }
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float g = __uint_as_float(r[j]);
                        r[j] = __float_as_uint(g / (1.0f + __expf(-g)) * (__uint_as_float(u[j]) * inv_rms));
                    }
                }
                if (GATED || mode == TC_STORE_BF16) {
                    // a thread's 32 columns are 64 contiguous bytes: store them directly, 16 bytes at a time
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(C) + (size_t)row * ldc + col0;
                    if (row < M) {
                        if (col0 + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint4 v;
                                v.x = pack2(r[j], r[j + 1]); v.y = pack2(r[j + 2], r[j + 3]);
                                v.z = pack2(r[j + 4], r[j + 5]); v.w = pack2(r[j + 6], r[j + 7]);
                                *reinterpret_cast<uint4*>(dst + j) = v;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < N) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
                        }
                    }
                    continue;
                }
                // float32: through shared memory, so that one instruction writes one row (128 contiguous bytes)
#pragma unroll
                for (int j = 0; j < 32; ++j) stage[lane * 33 + j] = __uint_as_float(r[j]);
                __syncwarp();
                const int col = col0 + lane;
                if (col < N) {
                    float* base = reinterpret_cast<float*>(C) + (size_t)(m0 + q * 32) * ldc + col;
                    const int rows = min(32, M - (m0 + q * 32));
                    if (mode == TC_ADD_F32) {
                        float old[32];   // read the 32 residual values first (independent loads), then add and write
#pragma unroll
                        for (int rr = 0; rr < 32; ++rr) old[rr] = rr < rows ? base[(size_t)rr * ldc] : 0.f;
                        if (norm.gain != nullptr) {
                            // producer half of a split RMSNorm: the new residual values go back into the tile as well
#pragma unroll
                            for (int rr = 0; rr < 32; ++rr) {
                                const float v = old[rr] + stage[rr * 33 + lane];
                                if (rr < rows) base[(size_t)rr * ldc] = v;
                                stage[rr * 33 + lane] = v;
                            }
                        } else {
#pragma unroll
                            for (int rr = 0; rr < 32; ++rr)
                                if (rr < rows) base[(size_t)rr * ldc] = old[rr] + stage[rr * 33 + lane];
                        }
                    } else {
#pragma unroll
                        for (int rr = 0; rr < 32; ++rr)
                            if (rr < rows) base[(size_t)rr * ldc] = stage[rr * 33 + lane];
                    }
                }
                __syncwarp();
                if (mode == TC_ADD_F32 && norm.gain != nullptr) {
                    // ... and come back row by row: this thread's row leaves as bfloat16(x * gain), 64 contiguous
                    // bytes, and adds its squares to the row's sum (columns beyond N hold what the zero-filled
                    // weight rows gave: nothing is stored or summed for them)
                    __nv_bfloat16* dst = norm.pre + (size_t)row * norm.ldp + col0;
                    uint32_t packed[16];
                    if (col0 + 32 <= N) {
                        const float4* g4 = reinterpret_cast<const float4*>(norm.gain + col0);   // 16-byte aligned (checked by the host)
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 g = g4[j >> 2];
                            const float v0 = stage[lane * 33 + j], v1 = stage[lane * 33 + j + 1];
                            const float v2 = stage[lane * 33 + j + 2], v3 = stage[lane * 33 + j + 3];
                            ssq = fmaf(v0, v0, ssq); ssq = fmaf(v1, v1, ssq); ssq = fmaf(v2, v2, ssq); ssq = fmaf(v3, v3, ssq);
                            packed[j >> 1] = pack2(__float_as_uint(v0 * g.x), __float_as_uint(v1 * g.y));
                            packed[(j >> 1) + 1] = pack2(__float_as_uint(v2 * g.z), __float_as_uint(v3 * g.w));
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            const bool in0 = col0 + j < N, in1 = col0 + j + 1 < N;
                            const float v0 = in0 ? stage[lane * 33 + j] : 0.f, v1 = in1 ? stage[lane * 33 + j + 1] : 0.f;
                            const float g0 = in0 ? norm.gain[col0 + j] : 0.f, g1 = in1 ? norm.gain[col0 + j + 1] : 0.f;
                            ssq = fmaf(v0, v0, ssq);
                            ssq = fmaf(v1, v1, ssq);
                            packed[j >> 1] = pack2(__float_as_uint(v0 * g0), __float_as_uint(v1 * g1));
                        }
                    }
                    if (row < M) {
                        if (col0 + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
                            for (int j = 0; j < 16; j += 4)
                                *reinterpret_cast<uint4*>(dst + 2 * j) = make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < N) dst[j] = __ushort_as_bfloat16((unsigned short)(packed[j >> 1] >> ((j & 1) * 16)));
                        }
                    }
                    __syncwarp();
                }
            }
            // this warp is done with the accumulator: hand it back to the MMA issuer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.tempty[acc]);
            if (!GATED && mode == TC_ADD_F32 && norm.gain != nullptr && row < M)
                norm.ss_out[(size_t)row * tiles_n + (tile / tiles_m)] = ssq;
        }
    }

    // ------------------------------------------------------------------------------- wind down
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        if (lane == 0 && sh.abort_flag) {
            // copies that were issued but never consumed may still be in flight: wait for them (bounded)
            for (int it = sh.consumed; it < sh.issued; ++it) {
                const long long t0 = clock64();
                while (!mbar_try_wait(&sh.full[it % STAGES], (it / STAGES) & 1) && clock64() - t0 < TC_WAIT_CYCLES) {}
            }
        }
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * BN) : "memory");
    }
}

// ------------------------------------------------------------------------------------------- host
// [rows, K] bfloat16, K contiguous, `ld` elements between rows; boxes of box_rows x 64, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows) {
    return tc_make_map_2d(map, base, rows, K, ld, box_rows, TC_BK, "gb_gemm_tcgen05");
}

template <int BN, bool GATED>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mw, void* c, int mode, int M, int N, int K,
                     long long ldc, int gate_rows, int* status, cudaStream_t stream, const TcQkv& qkv = TcQkv(),
                     const TcNorm& norm = TcNorm()) {
    using G = TcGeometry<BN, GATED>;
    auto kernel = gemm_tcgen05_kernel<BN, GATED>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM);
        GB_REQUIRE(e == cudaSuccess, "gb_gemm_tcgen05: %d bytes of shared memory refused: %s", G::SMEM, cudaGetErrorString(e));
        configured = true;
    }
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    const int ntiles = gb_ceil_div(M, TC_BM) * gb_ceil_div(N, G::BNO);
    const int grid = ntiles < sms ? ntiles : sms;   // persistent: one block per SM walks the tiles
    cudaError_t e = gb_launch(GB_PDL_GEMM, kernel, dim3(grid), dim3(192), G::SMEM, stream, ma, mw, c, mode, M, N, K, ldc, gate_rows, status, qkv, norm);
    GB_REQUIRE(e == cudaSuccess, "gb_gemm_tcgen05: launch failed: %s", cudaGetErrorString(e));
    return gb_check_launch("gb_gemm_tcgen05");
}

// 1 if the operands satisfy what TMA needs (16-byte aligned bases, row strides that are multiples of
// 8 elements).
GB_EXPORT int gb_gemm_tcgen05_supported(const void* a, const void* w, int M, int N, int K, long long lda,
                                        long long ldw) {
    return M > 0 && N > 0 && K > 0 && lda % 8 == 0 && ldw % 8 == 0 && lda >= K && ldw >= K &&
           (uintptr_t)a % 16 == 0 && (uintptr_t)w % 16 == 0;
}

static int tc_sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    return sms;
}

// Output tile width. A block's time for one tile is about 0.33 us per 64-wide k-block, whatever the width (at these
// sizes the operands come from L2 at a rate that the tile count, not the tile size, sets), plus an epilogue that
// grows with the width and with what it does; a launch takes as many rounds of tiles as its busiest block has.
// The width with the smallest estimate wins; ties go to the wider tile, which reads the A operand less often.
// Measured at 2048 rows on a B200, microseconds for widths 64 / 128 / 256: N 960, K 576 store 9.5 / 7.3 / 8.7;
// N 576, K 1536 add 13.1 / 15.6 / 19.9; N 1600, K 960 store 18.9 / 15.1 / 11.4; N 960, K 2560 add 30.3 / 21.4 / 25.1;
// gated, I 1536, K 576: 20.0 (128) / 22.3 (256); I 8192, K 2048: 153 / 107.
enum { TC_EPI_STORE = 0, TC_EPI_ADD = 1, TC_EPI_GATED = 2 };
static int pick_bn(int M, int N, int K, int epilogue, int narrowest = 64) {
    static const float epi_us[3][3] = {{1.5f, 2.5f, 4.5f}, {2.8f, 5.5f, 11.0f}, {0.f, 3.0f, 7.0f}};
    const long long tm = gb_ceil_div(M, TC_BM);
    const float main_us = 0.33f * (float)gb_ceil_div(K, TC_BK);
    int best = 0;
    float best_us = 0.f;
    for (int i = 0, bn = 64; bn <= 256; ++i, bn *= 2) {
        if (bn < narrowest) continue;
        const int out_cols = epilogue == TC_EPI_GATED ? bn / 2 : bn;
        const long long rounds = gb_ceil_div(tm * gb_ceil_div(N, out_cols), (long long)tc_sm_count());
        const float us = (float)rounds * (main_us + epi_us[epilogue][i]);
        if (best == 0 || us <= best_us) { best = bn; best_us = us; }
    }
    return best;
}

// Column tiles of gb_gemm_tcgen05's output for this shape: the second extent of the partial sums of squares
// that a producer of a split RMSNorm writes.
GB_EXPORT int gb_gemm_tcgen05_column_tiles(int M, int N, int K) { return gb_ceil_div(N, pick_bn(M, N, K, TC_EPI_ADD)); }

// mode: 0 store bfloat16, 1 store float32, 2 add into float32.
// Split RMSNorm (see TcNorm): with mode 2 and norm_gain != nullptr the launch also writes pre[M, N] =
// bfloat16(c * norm_gain) and ss_out[M, gb_gemm_tcgen05_column_tiles(M, N, K)]; with ss_in != nullptr the rows of
// the product are scaled by 1 / sqrt(sum_p ss_in[row, p] / K + eps) before they are stored or added.
GB_EXPORT int gb_gemm_tcgen05(const void* a, const void* w, void* c, int mode, int M, int N, int K, long long lda,
                              long long ldw, long long ldc, int* status, cudaStream_t stream, const float* norm_gain,
                              void* pre, long long ldp, float* ss_out, const float* ss_in, int ss_parts, float eps) {
    GB_REQUIRE(gb_gemm_tcgen05_supported(a, w, M, N, K, lda, ldw),
               "gb_gemm_tcgen05: operands must be 16-byte aligned with row strides that are multiples of 8 (M=%d N=%d K=%d)",
               M, N, K);
    GB_REQUIRE(mode >= 0 && mode <= 2 && ldc >= N && status != nullptr, "gb_gemm_tcgen05: bad mode, ldc or status");
    GB_REQUIRE(norm_gain == nullptr || (mode == TC_ADD_F32 && pre != nullptr && ss_out != nullptr && ldp >= N &&
                                        (uintptr_t)norm_gain % 16 == 0),
               "gb_gemm_tcgen05: a norm is prepared only by a product that adds into float32, into pre and ss_out");
    GB_REQUIRE(ss_in == nullptr || ss_parts > 0, "gb_gemm_tcgen05: ss_parts must be positive");
    const int bn = pick_bn(M, N, K, mode == TC_ADD_F32 ? TC_EPI_ADD : TC_EPI_STORE);
    CUtensorMap ma, mw;
    if (make_map(&ma, a, M, K, lda, TC_BM)) return 1;
    if (make_map(&mw, w, N, K, ldw, bn)) return 1;
    TcNorm norm = {};
    norm.gain = norm_gain; norm.pre = (__nv_bfloat16*)pre; norm.ldp = ldp; norm.ss_out = ss_out;
    norm.ss_in = ss_in; norm.ss_parts = ss_parts; norm.eps = eps;
    if (bn == 256) return launch_tc<256, false>(ma, mw, c, mode, M, N, K, ldc, 0, status, stream, TcQkv(), norm);
    if (bn == 128) return launch_tc<128, false>(ma, mw, c, mode, M, N, K, ldc, 0, status, stream, TcQkv(), norm);
    return launch_tc<64, false>(ma, mw, c, mode, M, N, K, ldc, 0, status, stream, TcQkv(), norm);
}

// Gated feed-forward input product: w = [gate rows; up rows] (2*inter rows), c bfloat16 [M, inter] =
// silu(a gate^T) * (a up^T). inter must be a multiple of 8 (TMA row addressing needs nothing more).
// ss_in != nullptr: a is the bfloat16(x * gain) of a split RMSNorm and the sums are scaled row by row (see TcNorm).
GB_EXPORT int gb_gemm_tcgen05_gated(const void* a, const void* w, void* c, int M, int inter, int K, long long lda,
                                    long long ldw, long long ldc, int* status, cudaStream_t stream, const float* ss_in,
                                    int ss_parts, float eps) {
    GB_REQUIRE(gb_gemm_tcgen05_supported(a, w, M, 2 * inter, K, lda, ldw),
               "gb_gemm_tcgen05_gated: operands must be 16-byte aligned with row strides that are multiples of 8 (M=%d I=%d K=%d)",
               M, inter, K);
    GB_REQUIRE(ldc >= inter && status != nullptr, "gb_gemm_tcgen05_gated: bad ldc or status");
    CUtensorMap ma, mw;
    if (make_map(&ma, a, M, K, lda, TC_BM)) return 1;
    const bool wide = pick_bn(M, inter, K, TC_EPI_GATED, 128) == 256;
    // the weight map covers only the rows that exist, so a box that runs past the gate rows of the last
    // tile reads up rows: those columns are >= inter and are never stored
    if (make_map(&mw, w, 2LL * inter, K, ldw, wide ? 128 : 64)) return 1;
    GB_REQUIRE(ss_in == nullptr || ss_parts > 0, "gb_gemm_tcgen05_gated: ss_parts must be positive");
    TcNorm norm = {};
    norm.ss_in = ss_in; norm.ss_parts = ss_parts; norm.eps = eps;
    return wide ? launch_tc<256, true>(ma, mw, c, TC_STORE_BF16, M, inter, K, ldc, inter, status, stream, TcQkv(), norm)
                : launch_tc<128, true>(ma, mw, c, TC_STORE_BF16, M, inter, K, ldc, inter, status, stream, TcQkv(), norm);
}

// 1 if gb_gemm_tcgen05_qkv takes this head size: whole heads must tile the 128 columns of an output tile and half
// a head must be a multiple of the 32 columns an epilogue thread reads at a time.
GB_EXPORT int gb_gemm_tcgen05_qkv_supported(int hd) { return hd == 64 || hd == 128; }

// Stacked QKV projection with rotary encoding and cache write in the epilogue: w = [q rows; k rows; v rows]
// ((nh + 2 nkv) * hd rows); q_out bfloat16 [M, >= nh*hd] receives the rotated queries; rotated keys and the
// values go to the cache slot of each row (unless write_kv == 0). rope == nullptr stores without rotation.
GB_EXPORT int gb_gemm_tcgen05_qkv(const void* a, const void* w, void* q_out, int M, int K, long long lda, long long ldw,
                                  long long ldq, const float* rope, int max_pos, const int* positions, const int* slots,
                                  void* kcache, void* vcache, int nh, int nkv, int hd, int page_size, long long num_pages,
                                  int write_kv, int* status, cudaStream_t stream, const float* ss_in, int ss_parts,
                                  float eps) {
    const int N = (nh + 2 * nkv) * hd;
    GB_REQUIRE(gb_gemm_tcgen05_supported(a, w, M, N, K, lda, ldw),
               "gb_gemm_tcgen05_qkv: operands must be 16-byte aligned with row strides that are multiples of 8 (M=%d N=%d K=%d)",
               M, N, K);
    GB_REQUIRE(gb_gemm_tcgen05_qkv_supported(hd) && nh > 0 && nkv > 0, "gb_gemm_tcgen05_qkv: head size %d is not built (64, 128)", hd);
    GB_REQUIRE(ldq >= (long long)nh * hd && ldq % 8 == 0 && (uintptr_t)q_out % 16 == 0 && (uintptr_t)kcache % 16 == 0 &&
                   (uintptr_t)vcache % 16 == 0,
               "gb_gemm_tcgen05_qkv: q_out and the cache must be 16-byte aligned");
    GB_REQUIRE(page_size > 0 && positions && slots && status, "gb_gemm_tcgen05_qkv: bad arguments");
    CUtensorMap ma, mw;
    if (make_map(&ma, a, M, K, lda, TC_BM)) return 1;
    const int bn = pick_bn(M, N, K, TC_EPI_STORE, 128);   // whole heads per tile
    if (make_map(&mw, w, N, K, ldw, bn)) return 1;
    TcQkv q = {};
    q.rope = (const float2*)rope; q.positions = positions; q.slots = slots;
    q.kcache = (__nv_bfloat16*)kcache; q.vcache = (__nv_bfloat16*)vcache;
    q.nh = nh; q.nkv = nkv; q.hd = hd; q.page_size = page_size; q.max_pos = max_pos; q.write_kv = write_kv;
    q.num_slots = num_pages * page_size;
    GB_REQUIRE(ss_in == nullptr || ss_parts > 0, "gb_gemm_tcgen05_qkv: ss_parts must be positive");
    TcNorm norm = {};
    norm.ss_in = ss_in; norm.ss_parts = ss_parts; norm.eps = eps;
    if (bn == 256) return launch_tc<256, false>(ma, mw, q_out, TC_ROPE_QKV, M, N, K, ldq, 0, status, stream, q, norm);
    return launch_tc<128, false>(ma, mw, q_out, TC_ROPE_QKV, M, N, K, ldq, 0, status, stream, q, norm);
}
