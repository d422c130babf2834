// The body of the weight-streaming product C[M, N] (+)= X[M, K] * W[N, K]^T for few rows (see gemm_stream.cu for
// the method), as a device function of a *virtual* block index, so that the same code serves two callers: the
// stand-alone kernel, whose blocks are the virtual blocks, and the persistent decode-program kernel
// (decode_program.cu), whose resident blocks walk over the virtual blocks of one product after another.
#pragma once

#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

enum { WS_STORE_BF16 = 0, WS_STORE_F32 = 1, WS_ADD_F32 = 2, WS_GLU_BF16 = 3, WS_ROPE_QKV = 4 };

constexpr int WS_PAD = 32;             // padding per activation row: row stride = 16 banks mod 32, so the
                                       // 16-byte operand loads of a quarter-warp never collide

struct StreamArgs {
    const __nv_bfloat16* X;   // [M, K] bfloat16 activations, or nullptr when `xres` is normalised instead
    long long ldx;
    const float* xres;        // [M, K] float32 rows to RMS-normalise (with X == nullptr)
    long long ldr;
    const float* gain;        // [K]
    float eps;
    const __nv_bfloat16* W;   // [N (+ pair rows), K]
    long long ldw;
    void* C;
    long long ldc;
    int mode, M, N, K;
    int pair_offset;          // rows between the two strips of a pair (gated: N; rotary: hd/2)
    // rotary + cache write
    const float2* rope;       // [max_pos, hd/2] (cos, sin) or nullptr (no rotation)
    const int* positions;     // [M]; a negative position marks a padding row
    const int* slots;         // [M]: page * page_size + offset
    __nv_bfloat16* kcache;    // [pages, nkv, page_size, hd]
    __nv_bfloat16* vcache;
    int nh, nkv, hd, page_size, max_pos, write_kv;
    long long num_slots;
    int* status;
    int kslice;               // k per block of a cluster (a multiple of the chunk); K without a cluster
    // a region to pull into L2 for a later kernel (its weights), or nullptr
    const unsigned char* prefetch;
    long long prefetch_bytes;
    int late_release;         // let the next kernel in the stream go only after this one's own wait (else at its start)
};

__device__ __forceinline__ void ws_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t ws_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Activations and residual rows: in a persistent kernel another block of the same launch wrote them, so they are read
// past L1 (which is not coherent between SMs); in the stand-alone kernel an earlier kernel wrote them and L1 may keep them.
template <bool PERSIST, typename V>
__device__ __forceinline__ V ld_act(const V* p) {
    if constexpr (PERSIST) return __ldcg(p);
    else return *p;
}

// Ask the memory system to bring the weights of virtual block `vblock` of a product into L2 (a hint; it writes and
// needs nothing): what a resident block of the persistent kernel does for its next product before it waits.
template <bool PAIR>
__device__ __forceinline__ void gemm_stream_prefetch_block(const StreamArgs& a, int vblock) {
    int n0;
    if (a.mode == WS_ROPE_QKV) {
        const int per_head = a.hd / 32;
        n0 = (vblock / per_head) * a.hd + (vblock % per_head) * 16;
    } else {
        n0 = vblock * 16;
    }
    const int lines_per_row = (a.K * 2 + 127) / 128;
    const int total = (PAIR ? 32 : 16) * lines_per_row;
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int rr = i / lines_per_row, line = i % lines_per_row;
        const int row = n0 + (rr & 15) + (rr >> 4) * a.pair_offset;
        if (row < (PAIR ? a.N + a.pair_offset : a.N))
            asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const unsigned char*>(a.W + (size_t)row * a.ldw) + (size_t)line * 128));
    }
}

// KC: k per shared-memory chunk (256 or 512); each warp has KC/128 blocks of 32 k in flight per strip row.
// PERSIST: called from a persistent kernel (no split of K over a cluster; `vblock` is the strip and its whole K),
// else from the stand-alone kernel (`vblock` = blockIdx.x). `sync` says how to wait for the work before (GbPdlSync
// in the stand-alone kernel).
// The caller provides the shared memory: `xs_raw` of gemm_stream_smem_bytes<NT, KC>() bytes, 16-byte aligned (the
// activation tile, reused for the partial sums), and `srow` of NT * 8 floats.
template <int NT, int KC>
__host__ __device__ constexpr int gemm_stream_smem_bytes() { return NT * 8 * (KC + WS_PAD) * 2; }

template <int NT, bool PAIR, int KC, bool PERSIST, class Sync>
__device__ __forceinline__ void gemm_stream_body(const StreamArgs& a, const int vblock, void* xs_raw, float* srow, Sync& sync) {
    constexpr int ROWS = NT * 8;   // activation rows held
    constexpr int SETS = PAIR ? 2 : 1;
    constexpr int WS_KC = KC;
    constexpr int WS_BPW = KC / 32 / 4;   // k32 blocks per warp per chunk
    __nv_bfloat16 (*xs)[WS_KC + WS_PAD] = reinterpret_cast<__nv_bfloat16 (*)[WS_KC + WS_PAD]>(xs_raw);
    // the partial sums of the four warps reuse the activation tile once the k loop is over
    static_assert(sizeof(float) * 4 * SETS * 16 * ROWS <= sizeof(__nv_bfloat16) * ROWS * (WS_KC + WS_PAD), "red fits in xs");
    float* red = reinterpret_cast<float*>(&xs[0][0]);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = lane >> 2, t = lane & 3;
    const int M = a.M, N = a.N, K = a.K;


    if (!a.late_release) sync.start();

    // a cluster shares one strip: block `crank` of `csize` takes k in [kbeg, kend)
    int csize = 1, crank = 0;
    if constexpr (!PERSIST) {
        cg::cluster_group cluster = cg::this_cluster();
        csize = (int)cluster.num_blocks();
        crank = (int)cluster.block_rank();
    }
    const int strip = vblock / csize;
    const int kbeg = PERSIST ? 0 : min(K, crank * a.kslice), kend = PERSIST ? K : min(K, kbeg + a.kslice);

    // first weight row of this block's strip (of its first strip, for a pair)
    int n0;
    if (a.mode == WS_ROPE_QKV) {
        const int per_head = a.hd / 32;   // strip pairs per head
        n0 = (strip / per_head) * a.hd + (strip % per_head) * 16;
    } else {
        n0 = strip * 16;
    }

    float acc[SETS][NT][4];
#pragma unroll
    for (int s = 0; s < SETS; ++s)
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[s][i][j] = 0.f;

    const int row_a = n0 + r, row_b = n0 + r + 8;
    const bool live_a = row_a < N, live_b = row_b < N;
    const __nv_bfloat16* wa[SETS];
    const __nv_bfloat16* wb[SETS];
#pragma unroll
    for (int s = 0; s < SETS; ++s) {
        wa[s] = a.W + (size_t)(row_a + s * a.pair_offset) * a.ldw;
        wb[s] = a.W + (size_t)(row_b + s * a.pair_offset) * a.ldw;
    }

    const int nchunks = (kend - kbeg + WS_KC - 1) / WS_KC;
    uint4 fa[SETS][WS_BPW], fb[SETS][WS_BPW];
    auto fetch = [&](int chunk) {
#pragma unroll
        for (int j = 0; j < WS_BPW; ++j) {
            const int k = kbeg + chunk * WS_KC + (j * 4 + warp) * 32 + 8 * t;
            const bool in = k < kend;
#pragma unroll
            for (int s = 0; s < SETS; ++s) {
                fa[s][j] = (in && live_a) ? ldg_stream(wa[s] + k) : make_uint4(0, 0, 0, 0);
                fb[s][j] = (in && live_b) ? ldg_stream(wb[s] + k) : make_uint4(0, 0, 0, 0);
            }
        }
    };

    if (nchunks > 0) fetch(0);   // weights do not depend on the previous kernel
    constexpr bool EARLY_ROPE = PAIR && NT <= 2;   // (the rotary mode runs with at most 16 rows)
    int rp_pos[EARLY_ROPE ? NT : 1], rp_slot[EARLY_ROPE ? NT : 1];
    float2 rp_cs[EARLY_ROPE ? NT : 1];
    {
        if (!PERSIST && a.prefetch != nullptr) {
            // While this kernel waits for its predecessor and works, the weights of a kernel further down
            // the stream travel from HBM to L2: each block asks for its share, one 128-byte line per thread.
            const long long lines = (a.prefetch_bytes + 127) / 128;
            for (long long i = (long long)blockIdx.x * 128 + tid; i < lines && blockIdx.y == 0; i += (long long)gridDim.x * 128)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(a.prefetch + i * 128));
        }
        // Rotary mode: a row's position, its (cos, sin) pair and its cache slot are step metadata that no kernel
        // writes. They are asked for now, so that the epilogue does not end on two dependent trips to memory.
        if constexpr (EARLY_ROPE) {
            if (a.mode == WS_ROPE_QKV) {
#pragma unroll
                for (int i = 0; i < NT; ++i) {
                    const int e = tid + i * 128, n = n0 + e % 16, tok = e / 16;
                    rp_pos[i] = -1;
                    rp_slot[i] = -1;
                    rp_cs[i] = make_float2(1.f, 0.f);
                    if (n < N && tok < M) {
                        const int pos = a.positions[tok];
                        rp_pos[i] = pos;
                        if (pos >= 0) {
                            rp_slot[i] = a.slots[tok];
                            if (n / a.hd < a.nh + a.nkv && a.rope != nullptr && pos < a.max_pos)
                                rp_cs[i] = a.rope[(size_t)pos * (a.hd / 2) + n % a.hd];
                        }
                    }
                }
            }
        }
        sync.wait();   // everything below reads what earlier work wrote
        if (a.late_release) sync.start();
        if (sync.gave_up()) return;
    }

    const bool normalise = a.X == nullptr;
    // One chunk holds the whole K (and no cluster shares it): a warp takes whole rows, two at a time, asks for all
    // their values (and the gains) at once, adds up the squares with shuffles and writes the normalised rows into
    // the tile: one trip to memory. Otherwise: a pass for the sums of squares, then the rows are read again chunk by
    // chunk. A lane adds up the same values in the same order either way (4 floats every 128), so the sums agree
    // to the bit.
    // (not in the 256-wide variant, which the largest matrices take: its register count decides how many blocks an SM holds)
    const bool norm_once = WS_KC >= 512 && normalise && nchunks == 1 && kbeg == 0 && kend == K;
    if (WS_KC >= 512 && norm_once) {
        constexpr int PPL = (WS_KC + 127) / 128;   // 4-float pieces of a row per lane
        const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
        float4 gn[PPL];
#pragma unroll
        for (int p = 0; p < PPL; ++p) {
            const int col = p * 128 + lane * 4;
            gn[p] = col < K ? *reinterpret_cast<const float4*>(a.gain + col) : zero4;
        }
        for (int m0 = warp; m0 < ROWS; m0 += 8) {
            float4 x[2][PPL];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int m = m0 + 4 * h;
#pragma unroll
                for (int p = 0; p < PPL; ++p) {
                    const int col = p * 128 + lane * 4;
                    x[h][p] = (m < M && col < K) ? ld_act<PERSIST>(reinterpret_cast<const float4*>(a.xres + (size_t)m * a.ldr + col)) : zero4;
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int m = m0 + 4 * h;
                if (m >= ROWS) continue;
                float ss = 0.f;
#pragma unroll
                for (int p = 0; p < PPL; ++p) {
                    const float4 v = x[h][p];
                    ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
                }
                ss = gb_warp_sum(ss);
                const float sc = 1.0f / sqrtf(ss / (float)K + a.eps);
#pragma unroll
                for (int p = 0; p < PPL; ++p) {
                    const int col = p * 128 + lane * 4;
                    if (col >= WS_KC) continue;
                    // rows beyond M and columns beyond K are zeros in the tile (x and the gain are zero there)
                    const float4 v = x[h][p], g4 = gn[p];
                    uint2 w;
                    w.x = ws_pack(g4.x * (v.x * sc), g4.y * (v.y * sc));
                    w.y = ws_pack(g4.z * (v.z * sc), g4.w * (v.w * sc));
                    *reinterpret_cast<uint2*>(&xs[m][col]) = w;
                }
            }
        }
    } else if (normalise) {
        for (int m = warp; m < ROWS; m += 4) {
            float ss = 0.f;
            if (m < M) {
                const float* xr = a.xres + (size_t)m * a.ldr;
                // four loads in flight at a time (the instructions issue in order: a load that is used at once
                // costs its whole latency, every time round); the squares are added in the order of k all the same
                for (int k0 = lane * 4; k0 < K; k0 += 512) {
                    float4 v[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        v[u] = k0 + 128 * u < K ? ld_act<PERSIST>(reinterpret_cast<const float4*>(xr + k0 + 128 * u)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        ss = fmaf(v[u].x, v[u].x, ss); ss = fmaf(v[u].y, v[u].y, ss);
                        ss = fmaf(v[u].z, v[u].z, ss); ss = fmaf(v[u].w, v[u].w, ss);
                    }
                }
            }
            ss = gb_warp_sum(ss);
            if (lane == 0) srow[m] = 1.0f / sqrtf(ss / (float)K + a.eps);
        }
    }

    // bfloat16 activations are fetched one chunk ahead into registers, so that their latency hides
    // behind the arithmetic of the chunk before (with 64 rows a chunk is 32 KB per block)
    constexpr int XPT = ROWS * (WS_KC / 8) / 128;   // 16-byte pieces per thread per chunk
    uint4 xr[XPT];
    auto xload = [&](int chunk) {
#pragma unroll
        for (int i = 0; i < XPT; ++i) {
            const int c = tid + i * 128;
            const int row = c / (WS_KC / 8), k = kbeg + chunk * WS_KC + (c % (WS_KC / 8)) * 8;
            xr[i] = (row < M && k < kend) ? ld_act<PERSIST>(reinterpret_cast<const uint4*>(a.X + (size_t)row * a.ldx + k)) : make_uint4(0, 0, 0, 0);
        }
    };
    if (!normalise && nchunks > 0) xload(0);

    for (int chunk = 0; chunk < nchunks; ++chunk) {
        // stage the activations of this chunk: ROWS x 256
        __syncthreads();
        if (norm_once) {
            // (the tile was written above)
        } else if (normalise) {
            constexpr int STAGE_UNROLL = NT <= 2 ? NT * WS_KC / 128 : 1;   // (rows are normalised on the way in only up to 16 of them)
#pragma unroll STAGE_UNROLL
            for (int c = tid; c < ROWS * (WS_KC / 8); c += 128) {
                const int row = c / (WS_KC / 8), col = (c % (WS_KC / 8)) * 8;
                const int k = kbeg + chunk * WS_KC + col;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (row < M && k < kend) {
                    const float* xrow = a.xres + (size_t)row * a.ldr + k;
                    const float4 x0 = ld_act<PERSIST>(reinterpret_cast<const float4*>(xrow)), x1 = ld_act<PERSIST>(reinterpret_cast<const float4*>(xrow + 4));
                    const float4 g0 = *reinterpret_cast<const float4*>(a.gain + k);
                    const float4 g1 = *reinterpret_cast<const float4*>(a.gain + k + 4);
                    const float s = srow[row];
                    v.x = ws_pack(g0.x * (x0.x * s), g0.y * (x0.y * s));
                    v.y = ws_pack(g0.z * (x0.z * s), g0.w * (x0.w * s));
                    v.z = ws_pack(g1.x * (x1.x * s), g1.y * (x1.y * s));
                    v.w = ws_pack(g1.z * (x1.z * s), g1.w * (x1.w * s));
                }
                *reinterpret_cast<uint4*>(&xs[row][col]) = v;
            }
        } else {
#pragma unroll
            for (int i = 0; i < XPT; ++i) {
                const int c = tid + i * 128;
                *reinterpret_cast<uint4*>(&xs[c / (WS_KC / 8)][(c % (WS_KC / 8)) * 8]) = xr[i];
            }
        }
        __syncthreads();
        if (!normalise && chunk + 1 < nchunks) xload(chunk + 1);
        uint4 ca[SETS][WS_BPW], cb[SETS][WS_BPW];
#pragma unroll
        for (int s = 0; s < SETS; ++s)
#pragma unroll
            for (int j = 0; j < WS_BPW; ++j) {
                ca[s][j] = fa[s][j];
                cb[s][j] = fb[s][j];
            }
        if (chunk + 1 < nchunks) fetch(chunk + 1);   // next chunk's weights fly while this one is used
#pragma unroll
        for (int j = 0; j < WS_BPW; ++j) {
            const int kb = (j * 4 + warp) * 32 + 8 * t;
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                // this thread's 8 consecutive k of token (8i + r): two k16 steps of 4 each
                const uint4 xv = *reinterpret_cast<const uint4*>(&xs[i * 8 + r][kb]);
#pragma unroll
                for (int s = 0; s < SETS; ++s) {
                    ws_mma(acc[s][i], ca[s][j].x, cb[s][j].x, ca[s][j].y, cb[s][j].y, xv.x, xv.y);
                    ws_mma(acc[s][i], ca[s][j].z, cb[s][j].z, ca[s][j].w, cb[s][j].w, xv.z, xv.w);
                }
            }
        }
    }

    // acc[s][i] = {(row r, token 8i+2t), (row r, token 8i+2t+1), (row r+8, ...), (row r+8, ...)}
    __syncthreads();
#pragma unroll
    for (int s = 0; s < SETS; ++s)
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int row = r + (j >> 1) * 8, tok = i * 8 + 2 * t + (j & 1);
                red[((warp * SETS + s) * 16 + row) * ROWS + tok] = acc[s][i][j];
            }
    __syncthreads();
    // each thread owns NT elements (strip row, token) of the block's tile and sums the four warps' parts
    float sum[NT][SETS];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        const int e = tid + i * 128, row = e % 16, tok = e / 16;
#pragma unroll
        for (int s = 0; s < SETS; ++s) {
            sum[i][s] = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) sum[i][s] += red[((w * SETS + s) * 16 + row) * ROWS + tok];
        }
    }
    if constexpr (!PERSIST) if (csize > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        // the first block's tile is free once every block of the cluster has passed this point; the others
        // write their sums into it, one plane per rank, and it adds them in rank order
        constexpr int PLANE = SETS * 16 * ROWS;
        cluster.sync();
        if (crank > 0) {
            float* dst = cluster.map_shared_rank(red, 0) + (size_t)(crank - 1) * PLANE;
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int s = 0; s < SETS; ++s) dst[s * 16 * ROWS + tid + i * 128] = sum[i][s];
        }
        cluster.sync();
        if (crank > 0) return;
        for (int rk = 1; rk < csize; ++rk)
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int s = 0; s < SETS; ++s) sum[i][s] += red[(rk - 1) * PLANE + s * 16 * ROWS + tid + i * 128];
    }
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        const int e = tid + i * 128;
        const int row = e % 16, tok = e / 16;   // consecutive threads -> consecutive n
        const int n = n0 + row;
        if (n >= N || tok >= M) continue;
        float v[2] = {sum[i][0], SETS > 1 ? sum[i][SETS - 1] : 0.f};
        if (a.mode == WS_ROPE_QKV) {
            const int ii = i;                    // (the channel index below takes the name i)
            int pos;
            if constexpr (EARLY_ROPE) pos = rp_pos[ii];
            else pos = a.positions[tok];
            if (pos < 0) continue;               // padding row
            const int half = a.hd / 2;
            const int head = n / a.hd, i = n % a.hd;   // i < hd/2: this thread holds channels i and i + hd/2
            float y0 = v[0], y1 = v[1];
            if (head < a.nh + a.nkv && a.rope != nullptr) {
                if (pos >= a.max_pos) {
                    atomicOr(a.status, GB_STATUS_BAD_POSITION);
                } else {
                    float2 cs;
                    if constexpr (EARLY_ROPE) cs = rp_cs[ii];
                    else cs = a.rope[(size_t)pos * half + i];
                    y0 = v[0] * cs.x - v[1] * cs.y;
                    y1 = v[1] * cs.x + v[0] * cs.y;
                }
            }
            if (head < a.nh) {
                __nv_bfloat16* q = reinterpret_cast<__nv_bfloat16*>(a.C) + (size_t)tok * a.ldc + (size_t)head * a.hd;
                q[i] = __float2bfloat16_rn(y0);
                q[i + half] = __float2bfloat16_rn(y1);
            } else if (a.write_kv) {
                long long slot;
                if constexpr (EARLY_ROPE) slot = rp_slot[ii];
                else slot = a.slots[tok];
                if (slot < 0 || slot >= a.num_slots) {
                    atomicOr(a.status, GB_STATUS_BAD_SLOT);
                } else {
                    const bool is_k = head < a.nh + a.nkv;
                    const int kvh = is_k ? head - a.nh : head - a.nh - a.nkv;
                    __nv_bfloat16* base = is_k ? a.kcache : a.vcache;
                    __nv_bfloat16* dst = base + (((slot / a.page_size) * a.nkv + kvh) * a.page_size + slot % a.page_size) * a.hd;
                    dst[i] = __float2bfloat16_rn(y0);
                    dst[i + half] = __float2bfloat16_rn(y1);
                }
            }
        } else if (a.mode == WS_GLU_BF16) {
            const float g = v[0] / (1.0f + __expf(-v[0])) * v[1];
            reinterpret_cast<__nv_bfloat16*>(a.C)[(size_t)tok * a.ldc + n] = __float2bfloat16_rn(g);
        } else if (a.mode == WS_STORE_BF16) {
            reinterpret_cast<__nv_bfloat16*>(a.C)[(size_t)tok * a.ldc + n] = __float2bfloat16_rn(v[0]);
        } else if (a.mode == WS_STORE_F32) {
            reinterpret_cast<float*>(a.C)[(size_t)tok * a.ldc + n] = v[0];
        } else {
            float* p = reinterpret_cast<float*>(a.C) + (size_t)tok * a.ldc + n;
            if constexpr (PERSIST) __stcg(p, __ldcg(p) + v[0]);
            else *p += v[0];
        }
    }
}

