// C[M, N] (+)= X[M, K] * W[N, K]^T for few rows (M <= 64, decoding): a weight-streaming kernel
// with the neighbouring element-wise work folded in.
//
// The weights are the big operand and each is needed once, so the kernel is organised around
// reading W from HBM at full speed: a block owns a strip of 16 weight rows (or a pair of strips),
// its four warps take interleaved blocks of 32 k-values and pull them with 16-byte loads straight
// into the register layout of the tensor-core instruction (mma.sync m16n8k16, bfloat16 in, float32
// accumulate); the few activation rows sit in shared memory as the other operand; the four
// partial sums are added through shared memory. Inside each block of 32 k-values a thread's 16
// bytes are 8 consecutive k; the instruction's k index is a fixed permutation of them, applied to
// both operands, so every dot product still sums the same products, in an order that depends on the
// matrix and on the bucket of the row count (8, 16, 32, 64), never on a row's place in the batch.
//
// Folded in:
//  * prologue: RMSNorm. Instead of bfloat16 activations the kernel can take the float32 residual
//    rows and a gain: it computes 1/sqrt(mean(x^2)+eps) per row and stages gain*(x*s) rounded to
//    bfloat16, exactly what the separate norm kernel would have written
//    (crates/glassbox-core/src/model.rs:94-100).
//  * epilogue: store bfloat16 / float32, add into float32 (the residual stream), gated
//    (act = silu(gate) * up with the gate strip and the up strip I rows apart, model.rs:335-340), or
//    rotary + cache write for a stacked QKV matrix: the two strips of a pair are hd/2 rows apart,
//    i.e. the two halves (i, i + hd/2) of one head; q is rotated and stored, k is rotated and
//    written to the row's cache slot, v is written to the cache slot (model.rs:266-276).
//  * programmatic dependent launch: the first weights are requested before the kernel waits for
//    its predecessor in the stream (they do not depend on it), and the successor is released at
//    once, so consecutive small kernels overlap their start-up with each other's tails.
//  * split K over a thread-block cluster: when the matrix has few strips and a long K (a 2048 x 8192
//    down projection has 128 strips), one block per strip leaves most of the memory system idle. The
//    strip is then given to a cluster of 2, 4 or 8 blocks, each with a contiguous slice of K; their sums
//    travel through distributed shared memory to the cluster's first block, which adds them in rank
//    order (a fixed order: the result does not depend on timing) and runs the epilogue.
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

// KC: k per shared-memory chunk (256 or 512); each warp has KC/128 blocks of 32 k in flight per strip row
template <int NT, bool PAIR, int KC>
__global__ void __launch_bounds__(128) gemm_stream_kernel(const StreamArgs a) {
    constexpr int ROWS = NT * 8;   // activation rows held
    constexpr int SETS = PAIR ? 2 : 1;
    constexpr int WS_KC = KC;
    constexpr int WS_BPW = KC / 32 / 4;   // k32 blocks per warp per chunk
    __shared__ __align__(16) __nv_bfloat16 xs[ROWS][WS_KC + WS_PAD];
    __shared__ float srow[ROWS];
    // the partial sums of the four warps reuse the activation tile once the k loop is over
    static_assert(sizeof(float) * 4 * SETS * 16 * ROWS <= sizeof(__nv_bfloat16) * ROWS * (WS_KC + WS_PAD), "red fits in xs");
    float* red = reinterpret_cast<float*>(&xs[0][0]);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = lane >> 2, t = lane & 3;
    const int M = a.M, N = a.N, K = a.K;

    // let the next kernel in the stream start its own prologue
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // a cluster shares one strip: block `crank` of `csize` takes k in [kbeg, kend)
    cg::cluster_group cluster = cg::this_cluster();
    const int csize = (int)cluster.num_blocks(), crank = (int)cluster.block_rank();
    const int strip = blockIdx.x / csize;
    const int kbeg = min(K, crank * a.kslice), kend = min(K, kbeg + a.kslice);

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
    if (a.prefetch != nullptr) {
        // While this kernel waits for its predecessor and works, the weights of a kernel further down
        // the stream travel from HBM to L2: each block asks for its share, one 128-byte line per thread.
        const long long lines = (a.prefetch_bytes + 127) / 128;
        for (long long i = (long long)blockIdx.x * 128 + tid; i < lines; i += (long long)gridDim.x * 128)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(a.prefetch + i * 128));
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");   // everything below reads what it wrote

    const bool normalise = a.X == nullptr;
    if (normalise) {
        for (int m = warp; m < ROWS; m += 4) {
            float ss = 0.f;
            if (m < M) {
                const float* xr = a.xres + (size_t)m * a.ldr;
                for (int k = lane * 4; k < K; k += 128) {
                    const float4 v = *reinterpret_cast<const float4*>(xr + k);
                    ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
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
            xr[i] = (row < M && k < kend) ? *reinterpret_cast<const uint4*>(a.X + (size_t)row * a.ldx + k) : make_uint4(0, 0, 0, 0);
        }
    };
    if (!normalise && nchunks > 0) xload(0);

    for (int chunk = 0; chunk < nchunks; ++chunk) {
        // stage the activations of this chunk: ROWS x 256
        __syncthreads();
        if (normalise) {
            for (int c = tid; c < ROWS * (WS_KC / 8); c += 128) {
                const int row = c / (WS_KC / 8), col = (c % (WS_KC / 8)) * 8;
                const int k = kbeg + chunk * WS_KC + col;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (row < M && k < kend) {
                    const float* xrow = a.xres + (size_t)row * a.ldr + k;
                    const float4 x0 = *reinterpret_cast<const float4*>(xrow), x1 = *reinterpret_cast<const float4*>(xrow + 4);
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
    if (csize > 1) {
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
            const int pos = a.positions[tok];
            if (pos < 0) continue;               // padding row
            const int half = a.hd / 2;
            const int head = n / a.hd, i = n % a.hd;   // i < hd/2: this thread holds channels i and i + hd/2
            float y0 = v[0], y1 = v[1];
            if (head < a.nh + a.nkv && a.rope != nullptr) {
                if (pos >= a.max_pos) {
                    atomicOr(a.status, GB_STATUS_BAD_POSITION);
                } else {
                    const float2 cs = a.rope[(size_t)pos * half + i];
                    y0 = v[0] * cs.x - v[1] * cs.y;
                    y1 = v[1] * cs.x + v[0] * cs.y;
                }
            }
            if (head < a.nh) {
                __nv_bfloat16* q = reinterpret_cast<__nv_bfloat16*>(a.C) + (size_t)tok * a.ldc + (size_t)head * a.hd;
                q[i] = __float2bfloat16_rn(y0);
                q[i + half] = __float2bfloat16_rn(y1);
            } else if (a.write_kv) {
                const long long slot = a.slots[tok];
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
            *p += v[0];
        }
    }
}

template <int NT, bool PAIR, int KC>
static int launch_stream(const StreamArgs& a, int strips, int split, int pdl, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(strips * split);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (split > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = split;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_stream_kernel<NT, PAIR, KC>, a);
    if (e != cudaSuccess) {
        gb_set_error("gb_gemm_stream: launch failed: %s", cudaGetErrorString(e));
        return 2;
    }
    return gb_check_launch("gb_gemm_stream");
}

// Overrides for measurements: chunk (0 = choose, 256, 512) and cluster size (0 = choose, 1, 2, 4, 8).
static int g_tune_chunk = 0, g_tune_split = 0;
GB_EXPORT void gb_gemm_stream_tune(int chunk, int split) {
    g_tune_chunk = chunk;
    g_tune_split = split;
}

static int stream_sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    return sms;
}

// blocks of one instantiation that the chip holds at a time
template <int NT, bool PAIR, int KC>
static int stream_slots() {
    static int slots = 0;
    if (slots == 0) {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_stream_kernel<NT, PAIR, KC>, 128, 0) != cudaSuccess || per_sm <= 0)
            per_sm = 1;
        slots = per_sm * stream_sm_count();
    }
    return slots;
}

static int slots_of(int nt, bool pair, int kc) {
#define GB_SL(NTT) return pair ? (kc == 512 ? stream_slots<NTT, true, 512>() : stream_slots<NTT, true, 256>()) \
                               : (kc == 512 ? stream_slots<NTT, false, 512>() : stream_slots<NTT, false, 256>());
    if (nt == 1) { GB_SL(1) }
    if (nt == 2) { GB_SL(2) }
    if (nt == 4) { GB_SL(4) }
    return pair ? stream_slots<8, true, 256>() : stream_slots<8, false, 256>();
#undef GB_SL
}

static int dispatch_stream(StreamArgs a, int strips, bool pair, int pdl, cudaStream_t stream) {
    const int nt = a.M <= 8 ? 1 : a.M <= 16 ? 2 : a.M <= 32 ? 4 : 8;
    // The wide chunk keeps twice the loads in flight per thread, at twice the registers: it is taken
    // where its blocks still fit the chip in one wave (and never by the variants with many rows, which
    // have neither the registers nor the shared memory for it).
    const bool wide_fits = nt <= (pair ? 2 : 4);
    int kc = (wide_fits && strips <= slots_of(nt, pair, 512)) ? 512 : 256;
    if (g_tune_chunk == 256 || (g_tune_chunk == 512 && wide_fits)) kc = g_tune_chunk;
    // Cluster size: one block per 512 k, rounded up to a power of two, as long as all blocks are on the
    // chip at once and the other ranks' sums fit the first block's activation tile. Chunk and cluster
    // size depend on the matrix and on the row bucket (8, 16, 32, 64), not on which rows are in the batch.
    const int max_split = (kc + 32) / 32 / (pair ? 2 : 1) + 1;   // (split - 1) * sets * 32 <= kc + 32
    const int slots = slots_of(nt, pair, kc);
    int split = 1;
    while (split < 8 && split < a.K / 512) split *= 2;
    while (split > 1 && (split > max_split || strips * split > slots)) split /= 2;
    if (g_tune_split >= 1 && g_tune_split <= 8 && g_tune_split <= max_split) split = g_tune_split;
    a.kslice = split == 1 ? a.K : ((a.K + split - 1) / split + kc - 1) / kc * kc;
#define GB_WS2(NTT, KCC) return pair ? launch_stream<NTT, true, KCC>(a, strips, split, pdl, stream) : launch_stream<NTT, false, KCC>(a, strips, split, pdl, stream);
#define GB_WS(NTT) if (kc == 512) { GB_WS2(NTT, 512) } else { GB_WS2(NTT, 256) }
    if (nt == 1) { GB_WS(1) }
    if (nt == 2) { GB_WS(2) }
    if (nt == 4) { GB_WS(4) }
    GB_WS2(8, 256)
#undef GB_WS
#undef GB_WS2
}

static int check_common(const char* who, const void* x, const float* xres, const void* w, int M, int N, int K,
                        long long ldx, long long ldr, long long ldw) {
    GB_REQUIRE(M >= 0 && M <= 64 && N > 0 && K > 0, "%s: sizes M=%d N=%d K=%d outside its range (M <= 64)", who, M, N, K);
    GB_REQUIRE(K % 8 == 0 && ldw % 8 == 0 && (uintptr_t)w % 16 == 0, "%s: K and the weight row stride must be multiples of 8, the weights 16-byte aligned", who);
    if (x != nullptr)
        GB_REQUIRE(ldx % 8 == 0 && (uintptr_t)x % 16 == 0, "%s: activations must be 16-byte aligned with a row stride that is a multiple of 8", who);
    else
        GB_REQUIRE(xres != nullptr && ldr % 4 == 0 && (uintptr_t)xres % 16 == 0, "%s: float32 rows to normalise must be 16-byte aligned", who);
    return 0;
}

// mode: 0 store bfloat16, 1 store float32, 2 add into float32, 3 gated (W = [gate rows; up rows],
// N = number of gate rows, c = bfloat16 [M, N]). With x == nullptr the float32 rows `xres` are
// RMS-normalised with `gain` and `eps` on the way in. `prefetch` (optional) names a region that the
// kernel asks the memory system to bring into L2 for a later kernel. pdl != 0 launches with programmatic stream
// serialisation (the kernel waits for its predecessor itself, after prefetching weights).
GB_EXPORT int gb_gemm_stream(const void* x, long long ldx, const float* xres, long long ldr, const float* gain, float eps,
                             const void* w, long long ldw, void* c, long long ldc, int mode, int M, int N, int K,
                             const void* prefetch, long long prefetch_bytes, int pdl, cudaStream_t stream) {
    if (check_common("gb_gemm_stream", x, xres, w, M, N, K, ldx, ldr, ldw)) return 1;
    GB_REQUIRE(mode >= 0 && mode <= 3, "gb_gemm_stream: unknown mode %d", mode);
    GB_REQUIRE(mode != WS_GLU_BF16 || N % 16 == 0, "gb_gemm_stream: the gated mode needs N to be a multiple of 16");
    GB_REQUIRE(x != nullptr || gain != nullptr, "gb_gemm_stream: normalising needs a gain");
    if (M == 0) return 0;
    StreamArgs a = {};
    a.X = (const __nv_bfloat16*)x; a.ldx = ldx; a.xres = xres; a.ldr = ldr; a.gain = gain; a.eps = eps;
    a.W = (const __nv_bfloat16*)w; a.ldw = ldw; a.C = c; a.ldc = ldc; a.mode = mode; a.M = M; a.N = N; a.K = K;
    a.pair_offset = mode == WS_GLU_BF16 ? N : 0;
    a.prefetch = (const unsigned char*)prefetch; a.prefetch_bytes = prefetch ? prefetch_bytes : 0;
    return dispatch_stream(a, (N + 15) / 16, mode == WS_GLU_BF16, pdl, stream);
}

// Stacked QKV projection with rotary encoding and cache write in the epilogue. W = [q rows; k rows; v
// rows] ((nh + 2 nkv) * hd rows); q_out bfloat16 [M, >= nh*hd] receives the rotated queries; rotated keys
// and the values go to the cache slot of each row (unless write_kv == 0). hd must be a multiple of 32;
// rope == nullptr stores without rotation.
GB_EXPORT int gb_gemm_stream_qkv(const void* x, long long ldx, const float* xres, long long ldr, const float* gain,
                                 float eps, const void* w, long long ldw, void* q_out, long long ldq, int M, int K,
                                 const float* rope, int max_pos, const int* positions, const int* slots, void* kcache,
                                 void* vcache, int nh, int nkv, int hd, int page_size, long long num_pages, int write_kv,
                                 int* status, const void* prefetch, long long prefetch_bytes, int pdl,
                                 cudaStream_t stream) {
    const int N = (nh + 2 * nkv) * hd;
    if (check_common("gb_gemm_stream_qkv", x, xres, w, M, N, K, ldx, ldr, ldw)) return 1;
    GB_REQUIRE(hd > 0 && hd % 32 == 0 && nh > 0 && nkv > 0, "gb_gemm_stream_qkv: head size %d must be a multiple of 32", hd);
    GB_REQUIRE(x != nullptr || gain != nullptr, "gb_gemm_stream_qkv: normalising needs a gain");
    GB_REQUIRE(page_size > 0 && positions && slots && status && ldq >= (long long)nh * hd, "gb_gemm_stream_qkv: bad arguments");
    if (M == 0) return 0;
    StreamArgs a = {};
    a.X = (const __nv_bfloat16*)x; a.ldx = ldx; a.xres = xres; a.ldr = ldr; a.gain = gain; a.eps = eps;
    a.W = (const __nv_bfloat16*)w; a.ldw = ldw; a.C = q_out; a.ldc = ldq; a.mode = WS_ROPE_QKV; a.M = M; a.N = N; a.K = K;
    a.pair_offset = hd / 2;
    a.rope = (const float2*)rope; a.positions = positions; a.slots = slots;
    a.kcache = (__nv_bfloat16*)kcache; a.vcache = (__nv_bfloat16*)vcache;
    a.nh = nh; a.nkv = nkv; a.hd = hd; a.page_size = page_size; a.max_pos = max_pos; a.write_kv = write_kv;
    a.num_slots = num_pages * page_size; a.status = status;
    a.prefetch = (const unsigned char*)prefetch; a.prefetch_bytes = prefetch ? prefetch_bytes : 0;
    return dispatch_stream(a, (nh + 2 * nkv) * (hd / 32), true, pdl, stream);
}
