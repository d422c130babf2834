// C[M, N] (+)= X[M, K] * W[N, K]^T for few rows (M <= 64, decoding): a weight-streaming kernel.
//
// The weights are the big operand and each is needed once, so the kernel is organised around
// reading W from HBM at full speed: every warp owns a strip of 16 weight rows and pulls them with
// 16-byte loads straight into the register layout of the tensor-core instruction
// (mma.sync m16n8k16, bfloat16 in, float32 accumulate); the few activation rows sit in shared
// memory as the other operand. Inside each block of 32 k-values a thread's 16 bytes are 8
// consecutive k; the instruction's k index is a fixed permutation of them, applied to both
// operands, so every dot product still sums the same products (in an order that depends only on
// K and the kernel variant, never on M or on a row's place in the batch).
//
// One strip per block: the four warps take interleaved k-blocks and their partial sums are added
// through shared memory, so even a 576-row matrix puts 36 x 4 warps to work. Output modes: store bfloat16 / float32,
// add into float32 (the residual stream), or gated: strips of the gate rows and of the up rows
// (I rows further down) are accumulated side by side and act = silu(gate) * up is stored
// (crates/glassbox-core/src/model.rs:335-340), which spares a kernel and the [M, 2I] round trip.
#include "common.cuh"

#include <mma.h>

enum { WS_STORE_BF16 = 0, WS_STORE_F32 = 1, WS_ADD_F32 = 2, WS_GLU_BF16 = 3 };

constexpr int WS_KC = 256;            // k per shared-memory chunk
constexpr int WS_PAD = 32;            // padding per activation row: row stride = 16 banks mod 32, so the
                                      // 16-byte operand loads of a quarter-warp never collide
constexpr int WS_BLOCKS = WS_KC / 32;  // k32 blocks per chunk

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
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

template <int NT, int KSPLIT, bool GLU>
__global__ void __launch_bounds__(128) gemm_stream_kernel(const __nv_bfloat16* __restrict__ X,
                                                          const __nv_bfloat16* __restrict__ W, void* __restrict__ C,
                                                          int mode, int M, int N, int K, long long ldx, long long ldw,
                                                          long long ldc, int glu_offset) {
    constexpr int ROWS = NT * 8;                          // activation rows held
    constexpr int BPW = WS_BLOCKS / KSPLIT;               // k32 blocks per warp per chunk
    constexpr int SETS = GLU ? 2 : 1;
    __shared__ __align__(16) __nv_bfloat16 xs[ROWS][WS_KC + WS_PAD];
    // the partial sums of the four warps reuse the activation tile once the k loop is over
    static_assert(sizeof(float) * 4 * SETS * 16 * ROWS <= sizeof(__nv_bfloat16) * ROWS * (WS_KC + WS_PAD), "red fits in xs");
    float* red = reinterpret_cast<float*>(&xs[0][0]);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = lane >> 2, t = lane & 3;
    const int strip = KSPLIT == 1 ? blockIdx.x * 4 + warp : blockIdx.x;
    const int n0 = strip * 16;
    // With GLU, N is the number of gate rows (= I) and the up rows start glu_offset rows below.
    const bool strip_live = n0 < N;

    float acc[SETS][NT][4];
#pragma unroll
    for (int s = 0; s < SETS; ++s)
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[s][i][j] = 0.f;

    const int row_a = n0 + r, row_b = n0 + r + 8;
    const bool live_a = strip_live && row_a < N, live_b = strip_live && row_b < N;
    const __nv_bfloat16* wa[SETS];
    const __nv_bfloat16* wb[SETS];
#pragma unroll
    for (int s = 0; s < SETS; ++s) {
        wa[s] = W + (size_t)(row_a + s * glu_offset) * ldw;
        wb[s] = W + (size_t)(row_b + s * glu_offset) * ldw;
    }

    const int nchunks = (K + WS_KC - 1) / WS_KC;
    uint4 fa[SETS][BPW], fb[SETS][BPW];
    auto fetch = [&](int chunk) {
#pragma unroll
        for (int j = 0; j < BPW; ++j) {
            const int blk = KSPLIT == 1 ? j : j * KSPLIT + warp;
            const int k = chunk * WS_KC + blk * 32 + 8 * t;
            const bool in = k < K;
#pragma unroll
            for (int s = 0; s < SETS; ++s) {
                fa[s][j] = (in && live_a) ? ldg_stream(wa[s] + k) : make_uint4(0, 0, 0, 0);
                fb[s][j] = (in && live_b) ? ldg_stream(wb[s] + k) : make_uint4(0, 0, 0, 0);
            }
        }
    };

    fetch(0);
    for (int chunk = 0; chunk < nchunks; ++chunk) {
        // stage the activations of this chunk: ROWS x 256, 16 bytes per thread and copy
        __syncthreads();
        for (int c = tid; c < ROWS * (WS_KC / 8); c += 128) {
            const int row = c / (WS_KC / 8), col = (c % (WS_KC / 8)) * 8;
            const int k = chunk * WS_KC + col;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < M && k < K) v = *reinterpret_cast<const uint4*>(X + (size_t)row * ldx + k);
            *reinterpret_cast<uint4*>(&xs[row][col]) = v;
        }
        __syncthreads();
        uint4 ca[SETS][BPW], cb[SETS][BPW];
#pragma unroll
        for (int s = 0; s < SETS; ++s)
#pragma unroll
            for (int j = 0; j < BPW; ++j) {
                ca[s][j] = fa[s][j];
                cb[s][j] = fb[s][j];
            }
        if (chunk + 1 < nchunks) fetch(chunk + 1);   // next chunk's weights fly while this one is used
#pragma unroll
        for (int j = 0; j < BPW; ++j) {
            const int blk = KSPLIT == 1 ? j : j * KSPLIT + warp;
            const int kb = blk * 32 + 8 * t;
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                // this thread's 8 consecutive k of token (8i + r): two k16 steps of 4 each
                const uint4 xv = *reinterpret_cast<const uint4*>(&xs[i * 8 + r][kb]);
#pragma unroll
                for (int s = 0; s < SETS; ++s) {
                    mma_bf16_16816(acc[s][i], ca[s][j].x, cb[s][j].x, ca[s][j].y, cb[s][j].y, xv.x, xv.y);
                    mma_bf16_16816(acc[s][i], ca[s][j].z, cb[s][j].z, ca[s][j].w, cb[s][j].w, xv.z, xv.w);
                }
            }
        }
    }

    // acc[s][i] = {(row r, token 8i+2t), (row r, token 8i+2t+1), (row r+8, ...), (row r+8, ...)}
    if (KSPLIT != 1) {
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
    }
    auto emit = [&](int row, int tok, float v0, float v1) {
        const int n = n0 + row;
        if (n >= N || tok >= M) return;
        if (mode == WS_GLU_BF16) {
            float a = v0 / (1.0f + __expf(-v0)) * v1;
            reinterpret_cast<__nv_bfloat16*>(C)[(size_t)tok * ldc + n] = __float2bfloat16_rn(a);
        } else if (mode == WS_STORE_BF16) {
            reinterpret_cast<__nv_bfloat16*>(C)[(size_t)tok * ldc + n] = __float2bfloat16_rn(v0);
        } else if (mode == WS_STORE_F32) {
            reinterpret_cast<float*>(C)[(size_t)tok * ldc + n] = v0;
        } else {
            float* p = reinterpret_cast<float*>(C) + (size_t)tok * ldc + n;
            *p += v0;
        }
    };
    if (KSPLIT == 1) {
        if (!strip_live) return;
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                emit(r + (j >> 1) * 8, i * 8 + 2 * t + (j & 1), acc[0][i][j], GLU ? acc[SETS - 1][i][j] : 0.f);
    } else {
        for (int e = tid; e < 16 * ROWS; e += 128) {
            const int row = e % 16, tok = e / 16;        // consecutive threads -> consecutive n
            float v[2] = {0.f, 0.f};
#pragma unroll
            for (int s = 0; s < SETS; ++s)
#pragma unroll
                for (int w = 0; w < 4; ++w) v[s] += red[((w * SETS + s) * 16 + row) * ROWS + tok];
            emit(row, tok, v[0], v[1]);
        }
    }
}

template <int NT, bool GLU>
static int launch_stream(const void* x, const void* w, void* c, int mode, int M, int N, int K, long long ldx,
                         long long ldw, long long ldc, int glu_offset, cudaStream_t stream) {
    const int strips = (N + 15) / 16;
    const __nv_bfloat16* X = (const __nv_bfloat16*)x;
    const __nv_bfloat16* W = (const __nv_bfloat16*)w;
    gemm_stream_kernel<NT, 4, GLU><<<strips, 128, 0, stream>>>(X, W, c, mode, M, N, K, ldx, ldw, ldc, glu_offset);
    return gb_check_launch("gb_gemm_stream");
}

// mode: 0 store bfloat16, 1 store float32, 2 add into float32, 3 gated (W = [gate rows; up rows],
// N = number of gate rows, c = bfloat16 [M, N]).
GB_EXPORT int gb_gemm_stream(const void* x, const void* w, void* c, int mode, int M, int N, int K, long long ldx,
                             long long ldw, long long ldc, cudaStream_t stream) {
    GB_REQUIRE(M >= 0 && M <= 64 && N > 0 && K > 0, "gb_gemm_stream: sizes M=%d N=%d K=%d outside its range (M <= 64)", M, N, K);
    GB_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0, "gb_gemm_stream: K and the row strides must be multiples of 8");
    GB_REQUIRE((uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0, "gb_gemm_stream: operands must be 16-byte aligned");
    GB_REQUIRE(mode >= 0 && mode <= 3, "gb_gemm_stream: unknown mode %d", mode);
    GB_REQUIRE(mode != WS_GLU_BF16 || N % 16 == 0, "gb_gemm_stream: the gated mode needs N to be a multiple of 16");
    if (M == 0) return 0;
    const int nt = M <= 8 ? 1 : M <= 16 ? 2 : M <= 32 ? 4 : 8;
    const bool glu = mode == WS_GLU_BF16;
#define GB_WS(NTT)                                                                                         \
    return glu ? launch_stream<NTT, true>(x, w, c, mode, M, N, K, ldx, ldw, ldc, N, stream)                 \
               : launch_stream<NTT, false>(x, w, c, mode, M, N, K, ldx, ldw, ldc, 0, stream);
    if (nt == 1) { GB_WS(1) }
    if (nt == 2) { GB_WS(2) }
    if (nt == 4) { GB_WS(4) }
    GB_WS(8)
#undef GB_WS
}
