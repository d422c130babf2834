// C[M, N] (+)= A[M, K] * W[N, K]^T on the CUDA cores with float32 FMA only.
//
// This is the true 32-bit matrix product (no TF32, no tensor cores) and also the generic
// fallback for any mix of float32 / bfloat16 operands at any size. Two kernels:
//   * a 64x64x16 register-tiled kernel for M > 8,
//   * a weight-streaming kernel for M <= 8 (one warp per output column), which is what a
//     decode step needs: every weight is read once, coalesced along K.
// Each output element is reduced over K in an order that depends only on K (and on which of
// the two kernels runs), never on M or on the element's place in the batch.
// Row-major [out, in] weights as in crates/glassbox-core/src/kernels.rs:381, 586-655.
#include "common.cuh"

enum { OUT_STORE = 0, OUT_ACCUMULATE = 1 };

template <typename T> struct Vec4Load;
template <> struct Vec4Load<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
};
template <> struct Vec4Load<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
        uint2 t = *reinterpret_cast<const uint2*>(p);
        __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&t.x);
        __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&t.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    }
};

template <typename TC>
__device__ __forceinline__ void store_out(TC* c, float v, int mode) {
    if (mode == OUT_ACCUMULATE) *c = gb_from_float<TC>(gb_to_float(*c) + v);
    else *c = gb_from_float<TC>(v);
}

// ------------------------------------------------------------------------------- tiled kernel
constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TW, typename TC, bool VEC>
__global__ void __launch_bounds__(256) gemm_tiled_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                         TC* __restrict__ C, int M, int N, int K, long long lda,
                                                         long long ldw, long long ldc, int mode) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;  // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    const int lr = tid / 4;        // 0..63: tile row this thread loads
    const int lk = (tid % 4) * 4;  // 0,4,8,12: first k of its 4 elements
    for (int k0 = 0; k0 < K; k0 += BK) {
        float a[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
        int gm = m0 + lr, gn = n0 + lr, gk = k0 + lk;
        if (gm < M) {
            const TA* p = A + (size_t)gm * lda + gk;
            if (VEC && gk + 3 < K) Vec4Load<TA>::load(p, a);
            else
#pragma unroll
                for (int e = 0; e < 4; ++e) if (gk + e < K) a[e] = gb_to_float(p[e]);
        }
        if (gn < N) {
            const TW* p = W + (size_t)gn * ldw + gk;
            if (VEC && gk + 3 < K) Vec4Load<TW>::load(p, w);
            else
#pragma unroll
                for (int e = 0; e < 4; ++e) if (gk + e < K) w[e] = gb_to_float(p[e]);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            As[lk + e][lr] = a[e];
            Ws[lk + e][lr] = w[e];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int gn = n0 + tx * 4 + j;
            if (gn < N) store_out<TC>(C + (size_t)gm * ldc + gn, acc[i][j], mode);
        }
    }
}

// ------------------------------------------------------------------- weight-streaming kernel
// One warp per output column n. Lanes stride over K four elements at a time; up to 8 rows of A
// are reduced against the same weight row, so the weight matrix is read exactly once.
template <typename TA, typename TW, typename TC, bool VEC>
__global__ void __launch_bounds__(256) gemm_skinny_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                          TC* __restrict__ C, int M, int N, int K, long long lda,
                                                          long long ldw, long long ldc, int mode) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + warp;
    if (n >= N) return;
    float acc[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) acc[m] = 0.f;
    const TW* wrow = W + (size_t)n * ldw;
    for (int k = lane * 4; k < K; k += 128) {
        float w[4] = {0.f, 0.f, 0.f, 0.f};
        if (VEC && k + 3 < K) Vec4Load<TW>::load(wrow + k, w);
        else
#pragma unroll
            for (int e = 0; e < 4; ++e) if (k + e < K) w[e] = gb_to_float(wrow[k + e]);
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            if (m < M) {
                float a[4] = {0.f, 0.f, 0.f, 0.f};
                const TA* arow = A + (size_t)m * lda + k;
                if (VEC && k + 3 < K) Vec4Load<TA>::load(arow, a);
                else
#pragma unroll
                    for (int e = 0; e < 4; ++e) if (k + e < K) a[e] = gb_to_float(arow[e]);
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[m] = fmaf(a[e], w[e], acc[m]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        if (m < M) {
            float v = gb_warp_sum(acc[m]);
            if (lane == 0) store_out<TC>(C + (size_t)m * ldc + n, v, mode);
        }
    }
}

template <typename TA, typename TW, typename TC>
static int launch_gemm(const void* a, const void* w, void* c, int M, int N, int K, long long lda, long long ldw,
                       long long ldc, int mode, cudaStream_t stream) {
    bool vec = (K % 4 == 0) && (lda % 4 == 0) && (ldw % 4 == 0) && ((uintptr_t)a % 16 == 0) &&
               ((uintptr_t)w % 16 == 0);
    const TA* A = (const TA*)a;
    const TW* W = (const TW*)w;
    TC* C = (TC*)c;
    if (M <= 8) {
        int warps = 8;
        dim3 grid(gb_ceil_div(N, warps));
        if (vec) gemm_skinny_kernel<TA, TW, TC, true><<<grid, warps * 32, 0, stream>>>(A, W, C, M, N, K, lda, ldw, ldc, mode);
        else gemm_skinny_kernel<TA, TW, TC, false><<<grid, warps * 32, 0, stream>>>(A, W, C, M, N, K, lda, ldw, ldc, mode);
    } else {
        dim3 grid(gb_ceil_div(N, BN), gb_ceil_div(M, BM));
        if (vec) gemm_tiled_kernel<TA, TW, TC, true><<<grid, 256, 0, stream>>>(A, W, C, M, N, K, lda, ldw, ldc, mode);
        else gemm_tiled_kernel<TA, TW, TC, false><<<grid, 256, 0, stream>>>(A, W, C, M, N, K, lda, ldw, ldc, mode);
    }
    return gb_check_launch("gb_gemm_simt");
}

// C dtype float32 with accumulate=1 adds into C (the residual stream); otherwise C is stored.
GB_EXPORT int gb_gemm_simt(const void* a, int a_dtype, const void* w, int w_dtype, void* c, int c_dtype,
                           int accumulate, int M, int N, int K, long long lda, long long ldw, long long ldc,
                           cudaStream_t stream) {
    GB_REQUIRE(M >= 0 && N > 0 && K > 0, "gb_gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
    GB_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gb_gemm_simt: a leading dimension is smaller than its row");
    GB_REQUIRE(!accumulate || c_dtype == GB_F32, "gb_gemm_simt: accumulation needs a float32 output");
    if (M == 0) return 0;
    int mode = accumulate ? OUT_ACCUMULATE : OUT_STORE;
#define GB_CASE(TA_, ta, TW_, tw, TC_, tc)                                                              \
    if (a_dtype == ta && w_dtype == tw && c_dtype == tc)                                                \
        return launch_gemm<TA_, TW_, TC_>(a, w, c, M, N, K, lda, ldw, ldc, mode, stream);
    GB_CASE(float, GB_F32, float, GB_F32, float, GB_F32)
    GB_CASE(__nv_bfloat16, GB_BF16, __nv_bfloat16, GB_BF16, __nv_bfloat16, GB_BF16)
    GB_CASE(__nv_bfloat16, GB_BF16, __nv_bfloat16, GB_BF16, float, GB_F32)
    GB_CASE(__nv_bfloat16, GB_BF16, float, GB_F32, __nv_bfloat16, GB_BF16)
    GB_CASE(__nv_bfloat16, GB_BF16, float, GB_F32, float, GB_F32)
    GB_CASE(float, GB_F32, __nv_bfloat16, GB_BF16, float, GB_F32)
#undef GB_CASE
    GB_REQUIRE(false, "gb_gemm_simt: unsupported dtype combination a=%d w=%d c=%d", a_dtype, w_dtype, c_dtype);
}
