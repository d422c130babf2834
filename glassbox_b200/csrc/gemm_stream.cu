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
#include "gemm_stream_body.cuh"

// (The one-strip variant with wide chunks is held to 128 registers, four blocks per SM: its choice of cluster size
// counts on that. The others leave the register count to the compiler: naming a minimum of one block per SM makes it
// spend 20 to 80 registers more per thread, which costs the large matrices a resident block per SM and a fifth of
// their bandwidth: 16384 x 2048 gated at one row 20.2 us against 14.2 us.)
template <int NT, bool PAIR, int KC>
__global__ void __launch_bounds__(128, (NT == 1 && !PAIR && KC == 512) ? 4 : 0) gemm_stream_kernel(const StreamArgs a) {
    __shared__ __align__(16) unsigned char xs[gemm_stream_smem_bytes<NT, KC>()];
    __shared__ float srow[NT * 8];
    GbPdlSync sync;
    gemm_stream_body<NT, PAIR, KC, false>(a, (int)blockIdx.x, xs, srow, sync);
}

// The same product with the rows in groups of eight along the grid's second dimension: block (x, y) does what block x of
// the one-group kernel does, for rows 8y .. 8y+7 only. Every group reads the weights again (from L2, after the first),
// so this is for small matrices, where a launch is a matter of latency and the eight-row variant is the fast one:
// at SmolLM2-135M shapes the four products of a layer take 11.6 us for 8 rows, 18.3 us for 16 rows in one group.
template <bool PAIR, int KC>
__global__ void __launch_bounds__(128, (!PAIR && KC == 512) ? 4 : 0) gemm_stream_rows_kernel(const StreamArgs a) {
    __shared__ __align__(16) unsigned char xs[gemm_stream_smem_bytes<1, KC>()];
    __shared__ float srow[8];
    StreamArgs b = a;
    const int r0 = (int)blockIdx.y * 8;
    b.M = min(8, a.M - r0);
    if (a.X != nullptr) b.X = a.X + (size_t)r0 * a.ldx;
    if (a.xres != nullptr) b.xres = a.xres + (size_t)r0 * a.ldr;
    const bool c32 = a.mode == WS_STORE_F32 || a.mode == WS_ADD_F32;
    b.C = c32 ? (void*)(reinterpret_cast<float*>(a.C) + (size_t)r0 * a.ldc) : (void*)(reinterpret_cast<__nv_bfloat16*>(a.C) + (size_t)r0 * a.ldc);
    if (a.positions != nullptr) b.positions = a.positions + r0;
    if (a.slots != nullptr) b.slots = a.slots + r0;
    GbPdlSync sync;
    gemm_stream_body<1, PAIR, KC, false>(b, (int)blockIdx.x, xs, srow, sync);
}

template <int NT, bool PAIR, int KC>
static int launch_stream(const StreamArgs& a, int strips, int split, int pdl, cudaStream_t stream, int groups = 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(strips * split, groups);
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
    cudaError_t e;
    if constexpr (NT == 1) {
        e = groups > 1 ? cudaLaunchKernelEx(&cfg, gemm_stream_rows_kernel<PAIR, KC>, a) : cudaLaunchKernelEx(&cfg, gemm_stream_kernel<NT, PAIR, KC>, a);
    } else {
        e = cudaLaunchKernelEx(&cfg, gemm_stream_kernel<NT, PAIR, KC>, a);
    }
    if (e != cudaSuccess) {
        gb_set_error("gb_gemm_stream: launch failed: %s", cudaGetErrorString(e));
        return 2;
    }
    return gb_check_launch("gb_gemm_stream");
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
#define GB_SL(NTT) return pair ? (kc == 640 ? stream_slots<NTT, true, 640>() : kc == 512 ? stream_slots<NTT, true, 512>() : stream_slots<NTT, true, 256>()) \
                               : (kc == 640 ? stream_slots<NTT, false, 640>() : kc == 512 ? stream_slots<NTT, false, 512>() : stream_slots<NTT, false, 256>());
    if (nt == 1) { GB_SL(1) }
    if (nt == 2) { GB_SL(2) }
    if (nt == 4) { return pair ? (kc == 512 ? stream_slots<4, true, 512>() : stream_slots<4, true, 256>())
                               : (kc == 512 ? stream_slots<4, false, 512>() : stream_slots<4, false, 256>()); }
    return pair ? stream_slots<8, true, 256>() : stream_slots<8, false, 256>();
#undef GB_SL
}

// Rows in groups of eight (see gemm_stream_rows_kernel): the number of groups, or 1 where one group takes all rows.
// Taken when the weights, read once per group, stay within a budget that L2 serves easily.
constexpr long long WS_GROUPED_WEIGHT_BYTES = 40ll << 20;
static int stream_row_groups(int M, int N, int K, bool pair) {
    const int groups = (M + 7) / 8;
    const long long weight_bytes = (long long)N * (pair ? 2 : 1) * K * 2;
    return (groups > 1 && weight_bytes * groups <= WS_GROUPED_WEIGHT_BYTES) ? groups : 1;
}

GB_EXPORT int gb_gemm_stream_row_groups(int M, int N, int K, int pair) { return stream_row_groups(M, N, K, pair != 0); }

static int dispatch_stream(StreamArgs a, int strips, bool pair, int pdl, cudaStream_t stream) {
    const int groups = stream_row_groups(a.M, a.mode == WS_ROPE_QKV ? a.N / 2 : a.N, a.K, pair);
    const int nt = groups > 1 ? 1 : a.M <= 8 ? 1 : a.M <= 16 ? 2 : a.M <= 32 ? 4 : 8;
    // The wide chunk keeps twice the loads in flight per thread, at twice the registers: it is taken
    // where its blocks still fit the chip in one wave (and never by the variants with many rows, which
    // have neither the registers nor the shared memory for it). A K just above 512 (576: SmolLM2-135M)
    // would leave a second chunk of a few columns that costs a whole round of staging and barriers: with at
    // most 16 rows such a K goes through as one chunk of 640.
    const bool wide_fits = nt <= (pair ? 2 : 4);
    const int blocks = strips * groups;   // per block of a cluster
    int kc = (wide_fits && blocks <= slots_of(nt, pair, 512)) ? 512 : 256;
    // (a launch of several row groups takes the one-round chunk even where its blocks then come in more than one wave:
    // 135M shapes, 64 rows, the four products of a layer: 24.9 -> 21.3 us)
    if (nt <= 2 && a.K > 512 && a.K <= 640 && (groups > 1 || (kc == 512 && blocks <= slots_of(nt, pair, 640)))) kc = 640;
    // Cluster size: one block per chunk, rounded up to a power of two, as long as all blocks are on the
    // chip at once and the other ranks' sums fit the first block's activation tile. Chunk and cluster
    // size depend on the matrix and on the row bucket (8, 16, 32, 64), not on which rows are in the batch.
    const int max_split = (kc + 32) / 32 / (pair ? 2 : 1) + 1;   // (split - 1) * sets * 32 <= kc + 32
    const int slots = slots_of(nt, pair, kc);
    int split = 1;
    // (with at most 16 rows a block should see one chunk: a second round of staging costs more than the cluster's
    // two barriers; with more rows the rounds carry real work and one block per 512 k is enough)
    while (split < 8 && (nt <= 2 ? split * kc < a.K : split < a.K / 512)) split *= 2;
    while (split > 1 && (split > max_split || blocks * split > slots)) split /= 2;
    a.kslice = split == 1 ? a.K : ((a.K + split - 1) / split + kc - 1) / kc * kc;
    // When the next kernel in the stream is let go: a launch without clusters only after its own wait (released at the
    // very start, kernels pile up two and three deep on the SMs, resident and waiting, in the way of the one that
    // works: 135M decode step at batch 8 0.767 -> 0.742 ms); a launch of clusters at its start, as before (its
    // successor is as a rule one too, and clusters take longer to place: 360M at batch 8, 1.20 ms against 1.26 ms).
    a.late_release = split == 1;
#define GB_WS2(NTT, KCC) return pair ? launch_stream<NTT, true, KCC>(a, strips, split, pdl, stream, groups) : launch_stream<NTT, false, KCC>(a, strips, split, pdl, stream, groups);
#define GB_WS(NTT) if (kc == 512) { GB_WS2(NTT, 512) } else { GB_WS2(NTT, 256) }
#define GB_WS3(NTT) if (kc == 640) { GB_WS2(NTT, 640) } else GB_WS(NTT)
    if (nt == 1) { GB_WS3(1) }
    if (nt == 2) { GB_WS3(2) }
    if (nt == 4) { GB_WS(4) }
    GB_WS2(8, 256)
#undef GB_WS3
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
