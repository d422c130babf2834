// A decode step's chain of small kernels as ONE persistent kernel that runs a *program*.
//
// Decoding a few rows through a small model is a chain of dependent kernels of a few microseconds each (five per
// layer: norm+QKV+rotation+cache write, attention, O projection, norm+gate/up+SwiGLU, down projection), each moving
// a megabyte or so: the step is bound by launch gaps, ramp-up and tails, not by bytes. Here the blocks stay
// resident for the whole chain. The host writes the chain down as an array of operations (a weight-streaming
// product with its folded-in prologue and epilogue, or a split-key decode attention: the very bodies the
// stand-alone kernels run, gemm_stream_body.cuh and attention_decode_mma_body.cuh), and a kernel walks the array.
// Two kernels do, and they differ in who shares an operation and how they wait for each other:
//
//  * by rows (decode_program_cluster_kernel): the rows of a decode step never read each other's activations, so a
//    group of rows (one row, with few rows) is given to one thread-block cluster, which runs the whole program for
//    it: every block of the cluster takes its share of each operation's virtual blocks, for the cluster's rows only,
//    and the cluster's hardware barrier (arrive.release / wait.acquire) stands between operations. Clusters never
//    wait for each other, so nothing has to be resident together and nothing can deadlock. Each cluster reads all the
//    weights; the first reads them from HBM, the others find them in L2.
//  * by operations (decode_program_grid_kernel): all resident blocks share every operation, for all rows, and meet
//    at a barrier in global memory. The launch is cooperative (all blocks resident, or the launch fails). Every wait
//    at that barrier is bounded by clock64: a block that waits too long records GB_STATUS_WAIT_TIMEOUT in the status
//    word and returns, and every other block sees that bit at its next look and returns too; nothing spins for ever
//    and nothing traps.
//
// In both, a barrier is split in two: a block arrives when its share of an operation is done, starts on the next
// operation with what does not depend on other blocks (it requests its first weights), and only then waits, at the
// point where the stand-alone kernel would wait for its predecessor in the stream.
// Loads come from this GPU's own memory only; blocks of a cluster exchange nothing through each other's shared
// memory and no load is multicast.
//
// The program knows nothing about models: parts call the same kernels.* functions as ever, and while a program is
// being recorded those calls append operations instead of launching (glassbox_b200/kernels.py).
#include "attention_decode_mma_body.cuh"
#include "gemm_stream_body.cuh"

enum { OP_GEMM = 1, OP_ATTENTION = 2 };

struct ProgramOp {
    int kind;
    int vblocks;   // virtual blocks: strips (or strip pairs) of a product; splits x kv heads x rows of an attention
    int pair;      // product: a block owns a pair of strips (gated, rotary QKV)
    int reserved;
    StreamArgs gemm;
    DecodeAttnArgs attn;
};

constexpr long long PROGRAM_WAIT_CYCLES = 4000000000ll;   // about two seconds: far beyond any step, short of a hang

struct ProgramSmem {
    ProgramOp op;
    int go;
};

// ------------------------------------------------------------------------------------ waiting, two ways
// The barrier in global memory of the grid kernel, split in two. arrive(): this block's share of the operation is
// done. wait(): every block's is (barrier number `index`: the one behind operation index - 1; 0 = nothing to wait
// for). A wait that is given up sets `failed`; the caller returns.
struct GridSync {
    unsigned* counter;
    int* status;
    int* go;
    unsigned arrivals, index;
    long long wait_cycles;
    bool waited, failed;

    __device__ __forceinline__ void start() {}
    __device__ __forceinline__ void arrive() {
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
        }
    }
    __device__ __forceinline__ void wait() {
        if (waited) return;
        waited = true;
        if (index == 0) return;
        if (threadIdx.x == 0) {
            const unsigned target = index * arrivals;
            const long long t0 = clock64();
            int ok = 1;
            unsigned polls = 0;
            for (;;) {
                unsigned seen;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
                if (seen >= target) break;
                if ((++polls & 31u) == 0) {
                    int st;
                    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(st) : "l"(status) : "memory");
                    if ((st & GB_STATUS_WAIT_TIMEOUT) || clock64() - t0 > wait_cycles) {
                        atomicOr(status, GB_STATUS_WAIT_TIMEOUT);
                        ok = 0;
                        break;
                    }
                }
            }
            __threadfence();
            *go = ok;
        }
        __syncthreads();
        if (*go == 0) failed = true;
    }
    __device__ __forceinline__ bool gave_up() const { return failed; }
    __device__ __forceinline__ int thread() const { return (int)threadIdx.x; }
    __device__ __forceinline__ void group_barrier() { __syncthreads(); }
};

// The hardware barrier of a thread-block cluster, split in two, for blocks in which every 128
// threads (a group) work on a virtual block of their own.
struct RowsSync {
    bool waited;
    int group, group_thread;
    __device__ __forceinline__ void start() {}
    __device__ __forceinline__ void arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
    __device__ __forceinline__ void wait() {
        if (waited) return;
        waited = true;
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    __device__ __forceinline__ bool gave_up() const { return false; }
    __device__ __forceinline__ int thread() const { return group_thread; }
    __device__ __forceinline__ void group_barrier() { asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory"); }
};

// The share of block `b` of `nb` in bringing the keys and values that an attention operation will read into L2.
__device__ __forceinline__ void attention_prefetch(const DecodeAttnArgs& a, int b, int nb, int row0, int nrows) {
    const int lines = (a.page_size * a.hd * 2) / 128;   // 128-byte lines per (page, kv head) tile
    if (lines <= 0) return;
    for (int row = row0; row < row0 + nrows; ++row) {
        const int pos = a.positions[row];
        if (pos < 0 || (pos >> a.page_shift) >= a.max_pages) continue;
        const int* table = a.block_tables + (size_t)a.row_seq[row] * a.max_pages;
        const int first = (a.window > 0 && pos + 1 > a.window) ? pos + 1 - a.window : 0;
        const int page_lo = first >> a.page_shift, page_hi = pos >> a.page_shift;
        const int tiles = (page_hi - page_lo + 1) * a.nkv;
        // one thread per (page, kv head) tile, walking its lines: no division in the inner loop
        for (int tile = b * (int)blockDim.x + (int)threadIdx.x; tile < tiles; tile += nb * (int)blockDim.x) {
            const long long page = table[page_lo + tile / a.nkv];
            if (page < 0 || page >= a.num_pages) continue;
            const long long off = ((page * a.nkv + tile % a.nkv) * (long long)a.page_size * a.hd) * 2;
            for (int line = 0; line < lines; ++line) {
                asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const unsigned char*>(a.kcache) + off + line * 128));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const unsigned char*>(a.vcache) + off + line * 128));
            }
        }
    }
}

// The bodies are called, not inlined: each keeps the register allocation it has as a kernel of its own instead of
// sharing one with everything else that is live in the operation loop.
template <int NT, bool PAIR, class Sync>
__device__ __noinline__ void program_gemm(const StreamArgs& a, int vb, void* xs, float* srow, Sync& sync) {
    gemm_stream_body<NT, PAIR, 512, true>(a, vb, xs, srow, sync);
}

template <int HD, int BK, class Sync>
__device__ __noinline__ void program_attention(const DecodeAttnArgs& a, int split, int kvh, int row, DecodeAttnSmem& sm, Sync& sync) {
    attention_decode_mma_body<HD, BK>(a, split, kvh, row, sm, sync);
}

__device__ __forceinline__ void load_op(ProgramSmem& ps, const ProgramOp* ops, int i) {
    const int* src = reinterpret_cast<const int*>(ops + i);
    int* dst = reinterpret_cast<int*>(&ps.op);
    for (int w = threadIdx.x; w < (int)(sizeof(ProgramOp) / sizeof(int)); w += blockDim.x) dst[w] = src[w];
}

// ----------------------------------------------------------------------------------------- by operations
// NT: row bucket of every product of the program (1: up to 8 rows, 2: up to 16). HD, BK: head size and keys per warp
// iteration of every attention of the program (HD 0: the program has no attention). `arrivals` is the number of
// blocks each barrier waits for: the grid size (a test passes more, so that the wait runs out); `wait_cycles` bounds
// each wait. With a trace buffer ([2, n_ops, 4] clock64 values) the first and the last block note, for every
// operation, when they started it, had issued their hints, had done their share, and had arrived at the barrier.
template <int NT, int HD, int BK>
__global__ void __launch_bounds__(128) decode_program_grid_kernel(const ProgramOp* __restrict__ ops, int n_ops,
                                                                  unsigned* __restrict__ barrier, int* __restrict__ status,
                                                                  unsigned arrivals, long long wait_cycles,
                                                                  long long* __restrict__ trace) {
    __shared__ __align__(16) unsigned char xs[gemm_stream_smem_bytes<NT, 512>()];
    __shared__ float srow[NT * 8];
    __shared__ DecodeAttnSmem attn_sm;
    __shared__ ProgramSmem ps;
    const int tid = threadIdx.x, nb = (int)gridDim.x, b = (int)blockIdx.x;
    const int traced = (trace != nullptr && tid == 0) ? (b == 0 ? 0 : (b == nb - 1 ? 1 : -1)) : -1;
    auto mark = [&](int i, int what) {
        if (traced >= 0) trace[((size_t)traced * n_ops + i) * 4 + what] = clock64();
    };
    GridSync sync;
    sync.counter = barrier; sync.status = status; sync.go = &ps.go; sync.arrivals = arrivals; sync.wait_cycles = wait_cycles;
    sync.failed = false;
    for (int i = 0; i < n_ops; ++i) {
        __syncthreads();
        mark(i, 0);
        load_op(ps, ops, i);
        __syncthreads();
        if (i + 1 < n_ops && ops[i + 1].kind == OP_ATTENTION)   // the keys and values of the attention behind this operation
            attention_prefetch(ops[i + 1].attn, b, nb, 0, ops[i + 1].attn.n);
        mark(i, 1);
        sync.index = (unsigned)i;
        sync.waited = false;
        const int kind = ps.op.kind, vblocks = ps.op.vblocks;
        if (kind == OP_GEMM) {
            const bool pair = ps.op.pair != 0;
            for (int vb = b; vb < vblocks && !sync.failed; vb += nb) {
                __syncthreads();
                if (pair) program_gemm<NT, true>(ps.op.gemm, vb, xs, srow, sync);
                else program_gemm<NT, false>(ps.op.gemm, vb, xs, srow, sync);
            }
        } else if (kind == OP_ATTENTION) {
            if constexpr (HD > 0) {
                const int splits = ps.op.attn.splits, nkv = ps.op.attn.nkv;
                for (int vb = b; vb < vblocks && !sync.failed; vb += nb) {
                    __syncthreads();
                    const int split = vb % splits, rest = vb / splits;
                    program_attention<HD, BK>(ps.op.attn, split, rest % nkv, rest / nkv, attn_sm, sync);
                }
            }
        }
        sync.wait();             // a block without a share of this operation still has to see the barrier before it
        if (sync.failed) return;
        mark(i, 2);
        if (i + 1 < n_ops) sync.arrive();
        mark(i, 3);
    }
}

// ------------------------------------------------------------------------------------------------ by rows
// One cluster of blocks of 256 threads runs the whole program for rows [cluster * R, ...). The rows of a decode step
// never read each other's activations, so the cluster's own barrier is all the waiting there is. A product is done
// the plain way for so few rows: a warp owns output features (or pairs of them, where the epilogue needs two: gate
// and up, the two halves of a rotated head), streams their weight rows in 16-byte pieces (one piece of 1,024 k ahead
// of the arithmetic, the very first before the wait for the operation before), multiplies with the activation
// row(s) held in shared memory in float32, and adds up with shuffles. Sums are float32 throughout; what the stand-alone
// kernel rounds to bfloat16 on the way in (the normalised activations) is rounded here too.
constexpr int ROWS_THREADS = 256, ROWS_WARPS = 8, ROWS_GROUPS = 2;   // (255 registers a thread: the bodies need them)
constexpr int ROWS_KC = 1024;   // k per piece: four 16-byte loads per lane and weight row

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// bfloat16 pair in a 32-bit word -> two floats (a bfloat16 is the upper half of a float)
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// acc += dot(8 bfloat16 weights in w, 8 floats x0 x1)
__device__ __forceinline__ float dot8(const uint4 w, const float4 x0, const float4 x1, float acc) {
    acc = fmaf(bf16_lo(w.x), x0.x, acc); acc = fmaf(bf16_hi(w.x), x0.y, acc);
    acc = fmaf(bf16_lo(w.y), x0.z, acc); acc = fmaf(bf16_hi(w.y), x0.w, acc);
    acc = fmaf(bf16_lo(w.z), x1.x, acc); acc = fmaf(bf16_hi(w.z), x1.y, acc);
    acc = fmaf(bf16_lo(w.w), x1.z, acc); acc = fmaf(bf16_hi(w.w), x1.w, acc);
    return acc;
}

// R: rows the cluster holds (1 or 2). xs: [R][K] floats; red: [R][ROWS_WARPS] floats.
template <int R>
__device__ __forceinline__ void rows_product(const StreamArgs& a, float* xs, float* red, const int row0, const int nrows,
                                             const int gwarp, const int nwarps, RowsSync& sync) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = a.K, mode = a.mode;
    const bool pair = mode == WS_GLU_BF16 || mode == WS_ROPE_QKV;
    const int half = a.hd / 2;
    const int units = mode == WS_ROPE_QKV ? (a.nh + 2 * a.nkv) * half : a.N;
    const int pieces = (K + ROWS_KC - 1) / ROWS_KC;
    auto rows_of = [&](int u, int& ra, int& rb) {
        if (mode == WS_ROPE_QKV) {
            ra = (u / half) * a.hd + u % half;
            rb = ra + half;
        } else {
            ra = u;
            rb = u + a.N;   // (gated: the up row)
        }
    };
    uint4 cur[2][4], nxt[2][4];
    auto fetch = [&](int u, int c, uint4 (&buf)[2][4]) {
        int ra, rb;
        rows_of(u, ra, rb);
        const __nv_bfloat16* wa = a.W + (size_t)ra * a.ldw;
        const __nv_bfloat16* wb = a.W + (size_t)rb * a.ldw;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = c * ROWS_KC + j * 256 + lane * 8;
            buf[0][j] = k < K ? ldg_stream(wa + k) : make_uint4(0, 0, 0, 0);
            if (pair) buf[1][j] = k < K ? ldg_stream(wb + k) : make_uint4(0, 0, 0, 0);
        }
    };
    int u = gwarp, c = 0;
    if (u < units) fetch(u, 0, cur);      // weights do not depend on the operation before
    sync.wait();                          // ... the activations do

    // ---- the cluster's activation rows into shared memory, as float32
    if (a.X != nullptr) {
        for (int idx = tid * 8; idx < nrows * K; idx += ROWS_THREADS * 8) {
            const int r = idx / K, k = idx - r * K;
            const uint4 v = __ldcg(reinterpret_cast<const uint4*>(a.X + (size_t)(row0 + r) * a.ldx + k));
            float4* dst = reinterpret_cast<float4*>(xs + (size_t)r * K + k);
            dst[0] = make_float4(bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y));
            dst[1] = make_float4(bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w));
        }
    } else {   // RMSNorm on the way in: gain * (x * s), rounded to bfloat16 as the separate norm kernel writes it
        float ss[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            ss[r] = 0.f;
            if (r < nrows) {
                const float* xr = a.xres + (size_t)(row0 + r) * a.ldr;
                for (int k = tid * 4; k < K; k += ROWS_THREADS * 4) {
                    const float4 v = __ldcg(reinterpret_cast<const float4*>(xr + k));
                    ss[r] = fmaf(v.x, v.x, ss[r]); ss[r] = fmaf(v.y, v.y, ss[r]);
                    ss[r] = fmaf(v.z, v.z, ss[r]); ss[r] = fmaf(v.w, v.w, ss[r]);
                }
            }
            ss[r] = gb_warp_sum(ss[r]);
            if (lane == 0) red[r * ROWS_WARPS + warp] = ss[r];
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (r >= nrows) continue;
            float tot = 0.f;
#pragma unroll
            for (int w = 0; w < ROWS_WARPS; ++w) tot += red[r * ROWS_WARPS + w];
            const float sc = 1.0f / sqrtf(tot / (float)K + a.eps);
            const float* xr = a.xres + (size_t)(row0 + r) * a.ldr;
            for (int k = tid * 4; k < K; k += ROWS_THREADS * 4) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(xr + k));
                const float4 g = *reinterpret_cast<const float4*>(a.gain + k);
                *reinterpret_cast<float4*>(xs + (size_t)r * K + k) =
                    make_float4(bf16_round(g.x * (v.x * sc)), bf16_round(g.y * (v.y * sc)), bf16_round(g.z * (v.z * sc)),
                                bf16_round(g.w * (v.w * sc)));
            }
        }
    }
    __syncthreads();

    // ---- this warp's output features: two register sets of weights take turns, one in flight while the other is used
    float acc[2][R];
#pragma unroll
    for (int s2 = 0; s2 < 2; ++s2)
#pragma unroll
        for (int r = 0; r < R; ++r) acc[s2][r] = 0.f;
    auto use = [&](const int uu, const int cc, const uint4 (&buf)[2][4]) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = cc * ROWS_KC + j * 256 + lane * 8;
            if (k < K) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    if (r >= nrows) continue;
                    const float4 x0 = *reinterpret_cast<const float4*>(xs + (size_t)r * K + k);
                    const float4 x1 = *reinterpret_cast<const float4*>(xs + (size_t)r * K + k + 4);
                    acc[0][r] = dot8(buf[0][j], x0, x1, acc[0][r]);
                    if (pair) acc[1][r] = dot8(buf[1][j], x0, x1, acc[1][r]);
                }
            }
        }
        if (cc != pieces - 1) return;
        // the feature's last piece: add up over the lanes, then lane r finishes row r
        float mine0 = 0.f, mine1 = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float s0 = gb_warp_sum(acc[0][r]);
            const float s1 = pair ? gb_warp_sum(acc[1][r]) : 0.f;
            if (lane == r) {
                mine0 = s0;
                mine1 = s1;
            }
            acc[0][r] = 0.f;
            acc[1][r] = 0.f;
        }
        if (lane >= nrows) return;
        const int tok = row0 + lane;
        if (mode == WS_ROPE_QKV) {
            const int pos = a.positions[tok];
            if (pos < 0) return;   // a padding row
            const int head = uu / half, i = uu % half;
            float y0 = mine0, y1 = mine1;
            if (head < a.nh + a.nkv && a.rope != nullptr) {
                if (pos >= a.max_pos) {
                    atomicOr(a.status, GB_STATUS_BAD_POSITION);
                } else {
                    const float2 cs = a.rope[(size_t)pos * half + i];
                    y0 = mine0 * cs.x - mine1 * cs.y;
                    y1 = mine1 * cs.x + mine0 * cs.y;
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
        } else if (mode == WS_GLU_BF16) {
            reinterpret_cast<__nv_bfloat16*>(a.C)[(size_t)tok * a.ldc + uu] = __float2bfloat16_rn(mine0 / (1.0f + __expf(-mine0)) * mine1);
        } else if (mode == WS_STORE_BF16) {
            reinterpret_cast<__nv_bfloat16*>(a.C)[(size_t)tok * a.ldc + uu] = __float2bfloat16_rn(mine0);
        } else if (mode == WS_STORE_F32) {
            reinterpret_cast<float*>(a.C)[(size_t)tok * a.ldc + uu] = mine0;
        } else {
            float* p = reinterpret_cast<float*>(a.C) + (size_t)tok * a.ldc + uu;
            __stcg(p, __ldcg(p) + mine0);
        }
    };
    auto step = [&](int& uu, int& cc) {   // the piece after (uu, cc) in this warp's order
        if (++cc >= pieces) {
            cc = 0;
            uu += nwarps;
        }
    };
    while (u < units) {
        int u1 = u, c1 = c;
        step(u1, c1);
        if (u1 < units) fetch(u1, c1, nxt);
        use(u, c, cur);
        if (u1 >= units) break;
        u = u1; c = c1;
        step(u, c);
        if (u < units) fetch(u, c, cur);
        use(u1, c1, nxt);
    }
}

template <int HD, int BK>
__device__ __noinline__ void rows_attention(const DecodeAttnArgs& a, int split, int kvh, int row, DecodeAttnSmem& sm, RowsSync& sync) {
    attention_decode_mma_body<HD, BK>(a, split, kvh, row, sm, sync);
}

// Dynamic shared memory: the attention groups' scratch, then R * (longest K of the program) floats. With a trace buffer ([2, n_ops, 4] clock64
// values) the first and the last block of the first cluster note, for every operation, when they started it, had its
// description, had done their share (and seen the barrier before it), and had arrived at the barrier behind it.
template <int R, int HD, int BK>
__global__ void __launch_bounds__(ROWS_THREADS, 1) decode_program_rows_kernel(const ProgramOp* __restrict__ ops, int n_ops,
                                                                              int total_rows, long long* __restrict__ trace) {
    extern __shared__ __align__(16) unsigned char dyn[];   // [ROWS_GROUPS] DecodeAttnSmem, then the activation rows
    DecodeAttnSmem* attn_sm = reinterpret_cast<DecodeAttnSmem*>(dyn);
    static_assert(sizeof(DecodeAttnSmem) % 16 == 0, "the activation rows behind the attention scratch are read 16 bytes at a time");
    float* xs_dyn = reinterpret_cast<float*>(dyn + ROWS_GROUPS * sizeof(DecodeAttnSmem));
    __shared__ float red[R * ROWS_WARPS];
    __shared__ ProgramSmem ps;
    unsigned rank, csize, cluster;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(csize));
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(cluster));
    const int tid = threadIdx.x, warp = tid >> 5;
    const int row0 = (int)cluster * R, nrows = min(R, total_rows - row0);
    const int traced = (trace != nullptr && tid == 0 && cluster == 0) ? (rank == 0 ? 0 : (rank == csize - 1 ? 1 : -1)) : -1;
    auto mark = [&](int i, int what) {
        if (traced >= 0) trace[((size_t)traced * n_ops + i) * 4 + what] = clock64();
    };
    RowsSync sync;
    sync.group = tid >> 7;
    sync.group_thread = tid & 127;
    for (int i = 0; i < n_ops; ++i) {
        __syncthreads();
        mark(i, 0);
        load_op(ps, ops, i);
        __syncthreads();
        mark(i, 1);
        sync.waited = (i == 0);
        const int kind = ps.op.kind;
        if (kind == OP_GEMM) {
            rows_product<R>(ps.op.gemm, xs_dyn, red, row0, nrows, (int)rank * ROWS_WARPS + warp, (int)csize * ROWS_WARPS, sync);
        } else if (kind == OP_ATTENTION) {
            if constexpr (HD > 0) {
                const int splits = ps.op.attn.splits, nkv = ps.op.attn.nkv;
                const int items = nrows * splits * nkv;
                for (int vb = (int)rank * ROWS_GROUPS + sync.group; vb < items; vb += (int)csize * ROWS_GROUPS) {
                    sync.group_barrier();
                    const int split = vb % splits, rest = vb / splits;
                    rows_attention<HD, BK>(ps.op.attn, split, rest % nkv, row0 + rest / nkv, attn_sm[sync.group], sync);
                }
            }
        }
        sync.wait();   // (threads that had no share still have to pass the barrier before this operation)
        __syncthreads();
        mark(i, 2);
        if (i + 1 < n_ops) sync.arrive();
        mark(i, 3);
    }
}

// ------------------------------------------------------------------------------------------ host side
GB_EXPORT int gb_program_op_bytes() { return (int)sizeof(ProgramOp); }

GB_EXPORT int gb_program_max_rows() { return 16; }

// Whether a product with these operands can be an operation of a program (the conditions of gb_gemm_stream, at most
// 16 rows).
static int encode_common(const char* who, const void* x, const float* xres, const void* w, int M, int N, int K, long long ldx,
                         long long ldr, long long ldw) {
    GB_REQUIRE(M >= 1 && M <= 16 && N > 0 && K > 0, "%s: sizes M=%d N=%d K=%d outside a program's range (1 <= M <= 16)", who, M, N, K);
    GB_REQUIRE(K % 8 == 0 && ldw % 8 == 0 && (uintptr_t)w % 16 == 0, "%s: K and the weight row stride must be multiples of 8, the weights 16-byte aligned", who);
    if (x != nullptr)
        GB_REQUIRE(ldx % 8 == 0 && (uintptr_t)x % 16 == 0, "%s: activations must be 16-byte aligned with a row stride that is a multiple of 8", who);
    else
        GB_REQUIRE(xres != nullptr && ldr % 4 == 0 && (uintptr_t)xres % 16 == 0, "%s: float32 rows to normalise must be 16-byte aligned", who);
    return 0;
}

// Write operation `op` (host memory, gb_program_op_bytes() bytes) for the product that gb_gemm_stream would launch.
GB_EXPORT int gb_program_encode_gemm(void* op, const void* x, long long ldx, const float* xres, long long ldr, const float* gain,
                                     float eps, const void* w, long long ldw, void* c, long long ldc, int mode, int M, int N,
                                     int K) {
    if (encode_common("gb_program_encode_gemm", x, xres, w, M, N, K, ldx, ldr, ldw)) return 1;
    GB_REQUIRE(mode >= 0 && mode <= 3, "gb_program_encode_gemm: unknown mode %d", mode);
    GB_REQUIRE(mode != WS_GLU_BF16 || N % 16 == 0, "gb_program_encode_gemm: the gated mode needs N to be a multiple of 16");
    GB_REQUIRE(x != nullptr || gain != nullptr, "gb_program_encode_gemm: normalising needs a gain");
    ProgramOp* o = static_cast<ProgramOp*>(op);
    *o = ProgramOp{};
    o->kind = OP_GEMM;
    o->vblocks = (N + 15) / 16;
    o->pair = mode == WS_GLU_BF16;
    StreamArgs& a = o->gemm;
    a.X = (const __nv_bfloat16*)x; a.ldx = ldx; a.xres = xres; a.ldr = ldr; a.gain = gain; a.eps = eps;
    a.W = (const __nv_bfloat16*)w; a.ldw = ldw; a.C = c; a.ldc = ldc; a.mode = mode; a.M = M; a.N = N; a.K = K;
    a.pair_offset = mode == WS_GLU_BF16 ? N : 0;
    a.kslice = K;
    return 0;
}

// ... for the stacked QKV product with rotation and cache write that gb_gemm_stream_qkv would launch.
GB_EXPORT int gb_program_encode_gemm_qkv(void* op, const void* x, long long ldx, const float* xres, long long ldr,
                                         const float* gain, float eps, const void* w, long long ldw, void* q_out, long long ldq,
                                         int M, int K, const float* rope, int max_pos, const int* positions, const int* slots,
                                         void* kcache, void* vcache, int nh, int nkv, int hd, int page_size, long long num_pages,
                                         int write_kv, int* status) {
    const int N = (nh + 2 * nkv) * hd;
    if (encode_common("gb_program_encode_gemm_qkv", x, xres, w, M, N, K, ldx, ldr, ldw)) return 1;
    GB_REQUIRE(hd > 0 && hd % 32 == 0 && nh > 0 && nkv > 0, "gb_program_encode_gemm_qkv: head size %d must be a multiple of 32", hd);
    GB_REQUIRE(x != nullptr || gain != nullptr, "gb_program_encode_gemm_qkv: normalising needs a gain");
    GB_REQUIRE(page_size > 0 && positions && slots && status && ldq >= (long long)nh * hd, "gb_program_encode_gemm_qkv: bad arguments");
    ProgramOp* o = static_cast<ProgramOp*>(op);
    *o = ProgramOp{};
    o->kind = OP_GEMM;
    o->vblocks = (nh + 2 * nkv) * (hd / 32);
    o->pair = 1;
    StreamArgs& a = o->gemm;
    a.X = (const __nv_bfloat16*)x; a.ldx = ldx; a.xres = xres; a.ldr = ldr; a.gain = gain; a.eps = eps;
    a.W = (const __nv_bfloat16*)w; a.ldw = ldw; a.C = q_out; a.ldc = ldq; a.mode = WS_ROPE_QKV; a.M = M; a.N = N; a.K = K;
    a.pair_offset = hd / 2;
    a.rope = (const float2*)rope; a.positions = positions; a.slots = slots;
    a.kcache = (__nv_bfloat16*)kcache; a.vcache = (__nv_bfloat16*)vcache;
    a.nh = nh; a.nkv = nkv; a.hd = hd; a.page_size = page_size; a.max_pos = max_pos; a.write_kv = write_kv;
    a.num_slots = num_pages * page_size; a.status = status;
    a.kslice = K;
    return 0;
}

// ... for the decode attention that gb_attention_decode_mma_pdl would launch. block_keys 0 = the default variant.
GB_EXPORT int gb_program_encode_attention(void* op, const void* q, long long q_stride, void* out, long long out_stride,
                                          const void* kcache, const void* vcache, const int* block_tables, int max_pages,
                                          const int* row_seq, const int* positions, int n, int nh, int nkv, int hd,
                                          int page_size, long long num_pages, float scale, int window, int splits,
                                          float* part_acc, float* part_ml, int* counters, int* status, int block_keys) {
    GB_REQUIRE(hd == 16 || hd == 32 || hd == 64 || hd == 128, "gb_program_encode_attention: head size %d is not built", hd);
    GB_REQUIRE(nkv > 0 && nh % nkv == 0 && nh / nkv <= 16, "gb_program_encode_attention: %d heads per kv head are not built", nkv > 0 ? nh / nkv : 0);
    GB_REQUIRE(page_size >= 16 && (page_size & (page_size - 1)) == 0, "gb_program_encode_attention: page size %d must be a power of two >= 16", page_size);
    GB_REQUIRE((long long)num_pages * nkv * page_size < (1ll << 31), "gb_program_encode_attention: the cache has too many rows");
    GB_REQUIRE(max_pages > 0 && splits >= 1 && splits <= MMA_MAX_MERGE / 4 && part_acc && part_ml && counters && status,
               "gb_program_encode_attention: bad page geometry, split count or scratch");
    GB_REQUIRE(n >= 1 && n <= 16, "gb_program_encode_attention: %d rows are outside a program's range", n);
    GB_REQUIRE(q_stride % 4 == 0 && (uintptr_t)q % 8 == 0, "gb_program_encode_attention: q must be 8-byte aligned");
    ProgramOp* o = static_cast<ProgramOp*>(op);
    *o = ProgramOp{};
    o->kind = OP_ATTENTION;
    o->vblocks = splits * nkv * n;
    DecodeAttnArgs& a = o->attn;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride; a.out = (__nv_bfloat16*)out; a.out_stride = out_stride;
    a.kcache = (const __nv_bfloat16*)kcache; a.vcache = (const __nv_bfloat16*)vcache; a.block_tables = block_tables;
    a.max_pages = max_pages; a.row_seq = row_seq; a.positions = positions; a.nh = nh; a.nkv = nkv; a.page_size = page_size;
    a.page_shift = page_shift; a.num_pages = num_pages; a.scale = scale; a.window = window; a.splits = splits;
    a.part_acc = part_acc; a.part_ml = part_ml; a.counters = counters; a.status = status; a.n = n; a.hd = hd;
    a.block_keys = (hd == 64 && block_keys == 16) ? 16 : (hd == 128 ? 16 : 32);
    return 0;
}

static int device_sms() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    return sms;
}

template <int NT, int HD, int BK>
static int launch_grid(const ProgramOp* ops, int n_ops, int max_vblocks, unsigned* barrier, int* status, int absent,
                       long long wait_cycles, long long* trace, cudaStream_t stream) {
    auto kernel = decode_program_grid_kernel<NT, HD, BK>;
    static int capacity = 0;   // blocks of this instantiation that the chip holds at once
    if (capacity == 0) {
        int per_sm = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 128, 0);
        GB_REQUIRE(e == cudaSuccess && per_sm > 0, "gb_program_launch: cannot size the grid: %s", cudaGetErrorString(e));
        capacity = device_sms() * per_sm;
    }
    const int grid = max_vblocks < capacity ? max_vblocks : capacity;
    cudaError_t e = cudaMemsetAsync(barrier, 0, sizeof(unsigned), stream);
    GB_REQUIRE(e == cudaSuccess, "gb_program_launch: clearing the barrier failed: %s", cudaGetErrorString(e));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(128);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kernel, ops, n_ops, barrier, status, (unsigned)(grid + absent), wait_cycles, trace);
    if (e != cudaSuccess) {
        gb_set_error("gb_program_launch: launch failed: %s", cudaGetErrorString(e));
        return 2;
    }
    return gb_check_launch("gb_program_launch");
}

// Clusters of 16 blocks where the chip can hold as many of them as there are row groups, else of 8. Returns -1 when the
// rows do not fit the clusters that can run at once (the caller then shares the work by operations).
template <int R, int HD, int BK>
static int launch_rows(const ProgramOp* ops, int n_ops, int rows, int max_k, long long* trace, cudaStream_t stream) {
    auto kernel = decode_program_rows_kernel<R, HD, BK>;
    const size_t smem = ROWS_GROUPS * sizeof(DecodeAttnSmem) + (size_t)R * max_k * sizeof(float);
    static int active16 = -1, active8 = -1;   // clusters of each size that can run at once (with the smallest buffer)
    static size_t smem_allowed = 0;
    if (smem > smem_allowed) {
        GB_REQUIRE(smem <= 200 * 1024, "gb_program_launch: K = %d is too long for a program's activation buffer", max_k);
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        GB_REQUIRE(e == cudaSuccess, "gb_program_launch: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
        smem_allowed = smem;
        active16 = -1;
    }
    if (active16 < 0) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        for (int size : {16, 8}) {
            cudaLaunchConfig_t probe = {};
            probe.gridDim = dim3(size * 32);
            probe.blockDim = dim3(ROWS_THREADS);
            probe.dynamicSmemBytes = smem_allowed;
            cudaLaunchAttribute pa[1];
            pa[0].id = cudaLaunchAttributeClusterDimension;
            pa[0].val.clusterDim.x = size; pa[0].val.clusterDim.y = 1; pa[0].val.clusterDim.z = 1;
            probe.attrs = pa;
            probe.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kernel, &probe) != cudaSuccess) n = 0;
            (size == 16 ? active16 : active8) = n;
        }
        cudaGetLastError();
    }
    const int clusters = (rows + R - 1) / R;
    int size = 0;
    if (active16 >= clusters) size = 16;
    else if (active8 >= clusters) size = 8;
    if (size == 0) return -1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(clusters * size);
    cfg.blockDim = dim3(ROWS_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = size; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ops, n_ops, rows, trace);
    if (e != cudaSuccess) {
        gb_set_error("gb_program_launch: cluster launch failed: %s", cudaGetErrorString(e));
        return 2;
    }
    return gb_check_launch("gb_program_launch");
}

enum { PROGRAM_BY_ROWS = 0, PROGRAM_BY_OPERATIONS = 1 };

static int program_dispatch(const void* ops, int n_ops, int rows, int hd, int block_keys, int max_vblocks, int max_k,
                            void* barrier, int* status, int how, int absent, long long wait_cycles, long long* trace,
                            cudaStream_t stream) {
    GB_REQUIRE(ops && n_ops >= 0 && barrier && status && max_vblocks >= 1 && max_k >= 8, "gb_program_launch: bad arguments");
    GB_REQUIRE(rows >= 1 && rows <= 16, "gb_program_launch: %d rows are outside a program's range (1..16)", rows);
    GB_REQUIRE(how == PROGRAM_BY_ROWS || how == PROGRAM_BY_OPERATIONS, "gb_program_launch: unknown way %d of sharing the work", how);
    if (n_ops == 0) return 0;
    const ProgramOp* o = static_cast<const ProgramOp*>(ops);
    unsigned* bar = static_cast<unsigned*>(barrier);
    // By rows: one row per cluster where that many clusters run at once, else two; if even that does not fit, by
    // operations. (A head size of 128 takes the 16-key variant either way.)
#define GB_PROG(NTT, HH, BB)                                                                                          \
    {                                                                                                                 \
        if (how == PROGRAM_BY_ROWS) {                                                                                 \
            constexpr int RB = HH == 64 ? 16 : BB;   /* blocks of 512 threads have 128 registers a thread */           \
            int rc = launch_rows<1, HH, RB>(o, n_ops, rows, max_k, trace, stream);                                    \
            if (rc == -1) rc = launch_rows<2, HH, RB>(o, n_ops, rows, max_k, trace, stream);                          \
            if (rc != -1) return rc;                                                                                  \
        }                                                                                                             \
        return launch_grid<NTT, HH, BB>(o, n_ops, max_vblocks, bar, status, absent, wait_cycles, trace, stream);      \
    }
#define GB_PROG_HD(NTT)                                   \
    if (hd == 0) { GB_PROG(NTT, 0, 32) }                  \
    if (hd == 16) { GB_PROG(NTT, 16, 32) }                \
    if (hd == 32) { GB_PROG(NTT, 32, 32) }                \
    if (hd == 64 && block_keys == 16) { GB_PROG(NTT, 64, 16) } \
    if (hd == 64) { GB_PROG(NTT, 64, 32) }                \
    if (hd == 128) { GB_PROG(NTT, 128, 16) }
    if (rows <= 8) { GB_PROG_HD(1) }
    GB_PROG_HD(2)
#undef GB_PROG_HD
#undef GB_PROG
    GB_REQUIRE(false, "gb_program_launch: head size %d is not built", hd);
}

// Run a program: `ops` on the device (n_ops operations written by the encode functions and copied there), every
// product with at most `rows` rows, every attention with head size `hd` (0: none) and `block_keys` keys per warp
// iteration; `max_vblocks` the most virtual blocks any operation has, `max_k` the longest K of its products;
// `barrier` one unsigned word on the device.
// how: 0 = by rows (a thread-block cluster per group of rows), 1 = by operations (all blocks share each operation).
GB_EXPORT int gb_program_launch(const void* ops, int n_ops, int rows, int hd, int block_keys, int max_vblocks, int max_k,
                                void* barrier, int* status, int how, cudaStream_t stream) {
    return program_dispatch(ops, n_ops, rows, hd, block_keys, max_vblocks, max_k, barrier, status, how, 0, PROGRAM_WAIT_CYCLES, nullptr, stream);
}

// For a test of the bounded wait: the by-operations kernel, but every barrier expects `absent` blocks more than the
// grid has and gives up after `wait_cycles` clock cycles. Nothing faults and nothing hangs: the first barrier's wait
// runs out, the blocks record GB_STATUS_WAIT_TIMEOUT and return, and the operations behind that barrier do not
// change anything.
GB_EXPORT int gb_program_launch_with_absent_blocks(const void* ops, int n_ops, int rows, int hd, int block_keys, int max_vblocks,
                                                   int max_k, void* barrier, int* status, int absent, long long wait_cycles,
                                                   cudaStream_t stream) {
    GB_REQUIRE(absent >= 0 && wait_cycles > 0 && wait_cycles <= PROGRAM_WAIT_CYCLES, "gb_program_launch_with_absent_blocks: bad arguments");
    return program_dispatch(ops, n_ops, rows, hd, block_keys, max_vblocks, max_k, barrier, status, PROGRAM_BY_OPERATIONS, absent,
                            wait_cycles, nullptr, stream);
}

// As gb_program_launch, and two blocks (the first and the last of the grid, or of the first cluster) write clock64
// values into `trace` (int64 [2, n_ops, 4] on the device): for each operation, when the block started it, had issued
// its hints, had done its share and waited for the others' share of the operation before, and had arrived at the
// barrier behind it. For measurements: where a step's time goes.
GB_EXPORT int gb_program_launch_traced(const void* ops, int n_ops, int rows, int hd, int block_keys, int max_vblocks, int max_k,
                                       void* barrier, int* status, int how, void* trace, cudaStream_t stream) {
    GB_REQUIRE(trace != nullptr, "gb_program_launch_traced: no trace buffer");
    return program_dispatch(ops, n_ops, rows, hd, block_keys, max_vblocks, max_k, barrier, status, how, 0, PROGRAM_WAIT_CYCLES,
                            static_cast<long long*>(trace), stream);
}
