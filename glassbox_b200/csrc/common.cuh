// Shared declarations for the kernel library: element types, error reporting, small helpers.
//
// Every exported function is `extern "C"`, takes raw device pointers plus a CUDA stream, and
// returns 0 on success. On failure it returns a non-zero code and leaves a message that
// `gb_last_error()` returns; nothing is printed and nothing traps. Kernels never assert: a bad
// index (token id, cache slot) is recorded in a caller-supplied status word and the access is
// skipped, so a faulty batch cannot fault the GPU.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define GB_EXPORT extern "C" __attribute__((visibility("default")))

enum GbDtype : int { GB_F32 = 0, GB_BF16 = 1 };

// Bits of the device status word.
enum GbStatusBits : int {
    GB_STATUS_BAD_TOKEN = 1,      // a token id outside the vocabulary
    GB_STATUS_BAD_SLOT = 2,       // a cache slot or page id outside the pool
    GB_STATUS_BAD_POSITION = 4,   // a position outside the rotary table, or beyond what a block table covers
    GB_STATUS_WAIT_TIMEOUT = 8,   // a bounded wait inside a kernel gave up
};

void gb_set_error(const char* fmt, ...);
int gb_check_launch(const char* what);

#define GB_REQUIRE(cond, ...)                 \
    do {                                      \
        if (!(cond)) {                        \
            gb_set_error(__VA_ARGS__);        \
            return 1;                         \
        }                                     \
    } while (0)

__device__ __forceinline__ float gb_to_float(float v) { return v; }
__device__ __forceinline__ float gb_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T gb_from_float(float v);
template <> __device__ __forceinline__ float gb_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 gb_from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float gb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float gb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

static inline int gb_ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// Programmatic dependent launch. A kernel launched through gb_launch (while the switch is on) may start
// while its predecessor in the stream is still running: it does its set-up, lets its own successor start
// (gb_pdl_launch_dependents) and then waits (gb_pdl_wait) until the predecessor has completed and its
// writes are visible; nothing before the wait may read what earlier kernels wrote, or write anything.
// Launched any other way, both instructions do nothing.
int gb_pdl_enabled();

__device__ __forceinline__ void gb_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void gb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// How a kernel body that can run in several settings meets the work before it. A body calls start() first and
// wait() at the point from which it reads what earlier work wrote; before wait() it may only read what no kernel of
// the step writes (weights, step metadata). A bounded wait may give up: the body then returns at once, having written nothing. Stand-alone kernels use GbPdlSync (programmatic dependent launch); a
// persistent kernel passes an object whose wait() is its barrier's wait.
struct GbPdlSync {
    __device__ __forceinline__ void start() { gb_pdl_launch_dependents(); }
    __device__ __forceinline__ void wait() { gb_pdl_wait(); }
    __device__ __forceinline__ bool gave_up() const { return false; }   // after wait(): true = do nothing more
    // the threads that share one virtual block: here the whole thread block
    __device__ __forceinline__ int thread() const { return (int)threadIdx.x; }
    __device__ __forceinline__ void group_barrier() { __syncthreads(); }
};

enum { GB_PDL_ELEMENTWISE = 1, GB_PDL_GEMM = 2, GB_PDL_ATTENTION = 4 };   // bits of the switch

template <typename... KArgs, typename... Args>
static inline cudaError_t gb_launch(int family, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (gb_pdl_enabled() & family) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
