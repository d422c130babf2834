// Error reporting shared by every exported function, and a few queries about the device.
#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>

static thread_local char g_error[1024] = "";

void gb_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int gb_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        gb_set_error("%s: launch failed: %s", what, cudaGetErrorString(e));
        return 2;
    }
    return 0;
}

GB_EXPORT const char* gb_last_error() { return g_error; }

// Which kernel families are launched with programmatic stream serialisation (bits GB_PDL_*; all by default).
static int g_pdl = 7;
int gb_pdl_enabled() { return g_pdl; }
GB_EXPORT void gb_set_pdl(int families) { g_pdl = families; }

// Compute capability of the current device as major*10+minor, or a negative CUDA error code.
GB_EXPORT int gb_device_arch() {
    int dev = 0, major = 0, minor = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (e != cudaSuccess) {
        gb_set_error("gb_device_arch: %s", cudaGetErrorString(e));
        return -(int)e;
    }
    return major * 10 + minor;
}

GB_EXPORT int gb_abi_version() { return 1; }

// One decode step's traffic in one call: the step's metadata block to the device, the step's recorded graph, the
// sampled tokens back to the host; all on `stream`, nothing is waited for. `graph_exec` is a cudaGraphExec_t.
GB_EXPORT int gb_step_io(const void* host_meta, void* dev_meta, long long meta_bytes, void* graph_exec, const void* sampled_dev,
                         void* sampled_host, long long sampled_bytes, cudaStream_t stream) {
    GB_REQUIRE(host_meta && dev_meta && graph_exec && meta_bytes > 0, "gb_step_io: bad arguments");
    cudaError_t e = cudaMemcpyAsync(dev_meta, host_meta, (size_t)meta_bytes, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph_exec), stream);
    if (e == cudaSuccess && sampled_bytes > 0)
        e = cudaMemcpyAsync(sampled_host, sampled_dev, (size_t)sampled_bytes, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) {
        gb_set_error("gb_step_io: %s", cudaGetErrorString(e));
        return 2;
    }
    return 0;
}
