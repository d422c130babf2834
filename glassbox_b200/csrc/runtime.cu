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
