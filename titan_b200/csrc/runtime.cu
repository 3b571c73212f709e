// Error reporting shared by all launchers, and small queries about the device.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

void tb_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

extern "C" const char* tb_last_error() { return g_error; }

// Compute capability of the current device as major * 10 + minor, or a negative CUDA error.
extern "C" int tb_device_arch() {
    int dev = 0, major = 0, minor = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return -2;
    if (cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) return -3;
    return major * 10 + minor;
}

extern "C" int tb_abi_version() { return 1; }

int g_tb_pdl = 1;
// Programmatic dependent launch on (1) or off (0) for every kernel launched afterwards.
extern "C" void tb_set_pdl(int on) { g_tb_pdl = on ? 1 : 0; }
