// Error reporting and device queries of the kernel library.
#include <stdarg.h>
#include <stdio.h>

#include "api.h"
#include "common.cuh"

static thread_local char g_error[512] = "";

int hb_fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return 1;
}

int hb_check_launch(const char* what) {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();
        return hb_fail("%s: launch failed: %s", what, cudaGetErrorString(e));
    }
    return 0;
}

extern "C" const char* hb_last_error(void) { return g_error; }

extern "C" int hb_device_info(int device, int* sm_major, int* sm_minor, int* sm_count) {
    cudaDeviceProp p;
    cudaError_t e = cudaGetDeviceProperties(&p, device);
    if (e != cudaSuccess) return hb_fail("device %d: %s", device, cudaGetErrorString(e));
    *sm_major = p.major;
    *sm_minor = p.minor;
    *sm_count = p.multiProcessorCount;
    return 0;
}
