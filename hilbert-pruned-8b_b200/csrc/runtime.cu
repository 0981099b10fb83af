// Error reporting and device queries of the kernel library.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

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

// HILBERT_B200_PDL=0 launches every kernel fully serialised (for debugging).
bool hb_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("HILBERT_B200_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
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
