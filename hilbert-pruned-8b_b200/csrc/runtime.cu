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

// Timeline marks (see common.cuh).  `marks` holds capacity pairs of 64-bit times, `count` one
// 32-bit counter; both are device memory of the caller.  A library built without
// -DHB_TIMELINE refuses.  `events` non-zero also records the events inside kernels that have
// some.  Passing null pointers switches the marks off again.
#ifdef HB_TIMELINE
static HbTimelineSetter g_tl_setters[64];
static int g_tl_setter_count = 0;
void hb_timeline_register(HbTimelineSetter fn) {
    if (g_tl_setter_count < 64) g_tl_setters[g_tl_setter_count++] = fn;
}
#endif
extern "C" int hb_timeline_set(void* marks, void* count, int capacity, int events) {
#ifdef HB_TIMELINE
    for (int i = 0; i < g_tl_setter_count; i++)
        g_tl_setters[i]((unsigned long long*)marks, (unsigned int*)count, (unsigned int)capacity, events);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return hb_fail("timeline: %s", cudaGetErrorString(e));
    return 0;
#else
    (void)marks, (void)count, (void)capacity, (void)events;
    return hb_fail("timeline: this library was built without -DHB_TIMELINE (set HILBERT_B200_TIMELINE=1 before the first use)");
#endif
}

extern "C" int hb_device_info(int device, int* sm_major, int* sm_minor, int* sm_count) {
    cudaDeviceProp p;
    cudaError_t e = cudaGetDeviceProperties(&p, device);
    if (e != cudaSuccess) return hb_fail("device %d: %s", device, cudaGetErrorString(e));
    *sm_major = p.major;
    *sm_minor = p.minor;
    *sm_count = p.multiProcessorCount;
    return 0;
}
