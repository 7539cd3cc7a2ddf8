// Error message store of the C entry points.
#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>

static thread_local char g_error[512] = "";

extern "C" const char* ti_last_error() { return g_error; }

int ti_fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return 1;
}

int ti_check_launch(const char* what) {
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) return 0;
    return ti_fail("%s: %s", what, cudaGetErrorString(err));
}

static int current_device_slot() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    return dev;
}

bool TiPerDevice::first_use() {
    const int dev = current_device_slot();
    return dev < 0 || !done[dev];
}

void TiPerDevice::mark() {
    const int dev = current_device_slot();
    if (dev >= 0) done[dev] = true;
}
