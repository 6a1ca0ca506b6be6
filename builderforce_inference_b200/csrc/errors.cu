// Error reporting shared by every exported function of one library.
#include "common.cuh"

static thread_local char g_error[1024] = "";

extern "C" const char* bfi_last_error() { return g_error; }

int bfi_fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return 1;
}

int bfi_check_launch(const char* what) {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();
        return bfi_fail("%s: launch failed: %s", what, cudaGetErrorString(e));
    }
    return 0;
}

// Identifies the build: the architecture the device code was compiled for.
extern "C" const char* bfi_build_arch() { return "sm_100a"; }
