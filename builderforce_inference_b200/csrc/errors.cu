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

// Off unless asked for: measured on the decode step, early launch of dependents did not pay.
int g_bfi_pdl = 1;

// Turns programmatic dependent launch on (1) or off (0) for every later launch of this library.
extern "C" int bfi_set_pdl(int on) {
    g_bfi_pdl = on ? 1 : 0;
    return 0;
}

// Identifies the build: the architecture the device code was compiled for.
extern "C" const char* bfi_build_arch() { return "sm_100a"; }
