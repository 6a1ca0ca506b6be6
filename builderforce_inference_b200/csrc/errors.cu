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

// Multiprocessors of the current device, asked of the driver once per device: launchers size
// their grids and work splits by it instead of by a constant.
int bfi_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = 148;      // no device to ask (a build check without a GPU): a B200's count
        }
        cached[dev] = n;
    }
    return cached[dev];
}

extern "C" int bfi_device_sm_count() { return bfi_sm_count(); }

// Identifies the build: the architecture the device code was compiled for.
extern "C" const char* bfi_build_arch() { return "sm_100a"; }
