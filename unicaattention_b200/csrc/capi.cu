// Error reporting and device checks behind the C entry points.
#include "capi.h"

#include <atomic>
#include <cstdio>
#include <cstring>

static thread_local char g_error[512] = "";

int unica_fail(int code, const char* message) {
    std::snprintf(g_error, sizeof g_error, "%s", message);
    return code;
}

int unica_check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return UNICA_B200_OK;
    std::snprintf(g_error, sizeof g_error, "%s: %s", what, cudaGetErrorString(e));
    return UNICA_B200_ERR_CUDA;
}

// The answer per device is looked up once (two runtime queries) and remembered: 0 unknown, 1 fine, 2 not a B200.
int unica_check_device() {
    constexpr int MAX_DEVICES = 64;
    static std::atomic<signed char> known[MAX_DEVICES];
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return unica_fail(UNICA_B200_ERR_CUDA, "cannot query the current CUDA device");
    signed char state = device < MAX_DEVICES ? known[device].load(std::memory_order_relaxed) : 0;
    if (state == 0) {
        int major = 0, minor = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess ||
            cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device) != cudaSuccess)
            return unica_fail(UNICA_B200_ERR_CUDA, "cannot query the current CUDA device");
        state = major == 10 && minor == 0 ? 1 : 2;  // sm_100a code runs on compute capability 10.0 only
        if (device < MAX_DEVICES) known[device].store(state, std::memory_order_relaxed);
    }
    if (state != 1) return unica_fail(UNICA_B200_ERR_DEVICE, "these kernels are built for sm_100a (B200, compute capability 10.0) only");
    return UNICA_B200_OK;
}

extern "C" const char* unica_b200_last_error(void) { return g_error; }
extern "C" int unica_b200_version(void) { return 1; }
