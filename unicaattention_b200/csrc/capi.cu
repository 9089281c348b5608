// Error reporting and device checks behind the C entry points.
#include "capi.h"

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

int unica_check_device() {
    int device = 0, major = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess)
        return unica_fail(UNICA_B200_ERR_CUDA, "cannot query the current CUDA device");
    if (major != 10) return unica_fail(UNICA_B200_ERR_DEVICE, "these kernels are built for sm_100a (B200) only");
    return UNICA_B200_OK;
}

extern "C" const char* unica_b200_last_error(void) { return g_error; }
extern "C" int unica_b200_version(void) { return 1; }
