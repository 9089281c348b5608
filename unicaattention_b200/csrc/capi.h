// Host-side plumbing shared by the C entry points: the thread-local error message and launch checks.
#pragma once

#include <cuda_runtime.h>

#include "../../include/unica_b200.h"
#include "common.cuh"

int unica_fail(int code, const char* message);
int unica_check_launch(const char* what);  // cudaGetLastError after a launch -> 0 or UNICA_B200_ERR_CUDA
int unica_check_device();                  // the current device must be compute capability 10.0 (cached per device)

static inline unica::TokenLayout to_layout(const unica_token_layout& l) {
    unica::TokenLayout t;
    t.batch = l.batch, t.head = l.head, t.token = l.token, t.heads = l.heads;
    return t;
}
