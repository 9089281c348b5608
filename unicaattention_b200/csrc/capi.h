// Host-side plumbing shared by the C entry points: the thread-local error message and launch checks.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/unica_b200.h"
#include "common.cuh"

int unica_fail(int code, const char* message);
int unica_check_launch(const char* what);  // cudaGetLastError after a launch -> 0 or UNICA_B200_ERR_CUDA
int unica_check_device();                  // the current device must be compute capability 10.0 (cached per device)

// Checks and copies a caller's list of peer output tensors (see PeerOutputs); n_peers == 0 leaves `peers` empty.
static inline int unica_peer_outputs(const void* out, void* const* peer_out, int n_peers, unica::PeerOutputs* peers) {
    peers->count = 0;
    if (n_peers == 0) return UNICA_B200_OK;
    if (n_peers < 0 || n_peers > unica::MAX_PEER_OUTPUTS || !peer_out) return unica_fail(UNICA_B200_ERR_ARGUMENT, "peer outputs: n_peers must be in 0..7 with a pointer list");
    for (int i = 0; i < n_peers; ++i) {
        if (!peer_out[i] || reinterpret_cast<uintptr_t>(peer_out[i]) % 16 || peer_out[i] == out)
            return unica_fail(UNICA_B200_ERR_ARGUMENT, "peer outputs: every pointer must be non-null, 16-byte aligned and different from out");
        peers->out[i] = static_cast<__nv_bfloat16*>(peer_out[i]);
    }
    peers->count = n_peers;
    return UNICA_B200_OK;
}

static inline unica::TokenLayout to_layout(const unica_token_layout& l) {
    unica::TokenLayout t;
    t.batch = l.batch, t.head = l.head, t.token = l.token, t.heads = l.heads, t.half = l.dtype == UNICA_B200_FLOAT16;
    return t;
}
