// Statistics and INT8 quantization passes of the accurate mode: HBM-bound kernels that read bf16 Q, K, V once in the
// caller's layout and write the 8-bit operands already arranged as the shared-memory images tcgen05.mma reads (no
// swizzle, K-major core matrices of 8 rows x 16 bytes), so that the attention kernel fetches each tile with one
// contiguous bulk copy.
//
// Numerics follow the reference bit for bit (bench/emulate.py quant(), csrc/flash.cu:334-372 and 590-630):
// amax over the scale block, scale = max(amax * (1/127), 1e-12), code = clamp(rint(x / scale), -127, 127) with an IEEE
// division and round-half-even.
#include <cstdio>

#include "quantize_int8.cuh"

namespace unica {

constexpr int STATS_TOKENS = 256;  // tokens per partial sum; the summation order below is part of the contract
constexpr int STATS_LANES = 16;

// Sum, min and max per channel over a block of 256 tokens of one head (the reference's rope_stats, csrc/flash.cu:287-327,
// without RoPE): thread = (lane of 16 tokens, chunk of 8 channels); lane l adds tokens l, l + 16, ... in order, then
// the 16 lanes are added in order.  partial: [heads][blocks][3][128].  Grid (blocks, heads).
// skip: [heads][n_tokens] bytes, 1 = the token takes no part (the outlier keys of V), or null.
// rope: x is rotated first (the rotated values exist nowhere in memory).
__global__ void __launch_bounds__(THREADS) channel_stats_kernel(const __nv_bfloat16* __restrict__ x, TokenLayout in,
                                                                 int n_tokens, float* __restrict__ partial,
                                                                 const uint8_t* __restrict__ skip = nullptr,
                                                                 RopeTable rope = RopeTable{nullptr, 0}) {
    const int chunk = threadIdx.x % 16, lane = threadIdx.x / 16;
    const int head = blockIdx.y, token0 = blockIdx.x * STATS_TOKENS;
    float sum[8], low[8], high[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) sum[i] = 0.0f, low[i] = INFINITY, high[i] = -INFINITY;
    const int end = min(token0 + STATS_TOKENS, n_tokens);
#pragma unroll 4
    for (int token = token0 + lane; token < end; token += STATS_LANES) {
        if (skip && skip[size_t(head) * n_tokens + token]) continue;
        float v[8];
        load8(v, x + in.offset(head, token) + chunk * 8, in.half);
        if (rope.table) rope8(v, rope.row(in, head, token), chunk * 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            sum[i] += v[i];
            low[i] = fminf(low[i], v[i]);
            high[i] = fmaxf(high[i], v[i]);
        }
    }
    __shared__ float stats[3][STATS_LANES][HEAD_DIM];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        stats[0][lane][chunk * 8 + i] = sum[i];
        stats[1][lane][chunk * 8 + i] = low[i];
        stats[2][lane][chunk * 8 + i] = high[i];
    }
    __syncthreads();
    if (threadIdx.x < HEAD_DIM) {
        float s = 0.0f, lo = INFINITY, hi = -INFINITY;
        for (int l = 0; l < STATS_LANES; ++l) {
            s += stats[0][l][threadIdx.x];
            lo = fminf(lo, stats[1][l][threadIdx.x]);
            hi = fmaxf(hi, stats[2][l][threadIdx.x]);
        }
        float* out = partial + (size_t(head) * gridDim.x + blockIdx.x) * 3 * HEAD_DIM + threadIdx.x;
        out[0] = s;
        out[HEAD_DIM] = lo;
        out[2 * HEAD_DIM] = hi;
    }
}

// The partials of each group of `blocks_per_group` blocks added in order (the reference leaves this to torch, whose
// order is unspecified: unica/__init__.py:603-612): mean = sum / true token count, min, max.  Grid (groups, heads), 128 threads.
__global__ void __launch_bounds__(HEAD_DIM) channel_stats_finish_kernel(const float* __restrict__ partial, int blocks,
                                                                        int blocks_per_group, int n_tokens,
                                                                        float* __restrict__ mean, float* __restrict__ low,
                                                                        float* __restrict__ high) {
    const int head = blockIdx.y, group = blockIdx.x, c = threadIdx.x;
    const int b0 = group * blocks_per_group, b1 = min(b0 + blocks_per_group, blocks);
    float s = 0.0f, lo = INFINITY, hi = -INFINITY;
    for (int b = b0; b < b1; ++b) {
        const float* p = partial + (size_t(head) * blocks + b) * 3 * HEAD_DIM + c;
        s += p[0];
        lo = fminf(lo, p[HEAD_DIM]);
        hi = fmaxf(hi, p[2 * HEAD_DIM]);
    }
    const int count = min(b1 * STATS_TOKENS, n_tokens) - b0 * STATS_TOKENS;
    const size_t o = (size_t(head) * gridDim.x + group) * HEAD_DIM + c;
    mean[o] = s / float(count);
    low[o] = lo;
    high[o] = hi;
}

// One block per tile.  Grid (tiles, heads).
template <int ROWS>
__global__ void __launch_bounds__(THREADS) quantize_rows_int8_kernel(const __nv_bfloat16* __restrict__ x, TokenLayout in,
                                                                      const float* __restrict__ mean, int n_tokens,
                                                                      int8_t* __restrict__ codes, float* __restrict__ scales,
                                                                      RopeTable rope) {
    __shared__ float scratch[THREADS / 32];
    const int head = blockIdx.y, tile = blockIdx.x;
    rows_int8_tile<ROWS>(x, in, mean ? mean + head * HEAD_DIM : nullptr, head, tile, n_tokens,
                         codes + (size_t(head) * gridDim.x + tile) * (ROWS * HEAD_DIM), scales + size_t(head) * gridDim.x + tile, rope, scratch);
}

template <bool PER_TOKEN>
__global__ void __launch_bounds__(THREADS) quantize_v_int8_kernel(const __nv_bfloat16* __restrict__ v, TokenLayout in,
                                                                   const float* __restrict__ low, const float* __restrict__ high,
                                                                   const uint8_t* __restrict__ skip, int n_tokens,
                                                                   int8_t* __restrict__ v8, float* __restrict__ v_scale,
                                                                   float* __restrict__ v_token) {
    __shared__ VTileSmem sm;
    const int head = blockIdx.y;
    v_int8_tile<PER_TOKEN>(v, in, low ? low + head * HEAD_DIM : nullptr, high ? high + head * HEAD_DIM : nullptr, skip, head, blockIdx.x,
                           gridDim.x, n_tokens, v8, v_scale, v_token, sm);
}

}  // namespace unica

// ---------------------------------------------------------------------------------------------------------------------
// C entry points (declared in include/unica_b200.h)

#include "capi.h"

using namespace unica;

static int channel_stats(const void* x, unica_token_layout layout, RopeTable rope, int heads, int n_tokens, int per, float* partial,
                         float* mean, float* low, float* high, void* stream) {
    if (!x || !partial || !mean || !low || !high) return unica_fail(UNICA_B200_ERR_ARGUMENT, "channel_stats: null pointer");
    if (heads <= 0 || n_tokens <= 0) return unica_fail(UNICA_B200_ERR_ARGUMENT, "channel_stats: heads and n_tokens must be positive");
    if (per != 0 && (per < 0 || per % STATS_TOKENS)) return unica_fail(UNICA_B200_ERR_ARGUMENT, "channel_stats: per must be 0 or a multiple of 256");
    const int blocks = (n_tokens + STATS_TOKENS - 1) / STATS_TOKENS;
    const int per_group = per ? per / STATS_TOKENS : blocks;
    const int groups = (blocks + per_group - 1) / per_group;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    channel_stats_kernel<<<dim3(blocks, heads), THREADS, 0, s>>>(static_cast<const __nv_bfloat16*>(x), to_layout(layout), n_tokens, partial,
                                                                 nullptr, rope);
    channel_stats_finish_kernel<<<dim3(groups, heads), HEAD_DIM, 0, s>>>(partial, blocks, per_group, n_tokens, mean, low, high);
    return unica_check_launch("channel_stats");
}

extern "C" int unica_b200_channel_stats(const void* x, unica_token_layout layout, int heads, int n_tokens, int per,
                                        float* partial, float* mean, float* low, float* high, void* stream) {
    return channel_stats(x, layout, RopeTable{nullptr, 0}, heads, n_tokens, per, partial, mean, low, high, stream);
}

extern "C" int unica_b200_channel_stats_rope(const void* x, unica_token_layout layout, const void* rope, long long rope_batch_stride,
                                             int heads, int n_tokens, int per, float* partial, float* mean, float* low, float* high,
                                             void* stream) {
    if (!rope) return unica_fail(UNICA_B200_ERR_ARGUMENT, "channel_stats_rope: null table");
    return channel_stats(x, layout, RopeTable{static_cast<const __half*>(rope), rope_batch_stride}, heads, n_tokens, per, partial, mean,
                         low, high, stream);
}

// ---------------------------------------------------------------------------------------------------------------------
// The statistics pass for callers that cannot hand over scratch memory.
//
// unica_b200_channel_stats wants a `partial` buffer from its caller.  Some callers have none to give and no way to get
// one: an attention hook that runs inside a sampler whose memory manager has already filled the card with staged
// weights (an allocation there fails, or pushes something else out), a host written in C that owns no device
// allocator, or a latency-critical loop that must not enter the CUDA allocator because cudaMalloc and cudaFree stall
// the whole device.  For them the partial sums live in the array below, which is part of the library image.  CUDA loads
// the image into a GPU's context lazily, on the first use of anything in this module on that GPU, and that is when the
// bytes are set aside there (until the process ends or the device is reset): the first call must come while memory is
// still available.
constexpr int STATIC_STATS_RECORDS = 6144;  // (head, 256-token block) pairs: 40 heads x 32760 tokens need 5120
static __device__ __align__(256) float g_stats_scratch[size_t(STATIC_STATS_RECORDS) * 3 * HEAD_DIM];  // 9 MiB

// In host code `g_stats_scratch` is only a handle for the symbol, not an address a kernel could use: the device address
// has to be asked for, per device, with that device current.
static float* stats_scratch_of_current_device(int* error) {
    constexpr int MAX_DEVICES = 64;
    static float* address[MAX_DEVICES] = {};
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) {
        *error = unica_fail(UNICA_B200_ERR_CUDA, "channel_stats_static: cannot tell the current device");
        return nullptr;
    }
    if (!address[device]) {  // first call on this device
        float* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_stats_scratch);
        if (e != cudaSuccess || !p) {
            static thread_local char message[256];
            snprintf(message, sizeof message,
                     "channel_stats_static: the built-in scratch could not be set up on this device (%s); the first call on a device "
                     "loads the module and reserves 9 MiB, which needs free device memory",
                     cudaGetErrorString(e));
            cudaGetLastError();  // the error is reported here, not by the next launch check
            *error = unica_fail(UNICA_B200_ERR_CUDA, message);
            return nullptr;
        }
        address[device] = p;  // the same value whichever thread gets here first
    }
    return address[device];
}

extern "C" int unica_b200_channel_stats_static(const void* x, unica_token_layout layout, int heads, int n_tokens, int per,
                                               float* mean, float* low, float* high, void* stream) {
    if (!x || !mean || !low || !high) return unica_fail(UNICA_B200_ERR_ARGUMENT, "channel_stats_static: null pointer");
    if (heads <= 0 || n_tokens <= 0) return unica_fail(UNICA_B200_ERR_ARGUMENT, "channel_stats_static: heads and n_tokens must be positive");
    if (per != 0 && (per < 0 || per % STATS_TOKENS)) return unica_fail(UNICA_B200_ERR_ARGUMENT, "channel_stats_static: per must be 0 or a multiple of 256");
    const int blocks = (n_tokens + STATS_TOKENS - 1) / STATS_TOKENS;
    if (static_cast<long long>(heads) * blocks > STATIC_STATS_RECORDS)
        return unica_fail(UNICA_B200_ERR_ARGUMENT,
                          "channel_stats_static: heads * ceil(n_tokens / 256) exceeds the built-in scratch of 6144 records; "
                          "use unica_b200_channel_stats with a buffer of your own");
    int error = UNICA_B200_OK;
    float* partial = stats_scratch_of_current_device(&error);
    if (!partial) return error;
    const int per_group = per ? per / STATS_TOKENS : blocks;
    const int groups = (blocks + per_group - 1) / per_group;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Nothing in the scratch has to start at zero: every record the second kernel reads is written whole by the first.
    channel_stats_kernel<<<dim3(blocks, heads), THREADS, 0, s>>>(static_cast<const __nv_bfloat16*>(x), to_layout(layout), n_tokens, partial);
    channel_stats_finish_kernel<<<dim3(groups, heads), HEAD_DIM, 0, s>>>(partial, blocks, per_group, n_tokens, mean, low, high);
    return unica_check_launch("channel_stats_static");
}

extern "C" int unica_b200_channel_stats_masked(const void* x, unica_token_layout layout, const uint8_t* skip, int heads, int n_tokens,
                                               float* partial, float* mean, float* low, float* high, void* stream) {
    if (!x || !skip || !partial || !mean || !low || !high) return unica_fail(UNICA_B200_ERR_ARGUMENT, "channel_stats_masked: null pointer");
    if (heads <= 0 || n_tokens <= 0) return unica_fail(UNICA_B200_ERR_ARGUMENT, "channel_stats_masked: heads and n_tokens must be positive");
    const int blocks = (n_tokens + STATS_TOKENS - 1) / STATS_TOKENS;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    channel_stats_kernel<<<dim3(blocks, heads), THREADS, 0, s>>>(static_cast<const __nv_bfloat16*>(x), to_layout(layout), n_tokens, partial, skip);
    channel_stats_finish_kernel<<<dim3(1, heads), HEAD_DIM, 0, s>>>(partial, blocks, blocks, n_tokens, mean, low, high);
    return unica_check_launch("channel_stats_masked");
}

static int quantize_int8(const void* x, unica_token_layout layout, const float* mean, RopeTable rope, int heads, int n_tokens,
                         int block_tokens, int tiles, int8_t* codes, float* scales, void* stream) {
    if (!x || !codes || !scales) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_int8: null pointer");
    if (heads <= 0 || n_tokens <= 0) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_int8: heads and n_tokens must be positive");
    if (block_tokens != 128 && block_tokens != 64) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_int8: block_tokens must be 128 (Q) or 64 (K)");
    if (tiles < (n_tokens + block_tokens - 1) / block_tokens) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_int8: tiles does not cover n_tokens");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
    if (block_tokens == 128)
        quantize_rows_int8_kernel<128><<<dim3(tiles, heads), THREADS, 0, s>>>(xb, to_layout(layout), mean, n_tokens, codes, scales, rope);
    else
        quantize_rows_int8_kernel<64><<<dim3(tiles, heads), THREADS, 0, s>>>(xb, to_layout(layout), mean, n_tokens, codes, scales, rope);
    return unica_check_launch("quantize_int8");
}

extern "C" int unica_b200_quantize_int8(const void* x, unica_token_layout layout, const float* mean, int heads, int n_tokens,
                                        int block_tokens, int tiles, int8_t* codes, float* scales, void* stream) {
    return quantize_int8(x, layout, mean, RopeTable{nullptr, 0}, heads, n_tokens, block_tokens, tiles, codes, scales, stream);
}

extern "C" int unica_b200_quantize_int8_rope(const void* x, unica_token_layout layout, const float* mean, const void* rope,
                                             long long rope_batch_stride, int heads, int n_tokens, int block_tokens, int tiles,
                                             int8_t* codes, float* scales, void* stream) {
    if (!rope) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_int8_rope: null table");
    return quantize_int8(x, layout, mean, RopeTable{static_cast<const __half*>(rope), rope_batch_stride}, heads, n_tokens, block_tokens,
                         tiles, codes, scales, stream);
}

extern "C" int unica_b200_quantize_v_int8(const void* v, unica_token_layout layout, const float* low, const float* high,
                                          const uint8_t* skip, int per_token, int heads, int n_tokens, int8_t* v8,
                                          float* v_scale, float* v_token, void* stream) {
    if (!v || !v8 || !v_scale) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_v_int8: null pointer");
    if (heads <= 0 || n_tokens <= 0) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_v_int8: heads and n_tokens must be positive");
    if (per_token ? !v_token : (!low || !high))
        return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_v_int8: per token needs v_token, per channel needs low and high");
    const int tiles = (n_tokens + KEY_TILE - 1) / KEY_TILE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const __nv_bfloat16* vb = static_cast<const __nv_bfloat16*>(v);
    if (per_token)
        quantize_v_int8_kernel<true><<<dim3(tiles, heads), THREADS, 0, s>>>(vb, to_layout(layout), low, high, skip, n_tokens, v8, v_scale, v_token);
    else
        quantize_v_int8_kernel<false><<<dim3(tiles, heads), THREADS, 0, s>>>(vb, to_layout(layout), low, high, skip, n_tokens, v8, v_scale, v_token);
    return unica_check_launch("quantize_v_int8");
}
