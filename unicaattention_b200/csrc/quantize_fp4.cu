// NVFP4 quantization passes of the fast mode: e2m1 codes with one e4m3 scale per 16 elements along the contraction
// and one FP32 "outer" scale (per head for Q and K, per channel for V), plus the exact Q-smoothing term.
//
// Numerics follow the reference bit for bit (bench/emulate.py:98-113 block_scaled "nvfp4"; csrc/flash.cu:1021-1050,
// 1183-1216): outer = max(amax * (1/2688), 1e-30); scale byte = e4m3(amax16 * (1/6) / outer), saturating; element code =
// e2m1(x / (e4m3 value * outer)), round to nearest even, saturating, 0 where the block scale is 0.
//
// Outputs are the operand images tcgen05.mma kind::mxf4nvf4 reads (K-major, no swizzle, two codes per byte, the lower
// contraction index in the low nibble), and the scale bytes in the order the attention kernel copies them into tensor
// memory.  Keys inside a 64-key tile are stored in the reference's slot order (bench/emulate.py:116-119): the 16-key
// scale blocks of P and V are defined on that order, so it is part of the numerics.
#include <cuda_fp8.h>

#include "capi.h"

namespace unica {

constexpr int FP4_THREADS = 256;
constexpr int V4_ROWS = 144;      // 128 channels + 16 rows of ones: their column of P.V is the running denominator
constexpr int V4_SF_WORDS = 256;  // scale words of a tile: two blocks of [32 lanes][4], the second for rows 128..143

__host__ __device__ __forceinline__ int slot_key(int k) { return 32 * (k / 32) + 8 * (k % 8 / 2) + 2 * (k % 32 / 8) + k % 2; }

__device__ __forceinline__ uint32_t to_e4m3(float x) { return __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3); }
__device__ __forceinline__ float from_e4m3(uint32_t byte) {
    return __half2float(__half(__nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3)));
}

// 8 floats -> 8 e2m1 codes, element i in nibble i.
__device__ __forceinline__ uint32_t pack_e2m1x8(const float* v) {
    uint32_t word;
    asm("{\n\t"
        ".reg .b8 b0, b1, b2, b3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
        "mov.b32 %0, {b0, b1, b2, b3};\n\t"
        "}"
        : "=r"(word)
        : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
    return word;
}

// One block of 16 values: scale byte and 16 codes (two words).
__device__ __forceinline__ void quantize_block16(float (&v)[16], float outer, uint32_t& byte, uint2& codes) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    byte = to_e4m3(__fdiv_rn(amax * (1.0f / 6.0f), outer));
    const float scale = from_e4m3(byte) * outer;
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = scale > 0.0f ? __fdiv_rn(v[i], scale) : 0.0f;
    codes = make_uint2(pack_e2m1x8(v), pack_e2m1x8(v + 8));
}

// outer[head] = max(max |x - mean| * (1/2688), 1e-30) from the per-channel (and per mean group) min and max of x:
// the extreme elements go through the same float subtraction as every element, so this is the head's exact maximum
// (unica/__init__.py:485-492).  mean/low/high: [heads][groups][128] (mean may be null).  Grid: heads, 128 threads.
__global__ void __launch_bounds__(HEAD_DIM) nvfp4_outer_rows_kernel(const float* __restrict__ mean, const float* __restrict__ low,
                                                                    const float* __restrict__ high, int groups,
                                                                    float* __restrict__ outer) {
    __shared__ float part[HEAD_DIM / 32];
    const int head = blockIdx.x, c = threadIdx.x;
    float amax = 0.0f;
    for (int g = 0; g < groups; ++g) {
        const size_t i = (size_t(head) * groups + g) * HEAD_DIM + c;
        const float m = mean ? mean[i] : 0.0f;
        amax = fmaxf(amax, fmaxf(fabsf(high[i] - m), fabsf(low[i] - m)));
    }
#pragma unroll
    for (int d = 16; d > 0; d /= 2) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    if (c % 32 == 0) part[c / 32] = amax;
    __syncthreads();
    if (c == 0) outer[head] = fmaxf(fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3])) * (1.0f / 2688.0f), 1e-30f);
}

// Q or K minus its mean in NVFP4 along the channels, one block per tile of ROWS tokens (128: Q, 64: K).
// SLOTS: row r of a tile holds token tile * 64 + slot_key(r) (K); else token tile * ROWS + r (Q).
// mean: [heads][groups][128], one group per mean_tokens tokens, or null.
// codes: [heads][tiles][4 chunks of 32 channels][ROWS][16] bytes; sf: Q [heads][tiles][2 halves of 64 channels][128][4]
// bytes, K [heads][tiles][32 lanes][4 words][4] bytes (see the store below).
template <int ROWS, bool SLOTS>
__global__ void __launch_bounds__(FP4_THREADS) quantize_rows_fp4_kernel(const __nv_bfloat16* __restrict__ x, TokenLayout in,
                                                                         const float* __restrict__ mean, int mean_tokens, int groups,
                                                                         const float* __restrict__ outer, int n_tokens,
                                                                         uint8_t* __restrict__ codes, uint8_t* __restrict__ sf,
                                                                         RopeTable rope) {
    const int head = blockIdx.y, tile = blockIdx.x;
    const float head_outer = outer[head];
    uint8_t* tile_codes = codes + (size_t(head) * gridDim.x + tile) * (ROWS * HEAD_DIM / 2);
    uint8_t* tile_sf = sf + (size_t(head) * gridDim.x + tile) * (ROWS * 8);
#pragma unroll
    for (int it = 0; it < ROWS * 8 / FP4_THREADS; ++it) {
        const int item = it * FP4_THREADS + threadIdx.x, row = item % ROWS, block = item / ROWS;  // block of 16 channels
        const int token = SLOTS ? tile * ROWS + slot_key(row) : tile * ROWS + row;
        float v[16];
        if (token < n_tokens) {
            const __nv_bfloat16* src = x + in.offset(head, token) + block * 16;
            const uint4 raw[2] = {load_bf16x8(src, in.half), load_bf16x8(src + 8, in.half)};
            const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(raw);
            const float* mu = mean ? mean + (size_t(head) * groups + token / mean_tokens) * HEAD_DIM + block * 16 : nullptr;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 f = __bfloat1622float2(pairs[i]);
                v[2 * i] = f.x, v[2 * i + 1] = f.y;
            }
            if (rope.table) {  // rotate first: the mean is the rotated x's
                const __half* f = rope.row(in, head, token);
                rope8(*reinterpret_cast<float(*)[8]>(v), f, block * 16);
                rope8(*reinterpret_cast<float(*)[8]>(v + 8), f, block * 16 + 8);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] -= mu ? mu[i] : 0.0f;
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0.0f;
        }
        uint32_t byte;
        uint2 packed;
        quantize_block16(v, head_outer, byte, packed);
        *reinterpret_cast<uint2*>(tile_codes + ((block / 2) * ROWS + row) * 16 + (block % 2) * 8) = packed;
        // the word of (K step = block / 4, row): Q [2][128] by row; K [32 lanes][4]: word 2 step + row / 32 of lane row % 32,
        // the 16 bytes tcgen05.cp hands to one tensor-memory lane
        const int word = ROWS == 64 ? (row % 32) * 4 + 2 * (block / 4) + row / 32 : (block / 4) * ROWS + row;
        tile_sf[word * 4 + block % 4] = uint8_t(byte);
    }
}

// V in NVFP4 along the keys, per channel, one block per tile of 64 keys (slot order).  low/high: the channel's min and
// max over the head ([heads][128]); v_outer [heads][128] is written by tile 0.
// codes: [heads][tiles][2 chunks of 32 slots][144 rows][16] bytes, rows 128..143 all ones (code 0x2);
// sf: [heads][tiles][2 blocks][32 lanes][4 words] of 4 bytes: block 0 word c / 32 of lane c % 32 = channel c's four
// bytes, block 1 word 0 of lanes 0..15 = ones (0x38) for rows 128..143, zeros elsewhere.
__global__ void __launch_bounds__(FP4_THREADS) quantize_v_fp4_kernel(const __nv_bfloat16* __restrict__ v, TokenLayout in,
                                                                      const float* __restrict__ low, const float* __restrict__ high,
                                                                      int n_tokens, uint8_t* __restrict__ codes, uint8_t* __restrict__ sf,
                                                                      float* __restrict__ v_outer) {
    __shared__ float tile[KEY_TILE][HEAD_DIM + 1];  // by slot
    const int head = blockIdx.y, t = blockIdx.x;
    for (int item = threadIdx.x; item < KEY_TILE * 16; item += FP4_THREADS) {
        const int slot = item / 16, chunk = item % 16, key = t * KEY_TILE + slot_key(slot);
        float f[8];
        if (key < n_tokens) {
            const uint4 raw = load_bf16x8(v + in.offset(head, key) + chunk * 8, in.half);
            const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 p = __bfloat1622float2(pairs[i]);
                f[2 * i] = p.x, f[2 * i + 1] = p.y;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) tile[slot][chunk * 8 + i] = f[i];
    }
    __syncthreads();
    uint8_t* tile_codes = codes + (size_t(head) * gridDim.x + t) * (V4_ROWS * 32);
    uint8_t* tile_sf = sf + (size_t(head) * gridDim.x + t) * (V4_SF_WORDS * 4);
    for (int item = threadIdx.x; item < HEAD_DIM * 4; item += FP4_THREADS) {
        const int c = item % HEAD_DIM, block = item / HEAD_DIM;  // block of 16 slots
        const int ci = head * HEAD_DIM + c;
        const float outer = fmaxf(fmaxf(high[ci], -low[ci]) * (1.0f / 2688.0f), 1e-30f);
        if (t == 0 && block == 0) v_outer[ci] = outer;
        float x[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = tile[block * 16 + i][c];
        uint32_t byte;
        uint2 packed;
        quantize_block16(x, outer, byte, packed);
        *reinterpret_cast<uint2*>(tile_codes + ((block / 2) * V4_ROWS + c) * 16 + (block % 2) * 8) = packed;
        tile_sf[((c % 32) * 4 + c / 32) * 4 + block] = uint8_t(byte);  // word c / 32 of lane c % 32
    }
    for (int item = threadIdx.x; item < 2 * 16 * 4; item += FP4_THREADS) {  // the rows of ones: 2 chunks x 16 rows x 4 words
        const int chunk = item / 64, row = 128 + item / 4 % 16, word = item % 4;
        reinterpret_cast<uint32_t*>(tile_codes + (chunk * V4_ROWS + row) * 16)[word] = 0x22222222u;
    }
    if (threadIdx.x < 128)  // second block: rows 128..143 (ones) are word 0 of lanes 0..15, the rest zeros
        reinterpret_cast<uint32_t*>(tile_sf)[128 + threadIdx.x] = threadIdx.x % 4 == 0 && threadIdx.x / 4 < 16 ? 0x38383838u : 0u;
}

// The part of the scores that Q smoothing took out, added back exactly (bench/emulate.py:308-309; the reference's
// smooth_bias kernel, csrc/flash.cu:1254-1322, gets there with three bf16 MMAs): for every block of `mean_tokens`
// queries and every key, q_mean[block] . (k - k_mean) to FP32 accuracy, times scale_log2, keys of a tile in slot
// order, -inf past the last key.  bias: [heads][q_blocks][k_tiles * 64].
//
// On the tensor core: D[128 keys][64 query blocks] = Kc . Qm^T as kind::tf32, every FP32 value split into two tf32
// parts and the product taken as hi.hi + lo.hi + hi.lo.  Keys are the rows, so a thread of the epilogue holds one
// key's terms for 16 query blocks and a warp's stores are 128 contiguous bytes of one table row.  A block keeps the
// images of its 64 query blocks' means and walks over pairs of key tiles of one head, half the channels at a time:
// centred K (rotated first when a table is given) -> images of 64 channels -> 24 instructions of K = 8, into one of two
// accumulators.  The instructions of one half run while the other half's images are made and the pair before is
// written out.  Grid (strips of key-tile pairs, heads, ceil(q_blocks / 64)).
constexpr int BIAS_KEYS = 2 * KEY_TILE;  // rows of an instruction: two K4 tiles
constexpr int BIAS_BLOCKS = 64;          // query blocks per pass (columns)
constexpr int BIAS_THREADS = 512;
constexpr int BIAS_HALF = HEAD_DIM / 2;  // channels per set of images
struct __align__(128) BiasSmem {
    float k_hi[2][BIAS_HALF / 4][BIAS_KEYS][4];  // operand images, one per half: [channel / 4][row][4 values]
    float k_lo[2][BIAS_HALF / 4][BIAS_KEYS][4];
    float q_hi[HEAD_DIM / 4][BIAS_BLOCKS][4];
    float q_lo[HEAD_DIM / 4][BIAS_BLOCKS][4];
    uint64_t done[2];  // the instructions of a half have completed (its images are free; after the second, the accumulator is whole)
    uint32_t tmem_base;
    int abort_flag;
};
constexpr uint32_t IDESC_BIAS = idesc_tf32(BIAS_KEYS, BIAS_BLOCKS);

// x = hi + lo with hi rounded to tf32's 11 significant bits (to nearest, ties away from zero) and lo exact: the tensor
// core drops what lo has below its own 11 bits, at most 2^-23 |x|.
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
    hi = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
    lo = x - hi;
}
__device__ __forceinline__ void split4(const float (&x)[4], float4& hi, float4& lo) {
    split_tf32(x[0], hi.x, lo.x);
    split_tf32(x[1], hi.y, lo.y);
    split_tf32(x[2], hi.z, lo.z);
    split_tf32(x[3], hi.w, lo.w);
}

__global__ void __launch_bounds__(BIAS_THREADS, 1) smooth_bias_kernel(const __nv_bfloat16* __restrict__ k, TokenLayout in,
                                                                      const float* __restrict__ k_mean, const float* __restrict__ q_mean,
                                                                      int q_blocks, int n_keys, float scale_log2, float* __restrict__ bias,
                                                                      RopeTable rope, int* status) {
    extern __shared__ __align__(128) uint8_t bias_smem_raw[];
    BiasSmem& sm = *reinterpret_cast<BiasSmem*>((reinterpret_cast<uintptr_t>(bias_smem_raw) + 127) & ~uintptr_t(127));
    const int head = blockIdx.y, b0 = blockIdx.z * BIAS_BLOCKS, warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int k_tiles = (n_keys + KEY_TILE - 1) / KEY_TILE, pairs = (k_tiles + 1) / 2;
    volatile int* abort_flag = &sm.abort_flag;
    if (threadIdx.x == 0) {
        sm.abort_flag = 0;
        mbar_init(&sm.done[0], 1);
        mbar_init(&sm.done[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(&sm.tmem_base, 2 * BIAS_BLOCKS);
    // the means of this pass's query blocks, rows past the last block zero
    for (int item = threadIdx.x; item < BIAS_BLOCKS * (HEAD_DIM / 4); item += BIAS_THREADS) {
        const int r = item % BIAS_BLOCKS, c4 = item / BIAS_BLOCKS;
        float x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (b0 + r < q_blocks) {
            const float4 m = *reinterpret_cast<const float4*>(q_mean + (size_t(head) * q_blocks + b0 + r) * HEAD_DIM + c4 * 4);
            x[0] = m.x, x[1] = m.y, x[2] = m.z, x[3] = m.w;
        }
        float4 hi, lo;
        split4(x, hi, lo);
        *reinterpret_cast<float4*>(sm.q_hi[c4][r]) = hi;
        *reinterpret_cast<float4*>(sm.q_lo[c4][r]) = lo;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    const float* mean = k_mean + head * HEAD_DIM;
    // A thread makes the images of one key (threads in key order: conflict-free 16-byte stores), 16 channels of each half
    const int r = threadIdx.x % BIAS_KEYS, g0 = 2 * (threadIdx.x / BIAS_KEYS);  // groups of 8 channels g0, g0 + 1 of a half
    float mine[2][16];  // the mean of K in this thread's channels
#pragma unroll
    for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int j = 0; j < 16; ++j) mine[half][j] = mean[half * BIAS_HALF + g0 * 8 + j];
    auto key_of = [&](int pair) { return (2 * pair + r / KEY_TILE) * KEY_TILE + slot_key(r % KEY_TILE); };
    auto fetch = [&](int pair, int half, uint4 (&raw)[2]) {  // 32 contiguous bytes of the key's row
        const int key = key_of(pair);
        if (key < n_keys) {
            const __nv_bfloat16* src = k + in.offset(head, key) + half * BIAS_HALF + g0 * 8;
            raw[0] = load_bf16x8(src, in.half), raw[1] = load_bf16x8(src + 8, in.half);
        } else {
            raw[0] = raw[1] = make_uint4(0, 0, 0, 0);
        }
    };
    auto make_images = [&](int pair, int half, const uint4 (&raw)[2]) {
        const int key = key_of(pair);
        const bool live = key < n_keys;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int g = g0 + i, channel = half * BIAS_HALF + g * 8;
            float x[8];
            const __nv_bfloat162* two = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(two[j]);
                x[2 * j] = f.x, x[2 * j + 1] = f.y;
            }
            if (live) {
                if (rope.table) rope8(x, rope.row(in, head, key), channel);
#pragma unroll
                for (int j = 0; j < 8; ++j) x[j] -= mine[half][i * 8 + j];
            }
            float4 hi, lo;
            split4(reinterpret_cast<const float(&)[4]>(x[0]), hi, lo);
            *reinterpret_cast<float4*>(sm.k_hi[half][2 * g][r]) = hi;
            *reinterpret_cast<float4*>(sm.k_lo[half][2 * g][r]) = lo;
            split4(reinterpret_cast<const float(&)[4]>(x[4]), hi, lo);
            *reinterpret_cast<float4*>(sm.k_hi[half][2 * g + 1][r]) = hi;
            *reinterpret_cast<float4*>(sm.k_lo[half][2 * g + 1][r]) = lo;
        }
    };
    // The block's pairs are counted by `turn`: accumulator turn & 1, and the barriers' phase parity turn & 1.
    // the 24 instructions of one half of a pair, by one thread; half 0 starts the accumulator afresh
    auto issue = [&](int turn, int half) {
        if (warp == 0 && elect_one()) {
            tc_fence_after();
            const uint32_t acc = tmem + (turn & 1) * BIAS_BLOCKS;
            const uint64_t k_hi = smem_desc(smem_u32(sm.k_hi[half]), BIAS_KEYS * 16, 128), k_lo = smem_desc(smem_u32(sm.k_lo[half]), BIAS_KEYS * 16, 128);
            const uint64_t q_hi = smem_desc(smem_u32(sm.q_hi[half * (BIAS_HALF / 4)]), BIAS_BLOCKS * 16, 128);
            const uint64_t q_lo = smem_desc(smem_u32(sm.q_lo[half * (BIAS_HALF / 4)]), BIAS_BLOCKS * 16, 128);
            // a descriptor's address counts 16-byte units; an instruction takes two chunks of each image
#pragma unroll
            for (int ks = 0; ks < BIAS_HALF / 8; ++ks) mma_tf32_ss(acc, k_hi + ks * (2 * BIAS_KEYS), q_hi + ks * (2 * BIAS_BLOCKS), IDESC_BIAS, half + ks > 0);
#pragma unroll
            for (int ks = 0; ks < BIAS_HALF / 8; ++ks) mma_tf32_ss(acc, k_lo + ks * (2 * BIAS_KEYS), q_hi + ks * (2 * BIAS_BLOCKS), IDESC_BIAS, true);
#pragma unroll
            for (int ks = 0; ks < BIAS_HALF / 8; ++ks) mma_tf32_ss(acc, k_hi + ks * (2 * BIAS_KEYS), q_lo + ks * (2 * BIAS_BLOCKS), IDESC_BIAS, true);
            mma_commit(&sm.done[half]);
        }
        __syncwarp();
    };
    // one warp watches the barrier, everybody learns the outcome
    auto wait_done = [&](int half, int turn) {
        return __syncthreads_and(warp != 0 || mbar_wait(&sm.done[half], turn & 1, abort_flag, status, STATUS_WAIT_SCORES)) != 0;
    };
    // warp w: the 32 keys of lane quarter w % 4, query blocks 16 (w / 4) .. + 15 of this pass
    auto write_out = [&](int pair, int turn) {
        float2 d[8];
        tc_fence_after();
        tmem_ld16_sync(tmem + (uint32_t((warp % 4) * 32) << 16) + (turn & 1) * BIAS_BLOCKS + (warp / 4) * 16, d);
        tc_fence_before();
        const int row = (warp % 4) * 32 + lane, tile = 2 * pair + row / KEY_TILE, slot = row % KEY_TILE;
        if (tile < k_tiles) {
            const bool live = tile * KEY_TILE + slot_key(slot) < n_keys;  // slots past the last key: -inf keeps them out of the softmax
            float* at = bias + (size_t(head) * q_blocks + b0 + (warp / 4) * 16) * (size_t(k_tiles) * KEY_TILE) + tile * KEY_TILE + slot;
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (b0 + (warp / 4) * 16 + j < q_blocks) at[size_t(j) * k_tiles * KEY_TILE] = live ? (j % 2 ? d[j / 2].y : d[j / 2].x) * scale_log2 : -INFINITY;
        }
    };

    bool ok = true;
    int last = -1, turn = 0;       // the pair whose instructions are in flight; this block's count of pairs
    int seen[2] = {0, 0}, sent[2] = {0, 0};  // per half: completions waited for, sets of instructions issued
    uint4 raw[2][2], ahead[2][2];  // this pair's and the next pair's 2 x 32 bytes of the thread's key: loaded a whole pair ahead
    if (blockIdx.x < pairs) fetch(blockIdx.x, 0, raw[0]), fetch(blockIdx.x, 1, raw[1]);
    for (int pair = blockIdx.x; pair < pairs; pair += gridDim.x, ++turn) {
        const int next = pair + gridDim.x;
        if (next < pairs) fetch(next, 0, ahead[0]), fetch(next, 1, ahead[1]);
        // images 0 were last read by the first half of the pair before: waited for at the end of that turn
        make_images(pair, 0, raw[0]);
        fence_proxy_async();  // the images, written through the generic proxy, are read by the tensor core
        __syncthreads();
        issue(turn, 0);
        ++sent[0];
        if (last >= 0) {
            ok = wait_done(1, turn - 1);  // the pair before is whole (and images 1 are free)
            if (!ok) break;
            ++seen[1];
            write_out(last, turn - 1);
        }
        make_images(pair, 1, raw[1]);
        fence_proxy_async();
        __syncthreads();  // also: the accumulator of the pair before has been read before anything is issued into it again
        issue(turn, 1);
        ++sent[1];
        last = pair;
        ok = wait_done(0, turn);  // images 0 are free for the next pair
        if (!ok) break;
        ++seen[0];
#pragma unroll
        for (int half = 0; half < 2; ++half) raw[half][0] = ahead[half][0], raw[half][1] = ahead[half][1];
    }
    if (ok && last >= 0) {
        ok = wait_done(1, turn - 1);
        if (ok) ++seen[1], write_out(last, turn - 1);
    }
    if (!ok && threadIdx.x == 0) {  // whatever was issued must finish before tensor memory is freed
        int never = 0;
        for (int half = 0; half < 2; ++half)
            if (sent[half] > seen[half]) mbar_wait(&sm.done[half], (sent[half] - 1) & 1, &never, nullptr, 0);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, 2 * BIAS_BLOCKS);
    }
}

}  // namespace unica

using namespace unica;

extern "C" int unica_b200_nvfp4_outer(const float* mean, const float* low, const float* high, int heads, int groups,
                                      float* outer, void* stream) {
    if (!low || !high || !outer) return unica_fail(UNICA_B200_ERR_ARGUMENT, "nvfp4_outer: null pointer");
    if (heads <= 0 || groups <= 0) return unica_fail(UNICA_B200_ERR_ARGUMENT, "nvfp4_outer: heads and groups must be positive");
    nvfp4_outer_rows_kernel<<<heads, HEAD_DIM, 0, static_cast<cudaStream_t>(stream)>>>(mean, low, high, groups, outer);
    return unica_check_launch("nvfp4_outer");
}

static int quantize_fp4_rows(const void* x, unica_token_layout layout, const float* mean, int mean_tokens, RopeTable rope,
                             const float* outer, int heads, int n_tokens, int rows_per_tile, int tiles, uint8_t* codes, uint8_t* sf,
                             void* stream) {
    if (!x || !outer || !codes || !sf) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_fp4_rows: null pointer");
    if (heads <= 0 || n_tokens <= 0) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_fp4_rows: heads and n_tokens must be positive");
    if (rows_per_tile != 128 && rows_per_tile != 64)
        return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_fp4_rows: rows_per_tile must be 128 (Q) or 64 (K, slot order)");
    if (tiles < (n_tokens + rows_per_tile - 1) / rows_per_tile) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_fp4_rows: tiles does not cover n_tokens");
    if (mean && mean_tokens <= 0) mean_tokens = n_tokens;
    if (!mean) mean_tokens = n_tokens;
    const int groups = (n_tokens + mean_tokens - 1) / mean_tokens;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
    if (rows_per_tile == 128)
        quantize_rows_fp4_kernel<128, false><<<dim3(tiles, heads), FP4_THREADS, 0, s>>>(xb, to_layout(layout), mean, mean_tokens, groups, outer, n_tokens, codes, sf, rope);
    else
        quantize_rows_fp4_kernel<64, true><<<dim3(tiles, heads), FP4_THREADS, 0, s>>>(xb, to_layout(layout), mean, mean_tokens, groups, outer, n_tokens, codes, sf, rope);
    return unica_check_launch("quantize_fp4_rows");
}

extern "C" int unica_b200_quantize_fp4_rows(const void* x, unica_token_layout layout, const float* mean, int mean_tokens,
                                            const float* outer, int heads, int n_tokens, int rows_per_tile, int tiles,
                                            uint8_t* codes, uint8_t* sf, void* stream) {
    return quantize_fp4_rows(x, layout, mean, mean_tokens, RopeTable{nullptr, 0}, outer, heads, n_tokens, rows_per_tile, tiles, codes, sf, stream);
}

extern "C" int unica_b200_quantize_fp4_rows_rope(const void* x, unica_token_layout layout, const float* mean, int mean_tokens,
                                                 const void* rope, long long rope_batch_stride, const float* outer, int heads,
                                                 int n_tokens, int rows_per_tile, int tiles, uint8_t* codes, uint8_t* sf, void* stream) {
    if (!rope) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_fp4_rows_rope: null table");
    return quantize_fp4_rows(x, layout, mean, mean_tokens, RopeTable{static_cast<const __half*>(rope), rope_batch_stride}, outer, heads,
                             n_tokens, rows_per_tile, tiles, codes, sf, stream);
}

extern "C" int unica_b200_quantize_v_fp4(const void* v, unica_token_layout layout, const float* low, const float* high,
                                         int heads, int n_tokens, uint8_t* codes, uint8_t* sf, float* v_outer, void* stream) {
    if (!v || !low || !high || !codes || !sf || !v_outer) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_v_fp4: null pointer");
    if (heads <= 0 || n_tokens <= 0) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_v_fp4: heads and n_tokens must be positive");
    const int tiles = (n_tokens + KEY_TILE - 1) / KEY_TILE;
    quantize_v_fp4_kernel<<<dim3(tiles, heads), FP4_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(v), to_layout(layout), low, high, n_tokens, codes, sf, v_outer);
    return unica_check_launch("quantize_v_fp4");
}

static int smooth_bias(const void* k, unica_token_layout layout, const float* k_mean, const float* q_mean, RopeTable rope, int heads,
                       int q_blocks, int n_keys, float scale_log2, float* bias, int* status, void* stream) {
    if (!k || !k_mean || !q_mean || !bias || !status) return unica_fail(UNICA_B200_ERR_ARGUMENT, "smooth_bias: null pointer");
    if (heads <= 0 || q_blocks <= 0 || n_keys <= 0) return unica_fail(UNICA_B200_ERR_ARGUMENT, "smooth_bias: heads, q_blocks and n_keys must be positive");
    if (int e = unica_check_device()) return e;
    const int tiles = (n_keys + KEY_TILE - 1) / KEY_TILE, pairs = (tiles + 1) / 2, passes = (q_blocks + BIAS_BLOCKS - 1) / BIAS_BLOCKS;
    if (heads > 65535 || passes > 65535) return unica_fail(UNICA_B200_ERR_ARGUMENT, "smooth_bias: more than 65535 heads or passes of 64 query blocks");
    constexpr int SMEM = int(sizeof(BiasSmem)) + 128;
    if (cudaFuncSetAttribute(smooth_bias_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
        return unica_check_launch("smooth_bias (shared memory size)");
    // a block per SM (its images take most of the shared memory); at most four full waves of blocks, each walking over
    // its strip of key-tile pairs with the query blocks' images built once
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
        return unica_check_launch("smooth_bias (device)");
    const long long others = (long long)heads * passes;
    const int strips = int(std::min<long long>(pairs, std::max<long long>(1, 4LL * sms / others)));
    smooth_bias_kernel<<<dim3(strips, heads, passes), BIAS_THREADS, SMEM, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(k), to_layout(layout), k_mean, q_mean, q_blocks, n_keys, scale_log2, bias, rope, status);
    return unica_check_launch("smooth_bias");
}

extern "C" int unica_b200_smooth_bias(const void* k, unica_token_layout layout, const float* k_mean, const float* q_mean,
                                      int heads, int q_blocks, int n_keys, float scale_log2, float* bias, int* status, void* stream) {
    return smooth_bias(k, layout, k_mean, q_mean, RopeTable{nullptr, 0}, heads, q_blocks, n_keys, scale_log2, bias, status, stream);
}

extern "C" int unica_b200_smooth_bias_rope(const void* k, unica_token_layout layout, const float* k_mean, const float* q_mean,
                                           const void* rope, long long rope_batch_stride, int heads, int q_blocks, int n_keys,
                                           float scale_log2, float* bias, int* status, void* stream) {
    if (!rope) return unica_fail(UNICA_B200_ERR_ARGUMENT, "smooth_bias_rope: null table");
    return smooth_bias(k, layout, k_mean, q_mean, RopeTable{static_cast<const __half*>(rope), rope_batch_stride}, heads, q_blocks, n_keys,
                       scale_log2, bias, status, stream);
}
