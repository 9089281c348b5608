// The INT8 quantizers' tile routines, shared by the one-tile-per-block kernels (quantize.cu) and the kernels that take a
// head's statistics and quantize it in one launch (quantize_fused.cu).
#pragma once

#include "common.cuh"

namespace unica {

constexpr int THREADS = 256;

__device__ __forceinline__ void load8(float (&v)[8], const __nv_bfloat16* src, bool half) {
    const uint4 raw = load_bf16x8(src, half);
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(pairs[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

template <int NT = THREADS>
__device__ __forceinline__ float block_max(float x, float* scratch) {
#pragma unroll
    for (int d = 16; d > 0; d /= 2) x = fmaxf(x, __shfl_xor_sync(0xffffffff, x, d));
    if (threadIdx.x % 32 == 0) scratch[threadIdx.x / 32] = x;
    __syncthreads();
    x = scratch[0];
#pragma unroll
    for (int w = 1; w < NT / 32; ++w) x = fmaxf(x, scratch[w]);
    return x;
}

// rint(x / scale) as the reference computes it (an IEEE division, then round to nearest even), two elements at a time and
// without the division: with y = rn(1 / scale), q0 = rn(x y), r = x - q0 scale (exact in a fused multiply-add) and
// q1 = rn(q0 + r y), q1 is the correctly rounded quotient (Markstein's correction step: it holds whenever y is the correctly
// rounded reciprocal and q0 a faithful quotient, which rn(x y) is unless the mantissa of scale is all ones; a tile whose
// scale is such a number takes the division itself, see needs_division).  q1 + 1.5 * 2^23 then has rint(q1), in two's
// complement, in its low mantissa bits.  No clamp: scale is at least max |x| / 127 rounded, so |q1| < 127.5.
__device__ __forceinline__ float2 sub2(float2 a, float2 b) {
    float2 d;
    asm("sub.rn.f32x2 %0, %1, %2;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
    return d;
}
__device__ __forceinline__ float2 quotient_code2(float2 x, float2 inv2, float2 minus_scale2) {
    const float2 q0 = mul2(x, inv2);
    const float2 q1 = fma2(fma2(q0, minus_scale2, x), inv2, q0);
    return add2(q1, make_float2(MAGIC, MAGIC));
}
__device__ __forceinline__ bool needs_division(float scale) { return (__float_as_uint(scale) & 0x7fffffu) == 0x7fffffu; }
__device__ __forceinline__ float code_by_division(float x, float scale) { return rintf(__fdiv_rn(x, scale)) + MAGIC; }
// the low bytes of four such floats in one word
__device__ __forceinline__ uint32_t low_bytes(float2 a, float2 b) {
    return __byte_perm(__byte_perm(__float_as_uint(a.x), __float_as_uint(a.y), 0x0040), __byte_perm(__float_as_uint(b.x), __float_as_uint(b.y), 0x0040),
                       0x5410);
}
// A tile staged in shared memory by the streaming kernels: 64 rows (tokens) of 256 bytes in token order, the eight
// 32-byte pieces of a row swapped about by the row number, so that threads on consecutive rows and the same channels
// (the quantizers' mapping: it keeps their stores to the operand image contiguous) fall on different banks.
// Address of the 32-byte piece `chunk` (channels 16 chunk .. + 15) of row `row`:
__device__ __forceinline__ const __nv_bfloat16* staged_chunk(const __nv_bfloat16* tile, int row, int chunk) {
    return tile + row * HEAD_DIM + ((chunk ^ (row & 7)) * 16);
}
__device__ __forceinline__ uint32_t staged_offset(int row, int piece16) {  // in bytes, of the 16-byte piece (channels 8 piece16 .. + 7)
    return uint32_t(row * 256 + ((((piece16 >> 1) ^ (row & 7)) << 5) | ((piece16 & 1) << 4)));
}

// eight bfloat16 (as load_bf16x8 returns them) as four float2
__device__ __forceinline__ void unpack8(const uint4 raw, float2 (&v)[4]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
}

// Q or K (minus `mean`, [heads][128] or null) in INT8 with one scale per tile of ROWS tokens (128: Q, 64: K).
// One block per tile; the tile stays in registers between the max and the write, so HBM is read once.
// codes: [heads][tiles][8 chunks of 16 channels][ROWS][16] bytes; rows past n_tokens and tiles past the last are zeros.
// scales: [heads][tiles].  Grid (tiles, heads).
// mean: this head's [128] (global or shared memory) or null; out: the tile's ROWS x 128 bytes; scale_out: its scale;
// scratch: NT / 32 floats of shared memory, free again after the next __syncthreads().  NT: the block's threads.
// staged: the tile's rows already in shared memory as the streaming kernels lay them out (see staged_chunk; then x is not
// read), or null.
template <int ROWS, int NT = THREADS>
__device__ __forceinline__ void rows_int8_tile(const __nv_bfloat16* __restrict__ x, const TokenLayout& in, const float* mean, int head,
                                               int tile, int n_tokens, int8_t* __restrict__ out, float* __restrict__ scale_out,
                                               const RopeTable& rope, float* scratch, const __nv_bfloat16* staged = nullptr) {
    constexpr int ITEMS = ROWS * 8 / NT;  // (row, 16-channel chunk) items per thread
    const int token0 = tile * ROWS;
    float2 v[ITEMS][8];
    float local = 0.0f;
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
        const int item = it * NT + threadIdx.x, row = item % ROWS, chunk = item / ROWS;
        if (token0 + row < n_tokens) {
            const __nv_bfloat16* src = staged ? staged_chunk(staged, row, chunk) : x + in.offset(head, token0 + row) + chunk * 16;
            float2 a[4], b[4];
            unpack8(load_bf16x8(src, in.half), a);
            unpack8(load_bf16x8(src + 8, in.half), b);
            if (rope.table) {  // rotate first, then take the mean (of the rotated x) away
                const __half* f = rope.row(in, head, token0 + row);
                rope8(*reinterpret_cast<float(*)[8]>(a), f, chunk * 16);
                rope8(*reinterpret_cast<float(*)[8]>(b), f, chunk * 16 + 8);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2* m2 = reinterpret_cast<const float2*>(mean + chunk * 16);
                v[it][i] = mean ? sub2(a[i], m2[i]) : a[i];
                v[it][4 + i] = mean ? sub2(b[i], m2[4 + i]) : b[i];
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[it][i] = make_float2(0.0f, 0.0f);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) local = max3(local, fabsf(v[it][i].x), fabsf(v[it][i].y));
    }
    const float scale = fmaxf(block_max<NT>(local, scratch) * (1.0f / 127.0f), 1e-12f);
    const float inv = __frcp_rn(scale);
    const float2 inv2 = make_float2(inv, inv), minus_scale2 = make_float2(-scale, -scale);
    const bool divide = needs_division(scale);  // practically never
    if (threadIdx.x == 0) *scale_out = scale;
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
        const int item = it * NT + threadIdx.x, row = item % ROWS, chunk = item / ROWS;
        float2 t[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) t[i] = quotient_code2(v[it][i], inv2, minus_scale2);
        if (divide) {
#pragma unroll
            for (int i = 0; i < 8; ++i) t[i] = make_float2(code_by_division(v[it][i].x, scale), code_by_division(v[it][i].y, scale));
        }
        *reinterpret_cast<uint4*>(out + (chunk * ROWS + row) * 16) =
            make_uint4(low_bytes(t[0], t[1]), low_bytes(t[2], t[3]), low_bytes(t[4], t[5]), low_bytes(t[6], t[7]));
    }
}

// V in INT8, one block per tile of 64 keys.  PER_TOKEN false: one scale per channel, max(|low|, |high|) * (1/127) from
// the channel's min and max over the head (low, high: [heads][128]); true: one scale per key over its channels, and
// v_token [heads][tiles][2][64] gets log2 s and 1 / s of the tile's keys (zeros past n_tokens).  skip: [heads][n_tokens],
// 1 = the key is written as zeros (outlier keys), or null.
// v8: [heads][tiles][4 chunks of 16 keys][128 channels][16] bytes: the K-major B operand of P.V.  v_scale [heads][128].
template <bool PER_TOKEN, int NT = THREADS, bool STAGED = false>
__device__ __forceinline__ void v_int8_emit(const __nv_bfloat16 (*tile)[HEAD_DIM], bool half, const float* key_scale, const float* key_inv,
                                            const float* low, const float* high, int head, int t, int tiles, int8_t* __restrict__ v8,
                                            float* __restrict__ v_scale);
struct VTileSmem {
    __align__(16) __nv_bfloat16 tile[KEY_TILE][HEAD_DIM];
    float key_scale[KEY_TILE], key_inv[KEY_TILE];
};
// low, high: this head's [128] (global or shared memory); tiles: key tiles per head; v_scale [heads][128] or null (the
// caller writes it); sm: free again after a __syncthreads().
template <bool PER_TOKEN>
__device__ __forceinline__ void v_int8_tile(const __nv_bfloat16* __restrict__ v, const TokenLayout& in, const float* low, const float* high,
                                            const uint8_t* __restrict__ skip, int head, int t, int tiles, int n_tokens,
                                            int8_t* __restrict__ v8, float* __restrict__ v_scale, float* __restrict__ v_token,
                                            VTileSmem& sm) {
    // The tile goes through shared memory as bf16, keys x channels, and comes out transposed: a thread then owns one
    // channel and 16 keys, i.e. one 16-byte row of the operand image, and a warp writes 512 contiguous bytes.
    auto& tile = sm.tile;
    auto& key_scale = sm.key_scale;
    auto& key_inv = sm.key_inv;
    const int token0 = t * KEY_TILE;
    const int chunk = threadIdx.x % 16;  // 8 channels
#pragma unroll
    for (int it = 0; it < KEY_TILE * 16 / THREADS; ++it) {
        const int key = it * (THREADS / 16) + threadIdx.x / 16;
        const bool valid = token0 + key < n_tokens;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (valid && !(skip && skip[size_t(head) * n_tokens + token0 + key]))
            raw = load_bf16x8(v + in.offset(head, token0 + key) + chunk * 8, in.half);
        *reinterpret_cast<uint4*>(&tile[key][chunk * 8]) = raw;
        if (PER_TOKEN) {  // one scale per key over its channels: the 16 threads of a key share their maxima
            const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(pairs[i]);
                amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
            }
#pragma unroll
            for (int d = 8; d > 0; d /= 2) amax = fmaxf(amax, __shfl_xor_sync(0xffffffff, amax, d));
            if (chunk == 0) {
                const float s = fmaxf(amax * (1.0f / 127.0f), 1e-12f);
                key_scale[key] = s;
                key_inv[key] = __frcp_rn(s);
                float* tok = v_token + (size_t(head) * tiles + t) * 2 * KEY_TILE;
                tok[key] = valid ? log2f(s) : 0.0f;
                tok[KEY_TILE + key] = valid ? __fdiv_rn(1.0f, s) : 0.0f;
            }
        }
    }
    __syncthreads();
    v_int8_emit<PER_TOKEN>(tile, false, key_scale, key_inv, low, high, head, t, tiles, v8, v_scale);
}

// The second half of v_int8_tile: the tile in shared memory (keys x channels, zeros past the last key; float16 bits if
// `half`, which then count as their bfloat16 rounding; STAGED: laid out as staged_chunk describes) to the operand image.
template <bool PER_TOKEN, int NT, bool STAGED>
__device__ __forceinline__ void v_int8_emit(const __nv_bfloat16 (*tile)[HEAD_DIM], bool half, const float* key_scale, const float* key_inv,
                                            const float* low, const float* high, int head, int t, int tiles, int8_t* __restrict__ v8,
                                            float* __restrict__ v_scale) {
    // Thread = (two channels, KEYS keys): KEYS loads of 32 bits down its column pair, KEYS bytes of two rows of the image out.
    constexpr int KEYS = (HEAD_DIM / 2) * KEY_TILE / NT;  // 16 with 256 threads, 8 with 512
    static_assert(KEYS == 16 || KEYS == 8, "a whole or half a 16-byte row per thread");
    const int c = threadIdx.x % (HEAD_DIM / 2) * 2, keys = threadIdx.x / (HEAD_DIM / 2) * KEYS;
    float2 scale2 = make_float2(1.0f, 1.0f), inv2 = make_float2(1.0f, 1.0f);
    if (!PER_TOKEN) {  // max(|low|, |high|) * (1/127) from the channel's minimum and maximum over the head
        scale2 = make_float2(fmaxf(fmaxf(high[c], -low[c]) * (1.0f / 127.0f), 1e-12f), fmaxf(fmaxf(high[c + 1], -low[c + 1]) * (1.0f / 127.0f), 1e-12f));
        inv2 = make_float2(__frcp_rn(scale2.x), __frcp_rn(scale2.y));
    }
    if (t == 0 && v_scale && keys == 0) *reinterpret_cast<float2*>(v_scale + head * HEAD_DIM + c) = scale2;
    float2 minus_scale2 = make_float2(-scale2.x, -scale2.y);
    bool divide = !PER_TOKEN && (needs_division(scale2.x) || needs_division(scale2.y));
    // row (16-key chunk, channel) of the image, this thread's KEYS bytes of it, eight keys at a time
    uint8_t* dst = reinterpret_cast<uint8_t*>(v8 + (size_t(head) * tiles + t) * (KEY_TILE * HEAD_DIM)) + ((keys / 16) * HEAD_DIM + c) * 16 + keys % 16;
#pragma unroll
    for (int step = 0; step < KEYS / 8; ++step) {
        float2 code[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int key = keys + 8 * step + j;
            const uint32_t two = STAGED ? *reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(tile) + staged_offset(key, c / 8) + c % 8 * 2)
                                        : *reinterpret_cast<const uint32_t*>(&tile[key][c]);
            float2 x;
            if (half) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&two));
                x = __bfloat1622float2(__floats2bfloat162_rn(f.x, f.y));
            } else {
                x = make_float2(__uint_as_float(two << 16), __uint_as_float(two & 0xffff0000u));
            }
            if (PER_TOKEN) {
                const float s = key_scale[key], inv = key_inv[key];
                scale2 = make_float2(s, s), inv2 = make_float2(inv, inv), minus_scale2 = make_float2(-s, -s);
                divide = needs_division(s);
            }
            code[j] = quotient_code2(x, inv2, minus_scale2);
            if (divide) code[j] = make_float2(code_by_division(x.x, scale2.x), code_by_division(x.y, scale2.y));
            if (!STAGED && !PER_TOKEN) {  // low and high come from the caller: a value outside them must not wrap around
                code[j].x = fminf(fmaxf(code[j].x, MAGIC - 127.0f), MAGIC + 127.0f);
                code[j].y = fminf(fmaxf(code[j].y, MAGIC - 127.0f), MAGIC + 127.0f);
            }
        }
        uint32_t first[2], second[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            first[i] = low_bytes(make_float2(code[4 * i].x, code[4 * i + 1].x), make_float2(code[4 * i + 2].x, code[4 * i + 3].x));
            second[i] = low_bytes(make_float2(code[4 * i].y, code[4 * i + 1].y), make_float2(code[4 * i + 2].y, code[4 * i + 3].y));
        }
        *reinterpret_cast<uint2*>(dst + 8 * step) = make_uint2(first[0], first[1]);
        *reinterpret_cast<uint2*>(dst + 16 + 8 * step) = make_uint2(second[0], second[1]);
    }
}

}  // namespace unica
