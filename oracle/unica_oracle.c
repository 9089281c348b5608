/* CPU oracle for the quantized-attention forward path.  TEST INFRASTRUCTURE ONLY: the checker the CUDA path is
 * compared with, and the timed CPU baseline.  Nothing in the product imports, links or runs it.
 *
 * A restatement in plain C of the arithmetic of the reference's emulator and quantizer kernels, function by function
 * (citations are paths inside the reference project):
 *
 *   uo_channel_stats      csrc/flash.cu:287-327 (rope_stats, fixed summation order) + unica/__init__.py:592-612
 *   uo_quantize_int8      bench/emulate.py:36-47,154-159 (token_scale, quant) == csrc/flash.cu:334-372
 *   uo_quantize_v_channel bench/emulate.py:288-290 == unica/__init__.py:426-427 + csrc/flash.cu:590-630
 *   uo_quantize_v_token   bench/emulate.py:279-287 == csrc/flash.cu:603-618
 *   uo_nvfp4_rows         bench/emulate.py:98-113 (block_scaled "nvfp4", dim -1) == csrc/flash.cu:1183-1216
 *   uo_nvfp4_v            bench/emulate.py:98-113 (dim -2, outer "channel", slot order 116-119) == csrc/flash.cu:1021-1050
 *   uo_attention_accurate bench/emulate.py:236-369 with TODAY (424) [+ v_token="float" | v_outliers=T]
 *   uo_attention_fast     bench/emulate.py:236-369 with the fast contract (tests/test_fp4.py:24-25,120-126)
 *   uo_reference_fp32     bench/emulate.py:25-33
 *
 * `recip` selects how "tensor / python scalar" is evaluated: 0 = an IEEE division (torch on CPU tensors), 1 = a
 * multiplication by the float reciprocal (torch on CUDA tensors, and the reference kernels: csrc/flash.cu:355-357).
 * With recip = 0 this file is pinned bit for bit (codes, scales) against the emulator run on the CPU
 * (tests/golden/); recip = 1 is the form the GPU kernels are held to.
 *
 * Layouts: every tensor is contiguous [heads][tokens][128]; bf16 values travel as uint16_t.  heads = batch * heads.
 * Build: gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC (oracle/Makefile).  -ffp-contract=off matters: a fused
 * multiply-add would change roundings the bit-exact comparisons rely on.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* Host threads of the OpenMP loops: a launcher may have set OMP_NUM_THREADS=1 for its worker processes. */
int uo_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

#define D 128
#define STATS_TOKENS 256 /* csrc/flash.cu:285 */
#define STATS_LANES 16   /* csrc/flash.cu:286 */
#define TILE 64          /* keys per tile, bench/emulate.py:176 (bc) */
#define LOG2E 1.4426950408889634

static inline float bf16_to_float(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* float -> bf16 -> float, round to nearest even (torch's .bfloat16()) */
static inline float round_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return f; /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    u &= 0xffff0000u;
    memcpy(&f, &u, 4);
    return f;
}

static inline float scalar_div(float a, float b, int recip) { return recip ? a * (1.0f / b) : a / b; }

/* ------------------------------------------------------------------------------------------------------------ */
/* e4m3 (float8_e4m3fn) and e2m1                                                                                  */

/* byte of the e4m3fn value nearest to x >= 0 (ties to even); x <= 448 expected (the callers clamp first,
 * bench/emulate.py:111).  Subnormals down to 2^-9; below half of that: 0. */
static uint8_t float_to_e4m3(float x) {
    if (!(x > 0.0f)) return 0;
    if (x > 448.0f) x = 448.0f;
    int e;
    float m = frexpf(x, &e); /* x = m * 2^e, m in [0.5, 1) */
    int exp = e - 1;         /* x = (2m) * 2^exp, 2m in [1, 2) */
    if (exp < -6) {          /* subnormal: units of 2^-9 */
        float q = rintf(ldexpf(x, 9));
        return (uint8_t)q; /* 0..8; 8 is the smallest normal, 0x08 */
    }
    float q = rintf(ldexpf(m, 4)); /* mantissa with 3 fraction bits: 2m * 8 in [8, 16] */
    if (q == 16.0f) {
        q = 8.0f;
        exp += 1;
    }
    return (uint8_t)(((exp + 7) << 3) | ((int)q - 8));
}

static float e4m3_to_float(uint8_t b) {
    int exp = (b >> 3) & 15, man = b & 7;
    if (exp == 0) return ldexpf((float)man, -9);
    return ldexpf((float)(8 + man), exp - 7 - 3);
}

/* nearest of 0, .5, 1, 1.5, 2, 3, 4, 6 with the sign of x, ties to even, saturating (bench/emulate.py:68-74).
 * Returns the 4-bit code: bit 3 the sign, bits 0-2 the index into that list. */
static const float E2M1_VALUE[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
static uint8_t float_to_e2m1(float x) {
    float a = fabsf(x);
    float step = a < 2.0f ? 0.5f : (a < 4.0f ? 1.0f : 2.0f);
    float r = rintf(a / step) * step;
    if (r > 6.0f) r = 6.0f;
    uint8_t idx = r < 2.0f ? (uint8_t)(r * 2.0f) : (r < 4.0f ? (uint8_t)(r + 2.0f) : (uint8_t)(r * 0.5f + 4.0f));
    /* r: 0,.5,1,1.5 -> 0..3; 2,3 -> 4,5; 4,6 -> 6,7 */
    return (uint8_t)(idx | (signbit(x) ? 8 : 0));
}
static inline float e2m1_to_float(uint8_t c) { return (c & 8) ? -E2M1_VALUE[c & 7] : E2M1_VALUE[c & 7]; }

uint8_t uo_float_to_e4m3(float x) { return float_to_e4m3(x); }
float uo_e4m3_to_float(uint8_t b) { return e4m3_to_float(b); }
uint8_t uo_float_to_e2m1(float x) { return float_to_e2m1(x); }
float uo_e2m1_to_float(uint8_t c) { return e2m1_to_float(c); }

/* slot -> key inside a tile of 64 (bench/emulate.py:116-119, csrc/flash.cu:973-975) */
static inline int slot_key(int k) { return 32 * (k / 32) + 8 * (k % 8 / 2) + 2 * (k % 32 / 8) + k % 2; }
int uo_slot_key(int slot) { return slot_key(slot); }

/* ------------------------------------------------------------------------------------------------------------ */
/* RoPE (bench/emulate.py:122-130)                                                                                */

/* x [heads][n][128] bf16 as float, rotated when rope is given: rope float [tables][n][64][2] = (cos, sin) per pair of
 * channels, already rounded to fp16; head h uses table h / heads_per_table.  out[2i] = c x[2i] - s x[2i+1],
 * out[2i+1] = s x[2i] + c x[2i+1], each product rounded, then the difference or sum (this file is compiled with
 * -ffp-contract=off).  The caller frees the result. */
static float* to_float_rotated(const uint16_t* x, const float* rope, int heads_per_table, int heads, int n) {
    float* out = (float*)malloc(sizeof(float) * (size_t)heads * n * D);
#pragma omp parallel for collapse(2) schedule(static)
    for (int h = 0; h < heads; ++h)
        for (int t = 0; t < n; ++t) {
            const uint16_t* src = x + ((size_t)h * n + t) * D;
            float* dst = out + ((size_t)h * n + t) * D;
            if (!rope) {
                for (int c = 0; c < D; ++c) dst[c] = bf16_to_float(src[c]);
                continue;
            }
            const float* f = rope + ((size_t)(h / heads_per_table) * n + t) * D;
            for (int i = 0; i < D / 2; ++i) {
                float c = f[2 * i], s = f[2 * i + 1], x0 = bf16_to_float(src[2 * i]), x1 = bf16_to_float(src[2 * i + 1]);
                float a = c * x0, b = s * x1, d = s * x0, e = c * x1;
                dst[2 * i] = a - b;
                dst[2 * i + 1] = d + e;
            }
        }
    return out;
}

void uo_rope(const uint16_t* x, const float* rope, int heads_per_table, int heads, int n, float* out) {
    float* r = to_float_rotated(x, rope, heads_per_table, heads, n);
    memcpy(out, r, sizeof(float) * (size_t)heads * n * D);
    free(r);
}

/* ------------------------------------------------------------------------------------------------------------ */
/* statistics                                                                                                     */

/* Per channel of each head: mean, min and max over each group of `per` tokens (per <= 0: the whole head).
 * Sums run in the order of csrc/flash.cu:296-326: inside a block of 256 tokens, lane l of 16 adds tokens l, l+16, ..
 * and the 16 lanes are added in order; the blocks of a group are then added in order and divided by the group's true
 * token count (unica/__init__.py:603-612; torch's own order over the partials is not specified, hence the reference
 * tests' 1e-6).  mean/low/high: [heads][groups][128], groups = ceil(n / per). */
static void channel_stats_f(const float* x, int heads, int n, int per, float* mean, float* low, float* high) {
    if (per <= 0) per = (n + STATS_TOKENS - 1) / STATS_TOKENS * STATS_TOKENS;
    int groups = (n + per - 1) / per;
#pragma omp parallel for collapse(2) schedule(static)
    for (int h = 0; h < heads; ++h)
        for (int g = 0; g < groups; ++g) {
            const float* xh = x + (size_t)h * n * D;
            int t0 = g * per, t1 = t0 + per < n ? t0 + per : n;
            float gs[D], glo[D], ghi[D];
            for (int c = 0; c < D; ++c) gs[c] = 0.0f, glo[c] = INFINITY, ghi[c] = -INFINITY;
            for (int b0 = t0; b0 < t1; b0 += STATS_TOKENS) {
                int b1 = b0 + STATS_TOKENS < t1 ? b0 + STATS_TOKENS : t1;
                float bs[D];
                for (int c = 0; c < D; ++c) bs[c] = 0.0f;
                for (int l = 0; l < STATS_LANES; ++l) {
                    float ls[D];
                    for (int c = 0; c < D; ++c) ls[c] = 0.0f;
                    for (int t = b0 + l; t < b1; t += STATS_LANES)
                        for (int c = 0; c < D; ++c) {
                            float v = xh[(size_t)t * D + c];
                            ls[c] += v;
                            glo[c] = fminf(glo[c], v);
                            ghi[c] = fmaxf(ghi[c], v);
                        }
                    for (int c = 0; c < D; ++c) bs[c] += ls[c];
                }
                for (int c = 0; c < D; ++c) gs[c] += bs[c];
            }
            size_t o = ((size_t)h * groups + g) * D;
            for (int c = 0; c < D; ++c) {
                mean[o + c] = gs[c] / (float)(t1 - t0);
                low[o + c] = glo[c];
                high[o + c] = ghi[c];
            }
        }
}

void uo_channel_stats_rope(const uint16_t* x, const float* rope, int heads_per_table, int heads, int n, int per, float* mean,
                           float* low, float* high) {
    float* xf = to_float_rotated(x, rope, heads_per_table, heads, n);
    channel_stats_f(xf, heads, n, per, mean, low, high);
    free(xf);
}

void uo_channel_stats(const uint16_t* x, int heads, int n, int per, float* mean, float* low, float* high) {
    uo_channel_stats_rope(x, NULL, 1, heads, n, per, mean, low, high);
}

/* ------------------------------------------------------------------------------------------------------------ */
/* INT8 quantizers                                                                                                */

/* x - mean ~ code * scale, one scale per `block` tokens over all channels.  mean: [heads][128] or NULL.
 * codes [heads][n][128], scales [heads][ceil(n / block)]. */
static void quantize_int8_f(const float* x, const float* mean, int heads, int n, int block, int recip, int8_t* codes,
                            float* scales) {
    int blocks = (n + block - 1) / block;
#pragma omp parallel for collapse(2) schedule(static)
    for (int h = 0; h < heads; ++h)
        for (int b = 0; b < blocks; ++b) {
            int t0 = b * block, t1 = t0 + block < n ? t0 + block : n;
            const float* mu = mean ? mean + (size_t)h * D : NULL;
            float amax = 0.0f;
            for (int t = t0; t < t1; ++t)
                for (int c = 0; c < D; ++c) {
                    float v = x[((size_t)h * n + t) * D + c] - (mu ? mu[c] : 0.0f);
                    amax = fmaxf(amax, fabsf(v));
                }
            float s = fmaxf(scalar_div(amax, 127.0f, recip), 1e-12f);
            scales[(size_t)h * blocks + b] = s;
            for (int t = t0; t < t1; ++t)
                for (int c = 0; c < D; ++c) {
                    float v = x[((size_t)h * n + t) * D + c] - (mu ? mu[c] : 0.0f);
                    codes[((size_t)h * n + t) * D + c] = (int8_t)fminf(fmaxf(rintf(v / s), -127.0f), 127.0f);
                }
        }
}

void uo_quantize_int8_rope(const uint16_t* x, const float* mean, const float* rope, int heads_per_table, int heads, int n,
                           int block, int recip, int8_t* codes, float* scales) {
    float* xf = to_float_rotated(x, rope, heads_per_table, heads, n);
    quantize_int8_f(xf, mean, heads, n, block, recip, codes, scales);
    free(xf);
}

void uo_quantize_int8(const uint16_t* x, const float* mean, int heads, int n, int block, int recip, int8_t* codes,
                      float* scales) {
    uo_quantize_int8_rope(x, mean, NULL, 1, heads, n, block, recip, codes, scales);
}

/* V with one scale per channel over all tokens of a head.  skip: [heads][n] bytes, 1 = the key is written as zeros
 * and left out of the scale (the outlier keys, bench/emulate.py:269-273), or NULL.  scale [heads][128]. */
void uo_quantize_v_channel(const uint16_t* v, const uint8_t* skip, int heads, int n, int recip, int8_t* codes,
                           float* scale) {
#pragma omp parallel for schedule(static)
    for (int h = 0; h < heads; ++h) {
        float amax[D];
        for (int c = 0; c < D; ++c) amax[c] = 0.0f;
        for (int t = 0; t < n; ++t) {
            if (skip && skip[(size_t)h * n + t]) continue;
            for (int c = 0; c < D; ++c) amax[c] = fmaxf(amax[c], fabsf(bf16_to_float(v[((size_t)h * n + t) * D + c])));
        }
        for (int c = 0; c < D; ++c) scale[(size_t)h * D + c] = fmaxf(scalar_div(amax[c], 127.0f, recip), 1e-12f);
        for (int t = 0; t < n; ++t)
            for (int c = 0; c < D; ++c) {
                float x = (skip && skip[(size_t)h * n + t]) ? 0.0f : bf16_to_float(v[((size_t)h * n + t) * D + c]);
                codes[((size_t)h * n + t) * D + c] =
                    (int8_t)fminf(fmaxf(rintf(x / scale[(size_t)h * D + c]), -127.0f), 127.0f);
            }
    }
}

/* V with one scale per token over its channels: s_tok [heads][n], plus log2 s and 1 / s as the loop uses them. */
void uo_quantize_v_token(const uint16_t* v, int heads, int n, int recip, int8_t* codes, float* s_tok, float* log_s,
                         float* inv_s) {
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < (size_t)heads * n; ++r) {
        float amax = 0.0f;
        for (int c = 0; c < D; ++c) amax = fmaxf(amax, fabsf(bf16_to_float(v[r * D + c])));
        float s = fmaxf(scalar_div(amax, 127.0f, recip), 1e-12f);
        s_tok[r] = s;
        log_s[r] = log2f(s);
        inv_s[r] = 1.0f / s;
        for (int c = 0; c < D; ++c)
            codes[r * D + c] = (int8_t)fminf(fmaxf(rintf(bf16_to_float(v[r * D + c]) / s), -127.0f), 127.0f);
    }
}

/* The `count` keys of each head with the largest max |v| (unica/__init__.py:384-399, bench/emulate.py:270): ties go
 * to the lower index.  keys [heads][count] (−1 where the head has fewer keys). */
void uo_v_outlier_keys(const uint16_t* v, int heads, int n, int count, int* keys) {
#pragma omp parallel for schedule(static)
    for (int h = 0; h < heads; ++h) {
        float* amax = (float*)malloc(sizeof(float) * (size_t)n);
        for (int t = 0; t < n; ++t) {
            float a = 0.0f;
            for (int c = 0; c < D; ++c) a = fmaxf(a, fabsf(bf16_to_float(v[((size_t)h * n + t) * D + c])));
            amax[t] = a;
        }
        for (int i = 0; i < count; ++i) {
            int best = -1;
            for (int t = 0; t < n; ++t)
                if (amax[t] >= 0.0f && (best < 0 || amax[t] > amax[best])) best = t;
            keys[(size_t)h * count + i] = best;
            if (best >= 0) amax[best] = -1.0f;
        }
        free(amax);
    }
}

/* ------------------------------------------------------------------------------------------------------------ */
/* NVFP4 quantizers                                                                                               */

/* x - mean in NVFP4 along the channels: one float `outer` per head, an e4m3 scale per 16 channels, e2m1 codes.
 * mean: [heads][groups][128] (one mean per `mean_tokens` tokens; mean_tokens <= 0: one per head) or NULL.
 * codes [heads][n][128] (4-bit codes, one per byte), sf [heads][n][8] (e4m3 bytes), outer [heads]. */
static void nvfp4_rows_f(const float* x, const float* mean, int mean_tokens, int heads, int n, int recip, uint8_t* codes,
                         uint8_t* sf, float* outer) {
    if (mean_tokens <= 0) mean_tokens = n;
    int groups = (n + mean_tokens - 1) / mean_tokens;
#pragma omp parallel for schedule(static)
    for (int h = 0; h < heads; ++h) {
        float amax = 0.0f;
        for (int t = 0; t < n; ++t) {
            const float* mu = mean ? mean + ((size_t)h * groups + t / mean_tokens) * D : NULL;
            for (int c = 0; c < D; ++c)
                amax = fmaxf(amax, fabsf(x[((size_t)h * n + t) * D + c] - (mu ? mu[c] : 0.0f)));
        }
        float o = fmaxf(scalar_div(amax, 6.0f * 448.0f, recip), 1e-30f);
        outer[h] = o;
        for (int t = 0; t < n; ++t) {
            const float* mu = mean ? mean + ((size_t)h * groups + t / mean_tokens) * D : NULL;
            for (int b = 0; b < D / 16; ++b) {
                float val[16], a16 = 0.0f;
                for (int i = 0; i < 16; ++i) {
                    int c = 16 * b + i;
                    val[i] = x[((size_t)h * n + t) * D + c] - (mu ? mu[c] : 0.0f);
                    a16 = fmaxf(a16, fabsf(val[i]));
                }
                uint8_t byte = float_to_e4m3(fminf(scalar_div(a16, 6.0f, recip) / o, 448.0f));
                float s = e4m3_to_float(byte) * o;
                sf[((size_t)h * n + t) * 8 + b] = byte;
                for (int i = 0; i < 16; ++i)
                    codes[((size_t)h * n + t) * D + 16 * b + i] = float_to_e2m1(val[i] / fmaxf(s, 1e-30f));
            }
        }
    }
}

void uo_nvfp4_rows_rope(const uint16_t* x, const float* mean, int mean_tokens, const float* rope, int heads_per_table,
                        int heads, int n, int recip, uint8_t* codes, uint8_t* sf, float* outer) {
    float* xf = to_float_rotated(x, rope, heads_per_table, heads, n);
    nvfp4_rows_f(xf, mean, mean_tokens, heads, n, recip, codes, sf, outer);
    free(xf);
}

void uo_nvfp4_rows(const uint16_t* x, const float* mean, int mean_tokens, int heads, int n, int recip, uint8_t* codes,
                   uint8_t* sf, float* outer) {
    uo_nvfp4_rows_rope(x, mean, mean_tokens, NULL, 1, heads, n, recip, codes, sf, outer);
}

/* V in NVFP4 along the keys, per channel: outer [heads][128] = max|v| / (6 * 448); inside each tile of 64 keys the
 * keys are taken in slot order and every 16 slots share an e4m3 scale; keys past n are zeros.
 * codes [heads][tiles * 64][128] indexed by SLOT position (tile * 64 + slot), sf [heads][tiles][4][128]. */
void uo_nvfp4_v(const uint16_t* v, int heads, int n, int recip, uint8_t* codes, uint8_t* sf, float* outer) {
    int tiles = (n + TILE - 1) / TILE;
#pragma omp parallel for schedule(static)
    for (int h = 0; h < heads; ++h) {
        float amax[D];
        for (int c = 0; c < D; ++c) amax[c] = 0.0f;
        for (int t = 0; t < n; ++t)
            for (int c = 0; c < D; ++c) amax[c] = fmaxf(amax[c], fabsf(bf16_to_float(v[((size_t)h * n + t) * D + c])));
        for (int c = 0; c < D; ++c) outer[(size_t)h * D + c] = fmaxf(scalar_div(amax[c], 6.0f * 448.0f, recip), 1e-30f);
        for (int tile = 0; tile < tiles; ++tile)
            for (int b = 0; b < 4; ++b)
                for (int c = 0; c < D; ++c) {
                    float val[16], a16 = 0.0f;
                    for (int i = 0; i < 16; ++i) {
                        int key = tile * TILE + slot_key(16 * b + i);
                        val[i] = key < n ? bf16_to_float(v[((size_t)h * n + key) * D + c]) : 0.0f;
                        a16 = fmaxf(a16, fabsf(val[i]));
                    }
                    float o = outer[(size_t)h * D + c];
                    uint8_t byte = float_to_e4m3(fminf(scalar_div(a16, 6.0f, recip) / o, 448.0f));
                    float s = e4m3_to_float(byte) * o;
                    sf[(((size_t)h * tiles + tile) * 4 + b) * D + c] = byte;
                    for (int i = 0; i < 16; ++i)
                        codes[((size_t)h * tiles * TILE + tile * TILE + 16 * b + i) * D + c] =
                            float_to_e2m1(val[i] / fmaxf(s, 1e-30f));
                }
    }
}

/* ------------------------------------------------------------------------------------------------------------ */
/* FP32 reference                                                                                                 */

void uo_reference_fp32_rope(const uint16_t* q, const uint16_t* k, const uint16_t* v, const float* rope, int heads_per_table,
                            int heads, int nq, int nk, int q_first, int q_count, float* out) {
    const float scale = 1.0f / sqrtf((float)D);
    float* q_rot = to_float_rotated(q, rope, heads_per_table, heads, nq);
    float* k_rot = to_float_rotated(k, rope, heads_per_table, heads, nk);
#pragma omp parallel
    {
        float* s = (float*)malloc(sizeof(float) * (size_t)nk);
#pragma omp for collapse(2) schedule(dynamic, 16)
        for (int h = 0; h < heads; ++h)
            for (int r = 0; r < q_count; ++r) {
                const float* qf = q_rot + ((size_t)h * nq + q_first + r) * D;
                float m = -INFINITY;
                for (int j = 0; j < nk; ++j) {
                    const float* kr = k_rot + ((size_t)h * nk + j) * D;
                    float dot = 0.0f;
                    for (int c = 0; c < D; ++c) dot += qf[c] * kr[c];
                    s[j] = dot * scale;
                    m = fmaxf(m, s[j]);
                }
                double den = 0.0;
                double acc[D];
                for (int c = 0; c < D; ++c) acc[c] = 0.0;
                for (int j = 0; j < nk; ++j) {
                    float p = expf(s[j] - m);
                    den += p;
                    const uint16_t* vr = v + ((size_t)h * nk + j) * D;
                    for (int c = 0; c < D; ++c) acc[c] += (double)p * bf16_to_float(vr[c]);
                }
                float* o = out + ((size_t)h * q_count + r) * D;
                for (int c = 0; c < D; ++c) o[c] = (float)(acc[c] / den);
            }
        free(s);
    }
    free(q_rot);
    free(k_rot);
}

void uo_reference_fp32(const uint16_t* q, const uint16_t* k, const uint16_t* v, int heads, int nq, int nk,
                       int q_first, int q_count, float* out) {
    uo_reference_fp32_rope(q, k, v, NULL, 1, heads, nq, nk, q_first, q_count, out);
}

/* ------------------------------------------------------------------------------------------------------------ */
/* accurate mode                                                                                                  */

enum { UO_V_CHANNEL = 0, UO_V_TOKEN = 1, UO_V_OUTLIERS = 2 };

/* Rows [q_first, q_first + q_count) of every head.  k_mean: [heads][128], or NULL to take uo_channel_stats's.
 * out: float [heads][q_count][128], already rounded to bf16 (bench/emulate.py:369).  Statistics (K mean, every
 * scale) come from the whole head whatever the row range, as in one whole call. */
void uo_attention_accurate_rope(const uint16_t* q, const uint16_t* k, const uint16_t* v, const float* rope, int heads_per_table,
                                int heads, int nq, int nk, int v_mode, int n_outliers, int recip, const float* k_mean,
                                int q_first, int q_count, float* out) {
    const float scale = (float)(1.0 / sqrt((double)D) * LOG2E); /* python double, then float32 tensor multiply */
    int q_blocks = (nq + 127) / 128, k_blocks = (nk + TILE - 1) / TILE;
    float* mean = (float*)malloc(sizeof(float) * (size_t)heads * D);
    if (k_mean)
        memcpy(mean, k_mean, sizeof(float) * (size_t)heads * D);
    else {
        float* lo = (float*)malloc(sizeof(float) * (size_t)heads * D * 2);
        uo_channel_stats_rope(k, rope, heads_per_table, heads, nk, 0, mean, lo, lo + (size_t)heads * D);
        free(lo);
    }
    int8_t* q8 = (int8_t*)malloc((size_t)heads * nq * D);
    int8_t* k8 = (int8_t*)malloc((size_t)heads * nk * D);
    int8_t* v8 = (int8_t*)malloc((size_t)heads * nk * D);
    float* sq = (float*)malloc(sizeof(float) * (size_t)heads * q_blocks);
    float* sk = (float*)malloc(sizeof(float) * (size_t)heads * k_blocks);
    float* sv = (float*)malloc(sizeof(float) * (size_t)heads * D);
    float *s_tok = NULL, *log_s = NULL, *inv_s = NULL;
    uint8_t* skip = NULL;
    int* okeys = NULL;
    uo_quantize_int8_rope(q, NULL, rope, heads_per_table, heads, nq, 128, recip, q8, sq);
    uo_quantize_int8_rope(k, mean, rope, heads_per_table, heads, nk, TILE, recip, k8, sk);
    if (v_mode == UO_V_TOKEN) {
        s_tok = (float*)malloc(sizeof(float) * (size_t)heads * nk * 3);
        log_s = s_tok + (size_t)heads * nk;
        inv_s = log_s + (size_t)heads * nk;
        uo_quantize_v_token(v, heads, nk, recip, v8, s_tok, log_s, inv_s);
        for (size_t i = 0; i < (size_t)heads * D; ++i) sv[i] = 1.0f;
    } else {
        if (v_mode == UO_V_OUTLIERS) {
            okeys = (int*)malloc(sizeof(int) * (size_t)heads * n_outliers);
            skip = (uint8_t*)calloc((size_t)heads * nk, 1);
            uo_v_outlier_keys(v, heads, nk, n_outliers, okeys);
            for (int h = 0; h < heads; ++h)
                for (int i = 0; i < n_outliers; ++i)
                    if (okeys[(size_t)h * n_outliers + i] >= 0) skip[(size_t)h * nk + okeys[(size_t)h * n_outliers + i]] = 1;
        }
        uo_quantize_v_channel(v, skip, heads, nk, recip, v8, sv);
    }

#pragma omp parallel for collapse(2) schedule(dynamic, 16)
    for (int h = 0; h < heads; ++h)
        for (int r = 0; r < q_count; ++r) {
            int row = q_first + r;
            const int8_t* qr = q8 + ((size_t)h * nq + row) * D;
            float s_q = sq[(size_t)h * q_blocks + row / 128];
            float m = -INFINITY, den = 0.0f, o[D];
            for (int c = 0; c < D; ++c) o[c] = 0.0f;
            for (int j0 = 0; j0 < nk; j0 += TILE) {
                int keys = nk - j0 < TILE ? nk - j0 : TILE;
                float s[TILE], s_k = sk[(size_t)h * k_blocks + j0 / TILE], m_tile = -INFINITY;
                for (int j = 0; j < keys; ++j) {
                    const int8_t* kr = k8 + ((size_t)h * nk + j0 + j) * D;
                    int dot = 0;
                    for (int c = 0; c < D; ++c) dot += (int)qr[c] * (int)kr[c];
                    s[j] = (float)dot * (s_q * s_k) * scale; /* bench/emulate.py:307 */
                    if (v_mode == UO_V_TOKEN) s[j] += log_s[(size_t)h * nk + j0 + j];
                    m_tile = fmaxf(m_tile, s[j]);
                }
                float m_new = fmaxf(m, m_tile);
                float alpha = exp2f(m - m_new), beta = exp2f(m_tile - m_new);
                int inner[D];
                for (int c = 0; c < D; ++c) inner[c] = 0;
                float row_sum = 0.0f;
                int isum = 0;
                for (int j = 0; j < keys; ++j) {
                    float p = exp2f(s[j] - m_tile);
                    if (v_mode == UO_V_TOKEN) row_sum += p * inv_s[(size_t)h * nk + j0 + j];
                    int ph = (int)fminf(fmaxf(rintf(p * 255.0f), 0.0f), 255.0f);
                    isum += ph;
                    const int8_t* vr = v8 + ((size_t)h * nk + j0 + j) * D;
                    for (int c = 0; c < D; ++c) inner[c] += ph * (int)vr[c];
                }
                if (v_mode != UO_V_TOKEN) row_sum = (float)isum / 255.0f; /* sum_rounded, bench/emulate.py:346 */
                den = den * alpha + row_sum * beta;
                for (int c = 0; c < D; ++c) o[c] = o[c] * alpha + (float)inner[c] * beta;
                m = m_new;
            }
            if (v_mode == UO_V_OUTLIERS) /* bench/emulate.py:361-365 */
                for (int i = 0; i < n_outliers; ++i) {
                    int key = okeys[(size_t)h * n_outliers + i];
                    if (key < 0) continue;
                    const int8_t* kr = k8 + ((size_t)h * nk + key) * D;
                    int dot = 0;
                    for (int c = 0; c < D; ++c) dot += (int)qr[c] * (int)kr[c];
                    float s_out = (float)dot * (s_q * sk[(size_t)h * k_blocks + key / TILE]) * scale;
                    float p = exp2f(s_out - m) * 255.0f;
                    for (int c = 0; c < D; ++c)
                        o[c] += p * (bf16_to_float(v[((size_t)h * nk + key) * D + c]) / sv[(size_t)h * D + c]);
                }
            float* dst = out + ((size_t)h * q_count + r) * D;
            for (int c = 0; c < D; ++c) dst[c] = round_bf16(o[c] * (sv[(size_t)h * D + c] / 255.0f) / den);
        }
    free(mean); free(q8); free(k8); free(v8); free(sq); free(sk); free(sv); free(s_tok); free(skip); free(okeys);
}

void uo_attention_accurate(const uint16_t* q, const uint16_t* k, const uint16_t* v, int heads, int nq, int nk,
                           int v_mode, int n_outliers, int recip, const float* k_mean, int q_first, int q_count,
                           float* out) {
    uo_attention_accurate_rope(q, k, v, NULL, 1, heads, nq, nk, v_mode, n_outliers, recip, k_mean, q_first, q_count, out);
}

/* ------------------------------------------------------------------------------------------------------------ */
/* fast mode                                                                                                      */

/* NVFP4 Q.K^T and P.V, Q mean-smoothed per `smooth_q` queries (0: no smoothing), keys in slot order, P in NVFP4
 * with outer scale 1 against p_mul = 1024.  k_mean [heads][128] / q_mean [heads][ceil(nq / smooth_q)][128] or NULL
 * (then uo_channel_stats's). */
/* p_codes (or NULL): the quantized probabilities of every row and key tile as the loop forms them, uint8
 * [heads][q_count][tiles][68]: 64 e2m1 codes in slot order, then the four e4m3 scale bytes. */
static void attention_fast_impl(const uint16_t* q, const uint16_t* k, const uint16_t* v, const float* rope, int heads_per_table,
                                int heads, int nq, int nk, int smooth_q, int recip, const float* k_mean, const float* q_mean,
                                int q_first, int q_count, float* out, uint8_t* p_codes) {
    const float scale = (float)(1.0 / sqrt((double)D) * LOG2E);
    const float p_mul = 1024.0f;
    float* k_rot = to_float_rotated(k, rope, heads_per_table, heads, nk); /* the smoothing term takes k in float */
    int tiles = (nk + TILE - 1) / TILE, npad = tiles * TILE;
    int q_groups = smooth_q ? (nq + smooth_q - 1) / smooth_q : 1;
    float* kmean = (float*)malloc(sizeof(float) * (size_t)heads * D);
    float* scratch = (float*)malloc(sizeof(float) * (size_t)heads * q_groups * D * 2);
    if (k_mean)
        memcpy(kmean, k_mean, sizeof(float) * (size_t)heads * D);
    else {
        float* lo = (float*)malloc(sizeof(float) * (size_t)heads * D * 2);
        uo_channel_stats_rope(k, rope, heads_per_table, heads, nk, 0, kmean, lo, lo + (size_t)heads * D);
        free(lo);
    }
    float* qmean = NULL;
    if (smooth_q) {
        qmean = (float*)malloc(sizeof(float) * (size_t)heads * q_groups * D);
        if (q_mean)
            memcpy(qmean, q_mean, sizeof(float) * (size_t)heads * q_groups * D);
        else
            uo_channel_stats_rope(q, rope, heads_per_table, heads, nq, smooth_q, qmean, scratch, scratch + (size_t)heads * q_groups * D);
    }
    uint8_t* qc = (uint8_t*)malloc((size_t)heads * nq * D);
    uint8_t* kc = (uint8_t*)malloc((size_t)heads * nk * D);
    uint8_t* vc = (uint8_t*)malloc((size_t)heads * npad * D);
    uint8_t* qsf = (uint8_t*)malloc((size_t)heads * nq * 8);
    uint8_t* ksf = (uint8_t*)malloc((size_t)heads * nk * 8);
    uint8_t* vsf = (uint8_t*)malloc((size_t)heads * tiles * 4 * D);
    float* qo = (float*)malloc(sizeof(float) * heads);
    float* ko = (float*)malloc(sizeof(float) * heads);
    float* vo = (float*)malloc(sizeof(float) * (size_t)heads * D);
    uo_nvfp4_rows_rope(q, qmean, smooth_q, rope, heads_per_table, heads, nq, recip, qc, qsf, qo);
    uo_nvfp4_rows_rope(k, kmean, 0, rope, heads_per_table, heads, nk, recip, kc, ksf, ko);
    uo_nvfp4_v(v, heads, nk, recip, vc, vsf, vo);
    /* dequantized K (x^ * s) and V, and the exact centred K for the smoothing term */
    float* kd = (float*)malloc(sizeof(float) * (size_t)heads * nk * D);
    float* vd = (float*)malloc(sizeof(float) * (size_t)heads * npad * D);
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < (size_t)heads * nk; ++r) {
        int h = (int)(r / nk);
        for (int c = 0; c < D; ++c)
            kd[r * D + c] = e2m1_to_float(kc[r * D + c]) * (e4m3_to_float(ksf[r * 8 + c / 16]) * ko[h]);
    }
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < (size_t)heads * npad; ++r) {
        int h = (int)(r / npad), pos = (int)(r % npad);
        for (int c = 0; c < D; ++c)
            vd[r * D + c] = e2m1_to_float(vc[r * D + c]) *
                            (e4m3_to_float(vsf[(((size_t)h * tiles + pos / TILE) * 4 + pos % TILE / 16) * D + c]) *
                             vo[(size_t)h * D + c]);
    }

#pragma omp parallel for collapse(2) schedule(dynamic, 16)
    for (int h = 0; h < heads; ++h)
        for (int r = 0; r < q_count; ++r) {
            int row = q_first + r;
            float qd[D], qbar[D];
            for (int c = 0; c < D; ++c) {
                size_t i = ((size_t)h * nq + row) * D + c;
                qd[c] = e2m1_to_float(qc[i]) * (e4m3_to_float(qsf[((size_t)h * nq + row) * 8 + c / 16]) * qo[h]);
                qbar[c] = smooth_q ? qmean[((size_t)h * q_groups + row / smooth_q) * D + c] : 0.0f;
            }
            float m = -INFINITY, den = 0.0f, o[D];
            for (int c = 0; c < D; ++c) o[c] = 0.0f;
            for (int tile = 0; tile < tiles; ++tile) {
                float s[TILE], m_new = m;
                for (int slot = 0; slot < TILE; ++slot) {
                    int key = tile * TILE + slot_key(slot);
                    if (key >= nk) {
                        s[slot] = -INFINITY;
                        continue;
                    }
                    const float* kr = kd + ((size_t)h * nk + key) * D;
                    float dot = 0.0f, bias = 0.0f;
                    for (int c = 0; c < D; ++c) dot += qd[c] * kr[c];
                    s[slot] = dot * scale;
                    if (smooth_q) { /* q_mean . (k - k_mean), unquantized (bench/emulate.py:308-309) */
                        for (int c = 0; c < D; ++c)
                            bias += qbar[c] * (k_rot[((size_t)h * nk + key) * D + c] - kmean[(size_t)h * D + c]);
                        s[slot] += bias * scale;
                    }
                    m_new = fmaxf(m_new, s[slot]);
                }
                float alpha = exp2f(m - m_new);
                float ph[TILE], row_sum = 0.0f;
                for (int b = 0; b < 4; ++b) {
                    float p[16], a16 = 0.0f;
                    for (int i = 0; i < 16; ++i) {
                        p[i] = exp2f(s[16 * b + i] - m_new) * p_mul;
                        a16 = fmaxf(a16, p[i]);
                    }
                    uint8_t sp_byte = float_to_e4m3(fminf(scalar_div(a16, 6.0f, recip), 448.0f));
                    float sp = e4m3_to_float(sp_byte);
                    uint8_t* rec = p_codes ? p_codes + ((((size_t)h * q_count + r) * tiles + tile) * 68) : NULL;
                    if (rec) rec[64 + b] = sp_byte;
                    for (int i = 0; i < 16; ++i) {
                        uint8_t code = float_to_e2m1(p[i] / fmaxf(sp, 1e-30f));
                        if (rec) rec[16 * b + i] = code;
                        ph[16 * b + i] = e2m1_to_float(code) * sp;
                        row_sum += ph[16 * b + i];
                    }
                }
                den = den * alpha + row_sum / p_mul;
                for (int c = 0; c < D; ++c) o[c] *= alpha;
                for (int slot = 0; slot < TILE; ++slot) {
                    if (ph[slot] == 0.0f) continue;
                    const float* vr = vd + ((size_t)h * npad + tile * TILE + slot) * D;
                    for (int c = 0; c < D; ++c) o[c] += ph[slot] * vr[c];
                }
                m = m_new;
            }
            float* dst = out + ((size_t)h * q_count + r) * D;
            for (int c = 0; c < D; ++c) dst[c] = round_bf16(o[c] * (1.0f / p_mul) / den);
        }
    free(kmean); free(scratch); free(qmean); free(qc); free(kc); free(vc); free(qsf); free(ksf); free(vsf);
    free(qo); free(ko); free(vo); free(kd); free(vd); free(k_rot);
}

void uo_attention_fast_rope(const uint16_t* q, const uint16_t* k, const uint16_t* v, const float* rope, int heads_per_table,
                            int heads, int nq, int nk, int smooth_q, int recip, const float* k_mean, const float* q_mean,
                            int q_first, int q_count, float* out) {
    attention_fast_impl(q, k, v, rope, heads_per_table, heads, nq, nk, smooth_q, recip, k_mean, q_mean, q_first, q_count, out, NULL);
}

/* The same, also returning the P^ codes (see attention_fast_impl). */
void uo_attention_fast_codes(const uint16_t* q, const uint16_t* k, const uint16_t* v, int heads, int nq, int nk, int smooth_q,
                             int recip, const float* k_mean, const float* q_mean, float* out, uint8_t* p_codes) {
    attention_fast_impl(q, k, v, NULL, 1, heads, nq, nk, smooth_q, recip, k_mean, q_mean, 0, nq, out, p_codes);
}

void uo_attention_fast(const uint16_t* q, const uint16_t* k, const uint16_t* v, int heads, int nq, int nk, int smooth_q,
                       int recip, const float* k_mean, const float* q_mean, int q_first, int q_count, float* out) {
    uo_attention_fast_rope(q, k, v, NULL, 1, heads, nq, nk, smooth_q, recip, k_mean, q_mean, q_first, q_count, out);
}
