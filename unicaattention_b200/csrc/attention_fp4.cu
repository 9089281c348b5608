// The fast mode's flash-attention loop on tcgen05 (replaces the reference's attention_fp4, csrc/flash.cu:1380-1524).
//
// Both contractions run as tcgen05.mma kind::mxf4nvf4.block_scale.scale_vec::4X (e2m1 codes, one ue4m3 scale per 16
// elements of the contraction, FP32 accumulators in tensor memory):
//   S[g]  = Q4[g] . K4(t)^T     128 x 64,  2 instructions of K = 64 channels
//   O[g] += P4[g](t) . V4(t)    128 x 144, 1 instruction of K = 64 keys; columns 0..127 are the output channels, column
//                               128 multiplies P by a row of ones: the running softmax denominator, rescaled with O
// One block = F4_TILES (2) tiles of 128 query rows of one head sharing every K and V tile, one thread per query row
// (on the row's tensor-memory lane: all 64 key slots of a tile in its registers, so a row's maximum needs no exchange
// between threads); the last warpgroup holds the producer warp (bulk TMA copies) and one MMA warp per query tile,
// one elected thread of which issues that tile's instructions and copies K's, V's and P's scale bytes into tensor
// memory.
//
// Numerics (bench/emulate.py:298-369 with the fast contract): scores x = S * (q_outer k_outer log2(e)/sqrt(d)) + bias,
// bias the exact q_mean . (k - k_mean) term of Q smoothing; running maximum m; P = 1024 * 2^(x - m) in NVFP4 along the
// keys of the tile in slot order with a fixed outer scale of 1: per 16 slots sp = e4m3(max P / 6), codes e2m1(P / sp),
// P / sp taken as 2^(x - m + 10 - log2 sp) in one ex2.approx; O = O * 2^(m_old - m) + P^ . V^; out = O / (sum of P^) *
// v_outer.  A code of P can therefore land on the other side of a rounding boundary than the emulation's (P / sp is off
// by some 1e-6 relative): results agree to rounding, not bit for bit.
//
// Scale bytes live in tensor memory, row r of an operand in lane r % 32 of column r / 32 of every 32-lane quarter.  Q's
// are stored once by the computing warps (tcgen05.st); K's, V's and P's are copied from shared memory by the issuing
// thread right before the MMA that reads them (tcgen05.cp 32x128b.warpx4: 16 bytes per lane, all four quarters), K's
// and V's as the quantizers laid them out, P's as the computing threads wrote them a moment earlier.
//
// Tensor memory per query tile (256 columns): S 0..63 | O 64..207 | SF of Q 208..215, K 216..219, P 220..223, V 224..231.
// All waits are bounded (common.cuh); none sleeps between probes: every hand-over here is on the loop's critical path.
#include <cuda_fp8.h>

#include "capi.h"
#include "fp4_common.cuh"

namespace unica {

constexpr int F4_TILES = 2;  // query tiles of 128 rows per block (tensor memory holds two: 2 x 232 of 512 columns)
constexpr int F4_COMPUTE_WARPS = 4 * F4_TILES;  // query tiles x 4 warps, a thread per row
constexpr int F4_THREADS = (F4_COMPUTE_WARPS + 4) * 32;
constexpr int F4_PRODUCER_WARP = F4_COMPUTE_WARPS, F4_MMA_WARP = F4_COMPUTE_WARPS + 1;
constexpr int F4_HALF_SLOTS = KEY_TILE / 2;  // one 16-byte piece of a row of P^: two scale blocks of 16 slots
constexpr int F4_STAGES = 4;
constexpr int Q4_BYTES = QUERY_TILE * HEAD_DIM / 2;  // 8192
constexpr int SFQ_BYTES = 2 * QUERY_TILE * 4;        // 1024
constexpr int K4_BYTES = KEY_TILE * HEAD_DIM / 2;    // 4096
constexpr int SFK_BYTES = 2 * KEY_TILE * 4;          // 512
constexpr int V4_TILE_ROWS = 144, V4_BYTES = 2 * V4_TILE_ROWS * 16;  // 4608
constexpr int SFV_BYTES = 256 * 4;                   // 1024: two blocks of 32 lanes x 4 words
constexpr int BIAS_BYTES = KEY_TILE * 4;             // 256
constexpr int P4_BYTES = QUERY_TILE * KEY_TILE / 2;  // 4096
constexpr int F4_TMEM_COLUMNS = 256 * F4_TILES;
constexpr int F4_S = 0, F4_O = 64, F4_SFQ = 208, F4_SFK = 216, F4_SFP = 220, F4_SFV = 224;
constexpr float P_LOG2_GAIN = 10.0f;  // P is taken times 2^10: its block scales (up to 1024 / 6) stay below e4m3's 448

// -DUNICA_TRACE: the first thread of each warpgroup of block (0, 0) adds up the cycles of each phase of its tile loop
// in registers and leaves the totals in g_trace_fp4 (see attention_int8.cu for the accurate kernel's).
#ifdef UNICA_TRACE
__device__ long long g_trace_fp4[4][8];
#define F4_TRACE_DECL long long trace_t0 = clock64(), trace_sum[8] = {}; const bool tracing = blockIdx.x == 0 && blockIdx.y == 0 && row == 0
#define F4_TRACE(phase)                              \
    do {                                             \
        if (tracing) {                               \
            const long long now = clock64();         \
            trace_sum[phase] += now - trace_t0;      \
            trace_t0 = now;                          \
        }                                            \
    } while (0)
#define F4_TRACE_END(slot)                                                    \
    do {                                                                      \
        if (tracing)                                                          \
            for (int i = 0; i < 8; ++i) g_trace_fp4[slot][i] = trace_sum[i];  \
    } while (0)
#else
#define F4_TRACE_DECL
#define F4_TRACE(phase)
#define F4_TRACE_END(slot)
#endif
enum { F4_TR_WAIT_S = 0, F4_TR_LOAD_S = 1, F4_TR_MAX = 2, F4_TR_QUANTIZE = 3, F4_TR_WAIT_O = 4, F4_TR_RESCALE = 5, F4_TR_EXCHANGE = 6, F4_TR_OTHER = 7 };

struct __align__(128) Fp4Smem {
    uint8_t q[F4_TILES][Q4_BYTES];
    uint32_t sfq[F4_TILES][2][QUERY_TILE];
    uint8_t k[F4_STAGES][K4_BYTES];
    uint32_t sfk[F4_STAGES][32][4];  // as tcgen05.cp takes them: lane, word 2 step + row / 32
    uint8_t v[F4_STAGES][V4_BYTES];
    uint32_t sfv[F4_STAGES][2][32][4];  // block 0: channel c = word c / 32 of lane c % 32; block 1: the ones rows
    float bias[F4_STAGES][KEY_TILE];
    float mask[2][KEY_TILE];  // what is added to the scores where there is no smoothing term: zeros / -inf in the last tile's empty slots
    uint8_t p[F4_TILES][P4_BYTES];
    uint32_t sfp[F4_TILES][32][4];  // P's scale words of a query tile: row r = word r / 32 of lane r % 32
    uint8_t staged[F4_COMPUTE_WARPS][32 * HEAD_DIM * 2];  // output rows on their way out (see store_staged_rows)
    float log2_e4m3[128];  // log2 of every non-negative e4m3 byte's value; +inf for the byte 0, so that 2^(x - that) = 0
    uint64_t q_full, k_full[F4_STAGES], k_empty[F4_STAGES], v_full[F4_STAGES], v_empty[F4_STAGES];
    uint64_t s_full[F4_TILES], s_free[F4_TILES], p_ready[F4_TILES], o_full[F4_TILES], drain[F4_TILES];
    uint32_t tmem_base;
    int abort_flag;
};

constexpr uint32_t IDESC_F4_QK = idesc_nvf4(QUERY_TILE, KEY_TILE);
constexpr uint32_t IDESC_F4_PV = idesc_nvf4(QUERY_TILE, V4_TILE_ROWS);

__device__ __forceinline__ float lg2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// eight floats -> eight e2m1 codes in one word, element i in nibble i
__device__ __forceinline__ uint32_t e2m1x8(const float2 (&v)[4]) {
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
        : "f"(v[0].x), "f"(v[0].y), "f"(v[1].x), "f"(v[1].y), "f"(v[2].x), "f"(v[2].y), "f"(v[3].x), "f"(v[3].y));
    return word;
}

__global__ void __launch_bounds__(F4_THREADS, 1)
    attention_fp4_kernel(const uint8_t* __restrict__ q4, const uint32_t* __restrict__ sfq, const uint8_t* __restrict__ k4,
                         const uint32_t* __restrict__ sfk, const uint8_t* __restrict__ v4, const uint32_t* __restrict__ sfv,
                         const float* __restrict__ qk_outer, const float* __restrict__ v_outer, const float* __restrict__ bias,
                         int q_blocks, int smooth_q, __nv_bfloat16* __restrict__ out, TokenLayout out_layout, const __grid_constant__ PeerOutputs peers, int n_queries,
                         int n_keys, float scale_log2, uint32_t* __restrict__ p_words, int* status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Fp4Smem& sm = *reinterpret_cast<Fp4Smem*>(smem_raw);
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int head = blockIdx.y;
    const int q_tiles = F4_TILES * gridDim.x;  // allocated Q tiles per head (even)
    const int k_tiles = (n_keys + KEY_TILE - 1) / KEY_TILE;
    volatile int* abort_flag = &sm.abort_flag;

    if (threadIdx.x == 0) {
        sm.abort_flag = 0;
        mbar_init(&sm.q_full, 1);
        for (int s = 0; s < F4_STAGES; ++s) {
            mbar_init(&sm.k_full[s], 1);
            mbar_init(&sm.k_empty[s], F4_TILES);  // every query tile's MMA thread commits to it
            mbar_init(&sm.v_full[s], 1);
            mbar_init(&sm.v_empty[s], F4_TILES);
        }
        for (int g = 0; g < F4_TILES; ++g) {
            mbar_init(&sm.s_full[g], 1);
            mbar_init(&sm.s_free[g], QUERY_TILE);  // every row's thread
            mbar_init(&sm.p_ready[g], QUERY_TILE);
            mbar_init(&sm.o_full[g], 1);
        }
        for (int g = 0; g < F4_TILES; ++g) mbar_init(&sm.drain[g], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 128) {
        const float value = __half2float(__half(__nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(threadIdx.x), __NV_E4M3)));
        sm.log2_e4m3[threadIdx.x] = value > 0.0f ? log2f(value) : INFINITY;  // byte 127 is NaN: never produced (satfinite)
    }
    if (threadIdx.x >= 128 && threadIdx.x < 128 + KEY_TILE) {
        const int slot = threadIdx.x - 128, j = slot % F4_HALF_SLOTS;
        const int key = (k_tiles - 1) * KEY_TILE + F4_HALF_SLOTS * (slot / F4_HALF_SLOTS) + 8 * (j % 8 / 2) + 2 * (j / 8) + j % 2;  // slot -> key
        sm.mask[0][slot] = 0.0f;
        sm.mask[1][slot] = key < n_keys ? 0.0f : -INFINITY;
    }
    if (warp == F4_MMA_WARP) tmem_alloc(&sm.tmem_base, F4_TMEM_COLUMNS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    if (warp == F4_PRODUCER_WARP) {
        // ------------------------------------------------------------------------------------------------ producer
        if (elect_one()) {  // one elected lane of a converged warp: see elect_one() in common.cuh
            const size_t q_first = size_t(head) * q_tiles + F4_TILES * blockIdx.x;
            mbar_expect_tx(&sm.q_full, F4_TILES * (Q4_BYTES + SFQ_BYTES));
            bulk_load(sm.q[0], q4 + q_first * Q4_BYTES, F4_TILES * Q4_BYTES, &sm.q_full);
            bulk_load(sm.sfq[0], sfq + q_first * (SFQ_BYTES / 4), F4_TILES * SFQ_BYTES, &sm.q_full);
            const float* bias_row = bias ? bias + (size_t(head) * q_blocks + (F4_TILES * blockIdx.x * QUERY_TILE) / smooth_q) * (size_t(k_tiles) * KEY_TILE) : nullptr;
            int issued = 0, issued_v = 0;  // K tiles / V tiles whose copies have been started
            for (int t = 0; t < k_tiles; ++t) {
                const int s = t % F4_STAGES, use = t / F4_STAGES;
                const size_t tile = size_t(head) * k_tiles + t;
                if (use > 0 && !mbar_wait<0>(&sm.k_empty[s], (use - 1) & 1, abort_flag, status, STATUS_WAIT_STAGE)) break;
                mbar_expect_tx(&sm.k_full[s], K4_BYTES + SFK_BYTES);
                bulk_load(sm.k[s], k4 + tile * K4_BYTES, K4_BYTES, &sm.k_full[s]);
                bulk_load(sm.sfk[s], sfk + tile * (SFK_BYTES / 4), SFK_BYTES, &sm.k_full[s]);
                if (use > 0 && !mbar_wait<0>(&sm.v_empty[s], (use - 1) & 1, abort_flag, status, STATUS_WAIT_STAGE)) {
                    issued = t + 1;
                    break;
                }
                mbar_expect_tx(&sm.v_full[s], V4_BYTES + SFV_BYTES + (bias_row ? BIAS_BYTES : 0));
                bulk_load(sm.v[s], v4 + tile * V4_BYTES, V4_BYTES, &sm.v_full[s]);
                bulk_load(sm.sfv[s], sfv + tile * (SFV_BYTES / 4), SFV_BYTES, &sm.v_full[s]);
                if (bias_row) bulk_load(sm.bias[s], bias_row + size_t(t) * KEY_TILE, BIAS_BYTES, &sm.v_full[s]);
                issued = issued_v = t + 1;
            }
            if (*abort_flag) {  // no copy may still be writing this block's shared memory when the block ends
                int never = 0;
                for (int t = max(0, issued - F4_STAGES); t < issued; ++t)
                    mbar_wait<0>(&sm.k_full[t % F4_STAGES], (t / F4_STAGES) & 1, &never, nullptr, 0);
                for (int t = max(0, issued_v - F4_STAGES); t < issued_v; ++t)
                    mbar_wait<0>(&sm.v_full[t % F4_STAGES], (t / F4_STAGES) & 1, &never, nullptr, 0);
                mbar_wait<0>(&sm.q_full, 0, &never, nullptr, 0);
            }
        }
    } else if (warp >= F4_MMA_WARP && warp < F4_MMA_WARP + F4_TILES) {
        // ------------------------------------------------------------------------------------------------ MMA issue
        // One elected thread per query tile, blocking on each operand in the order they become ready: the scores of key
        // tile t + 1 once the softmax threads have taken those of tile t; then P.V of tile t once P4(t) and the scale
        // bytes of P and V are in place.
        if (elect_one()) {  // one elected lane of a converged warp: see elect_one() in common.cuh
            const int g = warp - F4_MMA_WARP;
            const uint32_t q_addr = smem_u32(sm.q[g]), base = tmem + g * 256;
            auto scores = [&](int n) -> bool {
                const int stage = n % F4_STAGES;
                if (!mbar_wait<0>(&sm.k_full[stage], (n / F4_STAGES) & 1, abort_flag, status, STATUS_WAIT_TILE)) return false;
                if (!mbar_wait<0>(&sm.s_free[g], n & 1, abort_flag, status, STATUS_WAIT_FREE)) return false;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(sm.k[stage]);
                tmem_cp_32x128b(base + F4_SFK, smem_u32(sm.sfk[stage]));  // K's scale bytes; ordered before the MMAs below
#pragma unroll
                for (int ks = 0; ks < 2; ++ks)
                    mma_nvf4_ss(base + F4_S, smem_desc(q_addr + ks * 2 * QUERY_TILE * 16, QUERY_TILE * 16, 128),
                                smem_desc(k_addr + ks * 2 * KEY_TILE * 16, KEY_TILE * 16, 128), IDESC_F4_QK, base + F4_SFQ + 4 * ks,
                                base + F4_SFK + 2 * ks, ks > 0);
                mma_commit(&sm.s_full[g]);
                mma_commit(&sm.k_empty[stage]);
                return true;
            };
            bool ok = mbar_wait<0>(&sm.q_full, 0, abort_flag, status, STATUS_WAIT_TILE) && scores(0);
            for (int t = 0; ok && t < k_tiles; ++t) {
                if (t + 1 < k_tiles) ok = scores(t + 1);
                const int stage = t % F4_STAGES;
                ok = ok && mbar_wait<0>(&sm.v_full[stage], (t / F4_STAGES) & 1, abort_flag, status, STATUS_WAIT_TILE) &&
                     mbar_wait<0>(&sm.p_ready[g], t & 1, abort_flag, status, STATUS_WAIT_P);
                if (!ok) break;
                tc_fence_after();
                tmem_cp_32x128b(base + F4_SFP, smem_u32(sm.sfp[g]));  // the scale bytes of P^ and of V
                tmem_cp_32x128b(base + F4_SFV, smem_u32(sm.sfv[stage][0]));
                tmem_cp_32x128b(base + F4_SFV + 4, smem_u32(sm.sfv[stage][1]));
                mma_nvf4_ss(base + F4_O, smem_desc(smem_u32(sm.p[g]), QUERY_TILE * 16, 128),
                            smem_desc(smem_u32(sm.v[stage]), V4_TILE_ROWS * 16, 128), IDESC_F4_PV, base + F4_SFP, base + F4_SFV, t > 0);
                mma_commit(&sm.o_full[g]);
                mma_commit(&sm.v_empty[stage]);
            }
            if (!ok) {
                int never = 0;
                mma_commit(&sm.drain[g]);
                mbar_wait<0>(&sm.drain[g], 0, &never, nullptr, 0);
            }
        }
    } else if (warp < F4_COMPUTE_WARPS) {
        // ------------------------------------------------------------------------------------------------ softmax
        // One thread per query row: warp = 4 g + quarter on tensor-memory lanes 32 quarter .. + 31.
        const int g = warp / 4, row = (warp % 4) * 32 + lane;
        const int q_row = (F4_TILES * blockIdx.x + g) * QUERY_TILE + row;
        const uint32_t my = tmem + (uint32_t((warp % 4) * 32) << 16) + g * 256;
        const float c = qk_outer[head] * scale_log2;
        const float2 c2 = make_float2(c, c);
        const bool smoothed = bias != nullptr;
        float m = -INFINITY;
        bool ok = mbar_wait_warp<0>(&sm.q_full, 0, abort_flag, status, STATUS_WAIT_TILE) &&
                  mbar_wait_warp<0>(&sm.k_full[0], 0, abort_flag, status, STATUS_WAIT_TILE);
        if (ok) {  // scale bytes of Q, for the whole loop
#pragma unroll
            for (int s = 0; s < 2; ++s)
                tmem_st4(my + F4_SFQ + 4 * s, sm.sfq[g][s][lane], sm.sfq[g][s][32 + lane], sm.sfq[g][s][64 + lane], sm.sfq[g][s][96 + lane]);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&sm.s_free[g]);
        }

        F4_TRACE_DECL;
        for (int t = 0; ok && t < k_tiles; ++t) {
            const int stage = t % F4_STAGES;
            F4_TRACE(F4_TR_OTHER);
            // the scores, and V's tile, with which the smoothing term arrives: both probes in flight together
            ok = __all_sync(0xffffffffu, mbar_wait2<0>(&sm.s_full[g], t & 1, &sm.v_full[stage], (t / F4_STAGES) & 1, abort_flag, status,
                                                       STATUS_WAIT_SCORES));
            if (!ok) break;
            tc_fence_after();
            F4_TRACE(F4_TR_WAIT_S);
            float2 x[KEY_TILE / 2];
            tmem_ld64_sync(my + F4_S, x);
            tc_fence_before();
            mbar_arrive(&sm.s_free[g]);  // the scores are in registers: the buffer goes back
            // Has P.V of the previous tile completed?  Asked now, looked at after the exponentials: it usually has, and
            // the probe's latency (a few hundred cycles for a first look) is hidden behind them.
            const bool pv_done = t == 0 || mbar_try(&sm.o_full[g], (t - 1) & 1);
            F4_TRACE(F4_TR_LOAD_S);

            // Scores in the log2 domain plus the smoothing term (or zeros); -inf in the slots past the last key, which
            // keeps them out of the maxima and makes their P zero.
            {
                const float* added = smoothed ? sm.bias[stage] : sm.mask[(t + 1) * KEY_TILE > n_keys];
                const float2* b2 = reinterpret_cast<const float2*>(added);
#pragma unroll
                for (int j = 0; j < KEY_TILE / 2; ++j) x[j] = fma2(x[j], c2, b2[j]);
            }
            float block_max[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                float top = fmaxf(x[8 * b].x, x[8 * b].y);
#pragma unroll
                for (int i = 1; i < 8; ++i) top = max3(top, x[8 * b + i].x, x[8 * b + i].y);
                block_max[b] = top;
            }
            const float m_new = fmaxf(max3(m, block_max[0], block_max[1]), fmaxf(block_max[2], block_max[3]));
            const float alpha = ex2(m - m_new);
            m = m_new;
            F4_TRACE(F4_TR_MAX);

            // P in NVFP4: per 16 slots a scale byte sp = e4m3(max P / 6) with P = 1024 * 2^(x - m), then the codes of
            // P / sp = 2^(x - m + 10 - log2 sp) straight out of the exponent unit; log2 of every e4m3 value comes from a
            // table (a logarithm here would double the block's dependent chain).
            uint32_t codes[8], sf_word = 0;
            const float gain = P_LOG2_GAIN - m_new;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const float top = ex2(block_max[b] + gain) * (1.0f / 6.0f);
                const uint32_t byte = __nv_cvt_float_to_fp8(top, __NV_SATFINITE, __NV_E4M3);
                const float shift = gain - sm.log2_e4m3[byte];  // byte 0 (every P below e4m3's range): -inf, all codes zero
                const float2 shift2 = make_float2(shift, shift);
                sf_word |= byte << (8 * b);
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    float2 r[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 e = add2(x[8 * b + 4 * w + i], shift2);
                        r[i] = make_float2(ex2(e.x), ex2(e.y));
                    }
                    codes[2 * b + w] = e2m1x8(r);
                }
            }
            if (p_words && q_row < n_queries) {  // diagnostics: this row's P^ of the tile, 8 words of codes and the 4 scale bytes
                uint32_t* dst = p_words + ((size_t(head) * n_queries + q_row) * k_tiles + t) * 9;
#pragma unroll
                for (int i = 0; i < 8; ++i) dst[i] = codes[i];
                dst[8] = sf_word;
            }
            F4_TRACE(F4_TR_QUANTIZE);

            if (t > 0) {  // P.V of the previous tile must have read P, its scales and V's, and written O
                if (!__all_sync(0xffffffffu, pv_done)) {
                    ok = mbar_wait_warp<0>(&sm.o_full[g], (t - 1) & 1, abort_flag, status, STATUS_WAIT_PV);
                    if (!ok) break;
                }
                tc_fence_after();
                F4_TRACE(F4_TR_WAIT_O);
                if (!__all_sync(0xffffffffu, alpha == 1.0f)) {  // the maximum moved: O and the denominator shrink
                    const float2 alpha2 = make_float2(alpha, alpha);
                    // 128 channels, then the denominator's column (the 15 after it stay zero)
#pragma unroll
                    for (int first = 0; first < HEAD_DIM; first += 64) {
                        float2 o[4][8];
#pragma unroll
                        for (int i = 0; i < 4; ++i) tmem_ld16_async(my + F4_O + first + 16 * i, o[i]);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            reg_fence8(o[i]);
#pragma unroll
                            for (int j = 0; j < 8; ++j) o[i][j] = mul2(o[i][j], alpha2);
                            tmem_st16(my + F4_O + first + 16 * i, o[i]);
                        }
                    }
                    float2 sum[4];
                    tmem_ld8_async(my + F4_O + HEAD_DIM, sum);
                    tmem_wait_ld();
                    reg_fence4(sum);
#pragma unroll
                    for (int j = 0; j < 4; ++j) sum[j] = mul2(sum[j], alpha2);
                    tmem_st8(my + F4_O + HEAD_DIM, sum);
                }
            }
            // P.V of the previous tile has read P^: this tile's codes and scale bytes may take its place
            *reinterpret_cast<uint4*>(sm.p[g] + row * 16) = make_uint4(codes[0], codes[1], codes[2], codes[3]);
            *reinterpret_cast<uint4*>(sm.p[g] + QUERY_TILE * 16 + row * 16) = make_uint4(codes[4], codes[5], codes[6], codes[7]);
            sm.sfp[g][row % 32][row / 32] = sf_word;  // byte 2 piece + block
            F4_TRACE(F4_TR_RESCALE);
            tmem_wait_st();  // the rescaled O, if any
            tc_fence_before();
            fence_proxy_async();  // P^ and its scale bytes are read by the tensor pipe (tcgen05.cp, tcgen05.mma)
            mbar_arrive(&sm.p_ready[g]);
            F4_TRACE(F4_TR_EXCHANGE);
        }
        F4_TRACE_END(g);

        if (ok) ok = mbar_wait_warp<0>(&sm.o_full[g], (k_tiles - 1) & 1, abort_flag, status, STATUS_WAIT_PV);
        if (ok) {
            tc_fence_after();
            const float* scale = v_outer + head * HEAD_DIM;
            float2 last[4];
            tmem_ld8_async(my + F4_O + HEAD_DIM, last);  // column 128: the sum of P^
            tmem_wait_ld();
            reg_fence4(last);
            const float inv = 1.0f / last[0].x;
            uint8_t* staged = sm.staged[warp];
#pragma unroll
            for (int part = 0; part < HEAD_DIM / 16; ++part) {
                float2 o[8];
                tmem_ld16_sync(my + F4_O + part * 16, o);
                uint32_t w[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int c0 = part * 16 + 2 * i;
                    w[i] = output_pair(o[i].x * scale[c0] * inv, o[i].y * scale[c0 + 1] * inv, out_layout.half);
                }
                stage_piece(staged, lane, 2 * part, make_uint4(w[0], w[1], w[2], w[3]));
                stage_piece(staged, lane, 2 * part + 1, make_uint4(w[4], w[5], w[6], w[7]));
            }
            __syncwarp();
            store_staged_rows(staged, lane, q_row - lane, n_queries, head, out, out_layout, peers);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == F4_MMA_WARP) {
        tc_fence_after();
        tmem_dealloc(tmem, F4_TMEM_COLUMNS);
    }
}

}  // namespace unica

using namespace unica;

#ifdef UNICA_TRACE
// Trace builds only: copies the per-phase cycle totals of block (0, 0) to `host_out` (4 x 8 long long) and clears them.
extern "C" int unica_b200_trace_read_fp4(long long* host_out) {
    if (cudaMemcpyFromSymbol(host_out, g_trace_fp4, sizeof(long long) * 32) != cudaSuccess) return unica_check_launch("trace_read_fp4");
    static const long long zeros[32] = {};
    if (cudaMemcpyToSymbol(g_trace_fp4, zeros, sizeof zeros) != cudaSuccess) return unica_check_launch("trace_read_fp4");
    return UNICA_B200_OK;
}
#endif

static int attention_fp4(const uint8_t* q4, const void* sfq, const uint8_t* k4, const void* sfk, const uint8_t* v4, const void* sfv,
                         const float* qk_outer, const float* v_outer, const float* bias, int q_blocks, int smooth_q, void* out,
                         void* const* peer_out, int n_peers, unica_token_layout out_layout, int heads, int n_queries, int n_keys,
                         float scale_log2, uint32_t* p_words, int* status, void* stream) {
    if (!q4 || !sfq || !k4 || !sfk || !v4 || !sfv || !qk_outer || !v_outer || !out) return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_fp4: null pointer");
    if (heads <= 0 || heads > 65535 || n_queries <= 0 || n_keys <= 0)
        return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_fp4: heads must be in 1..65535, n_queries and n_keys positive");
    if (bias && (smooth_q <= 0 || smooth_q % 256 || q_blocks != (n_queries + smooth_q - 1) / smooth_q))
        return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_fp4: with a smoothing term, smooth_q must be a multiple of 256 and q_blocks = ceil(n_queries / smooth_q)");
    PeerOutputs peers = {};
    if (int e = unica_peer_outputs(out, peer_out, n_peers, &peers)) return e;
    if (int e = unica_check_device()) return e;
    const dim3 grid((n_queries + 2 * QUERY_TILE - 1) / (2 * QUERY_TILE) * (2 / F4_TILES), heads);  // Q4 holds an even number of tiles
    const size_t smem = sizeof(Fp4Smem) + 128;
    if (cudaFuncSetAttribute(attention_fp4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess ||
        cudaFuncSetAttribute(attention_fp4_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess)
        return unica_check_launch("attention_fp4 (shared memory size)");
    attention_fp4_kernel<<<grid, F4_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(
        q4, static_cast<const uint32_t*>(sfq), k4, static_cast<const uint32_t*>(sfk), v4, static_cast<const uint32_t*>(sfv), qk_outer,
        v_outer, bias, q_blocks, smooth_q > 0 ? smooth_q : 1, static_cast<__nv_bfloat16*>(out), to_layout(out_layout), peers, n_queries,
        n_keys, scale_log2, p_words, status);
    return unica_check_launch("attention_fp4");
}

extern "C" int unica_b200_attention_fp4(const uint8_t* q4, const void* sfq, const uint8_t* k4, const void* sfk, const uint8_t* v4,
                                        const void* sfv, const float* qk_outer, const float* v_outer, const float* bias,
                                        int q_blocks, int smooth_q, void* out, unica_token_layout out_layout, int heads,
                                        int n_queries, int n_keys, float scale_log2, int* status, void* stream) {
    return attention_fp4(q4, sfq, k4, sfk, v4, sfv, qk_outer, v_outer, bias, q_blocks, smooth_q, out, nullptr, 0, out_layout, heads,
                         n_queries, n_keys, scale_log2, nullptr, status, stream);
}

extern "C" int unica_b200_attention_fp4_peers(const uint8_t* q4, const void* sfq, const uint8_t* k4, const void* sfk,
                                              const uint8_t* v4, const void* sfv, const float* qk_outer, const float* v_outer,
                                              const float* bias, int q_blocks, int smooth_q, void* out, void* const* peer_out,
                                              int n_peers, unica_token_layout out_layout, int heads, int n_queries, int n_keys,
                                              float scale_log2, int* status, void* stream) {
    return attention_fp4(q4, sfq, k4, sfk, v4, sfv, qk_outer, v_outer, bias, q_blocks, smooth_q, out, peer_out, n_peers, out_layout, heads,
                         n_queries, n_keys, scale_log2, nullptr, status, stream);
}

extern "C" int unica_b200_attention_fp4_codes(const uint8_t* q4, const void* sfq, const uint8_t* k4, const void* sfk,
                                              const uint8_t* v4, const void* sfv, const float* qk_outer, const float* v_outer,
                                              const float* bias, int q_blocks, int smooth_q, void* out, unica_token_layout out_layout,
                                              int heads, int n_queries, int n_keys, float scale_log2, uint32_t* p_words, int* status,
                                              void* stream) {
    if (!p_words) return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_fp4_codes: null pointer");
    return attention_fp4(q4, sfq, k4, sfk, v4, sfv, qk_outer, v_outer, bias, q_blocks, smooth_q, out, nullptr, 0, out_layout, heads,
                         n_queries, n_keys, scale_log2, p_words, status, stream);
}
