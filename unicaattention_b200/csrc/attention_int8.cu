// The accurate mode's flash-attention loop on tcgen05 (replaces the reference's attention_int8pv_tma, csrc/flash.cu:806-959).
//
// One block = 256 query rows of one head = two tiles of 128 rows that share every K and V tile.  Per query tile g:
//   a softmax warpgroup  (warps 4g .. 4g+3):   thread = query row (tensor-memory lane), 64 scores of the tile -> P^ (u8)
//   a flush warpgroup    (warps 8+4g .. 11+4g): thread = query row, keeps out (float) in TENSOR MEMORY and folds every
//                                               tile's integer P^.V^ into it:  out = out * alpha + beta * float(acc)
// plus warp 16, which streams K8 / V8 tiles (contiguous 8 KB images written by the quantizers) into a ring of
// shared-memory stages with bulk TMA copies, and one thread of warp 17, which issues every tcgen05.mma as soon as its
// operands and its accumulator are free:
//   S[g]   = Q8[g] . K8(t)^T       kind::i8 s8 x s8 -> s32, 128 x 64, 4 instructions of K = 32
//   acc[g] = P^[g](t) . V8(t)[h]   kind::i8 u8 x s8 -> s32, 128 x 64 (channel half h), 2 instructions of K = 32
// Keeping `out` out of the registers is what lets 16 computing warps live on one SM (4 per scheduler): the arithmetic
// of this kernel is a chain of dependent FP32 operations per row, and only several warps per scheduler hide its latency.
//
// Tensor memory, per query tile (256 columns): S 64 | acc 64 (one channel half at a time) | out 128 (float).
//
// Numerics (bench/emulate.py:298-369 with the accurate contract): scores in the log2 domain, c = (q_scale * k_scale) *
// log2(e) / sqrt(d); P^ = rint(255 * 2^(x - tile max)) as u8 against the tile's own maximum; the denominator sums the
// rounded P^ (per channel) or p / s_j in float before rounding (per token); every tile is flushed with
// alpha = 2^(m_old - m_new), beta = 2^(m_tile - m_new).  The 255 stays in numerator and denominator alike (as
// csrc/flash.cu:409-414 does).  No int<->float conversion instruction runs in the loop (see MAGIC in common.cuh): they
// share the quarter-rate pipe with ex2, which is the unit this kernel keeps busiest.
// All waits are bounded (common.cuh).
#include "capi.h"

namespace unica {

constexpr int ATT_THREADS = 640;  // 8 softmax warps, 8 flush warps, and a warpgroup holding the producer and MMA warps
constexpr int SOFTMAX_REGISTERS = 112, FLUSH_REGISTERS = 112, SERVICE_REGISTERS = 32;
constexpr int PRODUCER_WARP = 16, MMA_WARP = 17;
constexpr int STAGES = 3;
constexpr int Q_BYTES = QUERY_TILE * HEAD_DIM;  // 16384
constexpr int K_BYTES = KEY_TILE * HEAD_DIM;    // 8192
constexpr int V_BYTES = KEY_TILE * HEAD_DIM;    // 8192
constexpr int TOK_BYTES = 2 * KEY_TILE * 4;     // 512
constexpr int P_BYTES = QUERY_TILE * KEY_TILE;  // 8192
constexpr int TMEM_COLUMNS = 512;
constexpr int COL_S = 0, COL_ACC = 64, COL_OUT = 128;  // inside a query tile's 256 columns

struct __align__(128) AttSmem {
    int8_t q[2][Q_BYTES];
    int8_t k[STAGES][K_BYTES];
    int8_t v[STAGES][V_BYTES];
    float tok[STAGES][2 * KEY_TILE];
    uint8_t p[2][2][P_BYTES];
    float2 alpha_beta[2][2][QUERY_TILE];
    float den[2][QUERY_TILE];
    uint64_t q_full, k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
    uint64_t s_full[2], s_free[2], p_ready[2][2], p_free[2][2], acc_full[2], acc_free[2], den_ready[2], drain;
    uint32_t tmem_base;
    int abort_flag;
};

// -DUNICA_TRACE: the first thread of each warpgroup of block (0, 0) adds up the cycles it spends in each phase of the
// tile loop (the reference has a TRACE build for the same purpose: csrc/legacy.cu, bench/timeline.py).
#ifdef UNICA_TRACE
__device__ long long g_trace[4][8];
#define TRACE_DECL(slot) long long trace_t0 = clock64(); const int trace_slot = (slot); const bool tracing = blockIdx.x == 0 && blockIdx.y == 0 && row == 0
#define TRACE(phase)                                      \
    do {                                                  \
        if (tracing) {                                    \
            const long long now = clock64();              \
            g_trace[trace_slot][phase] += now - trace_t0; \
            trace_t0 = now;                               \
        }                                                 \
    } while (0)
#else
#define TRACE_DECL(slot)
#define TRACE(phase)
#endif
// Trace builds also leave progress marks in status[1 ..] (block (0, 0) only): pass host-mapped memory to watch a run.
#ifdef UNICA_TRACE
#define MARK(slot, value)                                                    \
    do {                                                                     \
        if (status && blockIdx.x == status[32] && blockIdx.y == status[33]) { \
            reinterpret_cast<volatile int*>(status)[slot] = (value);         \
            __threadfence_system();                                          \
        }                                                                    \
    } while (0)
#else
#define MARK(slot, value)
#endif
enum { TR_WAIT = 0, TR_LOAD = 1, TR_MATH = 2, TR_STORE = 3, TR_WAIT2 = 4, TR_OTHER = 5 };

constexpr uint32_t IDESC_QK = idesc_i8(true, QUERY_TILE, KEY_TILE);
constexpr uint32_t IDESC_PV = idesc_i8(false, QUERY_TILE, HEAD_DIM / 2);

template <bool V_TOKEN>
__global__ void __launch_bounds__(ATT_THREADS, 1)
    attention_int8_kernel(const int8_t* __restrict__ q8, const float* __restrict__ q_scale, const int8_t* __restrict__ k8,
                          const float* __restrict__ k_scale, const int8_t* __restrict__ v8, const float* __restrict__ v_scale,
                          const float* __restrict__ v_token, __nv_bfloat16* __restrict__ out, TokenLayout out_layout,
                          int n_queries, int n_keys, float scale_log2, int* status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    AttSmem& sm = *reinterpret_cast<AttSmem*>(smem_raw);
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int head = blockIdx.y;
    const int q_tiles = 2 * gridDim.x;  // allocated Q tiles per head (even)
    const int k_tiles = (n_keys + KEY_TILE - 1) / KEY_TILE;
    volatile int* abort_flag = &sm.abort_flag;

    if (threadIdx.x == 0) {
        sm.abort_flag = 0;
        mbar_init(&sm.q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&sm.k_full[s], 1);
            mbar_init(&sm.k_empty[s], 1);
            mbar_init(&sm.v_full[s], 1);
            mbar_init(&sm.v_empty[s], 1);
        }
        for (int g = 0; g < 2; ++g) {
            mbar_init(&sm.s_full[g], 1);
            mbar_init(&sm.s_free[g], 128);
            for (int b = 0; b < 2; ++b) {
                mbar_init(&sm.p_ready[g][b], 128);
                mbar_init(&sm.p_free[g][b], 1);
            }
            mbar_init(&sm.acc_full[g], 1);
            mbar_init(&sm.acc_free[g], 128);
            mbar_init(&sm.den_ready[g], 128);
        }
        mbar_init(&sm.drain, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) tmem_alloc(&sm.tmem_base, TMEM_COLUMNS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    if (warp >= 16) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(SERVICE_REGISTERS));
      if (warp == PRODUCER_WARP) {
        // ------------------------------------------------------------------------------------------------ producer
        if (lane == 0) {
            const int8_t* q_src = q8 + (size_t(head) * q_tiles + 2 * blockIdx.x) * Q_BYTES;
            mbar_expect_tx(&sm.q_full, 2 * Q_BYTES);
            bulk_load(sm.q[0], q_src, Q_BYTES, &sm.q_full);
            bulk_load(sm.q[1], q_src + Q_BYTES, Q_BYTES, &sm.q_full);
            int issued = 0;
            for (int t = 0; t < k_tiles; ++t) {
                const int s = t % STAGES, use = t / STAGES;
                if (use > 0 && !mbar_wait(&sm.k_empty[s], (use - 1) & 1, abort_flag, status, STATUS_WAIT_STAGE)) break;
                mbar_expect_tx(&sm.k_full[s], K_BYTES);
                bulk_load(sm.k[s], k8 + (size_t(head) * k_tiles + t) * K_BYTES, K_BYTES, &sm.k_full[s]);
                if (use > 0 && !mbar_wait(&sm.v_empty[s], (use - 1) & 1, abort_flag, status, STATUS_WAIT_STAGE)) {
                    issued = t + 1;  // K of tile t is in flight, V is not
                    break;
                }
                mbar_expect_tx(&sm.v_full[s], V_BYTES + (V_TOKEN ? TOK_BYTES : 0));
                bulk_load(sm.v[s], v8 + (size_t(head) * k_tiles + t) * V_BYTES, V_BYTES, &sm.v_full[s]);
                if (V_TOKEN) bulk_load(sm.tok[s], v_token + (size_t(head) * k_tiles + t) * (2 * KEY_TILE), TOK_BYTES, &sm.v_full[s]);
                issued = t + 1;
                MARK(9, issued);
            }
            if (*abort_flag) {  // let the copies still in flight land before the block's shared memory goes away
                int never = 0;
                for (int t = max(0, issued - STAGES); t < issued; ++t)
                    mbar_wait(&sm.k_full[t % STAGES], (t / STAGES) & 1, &never, nullptr, 0);
                mbar_wait(&sm.q_full, 0, &never, nullptr, 0);
            }
        }
      } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------------------------------------ MMA issue
        // One thread polls what is ready and issues it: per query tile, the scores of the next key tile as soon as the
        // softmax threads have taken the previous ones, and each channel half of P.V as soon as the flush threads have
        // taken the previous half.
        if (lane == 0) {
            const uint32_t q_addr[2] = {smem_u32(sm.q[0]), smem_u32(sm.q[1])};
            bool ok = mbar_wait(&sm.q_full, 0, abort_flag, status, STATUS_WAIT_TILE);
            int s_next[2] = {0, 0};  // next key tile whose scores to issue
            int h_next[2] = {0, 0};  // next P.V half: 2 * tile + channel half
            long long idle_since = clock64();
            while (ok && (s_next[0] < k_tiles || s_next[1] < k_tiles || h_next[0] < 2 * k_tiles || h_next[1] < 2 * k_tiles)) {
                bool progress = false;
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    const int n = s_next[g];
                    if (n < k_tiles && mbar_test(&sm.k_full[n % STAGES], (n / STAGES) & 1) && mbar_test(&sm.s_free[g], n & 1)) {
                        tc_fence_after();
                        const uint32_t k_addr = smem_u32(sm.k[n % STAGES]);
#pragma unroll
                        for (int ks = 0; ks < HEAD_DIM / 32; ++ks)
                            mma_i8_ss(tmem + g * 256 + COL_S, smem_desc(q_addr[g] + ks * 2 * QUERY_TILE * 16, QUERY_TILE * 16, 128),
                                      smem_desc(k_addr + ks * 2 * KEY_TILE * 16, KEY_TILE * 16, 128), IDESC_QK, true);
                        mma_commit(&sm.s_full[g]);
                        s_next[g] = n + 1;
                        if (s_next[1 - g] > n) mma_commit(&sm.k_empty[n % STAGES]);  // both query tiles have read it
                        progress = true;
                    }
                    const int h = h_next[g], t = h >> 1, half = h & 1, buf = t & 1;
                    if (h < 2 * k_tiles && mbar_test(&sm.v_full[t % STAGES], (t / STAGES) & 1) &&
                        mbar_test(&sm.p_ready[g][buf], (t >> 1) & 1) && mbar_test(&sm.acc_free[g], h & 1)) {
                        tc_fence_after();
                        const uint32_t p_addr = smem_u32(sm.p[g][buf]), v_addr = smem_u32(sm.v[t % STAGES]) + half * (HEAD_DIM / 2) * 16;
#pragma unroll
                        for (int ks = 0; ks < KEY_TILE / 32; ++ks)
                            mma_i8_ss(tmem + g * 256 + COL_ACC, smem_desc(p_addr + ks * 2 * QUERY_TILE * 16, QUERY_TILE * 16, 128),
                                      smem_desc(v_addr + ks * 2 * HEAD_DIM * 16, HEAD_DIM * 16, 128), IDESC_PV, ks > 0);
                        mma_commit(&sm.acc_full[g]);
                        h_next[g] = h + 1;
                        if (half) {
                            mma_commit(&sm.p_free[g][buf]);
                            if (h_next[1 - g] > h) mma_commit(&sm.v_empty[t % STAGES]);
                        }
                        progress = true;
                    }
                }
                if (progress) {
                    MARK(5, s_next[0]);
                    MARK(6, s_next[1]);
                    MARK(7, h_next[0]);
                    MARK(8, h_next[1]);
                    idle_since = clock64();
                } else if (*abort_flag) {
                    ok = false;
                } else if (clock64() - idle_since > WAIT_LIMIT_CYCLES) {
                    *abort_flag = 1;
                    if (status) atomicCAS(status, 0, STATUS_WAIT_P);
                    ok = false;
                }
            }
            if (!ok) {  // whatever was issued must finish before tensor memory is freed
                int never = 0;
                mma_commit(&sm.drain);
                mbar_wait(&sm.drain, 0, &never, nullptr, 0);
            }
        }
      }
    } else if (warp < 8) {
        // ------------------------------------------------------------------------------------------------ softmax
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(SOFTMAX_REGISTERS));
        const int g = warp / 4, row = threadIdx.x % 128;
        const int q_tile = 2 * blockIdx.x + g;
        const uint32_t t_scores = tmem + (uint32_t((warp % 4) * 32) << 16) + g * 256 + COL_S;
        const float sq = q_scale[size_t(head) * q_tiles + q_tile];
        const float* sk = k_scale + size_t(head) * k_tiles;
        const float2 minus_magic = make_float2(-MAGIC, -MAGIC), plus_magic = make_float2(MAGIC, MAGIC);
        float m = -INFINITY, den = 0.0f;
        float sk_next = sk[0];
        bool ok = true;
        TRACE_DECL(g);

        // The score accumulator starts at MAGIC_BITS, so what comes back from tensor memory is already a float (common.cuh).
        tmem_fill32(t_scores, MAGIC_BITS);
        tmem_fill32(t_scores + 32, MAGIC_BITS);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&sm.s_free[g]);

        for (int t = 0; ok && t < k_tiles; ++t) {
            const int buf = t & 1, stage = t % STAGES;
            const int valid = min(KEY_TILE, n_keys - t * KEY_TILE);
            const float c = (sq * sk_next) * scale_log2;
            if (t + 1 < k_tiles) sk_next = sk[t + 1];  // needed a whole tile from now
            TRACE(TR_OTHER);
            if (row == 0) MARK(1 + g, t * 16 + 1);
            ok = mbar_wait_warp(&sm.s_full[g], t & 1, abort_flag, status, STATUS_WAIT_SCORES);
            if (ok && V_TOKEN) ok = mbar_wait_warp(&sm.v_full[stage], (t / STAGES) & 1, abort_flag, status, STATUS_WAIT_TILE);
            if (!ok) break;
            tc_fence_after();
            TRACE(TR_WAIT);
            if (row == 0) MARK(1 + g, t * 16 + 2);
            float2 x[KEY_TILE / 2];  // MAGIC + score, exactly
            tmem_ld64_sync(t_scores, x);
            tmem_fill32(t_scores, MAGIC_BITS);
            tmem_fill32(t_scores + 32, MAGIC_BITS);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&sm.s_free[g]);
            if (row == 0) MARK(1 + g, t * 16 + 3);
            TRACE(TR_LOAD);

            const float2 c2 = make_float2(c, c);
            float tile_max;
            if (!V_TOKEN) {
                if (valid < KEY_TILE) {  // keys past the end: below every real score (|score| < 2^21)
#pragma unroll
                    for (int j = 0; j < KEY_TILE; ++j)
                        if (j >= valid) (j % 2 ? x[j / 2].y : x[j / 2].x) = MAGIC - 4194303.0f;
                }
            } else {
                const float2* log_s = reinterpret_cast<const float2*>(sm.tok[stage]);
#pragma unroll
                for (int j = 0; j < KEY_TILE / 2; ++j) x[j] = fma2(add2(x[j], minus_magic), c2, log_s[j]);
                if (valid < KEY_TILE) {
#pragma unroll
                    for (int j = 0; j < KEY_TILE; ++j)
                        if (j >= valid) (j % 2 ? x[j / 2].y : x[j / 2].x) = -INFINITY;
                }
            }
            {  // the maximum as a tree: four independent chains
                float top[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) top[i] = fmaxf(x[i].x, x[i].y);
#pragma unroll
                for (int j = 4; j < KEY_TILE / 2; ++j) top[j % 4] = max3(top[j % 4], x[j].x, x[j].y);
                tile_max = fmaxf(fmaxf(top[0], top[1]), fmaxf(top[2], top[3]));
                if (!V_TOKEN) tile_max = (tile_max - MAGIC) * c;
            }
            const float m_new = fmaxf(m, tile_max);
            const float alpha = ex2(m - m_new), beta = ex2(tile_max - m_new);
            m = m_new;
            const float offset = LOG2_255 - tile_max;
            const float2 offset2 = make_float2(offset, offset);
            if (row == 0) MARK(1 + g, t * 16 + 4);
            if (t >= 2) {  // the P buffer is free once P.V of tile t - 2 has read it
                ok = mbar_wait_warp(&sm.p_free[g][buf], ((t >> 1) - 1) & 1, abort_flag, status, STATUS_WAIT_FREE);
                if (!ok) break;
            }
            uint8_t* p_row = sm.p[g][buf] + row * 16;
            unsigned isum[2] = {0, 0};
            float2 fsum = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int chunk = 0; chunk < KEY_TILE / 16; ++chunk) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t half[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int j = chunk * 8 + i * 2 + h;  // a pair of keys
                        const float2 e = V_TOKEN ? add2(x[j], offset2) : fma2(add2(x[j], minus_magic), c2, offset2);
                        const float2 p = make_float2(ex2(e.x), ex2(e.y));
                        if (V_TOKEN) fsum = fma2(p, reinterpret_cast<const float2*>(sm.tok[stage] + KEY_TILE)[j], fsum);
                        const float2 r = add2(p, plus_magic);  // the low byte of each is rint(p)
                        half[h] = __byte_perm(__float_as_uint(r.x), __float_as_uint(r.y), 0x0040);
                    }
                    w[i] = __byte_perm(half[0], half[1], 0x5410);
                    if (!V_TOKEN && valid < KEY_TILE) {  // keys past the end weigh nothing
                        const int left = valid - (chunk * 16 + i * 4);
                        w[i] = left >= 4 ? w[i] : left <= 0 ? 0u : (w[i] & ((1u << (8 * left)) - 1u));
                    }
                    if (!V_TOKEN) isum[i % 2] = __dp4a(w[i], 0x01010101u, isum[i % 2]);
                }
                *reinterpret_cast<uint4*>(p_row + chunk * (QUERY_TILE * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            sm.alpha_beta[g][buf][row] = make_float2(alpha, beta);
            TRACE(TR_MATH);
            fence_proxy_async();
            mbar_arrive(&sm.p_ready[g][buf]);
            if (row == 0) MARK(1 + g, t * 16 + 5);
            TRACE(TR_STORE);
            den = den * alpha + (V_TOKEN ? fsum.x + fsum.y : __uint2float_rn(isum[0] + isum[1])) * beta;
        }
        sm.den[g][row] = den;
        mbar_arrive(&sm.den_ready[g]);
    } else {
        // ------------------------------------------------------------------------------------------------ flush
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(FLUSH_REGISTERS));
        const int g = (warp - 8) / 4, row = threadIdx.x % 128;
        const int q_row = (2 * blockIdx.x + g) * QUERY_TILE + row;
        const uint32_t t_base = tmem + (uint32_t((warp % 4) * 32) << 16) + g * 256;
        const uint32_t t_acc = t_base + COL_ACC, t_out = t_base + COL_OUT;
        const float2 minus_magic = make_float2(-MAGIC, -MAGIC);
        bool ok = true;
        TRACE_DECL(2 + g);

#pragma unroll
        for (int c = 0; c < HEAD_DIM; c += 32) tmem_fill32(t_out + c, 0u);  // out = 0
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&sm.acc_free[g]);

        for (int t = 0; ok && t < k_tiles; ++t) {
            const int buf = t & 1;
            float2 ab = make_float2(1.0f, 1.0f);
            bool rescale = false;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                TRACE(TR_OTHER);
                if (row == 0) MARK(3 + g, (2 * t + half) * 16 + 1);
                ok = mbar_wait_warp(&sm.acc_full[g], (2 * t + half) & 1, abort_flag, status, STATUS_WAIT_PV);
                if (!ok) break;
                tc_fence_after();
                TRACE(TR_WAIT);
                if (half == 0) {
                    // alpha and beta were written before the arrival on p_ready, which P.V of this tile waited for; they
                    // are read before acc is released, because the second half's completion frees them for tile t + 2
                    ok = mbar_wait_warp(&sm.p_ready[g][buf], (t >> 1) & 1, abort_flag, status, STATUS_WAIT_P);
                    if (!ok) break;
                    ab = sm.alpha_beta[g][buf][row];
                    rescale = !__all_sync(0xffffffffu, ab.x == 1.0f);
                }
                if (row == 0) MARK(3 + g, (2 * t + half) * 16 + 2);
                float2 a[32];  // 64 channels of P^.V^, integers
                tmem_ld64_sync(t_acc, a);
                tc_fence_before();
                mbar_arrive(&sm.acc_free[g]);  // the other half (or the next tile) may start
                if (row == 0) MARK(3 + g, (2 * t + half) * 16 + 3);
                TRACE(TR_LOAD);
                const float2 alpha2 = make_float2(ab.x, ab.x), beta2 = make_float2(ab.y, ab.y);
#pragma unroll
                for (int part = 0; part < 4; ++part) {
                    float2 o[8];
                    tmem_ld16_sync(t_out + half * 64 + part * 16, o);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float2 f;  // float(acc): MAGIC_BITS + value read as a float is MAGIC + value
                        f.x = __uint_as_float(__float_as_uint(a[part * 8 + i].x) + MAGIC_BITS);
                        f.y = __uint_as_float(__float_as_uint(a[part * 8 + i].y) + MAGIC_BITS);
                        if (rescale) o[i] = mul2(o[i], alpha2);
                        o[i] = fma2(beta2, add2(f, minus_magic), o[i]);
                    }
                    tmem_st16(t_out + half * 64 + part * 16, o);
                }
                tmem_wait_st();
                if (row == 0) MARK(3 + g, (2 * t + half) * 16 + 4);
                TRACE(TR_MATH);
            }
        }

        if (ok) ok = mbar_wait_warp(&sm.den_ready[g], 0, abort_flag, status, STATUS_WAIT_P);
        ok = __all_sync(0xffffffffu, ok);  // the tensor-memory loads below are warp-wide: no lane may skip them
        if (ok) {
            const bool valid_row = q_row < n_queries;
            const float inv = 1.0f / sm.den[g][row];
            __nv_bfloat16* dst = out + out_layout.offset(head, valid_row ? q_row : 0);
#pragma unroll
            for (int part = 0; part < HEAD_DIM / 16; ++part) {
                float2 o[8];
                tmem_ld16_sync(t_out + part * 16, o);
                uint32_t w[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int c0 = part * 16 + 2 * i;
                    const __nv_bfloat162 pair = __floats2bfloat162_rn(o[i].x * v_scale[head * HEAD_DIM + c0] * inv,
                                                                      o[i].y * v_scale[head * HEAD_DIM + c0 + 1] * inv);
                    w[i] = *reinterpret_cast<const uint32_t*>(&pair);
                }
                if (valid_row) {
                    *reinterpret_cast<uint4*>(dst + part * 16) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(dst + part * 16 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
        }
    }

    if (lane == 0) MARK(10 + warp, 1);
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLUMNS);
    }
    if (threadIdx.x == 0) MARK(31, 1);
}

// ---------------------------------------------------------------------------------------------------------------------
// Self-test: one tcgen05.mma chain on operand images given by the caller, accumulator copied out as it lies in tensor memory.

__global__ void __launch_bounds__(128) selftest_mma_i8_kernel(const uint8_t* __restrict__ a_image, const uint8_t* __restrict__ b_image,
                                                              int n, int k, int a_unsigned, int variant, int32_t* __restrict__ d,
                                                              int* status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* a_s = smem_raw;             // [k / 16][128][16]
    uint8_t* b_s = smem_raw + 128 * k;   // [k / 16][n][16]
    __shared__ uint64_t done;
    __shared__ uint32_t tmem_base;
    __shared__ int abort_flag;
    for (int i = threadIdx.x; i < 128 * k / 16; i += 128) reinterpret_cast<uint4*>(a_s)[i] = reinterpret_cast<const uint4*>(a_image)[i];
    for (int i = threadIdx.x; i < n * k / 16; i += 128) reinterpret_cast<uint4*>(b_s)[i] = reinterpret_cast<const uint4*>(b_image)[i];
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_proxy_async();
    if (threadIdx.x / 32 == 0) tmem_alloc(&tmem_base, 128);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base;
    if (threadIdx.x == 0) {
        const uint32_t idesc = idesc_i8(!a_unsigned, 128, n);
        for (int ks = 0; ks < k / 32; ++ks) {
            uint64_t da, db;
            if (variant == 0) {
                da = smem_desc(smem_u32(a_s) + ks * 2 * 128 * 16, 128 * 16, 128);
                db = smem_desc(smem_u32(b_s) + ks * 2 * n * 16, n * 16, 128);
            } else {  // diagnostic: the two offsets exchanged
                da = smem_desc(smem_u32(a_s) + ks * 2 * 128 * 16, 128, 128 * 16);
                db = smem_desc(smem_u32(b_s) + ks * 2 * n * 16, 128, n * 16);
            }
            mma_i8_ss(tmem, da, db, idesc, ks > 0);
        }
        mma_commit(&done);
    }
    const bool ok = mbar_wait(&done, 0, &abort_flag, status, STATUS_WAIT_SCORES);
    tc_fence_after();
    if (ok) {
        const uint32_t lane_base = uint32_t((threadIdx.x / 32) * 32) << 16;
        for (int c0 = 0; c0 < n; c0 += 32) {
            uint32_t r[32];
            tmem_ld32(tmem + lane_base + c0, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) d[threadIdx.x * n + c0 + i] = int32_t(r[i]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x / 32 == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, 128);
    }
}

}  // namespace unica

using namespace unica;

extern "C" int unica_b200_attention_int8(const int8_t* q8, const float* q_scale, const int8_t* k8, const float* k_scale,
                                         const int8_t* v8, const float* v_scale, const float* v_token, int v_mode, void* out,
                                         unica_token_layout out_layout, int heads, int n_queries, int n_keys, float scale_log2,
                                         int* status, void* stream) {
    if (!q8 || !q_scale || !k8 || !k_scale || !v8 || !v_scale || !out) return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_int8: null pointer");
    if (heads <= 0 || heads > 65535 || n_queries <= 0 || n_keys <= 0)
        return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_int8: heads must be in 1..65535, n_queries and n_keys positive");
    if (v_mode != UNICA_B200_V_CHANNEL && v_mode != UNICA_B200_V_TOKEN) return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_int8: unknown v_mode");
    if (v_mode == UNICA_B200_V_TOKEN && !v_token) return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_int8: per-token mode needs v_token");
    if (int e = unica_check_device()) return e;
    const dim3 grid((n_queries + 2 * QUERY_TILE - 1) / (2 * QUERY_TILE), heads);
    const size_t smem = sizeof(AttSmem) + 128;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    auto launch = [&](auto kernel) -> int {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
            return unica_check_launch("attention_int8 (shared memory size)");
        kernel<<<grid, ATT_THREADS, smem, s>>>(q8, q_scale, k8, k_scale, v8, v_scale, v_token, static_cast<__nv_bfloat16*>(out),
                                               to_layout(out_layout), n_queries, n_keys, scale_log2, status);
        return unica_check_launch("attention_int8");
    };
    return v_mode == UNICA_B200_V_TOKEN ? launch(attention_int8_kernel<true>) : launch(attention_int8_kernel<false>);
}

#ifdef UNICA_TRACE
// Trace builds only: copies the per-phase cycle totals of block (0, 0) to `host_out` (4 x 8 long long) and clears them.
extern "C" int unica_b200_trace_read(long long* host_out) {
    if (cudaMemcpyFromSymbol(host_out, g_trace, sizeof(long long) * 32) != cudaSuccess) return unica_check_launch("trace_read");
    static const long long zeros[32] = {};
    if (cudaMemcpyToSymbol(g_trace, zeros, sizeof zeros) != cudaSuccess) return unica_check_launch("trace_read");
    return UNICA_B200_OK;
}
#endif

extern "C" int unica_b200_selftest_mma_i8(const void* a_image, const void* b_image, int n, int k, int a_unsigned, int variant,
                                          int32_t* d, void* stream) {
    if (!a_image || !b_image || !d) return unica_fail(UNICA_B200_ERR_ARGUMENT, "selftest_mma_i8: null pointer");
    if (n < 32 || n > 128 || n % 32 || k < 32 || k > 128 || k % 32)
        return unica_fail(UNICA_B200_ERR_ARGUMENT, "selftest_mma_i8: n and k must be multiples of 32 in 32..128");
    if (int e = unica_check_device()) return e;
    const size_t smem = size_t(128 + n) * k + 128;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int* status = nullptr;
    if (cudaMalloc(&status, sizeof(int)) != cudaSuccess || cudaMemsetAsync(status, 0, sizeof(int), s) != cudaSuccess)
        return unica_check_launch("selftest_mma_i8 (status word)");
    selftest_mma_i8_kernel<<<1, 128, smem, s>>>(static_cast<const uint8_t*>(a_image), static_cast<const uint8_t*>(b_image), n, k,
                                                a_unsigned, variant, d, status);
    int host_status = 0;
    cudaError_t e = cudaMemcpyAsync(&host_status, status, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaFree(status);
    if (e != cudaSuccess) {
        unica_fail(UNICA_B200_ERR_CUDA, cudaGetErrorString(e));
        return UNICA_B200_ERR_CUDA;
    }
    if (host_status) return unica_fail(UNICA_B200_ERR_KERNEL, "selftest_mma_i8: the tensor-core instruction never completed");
    return UNICA_B200_OK;
}
