// The accurate mode's flash-attention loop on tcgen05 (replaces the reference's attention_int8pv_tma, csrc/flash.cu:806-959).
//
// One block = one tile of 128 query rows of one head, one block per SM, 16 warps in four warpgroups with three kinds of
// work (a thread of a computing warpgroup owns one query row = one tensor-memory lane, so row maxima and sums need no
// shuffles):
//
//   softmax A, B   key tiles t = 0, 2, 4 .. and 1, 3, 5 ..: the scores S(t) of tensor memory, read once into registers,
//                  become the bytes P^(t) = rint(255 * 2^(x - tile max)) of the A-operand image in shared memory; the tile
//                  maximum and the row sum go to the flush threads through shared memory.  They carry nothing from tile to
//                  tile.
//   flush          out = out * alpha + beta * float(acc(t)) for every key tile t, the row's 128 outputs in registers;
//                  they own the running exponent and the denominator, and write the result.
//   service        four warps, one elected thread each, two per key-tile parity: one issues the scores, one issues P.V and
//                  copies K8 / V8 tiles (contiguous 8 KB images written by the quantizers, bulk TMA) into a ring of
//                  shared-memory stages:
//
//   S(t)   = Q8 . K8(t)^T      kind::i8 s8 x s8 -> s32, 128 x 64, 4 instructions of K = 32, a ring of 4 buffers
//   acc(t) = P^(t) . V8(t)     kind::i8 u8 x s8 -> s32, 128 x 128, 2 instructions of K = 32, two accumulators (t even / odd)
//
// What was measured on the way here (B200): the exponentials of two softmax warps per scheduler alone take 567 cycles
// per 128 x 64 tile and overlap with a flush warp's conversions almost freely, the tensor pipe alone 476; what decides
// the kernel's speed is the chain of hand-overs between the roles.  A lone thread pays some 250 cycles for an mbarrier
// probe, so MMA issue is dealt out to four threads and a thread waits for two barriers with both probes in flight.  A
// thread or warp that has to wait longer is suspended by the hardware on the barrier (mbarrier.try_wait with a time
// hint) instead of spinning: a spinning waiter takes issue slots from the computing warps of its scheduler.  Per token
// the completion of tcgen05.mma is instead passed on by the issuing thread through words in shared memory that a
// waiting warp reads in 30 cycles.
//
// Numerics (bench/emulate.py:298-369 with the accurate contract): scores in the log2 domain, c = (q_scale * k_scale) *
// log2(e) / sqrt(d); P^ as u8 against the tile's own maximum; the denominator sums the rounded P^ (per channel) or
// p / s_j in float before rounding (per token); every tile is flushed as out = out * alpha + beta * float(acc) with
// beta = 2^(m_tile - m) and alpha = 2^(m_old - m_new), where m is a reference exponent that follows the running maximum
// only in large steps (the common factor cancels against the denominator's).  The 255 stays in numerator and
// denominator alike (as csrc/flash.cu:409-414 does).
//
// Tensor memory (all 512 columns): S ring 4 x 64 | acc 2 x 128.  All waits are bounded (common.cuh).
#include <atomic>
#include <type_traits>

#include "capi.h"

namespace unica {

constexpr int FLUSH_WARP = 8, SERVICE_WARP = 12, ATT_WARPS = 16, ATT_THREADS = ATT_WARPS * 32;
// registers per thread after setmaxnreg; the block is launched with ATT_THREADS x LAUNCH_REGISTERS = 65536
constexpr int LAUNCH_REGISTERS = 128, SOFTMAX_REGISTERS = 120, FLUSH_REGISTERS = 232, SERVICE_REGISTERS = 32;
static_assert(128 * (2 * SOFTMAX_REGISTERS + FLUSH_REGISTERS + SERVICE_REGISTERS) <= ATT_THREADS * LAUNCH_REGISTERS, "the split must fit the launch");
template <int REGISTERS>
__device__ __forceinline__ void set_registers() {  // every warp of a warpgroup executes it
    if constexpr (REGISTERS > LAUNCH_REGISTERS)
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGISTERS));
    else
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGISTERS));
}
constexpr int STAGES = 6;   // K8 / V8 tiles in shared memory
constexpr int S_RING = 4;   // score buffers in tensor memory
constexpr int P_RING = STAGES;  // P^ images in shared memory: one per stage (see the P.V issuing thread)
static_assert(STAGES % 2 == 0 && STAGES > S_RING, "a softmax warpgroup steps through the stages two at a time");
constexpr int ST_RING = 8;  // (tile maximum, row sum) records on their way from the softmax to the flush threads
constexpr int Q_BYTES = QUERY_TILE * HEAD_DIM;  // 16384
constexpr int K_BYTES = KEY_TILE * HEAD_DIM;    // 8192
constexpr int V_BYTES = KEY_TILE * HEAD_DIM;    // 8192
constexpr int TOK_BYTES = 2 * KEY_TILE * 4;     // 512
constexpr int P_BYTES = QUERY_TILE * KEY_TILE;  // 8192
constexpr int TMEM_COLUMNS = 512;
constexpr int COL_S = 0, COL_ACC = 256;
constexpr int OUTLIER_BATCH = 16;  // outlier keys whose rows are in shared memory at a time (the epilogue of the outliers mode)
constexpr float REFERENCE_SLACK = 60.0f;  // log2: how far a tile maximum may rise above a row's reference exponent

struct __align__(128) AttSmem {
    int8_t q[Q_BYTES];
    int8_t k[STAGES][K_BYTES];
    int8_t v[STAGES][V_BYTES];
    float tok[STAGES][2 * KEY_TILE];
    uint8_t p[P_RING][P_BYTES];
    float2 st[ST_RING][QUERY_TILE];
    uint64_t q_full, kv_full[STAGES], kv_empty[STAGES];
    uint64_t s_ready, s_full[S_RING], soft_done[ST_RING], acc_free[2], drain[4];
    int s_done[S_RING], acc_done[2];  // key tile + 1 of the last S / P.V seen complete in each buffer (see flag_publish)
    uint32_t tmem_base;
    int abort_flag;
};

// -DUNICA_TRACE: thread 0 of each role of block (0, 0) adds up the cycles it spends in each phase of its tile loop and
// notes when key tiles EVENT_FIRST .. + 15 passed from role to role (the reference has a TRACE build for the same
// purpose: csrc/legacy.cu, bench/timeline.py).  Rows of g_trace: softmax A, softmax B, flush, P.V-issuing thread,
// scores-issuing thread.  The totals stay in registers until the end: tracing costs a clock read per phase.
#ifndef UNICA_SERVICE_SLEEP_NS
#define UNICA_SERVICE_SLEEP_NS 0
#endif
constexpr unsigned SERVICE_SLEEP = UNICA_SERVICE_SLEEP_NS;  // the service threads pass events on: they do not sleep between probes
#ifdef UNICA_TRACE
__device__ long long g_trace[5][8];
__device__ long long g_events[8][16];
constexpr int EVENT_FIRST = 64;
#define EVENT(kind, tile) do { if (tracing && (tile) >= EVENT_FIRST && (tile) < EVENT_FIRST + 16) g_events[kind][(tile) - EVENT_FIRST] = clock64(); } while (0)
#define TRACE_DECL(on) long long trace_t0 = clock64(), trace_sum[8] = {}; const bool tracing = blockIdx.x == 0 && blockIdx.y == 0 && (on)
#define TRACE(phase)                                 \
    do {                                             \
        if (tracing) {                               \
            const long long now = clock64();         \
            trace_sum[phase] += now - trace_t0;      \
            trace_t0 = now;                          \
        }                                            \
    } while (0)
#define TRACE_END(slot)                                                   \
    do {                                                                  \
        if (tracing)                                                      \
            for (int i = 0; i < 8; ++i) g_trace[slot][i] = trace_sum[i];  \
    } while (0)
#else
#define TRACE_DECL(on)
#define TRACE(phase)
#define TRACE_END(slot)
#define EVENT(kind, tile)
#endif

constexpr uint32_t IDESC_QK = idesc_i8(true, QUERY_TILE, KEY_TILE);
constexpr uint32_t IDESC_PV = idesc_i8(false, QUERY_TILE, HEAD_DIM);

// One step of a row's sums: the reference exponent `m` and the factors of the tile whose maximum is `tile_max`.
// `m` is the exponent the sums are kept at, not the running maximum: out = sum over tiles of 2^(tile max - m) * acc, the
// same for the denominator, and the common factor cancels at the end.  The textbook form moves m to every new maximum
// and multiplies out and den by alpha = 2^(m_old - m_new) each time; here m moves only when a tile maximum is more than
// 2^REFERENCE_SLACK above it, so that multiplication all but disappears.  The difference is rounding only.
__device__ __forceinline__ void reference_step(float& m, float tile_max, float& alpha, float& beta) {
    const bool first = m == -INFINITY;
    const float m_new = tile_max > m + REFERENCE_SLACK ? tile_max : m;
    alpha = first ? 1.0f : ex2(m - m_new);
    beta = ex2(tile_max - m_new);
    m = m_new;
}

// 32 accumulator values (plain integers: every tile's P.V overwrites the accumulator) into 32 of a row's sums.
__device__ __forceinline__ void flush32(float2 (&y)[16], float2* o, float alpha, float beta, bool rescale) {
    const float2 alpha2 = make_float2(alpha, alpha), beta2 = make_float2(beta, beta);
    if (rescale) {
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = mul2(o[i], alpha2);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) y[i] = make_float2(__int2float_rn(__float_as_int(y[i].x)), __int2float_rn(__float_as_int(y[i].y)));
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i] = fma2(beta2, y[i], o[i]);
}

template <bool V_TOKEN, bool OUTLIERS>
__global__ void __launch_bounds__(ATT_THREADS, 1)
    attention_int8_kernel(const int8_t* __restrict__ q8, const float* __restrict__ q_scale, const int8_t* __restrict__ k8,
                          const float* __restrict__ k_scale, const int8_t* __restrict__ v8, const float* __restrict__ v_scale,
                          const float* __restrict__ v_token, const int* __restrict__ outlier_keys,
                          const float* __restrict__ outlier_rows, int n_outliers, __nv_bfloat16* __restrict__ out,
                          TokenLayout out_layout, const __grid_constant__ PeerOutputs peers, int n_queries, int n_keys, float scale_log2, int* status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    AttSmem& sm = *reinterpret_cast<AttSmem*>(smem_raw);
    const int warp = threadIdx.x / 32;
    const int head = blockIdx.y;
    const int q_tiles = gridDim.x;  // allocated Q tiles per head (even)
    const int q_tile = blockIdx.x;
    if (q_tile * QUERY_TILE >= n_queries) return;  // the padding tile of an odd count: nothing to do
    const int k_tiles = (n_keys + KEY_TILE - 1) / KEY_TILE;
    volatile int* abort_flag = &sm.abort_flag;
    // How the softmax and flush warps learn that S(t) / P.V(t) is complete.  Per channel and with outliers they wait on the
    // instructions' own barrier, suspended by the hardware; per token that measured 1 % slower than looking at a word
    // in shared memory that the issuing thread, which watches the barrier anyway, advances (flag_publish).
    constexpr bool FLAG_WAITS = V_TOKEN;

    if (threadIdx.x == 0) {
        sm.abort_flag = 0;
        mbar_init(&sm.q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&sm.kv_full[s], 1);
            mbar_init(&sm.kv_empty[s], 1);
        }
        mbar_init(&sm.s_ready, 256);
        for (int b = 0; b < S_RING; ++b) mbar_init(&sm.s_full[b], 1), sm.s_done[b] = 0;
        for (int b = 0; b < ST_RING; ++b) mbar_init(&sm.soft_done[b], 128);
        for (int b = 0; b < 2; ++b) mbar_init(&sm.acc_free[b], 128), sm.acc_done[b] = 0;
        for (int i = 0; i < 4; ++i) mbar_init(&sm.drain[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == SERVICE_WARP) tmem_alloc(&sm.tmem_base, TMEM_COLUMNS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    const int row = threadIdx.x % 128, q_row = q_tile * QUERY_TILE + row;
    const uint32_t lane_base = uint32_t((warp % 4) * 32) << 16;
    const bool ragged = n_keys % KEY_TILE != 0;  // the last key tile needs masking

    if (warp >= SERVICE_WARP) {
      set_registers<SERVICE_REGISTERS>();
      // Four service warps, one elected thread each, two per key-tile parity.  A thread that issues tcgen05.mma runs a
      // chain of dependent barrier probes and instruction issues that takes several hundred cycles per tile (a probe
      // alone, by a lone thread, some 250), so the tiles are dealt out: no thread sees more than every other tile.
      const int parity = (warp - SERVICE_WARP) & 1;
      if (warp < SERVICE_WARP + 2) {
        // -------------------------------------------------------------------------- scores S(n), n = parity, parity + 2, ..
        // S(n) = Q8 . K8(n)^T goes out as soon as K8(n) has landed and the softmax of tile n - 4 (the same warpgroup's
        // last tile but one) has handed the scores buffer back.
        if (elect_one()) {  // one elected lane of a converged warp: see elect_one() in common.cuh
            const uint64_t q_desc0 = smem_desc(smem_u32(sm.q), QUERY_TILE * 16, 128), k_desc0 = smem_desc(smem_u32(sm.k[0]), KEY_TILE * 16, 128);
            bool ok = mbar_wait2<SERVICE_SLEEP>(&sm.q_full, 0, &sm.s_ready, 0, abort_flag, status, STATUS_WAIT_TILE);  // s_ready: the score buffers hold their start value
            TRACE_DECL(true);
            for (int n = parity, stage = parity, phase = 0; ok && n < k_tiles; n += 2) {
                const int buf = n % S_RING;
                TRACE(7);
                ok = mbar_wait2<SERVICE_SLEEP>(&sm.kv_full[stage], phase, &sm.soft_done[(n - S_RING) & (ST_RING - 1)], n >= S_RING ? ((n - S_RING) / ST_RING) & 1 : -1,
                                abort_flag, status, STATUS_WAIT_TILE);
                TRACE(0);
                if (!ok) break;
                tc_fence_after();
                const uint64_t k_desc = k_desc0 + uint64_t(stage * (K_BYTES / 16));
#pragma unroll
                for (int ks = 0; ks < HEAD_DIM / 32; ++ks)
                    mma_i8_ss(tmem + COL_S + buf * 64, q_desc0 + ks * (2 * QUERY_TILE * 16 / 16), k_desc + ks * (2 * KEY_TILE * 16 / 16), IDESC_QK, true);
                mma_commit(&sm.s_full[buf]);
                TRACE(2);
                EVENT(6, n);
                // the thread watches its own instructions complete before it turns to its next tile (going on at once
                // measured slower) and, per token, tells the softmax threads through a word they can look at cheaply
                ok = mbar_wait<SERVICE_SLEEP>(&sm.s_full[buf], (n / S_RING) & 1, abort_flag, status, STATUS_WAIT_SCORES);
                if (!ok) break;
                if (FLAG_WAITS) {
                    tc_fence_before();
                    flag_publish(&sm.s_done[buf], n + 1);
                }
                TRACE(3);
                stage += 2;
                if (stage >= STAGES) stage -= STAGES, phase ^= 1;
            }
            if (parity == 0) TRACE_END(4);
            if (!ok) {  // whatever was issued must finish before tensor memory is freed
                int never = 0;
                mma_commit(&sm.drain[parity]);
                mbar_wait(&sm.drain[parity], 0, &never, nullptr, 0);
            }
        }
      } else {
        // -------------------------------------------------------------------------- P.V(t) and the K8 / V8 copies, t = parity, parity + 2, ..
        // P.V(t), into accumulator `parity`, goes out as soon as P^(t) is delivered and the flush of tile t - 2 has read the
        // accumulator.  When it completes, its stage is free and the same thread copies tile t + STAGES into it (contiguous
        // 8 KB images written by the quantizers, bulk TMA).  The P^ ring relies on that order: scores S(t) can only be issued
        // once K8(t) has landed in the stage P.V(t - STAGES) has released, so when they complete, the P^ image of tile
        // t - STAGES has been read.  V8(t) landed before S(t) was issued, which the softmax of tile t waited for before it
        // delivered P^(t).
        if (elect_one()) {
            const int8_t* k_src = k8 + size_t(head) * k_tiles * K_BYTES;
            const int8_t* v_src = v8 + size_t(head) * k_tiles * V_BYTES;
            const float* tok_src = V_TOKEN ? v_token + size_t(head) * k_tiles * (2 * KEY_TILE) : nullptr;
            int issued = 0;  // copies of this parity's tiles issued so far
            TRACE_DECL(true);
            auto copy_tile = [&](int tile, int stage) {
                mbar_expect_tx(&sm.kv_full[stage], K_BYTES + V_BYTES + (V_TOKEN ? TOK_BYTES : 0));
                bulk_load(sm.k[stage], k_src + size_t(tile) * K_BYTES, K_BYTES, &sm.kv_full[stage]);
                bulk_load(sm.v[stage], v_src + size_t(tile) * V_BYTES, V_BYTES, &sm.kv_full[stage]);
                if (V_TOKEN) bulk_load(sm.tok[stage], tok_src + size_t(tile) * (2 * KEY_TILE), TOK_BYTES, &sm.kv_full[stage]);
                ++issued;
                EVENT(7, tile);
            };
            if (parity == 0) {
                mbar_expect_tx(&sm.q_full, Q_BYTES);
                bulk_load(sm.q, q8 + (size_t(head) * q_tiles + q_tile) * Q_BYTES, Q_BYTES, &sm.q_full);
            }
            for (int n = parity; n < min(k_tiles, STAGES); n += 2) copy_tile(n, n);
            bool ok = true;
            const int b = parity;
            const uint64_t p_desc0 = smem_desc(smem_u32(sm.p[0]), QUERY_TILE * 16, 128), v_desc0 = smem_desc(smem_u32(sm.v[0]), HEAD_DIM * 16, 128);
            for (int t = parity, stage = parity, phase = 0; ok && t < k_tiles; t += 2) {
                TRACE(7);
                const int free_parity = t >= 2 ? ((t - 2) >> 1) & 1 : -1;  // the flushes of tile t - 2 have read the accumulator
                ok = mbar_wait2<SERVICE_SLEEP>(&sm.soft_done[t % ST_RING], (t / ST_RING) & 1, &sm.acc_free[b], free_parity, abort_flag, status, STATUS_WAIT_P);
                TRACE(3);
                if (!ok) break;
                tc_fence_after();
                // a descriptor's address field counts 16-byte units: the images of stage `stage`, K step ks
                const uint64_t p_desc = p_desc0 + uint64_t(stage * (P_BYTES / 16)), v_desc = v_desc0 + uint64_t(stage * (V_BYTES / 16));
#pragma unroll
                for (int ks = 0; ks < KEY_TILE / 32; ++ks)
                    mma_i8_ss(tmem + COL_ACC + b * 128, p_desc + ks * (2 * QUERY_TILE * 16 / 16), v_desc + ks * (2 * HEAD_DIM * 16 / 16), IDESC_PV,
                              ks > 0);  // the first instruction of a tile overwrites the accumulator
                mma_commit(&sm.kv_empty[stage]);
                TRACE(4);
                EVENT(2, t);
                // P.V(t) complete: the stage is free (and, per token, the flush threads are told through a word)
                ok = mbar_wait<SERVICE_SLEEP>(&sm.kv_empty[stage], phase, abort_flag, status, STATUS_WAIT_STAGE);
                if (!ok) break;
                if (FLAG_WAITS) {
                    tc_fence_before();
                    flag_publish(&sm.acc_done[b], t + 1);
                }
                if (t + STAGES < k_tiles) copy_tile(t + STAGES, stage);
                TRACE(5);
                stage += 2;
                if (stage >= STAGES) stage -= STAGES, phase ^= 1;
            }
            if (parity == 0) TRACE_END(3);
            if (!ok) {
                int never = 0;
                mma_commit(&sm.drain[2 + parity]);
                mbar_wait(&sm.drain[2 + parity], 0, &never, nullptr, 0);
            }
            if (*abort_flag) {  // let the copies still in flight land before the block's shared memory goes away
                int never = 0;
                for (int i = max(0, issued - STAGES / 2); i < issued; ++i) {
                    const int tile = parity + 2 * i;
                    mbar_wait(&sm.kv_full[tile % STAGES], (tile / STAGES) & 1, &never, nullptr, 0);
                }
                mbar_wait(&sm.q_full, 0, &never, nullptr, 0);
            }
        }
      }
    } else if (warp < FLUSH_WARP) {
        // ------------------------------------------------------------------------------------------------ softmax
        set_registers<SOFTMAX_REGISTERS>();
        const int parity = warp / 4;  // this warpgroup's key tiles: t = parity, parity + 2, ..
        const uint32_t t_s = tmem + lane_base + COL_S;
        const float sq = q_scale[size_t(head) * q_tiles + q_tile];
        const float* sk = k_scale + size_t(head) * k_tiles;
        // The K scale of the tile after this one, loaded a whole tile ahead of its use (volatile: the compiler would
        // otherwise sink the load to the use and expose its latency on every tile).
        auto load_scale = [](const float* p) {
            float v;
            asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
            return v;
        };
        // The score buffers start at MAGIC_BITS, so what comes back from tensor memory is already a float (common.cuh).
        uint32_t magic[FILL_BLOCK];
        fill_block_init(magic, MAGIC_BITS);
        tmem_fill<KEY_TILE>(t_s + parity * 64, magic);
        tmem_fill<KEY_TILE>(t_s + (parity + 2) * 64, magic);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&sm.s_ready);
        float sk_reg = parity < k_tiles ? load_scale(sk + parity) : 0.0f;

        TRACE_DECL(row == 0);
        // One key tile: scores -> P^ bytes in shared memory, (tile maximum, row sum) -> the flush threads.
        auto softmax_tile = [&](auto masked_c, int t, float c, int buf, int stage, int kv_phase, int record) -> bool {
            constexpr bool MASKED = decltype(masked_c)::value;
            const int valid = MASKED ? n_keys - t * KEY_TILE : KEY_TILE;
            const uint32_t ts = t_s + buf * 64;
            TRACE(7);
            // Per token: the keys' scales came with the V tile.  That tile has long landed when its scores are there (the
            // scores were issued after it), so the barrier is only looked at, and the look is started before the wait for
            // the scores so that its latency hides behind that.
            const bool scales_there = !V_TOKEN || mbar_try(&sm.kv_full[stage], kv_phase);
            if (FLAG_WAITS ? !flag_wait_warp(&sm.s_done[buf], t + 1, abort_flag, status, STATUS_WAIT_SCORES)
                           : !mbar_wait_warp<0>(&sm.s_full[buf], (t / S_RING) & 1, abort_flag, status, STATUS_WAIT_SCORES))
                return false;
            TRACE(0);
            EVENT(0, t);
            if (V_TOKEN && !__all_sync(0xffffffffu, scales_there) && !mbar_wait_warp(&sm.kv_full[stage], kv_phase, abort_flag, status, STATUS_WAIT_TILE))
                return false;
            tc_fence_after();
#if defined(UNICA_STUB) && (UNICA_STUB & 1)  // measurement only: the protocol without the arithmetic (results are wrong)
            sm.st[record][row] = make_float2(0.0f, 1.0f);
            tc_fence_before();
            fence_proxy_async();
            mbar_arrive(&sm.soft_done[record]);
            return true;
#endif
            const float2 c2 = make_float2(c, c), minus_magic = make_float2(-MAGIC, -MAGIC), plus_magic = make_float2(MAGIC, MAGIC);
            const float4* log_s4 = reinterpret_cast<const float4*>(sm.tok[stage]);
            const float4* inv_s4 = reinterpret_cast<const float4*>(sm.tok[stage] + KEY_TILE);
            uint8_t* p_row = sm.p[stage] + row * 16;  // the P^ ring runs with the stages
            // The row's 64 scores, read once and kept in registers; the buffer goes back to its start value for S(t + 4)
            // at once (the stores run while the arithmetic does; they are waited for at the hand-over).
            float2 x[KEY_TILE / 16][8];
            tmem_ld64_sync(ts, reinterpret_cast<float2(&)[KEY_TILE / 2]>(x));
            tmem_fill<KEY_TILE>(ts, magic);
            float top[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int step = 0; step < KEY_TILE / 16; ++step) {
                float2(&y)[8] = x[step];
                if (V_TOKEN) {  // log2 s_j joins the scores before the maximum
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        const float4 l = log_s4[step * 4 + j / 2];
                        y[j] = fma2(add2(y[j], minus_magic), c2, make_float2(l.x, l.y));
                        y[j + 1] = fma2(add2(y[j + 1], minus_magic), c2, make_float2(l.z, l.w));
                    }
                }
                if (MASKED) {  // keys past the end: below every real score (|score| < 2^21)
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (step * 16 + j >= valid) (j % 2 ? y[j / 2].y : y[j / 2].x) = V_TOKEN ? -INFINITY : MAGIC - 4194303.0f;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) top[j % 4] = max3(top[j % 4], y[j].x, y[j].y);
            }
            float tile_max = fmaxf(fmaxf(top[0], top[1]), fmaxf(top[2], top[3]));
            TRACE(1);
            if (!V_TOKEN) tile_max = (tile_max - MAGIC) * c;
            // P^ = rint(255 * 2^(score * c - tile max)).  Per channel the float read back is MAGIC + score, so the exponent is
            // x * c + (offset - MAGIC * c) in ONE fused multiply-add; what the rounding of that constant loses (it is about
            // 2^11 in size) is put back exactly: `low` is the lost part, and the product p * 2^low happens inside the
            // multiply-add that rounds p to a byte.
            const float offset = LOG2_255 - tile_max;
            float2 base2 = make_float2(offset, offset), k2 = make_float2(1.0f, 1.0f);
            if (!V_TOKEN) {
                const float a_hi = __fmul_rn(-MAGIC, c), a_lo = __fmaf_rn(-MAGIC, c, -a_hi);  // -MAGIC * c = a_hi + a_lo exactly
                const float sum = __fadd_rn(a_hi, offset), bb = __fsub_rn(sum, a_hi);
                const float low = __fadd_rn(__fadd_rn(__fsub_rn(a_hi, __fsub_rn(sum, bb)), __fsub_rn(offset, bb)), a_lo);  // a_hi + offset = sum + ..
                const float k = __fmaf_rn(low, 0.693147181f, 1.0f);  // 2^low, |low| < 2^-12
                base2 = make_float2(sum, sum), k2 = make_float2(k, k);
            }
            unsigned isum[2] = {0, 0};
            float2 fsum = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int step = 0; step < KEY_TILE / 16; ++step) {
                // Sixteen keys, written stage by stage (exponents, exponentials, rounding, packing) so that every
                // instruction has fifteen independent ones around it: the exponential unit takes a warp every 8 cycles
                // and answers after some twenty, and a thread that asks for one result at a time waits for each.
                float2(&y)[8] = x[step];
                float2 e[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) e[j] = V_TOKEN ? add2(y[j], base2) : fma2(y[j], c2, base2);
#pragma unroll
                for (int j = 0; j < 8; ++j) e[j] = make_float2(ex2(e[j].x), ex2(e[j].y));
                if (V_TOKEN) {  // the denominator sums p / s_j before rounding
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        const float4 r = inv_s4[step * 4 + j / 2];
                        fsum = fma2(e[j], make_float2(r.x, r.y), fsum);
                        fsum = fma2(e[j + 1], make_float2(r.z, r.w), fsum);
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) e[j] = V_TOKEN ? add2(e[j], plus_magic) : fma2(e[j], k2, plus_magic);  // the low byte of each is rint(p)
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t lo = __byte_perm(__float_as_uint(e[2 * i].x), __float_as_uint(e[2 * i].y), 0x0040);
                    const uint32_t hi = __byte_perm(__float_as_uint(e[2 * i + 1].x), __float_as_uint(e[2 * i + 1].y), 0x0040);
                    w[i] = __byte_perm(lo, hi, 0x5410);
                    if (!V_TOKEN && MASKED) {  // keys past the end weigh nothing
                        const int left = valid - (step * 16 + i * 4);
                        w[i] = left >= 4 ? w[i] : left <= 0 ? 0u : (w[i] & ((1u << (8 * left)) - 1u));
                    }
                    if (!V_TOKEN) isum[i % 2] = __dp4a(w[i], 0x01010101u, isum[i % 2]);
                }
                *reinterpret_cast<uint4*>(p_row + step * (QUERY_TILE * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            TRACE(2);
            sm.st[record][row] = make_float2(tile_max, V_TOKEN ? fsum.x + fsum.y : __uint2float_rn(isum[0] + isum[1]));
            tmem_wait_st();
            tc_fence_before();
            fence_proxy_async();
            mbar_arrive(&sm.soft_done[record]);  // P^(t) and its record delivered, the scores buffer back at its start value
            TRACE(3);
            EVENT(1, t);
            return true;
        };

        bool ok = true;
        // this warpgroup's tiles advance by two: ring positions and barrier phases are kept as counters
        int buf = parity, stage = parity, kv_phase = 0, record = parity;
        for (int t = parity; ok && t < k_tiles; t += 2) {
            const float c = (sq * sk_reg) * scale_log2;
            if (t + 2 < k_tiles) sk_reg = load_scale(sk + t + 2);
            ok = ragged && t + 1 == k_tiles ? softmax_tile(std::true_type{}, t, c, buf, stage, kv_phase, record)
                                            : softmax_tile(std::false_type{}, t, c, buf, stage, kv_phase, record);
            buf ^= 2;
            stage += 2;
            if (stage >= STAGES) stage -= STAGES, kv_phase ^= 1;
            record = (record + 2) % ST_RING;
        }
        TRACE_END(parity);
    } else {
        // ------------------------------------------------------------------------------------------------ flush
        set_registers<FLUSH_REGISTERS>();
        const uint32_t t_acc = tmem + lane_base + COL_ACC;
        float m = -INFINITY, den = 0.0f;
        float2 o[HEAD_DIM / 2];
#pragma unroll
        for (int i = 0; i < HEAD_DIM / 2; ++i) o[i] = make_float2(0.0f, 0.0f);

        bool ok = true;
        TRACE_DECL(row == 0);
        for (int t = 0; ok && t < k_tiles; ++t) {
            const int b = t & 1;
            TRACE(7);
            // P.V(t) was issued after the softmax of tile t had delivered its record, so the record is there too
            if (FLAG_WAITS ? !flag_wait_warp(&sm.acc_done[b], t + 1, abort_flag, status, STATUS_WAIT_PV)
                           : !mbar_wait_warp<0>(&sm.kv_empty[t % STAGES], (t / STAGES) & 1, abort_flag, status, STATUS_WAIT_PV)) {
                ok = false;
                break;
            }
            tc_fence_after();
            // 32 channels per load, three loads out at once and the fourth as soon as the first values are used: the
            // accumulator is handed back a few hundred cycles after it was seen, long before the arithmetic is done
            float2 a[3][16];
            tmem_ld32_async(t_acc + b * 128, a[0]);
            tmem_ld32_async(t_acc + b * 128 + 32, a[1]);
            tmem_ld32_async(t_acc + b * 128 + 64, a[2]);
            TRACE(1);
            EVENT(3, t);
#if defined(UNICA_STUB) && (UNICA_STUB & 2)  // measurement only
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(&sm.acc_free[b]);
            continue;
#endif
            const float2 record = sm.st[t % ST_RING][row];  // tile maximum, row sum
            float alpha, beta;
            reference_step(m, record.x, alpha, beta);
            den = den * alpha + record.y * beta;
            const bool rescale = !__all_sync(0xffffffffu, alpha == 1.0f);
            tmem_wait_ld();
            reg_fence16(a[0]);
            reg_fence16(a[1]);
            reg_fence16(a[2]);
            flush32(a[0], o, alpha, beta, rescale);
            reg_fence16(a[0]);
            tmem_ld32_async(t_acc + b * 128 + 96, a[0]);
            tmem_wait_ld();
            reg_fence16(a[0]);
            tc_fence_before();
            mbar_arrive(&sm.acc_free[b]);  // the accumulator has been read: P.V(t + 2) may overwrite it
            EVENT(4, t);
            flush32(a[1], o + 16, alpha, beta, rescale);
            flush32(a[2], o + 32, alpha, beta, rescale);
            flush32(a[0], o + 48, alpha, beta, rescale);
            TRACE(3);
            EVENT(5, t);
        }
        TRACE_END(2);

        if constexpr (OUTLIERS) {
            // The outlier keys were zeros in V8: their exact share p * v / v_scale, with p = 255 * 2^(score - final max),
            // from this row's Q^ (still in shared memory) and the key's K^ row and scale (csrc/flash.cu:748-790).
            // The keys' K^ rows and V rows are the same for all 128 rows: the flush warps bring them into two P^ slots
            // that nobody uses any more (sixteen outliers at a time) and meet at a barrier of their own, which every
            // flush warp reaches whatever happened to it.
            if (ok) ok = mbar_wait_warp(&sm.q_full, 0, abort_flag, status, STATUS_WAIT_TILE);
            static_assert(P_RING >= 6 && OUTLIER_BATCH * HEAD_DIM * 4 <= P_BYTES, "two spare P^ slots hold a batch of outlier rows");
            float* rows_s = reinterpret_cast<float*>(sm.p[4]);                            // [OUTLIER_BATCH][128]
            uint4* k_rows_s = reinterpret_cast<uint4*>(sm.p[5]);                          // [OUTLIER_BATCH][8]: the key's 128 codes
            int* keys_s = reinterpret_cast<int*>(sm.p[5] + OUTLIER_BATCH * HEAD_DIM);     // [OUTLIER_BATCH], -1: no such key
            const int mine = threadIdx.x - FLUSH_WARP * 32;
            const float sq = q_scale[size_t(head) * q_tiles + q_tile];
            const float* sk = k_scale + size_t(head) * k_tiles;
            const uint4* q_row8 = reinterpret_cast<const uint4*>(sm.q + row * 16);  // chunk c: QUERY_TILE uint4 further
            for (int i0 = 0; i0 < n_outliers; i0 += OUTLIER_BATCH) {
                const int n = min(OUTLIER_BATCH, n_outliers - i0);
                asm volatile("bar.sync 1, 128;" ::: "memory");  // the batch before has been used
                for (int item = mine; item < n * (HEAD_DIM / 4); item += 128)
                    reinterpret_cast<float4*>(rows_s)[item] =
                        reinterpret_cast<const float4*>(outlier_rows + (size_t(head) * n_outliers + i0) * HEAD_DIM)[item];
                for (int item = mine; item < n * (HEAD_DIM / 16); item += 128) {
                    const int i = item / (HEAD_DIM / 16), c = item % (HEAD_DIM / 16);
                    const int key = outlier_keys[size_t(head) * n_outliers + i0 + i];
                    const bool there = key >= 0 && key < n_keys;
                    k_rows_s[item] = there ? reinterpret_cast<const uint4*>(k8 + (size_t(head) * k_tiles + key / KEY_TILE) * K_BYTES + (key % KEY_TILE) * 16)[c * KEY_TILE]
                                           : make_uint4(0, 0, 0, 0);
                    if (c == 0) keys_s[i] = there ? key : -1;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (!ok) continue;
                for (int i = 0; i < n; ++i) {
                    const int key = keys_s[i];
                    if (key < 0) continue;
                    int dot = 0;
#pragma unroll
                    for (int c = 0; c < HEAD_DIM / 16; ++c) {
                        const uint4 qv = q_row8[c * QUERY_TILE], kv = k_rows_s[i * (HEAD_DIM / 16) + c];
                        dot = __dp4a(int(qv.x), int(kv.x), dot);
                        dot = __dp4a(int(qv.y), int(kv.y), dot);
                        dot = __dp4a(int(qv.z), int(kv.z), dot);
                        dot = __dp4a(int(qv.w), int(kv.w), dot);
                    }
                    const float p = ex2(__int2float_rn(dot) * ((sq * sk[key / KEY_TILE]) * scale_log2) - m) * 255.0f;
                    const float2 p2 = make_float2(p, p);
                    const float2* v_row = reinterpret_cast<const float2*>(rows_s + i * HEAD_DIM);
#pragma unroll
                    for (int j = 0; j < HEAD_DIM / 2; ++j) o[j] = fma2(p2, v_row[j], o[j]);
                }
            }
        }

        // Out through shared memory (stage_piece / store_staged_rows).  The warp's 32 rows take one P^ slot: the last
        // P.V, which the loop above has seen complete, was its last reader.
        if (__all_sync(0xffffffffu, ok)) {
            const int lane = threadIdx.x % 32;
            uint8_t* staged = sm.p[warp - FLUSH_WARP];
            const float inv = 1.0f / den;
            const float* vs = v_scale + head * HEAD_DIM;
#pragma unroll
            for (int chunk = 0; chunk < HEAD_DIM / 8; ++chunk) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c0 = chunk * 8 + 2 * i;
                    const float2 v = o[chunk * 4 + i];
                    w[i] = output_pair(v.x * vs[c0] * inv, v.y * vs[c0 + 1] * inv, out_layout.half);
                }
                stage_piece(staged, lane, chunk, make_uint4(w[0], w[1], w[2], w[3]));
            }
            __syncwarp();
            store_staged_rows(staged, lane, q_tile * QUERY_TILE + (warp - FLUSH_WARP) * 32, n_queries, head, out, out_layout, peers);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == SERVICE_WARP) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLUMNS);
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Self-test: one tcgen05.mma chain on operand images given by the caller, accumulator copied out as it lies in tensor memory.

__global__ void __launch_bounds__(128) selftest_mma_i8_kernel(const uint8_t* __restrict__ a_image, const uint8_t* __restrict__ b_image,
                                                              int n, int k, int a_unsigned, int32_t* __restrict__ d, int* status) {
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
        for (int ks = 0; ks < k / 32; ++ks) {
            const uint64_t a_desc = smem_desc(smem_u32(a_s) + ks * 2 * 128 * 16, 128 * 16, 128), b_desc = smem_desc(smem_u32(b_s) + ks * 2 * n * 16, n * 16, 128);
            if (a_unsigned == 2)  // kind::tf32: the images hold floats, k / 4 per row; an instruction takes 8 = 32 bytes of a row
                mma_tf32_ss(tmem, a_desc, b_desc, idesc_tf32(128, n), ks > 0);
            else
                mma_i8_ss(tmem, a_desc, b_desc, idesc_i8(!a_unsigned, 128, n), ks > 0);
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

static int attention_int8(const int8_t* q8, const float* q_scale, const int8_t* k8, const float* k_scale, const int8_t* v8,
                          const float* v_scale, const float* v_token, int v_mode, const int* outlier_keys, const float* outlier_rows,
                          int n_outliers, void* out, void* const* peer_out, int n_peers, unica_token_layout out_layout, int heads,
                          int n_queries, int n_keys, float scale_log2, int* status, void* stream) {
    if (!q8 || !q_scale || !k8 || !k_scale || !v8 || !v_scale || !out) return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_int8: null pointer");
    if (heads <= 0 || heads > 65535 || n_queries <= 0 || n_keys <= 0)
        return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_int8: heads must be in 1..65535, n_queries and n_keys positive");
    if (v_mode != UNICA_B200_V_CHANNEL && v_mode != UNICA_B200_V_TOKEN && v_mode != UNICA_B200_V_OUTLIERS)
        return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_int8: unknown v_mode");
    if (v_mode == UNICA_B200_V_OUTLIERS && (!outlier_keys || !outlier_rows || n_outliers < 1 || n_outliers > 8))
        return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_int8: the outliers mode needs outlier_keys, outlier_rows and 1..8 outliers");
    if (v_mode == UNICA_B200_V_TOKEN && !v_token) return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_int8: per-token mode needs v_token");
    PeerOutputs peers = {};
    if (int e = unica_peer_outputs(out, peer_out, n_peers, &peers)) return e;
    if (int e = unica_check_device()) return e;
    const dim3 grid((n_queries + 2 * QUERY_TILE - 1) / (2 * QUERY_TILE) * 2, heads);  // Q8 holds an even number of tiles
    const size_t smem = sizeof(AttSmem) + 128;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    auto launch = [&](auto kernel, int instance) -> int {
        // Set up once per kernel instance and device: the shared-memory size, and a check that the build holds the
        // registers its setmaxnreg split needs (setmaxnreg only moves registers the block already has: asking for more
        // than the launch gives would make the flush warps wait for ever).
        constexpr int MAX_DEVICES = 64;
        static std::atomic<signed char> done[3][MAX_DEVICES];  // the three instances share this lambda's one instantiation
        std::atomic<signed char>* ready = done[instance];
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess) return unica_check_launch("attention_int8 (device)");
        if (device >= MAX_DEVICES || ready[device].load(std::memory_order_acquire) == 0) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess ||
                cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess)
                return unica_check_launch("attention_int8 (shared memory size)");
            cudaFuncAttributes attributes;
            if (cudaFuncGetAttributes(&attributes, kernel) != cudaSuccess) return unica_check_launch("attention_int8 (attributes)");
            if (attributes.numRegs * ATT_THREADS < 128 * (2 * SOFTMAX_REGISTERS + FLUSH_REGISTERS + SERVICE_REGISTERS))
                return unica_fail(UNICA_B200_ERR_KERNEL, "attention_int8: this build holds fewer registers per block than its setmaxnreg split needs");
            if (device < MAX_DEVICES) ready[device].store(1, std::memory_order_release);
        }
        kernel<<<grid, ATT_THREADS, smem, s>>>(q8, q_scale, k8, k_scale, v8, v_scale, v_token, outlier_keys, outlier_rows, n_outliers,
                                               static_cast<__nv_bfloat16*>(out), to_layout(out_layout), peers, n_queries, n_keys,
                                               scale_log2, status);
        return unica_check_launch("attention_int8");
    };
    return v_mode == UNICA_B200_V_TOKEN      ? launch(attention_int8_kernel<true, false>, 1)
           : v_mode == UNICA_B200_V_OUTLIERS ? launch(attention_int8_kernel<false, true>, 2)
                                             : launch(attention_int8_kernel<false, false>, 0);
}

extern "C" int unica_b200_attention_int8(const int8_t* q8, const float* q_scale, const int8_t* k8, const float* k_scale,
                                         const int8_t* v8, const float* v_scale, const float* v_token, int v_mode,
                                         const int* outlier_keys, const float* outlier_rows, int n_outliers, void* out,
                                         unica_token_layout out_layout, int heads, int n_queries, int n_keys, float scale_log2,
                                         int* status, void* stream) {
    return attention_int8(q8, q_scale, k8, k_scale, v8, v_scale, v_token, v_mode, outlier_keys, outlier_rows, n_outliers, out, nullptr, 0,
                          out_layout, heads, n_queries, n_keys, scale_log2, status, stream);
}

extern "C" int unica_b200_attention_int8_peers(const int8_t* q8, const float* q_scale, const int8_t* k8, const float* k_scale,
                                               const int8_t* v8, const float* v_scale, const float* v_token, int v_mode,
                                               const int* outlier_keys, const float* outlier_rows, int n_outliers, void* out,
                                               void* const* peer_out, int n_peers, unica_token_layout out_layout, int heads,
                                               int n_queries, int n_keys, float scale_log2, int* status, void* stream) {
    return attention_int8(q8, q_scale, k8, k_scale, v8, v_scale, v_token, v_mode, outlier_keys, outlier_rows, n_outliers, out, peer_out,
                          n_peers, out_layout, heads, n_queries, n_keys, scale_log2, status, stream);
}

#ifdef UNICA_TRACE
// Trace builds only: copies the per-phase cycle totals of block (0, 0) to `host_out` (5 x 8 long long) and clears them.
extern "C" int unica_b200_trace_events(long long* host_out) {  // 8 kinds x 16 tiles
    if (cudaMemcpyFromSymbol(host_out, g_events, sizeof(long long) * 128) != cudaSuccess) return unica_check_launch("trace_events");
    return UNICA_B200_OK;
}
extern "C" int unica_b200_trace_read(long long* host_out) {
    if (cudaMemcpyFromSymbol(host_out, g_trace, sizeof(long long) * 40) != cudaSuccess) return unica_check_launch("trace_read");
    static const long long zeros[40] = {};
    if (cudaMemcpyToSymbol(g_trace, zeros, sizeof zeros) != cudaSuccess) return unica_check_launch("trace_read");
    return UNICA_B200_OK;
}
#endif


extern "C" int unica_b200_selftest_mma_i8(const void* a_image, const void* b_image, int n, int k, int a_unsigned, int variant,
                                          int32_t* d, void* stream) {
    if (!a_image || !b_image || !d) return unica_fail(UNICA_B200_ERR_ARGUMENT, "selftest_mma_i8: null pointer");
    if (n < 32 || n > 128 || n % 32 || k < 32 || k > 128 || k % 32)
        return unica_fail(UNICA_B200_ERR_ARGUMENT, "selftest_mma_i8: n and k must be multiples of 32 in 32..128");
    if (variant != 0) return unica_fail(UNICA_B200_ERR_ARGUMENT, "selftest_mma_i8: variant must be 0");
    if (int e = unica_check_device()) return e;
    const size_t smem = size_t(128 + n) * k + 128;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int* status = nullptr;
    if (cudaMalloc(&status, sizeof(int)) != cudaSuccess || cudaMemsetAsync(status, 0, sizeof(int), s) != cudaSuccess) {
        const int e = unica_check_launch("selftest_mma_i8 (status word)");
        cudaFree(status);  // a no-op when the allocation itself failed
        return e;
    }
    selftest_mma_i8_kernel<<<1, 128, smem, s>>>(static_cast<const uint8_t*>(a_image), static_cast<const uint8_t*>(b_image), n, k,
                                                a_unsigned, d, status);
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
