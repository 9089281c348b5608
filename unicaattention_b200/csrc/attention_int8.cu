// The accurate mode's flash-attention loop on tcgen05 (replaces the reference's attention_int8pv_tma, csrc/flash.cu:806-959).
//
// One block = TILES tiles of 128 query rows of one head, each owned by one warpgroup of 4 warps in which a thread owns
// one query row (tensor-memory lane = row, so row maxima and sums need no shuffles) and keeps that row's 128 output
// channels in registers.  TILES = 1 (the default): 256 threads, two blocks per SM, which run out of step and fill each
// other's waits; TILES = 2: 384 threads, one block per SM whose two tiles share every K and V tile (half the traffic
// from L2, a few per cent slower).  The last warpgroup of a block holds the producer warp, which streams K8 / V8 tiles
// (contiguous 8 KB images written by the quantizers) into a ring of shared-memory stages with bulk TMA copies, and one
// MMA warp per query tile, one elected thread of which issues that tile's tcgen05.mma:
//
//   S[g]   = Q8[g] . K8(t)^T      kind::i8 s8 x s8 -> s32, 128 x 64, 4 instructions of K = 32, double-buffered in tensor memory
//   acc[g] = P^[g](t) . V8(t)     kind::i8 u8 x s8 -> s32, 128 x 128, 2 instructions of K = 32, one accumulator per tile
//
// The loop runs in steps: step t turns the scores of key tile t into P^ and, in the same straight run of instructions,
// flushes the accumulator of tile t - 1 into the row's outputs (see tile_step below); one arrival per step tells the
// issuing thread that P^(t) is delivered, a scores buffer empty and the accumulator read.
//
// Numerics (bench/emulate.py:298-369 with the accurate contract): scores in the log2 domain, c = (q_scale * k_scale) *
// log2(e) / sqrt(d); P^ = rint(255 * 2^(x - tile max)) as u8 against the tile's own maximum; the denominator sums the
// rounded P^ (per channel) or p / s_j in float before rounding (per token); every tile is flushed as
// out = out * alpha + beta * float(acc) with beta = 2^(m_tile - m) and alpha = 2^(m_old - m_new), where m is a reference
// exponent that follows the running maximum only in large steps (the common factor cancels against the denominator's).
// The 255 stays in numerator and denominator alike (as csrc/flash.cu:409-414 does).
//
// What bounds it (measured on B200 with the micro-benchmarks of peak.cu): ex2 issues once per 8 cycles per scheduler,
// float -> int conversions too, so rounding goes through the float bias MAGIC (common.cuh) instead; int -> float runs on
// the ALU pipe at 2 cycles; a tensor-memory load costs ~180 cycles of latency and a barrier probe as much, so loads are
// issued a step ahead and a step has one wait.
//
// Tensor memory: 256 columns per query tile = S x 2 (64 each) + acc (128).  All waits are bounded (common.cuh).
#include <type_traits>

#include "capi.h"

namespace unica {

#ifndef UNICA_TILES
#define UNICA_TILES 1
#endif
constexpr int TILES = UNICA_TILES;  // query tiles of 128 rows per block: 2 (one block per SM), or 1 (two blocks per SM)
constexpr int ATT_THREADS = (4 * TILES + 4) * 32;  // a warpgroup per query tile + one holding the producer and MMA warps
// registers move from the service warpgroup to those that hold `out`: 256 x 232 + 128 x 40 = 384 x 168, 128 x 224 + 128 x 32 = 256 x 128
constexpr int COMPUTE_REGISTERS = TILES == 2 ? 232 : 224, SERVICE_REGISTERS = TILES == 2 ? 40 : 32;
constexpr int PRODUCER_WARP = 4 * TILES, MMA_WARP = PRODUCER_WARP + 1;
constexpr int STAGES = 3;
constexpr int Q_BYTES = QUERY_TILE * HEAD_DIM;  // 16384
constexpr int K_BYTES = KEY_TILE * HEAD_DIM;    // 8192
constexpr int V_BYTES = KEY_TILE * HEAD_DIM;    // 8192
constexpr int TOK_BYTES = 2 * KEY_TILE * 4;     // 512
constexpr int P_BYTES = QUERY_TILE * KEY_TILE;  // 8192
constexpr int TMEM_COLUMNS = 256 * TILES;
constexpr float REFERENCE_SLACK = 60.0f;  // log2: how far a tile maximum may rise above a row's reference exponent
constexpr int COL_S = 0, COL_ACC = 128;  // inside a query tile's 256 columns: S buffers at 0 and 64, acc at 128

struct __align__(128) AttSmem {
    int8_t q[TILES][Q_BYTES];
    int8_t k[STAGES][K_BYTES];
    int8_t v[STAGES][V_BYTES];
    float tok[STAGES][2 * KEY_TILE];
    uint8_t p[TILES][2][P_BYTES];
    uint64_t q_full, k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
    uint64_t s_full[TILES][2], s_free[TILES][2], acc_full[TILES], step_done[TILES], drain[TILES];
    uint32_t tmem_base;
    int abort_flag;
};

// -DUNICA_TRACE: the first thread of each warpgroup of block (0, 0) adds up the cycles it spends in each phase of the
// tile loop (the reference has a TRACE build for the same purpose: csrc/legacy.cu, bench/timeline.py).  The totals
// stay in registers until the end, so tracing itself costs a clock read per phase.
#ifdef UNICA_TRACE
__device__ long long g_trace[4][8];
#define TRACE_DECL long long trace_t0 = clock64(), trace_sum[8] = {}; const bool tracing = blockIdx.x == 0 && blockIdx.y == 0 && row == 0
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
#define TRACE_DECL
#define TRACE(phase)
#define TRACE_END(slot)
#endif
enum { TR_WAIT_S = 0, TR_LOAD_S = 1, TR_SOFTMAX = 2, TR_STORE_P = 3, TR_WAIT_PV = 4, TR_FLUSH = 5, TR_OTHER = 6 };

constexpr uint32_t IDESC_QK = idesc_i8(true, QUERY_TILE, KEY_TILE);
constexpr uint32_t IDESC_PV = idesc_i8(false, QUERY_TILE, HEAD_DIM);

template <bool V_TOKEN, bool OUTLIERS>
__global__ void __launch_bounds__(ATT_THREADS, 3 - TILES)
    attention_int8_kernel(const int8_t* __restrict__ q8, const float* __restrict__ q_scale, const int8_t* __restrict__ k8,
                          const float* __restrict__ k_scale, const int8_t* __restrict__ v8, const float* __restrict__ v_scale,
                          const float* __restrict__ v_token, const int* __restrict__ outlier_keys,
                          const float* __restrict__ outlier_rows, int n_outliers, __nv_bfloat16* __restrict__ out,
                          TokenLayout out_layout, int n_queries, int n_keys, float scale_log2, int* status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    AttSmem& sm = *reinterpret_cast<AttSmem*>(smem_raw);
    const int warp = threadIdx.x / 32;
    const int head = blockIdx.y;
    const int q_tiles = TILES * gridDim.x;  // allocated Q tiles per head (even)
    if (TILES == 1 && blockIdx.x * QUERY_TILE >= n_queries) return;  // the padding tile of an odd count: nothing to do
    const int k_tiles = (n_keys + KEY_TILE - 1) / KEY_TILE;
    volatile int* abort_flag = &sm.abort_flag;

    if (threadIdx.x == 0) {
        sm.abort_flag = 0;
        mbar_init(&sm.q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&sm.k_full[s], 1);
            mbar_init(&sm.k_empty[s], TILES);  // every query tile's MMA thread commits to it
            mbar_init(&sm.v_full[s], 1);
            mbar_init(&sm.v_empty[s], TILES);
        }
        for (int g = 0; g < TILES; ++g) {
            for (int b = 0; b < 2; ++b) {
                mbar_init(&sm.s_full[g][b], 1);
                mbar_init(&sm.s_free[g][b], 128);
            }
            mbar_init(&sm.acc_full[g], 1);
            mbar_init(&sm.step_done[g], 128);
        }
        for (int g = 0; g < TILES; ++g) mbar_init(&sm.drain[g], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) tmem_alloc(&sm.tmem_base, TMEM_COLUMNS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    if (warp >= PRODUCER_WARP) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(SERVICE_REGISTERS));
      if (warp == PRODUCER_WARP) {
        // ------------------------------------------------------------------------------------------------ producer
        if (elect_one()) {  // one elected lane of a converged warp: see elect_one() in common.cuh
            const int8_t* q_src = q8 + (size_t(head) * q_tiles + TILES * blockIdx.x) * Q_BYTES;
            mbar_expect_tx(&sm.q_full, TILES * Q_BYTES);
            for (int g = 0; g < TILES; ++g) bulk_load(sm.q[g], q_src + g * Q_BYTES, Q_BYTES, &sm.q_full);
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
            }
            if (*abort_flag) {  // let the copies still in flight land before the block's shared memory goes away
                int never = 0;
                for (int t = max(0, issued - STAGES); t < issued; ++t)
                    mbar_wait(&sm.k_full[t % STAGES], (t / STAGES) & 1, &never, nullptr, 0);
                mbar_wait(&sm.q_full, 0, &never, nullptr, 0);
            }
        }
      } else if (warp >= MMA_WARP && warp < MMA_WARP + TILES) {
        // ------------------------------------------------------------------------------------------------ MMA issue
        // One elected thread per query tile issues that tile's tcgen05.mma in the order
        // its operands become ready: P.V of key tile t once P^(t) is written, V(t) has landed and the flush of tile t - 1
        // has read the accumulator; then the scores of tile t + 2 into the buffer the softmax of tile t has emptied.
        // Each wait blocks in hardware (mbarrier.try_wait) and wakes as the phase completes; a stage of K or V is
        // released by the last of the tiles' commits.
        if (elect_one()) {  // one elected lane of a converged warp: see elect_one() in common.cuh
            const int g = warp - MMA_WARP;
            const uint32_t q_addr = smem_u32(sm.q[g]), base = tmem + g * 256;
            // Per channel / outliers: a query tile's threads end every step with ONE arrival (step_done): step t holds
            // the softmax of key tile t and the flush of tile t - 1, so its end frees the accumulator, delivers P^(t) and
            // empties a scores buffer at once, and P.V(t) and the scores of tile t + 2 go out back to back after a single
            // wake-up.  Per token the softmax and the flush end at different times and keep a barrier each.
            auto scores = [&](int n) -> bool {
                const int stage = n % STAGES, buf = n & 1;
                if (!mbar_wait(&sm.k_full[stage], (n / STAGES) & 1, abort_flag, status, STATUS_WAIT_TILE)) return false;
                if (n < 2 && !mbar_wait(&sm.s_free[g][buf], (n >> 1) & 1, abort_flag, status, STATUS_WAIT_FREE)) return false;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(sm.k[stage]);
#pragma unroll
                for (int ks = 0; ks < HEAD_DIM / 32; ++ks)
                    mma_i8_ss(base + COL_S + buf * 64, smem_desc(q_addr + ks * 2 * QUERY_TILE * 16, QUERY_TILE * 16, 128),
                              smem_desc(k_addr + ks * 2 * KEY_TILE * 16, KEY_TILE * 16, 128), IDESC_QK, true);
                mma_commit(&sm.s_full[g][buf]);
                mma_commit(&sm.k_empty[stage]);
                return true;
            };
            bool ok = mbar_wait(&sm.q_full, 0, abort_flag, status, STATUS_WAIT_TILE);
            for (int n = 0; ok && n < min(2, k_tiles); ++n) ok = scores(n);
            for (int t = 0; ok && t < k_tiles; ++t) {
                const int stage = t % STAGES, buf = t & 1;
                ok = mbar_wait(&sm.v_full[stage], (t / STAGES) & 1, abort_flag, status, STATUS_WAIT_TILE);
                // K(t + 2) has long landed: probing it before the step's end keeps that probe off the critical path
                if (t + 2 < k_tiles) ok = ok && mbar_wait(&sm.k_full[(t + 2) % STAGES], ((t + 2) / STAGES) & 1, abort_flag, status, STATUS_WAIT_TILE);
                ok = ok && mbar_wait(&sm.step_done[g], t & 1, abort_flag, status, STATUS_WAIT_P);
                if (!ok) break;
                tc_fence_after();
                const uint32_t p_addr = smem_u32(sm.p[g][buf]), v_addr = smem_u32(sm.v[stage]);
#pragma unroll
                for (int ks = 0; ks < KEY_TILE / 32; ++ks)
                    mma_i8_ss(base + COL_ACC, smem_desc(p_addr + ks * 2 * QUERY_TILE * 16, QUERY_TILE * 16, 128),
                              smem_desc(v_addr + ks * 2 * HEAD_DIM * 16, HEAD_DIM * 16, 128), IDESC_PV, ks > 0);  // the first instruction of a tile overwrites the accumulator
                mma_commit(&sm.acc_full[g]);
                mma_commit(&sm.v_empty[stage]);
                if (t + 2 < k_tiles) ok = scores(t + 2);
            }
            if (!ok) {  // whatever was issued must finish before tensor memory is freed
                int never = 0;
                mma_commit(&sm.drain[g]);
                mbar_wait(&sm.drain[g], 0, &never, nullptr, 0);
            }
        }
      }
    } else {
        // ------------------------------------------------------------------------------------- softmax and flush
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(COMPUTE_REGISTERS));
        const int g = warp / 4, row = threadIdx.x % 128;
        const int q_tile = TILES * blockIdx.x + g, q_row = q_tile * QUERY_TILE + row;
        const uint32_t lane_base = uint32_t((warp % 4) * 32) << 16;
        const uint32_t t_scores = tmem + lane_base + g * 256 + COL_S, t_acc = tmem + lane_base + g * 256 + COL_ACC;
        const float sq = q_scale[size_t(head) * q_tiles + q_tile];
        const float* sk = k_scale + size_t(head) * k_tiles;
        const float2 minus_magic = make_float2(-MAGIC, -MAGIC), plus_magic = make_float2(MAGIC, MAGIC);
        float m = -INFINITY, den = 0.0f;
        // The K scale of the tile the next step takes, loaded a whole tile ahead of its use (volatile: the compiler
        // would otherwise sink the load to the use and expose its latency on every tile).
        auto load_scale = [](const float* p) {
            float v;
            asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
            return v;
        };
        float sk_reg = load_scale(sk);
        float2 o[HEAD_DIM / 2];
#pragma unroll
        for (int i = 0; i < HEAD_DIM / 2; ++i) o[i] = make_float2(0.0f, 0.0f);
        bool ok = true;
        TRACE_DECL;

        // The score buffers start at MAGIC_BITS, so what comes back from tensor memory is already a float (common.cuh).
        uint32_t magic[FILL_BLOCK];
        fill_block_init(magic, MAGIC_BITS);
        tmem_fill<128>(t_scores, magic);  // both score buffers
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&sm.s_free[g][0]);
        mbar_arrive(&sm.s_free[g][1]);

        {
            // One step of the loop: the scores of key tile `ts` become P^ in shared memory (SOFT) while the accumulator of
            // tile `tf` is flushed into `out` (FLUSH).  In the steady state both happen, interleaved 16 keys and 32 channels
            // at a time in one straight run of instructions, so that the exponentials (XU), the flush's multiply-adds (FMA
            // pipe) and the packing (ALU) overlap inside one warp, and one wait covers the tensor-memory loads of both.
            // Every choice is a template argument: a test inside the run would cut it into short basic blocks and leave
            // the latencies exposed.  alpha_s, beta_s: of tile ts, for its flush one step later.
            auto tile_step = [&](auto soft_c, auto flush_c, auto masked_c, auto rescale_c, int ts, int tf, float& alpha_s, float& beta_s,
                                 float alpha_f, float beta_f, bool last_of_step = true) -> bool {
                constexpr bool SOFT = decltype(soft_c)::value, FLUSH = decltype(flush_c)::value;
                constexpr bool MASKED = decltype(masked_c)::value, RESCALE = decltype(rescale_c)::value;
                const int buf = ts & 1, stage = SOFT ? ts % STAGES : 0;
                const int valid = min(KEY_TILE, n_keys - ts * KEY_TILE);
                float c = 0.0f, offset = 0.0f;
                TRACE(TR_OTHER);
                if (SOFT) {
                    c = (sq * sk_reg) * scale_log2;
                    if (ts + 1 < k_tiles) sk_reg = load_scale(sk + ts + 1);
                    // One wait serves both halves of a full step: the tile's issuing thread queued S(ts) before P.V(tf)
                    // (tf = ts - 1), tcgen05.mma of one thread complete in order, and a commit covers everything issued
                    // before it, so when the accumulator's barrier has flipped the scores are there too.
                    if (FLUSH ? !mbar_wait_warp(&sm.acc_full[g], tf & 1, abort_flag, status, STATUS_WAIT_PV)
                              : !mbar_wait_warp(&sm.s_full[g][buf], (ts >> 1) & 1, abort_flag, status, STATUS_WAIT_SCORES))
                        return false;
                    if (V_TOKEN && !mbar_wait_warp(&sm.v_full[stage], (ts / STAGES) & 1, abort_flag, status, STATUS_WAIT_TILE)) return false;
                    tc_fence_after();
                }
                TRACE(TR_WAIT_S);
#ifdef UNICA_TRACE
                if (tracing && ts >= 100 && ts < 108) g_trace[2 + g][ts - 100] = clock64();  // when the steps of tiles 100..107 began
#endif
                const float2 c2 = make_float2(c, c);
                const float4* log_s4 = reinterpret_cast<const float4*>(sm.tok[stage]);
                const float4* inv_s4 = reinterpret_cast<const float4*>(sm.tok[stage] + KEY_TILE);
                if (SOFT) {
                    // Pass 1: the tile maximum.  The 64 scores are not kept: the row's 128 output channels and the flush's
                    // accumulator values fill the register file, so pass 2 reads the scores again, 16 at a time.
                    float tile_max;
                    if (!V_TOKEN) {
                        float2 x[KEY_TILE / 2];  // MAGIC + score, exactly
                        tmem_ld64_sync(t_scores + buf * 64, x);
                        if (MASKED) {  // keys past the end: below every real score (|score| < 2^21)
#pragma unroll
                            for (int j = 0; j < KEY_TILE; ++j)
                                if (j >= valid) (j % 2 ? x[j / 2].y : x[j / 2].x) = MAGIC - 4194303.0f;
                        }
                        float top[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) top[i] = fmaxf(x[i].x, x[i].y);
#pragma unroll
                        for (int j = 4; j < KEY_TILE / 2; ++j) top[j % 4] = max3(top[j % 4], x[j].x, x[j].y);
                        tile_max = (fmaxf(fmaxf(top[0], top[1]), fmaxf(top[2], top[3])) - MAGIC) * c;
                    } else {  // log2 s_j joins the scores before the maximum; 32 keys at a time (registers)
                        float top[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                        for (int part = 0; part < 2; ++part) {
                            float2 x[KEY_TILE / 4];
                            tmem_ld32_async(t_scores + buf * 64 + part * 32, x);
                            tmem_wait_ld();
                            reg_fence16(x);
#pragma unroll
                            for (int j = 0; j < KEY_TILE / 4; j += 2) {  // 16-byte loads: the loop is short of load slots, not of bytes
                                const float4 l = log_s4[part * 8 + j / 2];
                                x[j] = fma2(add2(x[j], minus_magic), c2, make_float2(l.x, l.y));
                                x[j + 1] = fma2(add2(x[j + 1], minus_magic), c2, make_float2(l.z, l.w));
                            }
                            if (MASKED) {
#pragma unroll
                                for (int j = 0; j < KEY_TILE / 2; ++j)
                                    if (part * 32 + j >= valid) (j % 2 ? x[j / 2].y : x[j / 2].x) = -INFINITY;
                            }
#pragma unroll
                            for (int j = 0; j < KEY_TILE / 4; ++j) top[j % 4] = max3(top[j % 4], x[j].x, x[j].y);
                        }
                        tile_max = fmaxf(fmaxf(top[0], top[1]), fmaxf(top[2], top[3]));
                    }
                    // `m` is the exponent the row's sums are kept at, not the running maximum: out = sum over tiles of
                    // 2^(tile max - m) * acc, the same for the denominator, and the common factor cancels at the end.  The
                    // textbook form moves m to every new maximum and multiplies out and den by alpha = 2^(m_old - m_new)
                    // each time; here m moves only when a tile maximum is more than 2^REFERENCE_SLACK above it, so that
                    // multiplication (128 per row) all but disappears.  The difference is rounding only.
                    const bool first = m == -INFINITY;
                    const float m_new = tile_max > m + REFERENCE_SLACK ? tile_max : m;
                    alpha_s = first ? 1.0f : ex2(m - m_new);
                    beta_s = ex2(tile_max - m_new);
                    m = m_new;
                    offset = LOG2_255 - tile_max;
                }
                TRACE(TR_LOAD_S);
                if (FLUSH && !SOFT) {
                    if (!mbar_wait_warp(&sm.acc_full[g], tf & 1, abort_flag, status, STATUS_WAIT_PV)) return false;
                    tc_fence_after();
                }
                TRACE(TR_WAIT_PV);
                const float2 offset2 = make_float2(offset, offset), alpha2 = make_float2(alpha_f, alpha_f), beta2 = make_float2(beta_f, beta_f);
                uint8_t* p_row = sm.p[g][buf] + row * 16;
                unsigned isum[2] = {0, 0};
                float2 fsum = make_float2(0.0f, 0.0f);
                float2 x[2][8], a[2][8];  // 16 scores ahead; the 32 accumulator channels of the step
                if (SOFT) tmem_ld16_async(t_scores + buf * 64, x[0]);
                if (FLUSH) {
                    tmem_ld16_async(t_acc, a[0]);
                    tmem_ld16_async(t_acc + 16, a[1]);
                }
#pragma unroll
                for (int step = 0; step < KEY_TILE / 16; ++step) {
                    tmem_wait_ld();  // every load issued so far
                    if (SOFT) {
                        reg_fence8(x[step % 2]);
                        if (step + 1 < KEY_TILE / 16) tmem_ld16_async(t_scores + buf * 64 + (step + 1) * 16, x[(step + 1) % 2]);
                    }
                    // Per channel the accumulator values are converted at once and their registers go back to the next loads;
                    // per token (log2 s_j and 1 / s_j on top) the registers do not reach that far: the values are used where
                    // they are and the next loads follow the flush arithmetic, with the exponentials still ahead to cover them.
                    constexpr bool STAGED = !V_TOKEN;
                    float2 f[STAGED ? 16 : 1];
                    if (FLUSH) {
                        reg_fence8(a[0]);
                        reg_fence8(a[1]);
                        if (STAGED) {
#pragma unroll
                            for (int i = 0; i < 16; ++i)  // the accumulator is overwritten by every tile's P.V: plain integers
                                f[STAGED ? i : 0] = make_float2(__int2float_rn(__float_as_int(a[i / 8][i % 8].x)), __int2float_rn(__float_as_int(a[i / 8][i % 8].y)));
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                float2 v = o[step * 16 + i];
                                if (RESCALE) v = mul2(v, alpha2);
                                o[step * 16 + i] = fma2(beta2, make_float2(__int2float_rn(__float_as_int(a[i / 8][i % 8].x)), __int2float_rn(__float_as_int(a[i / 8][i % 8].y))), v);
                            }
                        }
                        if (step + 1 < KEY_TILE / 16) {
                            reg_fence8(a[0]);
                            reg_fence8(a[1]);
                            tmem_ld16_async(t_acc + (step + 1) * 32, a[0]);
                            tmem_ld16_async(t_acc + (step + 1) * 32 + 16, a[1]);
                        }
                    }
                    uint32_t w[4];
                    if (SOFT) {  // P^ = rint(255 * 2^(x - tile max)), keys 16 step .. 16 step + 15
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint32_t pair[2];
                            float4 l = make_float4(0.0f, 0.0f, 0.0f, 0.0f), r = l;  // log2 s and 1 / s of the four keys
                            if (V_TOKEN) l = log_s4[step * 4 + i], r = inv_s4[step * 4 + i];
#pragma unroll
                            for (int h = 0; h < 2; ++h) {  // a pair of keys
                                float2 e = fma2(add2(x[step % 2][i * 2 + h], minus_magic), c2, V_TOKEN ? (h ? make_float2(l.z, l.w) : make_float2(l.x, l.y)) : offset2);
                                if (V_TOKEN) e = add2(e, offset2);
                                const float2 p = make_float2(ex2(e.x), ex2(e.y));
                                if (V_TOKEN) fsum = fma2(p, h ? make_float2(r.z, r.w) : make_float2(r.x, r.y), fsum);
                                const float2 r = add2(p, plus_magic);  // the low byte of each is rint(p)
                                pair[h] = __byte_perm(__float_as_uint(r.x), __float_as_uint(r.y), 0x0040);
                            }
                            w[i] = __byte_perm(pair[0], pair[1], 0x5410);
                            if (!V_TOKEN && MASKED) {  // keys past the end weigh nothing
                                const int left = valid - (step * 16 + i * 4);
                                w[i] = left >= 4 ? w[i] : left <= 0 ? 0u : (w[i] & ((1u << (8 * left)) - 1u));
                            }
                            if (!V_TOKEN) isum[i % 2] = __dp4a(w[i], 0x01010101u, isum[i % 2]);
                        }
                    }
                    if (FLUSH && STAGED) {  // out = out * alpha + beta * float(acc), channels 32 step .. 32 step + 31
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            float2 v = o[step * 16 + i];
                            if (RESCALE) v = mul2(v, alpha2);
                            o[step * 16 + i] = fma2(beta2, f[STAGED ? i : 0], v);
                        }
                    }
                    if (SOFT) *reinterpret_cast<uint4*>(p_row + step * (QUERY_TILE * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
                if (SOFT) tmem_fill<KEY_TILE>(t_scores + buf * 64, magic);  // every score has been read: refill the buffer
                tmem_wait_st();
                tc_fence_before();
                TRACE(TR_SOFTMAX);
                if (SOFT) {
                    fence_proxy_async();
                    den = den * alpha_s + (V_TOKEN ? fsum.x + fsum.y : __uint2float_rn(isum[0] + isum[1])) * beta_s;
                }
                if (last_of_step) mbar_arrive(&sm.step_done[g]);  // P^(ts) delivered, its scores buffer and the accumulator free
                TRACE(TR_STORE_P);
                return true;
            };
            using yes = std::true_type;
            using no = std::false_type;
            float unused_a = 1.0f, unused_b = 1.0f;
            auto flush_only = [&](int tf, float alpha_f, float beta_f) -> bool {
                return __all_sync(0xffffffffu, alpha_f == 1.0f) ? tile_step(no{}, yes{}, no{}, no{}, -1, tf, unused_a, unused_b, alpha_f, beta_f)
                                                                : tile_step(no{}, yes{}, no{}, yes{}, -1, tf, unused_a, unused_b, alpha_f, beta_f);
            };
            const bool ragged = n_keys % KEY_TILE != 0;  // the last key tile needs masking: it is taken apart from the flush

            float alpha = 1.0f, beta = 1.0f;
            if (ok) ok = k_tiles == 1 && ragged ? tile_step(yes{}, no{}, yes{}, no{}, 0, -1, alpha, beta, 1.0f, 1.0f)
                                                : tile_step(yes{}, no{}, no{}, no{}, 0, -1, alpha, beta, 1.0f, 1.0f);
            for (int t = 0; ok && t < k_tiles; ++t) {
                float alpha_next = 1.0f, beta_next = 1.0f;
                if (t + 1 == k_tiles) {
                    ok = flush_only(t, alpha, beta);
                } else if (t + 2 == k_tiles && ragged) {
                    ok = tile_step(yes{}, no{}, yes{}, no{}, t + 1, -1, alpha_next, beta_next, 1.0f, 1.0f, false) && flush_only(t, alpha, beta);
                } else if (__all_sync(0xffffffffu, alpha == 1.0f)) {
                    ok = tile_step(yes{}, yes{}, no{}, no{}, t + 1, t, alpha_next, beta_next, alpha, beta);
                } else {
                    ok = tile_step(yes{}, yes{}, no{}, yes{}, t + 1, t, alpha_next, beta_next, alpha, beta);
                }
                alpha = alpha_next;
                beta = beta_next;
            }
        }
        TRACE_END(g);

        if constexpr (OUTLIERS) {
            // The outlier keys were zeros in V8: their exact share p * v / v_scale, with p = 255 * 2^(score - final max),
            // from this row's Q^ (still in shared memory) and the key's K^ row and scale (csrc/flash.cu:748-790).
            if (ok) ok = mbar_wait_warp(&sm.q_full, 0, abort_flag, status, STATUS_WAIT_TILE);
            if (ok) {
                const uint4* q_row8 = reinterpret_cast<const uint4*>(sm.q[g] + row * 16);  // chunk c: QUERY_TILE uint4 further
                for (int i = 0; i < n_outliers; ++i) {
                    const int key = outlier_keys[size_t(head) * n_outliers + i];
                    if (key < 0 || key >= n_keys) continue;
                    const uint4* k_row8 = reinterpret_cast<const uint4*>(k8 + (size_t(head) * k_tiles + key / KEY_TILE) * K_BYTES + (key % KEY_TILE) * 16);
                    int dot = 0;
#pragma unroll
                    for (int c = 0; c < HEAD_DIM / 16; ++c) {
                        const uint4 qv = q_row8[c * QUERY_TILE], kv = k_row8[c * KEY_TILE];
                        dot = __dp4a(int(qv.x), int(kv.x), dot);
                        dot = __dp4a(int(qv.y), int(kv.y), dot);
                        dot = __dp4a(int(qv.z), int(kv.z), dot);
                        dot = __dp4a(int(qv.w), int(kv.w), dot);
                    }
                    const float p = ex2(__int2float_rn(dot) * ((sq * sk[key / KEY_TILE]) * scale_log2) - m) * 255.0f;
                    const float2 p2 = make_float2(p, p);
                    const float2* v_row = reinterpret_cast<const float2*>(outlier_rows + (size_t(head) * n_outliers + i) * HEAD_DIM);
#pragma unroll
                    for (int j = 0; j < HEAD_DIM / 2; ++j) o[j] = fma2(p2, v_row[j], o[j]);
                }
            }
        }

        if (ok && q_row < n_queries) {
            const float inv = 1.0f / den;
            __nv_bfloat16* dst = out + out_layout.offset(head, q_row);
#pragma unroll
            for (int chunk = 0; chunk < HEAD_DIM / 8; ++chunk) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c0 = chunk * 8 + 2 * i;
                    const float2 v = o[chunk * 4 + i];
                    const __nv_bfloat162 pair = __floats2bfloat162_rn(v.x * v_scale[head * HEAD_DIM + c0] * inv,
                                                                      v.y * v_scale[head * HEAD_DIM + c0 + 1] * inv);
                    w[i] = *reinterpret_cast<const uint32_t*>(&pair);
                }
                *reinterpret_cast<uint4*>(dst + chunk * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLUMNS);
    }
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
                                         const int8_t* v8, const float* v_scale, const float* v_token, int v_mode,
                                         const int* outlier_keys, const float* outlier_rows, int n_outliers, void* out,
                                         unica_token_layout out_layout, int heads, int n_queries, int n_keys, float scale_log2,
                                         int* status, void* stream) {
    if (!q8 || !q_scale || !k8 || !k_scale || !v8 || !v_scale || !out) return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_int8: null pointer");
    if (heads <= 0 || heads > 65535 || n_queries <= 0 || n_keys <= 0)
        return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_int8: heads must be in 1..65535, n_queries and n_keys positive");
    if (v_mode != UNICA_B200_V_CHANNEL && v_mode != UNICA_B200_V_TOKEN && v_mode != UNICA_B200_V_OUTLIERS)
        return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_int8: unknown v_mode");
    if (v_mode == UNICA_B200_V_OUTLIERS && (!outlier_keys || !outlier_rows || n_outliers < 1 || n_outliers > 8))
        return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_int8: the outliers mode needs outlier_keys, outlier_rows and 1..8 outliers");
    if (v_mode == UNICA_B200_V_TOKEN && !v_token) return unica_fail(UNICA_B200_ERR_ARGUMENT, "attention_int8: per-token mode needs v_token");
    if (int e = unica_check_device()) return e;
    const dim3 grid((n_queries + 2 * QUERY_TILE - 1) / (2 * QUERY_TILE) * (2 / TILES), heads);  // Q8 holds an even number of tiles
    const size_t smem = sizeof(AttSmem) + 128;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    auto launch = [&](auto kernel) -> int {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess ||
            cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess)
            return unica_check_launch("attention_int8 (shared memory size)");
        // setmaxnreg only moves registers the block already holds: the split must not ask for more than the launch gives,
        // or the computing warps would wait for registers for ever
        cudaFuncAttributes attributes;
        if (cudaFuncGetAttributes(&attributes, kernel) != cudaSuccess) return unica_check_launch("attention_int8 (attributes)");
        if (attributes.numRegs * ATT_THREADS < 128 * TILES * COMPUTE_REGISTERS + 128 * SERVICE_REGISTERS)
            return unica_fail(UNICA_B200_ERR_KERNEL, "attention_int8: this build holds fewer registers per block than its setmaxnreg split needs");
        kernel<<<grid, ATT_THREADS, smem, s>>>(q8, q_scale, k8, k_scale, v8, v_scale, v_token, outlier_keys, outlier_rows, n_outliers,
                                               static_cast<__nv_bfloat16*>(out), to_layout(out_layout), n_queries, n_keys, scale_log2,
                                               status);
        return unica_check_launch("attention_int8");
    };
    return v_mode == UNICA_B200_V_TOKEN      ? launch(attention_int8_kernel<true, false>)
           : v_mode == UNICA_B200_V_OUTLIERS ? launch(attention_int8_kernel<false, true>)
                                             : launch(attention_int8_kernel<false, false>);
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
