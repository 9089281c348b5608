// The accurate mode's flash-attention loop on tcgen05 (replaces the reference's attention_int8pv_tma, csrc/flash.cu:806-959).
//
// One block = one tile of 128 query rows of one head, one block per SM, 20 warps in five warpgroups with three kinds of
// work (a thread of a computing warpgroup owns one query row = one tensor-memory lane, so row maxima and sums need no
// shuffles):
//
//   softmax A, B   key tiles t = 0, 2, 4 .. and 1, 3, 5 ..: the scores S(t) of tensor memory become the bytes
//                  P^(t) = rint(255 * 2^(x - tile max)) of the A-operand image in shared memory.  They carry nothing from
//                  tile to tile: the tile maximum and the row sum go to the flush threads through shared memory.
//   flush 0, 1     output channels 0..63 and 64..127: out = out * alpha + beta * float(acc(t)) for every key tile t, the
//                  row's 64 outputs in registers; they own the running exponent and the denominator, and write the result.
//   service        one producer warp (bulk TMA copies of K8 / V8 tiles, contiguous 8 KB images written by the quantizers,
//                  into a ring of shared-memory stages) and one MMA warp, one elected thread of which issues
//
//   S(t)   = Q8 . K8(t)^T      kind::i8 s8 x s8 -> s32, 128 x 64, 4 instructions of K = 32, a ring of 4 buffers
//   acc(t) = P^(t) . V8(t)     kind::i8 u8 x s8 -> s32, 128 x 128, 2 instructions of K = 32, two accumulators (t even / odd)
//
// Two softmax warpgroups on alternate key tiles keep two warps per scheduler on the exponential unit, the flush runs
// beside them on the ALU and FMA pipes, and neither waits for the other: the scores of tile t + 4 are issued as soon as
// tile t's are consumed, P.V(t) as soon as P^(t) is delivered and the flush of tile t - 2 has read its accumulator.
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

constexpr int ATT_WARPS = 20, ATT_THREADS = ATT_WARPS * 32;
constexpr int FLUSH_WARP = 8, PRODUCER_WARP = 16, MMA_WARP = 17;
// registers per thread after setmaxnreg: 128 x (2 x 80 + 2 x 144 + 32) = 640 x 96, what the block is launched with
constexpr int SOFTMAX_REGISTERS = 80, FLUSH_REGISTERS = 144, SERVICE_REGISTERS = 32;
constexpr int STAGES = 6;   // K8 / V8 tiles in shared memory
constexpr int S_RING = 4;   // score buffers in tensor memory
constexpr int P_RING = STAGES;  // P^ images in shared memory: as many as stages (see the P.V issuing thread)
constexpr int ST_RING = 8;  // (tile maximum, row sum) records on their way from the softmax to the flush threads
constexpr int Q_BYTES = QUERY_TILE * HEAD_DIM;  // 16384
constexpr int K_BYTES = KEY_TILE * HEAD_DIM;    // 8192
constexpr int V_BYTES = KEY_TILE * HEAD_DIM;    // 8192
constexpr int TOK_BYTES = 2 * KEY_TILE * 4;     // 512
constexpr int P_BYTES = QUERY_TILE * KEY_TILE;  // 8192
constexpr int TMEM_COLUMNS = 512;
constexpr int COL_S = 0, COL_ACC = 256;
constexpr float REFERENCE_SLACK = 60.0f;  // log2: how far a tile maximum may rise above a row's reference exponent

struct __align__(128) AttSmem {
    int8_t q[Q_BYTES];
    int8_t k[STAGES][K_BYTES];
    int8_t v[STAGES][V_BYTES];
    float tok[STAGES][2 * KEY_TILE];
    uint8_t p[P_RING][P_BYTES];
    float2 st[ST_RING][QUERY_TILE];
    uint64_t q_full, kv_full[STAGES], kv_empty[STAGES];
    uint64_t s_ready, s_full[S_RING], soft_done[ST_RING], acc_full[2], acc_free[2], drain[2];
    uint32_t tmem_base;
    int abort_flag;
};

// -DUNICA_TRACE: thread 0 of each role of block (0, 0) adds up the cycles it spends in each phase of its tile loop (the
// reference has a TRACE build for the same purpose: csrc/legacy.cu, bench/timeline.py).  Rows of g_trace: softmax A,
// softmax B, flush 0, MMA thread.  The totals stay in registers until the end: tracing costs a clock read per phase.
#ifdef UNICA_TRACE
__device__ long long g_trace[4][8];
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
#endif

constexpr uint32_t IDESC_QK = idesc_i8(true, QUERY_TILE, KEY_TILE);
constexpr uint32_t IDESC_PV = idesc_i8(false, QUERY_TILE, HEAD_DIM);

template <bool V_TOKEN, bool OUTLIERS>
__global__ void __launch_bounds__(ATT_THREADS, 1)
    attention_int8_kernel(const int8_t* __restrict__ q8, const float* __restrict__ q_scale, const int8_t* __restrict__ k8,
                          const float* __restrict__ k_scale, const int8_t* __restrict__ v8, const float* __restrict__ v_scale,
                          const float* __restrict__ v_token, const int* __restrict__ outlier_keys,
                          const float* __restrict__ outlier_rows, int n_outliers, __nv_bfloat16* __restrict__ out,
                          TokenLayout out_layout, int n_queries, int n_keys, float scale_log2, int* status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    AttSmem& sm = *reinterpret_cast<AttSmem*>(smem_raw);
    const int warp = threadIdx.x / 32;
    const int head = blockIdx.y;
    const int q_tiles = gridDim.x;  // allocated Q tiles per head (even)
    const int q_tile = blockIdx.x;
    if (q_tile * QUERY_TILE >= n_queries) return;  // the padding tile of an odd count: nothing to do
    const int k_tiles = (n_keys + KEY_TILE - 1) / KEY_TILE;
    volatile int* abort_flag = &sm.abort_flag;

    if (threadIdx.x == 0) {
        sm.abort_flag = 0;
        mbar_init(&sm.q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&sm.kv_full[s], 1);
            mbar_init(&sm.kv_empty[s], 1);
        }
        mbar_init(&sm.s_ready, 256);
        for (int b = 0; b < S_RING; ++b) mbar_init(&sm.s_full[b], 1);
        for (int b = 0; b < ST_RING; ++b) mbar_init(&sm.soft_done[b], 128);
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sm.acc_full[b], 1);
            mbar_init(&sm.acc_free[b], 256);
        }
        mbar_init(&sm.drain[0], 1);
        mbar_init(&sm.drain[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) tmem_alloc(&sm.tmem_base, TMEM_COLUMNS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    const int row = threadIdx.x % 128, q_row = q_tile * QUERY_TILE + row;
    const uint32_t lane_base = uint32_t((warp % 4) * 32) << 16;
    const bool ragged = n_keys % KEY_TILE != 0;  // the last key tile needs masking

    if (warp >= PRODUCER_WARP) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(SERVICE_REGISTERS));
      if (warp == PRODUCER_WARP) {
        // ------------------------------------------------------------------------------------------------ producer
        if (elect_one()) {  // one elected lane of a converged warp: see elect_one() in common.cuh
            mbar_expect_tx(&sm.q_full, Q_BYTES);
            bulk_load(sm.q, q8 + (size_t(head) * q_tiles + q_tile) * Q_BYTES, Q_BYTES, &sm.q_full);
            int issued = 0;
            for (int t = 0; t < k_tiles; ++t) {
                const int s = t % STAGES, use = t / STAGES;
                if (use > 0 && !mbar_wait(&sm.kv_empty[s], (use - 1) & 1, abort_flag, status, STATUS_WAIT_STAGE)) break;
                mbar_expect_tx(&sm.kv_full[s], K_BYTES + V_BYTES + (V_TOKEN ? TOK_BYTES : 0));
                bulk_load(sm.k[s], k8 + (size_t(head) * k_tiles + t) * K_BYTES, K_BYTES, &sm.kv_full[s]);
                bulk_load(sm.v[s], v8 + (size_t(head) * k_tiles + t) * V_BYTES, V_BYTES, &sm.kv_full[s]);
                if (V_TOKEN) bulk_load(sm.tok[s], v_token + (size_t(head) * k_tiles + t) * (2 * KEY_TILE), TOK_BYTES, &sm.kv_full[s]);
                issued = t + 1;
            }
            if (*abort_flag) {  // let the copies still in flight land before the block's shared memory goes away
                int never = 0;
                for (int t = max(0, issued - STAGES); t < issued; ++t) mbar_wait(&sm.kv_full[t % STAGES], (t / STAGES) & 1, &never, nullptr, 0);
                mbar_wait(&sm.q_full, 0, &never, nullptr, 0);
            }
        }
      } else if (warp == MMA_WARP) {
        // ---------------------------------------------------------------------------------------- MMA issue: P.V
        // One elected thread issues P.V(t) for every key tile as soon as P^(t) is delivered and the flush of tile t - 2
        // has read the accumulator.  Its commit also hands the K8 / V8 stage back to the producer (the scores of the
        // tile were issued four tiles earlier), which the P^ ring relies on: scores S(t) can only be issued into a stage
        // P.V(t - STAGES) has released, so when they complete, the P^ image of tile t - STAGES has been read.
        if (elect_one()) {
            TRACE_DECL(true);
            bool ok = true;
            for (int t = 0; ok && t < k_tiles; ++t) {
                const int stage = t % STAGES, b = t & 1;
                TRACE(7);
                ok = mbar_wait(&sm.kv_full[stage], (t / STAGES) & 1, abort_flag, status, STATUS_WAIT_TILE);  // landed long ago: V8(t) made visible to this thread
                TRACE(0);
                if (t >= 2) ok = ok && mbar_wait(&sm.acc_free[b], ((t - 2) >> 1) & 1, abort_flag, status, STATUS_WAIT_FREE);
                TRACE(2);
                ok = ok && mbar_wait(&sm.soft_done[t % ST_RING], (t / ST_RING) & 1, abort_flag, status, STATUS_WAIT_P);
                TRACE(3);
                if (!ok) break;
                tc_fence_after();
                const uint32_t p_addr = smem_u32(sm.p[t % P_RING]), v_addr = smem_u32(sm.v[stage]);
#pragma unroll
                for (int ks = 0; ks < KEY_TILE / 32; ++ks)
                    mma_i8_ss(tmem + COL_ACC + b * 128, smem_desc(p_addr + ks * 2 * QUERY_TILE * 16, QUERY_TILE * 16, 128),
                              smem_desc(v_addr + ks * 2 * HEAD_DIM * 16, HEAD_DIM * 16, 128), IDESC_PV, ks > 0);  // the first instruction of a tile overwrites the accumulator
                mma_commit(&sm.acc_full[b]);
                mma_commit(&sm.kv_empty[stage]);
                TRACE(4);
            }
            TRACE_END(3);
            if (!ok) {  // whatever was issued must finish before tensor memory is freed
                int never = 0;
                mma_commit(&sm.drain[0]);
                mbar_wait(&sm.drain[0], 0, &never, nullptr, 0);
            }
        }
      } else if (warp == MMA_WARP + 1) {
        // ---------------------------------------------------------------------------------------- MMA issue: scores
        // A second elected thread issues S(n) = Q8 . K8(n)^T as soon as K8(n) has landed and the softmax of tile n - 4
        // has handed the scores buffer back.
        if (elect_one()) {
            const uint32_t q_addr = smem_u32(sm.q);
            bool ok = mbar_wait(&sm.q_full, 0, abort_flag, status, STATUS_WAIT_TILE) &&
                      mbar_wait(&sm.s_ready, 0, abort_flag, status, STATUS_WAIT_FREE);  // the score buffers hold their start value
            for (int n = 0; ok && n < k_tiles; ++n) {
                const int stage = n % STAGES, buf = n % S_RING;
                ok = mbar_wait(&sm.kv_full[stage], (n / STAGES) & 1, abort_flag, status, STATUS_WAIT_TILE);
                if (n >= S_RING)
                    ok = ok && mbar_wait(&sm.soft_done[(n - S_RING) % ST_RING], ((n - S_RING) / ST_RING) & 1, abort_flag, status, STATUS_WAIT_FREE);
                if (!ok) break;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(sm.k[stage]);
#pragma unroll
                for (int ks = 0; ks < HEAD_DIM / 32; ++ks)
                    mma_i8_ss(tmem + COL_S + buf * 64, smem_desc(q_addr + ks * 2 * QUERY_TILE * 16, QUERY_TILE * 16, 128),
                              smem_desc(k_addr + ks * 2 * KEY_TILE * 16, KEY_TILE * 16, 128), IDESC_QK, true);
                mma_commit(&sm.s_full[buf]);
            }
            if (!ok) {
                int never = 0;
                mma_commit(&sm.drain[1]);
                mbar_wait(&sm.drain[1], 0, &never, nullptr, 0);
            }
        }
      }
    } else if (warp < FLUSH_WARP) {
        // ------------------------------------------------------------------------------------------------ softmax
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(SOFTMAX_REGISTERS));
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
        auto softmax_tile = [&](auto masked_c, int t, float c) -> bool {
            constexpr bool MASKED = decltype(masked_c)::value;
            const int buf = t % S_RING, stage = t % STAGES;
            const int valid = min(KEY_TILE, n_keys - t * KEY_TILE);
            const uint32_t ts = t_s + buf * 64;
            TRACE(7);
            if (!mbar_wait_warp(&sm.s_full[buf], (t / S_RING) & 1, abort_flag, status, STATUS_WAIT_SCORES)) return false;
            TRACE(0);
            if (V_TOKEN && !mbar_wait_warp(&sm.kv_full[stage], (t / STAGES) & 1, abort_flag, status, STATUS_WAIT_TILE)) return false;
            tc_fence_after();
            const float2 c2 = make_float2(c, c), minus_magic = make_float2(-MAGIC, -MAGIC);
            const float4* log_s4 = reinterpret_cast<const float4*>(sm.tok[stage]);
            const float4* inv_s4 = reinterpret_cast<const float4*>(sm.tok[stage] + KEY_TILE);
            float2 x[2][8];  // 16 scores in use, 16 on their way

            // Pass 1: the tile maximum (the 64 scores are read again below: they would not fit next to the rest).
            float top[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            tmem_ld16_async(ts, x[0]);
            tmem_ld16_async(ts + 16, x[1]);
#pragma unroll
            for (int step = 0; step < KEY_TILE / 16; ++step) {
                float2(&y)[8] = x[step % 2];
                if (step % 2 == 0) tmem_wait_ld();  // both loads in flight
                reg_fence8(y);
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
                if (step + 2 < KEY_TILE / 16) {
                    reg_fence8(y);
                    tmem_ld16_async(ts + (step + 2) * 16, y);
                }
            }
            float tile_max = fmaxf(fmaxf(top[0], top[1]), fmaxf(top[2], top[3]));
            TRACE(1);
            if (!V_TOKEN) tile_max = (tile_max - MAGIC) * c;
            const float offset = LOG2_255 - tile_max;

            // Pass 2: P^ = rint(255 * 2^(score * c - tile max)), 16 keys at a time.  Per channel the float read back is
            // MAGIC + score, so the exponent is x * c + (offset - MAGIC * c) in ONE fused multiply-add; what the rounding
            // of that constant loses (it is about 2^11 in size) is put back exactly: `low` is the lost part, and the
            // product p * 2^low happens inside the multiply-add that rounds p to a byte.
            float2 base2, k2;
            if (!V_TOKEN) {
                const float a_hi = __fmul_rn(-MAGIC, c), a_lo = __fmaf_rn(-MAGIC, c, -a_hi);  // -MAGIC * c = a_hi + a_lo exactly
                const float s = __fadd_rn(a_hi, offset), bb = __fsub_rn(s, a_hi);
                const float low = __fadd_rn(__fadd_rn(__fsub_rn(a_hi, __fsub_rn(s, bb)), __fsub_rn(offset, bb)), a_lo);  // a_hi + offset = s + ..
                const float k = __fmaf_rn(low, 0.693147181f, 1.0f);  // 2^low, |low| < 2^-12
                base2 = make_float2(s, s), k2 = make_float2(k, k);
            } else {
                base2 = make_float2(offset, offset), k2 = make_float2(1.0f, 1.0f);
            }
            const float2 plus_magic = make_float2(MAGIC, MAGIC);
            uint8_t* p_row = sm.p[t % P_RING] + row * 16;
            unsigned isum[2] = {0, 0};
            float2 fsum = make_float2(0.0f, 0.0f);
            tmem_ld16_async(ts, x[0]);
#pragma unroll
            for (int step = 0; step < KEY_TILE / 16; ++step) {
                float2(&y)[8] = x[step % 2];
                tmem_wait_ld();
                reg_fence8(y);
                if (step + 1 < KEY_TILE / 16) {
                    tmem_ld16_async(ts + (step + 1) * 16, x[(step + 1) % 2]);
                } else {  // every score has been read: the buffer goes back to its start value for S(t + 4)
                    tmem_fill<KEY_TILE>(ts, magic);
                }
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t pair[2];
                    float4 l = make_float4(0.0f, 0.0f, 0.0f, 0.0f), r = l;  // log2 s and 1 / s of the four keys
                    if (V_TOKEN) l = log_s4[step * 4 + i], r = inv_s4[step * 4 + i];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {  // a pair of keys
                        float2 e;
                        if (V_TOKEN)
                            e = add2(fma2(add2(y[i * 2 + h], minus_magic), c2, h ? make_float2(l.z, l.w) : make_float2(l.x, l.y)), base2);
                        else
                            e = fma2(y[i * 2 + h], c2, base2);
                        const float2 p = make_float2(ex2(e.x), ex2(e.y));
                        if (V_TOKEN) fsum = fma2(p, h ? make_float2(r.z, r.w) : make_float2(r.x, r.y), fsum);
                        const float2 rounded = V_TOKEN ? add2(p, plus_magic) : fma2(p, k2, plus_magic);  // the low byte of each is rint(p)
                        pair[h] = __byte_perm(__float_as_uint(rounded.x), __float_as_uint(rounded.y), 0x0040);
                    }
                    w[i] = __byte_perm(pair[0], pair[1], 0x5410);
                    if (!V_TOKEN && MASKED) {  // keys past the end weigh nothing
                        const int left = valid - (step * 16 + i * 4);
                        w[i] = left >= 4 ? w[i] : left <= 0 ? 0u : (w[i] & ((1u << (8 * left)) - 1u));
                    }
                    if (!V_TOKEN) isum[i % 2] = __dp4a(w[i], 0x01010101u, isum[i % 2]);
                }
                *reinterpret_cast<uint4*>(p_row + step * (QUERY_TILE * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            TRACE(2);
            sm.st[t % ST_RING][row] = make_float2(tile_max, V_TOKEN ? fsum.x + fsum.y : __uint2float_rn(isum[0] + isum[1]));
            tmem_wait_st();
            tc_fence_before();
            fence_proxy_async();
            mbar_arrive(&sm.soft_done[t % ST_RING]);  // P^(t) and its record delivered, the scores buffer back at its start value
            TRACE(3);
            return true;
        };

        bool ok = true;
        for (int t = parity; ok && t < k_tiles; t += 2) {
            const float c = (sq * sk_reg) * scale_log2;
            if (t + 2 < k_tiles) sk_reg = load_scale(sk + t + 2);
            ok = ragged && t + 1 == k_tiles ? softmax_tile(std::true_type{}, t, c) : softmax_tile(std::false_type{}, t, c);
        }
        TRACE_END(parity);
    } else {
        // ------------------------------------------------------------------------------------------------ flush
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(FLUSH_REGISTERS));
        const int half = (warp - FLUSH_WARP) / 4;  // output channels 64 half .. 64 half + 63
        const uint32_t t_acc = tmem + lane_base + COL_ACC + half * 64;
        float m = -INFINITY, den = 0.0f;
        float2 o[HEAD_DIM / 4];
#pragma unroll
        for (int i = 0; i < HEAD_DIM / 4; ++i) o[i] = make_float2(0.0f, 0.0f);

        auto flush_tile = [&](auto rescale_c, const float2 (&a0)[16], const float2 (&a1)[16], float alpha, float beta) {
            constexpr bool RESCALE = decltype(rescale_c)::value;
            const float2 alpha2 = make_float2(alpha, alpha), beta2 = make_float2(beta, beta);
#pragma unroll
            for (int i = 0; i < 32; ++i) {  // the accumulator is overwritten by every tile's P.V: plain integers
                const float2 raw = i < 16 ? a0[i % 16] : a1[i % 16];
                const float2 f = make_float2(__int2float_rn(__float_as_int(raw.x)), __int2float_rn(__float_as_int(raw.y)));
                o[i] = fma2(beta2, f, RESCALE ? mul2(o[i], alpha2) : o[i]);
            }
        };

        bool ok = true;
        TRACE_DECL(row == 0 && half == 0);
        for (int t = 0; ok && t < k_tiles; ++t) {
            const int b = t & 1;
            TRACE(7);
            if (!mbar_wait_warp(&sm.soft_done[t % ST_RING], (t / ST_RING) & 1, abort_flag, status, STATUS_WAIT_P)) {
                ok = false;
                break;
            }
            // `m` is the exponent the row's sums are kept at, not the running maximum: out = sum over tiles of
            // 2^(tile max - m) * acc, the same for the denominator, and the common factor cancels at the end.  The
            // textbook form moves m to every new maximum and multiplies out and den by alpha = 2^(m_old - m_new) each
            // time; here m moves only when a tile maximum is more than 2^REFERENCE_SLACK above it, so that
            // multiplication all but disappears.  The difference is rounding only.
            TRACE(0);
            const float2 record = sm.st[t % ST_RING][row];  // tile maximum, row sum
            const bool first = m == -INFINITY;
            const float m_new = record.x > m + REFERENCE_SLACK ? record.x : m;
            const float alpha = first ? 1.0f : ex2(m - m_new), beta = ex2(record.x - m_new);
            m = m_new;
            den = den * alpha + record.y * beta;
            if (!mbar_wait_warp(&sm.acc_full[b], (t >> 1) & 1, abort_flag, status, STATUS_WAIT_PV)) {
                ok = false;
                break;
            }
            TRACE(1);
            tc_fence_after();
            float2 a0[16], a1[16];
            tmem_ld32_async(t_acc + b * 128, a0);
            tmem_ld32_async(t_acc + b * 128 + 32, a1);
            tmem_wait_ld();
            reg_fence16(a0);
            reg_fence16(a1);
            tc_fence_before();
            mbar_arrive(&sm.acc_free[b]);  // P.V(t + 2) may overwrite the accumulator
            TRACE(2);
            if (__all_sync(0xffffffffu, alpha == 1.0f))
                flush_tile(std::false_type{}, a0, a1, alpha, beta);
            else
                flush_tile(std::true_type{}, a0, a1, alpha, beta);
            TRACE(3);
        }
        TRACE_END(2);

        if constexpr (OUTLIERS) {
            // The outlier keys were zeros in V8: their exact share p * v / v_scale, with p = 255 * 2^(score - final max),
            // from this row's Q^ (still in shared memory) and the key's K^ row and scale (csrc/flash.cu:748-790).
            if (ok) ok = mbar_wait_warp(&sm.q_full, 0, abort_flag, status, STATUS_WAIT_TILE);
            if (ok) {
                const float sq = q_scale[size_t(head) * q_tiles + q_tile];
                const float* sk = k_scale + size_t(head) * k_tiles;
                const uint4* q_row8 = reinterpret_cast<const uint4*>(sm.q + row * 16);  // chunk c: QUERY_TILE uint4 further
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
                    const float2* v_row = reinterpret_cast<const float2*>(outlier_rows + (size_t(head) * n_outliers + i) * HEAD_DIM + half * 64);
#pragma unroll
                    for (int j = 0; j < HEAD_DIM / 4; ++j) o[j] = fma2(p2, v_row[j], o[j]);
                }
            }
        }

        if (ok && q_row < n_queries) {
            const float inv = 1.0f / den;
            __nv_bfloat16* dst = out + out_layout.offset(head, q_row) + half * 64;
            const float* vs = v_scale + head * HEAD_DIM + half * 64;
#pragma unroll
            for (int chunk = 0; chunk < HEAD_DIM / 16; ++chunk) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c0 = chunk * 8 + 2 * i;
                    const float2 v = o[chunk * 4 + i];
                    const __nv_bfloat162 pair = __floats2bfloat162_rn(v.x * vs[c0] * inv, v.y * vs[c0 + 1] * inv);
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
        const uint32_t idesc = idesc_i8(!a_unsigned, 128, n);
        for (int ks = 0; ks < k / 32; ++ks) {
            mma_i8_ss(tmem, smem_desc(smem_u32(a_s) + ks * 2 * 128 * 16, 128 * 16, 128), smem_desc(smem_u32(b_s) + ks * 2 * n * 16, n * 16, 128),
                      idesc, ks > 0);
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
            if (attributes.numRegs * ATT_THREADS < 128 * (2 * SOFTMAX_REGISTERS + 2 * FLUSH_REGISTERS + SERVICE_REGISTERS))
                return unica_fail(UNICA_B200_ERR_KERNEL, "attention_int8: this build holds fewer registers per block than its setmaxnreg split needs");
            if (device < MAX_DEVICES) ready[device].store(1, std::memory_order_release);
        }
        kernel<<<grid, ATT_THREADS, smem, s>>>(q8, q_scale, k8, k_scale, v8, v_scale, v_token, outlier_keys, outlier_rows, n_outliers,
                                               static_cast<__nv_bfloat16*>(out), to_layout(out_layout), n_queries, n_keys, scale_log2,
                                               status);
        return unica_check_launch("attention_int8");
    };
    return v_mode == UNICA_B200_V_TOKEN      ? launch(attention_int8_kernel<true, false>, 1)
           : v_mode == UNICA_B200_V_OUTLIERS ? launch(attention_int8_kernel<false, true>, 2)
                                             : launch(attention_int8_kernel<false, false>, 0);
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
