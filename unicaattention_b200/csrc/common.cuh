// Shared device-side helpers for the sm_100a kernels: the caller's tensor layout, bounded mbarrier waits, bulk (TMA)
// copies, tensor-memory allocation and the tcgen05 instructions the attention kernels issue.
//
// Every wait here is bounded: a wait that does not complete within WAIT_LIMIT_CYCLES records a status code and
// returns false, and the kernels then leave their loops, drain what they started and free their tensor memory.  A
// kernel therefore always terminates, whatever went wrong with its pipeline.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#ifndef UNICA_FILL_BLOCK
#define UNICA_FILL_BLOCK 8
#endif

namespace unica {

constexpr int HEAD_DIM = 128;
constexpr int KEY_TILE = 64;     // keys per tile: the K scale block and the softmax tile of the numerics contract
constexpr int QUERY_TILE = 128;  // query rows per tile: the Q scale block, and M of one tcgen05.mma
constexpr float LOG2_255 = 7.99435343685886f;

// Where token `token` of head `head_index` (= batch * heads + head) starts in a [batch, heads, tokens, 128] tensor with
// a contiguous last dimension and any other strides; strides in elements.  Field for field the reference's struct
// (csrc/flash.cu:231-237), so a caller fills it the same way.
struct TokenLayout {
    long long batch, head, token;
    int heads;
    int half;  // the elements are float16, not bfloat16 (see load_bf16x8 / the kernels' epilogues)
    __host__ __device__ __forceinline__ size_t offset(int head_index, int token_index) const {
        return size_t(head_index / heads) * batch + size_t(head_index % heads) * head + size_t(token_index) * token;
    }
};

// Eight consecutive input elements as bfloat16 bits.  float16 input is rounded to bfloat16 here, in registers (round to
// nearest even, what torch's .to(bfloat16) does), so every pass downstream sees exactly what it would see had the caller
// converted the tensor first, without that conversion's trip through memory (the reference converts: unica/__init__.py:236).
__device__ __forceinline__ uint4 load_bf16x8(const __nv_bfloat16* src, bool half) {
    uint4 raw = *reinterpret_cast<const uint4*>(src);
    if (half) {
        uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
            w[i] = *reinterpret_cast<const uint32_t*>(&b);
        }
    }
    return raw;
}
// Two output values as the 32 bits the output tensor takes: bfloat16, or for a float16 tensor the float16 of that
// bfloat16 (what converting the bfloat16 result gives; exact unless the value leaves float16's range).
__device__ __forceinline__ uint32_t output_pair(float x, float y, bool half) {
    const __nv_bfloat162 b = __floats2bfloat162_rn(x, y);
    if (!half) return *reinterpret_cast<const uint32_t*>(&b);
    const float2 f = __bfloat1622float2(b);
    const __half2 h = __floats2half2_rn(f.x, f.y);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// The same output tensor on other GPUs (peer mappings of their memory): the attention kernels store every output row
// they compute to `out` and to each of these, at the same offsets.  Plain stores only; nothing is read from a peer.
constexpr int MAX_PEER_OUTPUTS = 7;
struct PeerOutputs {
    __nv_bfloat16* out[MAX_PEER_OUTPUTS];
    int count;
};

// Output rows on their way out through shared memory, so that a warp writes whole 256-byte rows (two per instruction)
// instead of 32 separate pieces of 16 bytes: that matters little for this GPU's memory and much for rows that cross
// NVLink to a peer.  A warp owns 32 rows of 128 bf16 in `staged` (8 KB); the 16-byte pieces of a row are swapped about
// by the row number, so neither the row-per-thread writes nor the row-per-half-warp reads meet bank conflicts.
__device__ __forceinline__ void stage_piece(uint8_t* staged, int row_in_warp, int piece, uint4 value) {
    *reinterpret_cast<uint4*>(staged + row_in_warp * 256 + ((piece ^ (row_in_warp & 15)) * 16)) = value;
}
// The warp's 32 staged rows (query rows first_row ..) to `out` and to every peer; all lanes call it after __syncwarp().
__device__ __forceinline__ void store_staged_rows(const uint8_t* staged, int lane, int first_row, int n_queries, int head,
                                                  __nv_bfloat16* out, const TokenLayout& layout, const PeerOutputs& peers) {
    const int piece = lane % 16;
#pragma unroll 4
    for (int pair = 0; pair < 16; ++pair) {
        const int r = 2 * pair + lane / 16;
        const uint4 value = *reinterpret_cast<const uint4*>(staged + r * 256 + ((piece ^ (r & 15)) * 16));
        if (first_row + r < n_queries) {
            const size_t at = layout.offset(head, first_row + r) + piece * 8;
            *reinterpret_cast<uint4*>(out + at) = value;
            for (int peer = 0; peer < peers.count; ++peer) *reinterpret_cast<uint4*>(peers.out[peer] + at) = value;
        }
    }
}

// RoPE inside the quantizers (the reference's rope_chunk, csrc/flash.cu:250-268): (cos, sin) per pair of channels in fp16,
// [batch or 1][n_tokens][64][2]; batch_stride in halves, 0 when one table serves every batch.  table null: no rotation.
struct RopeTable {
    const __half* table;
    long long batch_stride;
    __device__ __forceinline__ const __half* row(const TokenLayout& in, int head_index, int token_index) const {
        return table + size_t(head_index / in.heads) * batch_stride + size_t(token_index) * 128;
    }
};

// Eight channels starting at channel `dim` (a multiple of 8) of one token, rotated: out[2i] = c x[2i] - s x[2i+1],
// out[2i+1] = s x[2i] + c x[2i+1], each product rounded, then the difference or sum: no fused multiply-add, as the
// emulator computes it (bench/emulate.py:122-130).
__device__ __forceinline__ void rope8(float (&v)[8], const __half* token_row, int dim) {
    const uint4 raw = *reinterpret_cast<const uint4*>(token_row + dim);
    const __half2* cs = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 r = __half22float2(cs[j]);  // (cos, sin)
        const float x0 = v[2 * j], x1 = v[2 * j + 1];
        v[2 * j] = __fsub_rn(__fmul_rn(r.x, x0), __fmul_rn(r.y, x1));
        v[2 * j + 1] = __fadd_rn(__fmul_rn(r.y, x0), __fmul_rn(r.x, x1));
    }
}

// status codes a kernel leaves in its status word (0: fine)
enum Status : int {
    STATUS_OK = 0,
    STATUS_WAIT_TILE = 1,     // a K/V/Q tile never arrived
    STATUS_WAIT_SCORES = 2,   // S = Q.K^T never completed
    STATUS_WAIT_P = 3,        // the softmax threads never delivered P
    STATUS_WAIT_PV = 4,       // P.V never completed
    STATUS_WAIT_FREE = 5,     // a buffer was never released
    STATUS_WAIT_STAGE = 6,    // the producer never got a stage back
    STATUS_WAIT_PARTNER = 7,  // the other thread of a query row never published its value
    STATUS_WAIT_GROUP = 8,    // a block of a one-launch quantizer never saw its group's statistics
};

constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;  // about a second

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// ---------------------------------------------------------------------------------------------------------------------
// mbarrier

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Non-blocking: has the phase of parity `parity` completed?
__device__ __forceinline__ bool mbar_test(uint64_t* bar, int parity) {
    uint32_t done;
    asm volatile(
        "{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, int parity) {
    uint32_t done;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// The same probe, but the thread may be suspended by the hardware for up to UNICA_WAIT_HINT_NS until the phase completes:
// a waiting thread then issues no instructions, where a loop of plain probes takes issue slots from the computing
// warps of its scheduler.
#ifndef UNICA_WAIT_HINT_NS
#define UNICA_WAIT_HINT_NS 2000
#endif
__device__ __forceinline__ bool mbar_try_suspended(uint64_t* bar, int parity) {
    uint32_t done;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3; selp.u32 %0, 1, 0, p; }"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity), "r"(uint32_t(UNICA_WAIT_HINT_NS))
        : "memory");
    return done != 0;
}

// Waits for the phase of parity `parity`.  abort_flag: a word in shared memory any thread of the block sets when it
// gave up; everyone else then stops waiting at once.  Returns false when the wait was abandoned.
// A waiting warp shares its scheduler with computing warps and every instruction of its loop takes an issue slot from
// them (the probe itself returns within a few dozen cycles when the phase has not completed), so after a failed probe
// the warp sleeps for WAIT_SLEEP_NS before the next one, and the loop is the probe, the sleep, a counter and a branch,
// written in PTX so that nothing else gets into it; the abort word and the clock are looked at once in WAIT_PROBES
// probes.
#ifndef UNICA_WAIT_SLEEP_NS
#define UNICA_WAIT_SLEEP_NS 64
#endif
constexpr unsigned WAIT_PROBES = 2048, WAIT_SLEEP_NS = UNICA_WAIT_SLEEP_NS;
template <unsigned SLEEP_NS = WAIT_SLEEP_NS>
__device__ __forceinline__ bool mbar_probe_many(uint64_t* bar, int parity) {
    uint32_t done;
    if constexpr (SLEEP_NS > 0) {
        asm volatile(
            "{\n\t"
            ".reg .pred p, q;\n\t"
            ".reg .u32 left;\n\t"
            "mov.u32 left, %3;\n"
            "UNICA_WAIT_AGAIN:\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "@p bra UNICA_WAIT_DONE;\n\t"
            "nanosleep.u32 %4;\n\t"
            "sub.u32 left, left, 1;\n\t"
            "setp.ne.u32 q, left, 0;\n\t"
            "@q bra UNICA_WAIT_AGAIN;\n"
            "UNICA_WAIT_DONE:\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}"
            : "=r"(done)
            : "r"(smem_u32(bar)), "r"(parity), "n"(WAIT_PROBES), "n"(SLEEP_NS)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p, q;\n\t"
            ".reg .u32 left;\n\t"
            "mov.u32 left, %3;\n"
            "UNICA_SPIN_AGAIN:\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "@p bra UNICA_SPIN_DONE;\n\t"
            "sub.u32 left, left, 1;\n\t"
            "setp.ne.u32 q, left, 0;\n\t"
            "@q bra UNICA_SPIN_AGAIN;\n"
            "UNICA_SPIN_DONE:\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}"
            : "=r"(done)
            : "r"(smem_u32(bar)), "r"(parity), "n"(WAIT_PROBES)
            : "memory");
    }
    return done != 0;
}
// SLEEP_NS 0: for waits whose end is on everybody's critical path; the loop then is the plain one (probe, abort word,
// clock), which measured faster than a bare run of probes: back-to-back probes crowd the queue that shared-memory
// accesses and exponentials of the computing warps go through.
template <unsigned SLEEP_NS = WAIT_SLEEP_NS>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, int parity, volatile int* abort_flag, int* status, int code) {
    if constexpr (SLEEP_NS == 0) {
        if (mbar_try(bar, parity)) return true;
        const long long start = clock64();
        while (true) {
            if (UNICA_WAIT_HINT_NS > 0 ? mbar_try_suspended(bar, parity) : mbar_try(bar, parity)) return true;
            if (*abort_flag) return false;
            if (clock64() - start > WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                if (status) atomicCAS(status, 0, code);
                return false;
            }
        }
    } else {
        if (mbar_probe_many<SLEEP_NS>(bar, parity)) return true;
        const long long start = clock64();
        while (true) {
            if (mbar_probe_many<SLEEP_NS>(bar, parity)) return true;
            if (*abort_flag) return false;
            if (clock64() - start > WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                if (status) atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

// Two barriers at once: both probes are in flight together, so a lone thread pays one probe latency (some 250 cycles)
// instead of two.  parity_b < 0: there is no second barrier.
template <unsigned SLEEP_NS = WAIT_SLEEP_NS>
__device__ __forceinline__ bool mbar_probe_many2(uint64_t* bar_a, int parity_a, uint64_t* bar_b, int parity_b) {
    uint32_t done;
    if constexpr (SLEEP_NS > 0) {
        asm volatile(
            "{\n\t"
            ".reg .pred p, q, r;\n\t"
            ".reg .u32 left;\n\t"
            "mov.u32 left, %5;\n"
            "UNICA_WAIT2_AGAIN:\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 q, [%3], %4;\n\t"
            "and.pred r, p, q;\n\t"
            "@r bra UNICA_WAIT2_DONE;\n\t"
            "nanosleep.u32 %6;\n\t"
            "sub.u32 left, left, 1;\n\t"
            "setp.ne.u32 q, left, 0;\n\t"
            "@q bra UNICA_WAIT2_AGAIN;\n"
            "UNICA_WAIT2_DONE:\n\t"
            "selp.u32 %0, 1, 0, r;\n\t"
            "}"
            : "=r"(done)
            : "r"(smem_u32(bar_a)), "r"(parity_a), "r"(smem_u32(bar_b)), "r"(parity_b), "n"(WAIT_PROBES), "n"(SLEEP_NS)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p, q, r;\n\t"
            ".reg .u32 left;\n\t"
            "mov.u32 left, %5;\n"
            "UNICA_SPIN2_AGAIN:\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 q, [%3], %4;\n\t"
            "and.pred r, p, q;\n\t"
            "@r bra UNICA_SPIN2_DONE;\n\t"
            "sub.u32 left, left, 1;\n\t"
            "setp.ne.u32 q, left, 0;\n\t"
            "@q bra UNICA_SPIN2_AGAIN;\n"
            "UNICA_SPIN2_DONE:\n\t"
            "selp.u32 %0, 1, 0, r;\n\t"
            "}"
            : "=r"(done)
            : "r"(smem_u32(bar_a)), "r"(parity_a), "r"(smem_u32(bar_b)), "r"(parity_b), "n"(WAIT_PROBES)
            : "memory");
    }
    return done != 0;
}
template <unsigned SLEEP_NS = WAIT_SLEEP_NS>
__device__ __forceinline__ bool mbar_wait2(uint64_t* bar_a, int parity_a, uint64_t* bar_b, int parity_b, volatile int* abort_flag, int* status,
                                           int code) {
    if (parity_b < 0) return mbar_wait<SLEEP_NS>(bar_a, parity_a, abort_flag, status, code);
    if constexpr (SLEEP_NS == 0 && UNICA_WAIT_HINT_NS > 0) {  // one look at both with the probes in flight together, then suspended waits
        uint32_t seen;
        asm volatile(
            "{\n\t"
            ".reg .pred p, q;\n\t"
            ".reg .u32 a, b;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 q, [%3], %4;\n\t"
            "selp.u32 a, 1, 0, p;\n\t"
            "selp.u32 b, 2, 0, q;\n\t"
            "or.b32 %0, a, b;\n\t"
            "}"
            : "=r"(seen)
            : "r"(smem_u32(bar_a)), "r"(parity_a), "r"(smem_u32(bar_b)), "r"(parity_b)
            : "memory");
        if (seen == 3) return true;
        if (!(seen & 1) && !mbar_wait<0>(bar_a, parity_a, abort_flag, status, code)) return false;
        return (seen & 2) || mbar_wait<0>(bar_b, parity_b, abort_flag, status, code);
    }
    if (mbar_probe_many2<SLEEP_NS>(bar_a, parity_a, bar_b, parity_b)) return true;
    const long long start = clock64();
    while (true) {
        if (mbar_probe_many2<SLEEP_NS>(bar_a, parity_a, bar_b, parity_b)) return true;
        if (*abort_flag) return false;
        if (clock64() - start > WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            if (status) atomicCAS(status, 0, code);
            return false;
        }
    }
}

// A word in shared memory that one thread of the block advances and others wait for.  Looking at a word costs a waiting
// warp an ordinary shared-memory load (some 30 cycles), a tenth of an mbarrier probe, so where the event is first seen by
// a thread that has to watch it anyway (the completion of tcgen05.mma by the thread that issued them), that thread passes
// it on through such a word.  Release / acquire at block scope; bounded like every other wait here.
#ifndef UNICA_FLAG_SLEEP_NS
#define UNICA_FLAG_SLEEP_NS 0
#endif
__device__ __forceinline__ void flag_publish(int* flag, int value) {
    asm volatile("st.release.cta.shared::cta.s32 [%0], %1;" ::"r"(smem_u32(flag)), "r"(value) : "memory");
}
__device__ __forceinline__ bool flag_wait(const int* flag, int at_least, volatile int* abort_flag, int* status, int code) {
    long long start = 0;
    for (int looks = 1;; ++looks) {
        int value;
        asm volatile("ld.acquire.cta.shared::cta.s32 %0, [%1];" : "=r"(value) : "r"(smem_u32(flag)) : "memory");
        if (value >= at_least) return true;
#if UNICA_FLAG_SLEEP_NS > 0
        __nanosleep(UNICA_FLAG_SLEEP_NS);  // back-to-back looks crowd the queue the computing warps' exponentials go through
#endif
        if (looks % 256 == 0) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (start == 0) start = now;
            if (now - start > WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                if (status) atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool flag_wait_warp(const int* flag, int at_least, volatile int* abort_flag, int* status, int code) {
    return __all_sync(0xffffffffu, flag_wait(flag, at_least, abort_flag, status, code));
}

// The same for a whole warp: every lane waits, and all get the same answer.  The vote also reconverges the warp, which
// the .sync.aligned tensor-memory instructions that usually follow require: a tcgen05.ld executed by part of a warp
// never completes.
template <unsigned SLEEP_NS = WAIT_SLEEP_NS>
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, int parity, volatile int* abort_flag, int* status, int code) {
    return __all_sync(0xffffffffu, mbar_wait<SLEEP_NS>(bar, parity, abort_flag, status, code));
}

// ---------------------------------------------------------------------------------------------------------------------
// bulk copies (the untiled TMA path): global -> shared, completion counted in bytes on an mbarrier.
// dst, src 16-byte aligned, bytes a multiple of 16.

__device__ __forceinline__ void bulk_load(void* dst, const void* src, int bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// generic-proxy writes to shared memory made visible to the async proxy (tcgen05.mma operand reads)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------------------------------
// tensor memory

// One warp allocates `columns` (a power of two >= 32) and leaves the base address in *dst (shared memory).
__device__ __forceinline__ void tmem_alloc(uint32_t* dst, int columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, int columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 consecutive 32-bit columns of this thread's lane (lane = 32 * (warp % 4) + lane id): r[i] = column i.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// 64 consecutive columns as 32 float2 (bit patterns untouched), load and wait in ONE statement so that no use of the
// registers can be scheduled before the wait.
__device__ __forceinline__ void tmem_ld64_sync(uint32_t taddr, float2 (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
        "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
        "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=f"(v[0].x), "=f"(v[0].y), "=f"(v[1].x), "=f"(v[1].y), "=f"(v[2].x), "=f"(v[2].y), "=f"(v[3].x), "=f"(v[3].y),
          "=f"(v[4].x), "=f"(v[4].y), "=f"(v[5].x), "=f"(v[5].y), "=f"(v[6].x), "=f"(v[6].y), "=f"(v[7].x), "=f"(v[7].y),
          "=f"(v[8].x), "=f"(v[8].y), "=f"(v[9].x), "=f"(v[9].y), "=f"(v[10].x), "=f"(v[10].y), "=f"(v[11].x), "=f"(v[11].y),
          "=f"(v[12].x), "=f"(v[12].y), "=f"(v[13].x), "=f"(v[13].y), "=f"(v[14].x), "=f"(v[14].y), "=f"(v[15].x), "=f"(v[15].y),
          "=f"(v[16].x), "=f"(v[16].y), "=f"(v[17].x), "=f"(v[17].y), "=f"(v[18].x), "=f"(v[18].y), "=f"(v[19].x), "=f"(v[19].y),
          "=f"(v[20].x), "=f"(v[20].y), "=f"(v[21].x), "=f"(v[21].y), "=f"(v[22].x), "=f"(v[22].y), "=f"(v[23].x), "=f"(v[23].y),
          "=f"(v[24].x), "=f"(v[24].y), "=f"(v[25].x), "=f"(v[25].y), "=f"(v[26].x), "=f"(v[26].y), "=f"(v[27].x), "=f"(v[27].y),
          "=f"(v[28].x), "=f"(v[28].y), "=f"(v[29].x), "=f"(v[29].y), "=f"(v[30].x), "=f"(v[30].y), "=f"(v[31].x), "=f"(v[31].y)
        : "r"(taddr)
        : "memory");
}

// 32 consecutive columns as 16 float2, issued without waiting; tmem_wait_ld() then reg_fence16() before the first use.
__device__ __forceinline__ void tmem_ld32_async(uint32_t taddr, float2 (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=f"(v[0].x), "=f"(v[0].y), "=f"(v[1].x), "=f"(v[1].y), "=f"(v[2].x), "=f"(v[2].y), "=f"(v[3].x), "=f"(v[3].y),
          "=f"(v[4].x), "=f"(v[4].y), "=f"(v[5].x), "=f"(v[5].y), "=f"(v[6].x), "=f"(v[6].y), "=f"(v[7].x), "=f"(v[7].y),
          "=f"(v[8].x), "=f"(v[8].y), "=f"(v[9].x), "=f"(v[9].y), "=f"(v[10].x), "=f"(v[10].y), "=f"(v[11].x), "=f"(v[11].y),
          "=f"(v[12].x), "=f"(v[12].y), "=f"(v[13].x), "=f"(v[13].y), "=f"(v[14].x), "=f"(v[14].y), "=f"(v[15].x), "=f"(v[15].y)
        : "r"(taddr)
        : "memory");
}

// Emits nothing; ties the 32 registers to this point of the (volatile-ordered) instruction stream, so that uses of
// an asynchronous tensor-memory load cannot move above the tcgen05.wait::ld that precedes this call.
__device__ __forceinline__ void reg_fence16(float2 (&v)[16]) {
    asm volatile(""
                 : "+f"(v[0].x), "+f"(v[0].y), "+f"(v[1].x), "+f"(v[1].y), "+f"(v[2].x), "+f"(v[2].y), "+f"(v[3].x), "+f"(v[3].y),
                   "+f"(v[4].x), "+f"(v[4].y), "+f"(v[5].x), "+f"(v[5].y), "+f"(v[6].x), "+f"(v[6].y), "+f"(v[7].x), "+f"(v[7].y),
                   "+f"(v[8].x), "+f"(v[8].y), "+f"(v[9].x), "+f"(v[9].y), "+f"(v[10].x), "+f"(v[10].y), "+f"(v[11].x), "+f"(v[11].y),
                   "+f"(v[12].x), "+f"(v[12].y), "+f"(v[13].x), "+f"(v[13].y), "+f"(v[14].x), "+f"(v[14].y), "+f"(v[15].x), "+f"(v[15].y)
                 :
                 : "memory");
}

// 16 consecutive columns as 8 float2, load and wait in one statement / store (tmem_wait_st() before they are read back).
__device__ __forceinline__ void tmem_ld16_sync(uint32_t taddr, float2 (&v)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=f"(v[0].x), "=f"(v[0].y), "=f"(v[1].x), "=f"(v[1].y), "=f"(v[2].x), "=f"(v[2].y), "=f"(v[3].x), "=f"(v[3].y),
          "=f"(v[4].x), "=f"(v[4].y), "=f"(v[5].x), "=f"(v[5].y), "=f"(v[6].x), "=f"(v[6].y), "=f"(v[7].x), "=f"(v[7].y)
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float2 (&v)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "f"(v[0].x), "f"(v[0].y), "f"(v[1].x), "f"(v[1].y), "f"(v[2].x), "f"(v[2].y), "f"(v[3].x), "f"(v[3].y), "f"(v[4].x),
        "f"(v[4].y), "f"(v[5].x), "f"(v[5].y), "f"(v[6].x), "f"(v[6].y), "f"(v[7].x), "f"(v[7].y)
        : "memory");
}

// 16 consecutive columns issued without waiting; tmem_wait_ld() then reg_fence8() before the first use.
__device__ __forceinline__ void tmem_ld16_async(uint32_t taddr, float2 (&v)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=f"(v[0].x), "=f"(v[0].y), "=f"(v[1].x), "=f"(v[1].y), "=f"(v[2].x), "=f"(v[2].y), "=f"(v[3].x), "=f"(v[3].y),
          "=f"(v[4].x), "=f"(v[4].y), "=f"(v[5].x), "=f"(v[5].y), "=f"(v[6].x), "=f"(v[6].y), "=f"(v[7].x), "=f"(v[7].y)
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void reg_fence8(float2 (&v)[8]) {
    asm volatile(""
                 : "+f"(v[0].x), "+f"(v[0].y), "+f"(v[1].x), "+f"(v[1].y), "+f"(v[2].x), "+f"(v[2].y), "+f"(v[3].x), "+f"(v[3].y),
                   "+f"(v[4].x), "+f"(v[4].y), "+f"(v[5].x), "+f"(v[5].y), "+f"(v[6].x), "+f"(v[6].y), "+f"(v[7].x), "+f"(v[7].y)
                 :
                 : "memory");
}

// 8 consecutive columns as 4 float2: load issued without waiting (tmem_wait_ld() then reg_fence4() before the first
// use) / store.
__device__ __forceinline__ void tmem_ld8_async(uint32_t taddr, float2 (&v)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=f"(v[0].x), "=f"(v[0].y), "=f"(v[1].x), "=f"(v[1].y), "=f"(v[2].x), "=f"(v[2].y), "=f"(v[3].x), "=f"(v[3].y)
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const float2 (&v)[4]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "f"(v[0].x), "f"(v[0].y),
                 "f"(v[1].x), "f"(v[1].y), "f"(v[2].x), "f"(v[2].y), "f"(v[3].x), "f"(v[3].y)
                 : "memory");
}
__device__ __forceinline__ void reg_fence4(float2 (&v)[4]) {
    asm volatile("" : "+f"(v[0].x), "+f"(v[0].y), "+f"(v[1].x), "+f"(v[1].y), "+f"(v[2].x), "+f"(v[2].y), "+f"(v[3].x), "+f"(v[3].y) : : "memory");
}

// 32 consecutive columns of this thread's lane set to one value.
__device__ __forceinline__ void tmem_fill32(uint32_t taddr, uint32_t v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr),
        "r"(v)
        : "memory");
}

// The same from a block of registers the caller keeps alive: tcgen05.st takes consecutive registers, so a single value
// would be copied into as many registers before every store.  fill_block_init() makes the block; the `volatile` moves
// keep the compiler from folding it back into one register.
constexpr int FILL_BLOCK = UNICA_FILL_BLOCK;
__device__ __forceinline__ void fill_block_init(uint32_t (&r)[FILL_BLOCK], uint32_t v) {
#pragma unroll
    for (int i = 0; i < FILL_BLOCK; ++i) asm volatile("mov.b32 %0, %1;" : "=r"(r[i]) : "r"(v));
}
__device__ __forceinline__ void tmem_fill_block(uint32_t taddr, const uint32_t (&r)[FILL_BLOCK]) {
#if UNICA_FILL_BLOCK == 16
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
                 "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
                 "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
#else
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]),
                 "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
#endif
}
// `columns` (a multiple of FILL_BLOCK) consecutive columns of this thread's lane set to the block's value.
template <int COLUMNS>
__device__ __forceinline__ void tmem_fill(uint32_t taddr, const uint32_t (&r)[FILL_BLOCK]) {
#pragma unroll
    for (int c = 0; c < COLUMNS; c += FILL_BLOCK) tmem_fill_block(taddr + c, r);
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// ---------------------------------------------------------------------------------------------------------------------
// tcgen05.mma operands

// Shared-memory matrix descriptor, no swizzle, K-major.  The operand is stored as core matrices of 8 rows x 16 bytes,
// each 128 contiguous bytes; `k_step_bytes` separates the two core matrices one instruction reads along K (the
// "leading" offset), `row_group_bytes` separates groups of 8 rows (the "stride" offset).
__device__ __forceinline__ uint64_t smem_desc(uint32_t smem_addr, uint32_t k_step_bytes, uint32_t row_group_bytes) {
    uint64_t d = 0;
    d |= uint64_t((smem_addr >> 4) & 0x3fff);
    d |= uint64_t((k_step_bytes >> 4) & 0x3fff) << 16;
    d |= uint64_t((row_group_bytes >> 4) & 0x3fff) << 32;
    d |= uint64_t(1) << 46;  // descriptor version of this architecture
    return d;                // base offset 0, layout type 0: no swizzle
}

// Instruction descriptor of kind::i8: D s32; A u8 or s8; B s8; both K-major; M x N.
__host__ __device__ constexpr uint32_t idesc_i8(bool a_signed, int m, int n) {
    return (2u << 4) | (uint32_t(a_signed) << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// Instruction descriptor of kind::tf32: D f32; A and B tf32 (32-bit words whose low 13 bits the tensor core ignores);
// both K-major; M x N.  The operand images have the byte geometry of the 8-bit ones: 16 bytes (four values) per row and
// chunk, an instruction takes K = 8 values = two chunks.
__host__ __device__ constexpr uint32_t idesc_tf32(int m, int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}
__device__ __forceinline__ void mma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate))
        : "memory");
}
// x = hi + lo up to 2^-24 |x|, both with tf32's 11 significant bits (round to nearest): three tf32 products
// hi.hi + lo.hi + hi.lo then carry an FP32 product to about 2^-22.
__device__ __forceinline__ void tf32_split(float x, float& hi, float& lo) {
    uint32_t bits;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bits) : "f"(x));
    hi = __uint_as_float(bits);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bits) : "f"(x - hi));  // the difference is exact
    lo = __uint_as_float(bits);
}

// D[tmem] (+)= A[smem] . B[smem]^T, issued by one thread.
__device__ __forceinline__ void mma_i8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate))
        : "memory");
}

// True in exactly one lane of a converged warp.  tcgen05.mma and tcgen05.commit take their operands from uniform
// registers: issued under `if (elect_one())` by a warp whose control flow is otherwise uniform they cost a few cycles;
// issued by one lane of a diverged warp (`if (lane == 0) { loop }`) each costs ~190 cycles (measured), because every
// operand is then moved into the uniform file the slow way.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{ .reg .b32 r; .reg .pred p; elect.sync r|p, 0xffffffff; selp.b32 %0, 1, 0, p; }" : "=r"(pred));
    return pred != 0;
}

// The mbarrier gets one arrival once every tcgen05.mma this thread issued before has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---------------------------------------------------------------------------------------------------------------------
// arithmetic helpers

// Packed FP32: one instruction for two lanes of a float2 (sm_100 has FFMA2 / FADD2 / FMUL2).
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)),
          "l"(reinterpret_cast<unsigned long long&>(c)));
    return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 d;
    asm("add.rn.f32x2 %0, %1, %2;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
    return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 d;
    asm("mul.rn.f32x2 %0, %1, %2;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// An s32 accumulator that starts at MAGIC_BITS instead of 0 reads back as the float MAGIC + value, exactly, for
// |value| < 2^22: the conversion to float costs one FADD instead of an I2F on the quarter-rate conversion pipe.
// Adding MAGIC to a float in [0, 2^22) likewise leaves its round-half-even integer in the low mantissa bits.
constexpr uint32_t MAGIC_BITS = 0x4B400000u;
constexpr float MAGIC = 12582912.0f;  // 1.5 * 2^23

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace unica
