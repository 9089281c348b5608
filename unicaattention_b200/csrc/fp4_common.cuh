// tcgen05 block-scaled FP4 helpers shared by the fast-mode kernel and its self-test.
#pragma once

#include "common.cuh"

namespace unica {

// Instruction descriptor of kind::mxf4nvf4: A and B e2m1, scales ue4m3 (one per 16 elements: scale_vec::4X), D f32,
// both K-major, M x N, K = 64 per instruction.
__host__ __device__ constexpr uint32_t idesc_nvf4(int m, int n) {
    return (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (0u << 23) | (uint32_t(m >> 4) << 24);
}

// D[tmem] (+)= (A . sfa) . (B . sfb)^T.  sfa / sfb: tensor-memory addresses of the scale bytes: row r of the operand has
// its four bytes (one per 16 elements of K) in lane r % 32 of column r / 32, the same in each of the four 32-lane quarters.
__device__ __forceinline__ void mma_nvf4_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa,
                                            uint32_t sfb, bool accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(uint32_t(accumulate))
        : "memory");
}

// n consecutive columns of this thread's lane from registers (n = 1, 2, 4).
__device__ __forceinline__ void tmem_st1(uint32_t taddr, uint32_t a) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(a) : "memory");
}
__device__ __forceinline__ void tmem_st2(uint32_t taddr, uint32_t a, uint32_t b) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};" ::"r"(taddr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Scale bytes from shared memory into tensor memory by the tensor-core pipe itself: 32 rows of 16 bytes at `src`
// (row i = the four 32-bit words that lane i of columns taddr .. taddr + 3 gets), copied into all four 32-lane quarters.
// Issued by one thread; ordered with the tcgen05.mma that the same thread issues after it.
__device__ __forceinline__ void tmem_cp_32x128b(uint32_t taddr, uint32_t src) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc(src, 16, 128)) : "memory");
}

}  // namespace unica
