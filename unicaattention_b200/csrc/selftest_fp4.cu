// Self-test of the block-scaled FP4 tensor-core path: one tcgen05.mma kind::mxf4nvf4 chain on operand images and scale
// bytes given by the caller; with small values every product and sum is exact in float, so a wrong nibble order,
// scale position or layout cannot hide (the idea of the reference's tests/test_mma.py).
#include "capi.h"
#include "fp4_common.cuh"

namespace unica {

// a_image [k / 32][128][16], b_image [k / 32][n][16] (two codes per byte); sfa [k / 64][128] words, sfb [k / 64][n]
// words (byte i of a word scales elements 16 i .. 16 i + 15 of that K step); d float [128][n].
// variant 0: scale words stored into tensor memory by the threads (tcgen05.st); 2: A's copied from shared memory by
// the issuing thread (tcgen05.cp); 1: a deliberately wrong layout (diagnostic).
__global__ void __launch_bounds__(128) selftest_mma_nvf4_kernel(const uint8_t* __restrict__ a_image, const uint8_t* __restrict__ b_image,
                                                                const uint32_t* __restrict__ sfa, const uint32_t* __restrict__ sfb,
                                                                int n, int k, int variant, float* __restrict__ d, int* status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* a_s = smem_raw;               // 64 k bytes
    uint8_t* b_s = smem_raw + 64 * k;      // n k / 2 bytes
    __shared__ uint64_t done;
    __shared__ uint32_t tmem_base;
    __shared__ int abort_flag;
    __shared__ __align__(128) uint32_t sfa_s[2][32][4];  // variant 2: A's scale words as tcgen05.cp takes them, [K step][lane][row / 32]
    if (variant == 2)
        for (int i = threadIdx.x; i < (k / 64) * 128; i += 128) sfa_s[i / 128][i % 32][i % 128 / 32] = sfa[i];
    for (int i = threadIdx.x; i < 64 * k / 16; i += 128) reinterpret_cast<uint4*>(a_s)[i] = reinterpret_cast<const uint4*>(a_image)[i];
    for (int i = threadIdx.x; i < n * k / 32; i += 128) reinterpret_cast<uint4*>(b_s)[i] = reinterpret_cast<const uint4*>(b_image)[i];
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_proxy_async();
    if (threadIdx.x / 32 == 0) tmem_alloc(&tmem_base, 256);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t my = tmem + (uint32_t(warp * 32) << 16);
    const int k_steps = k / 64, b_cols = (n + 31) / 32;
    const uint32_t col_sfa = 160, col_sfb = 192;  // D takes columns 0 .. n - 1 (n <= 160)
    // scale bytes into tensor memory: every 32-lane quarter holds all rows
    for (int s = 0; s < k_steps; ++s) {
        if (variant == 0)  // variant 2: A's scale words are copied from shared memory by the issuing thread below
            tmem_st4(my + col_sfa + 4 * s, sfa[s * 128 + lane], sfa[s * 128 + 32 + lane], sfa[s * 128 + 64 + lane], sfa[s * 128 + 96 + lane]);
        for (int c = 0; c < b_cols; ++c) {
            const int row = 32 * c + lane;
            tmem_st1(my + col_sfb + b_cols * s + c, row < n ? sfb[s * n + row] : 0u);
        }
    }
    tmem_wait_st();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (threadIdx.x == 0) {
        const uint32_t idesc = idesc_nvf4(128, n);
        if (variant == 2)
            for (int s = 0; s < k_steps; ++s) tmem_cp_32x128b(tmem + col_sfa + 4 * s, smem_u32(&sfa_s[s][0][0]));
        for (int s = 0; s < k_steps; ++s)
            mma_nvf4_ss(tmem, smem_desc(smem_u32(a_s) + s * 2 * 128 * 16, 128 * 16, 128), smem_desc(smem_u32(b_s) + s * 2 * n * 16, n * 16, 128),
                        idesc, tmem + col_sfa + 4 * s, tmem + col_sfb + b_cols * s, s > 0);
        mma_commit(&done);
    }
    const bool ok = mbar_wait_warp(&done, 0, &abort_flag, status, STATUS_WAIT_SCORES);
    tc_fence_after();
    if (ok) {
        for (int c0 = 0; c0 < n; c0 += 16) {
            uint32_t r[16];
            tmem_ld16(my + c0, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (c0 + i < n) d[threadIdx.x * n + c0 + i] = __uint_as_float(r[i]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x / 32 == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, 256);
    }
}

}  // namespace unica

using namespace unica;

extern "C" int unica_b200_selftest_mma_nvf4(const void* a_image, const void* b_image, const void* sfa, const void* sfb, int n, int k,
                                            int variant, float* d, void* stream) {
    if (!a_image || !b_image || !sfa || !sfb || !d) return unica_fail(UNICA_B200_ERR_ARGUMENT, "selftest_mma_nvf4: null pointer");
    if (n < 16 || n > 160 || n % 16 || (k != 64 && k != 128))
        return unica_fail(UNICA_B200_ERR_ARGUMENT, "selftest_mma_nvf4: n must be a multiple of 16 in 16..160, k 64 or 128");
    if (variant != 0 && variant != 2) return unica_fail(UNICA_B200_ERR_ARGUMENT, "selftest_mma_nvf4: variant must be 0 or 2");
    if (int e = unica_check_device()) return e;
    const size_t smem = size_t(128 + n) * k / 2 + 128;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int* status = nullptr;
    if (cudaMalloc(&status, sizeof(int)) != cudaSuccess || cudaMemsetAsync(status, 0, sizeof(int), s) != cudaSuccess) {
        const int e = unica_check_launch("selftest_mma_nvf4 (status word)");
        cudaFree(status);  // a no-op when the allocation itself failed
        return e;
    }
    selftest_mma_nvf4_kernel<<<1, 128, smem, s>>>(static_cast<const uint8_t*>(a_image), static_cast<const uint8_t*>(b_image),
                                                  static_cast<const uint32_t*>(sfa), static_cast<const uint32_t*>(sfb), n, k, variant, d, status);
    int host_status = 0;
    cudaError_t e = cudaMemcpyAsync(&host_status, status, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaFree(status);
    if (e != cudaSuccess) return unica_fail(UNICA_B200_ERR_CUDA, cudaGetErrorString(e));
    if (host_status) return unica_fail(UNICA_B200_ERR_KERNEL, "selftest_mma_nvf4: the tensor-core instruction never completed");
    return UNICA_B200_OK;
}
