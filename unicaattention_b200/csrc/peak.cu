// Peak-rate micro-benchmarks: what one SM sustains for the instructions the attention kernels are made of, so that their
// speed can be held against measured ceilings instead of datasheet ones (the reference does the same for its mma.sync
// forms: csrc/peak.cu, bench/peak.py).  One block per SM.
//
//   tensor kinds: a chain of tcgen05.mma on shared-memory operands in this library's layout (K-major, no swizzle),
//                 round-robin over the accumulators that fit in tensor memory, one commit at the end
//   scalar kinds: 8 independent chains per thread of one instruction, 4 warps per scheduler
#include "capi.h"
#include "fp4_common.cuh"

namespace unica {

enum PeakKind { PEAK_I8 = 0, PEAK_NVF4 = 1, PEAK_EX2 = 2, PEAK_FMA2 = 3, PEAK_FMA = 4, PEAK_PRMT = 5, PEAK_I2F = 6, PEAK_F2I = 7 };

// cycles[block] = clock64 span of `count` MMAs of shape 128 x n x (32 for i8, 64 for nvf4).
__global__ void __launch_bounds__(128) peak_mma_kernel(int kind, int n, int count, int layout_type, int run_length, long long* cycles, int* status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];  // A: 128 rows x 32 bytes, B: n rows x 32 bytes (zeros)
    __shared__ uint64_t done;
    __shared__ uint32_t tmem_base;
    __shared__ int abort_flag;
    for (int i = threadIdx.x; i < ((128 + n) * 128 + 1024) / 16; i += 128) reinterpret_cast<uint4*>(smem_raw)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_proxy_async();
    if (threadIdx.x / 32 == 0) tmem_alloc(&tmem_base, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base;
    // scale bytes (nvf4): zeros everywhere would do, but keep them defined: columns 480..511
    for (int c = 480; c < 512; c += 1) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(tmem + (uint32_t(threadIdx.x / 32 * 32) << 16) + c), "r"(0x38383838u) : "memory");
    }
    tmem_wait_st();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (threadIdx.x / 32 == 0) {  // the whole warp runs the loop; one elected lane issues (see elect_one)
        const int m = layout_type >= 10 ? 64 : 128;  // diagnostic: 10 + layout type times M = 64
        if (layout_type >= 10) layout_type -= 10;
        uint64_t a = smem_desc(smem_u32(smem_raw), 128 * 16, 128), b = smem_desc(smem_u32(smem_raw) + 128 * 32, n * 16, 128);
        if (layout_type) {  // timing only (operands are zeros): a swizzled layout type, rows of 8 x 16 bytes apart
            a = (smem_desc(smem_u32(smem_raw), 16, layout_type == 2 ? 1024 : layout_type == 4 ? 512 : 256) | (uint64_t(layout_type) << 61));
            b = (smem_desc(smem_u32(smem_raw) + 128 * 32, 16, layout_type == 2 ? 1024 : layout_type == 4 ? 512 : 256) | (uint64_t(layout_type) << 61));
        }
        const int accumulators = run_length ? 480 / n : 1;  // which accumulator: changes every `run_length` MMAs (0: never)
        const uint32_t idesc = kind == PEAK_I8 ? idesc_i8(true, m, n) : idesc_nvf4(m, n);
        const long long t0 = clock64();
        if (elect_one()) {  // one elected lane runs the whole chain
            int run = 0, slot = 0;
            for (int i = 0; i < count; ++i) {
                const uint32_t d = tmem + slot * n;
                if (kind == PEAK_I8)
                    mma_i8_ss(d, a, b, idesc, true);
                else
                    mma_nvf4_ss(d, a, b, idesc, tmem + 480, tmem + 488, true);
                if (run_length && ++run == run_length) {
                    run = 0;
                    slot = slot + 1 == accumulators ? 0 : slot + 1;
                }
            }
            mma_commit(&done);
        }
        __syncwarp();
        const bool ok = mbar_wait_warp(&done, 0, &abort_flag, status, STATUS_WAIT_SCORES);
        if (threadIdx.x == 0) cycles[blockIdx.x] = ok ? clock64() - t0 : -1;
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x / 32 == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// cycles[block] = clock64 span of `iters` x 8 independent instructions per thread, 512 threads (4 warps per scheduler).
__global__ void __launch_bounds__(512) peak_scalar_kernel(int kind, int iters, long long* cycles, float* sink, float seed) {
    float2 v[8];
    unsigned u[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = make_float2(seed + i + threadIdx.x * 1e-3f, seed * 0.5f + i), u[i] = threadIdx.x * 7 + i;
    const float2 c2 = make_float2(1.0001f, 0.9999f), d2 = make_float2(1e-3f, -1e-3f);
    __syncthreads();
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (kind == PEAK_EX2) v[i].x = ex2(v[i].x);
            if (kind == PEAK_FMA2) v[i] = fma2(v[i], c2, d2);
            if (kind == PEAK_FMA) v[i].x = fmaf(v[i].x, 1.0001f, 1e-3f);
            if (kind == PEAK_PRMT) u[i] = __byte_perm(u[i], u[(i + 1) % 8], 0x5410);
            if (kind == PEAK_I2F) v[i].x = __int2float_rn(__float_as_int(v[i].x));
            if (kind == PEAK_F2I) u[i] = __float2uint_rn(__uint_as_float(u[i]));
        }
    }
    const long long t1 = clock64();
    float acc = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += v[i].x + v[i].y + u[i];
    sink[blockIdx.x * blockDim.x + threadIdx.x] = acc;
    if (threadIdx.x == 0) cycles[blockIdx.x] = t1 - t0;
}

}  // namespace unica

using namespace unica;

// kind 0: tcgen05 kind::i8 (128 x n x 32), 1: kind::mxf4nvf4 (128 x n x 64), 2..7: ex2, fma.f32x2, fma.f32, prmt, cvt s32->f32,
// cvt f32->u32.  Runs `blocks` blocks (one per SM is the point) and returns the MEDIAN block's cycles per instruction
// (tensor kinds: per MMA; scalar kinds: per warp instruction per scheduler) in *cycles_per_instruction.
// Allocates scratch and synchronises: a measurement tool, not part of the hot path.
extern "C" int unica_b200_peak(int kind, int n, int count, int blocks, double* cycles_per_instruction, void* stream) {
    if (!cycles_per_instruction || count <= 0 || blocks <= 0 || blocks > 1024) return unica_fail(UNICA_B200_ERR_ARGUMENT, "peak: bad arguments");
    if (kind % 100 < 0 || kind % 100 > PEAK_F2I) return unica_fail(UNICA_B200_ERR_ARGUMENT, "peak: unknown kind");
    if (kind % 100 <= PEAK_NVF4 && (n < 16 || n > 240 || n % 16)) return unica_fail(UNICA_B200_ERR_ARGUMENT, "peak: n must be a multiple of 16 in 16..240");
    if (kind % 100 <= PEAK_NVF4) {  // the descriptor's layout-type field takes these values only; + 10: the same with M = 64
        const int layout = kind / 100 % 100 % 10, m64 = kind / 100 % 100 / 10;
        if (m64 > 1 || (layout != 0 && layout != 1 && layout != 2 && layout != 4 && layout != 6))
            return unica_fail(UNICA_B200_ERR_ARGUMENT, "peak: the layout digit must be 0, 1, 2, 4 or 6 (plus 10 for M = 64)");
    } else if (kind >= 100) {
        return unica_fail(UNICA_B200_ERR_ARGUMENT, "peak: scalar kinds take no variant digits");
    }
    if (int e = unica_check_device()) return e;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    long long* cycles = nullptr;
    float* sink = nullptr;
    int* status = nullptr;
    auto release = [&]() { cudaFree(cycles), cudaFree(sink), cudaFree(status); };  // cudaFree(nullptr) is a no-op
    if (cudaMalloc(&cycles, sizeof(long long) * blocks) != cudaSuccess || cudaMalloc(&sink, sizeof(float) * blocks * 512) != cudaSuccess ||
        cudaMalloc(&status, sizeof(int)) != cudaSuccess || cudaMemsetAsync(status, 0, sizeof(int), s) != cudaSuccess) {
        const int e = unica_check_launch("peak (scratch)");
        release();
        return e;
    }
    for (int rep = 0; rep < 2; ++rep) {  // the second run is the measured one
        if (kind % 100 <= PEAK_NVF4)
            peak_mma_kernel<<<blocks, 128, (128 + n) * 128 + 1024 + 128, s>>>(kind % 100, n, count, kind / 100 % 100, kind / 10000, cycles, status);
        else
            peak_scalar_kernel<<<blocks, 128 * (n >= 1 && n <= 4 ? n : 4), 0, s>>>(kind, count, cycles, sink, 0.3f);  // n: warps per scheduler
    }
    long long host[1024];
    cudaError_t e = cudaMemcpyAsync(host, cycles, sizeof(long long) * blocks, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    release();
    if (e != cudaSuccess) return unica_fail(UNICA_B200_ERR_CUDA, cudaGetErrorString(e));
    for (int i = 1; i < blocks; ++i)  // insertion sort: blocks <= 1024
        for (int j = i; j > 0 && host[j - 1] > host[j]; --j) {
            const long long t = host[j];
            host[j] = host[j - 1], host[j - 1] = t;
        }
    const long long median = host[blocks / 2];
    if (median < 0) return unica_fail(UNICA_B200_ERR_KERNEL, "peak: the tensor-core chain never completed");
    // scalar kinds: 8 chains x 4 warps per scheduler -> per warp instruction per scheduler
    *cycles_per_instruction = kind % 100 <= PEAK_NVF4 ? double(median) / count : double(median) / (double(count) * 8 * (n >= 1 && n <= 4 ? n : 4));
    return UNICA_B200_OK;
}
