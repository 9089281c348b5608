// The INT8 quantizers as streaming kernels: persistent blocks that pull 64-token tiles through a ring of shared-memory
// stages with cp.async (several tiles in flight per block whatever the arithmetic is doing), for
//   Q: codes with a scale per 128 queries, one pass;
//   K: the mean over the tokens, then codes of k - mean with a scale per 64 keys;
//   V: minimum and maximum per channel over the tokens, then codes with a scale per channel.
// For K and V the separate passes (quantize.cu) read the operand from HBM twice, once for the statistics and once to
// quantize.  Here both happen in one launch and the second read comes out of L2: only a few heads are in flight at a
// time (a head of 32760 tokens is 8.4 MB of the 126 MB), and a head's blocks go back over the very tokens they have just
// read.
//
// K and V: one persistent block per resident slot (cooperative launch, so that all blocks are on the GPU together), dealt
// into `groups` groups of `per_group` blocks; group g takes heads g, g + groups, ...  Per head a block
//   1. adds up sum, min and max per channel over its share of the head's tiles and leaves them in `partial`,
//   2. takes a ticket; the block with the last ticket of the round adds all partials of the group in block order (so the
//      result does not depend on who came last), publishes the head's statistics and raises the group's `ready` count;
//      the others wait for that count (bounded: on a time-out they set the status word and give up),
//   3. quantizes its tiles with the tile routines of quantize_int8.cuh.
// The ring does not stop at the wait: the tiles of step 3 are on their way while the block waits in step 2.
// Numerics are those of the separate passes except for the order in which a mean's terms are added.  That order is fixed
// here too: a head's tiles are dealt to `per_group` blocks, and `per_group` follows from the device and the token count
// alone, not from how many heads the call holds, so a head's operands do not depend on what it is quantized with.
#include "capi.h"
#include "quantize_int8.cuh"

namespace unica {

constexpr int STREAM_THREADS = 512;  // two blocks of 16 warps per SM at 64 registers a thread
constexpr int FUSED_LANES = STREAM_THREADS / 16;  // token lanes: thread = (lane, chunk of 8 channels)
constexpr int FUSED_MAX_GROUPS = 12;  // heads in flight at most: more would only thin out the blocks a head gets
constexpr int RING_STAGES = 4;                       // tiles in flight per block: three ahead of the one in hand
constexpr int RING_TILE_BYTES = KEY_TILE * HEAD_DIM * 2;  // 16 KB
constexpr int RING_BYTES = RING_STAGES * RING_TILE_BYTES;

struct FusedScratch {  // carved out of the caller's scratch buffer
    float* partial;      // [groups][per_group][3][128]
    float* head_stats;   // [groups][3][128]: mean, min, max of the head the group is on
    unsigned* counters;  // [groups][2]: tickets taken, heads published
};

__device__ __forceinline__ unsigned load_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void store_release(unsigned* p, unsigned v) { asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }

// A thread's share of every tile copy: the same two 16-byte pieces (row, piece of the row) of each tile, so their offsets
// in the stage and from the tile's first token are worked out once.
struct FetchLane {
    uint32_t in_stage[KEY_TILE * 16 / STREAM_THREADS];
    long long from_tile[KEY_TILE * 16 / STREAM_THREADS];  // in elements
    int row[KEY_TILE * 16 / STREAM_THREADS];
    __device__ __forceinline__ explicit FetchLane(long long token_stride) {
#pragma unroll
        for (int it = 0; it < KEY_TILE * 16 / STREAM_THREADS; ++it) {
            const int piece = it * STREAM_THREADS + threadIdx.x, piece16 = piece % 16;
            row[it] = piece / 16;
            in_stage[it] = staged_offset(row[it], piece16);
            from_tile[it] = row[it] * token_stride + piece16 * 8;
        }
    }
};
// 64 tokens x 256 bytes into a stage (laid out as staged_chunk describes), 16 bytes per copy, two copies per thread; rows
// past the last token arrive as zeros.  tile_base: the tile's first token (token0) in the head.
__device__ __forceinline__ void ring_fetch(uint8_t* stage, const __nv_bfloat16* __restrict__ tile_base, int token0, int n_tokens,
                                           const FetchLane& lane) {
    const uint32_t stage_address = smem_u32(stage);
#pragma unroll
    for (int it = 0; it < KEY_TILE * 16 / STREAM_THREADS; ++it) {
        const bool valid = token0 + lane.row[it] < n_tokens;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(stage_address + lane.in_stage[it]),
                     "l"(valid ? tile_base + lane.from_tile[it] : tile_base), "r"(valid ? 16 : 0)
                     : "memory");
    }
}
__device__ __forceinline__ void ring_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// at most RING_STAGES - 2 of the newest groups still in flight: the tile in hand has arrived (for this thread's copies)
__device__ __forceinline__ void ring_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(RING_STAGES - 2) : "memory"); }

// Q: [heads][tiles of 128 queries], one scale per tile; rows past n_tokens and tiles past the last are zeros.
// Persistent blocks take (head, tile) pairs blockIdx.x, blockIdx.x + gridDim.x, ...; a tile is two stages of the ring.
// HALF: the input is float16 (a template parameter so that the bfloat16 path carries none of the conversion).
template <bool HALF>
__global__ void __launch_bounds__(STREAM_THREADS, 2) quantize_q_int8_stream_kernel(const __nv_bfloat16* __restrict__ x, TokenLayout in, int heads,
                                                                          int n_tokens, int tiles, int8_t* __restrict__ codes,
                                                                          float* __restrict__ scales) {
    in.half = HALF;
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ float scratch_max[STREAM_THREADS / 32];
    // 32-bit counters throughout: the host checks that heads * tiles fits, and 64-bit divisions here would cost more than
    // the quantization itself
    const int mine = (heads * tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x);  // this block's tiles
    const FetchLane lane(in.token);
    int fetched = 0, fetch_t = 0;  // half tiles whose copies have been started; the tile of the head the next one is in
    const __nv_bfloat16* fetch_head = x;
    auto fetch = [&]() {  // the next half tile of 64 queries
        if (fetched < 2 * mine) {
            if (fetched % 2 == 0) {  // a new tile: one division for both halves
                const int tile = int(blockIdx.x) + (fetched / 2) * int(gridDim.x), head = tile / tiles;
                fetch_t = tile - head * tiles;
                fetch_head = x + in.offset(head, 0);
            }
            const int token0 = fetch_t * 128 + (fetched % 2) * KEY_TILE;
            ring_fetch(ring + (fetched % RING_STAGES) * RING_TILE_BYTES, fetch_head + token0 * in.token, token0, n_tokens, lane);
        }
        ++fetched;
        ring_commit();
    };
    static_assert(RING_STAGES == 4, "a tile in hand and a tile in flight, two stages each");
    for (int i = 0; i < RING_STAGES; ++i) fetch();
    for (int i = 0; i < mine; ++i) {
        ring_wait();  // all but the two newest groups: both halves of this tile are there
        __syncthreads();
        const int tile = int(blockIdx.x) + i * int(gridDim.x), head = tile / tiles, t = tile - head * tiles;
        rows_int8_tile<128, STREAM_THREADS>(x, in, nullptr, head, t, n_tokens, codes + size_t(tile) * (128 * HEAD_DIM), scales + tile,
                                            RopeTable{nullptr, 0}, scratch_max,
                                            reinterpret_cast<const __nv_bfloat16*>(ring + (2 * i % RING_STAGES) * RING_TILE_BYTES));
        __syncthreads();  // its two stages are free
        fetch();
        fetch();
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
}

// IS_V false: x = K, out_codes K8 [heads][tiles][8][64][16], out_scale [heads][tiles], out_stat = the means [heads][128].
// IS_V true: x = V, out_codes V8 [heads][tiles][4][128][16], out_scale = v_scale [heads][128], out_stat unused.
template <bool IS_V, bool HALF>
__global__ void __launch_bounds__(STREAM_THREADS, 2) quantize_head_int8_kernel(const __nv_bfloat16* __restrict__ x, TokenLayout in, int heads,
                                                                      int n_tokens, int tiles, int groups, int per_group,
                                                                      FusedScratch scratch, int8_t* __restrict__ out_codes,
                                                                      float* __restrict__ out_scale, float* __restrict__ out_stat,
                                                                      int* status) {
    in.half = HALF;
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ float lanes[2][FUSED_LANES][HEAD_DIM];  // 32 KB: per-lane sums (K) or minima and maxima (V) on their way to one row
    __shared__ float head_stats[3][HEAD_DIM];          // mean, min, max of the head in hand
    __shared__ float scratch_max[STREAM_THREADS / 32];
    __shared__ unsigned ticket_s;
    __shared__ int gave_up;
    const int group = blockIdx.x / per_group, member = blockIdx.x % per_group;
    if (group >= groups) return;  // the blocks left over after the division
    const int chunk = threadIdx.x % 16, lane = threadIdx.x / 16;
    const int tile0 = int(static_cast<long long>(tiles) * member / per_group), tile1 = int(static_cast<long long>(tiles) * (member + 1) / per_group);
    const int mine = tile1 - tile0;  // this block's tiles of every head of its group
    const int rounds = (heads - group + groups - 1) / groups;
    float* my_partial = scratch.partial + (size_t(group) * per_group + member) * 3 * HEAD_DIM;
    float* group_stats = scratch.head_stats + size_t(group) * 3 * HEAD_DIM;
    unsigned* tickets = scratch.counters + 2 * group;
    unsigned* ready = tickets + 1;
    if (threadIdx.x == 0) gave_up = 0;

    // The block's stream of tiles: per head its tiles once for the statistics, then once more to be quantized.  The fetches
    // walk it with counters of their own (no divisions on the way).
    const FetchLane copies(in.token);
    const long long tile_step = KEY_TILE * in.token;
    int fetch_round = 0, fetch_pass = 0, fetch_tile = tile0, fetched = 0;
    const __nv_bfloat16* fetch_first = x + in.offset(group, 0) + tile0 * tile_step;  // the block's first tile of the head
    const __nv_bfloat16* fetch_at = fetch_first;
    auto fetch = [&]() {
        if (fetch_round < rounds && mine > 0) {
            ring_fetch(ring + (fetched % RING_STAGES) * RING_TILE_BYTES, fetch_at, fetch_tile * KEY_TILE, n_tokens, copies);
            fetch_at += tile_step;
            if (++fetch_tile == tile1) {
                fetch_tile = tile0;
                if (++fetch_pass == 2) {
                    fetch_pass = 0;
                    if (++fetch_round < rounds) fetch_first = x + in.offset(group + fetch_round * groups, 0) + tile0 * tile_step;
                }
                fetch_at = fetch_first;
            }
        }
        ++fetched;
        ring_commit();
    };
    auto arrived = [&](int i) -> const uint8_t* {  // waits for tile i of the stream, starts the fetch three ahead
        ring_wait();
        __syncthreads();  // everybody's copies of tile i are there, and everybody is done with tile i - 1, whose stage goes next
        fetch();
        return ring + (i % RING_STAGES) * RING_TILE_BYTES;
    };
    for (int i = 0; i < RING_STAGES - 1; ++i) fetch();

    int at = 0;
    for (int round = 0; round < rounds; ++round) {
        const int head = group + round * groups;
        // ---- 1. this block's share of the statistics
        // K needs the sums only (in FP32), V the minima and maxima only, which are exact in any format: taken on the
        // bfloat16 pairs as they come, two elements per instruction.
        float2 sum[4];
        __nv_bfloat162 low[4], high[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            sum[i] = make_float2(0.0f, 0.0f);
            low[i] = __floats2bfloat162_rn(INFINITY, INFINITY);
            high[i] = __floats2bfloat162_rn(-INFINITY, -INFINITY);
        }
        for (int t = tile0; t < tile1; ++t, ++at) {
            const uint8_t* stage = arrived(at);
#pragma unroll
            for (int j = 0; j < KEY_TILE / FUSED_LANES; ++j) {
                const int row = lane + j * FUSED_LANES;
                if (t * KEY_TILE + row < n_tokens) {
                    const uint4 raw = load_bf16x8(reinterpret_cast<const __nv_bfloat16*>(stage + staged_offset(row, chunk)), in.half);
                    if (IS_V) {
                        const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                        for (int i = 0; i < 4; ++i) low[i] = __hmin2(low[i], pairs[i]), high[i] = __hmax2(high[i], pairs[i]);
                    } else {
                        float2 v[4];
                        unpack8(raw, v);
#pragma unroll
                        for (int i = 0; i < 4; ++i) sum[i] = add2(sum[i], v[i]);
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            *reinterpret_cast<float2*>(&lanes[0][lane][chunk * 8 + 2 * i]) = IS_V ? __bfloat1622float2(low[i]) : sum[i];
            *reinterpret_cast<float2*>(&lanes[1][lane][chunk * 8 + 2 * i]) = __bfloat1622float2(high[i]);
        }
        __syncthreads();
        if (threadIdx.x < HEAD_DIM) {
            float s = 0.0f, lo = INFINITY, hi = -INFINITY;
            for (int l = 0; l < FUSED_LANES; ++l) {
                if (IS_V) {
                    lo = fminf(lo, lanes[0][l][threadIdx.x]);
                    hi = fmaxf(hi, lanes[1][l][threadIdx.x]);
                } else {
                    s += lanes[0][l][threadIdx.x];
                }
            }
            my_partial[threadIdx.x] = s;
            my_partial[HEAD_DIM + threadIdx.x] = lo;
            my_partial[2 * HEAD_DIM + threadIdx.x] = hi;
            __threadfence();
        }
        __syncthreads();
        // ---- 2. the group's statistics: the last block of the round to get here adds them up, the others wait for it
        if (threadIdx.x == 0) ticket_s = atomicAdd(tickets, 1u);
        __syncthreads();
        if (ticket_s == unsigned(round + 1) * per_group - 1) {
            __threadfence();
            if (threadIdx.x < HEAD_DIM) {
                float s = 0.0f, lo = INFINITY, hi = -INFINITY;
                const float* p = scratch.partial + size_t(group) * per_group * 3 * HEAD_DIM + threadIdx.x;
                for (int b = 0; b < per_group; ++b, p += 3 * HEAD_DIM) {
                    s += __ldcg(p);
                    lo = fminf(lo, __ldcg(p + HEAD_DIM));
                    hi = fmaxf(hi, __ldcg(p + 2 * HEAD_DIM));
                }
                const float mean = s / float(n_tokens);
                group_stats[threadIdx.x] = mean;
                group_stats[HEAD_DIM + threadIdx.x] = lo;
                group_stats[2 * HEAD_DIM + threadIdx.x] = hi;
                if (IS_V)
                    out_scale[size_t(head) * HEAD_DIM + threadIdx.x] = fmaxf(fmaxf(hi, -lo) * (1.0f / 127.0f), 1e-12f);
                else
                    out_stat[size_t(head) * HEAD_DIM + threadIdx.x] = mean;
                __threadfence();
            }
            __syncthreads();
            if (threadIdx.x == 0) store_release(ready, unsigned(round + 1));
        } else if (threadIdx.x == 0) {
            const long long start = clock64();
            while (load_acquire(ready) < unsigned(round + 1)) {
                if (clock64() - start > WAIT_LIMIT_CYCLES || (status && *reinterpret_cast<volatile int*>(status) != 0)) {
                    if (status) atomicCAS(status, 0, int(STATUS_WAIT_GROUP));
                    gave_up = 1;
                    break;
                }
                __nanosleep(100);
            }
        }
        __syncthreads();
        if (gave_up) break;
        for (int i = threadIdx.x; i < 3 * HEAD_DIM; i += STREAM_THREADS) head_stats[i / HEAD_DIM][i % HEAD_DIM] = __ldcg(group_stats + i);
        __syncthreads();
        // ---- 3. this block's tiles again (out of L2), quantized
        for (int t = tile0; t < tile1; ++t, ++at) {
            const uint8_t* stage = arrived(at);
            if (IS_V) {
                v_int8_emit<false, STREAM_THREADS, true>(reinterpret_cast<const __nv_bfloat16(*)[HEAD_DIM]>(stage), in.half, nullptr, nullptr, head_stats[1], head_stats[2],
                                   head, t, tiles, out_codes, nullptr);
            } else {
                rows_int8_tile<KEY_TILE, STREAM_THREADS>(x, in, head_stats[0], head, t, n_tokens, out_codes + (size_t(head) * tiles + t) * (KEY_TILE * HEAD_DIM),
                                         out_scale + size_t(head) * tiles + t, RopeTable{nullptr, 0}, scratch_max,
                                         reinterpret_cast<const __nv_bfloat16*>(stage));
            }
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");  // no copy may still be writing this block's shared memory when it ends
}

}  // namespace unica

using namespace unica;

// Persistent blocks the device holds for `kernel` with the ring in shared memory: at most four per SM.
static int resident_blocks(const void* kernel, const char* name, int* blocks) {
    int device = 0, sms = 0, per_sm = 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, RING_BYTES) != cudaSuccess ||
        cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, STREAM_THREADS, RING_BYTES) != cudaSuccess)
        return unica_check_launch(name);
    if (per_sm < 1) return unica_fail(UNICA_B200_ERR_DEVICE, "quantize: the device cannot hold a block of the streaming quantizers");
    *blocks = sms * (per_sm < 4 ? per_sm : 4);
    return UNICA_B200_OK;
}

// Launch plan of the K and V kernels: how many persistent blocks, in how many groups.  A group is on one head at a time,
// so up to `groups` heads are in flight: as many as fit in about 96 MB of L2 with their output.  per_group must not depend
// on `heads` (see the top of the file), so a call with few heads leaves groups idle rather than spreading a head over
// more blocks.
static int fused_plan(const void* kernel, const char* name, int heads, int n_tokens, int* groups, int* per_group, int* grid) {
    int device = 0, cooperative = 0, blocks = 0;
    if (int e = resident_blocks(kernel, name, &blocks)) return e;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, device) != cudaSuccess)
        return unica_check_launch(name);
    if (!cooperative) return unica_fail(UNICA_B200_ERR_DEVICE, "quantize: the device has no cooperative launch");
    const long long head_bytes = static_cast<long long>(n_tokens) * HEAD_DIM * 3;  // read as 16 bits, written as 8
    long long in_flight = (96LL << 20) / head_bytes;
    in_flight = in_flight < 1 ? 1 : in_flight;
    in_flight = in_flight > FUSED_MAX_GROUPS ? FUSED_MAX_GROUPS : in_flight;
    in_flight = in_flight > blocks ? blocks : in_flight;
    *per_group = blocks / int(in_flight);
    const int rounds = int((heads + in_flight - 1) / in_flight);
    *groups = (heads + rounds - 1) / rounds;  // the same number of rounds with the heads spread evenly over them
    *grid = *groups * *per_group;
    return UNICA_B200_OK;
}

static int quantize_fused(bool is_v, const void* x, unica_token_layout layout, int heads, int n_tokens, int tiles, void* scratch,
                          size_t scratch_bytes, int8_t* codes, float* scales, float* stat, int* status, void* stream) {
    const char* name = is_v ? "quantize_v_int8_fused" : "quantize_k_int8_fused";
    if (!x || !scratch || !codes || !scales || (!is_v && !stat)) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize (one launch): null pointer");
    if (heads <= 0 || n_tokens <= 0) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize (one launch): heads and n_tokens must be positive");
    if (tiles != (n_tokens + KEY_TILE - 1) / KEY_TILE) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize (one launch): tiles must be ceil(n_tokens / 64)");
    if (static_cast<long long>(heads) * tiles > (1LL << 29)) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize (one launch): more than 2^29 tiles");
    if (scratch_bytes < UNICA_B200_FUSED_SCRATCH_BYTES || reinterpret_cast<uintptr_t>(scratch) % 16)
        return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize (one launch): scratch must be 16-byte aligned and hold UNICA_B200_FUSED_SCRATCH_BYTES");
    if (int e = unica_check_device()) return e;
    const bool half = layout.dtype == UNICA_B200_FLOAT16;
    const void* kernel = is_v ? (half ? reinterpret_cast<const void*>(quantize_head_int8_kernel<true, true>) : reinterpret_cast<const void*>(quantize_head_int8_kernel<true, false>))
                              : (half ? reinterpret_cast<const void*>(quantize_head_int8_kernel<false, true>) : reinterpret_cast<const void*>(quantize_head_int8_kernel<false, false>));
    int groups = 0, per_group = 0, grid = 0;
    if (int e = fused_plan(kernel, name, heads, n_tokens, &groups, &per_group, &grid)) return e;
    FusedScratch carve;
    carve.partial = static_cast<float*>(scratch);
    carve.head_stats = carve.partial + size_t(grid) * 3 * HEAD_DIM;
    carve.counters = reinterpret_cast<unsigned*>(carve.head_stats + size_t(groups) * 3 * HEAD_DIM);
    if (size_t(reinterpret_cast<char*>(carve.counters + 2 * groups) - static_cast<char*>(scratch)) > UNICA_B200_FUSED_SCRATCH_BYTES)
        return unica_fail(UNICA_B200_ERR_KERNEL, "quantize (one launch): the launch plan outgrew the scratch");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(carve.counters, 0, sizeof(unsigned) * 2 * groups, s) != cudaSuccess) return unica_check_launch(name);
    const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
    TokenLayout in = to_layout(layout);
    void* args[] = {&xb, &in, &heads, &n_tokens, &tiles, &groups, &per_group, &carve, &codes, &scales, &stat, &status};
    if (cudaLaunchCooperativeKernel(kernel, dim3(grid), dim3(STREAM_THREADS), args, RING_BYTES, s) != cudaSuccess) return unica_check_launch(name);
    return unica_check_launch(name);
}

extern "C" int unica_b200_quantize_k_int8_fused(const void* k, unica_token_layout layout, int heads, int n_tokens, int tiles, void* scratch,
                                                size_t scratch_bytes, int8_t* codes, float* scales, float* mean, int* status, void* stream) {
    return quantize_fused(false, k, layout, heads, n_tokens, tiles, scratch, scratch_bytes, codes, scales, mean, status, stream);
}

extern "C" int unica_b200_quantize_v_int8_fused(const void* v, unica_token_layout layout, int heads, int n_tokens, void* scratch,
                                                size_t scratch_bytes, int8_t* v8, float* v_scale, int* status, void* stream) {
    return quantize_fused(true, v, layout, heads, n_tokens, (n_tokens + KEY_TILE - 1) / KEY_TILE, scratch, scratch_bytes, v8, v_scale, nullptr,
                          status, stream);
}

extern "C" int unica_b200_quantize_q_int8_stream(const void* q, unica_token_layout layout, int heads, int n_tokens, int tiles, int8_t* codes,
                                                 float* scales, void* stream) {
    if (!q || !codes || !scales) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_q_int8_stream: null pointer");
    if (heads <= 0 || n_tokens <= 0) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_q_int8_stream: heads and n_tokens must be positive");
    if (tiles < (n_tokens + 127) / 128) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_q_int8_stream: tiles does not cover n_tokens");
    if (static_cast<long long>(heads) * tiles > (1LL << 30)) return unica_fail(UNICA_B200_ERR_ARGUMENT, "quantize_q_int8_stream: more than 2^30 tiles");
    if (int e = unica_check_device()) return e;
    int blocks = 0;
    const bool half = layout.dtype == UNICA_B200_FLOAT16;
    auto kernel = half ? quantize_q_int8_stream_kernel<true> : quantize_q_int8_stream_kernel<false>;
    if (int e = resident_blocks(reinterpret_cast<const void*>(kernel), "quantize_q_int8_stream", &blocks)) return e;
    const long long work = static_cast<long long>(heads) * tiles;
    const int grid = int(work < blocks ? work : blocks);
    kernel<<<grid, STREAM_THREADS, RING_BYTES, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(q), to_layout(layout), heads,
                                                                                      n_tokens, tiles, codes, scales);
    return unica_check_launch("quantize_q_int8_stream");
}
