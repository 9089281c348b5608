/* unica_b200: C ABI of the B200 (sm_100a) forward quantized attention.
 *
 * The reference reaches its kernels through the CUDA driver API from Python: `module("flash")[name](grid, block, *args)`
 * looks an `extern "C" __global__` symbol up by name and launches it with positional arguments (unica/cuda.py:138-160;
 * call sites in unica/__init__.py).  This library replaces that boundary by host entry points, one per reference
 * kernel launch, with plain pointers and sizes: the launch geometry, shared-memory sizes and tensor-memory use are its
 * own business.  A binding needs nothing but dlopen / ctypes.
 *
 * Conventions
 *   - every pointer is a device pointer on the current CUDA device unless said otherwise; nothing here allocates,
 *     frees or synchronises (except where an entry point says so); work is queued on `stream` (a cudaStream_t; NULL
 *     is the default stream);
 *   - `heads` is batch * heads; inputs are bf16 (or float16) [batch, heads, tokens, 128] in any strides with a contiguous last
 *     dimension and 16-byte aligned tokens, described by unica_token_layout;
 *   - return value 0 = queued; otherwise one of the UNICA_B200_ERR_* codes, and unica_b200_last_error() gives the
 *     message (thread-local).
 *
 * Operand layouts written by the quantizers and read by the attention kernels (all per head, tiles in token order):
 *   Q8   [q_tiles][8][128 rows][16]  int8, q_tiles rounded up to even, 16 KB per tile of 128 queries
 *   K8   [k_tiles][8][ 64 rows][16]  int8, 8 KB per tile of 64 keys          (chunk c, row r: channels 16c..16c+15 of key r)
 *   V8   [k_tiles][4][128 chan][16]  int8, 8 KB per tile                     (chunk c, channel d: keys 16c..16c+15)
 *   v_token [k_tiles][2][64] float: log2 s_j then 1 / s_j of the tile's keys (per-token mode)
 * These are the shared-memory images tcgen05.mma reads (K-major, no swizzle: core matrices of 8 rows x 16 bytes), so a
 * tile is one contiguous bulk copy.  Rows past the last token are zeros.
 */
#ifndef UNICA_B200_H
#define UNICA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Strides in elements of a [batch, heads, tokens, 128] tensor, and its heads: the reference's TokenLayout
 * (csrc/flash.cu:231-237, unica/__init__.py:92-100), field for field. */
typedef struct {
    long long batch, head, token;
    int heads;
    int dtype; /* UNICA_B200_BFLOAT16 (0) or UNICA_B200_FLOAT16: see below */
} unica_token_layout;

/* Element types of the q, k, v a quantizer or statistics pass reads and of the output an attention kernel writes.
 * float16 input is rounded to bfloat16 as it is read (the reference converts the tensor first,
 * unica/__init__.py:236: same numbers, one pass through memory less); a float16 output gets the float16 of the
 * bfloat16 result. */
enum { UNICA_B200_BFLOAT16 = 0, UNICA_B200_FLOAT16 = 1 };

enum {
    UNICA_B200_OK = 0,
    UNICA_B200_ERR_ARGUMENT = 1, /* a size, pointer or mode the entry point does not take */
    UNICA_B200_ERR_CUDA = 2,     /* the CUDA runtime refused the launch or a set-up call */
    UNICA_B200_ERR_DEVICE = 3,   /* not an sm_100 device */
    UNICA_B200_ERR_KERNEL = 4    /* a kernel reported a non-zero status word (unica_b200_read_status) */
};

/* V scale modes of the accurate kernel (the reference's V_TOKEN / V_OUTLIERS build settings, unica/__init__.py:88-89) */
enum { UNICA_B200_V_CHANNEL = 0, UNICA_B200_V_TOKEN = 1, UNICA_B200_V_OUTLIERS = 2 };

const char* unica_b200_last_error(void);
int unica_b200_version(void);

/* Replaces rope_stats + the torch reduction over its partials (csrc/flash.cu:287-327; unica/__init__.py:580-612).
 * Per channel of each head, over each group of `per` tokens (0: the whole head; else a multiple of 256): mean, min,
 * max, float [heads][groups][128].  partial: scratch, float [heads][ceil(n_tokens / 256)][3][128].  Sums run in a
 * fixed order, so results do not depend on how many heads a call holds. */
int unica_b200_channel_stats(const void* x, unica_token_layout layout, int heads, int n_tokens, int per, float* partial,
                             float* mean, float* low, float* high, void* stream);

/* unica_b200_channel_stats over the whole head without the tokens whose byte in skip [heads][n_tokens] is 1: min and
 * max of V without its outlier keys (the second pass of v_outliers, unica/__init__.py:384-399).  The mean divides by
 * n_tokens and is of no use here. */
int unica_b200_channel_stats_masked(const void* x, unica_token_layout layout, const uint8_t* skip, int heads, int n_tokens,
                                    float* partial, float* mean, float* low, float* high, void* stream);

/* No counterpart in the reference.  unica_b200_channel_stats for callers that cannot provide the `partial` scratch:
 * code running where device memory cannot be had (a hook inside a pipeline that keeps the card full, a C host without
 * an allocator of its own) or must not be asked for (cudaMalloc / cudaFree stall the device).  The partial sums go to
 * a 9 MiB array built into the library.  CUDA loads a library's device code into a GPU's context when it is first
 * used there (lazy module loading), so the 9 MiB are reserved on a GPU by the first call of this entry point (or of any
 * kernel of the same module) on that GPU, and held until the process exits or the device is reset: make that first call
 * while memory is still to be had; on a card that is already full it fails with UNICA_B200_ERR_CUDA and a message
 * that says so.
 *   - limit: heads * ceil(n_tokens / 256) <= 6144 (40 heads x 32760 tokens need 5120); larger calls are refused with
 *     UNICA_B200_ERR_ARGUMENT and should use unica_b200_channel_stats;
 *   - apart from that first load of the module it allocates and frees nothing, here or in anything it calls; mean,
 *     low, high are still the caller's;
 *   - the first call on each device also looks the array's device address up (the device must be current) and keeps
 *     it: make that first call before starting any stream capture, and do not reset the device afterwards (the kept
 *     address would point into the old context);
 *   - all calls on a device share the one array, which keeps whatever the last call left in it (nothing in it needs
 *     clearing between calls); two calls whose kernels may run at the same time, e.g. on different streams, race on
 *     it and give wrong statistics: keep them ordered.
 * Results are bit for bit those of unica_b200_channel_stats. */
int unica_b200_channel_stats_static(const void* x, unica_token_layout layout, int heads, int n_tokens, int per, float* mean,
                                    float* low, float* high, void* stream);

/* Replaces quantize_int8 (csrc/flash.cu:334-372; unica/__init__.py:363-378).  x - mean (mean float [heads][128] or
 * NULL) in INT8 with one scale per block_tokens tokens: 128 for Q, 64 for K.  `tiles` >= ceil(n_tokens /
 * block_tokens) tiles are written (the extra ones zeros): the attention kernel wants Q8 with an even tile count.
 * codes: Q8 / K8 layout above; scales: float [heads][tiles]. */
int unica_b200_quantize_int8(const void* x, unica_token_layout layout, const float* mean, int heads, int n_tokens,
                             int block_tokens, int tiles, int8_t* codes, float* scales, void* stream);

/* Replaces quantize_v and the torch aminmax before it (csrc/flash.cu:590-630; unica/__init__.py:402-444).
 * per_token = 0: one scale per channel from the channel's min and max over the head (low, high float [heads][128],
 * from unica_b200_channel_stats), written to v_scale [heads][128].  per_token = 1: one scale per key over its
 * channels; v_scale becomes ones and v_token gets {log2 s, 1 / s}.  skip: uint8 [heads][n_tokens], 1 = write the key
 * as zeros (the outlier keys), or NULL. */
int unica_b200_quantize_v_int8(const void* v, unica_token_layout layout, const float* low, const float* high,
                               const uint8_t* skip, int per_token, int heads, int n_tokens, int8_t* v8, float* v_scale,
                               float* v_token, void* stream);

/* unica_b200_quantize_int8 for Q (block_tokens 128, no mean, no rotation) as a streaming kernel: persistent blocks with
 * several tiles in flight each; the same bits, about twice the bandwidth. */
int unica_b200_quantize_q_int8_stream(const void* q, unica_token_layout layout, int heads, int n_tokens, int tiles, int8_t* codes,
                                      float* scales, void* stream);

/* Statistics and quantization of K in one launch: what unica_b200_channel_stats (per = 0) followed by
 * unica_b200_quantize_int8 (block_tokens 64, mean = the statistics' mean) do (csrc/flash.cu:287-372; unica/__init__.py:
 * 363-378, 592-612), with the second read of K served by L2 instead of HBM.  codes, scales as unica_b200_quantize_int8
 * writes them, tiles = ceil(n_tokens / 64); mean [heads][128] is written too (the order in which its terms are added
 * differs from unica_b200_channel_stats', so its last bit can; it is fixed for a device and a token count).
 * scratch: UNICA_B200_FUSED_SCRATCH_BYTES of device memory, 16-byte aligned, that no other call uses at the same time;
 * its contents do not matter.  status: as for the attention kernels (a block that never sees its group's statistics
 * gives up after about a second and leaves STATUS 8 there), or NULL.  A cooperative launch of persistent blocks. */
#define UNICA_B200_FUSED_SCRATCH_BYTES (2u << 20)
int unica_b200_quantize_k_int8_fused(const void* k, unica_token_layout layout, int heads, int n_tokens, int tiles, void* scratch,
                                     size_t scratch_bytes, int8_t* codes, float* scales, float* mean, int* status, void* stream);

/* The same for V with one scale per channel: unica_b200_channel_stats followed by unica_b200_quantize_v_int8
 * (per_token 0, no skip): v8 and v_scale [heads][128] bit for bit as those two write them (minimum and maximum do not
 * depend on the order they are taken in). */
int unica_b200_quantize_v_int8_fused(const void* v, unica_token_layout layout, int heads, int n_tokens, void* scratch,
                                     size_t scratch_bytes, int8_t* v8, float* v_scale, int* status, void* stream);

/* Replaces attention_int8pv_tma (csrc/flash.cu:806-959; launched from unica/__init__.py:179-189).  The accurate mode:
 * S = Q8.K8^T on tcgen05 kind::i8, softmax in the log2 domain against each 64-key tile's own maximum, P as u8,
 * P.V8 on kind::i8 (u8 x s8), flushed into a float accumulator with alpha / beta every tile.
 * out: bf16 in out_layout.  scale_log2 = log2(e) / sqrt(128).  status: device int the kernel leaves non-zero if one
 * of its bounded waits gave up (must be 0 on entry), or NULL.
 * v_mode UNICA_B200_V_OUTLIERS (the reference's V_OUTLIERS, csrc/flash.cu:748-790): V8 per channel with each head's
 * n_outliers (<= 8) outlier keys written as zeros; their share of P.V is added exactly at the end from outlier_keys
 * int [heads][n_outliers] (-1: none) and outlier_rows float [heads][n_outliers][128] = their V rows over v_scale.
 * Both are NULL / 0 in the other modes. */
int unica_b200_attention_int8(const int8_t* q8, const float* q_scale, const int8_t* k8, const float* k_scale,
                              const int8_t* v8, const float* v_scale, const float* v_token, int v_mode,
                              const int* outlier_keys, const float* outlier_rows, int n_outliers, void* out,
                              unica_token_layout out_layout, int heads, int n_queries, int n_keys, float scale_log2,
                              int* status, void* stream);

/* ---- fast mode (NVFP4) ------------------------------------------------------------------------------------------
 * Operand layouts, per head (two e2m1 codes per byte, the lower contraction index in the low nibble; one e4m3 scale
 * byte per 16 elements along the contraction; keys of a 64-key tile in the reference's slot order, bench/emulate.py:116-119):
 *   Q4  [q_tiles (even)][4 chunks of 32 channels][128 rows][16]  8 KB/tile   SFQ [q_tiles][2 halves of 64 channels][128][4]
 *   K4  [k_tiles][4][64 slots][16]                               4 KB/tile   SFK [k_tiles][32 lanes][4 words][4]
 *   V4  [k_tiles][2 chunks of 32 slots][144 rows][16]            4.5 KB      SFV [k_tiles][2 blocks][32 lanes][4 words][4]
 *       rows 0..127 channels, rows 128..143 ones (their column of P.V is the softmax denominator)
 *   K's and V's scale bytes lie as tcgen05.cp (32x128b) takes them, 16 bytes per tensor-memory lane: the word (four
 *   bytes, one per 16-element block of a K = 64 step) of operand row r is word r / 32 of lane r % 32; K's two steps
 *   follow each other (word 2 step + r / 32); V's second block holds rows 128..143 (word 0 of lanes 0..15: ones).
 *   bias [q_blocks][k_tiles * 64] float: the Q-smoothing term, already times log2(e)/sqrt(128), slot order */

/* outer = max(max|x - mean| * (1/2688), 1e-30) per head from per-channel statistics (mean may be NULL; all
 * [heads][groups][128]).  Replaces the torch lines of unica/__init__.py:485-492. */
int unica_b200_nvfp4_outer(const float* mean, const float* low, const float* high, int heads, int groups, float* outer,
                           void* stream);

/* Replaces quantize_fp4_rows (csrc/flash.cu:1183-1216; unica/__init__.py:473-500).  rows_per_tile 128: Q (token
 * order), 64: K (slot order).  mean: [heads][ceil(n_tokens / mean_tokens)][128] or NULL (mean_tokens <= 0: one mean
 * per head).  outer: [heads] from unica_b200_nvfp4_outer. */
int unica_b200_quantize_fp4_rows(const void* x, unica_token_layout layout, const float* mean, int mean_tokens,
                                 const float* outer, int heads, int n_tokens, int rows_per_tile, int tiles,
                                 uint8_t* codes, uint8_t* sf, void* stream);

/* Replaces quantize_v4 and the torch aminmax before it (csrc/flash.cu:1021-1050; unica/__init__.py:452-466).
 * low, high: per-channel min and max over the head; v_outer [heads][128] is written. */
int unica_b200_quantize_v_fp4(const void* v, unica_token_layout layout, const float* low, const float* high, int heads,
                              int n_tokens, uint8_t* codes, uint8_t* sf, float* v_outer, void* stream);

/* Replaces smooth_bias (csrc/flash.cu:1254-1322; unica/__init__.py:503-521): q_mean[block] . (k - k_mean) in FP32 for
 * every block of smoothed queries and every key, times scale_log2.  q_mean [heads][q_blocks][128], k_mean [heads][128].
 * bias [heads][q_blocks][ceil(n_keys / 64) * 64] in the slot order of K4's tiles; the slots past the last key hold -inf
 * (the attention kernel adds the table to the scores, which takes those slots out of the softmax).  Computed on the
 * tensor core (kind::tf32, every FP32 value as two tf32 parts, three products): accurate to about 2^-22 of
 * sum |q_mean| |k - k_mean|.  status: as for unica_b200_attention_int8 (the kernel waits for its tensor-core
 * instructions with a time limit). */
int unica_b200_smooth_bias(const void* k, unica_token_layout layout, const float* k_mean, const float* q_mean, int heads,
                           int q_blocks, int n_keys, float scale_log2, float* bias, int* status, void* stream);

/* ---- RoPE inside the quantizers -----------------------------------------------------------------------------------
 * Replace the reference's `freqs, freqs_batch` kernel arguments (rope_chunk / load_chunk_rope, csrc/flash.cu:250-279;
 * rope_args, unica/__init__.py:571-577): x is rotated in float before anything else is done with it, so the rotated
 * tensor is never written.  rope: (cos, sin) per pair of channels in fp16, [batch or 1][n_tokens][64][2];
 * rope_batch_stride: halves between the tables of two batches, 0 when one table serves all.  out[2i] = c x[2i] - s x[2i+1],
 * out[2i+1] = s x[2i] + c x[2i+1], products rounded before the sum (bench/emulate.py:122-130).  The other arguments
 * are those of the entry point without the suffix; a mean passed in is the rotated x's. */
int unica_b200_channel_stats_rope(const void* x, unica_token_layout layout, const void* rope, long long rope_batch_stride,
                                  int heads, int n_tokens, int per, float* partial, float* mean, float* low, float* high,
                                  void* stream);
int unica_b200_quantize_int8_rope(const void* x, unica_token_layout layout, const float* mean, const void* rope,
                                  long long rope_batch_stride, int heads, int n_tokens, int block_tokens, int tiles,
                                  int8_t* codes, float* scales, void* stream);
int unica_b200_quantize_fp4_rows_rope(const void* x, unica_token_layout layout, const float* mean, int mean_tokens,
                                      const void* rope, long long rope_batch_stride, const float* outer, int heads,
                                      int n_tokens, int rows_per_tile, int tiles, uint8_t* codes, uint8_t* sf, void* stream);
int unica_b200_smooth_bias_rope(const void* k, unica_token_layout layout, const float* k_mean, const float* q_mean,
                                const void* rope, long long rope_batch_stride, int heads, int q_blocks, int n_keys,
                                float scale_log2, float* bias, int* status, void* stream);

/* No counterpart in the reference (which runs on one GPU).  unica_b200_attention_int8 for a job that shards the heads
 * over several GPUs and wants every GPU to end up with all heads: each output row is stored to `out` and, at the same
 * offsets, to the n_peers (0..7) tensors of peer_out, which are this process's mappings of the other GPUs' output tensors
 * (peer access or an imported IPC / fabric handle; `out` and each peer_out[i] already offset to this call's first head).
 * The kernel only stores to peer memory, with plain stores, and reads nothing from it.  Ordering against the peers'
 * own streams is the caller's business: nobody may read or overwrite those rows between this call's launch and a
 * barrier after its completion.  peer_out is read before the call returns (host memory). */
int unica_b200_attention_int8_peers(const int8_t* q8, const float* q_scale, const int8_t* k8, const float* k_scale,
                                    const int8_t* v8, const float* v_scale, const float* v_token, int v_mode,
                                    const int* outlier_keys, const float* outlier_rows, int n_outliers, void* out,
                                    void* const* peer_out, int n_peers, unica_token_layout out_layout, int heads, int n_queries,
                                    int n_keys, float scale_log2, int* status, void* stream);

/* Hardware self-test of the tensor-core path (the idea of the reference's tests/test_mma.py: small integers make every
 * result exact, so a wrong lane or layout cannot hide).  One tcgen05.mma kind::i8 chain D[128 x n] = A[128 x k] . B[n x k]^T
 * with A (u8 if a_unsigned, else s8) and B (s8) given as the shared-memory images described above
 * ([k / 16][rows][16] bytes); d gets int32 [128][n] row-major.  The operands are described as the attention
 * kernels describe theirs; variant must be 0.  a_unsigned = 2: the same chain as kind::tf32 (what
 * unica_b200_smooth_bias issues): the images hold floats, [k / 16][rows][4], k / 4 of them per row, and d receives the
 * bits of the float results.
 * Allocates a status word and synchronises the stream: not for the hot path. */
int unica_b200_selftest_mma_i8(const void* a_image, const void* b_image, int n, int k, int a_unsigned, int variant,
                               int32_t* d, void* stream);

/* Replaces attention_fp4 with SMOOTH_Q (csrc/flash.cu:1380-1524; launched from unica/__init__.py:179-189).  The fast
 * mode: both contractions on tcgen05 kind::mxf4nvf4 with block scales in tensor memory, running-max softmax, P in NVFP4
 * (1024 * 2^(x - m), one e4m3 scale per 16 slots), the denominator taken from a column of ones in V4.
 * qk_outer [heads] = max(q_outer * k_outer, 1e-30); v_outer [heads][128]; bias: the table of unica_b200_smooth_bias or
 * NULL (no Q smoothing), q_blocks = ceil(n_queries / smooth_q) its rows per head, smooth_q a multiple of 256.
 * out, out_layout, scale_log2, status as for unica_b200_attention_int8. */
int unica_b200_attention_fp4(const uint8_t* q4, const void* sfq, const uint8_t* k4, const void* sfk, const uint8_t* v4,
                             const void* sfv, const float* qk_outer, const float* v_outer, const float* bias, int q_blocks,
                             int smooth_q, void* out, unica_token_layout out_layout, int heads, int n_queries, int n_keys,
                             float scale_log2, int* status, void* stream);

/* No counterpart in the reference: unica_b200_attention_fp4 with peer outputs, as unica_b200_attention_int8_peers. */
int unica_b200_attention_fp4_peers(const uint8_t* q4, const void* sfq, const uint8_t* k4, const void* sfk, const uint8_t* v4,
                                   const void* sfv, const float* qk_outer, const float* v_outer, const float* bias, int q_blocks,
                                   int smooth_q, void* out, void* const* peer_out, int n_peers, unica_token_layout out_layout,
                                   int heads, int n_queries, int n_keys, float scale_log2, int* status, void* stream);

/* No counterpart in the reference (its emulator shows P^, its kernel does not): unica_b200_attention_fp4 that also
 * leaves every row's quantized probabilities in p_words, uint32 [heads][n_queries][ceil(n_keys / 64)][9]: per key tile
 * eight words of e2m1 codes (slot s of the tile in nibble s % 8 of word s / 8) and one word with the four e4m3 scale
 * bytes (slots 16 b .. 16 b + 15 in byte b).  For tests that count how many codes differ from an emulation's; the
 * extra stores make it slower than the plain entry. */
int unica_b200_attention_fp4_codes(const uint8_t* q4, const void* sfq, const uint8_t* k4, const void* sfk, const uint8_t* v4,
                                   const void* sfv, const float* qk_outer, const float* v_outer, const float* bias, int q_blocks,
                                   int smooth_q, void* out, unica_token_layout out_layout, int heads, int n_queries, int n_keys,
                                   float scale_log2, uint32_t* p_words, int* status, void* stream);

/* The same for the block-scaled FP4 path: D[128 x n] = (A . sfa) . (B . sfb)^T with one tcgen05.mma
 * kind::mxf4nvf4.block_scale.scale_vec::4X per 64 elements of k (k = 64 or 128).  a_image [k / 32][128][16],
 * b_image [k / 32][n][16] bytes (two e2m1 codes per byte, low nibble first); sfa uint32 [k / 64][128], sfb uint32
 * [k / 64][n]: byte i of a word is the e4m3 scale of elements 16 i .. 16 i + 15 of that 64-element step.  d: float
 * [128][n].  variant 0: the computing threads store the scale words into tensor memory (as the attention kernel does for Q's);
 * 2: A's are copied from shared memory by the issuing thread (tcgen05.cp, as it does for K's, V's and P's).
 * Allocates a status word and synchronises the stream: not for the hot path. */
int unica_b200_selftest_mma_nvf4(const void* a_image, const void* b_image, const void* sfa, const void* sfb, int n, int k,
                                 int variant, float* d, void* stream);

/* Peak-rate micro-benchmark (the reference's csrc/peak.cu + bench/peak.py, for the instructions used here): cycles per
 * instruction on one SM, median over `blocks` blocks.  kind 0: tcgen05.mma kind::i8 128 x n x 32; 1: kind::mxf4nvf4
 * 128 x n x 64 (both on shared-memory operands in this library's layout; per MMA); 2..7: ex2.approx, fma.f32x2, fma.f32,
 * prmt, cvt s32->f32, cvt f32->u32 (per warp instruction per scheduler; n = warps per scheduler, 1..4, else 4).
 * count: instructions in the chain.  Tensor kinds take diagnostic variants in the higher decimal digits of `kind`:
 * + 100 x L: shared-memory layout type L of the descriptor (0: none, as the library uses; 1, 2, 4, 6: the swizzled
 * types, timing only; anything else is refused); + 1000: M = 64 instead of 128; + 10000 x R: move to the next accumulator every R instructions
 * (0: one accumulator).  Allocates scratch and synchronises the stream: a measurement tool. */
int unica_b200_peak(int kind, int n, int count, int blocks, double* cycles_per_instruction, void* stream);

#ifdef __cplusplus
}
#endif
#endif
