/*
 * nvfp4_b200.h -- C ABI of the B200 (sm_100a) NVFP4 quantize + block-scaled
 * FP4 GEMM library (libnvfp4_b200.so).
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream
 * (passed as void*, i.e. a cudaStream_t), launches asynchronously on that
 * stream, never synchronises with the host, never allocates, and returns an
 * nvfp4_status.  Nothing falls back to the CPU: on a device that is not
 * compute capability 10.x the calls return NVFP4_ERR_UNSUPPORTED_ARCH.
 *
 * Packed-tensor layout (identical to the reference's):
 *   data    uint8 [rows, cols/2]   two E2M1 codes per byte, even element in
 *                                  the low nibble
 *   scales  uint8 [rows, cols/16]  FP8-E4M3 bits, one per 16-element K-block,
 *                                  linear row-major
 *   global  float                  the FP32 per-tensor scale amax/(6*448)
 * The GEMM additionally reads scales in the tensor-core layout ("swizzled":
 * 512-byte atoms of 128 rows x 4 K-blocks ordered [32][4][4], rows padded to
 * 256 and K-blocks to 16); quantize emits it directly, and
 * nvfp4_swizzle_scales converts a linear buffer.
 *
 * Reference interfaces are cited by path inside the reference project.
 */
#ifndef NVFP4_B200_H_
#define NVFP4_B200_H_

#include <stdint.h>

#if defined(__GNUC__)
#define NVFP4_API __attribute__((visibility("default")))
#else
#define NVFP4_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum nvfp4_status {
  NVFP4_OK = 0,
  NVFP4_ERR_BAD_ARG = 1,          /* null pointer, negative size, cols % 16 != 0 ... */
  NVFP4_ERR_BAD_ALIGN = 2,        /* pointer or leading dimension not 16-byte aligned */
  NVFP4_ERR_UNSUPPORTED_ARCH = 3, /* current device is not sm_100 */
  NVFP4_ERR_LAUNCH_FAILED = 4,    /* cudaGetLastError() after the launch */
  NVFP4_ERR_TIMEOUT = 5           /* a device-side bounded wait gave up */
} nvfp4_status;

/* Epilogue activation selector of nvfp4_gemm. */
#define NVFP4_ACT_NONE 0
#define NVFP4_ACT_GELU_TANH 1

/* Human-readable name of a status code (static storage). */
NVFP4_API const char* nvfp4_status_string(int status);

/* Library version, major*10000 + minor*100 + patch. */
NVFP4_API int nvfp4_version(void);

/* Replaces the module-level init() of fx/src/s4/nvfp4/bindings.cpp:16-31,
 * which refuses compute capability < 12: here the requirement is exactly
 * 10.x.  Writes major/minor when the pointers are non-null. */
NVFP4_API int nvfp4_init(int device, int* cc_major, int* cc_minor);

/* Per-tensor max|x| into a device fp32 slot (zeroed by this call, on the
 * stream).  Replaces the host-synchronising input.abs().max().item() of
 * fx/src/s4/nvfp4/tensor.cpp:54 and linear/nvfp4_linear.cpp:79. */
NVFP4_API int nvfp4_amax_bf16(const void* x_bf16, int64_t n, float* amax_dev, void* stream);

/* Bytes of the swizzled scale buffer for a [rows, cols] tensor. */
NVFP4_API int64_t nvfp4_swizzled_scale_bytes(int64_t rows, int64_t cols);

/* bf16 [rows, cols] -> packed E2M1 + E4M3 block scales + FP32 tensor scale,
 * the tensor amax being read from a device slot (no host sync).  Replaces
 * launch_block_1d_quantization_cuda_te (fx/src/s4/nvfp4/quantization.cuh:
 * 52-54) with its global_amax argument moved to device memory.
 *   scales_linear   may be null (skip the linear copy)
 *   scales_swizzled may be null (skip the tensor-core copy)
 *   global_scale_dev may be null; otherwise receives amax/(6*448) as 1/S_enc */
NVFP4_API int nvfp4_quantize_bf16(const void* x_bf16, int64_t rows, int64_t cols, const float* amax_dev,
                        uint8_t* packed, uint8_t* scales_linear, uint8_t* scales_swizzled,
                        float* global_scale_dev, void* stream);

/* Same arithmetic with the reference launcher's exact argument list: flat
 * element count and global_amax by value.  Replaces
 * launch_block_1d_quantization_cuda_te (fx/src/s4/nvfp4/quantization.cuh:52-54).
 * n must be a multiple of 16. */
NVFP4_API int nvfp4_quantize_bf16_amax(const void* x_bf16, uint8_t* packed, uint8_t* scales, int64_t n,
                             float global_amax, void* stream);

/* packed + linear scales -> bf16, the tensor amax read from the device slot
 * nvfp4_amax_bf16 filled.  Replaces launch_block_1d_dequantization_cuda_te
 * (fx/src/s4/nvfp4/quantization.cuh:56-58). */
NVFP4_API int nvfp4_dequantize_bf16(const uint8_t* packed, const uint8_t* scales_linear, int64_t rows,
                          int64_t cols, const float* amax_dev, void* out_bf16, void* stream);

/* Same with global_amax by value, the reference launcher's argument list
 * (fx/src/s4/nvfp4/quantization.cuh:56-58). */
NVFP4_API int nvfp4_dequantize_bf16_amax(const uint8_t* packed, const uint8_t* scales, void* out_bf16,
                               int64_t n, float global_amax, void* stream);

/* Linear [rows, cols/16] scales -> swizzled layout (pad bytes zeroed).
 * Reconciles fx/src/s4/nvfp4/tensor.cpp:15 (linear scales) with the layout
 * fx/src/s4/nvfp4/kernel.cu:91-96 expects. */
NVFP4_API int nvfp4_swizzle_scales(const uint8_t* scales_linear, int64_t rows, int64_t cols,
                         uint8_t* scales_swizzled, void* stream);

/* Block-scaled FP4 GEMM on the tcgen05 tensor cores:
 *   D[M,N] (bf16) = beta * C + gate[n] * act( alpha * ga * gb * sum_k a*sfa * b*sfb + bias[n] )
 * A is [M, K/2] packed, B is [N, K/2] packed (both K-contiguous), scales are
 * swizzled, ga/gb are the device FP32 tensor scales (null = 1).  bias (bf16
 * [N]), gate (fp32 [N]) and C (bf16 [M,N]) may be null.  Replaces
 * blackwell_fp4_gemm_prequantized (fx/src/s4/nvfp4/kernel.cuh:13-18,
 * kernel.cu:15-159) without its M,N,K % 128 restriction: any M >= 1,
 * N % 8 == 0, K % 32 == 0.  d_amax_dev (nullable) receives max|D| over the stored bf16
 * values by atomic max (the slot is zeroed by this call, on the stream) so that a following
 * nvfp4_quantize_bf16 of D needs no separate amax pass.  status_dev (nullable) is a device
 * int the kernel sets non-zero if a bounded wait expires. */
NVFP4_API int nvfp4_gemm(const uint8_t* a_packed, const uint8_t* b_packed, const uint8_t* a_scales_swizzled,
               const uint8_t* b_scales_swizzled, const float* a_global_scale_dev,
               const float* b_global_scale_dev, int64_t M, int64_t N, int64_t K, float alpha,
               float beta, const void* c_bf16, const void* bias_bf16, const float* gate_f32,
               int act, void* d_bf16, float* d_amax_dev, int* status_dev, void* stream);

/* Which N tiling nvfp4_gemm uses: 0 = chosen per shape (the default; today always uniform),
 * 1 = uniform 256-wide tiles, 2 = 448-column pairs of a 256-wide and a 192-wide tile (two
 * disjoint accumulators in tensor memory: no hand-off between consecutive tiles, 8 % more
 * operand bytes per flop; measured 3-8 % slower than uniform on B200, kept selectable).
 * Process-wide; results do not depend on it: every output element is the same sum over K
 * either way.  A tuning and test knob with no counterpart in
 * the reference, whose CUTLASS instantiation fixes one 128x128x128 tile
 * (fx/src/s4/nvfp4/kernel.cu:61-82). */
NVFP4_API int nvfp4_gemm_set_tiling(int mode);

/* One GEMM against several weights stacked along N: B is [N, K/2] packed with N a multiple of
 * b_rows_per_weight (itself a multiple of 256), weight i occupying rows [i*b_rows_per_weight,
 * (i+1)*b_rows_per_weight) with its own FP32 tensor scale b_global_scales_dev[i]; swizzled
 * scales and bias stacked the same way.  D[M, N] = ga * gb[n / b_rows_per_weight] * sum + bias.
 * Every output element equals what nvfp4_gemm gives for that weight alone.  Used to compute the
 * cross-attention K/V projections of the text context for all DiT blocks in one launch before
 * the block loop (the context does not change from block to block; the reference's TE model
 * hoists this projection likewise, fx/src/s4/models/wan22/wan_transformer_megaupload.py:379-382,
 * 411-426) instead of one launch-bound M = 512 GEMM per block. */
NVFP4_API int nvfp4_gemm_stacked(const uint8_t* a_packed, const uint8_t* b_packed,
                                 const uint8_t* a_scales_swizzled, const uint8_t* b_scales_swizzled,
                                 const float* a_global_scale_dev, const float* b_global_scales_dev,
                                 int64_t b_rows_per_weight, int64_t M, int64_t N, int64_t K,
                                 const void* bias_bf16, void* d_bf16, int* status_dev,
                                 void* stream);

/* LayerNorm (rms = 0) or RMSNorm (rms = 1) over each row of x [rows, cols] in fp32, optional
 * affine weight/bias [cols] and adaLN modulation (1 + scale[cols]) * y + shift[cols] (all fp32,
 * all nullable), result rounded to bf16 -- the producer chain in front of the DiT block's QKV,
 * cross-attention Q and FFN-up linears (fx/src/s4/models/wan22/wan_transformer.py:204-206,
 * 210, 218-220) -- fused with the NVFP4 quantizer in two sweeps over x:
 *   sweep 1 (nvfp4_norm_mod_amax_bf16): per-row mean and rstd into row_stats [rows, 2] and the
 *     tensor amax of the bf16 result into amax_dev (zeroed by the call); h_out_bf16 (nullable)
 *     additionally receives the bf16 result itself;
 *   sweep 2 (nvfp4_norm_mod_quantize_bf16): recomputes the result from x and row_stats and
 *     writes packed nibbles, scales (linear and/or swizzled, either nullable) and the FP32
 *     tensor scale, exactly as nvfp4_quantize_bf16 would from the bf16 result.
 * cols % 16 == 0 and cols <= 16384.  Rows reach the SMs as bulk copies into shared memory;
 * a copy that does not arrive within about two seconds makes the kernel give up and store
 * 0x900 in *status_dev (nullable; the caller zeroes it once and may poll it at any time). */
NVFP4_API int nvfp4_norm_mod_amax_bf16(const void* x_bf16, int64_t rows, int64_t cols,
                                       const float* weight, const float* bias, const float* scale,
                                       const float* shift, int rms, float eps, float* row_stats,
                                       float* amax_dev, void* h_out_bf16, int* status_dev,
                                       void* stream);
NVFP4_API int nvfp4_norm_mod_quantize_bf16(const void* x_bf16, int64_t rows, int64_t cols,
                                           const float* weight, const float* bias,
                                           const float* scale, const float* shift,
                                           const float* row_stats, const float* amax_dev,
                                           uint8_t* packed, uint8_t* scales_linear,
                                           uint8_t* scales_swizzled, float* global_scale_dev,
                                           int* status_dev, void* stream);

/* q/k RMSNorm across heads + rotary embedding in one pass over the QKV linear's output: what
 * the reference block does with separate torch ops between to_qkv and attention
 * (fx/src/s4/models/wan22/wan_transformer.py:91-92,114-115 norm_q/norm_k; :61-75
 * apply_rotary_emb).  q_in / k_in (/ v_in, nullable) are bf16 [rows, heads*head_dim] views
 * with a common row stride in elements (e.g. the three column blocks of a [rows, 3*dim]
 * tensor); gains are fp32 [heads*head_dim] or null for 1; cos_sin is fp32
 * [rows, head_dim/2, 2] = (cos, sin) of each rotated pair.  Element (row, head, d) of an
 * output lands at out + row*out_row_stride + head*out_head_stride + d (strides in elements),
 * so one call can fill either three [rows, heads, head_dim] tensors or one packed
 * [rows, heads, 3*head_dim] buffer; v is copied unchanged when given.  k_in/k_out may be null
 * (q only), and cos_sin may be null (RMSNorm only, as for the cross-attention query).
 * head_dim % 16 == 0, heads*head_dim <= 8192, strides % 8 == 0.  A row group that does not
 * arrive in shared memory within about two seconds stores 0xA00 in *status_dev (nullable). */
NVFP4_API int nvfp4_qk_norm_rope_bf16(const void* q_in, const void* k_in, const void* v_in,
                                      int64_t in_row_stride, int64_t rows, int heads,
                                      int head_dim, const float* gain_q, const float* gain_k,
                                      float eps, const float* cos_sin, void* q_out, void* k_out,
                                      void* v_out, int64_t out_row_stride,
                                      int64_t out_head_stride, int* status_dev, void* stream);

/* The same kernel fused with the head/sequence exchange of sequence-parallel attention (no
 * reference counterpart: the reference has no distributed code).  `heads` are dealt out to
 * `world` ranks in order; rank_buffers[r] (a HOST array of `world` device pointers) is rank r's
 * bf16 [tokens_total, heads/world, 3*head_dim] buffer as mapped in THIS process (its own buffer
 * for r = this rank, peer-mapped memory otherwise).  Each thread stores its q | k | v pieces of
 * this rank's `rows` tokens, global token index row_offset + row, straight into the buffer of
 * the rank that owns the head: plain stores over NVLink, no staging copy, no collective.
 * sync_blocks (nullable; a HOST array of `world` device pointers to every rank's sync block of
 * nvfp4_exchange_sync_bytes() bytes, zeroed once, mapped in this process) makes the CTA that
 * finishes last raise this rank's flag of kind 0 on every rank; the consumers then order
 * themselves with nvfp4_exchange_wait.  Without it the caller orders the consumers after all
 * ranks' kernels itself (a barrier on the same streams). */
NVFP4_API int nvfp4_qk_norm_rope_exchange_bf16(const void* q_in, const void* k_in, const void* v_in,
                                               int64_t in_row_stride, int64_t rows, int heads,
                                               int head_dim, const float* gain_q,
                                               const float* gain_k, float eps,
                                               const float* cos_sin, void* const* rank_buffers,
                                               int world, int64_t row_offset,
                                               void* const* sync_blocks, int rank,
                                               int* status_dev, void* stream);

/* Bytes of one rank's sync block (flags, epochs and partial maxima of the exchanges). */
NVFP4_API int64_t nvfp4_exchange_sync_bytes(void);

/* Wait, on the stream, until every rank's flag of `kind` (0: the q|k|v pieces before attention,
 * 1: the attention output after it) in THIS rank's sync block has reached this rank's next
 * epoch, i.e. until all ranks' producer kernels of this exchange have finished storing.  One
 * tiny kernel that polls with plain loads; limit_ns bounds the wait: when it runs out the
 * kernel stores 0xB00 + (the first missing rank) in *status_dev (nullable) and returns
 * normally -- the GPU is never left spinning; while *status_dev stays non-zero later waits
 * return at once, so a missing rank costs one limit per step, not one per exchange.  For kind 1, amax_out_dev (nullable) receives the
 * tensor amax of the assembled attention output (the maximum over the sources' partial maxima),
 * ready for nvfp4_quantize_bf16.  No reference counterpart. */
NVFP4_API int nvfp4_exchange_wait(void* sync_block, int kind, int world, int64_t limit_ns,
                                  float* amax_out_dev, int* status_dev, void* stream);

/* The head -> sequence return exchange after attention, as one kernel of plain stores: o is
 * this rank's attention output, bf16 [tokens_total, heads_local, head_dim] with the given
 * token and head strides (in elements); the rows of rank s's tokens go into rank_buffers[s]
 * (bf16 [tokens_total/world, heads_local*world, head_dim], mapped here) at this rank's head
 * columns.  The same pass takes max|o| per destination; the last CTA publishes those maxima
 * and raises this rank's flag of kind 1 on every rank (see nvfp4_exchange_wait).  Replaces the
 * second all-to-all of the Ulysses exchange and the amax pass of the attention-out linear's
 * quantizer; the reference's attention call sites are fx/src/s4/models/wan22/
 * wan_transformer.py:126-129 (no distributed counterpart). */
NVFP4_API int nvfp4_attn_return_exchange_bf16(const void* o_bf16, int64_t o_row_stride,
                                              int64_t o_head_stride, int64_t tokens_total,
                                              int heads_local, int head_dim,
                                              void* const* rank_buffers, void* const* sync_blocks,
                                              int world, int rank, void* stream);

/* Non-causal bf16 attention, head_dim == 128: o = softmax(q k^T * softmax_scale) v per head, on
 * the tensor cores of sm_100a (tcgen05, accumulators and the probabilities in tensor memory,
 * operands by TMA).  q is bf16 [q_len, heads, 128], k and v are bf16 [kv_len, heads, 128], o is
 * bf16 [q_len, heads, 128]; every tensor is addressed by a token stride and a head stride in
 * elements (multiples of 8), so the column blocks of a fused QKV projection can be passed
 * without a copy.  amax_dev (nullable) receives max|o| by an atomic maximum on the float's bit
 * pattern: zero it before the call and hand it to nvfp4_quantize_bf16 afterwards -- the
 * quantizer of the attention-out linear then needs no amax pass.  status_dev (nullable) records
 * 0xA00 + a code if a device-side wait gives up.  q_len == 0 is a no-op; kv_len must be at least 1.  Replaces flash_attn_qkvpacked_func at
 * fx/src/s4/models/wan22/wan_transformer_fast.py:47-58 and F.scaled_dot_product_attention at
 * fx/src/s4/models/wan22/wan_transformer.py:126-129,164-167. */
NVFP4_API int nvfp4_attention_bf16(const void* q_bf16, int64_t q_row_stride, int64_t q_head_stride,
                                   const void* k_bf16, int64_t k_row_stride, int64_t k_head_stride,
                                   const void* v_bf16, int64_t v_row_stride, int64_t v_head_stride,
                                   int64_t q_len, int64_t kv_len, int heads, int head_dim,
                                   float softmax_scale, void* o_bf16, int64_t o_row_stride,
                                   int64_t o_head_stride, float* amax_dev, int* status_dev,
                                   void* stream);

/* Has no counterpart in the reference.  One whole linear, y = act(x W^T + bias), for
 * callers that cannot allocate device memory (code inside a region where cudaMalloc is not
 * allowed, fixed-budget real-time loops, plug-ins handed only input and output pointers):
 * the packed activation, its scales and the amax / tensor-scale slots live in a fixed
 * device array inside the library (about 5 MiB, held by every GPU that loads the library
 * until the process exits).  x is bf16 [M, K]; the weight is given pre-quantized (packed
 * [N, K/2], swizzled scales, device tensor scale); y is bf16 [M, N]; bias may be null.
 * Limits: M*K <= nvfp4_linear_bf16_static_max_elements() (8 Mi), K % 32 == 0, N % 8 == 0, and
 * the padded scale layout must fit 1 MiB: ceil(M/256) * ceil(K/256) <= 256 (rows pad to 256 and
 * K to 256 elements, so a very skinny activation such as M = 1, K = 131072 is refused although
 * it has few elements); anything larger returns NVFP4_ERR_BAD_ARG.  The first call on each device resolves the
 * array's device address (with that device current); make that first call outside any
 * stream capture.  No call allocates.  All calls on a device share the one array: two calls
 * whose kernels can overlap on the GPU (different streams without ordering) race; calls on
 * one stream are safe, and nothing is carried from one call to the next. */
NVFP4_API int nvfp4_linear_bf16_static(const void* x_bf16, int64_t M, int64_t K,
                                       const uint8_t* w_packed, const uint8_t* w_scales_swizzled,
                                       const float* w_global_scale_dev, int64_t N,
                                       const void* bias_bf16, int act, void* y_bf16,
                                       int* status_dev, void* stream);
NVFP4_API int64_t nvfp4_linear_bf16_static_max_elements(void);

#ifdef __cplusplus
}
#endif
#endif /* NVFP4_B200_H_ */
