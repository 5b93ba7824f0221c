/* bfp8.h - C ABI of libbfp8.so: block-scaled E4M3 GEMM and E4M3 codec kernels for NVIDIA B200.
 *
 * Conventions (all entry points):
 *   - extern "C", plain pointers and 64-bit sizes; no C++ or framework types cross the boundary.
 *   - Every pointer named *_dev (and every data pointer) is a device pointer on the current
 *     CUDA device; `stream` is a cudaStream_t passed as void* (NULL = default stream).
 *   - The return value is 0 or a negative BFP8_ERR_* code for conditions the host can see
 *     (null pointer, misalignment, bad shape, workspace too small).  Nothing is launched when an
 *     error is returned.  Work is enqueued asynchronously on `stream`.
 *   - Conditions only the device can see are OR-ed into a caller-owned 32-bit status word
 *     (BFP8_STATUS_* bits).  The caller zeroes it before the first call and reads it after
 *     synchronising; several calls may share one word.
 *   - The library's only mutable global state is caches of facts about the device (driver entry points, SM
 *     count, per-kernel shared-memory and cluster limits), the switch of bfp8_set_weights_at_rest and the
 *     fixed scratch of bfp8_gemm_block128_noalloc; calls are re-entrant and may be issued from several host threads on
 *     different streams (that one entry point excepted, see there).  The caches are keyed by device ordinal
 *     and are not rebuilt after cudaDeviceReset: a process that resets a device must not call the library
 *     on it again.
 *
 * These conventions mirror the reference glue's: integer status codes instead of exceptions, caller-owned
 * buffers, and a size query before any call that needs scratch (two-phase protocol of
 * csrc/host/generic_attention_glue.hpp:84-90 in tracycam/gaudi-kernels).
 */
#ifndef BFP8_H_
#define BFP8_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BFP8_OK               0
#define BFP8_ERR_NULL        -1   /* a required pointer is NULL */
#define BFP8_ERR_ALIGN       -2   /* a pointer or leading dimension breaks the stated alignment */
#define BFP8_ERR_SHAPE       -3   /* a size is zero, negative or outside the supported range */
#define BFP8_ERR_WORKSPACE   -4   /* workspace smaller than bfp8_*_workspace_bytes() */
#define BFP8_ERR_CUDA        -5   /* a CUDA runtime / driver call failed (see bfp8_last_cuda_error) */
#define BFP8_ERR_UNSUPPORTED -6   /* not an sm_100 part, or a configuration the entry point states it does not take */
#define BFP8_ERR_TOO_LARGE   -7   /* the problem exceeds the fixed scratch of bfp8_gemm_block128_noalloc */

#define BFP8_STATUS_NONFINITE_CODE 0x1u  /* an input byte was 0x7f or 0xff (OCP E4M3FN NaN) */
#define BFP8_STATUS_BAD_SCALE      0x2u  /* a scale was negative, non-finite, or overflowed when doubled */
#define BFP8_STATUS_WAIT_TIMEOUT   0x4u  /* a bounded barrier wait inside a kernel gave up */
#define BFP8_STATUS_NONFINITE_INPUT 0x8u /* an activation was inf or NaN */

#define BFP8_OUT_F32  0
#define BFP8_OUT_BF16 1

int bfp8_version(void);
const char* bfp8_error_string(int code);
/* cudaError_t value of the most recent failing CUDA call on this host thread (0 if none). */
int bfp8_last_cuda_error(void);

/* OCP E4M3FN -> Gaudi2 half-range E4M3 byte map, with the scale doubling that goes with it.
 * Replaces gaudi_kernels.fp8_codec.reencode_e4m3fn_half (python/gaudi_kernels/fp8_codec.py:14-53):
 *   codes_out[i] = sign | half(magnitude) with round-to-nearest-even on the low end (:36-40);
 *   scales_out[j] = 2 * scales_in[j] (:30);
 *   *rounded_dev += number of codes whose halving was inexact (:50)  (caller zeroes it first);
 *   status |= NONFINITE_CODE for any 0x7f/0xff (:48-49), BAD_SCALE for the conditions of :25-32.
 * n > 0 codes; n_scales may be 0 (then scales_* may be NULL).  In-place (codes_out == codes_in) is allowed. */
int bfp8_reencode_half(const uint8_t* codes_in, uint8_t* codes_out, int64_t n,
                       const float* scales_in, float* scales_out, int64_t n_scales,
                       unsigned long long* rounded_dev, uint32_t* status_dev, void* stream);

/* The input checks of bfp8_reencode_half without the re-encoding, for checkpoints whose OCP codes are used
 * unchanged: status |= NONFINITE_CODE for any 0x7f / 0xff code (python/gaudi_kernels/fp8_codec.py:48-49;
 * python/gaudi_kernels/block_fp8_oracle.py:22-24 rejects the same inputs), BAD_SCALE for a negative or
 * non-finite scale (fp8_codec.py:25-29).  Nothing is written but the status word.  n > 0; n_scales may be 0. */
int bfp8_validate_e4m3(const uint8_t* codes, int64_t n, const float* scales, int64_t n_scales,
                       uint32_t* status_dev, void* stream);

/* 128x128 block-amax quantizer, fp32 [rows, cols] (row stride ld, elements) -> E4M3 codes
 * [rows, cols] (row stride ld_codes) + fp32 scales [ceil(rows/128), ceil(cols/128)] (dense).
 * Per tile: scale = max(amax, 1e-10) * fp32(1/448); code = RNE_e4m3(clamp(x / scale, +-448)) -
 * the rule of python/gaudi_kernels/block_fp8_oracle.py:27-28 applied to a square tile (the reference
 * has no weight quantizer of its own).  native_half != 0 additionally applies the half-range map
 * and stores 2*scale (block_fp8_oracle.py:31-35), in the same pass. */
int bfp8_quant_block128_f32(const float* w, int64_t rows, int64_t cols, int64_t ld,
                            uint8_t* codes, int64_t ld_codes, float* scales,
                            int native_half, void* stream);

/* 1x128 activation quantizer, bf16 [m, k] (row stride ldx) -> E4M3 codes [m, k] (row stride
 * ld_codes) + fp32 scales addressed as scales[row * scale_stride_m + group * scale_stride_g].
 * Replaces python/gaudi_kernels/block_fp8_oracle.py:25-28 (and :31-34 when native_half != 0); the
 * Gaudi2 counterpart is gk_fp8_block_quant_bf16_v1 (csrc/tpc/block_fp8_framework/activation_native.c:9-29).
 * A ragged last group (k % 128 != 0) is treated as zero-padded.  status_dev may be NULL; otherwise
 * NONFINITE_INPUT is raised for an inf/NaN activation (the check of block_fp8_oracle.py:22). */
int bfp8_quant_act_1x128_bf16(const uint16_t* x, int64_t m, int64_t k, int64_t ldx,
                              uint8_t* codes, int64_t ld_codes,
                              float* scales, int64_t scale_stride_m, int64_t scale_stride_g,
                              int native_half, uint32_t* status_dev, void* stream);

/* value(code) * block scale -> fp32 or bf16 [rows, cols].  value() is the E4M3 decode of
 * tests/test_fp8_codec.py:8-12; the Gaudi2 counterpart of the scaling is
 * gk_fp8_dequant_weight_fp16_1k_v1 (csrc/tpc/block_fp8_framework/dequant_weight_fp16_1k.c:5-30).
 * scales is [ceil(rows/128), ceil(cols/128)] dense.  out_dtype: BFP8_OUT_F32 or BFP8_OUT_BF16;
 * ld_out in elements of that type. */
int bfp8_decode_block128(const uint8_t* codes, int64_t rows, int64_t cols, int64_t ld,
                         const float* scales, void* out, int out_dtype, int64_t ld_out,
                         void* stream);

/* Block-scaled E4M3 GEMM:
 *   out[i, j] = sum_g a_scales[g, i] * w_scales[j / 128, g] * sum_{t < 128} a(i, 128 g + t) * w(j, 128 g + t) (+ bias[j])
 * Replaces the numerical contract of gaudi_kernels.block_fp8_oracle.reference
 * (python/gaudi_kernels/block_fp8_oracle.py:38-46) for operands that are already quantized; on Gaudi2 the
 * same contraction is an MME batched GEMM followed by gk_fp8_block_reduce_bf16_v1
 * (csrc/tpc/block_fp8_framework/reduce_bias.c:13-61).
 *   a_codes  uint8 E4M3 [m, k], row stride lda bytes (lda % 16 == 0, base 16-byte aligned)
 *   a_scales fp32, element (g, i) at a_scales[g * ldsa + i]   (group-major, ldsa >= m)
 *   w_codes  uint8 E4M3 [n, k], row stride ldw bytes (ldw % 16 == 0, base 16-byte aligned)
 *   w_scales fp32 [ceil(n/128), ceil(k/128)] dense
 *   bias     fp32 [n] or NULL
 *   out      fp32 or bf16 [m, n], row stride ldo elements (bf16: ldo % 8 == 0 and base 16-byte aligned)
 * Codes are consumed as OCP E4M3 by the tensor cores; Gaudi2 half-range codes (magnitude <= 0x76)
 * mean the same values under that format.  Each 128-wide block dot product is accumulated by the
 * tensor core in fp32 (TMEM); the promotion across K blocks is an fp32 FMA chain in g order.
 * workspace: bfp8_gemm_block128_workspace_bytes(m, n, k) bytes, 256-byte aligned (may be NULL if 0).
 *   Its first 64 KB hold arrival counters: they must be zero before the first call and every call that
 *   completes normally leaves them zero, so one zero-initialised buffer serves any sequence of calls on
 *   one stream.  Calls that may overlap on the device need separate workspaces.
 * status |= WAIT_TIMEOUT if an internal barrier wait gave up; the output is then undefined and counters may
 *   have been left non-zero: zero the first 64 KB of the workspace again before it is reused. */
size_t bfp8_gemm_block128_workspace_bytes(int64_t m, int64_t n, int64_t k);
int bfp8_gemm_block128(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                       const uint8_t* w_codes, int64_t ldw, const float* w_scales,
                       const float* bias, void* out, int out_dtype, int64_t ldo,
                       int64_t m, int64_t n, int64_t k,
                       void* workspace, size_t workspace_bytes,
                       uint32_t* status_dev, void* stream);


/* Same as bfp8_gemm_block128 with tuning / diagnostic knobs (0 = default for each):
 *   schedule           0 automatic; 1 large-tile schedule (one CTA per 128x256 tile); 2 small-M weight-streaming
 *                      schedule (m <= 128); 3 CTA-pair schedule (clusters of two CTAs per 256x256 tile)
 *   max_ctas           upper bound on the persistent grid
 *   wait_limit_cycles  SM-clock budget of every internal barrier wait before WAIT_TIMEOUT is raised
 * The reference has no counterpart; its launch geometry is fixed per GUID in
 * csrc/host/generic_fp8_glue.hpp:95-98,125-130. */
int bfp8_gemm_block128_ex(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                          const uint8_t* w_codes, int64_t ldw, const float* w_scales,
                          const float* bias, void* out, int out_dtype, int64_t ldo,
                          int64_t m, int64_t n, int64_t k,
                          void* workspace, size_t workspace_bytes,
                          uint32_t* status_dev, void* stream,
                          int schedule, int max_ctas, int64_t wait_limit_cycles);

/* Per-token activation quantizer, bf16 [m, k] -> E4M3 codes [m, k] + one fp32 scale per row (scales[m]).
 * Replaces gk_fp8_token_quant_bf16_v1 (csrc/tpc/block_fp8_framework/activation_token.c:4-26): amax over the
 * whole row, 1 substituted for the amax of an all-zero row (:17), scale = amax / 448 (IEEE division - the
 * value the kernel's FMA-corrected product computes, activation_quant_common.h:3-7), code = RNE_e4m3(x / scale)
 * clamped to +-448; native_half != 0 halves the codes (RNE) and stores 2 * scale (:21,24), as that kernel
 * always does.  status_dev may be NULL; NONFINITE_INPUT is raised for inf / NaN activations. */
int bfp8_quant_act_token_bf16(const uint16_t* x, int64_t m, int64_t k, int64_t ldx,
                              uint8_t* codes, int64_t ld_codes, float* scales,
                              int native_half, uint32_t* status_dev, void* stream);

/* Token/channel-scaled E4M3 GEMM:
 *   out[i, j] = (sum_t a(i, t) * w(j, t)) * a_scales[i] * w_scales[j] (+ bias[j])
 * Replaces the Gaudi2 pair "MME GEMM + gk_fp8_channel_finish_bf16_v1"
 * (csrc/tpc/block_fp8_framework/channel_finish.c:2-18; glue csrc/host/generic_fp8_glue.hpp:56-82): the whole K
 * range accumulates in TMEM and the finish (partial * act) * w_scale + bias, bf16 rounding included, is the
 * kernel's epilogue.  Operand and output requirements are those of bfp8_gemm_block128; a_scales is fp32 [m],
 * w_scales fp32 [n].  No workspace. */
int bfp8_gemm_token_channel(const uint8_t* a_codes, int64_t lda, const float* a_scales,
                            const uint8_t* w_codes, int64_t ldw, const float* w_scales,
                            const float* bias, void* out, int out_dtype, int64_t ldo,
                            int64_t m, int64_t n, int64_t k, uint32_t* status_dev, void* stream);

/* Declares, for the whole process, whether the weight operands (w_codes) of the decode-bucket GEMMs (m <= 128:
 * bfp8_gemm_block128, _ex, _swiglu, _push, _noalloc) are at rest.  These kernels are launched so that their
 * set-up overlaps the end of the previous kernel of the stream, and normally touch no global memory until that
 * kernel has finished.  With on != 0 the caller promises that no work still in flight when such a GEMM is
 * enqueued writes its w_codes (weights were prepared at load time and the device was synchronised since); the
 * kernel then requests the first weight tiles of every CTA before it waits for the previous kernel, so the
 * stream from HBM does not pause between the kernels of a decode step.  Activations, scales, bias, workspace
 * and output are still touched only after the wait, and results do not change.  Off by default; returns the
 * previous setting.  The reference has no counterpart (its weights are bound to the graph at compile time,
 * csrc/host/generic_fp8_glue.hpp:125-130). */
int bfp8_set_weights_at_rest(int on);

/* bfp8_gemm_block128 for callers that cannot allocate a workspace where they make the call (for
 * example a server that handed all device memory to its own pools at start-up, or host code running
 * where CUDA allocation calls are not allowed).  This entry point has no counterpart in the reference.
 * The scratch of the small-M schedule lives in a fixed 5,308,416-byte array inside the library (held by
 * every GPU that loads it), so the size is limited: m <= 32 and n <= 2,097,152, otherwise
 * BFP8_ERR_TOO_LARGE is returned and nothing is launched.  Arguments and results are those of
 * bfp8_gemm_block128 without the workspace.  No cudaMalloc / cudaFree or allocating library routine
 * is called.  Every call asks the runtime for the array's device address (a host-side query, made with the
 * call's device current); the first call on a device also loads the library's device code and raises the
 * kernel's shared-memory limit, so make that first call before any stream capture.
 * All calls on a device share the array: calls that may overlap on the GPU race on it. */
int bfp8_gemm_block128_noalloc(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                               const uint8_t* w_codes, int64_t ldw, const float* w_scales,
                               const float* bias, void* out, int out_dtype, int64_t ldo,
                               int64_t m, int64_t n, int64_t k,
                               uint32_t* status_dev, void* stream);

/* Load-time repack for bfp8_gemm_block128_swiglu: w_codes is the fused gate/up weight [2 * inter, k] (rows
 * [0, inter) gate, rows [inter, 2 * inter) up - the column order csrc/tpc/generic_dense/silu_and_mul_bf16.c:29
 * reads, `col` and `col + width`); out receives the same rows interleaved in chunks of 64: chunk c holds gate
 * rows 64c..64c+63 followed by up rows 64c..64c+63.  Codes are copied unchanged, the scale grid is not
 * touched.  inter must be a multiple of 128 (BFP8_ERR_UNSUPPORTED otherwise), k and both leading
 * dimensions multiples of 16; not in place. */
int bfp8_swiglu_interleave_weight(const uint8_t* w_codes, int64_t ld_src, uint8_t* out, int64_t ld_dst,
                                  int64_t inter, int64_t k, void* stream);

/* Gate/up GEMM with the SwiGLU step fused into its epilogue:
 *   gate = bf16(A . Wgate^T (+ bias[0:inter])),  up = bf16(A . Wup^T (+ bias[inter:2 inter])),
 *   out[i, j] = bf16( silu(gate[i, j]) * up[i, j] )                                    out: bf16 [m, inter]
 * Replaces "block-scaled GEMM to bf16 [m, 2 * inter], then gk_silu_and_mul_bf16_v1"
 * (csrc/tpc/generic_dense/silu_and_mul_bf16.c:4-13,16-75; glue csrc/host/generic_dense_glue.cpp:196-216):
 * both factors are rounded to bf16 exactly where the unfused pair rounds them, silu(g) = g / (1 + exp(-g))
 * with 0 for g <= -88, and the product is rounded once.  w_codes is the output of
 * bfp8_swiglu_interleave_weight; w_scales ([2 * inter / 128, ceil(k/128)]) and bias ([2 * inter] or NULL)
 * keep the fused weight's original order (gate first).  Other requirements as bfp8_gemm_block128;
 * inter % 128 == 0.  One weight copy serves both buckets: with m <= 128 and a workspace of
 * bfp8_gemm_block128_workspace_bytes(m, 2 * inter, k) bytes (256-byte aligned, first 64 KB zero as for
 * bfp8_gemm_block128) the weight-streaming schedule runs with the same epilogue - bit-identical to the
 * small-M GEMM over the un-interleaved weight followed by bfp8_silu_and_mul_bf16; without a workspace
 * (NULL) or with larger m the large-tile schedule runs. */
int bfp8_gemm_block128_swiglu(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                              const uint8_t* w_codes, int64_t ldw, const float* w_scales,
                              const float* bias, void* out, int64_t ldo,
                              int64_t m, int64_t inter, int64_t k,
                              void* workspace, size_t workspace_bytes, uint32_t* status_dev, void* stream);

/* The SwiGLU step on its own: out[r, c] = bf16( silu(gate_up[r, c]) * gate_up[r, inter + c] ), bf16 in and out.
 * Replaces gk_silu_and_mul_bf16_v1 (csrc/tpc/generic_dense/silu_and_mul_bf16.c:16-75, input [rows, 2 * inter], glue
 * csrc/host/generic_dense_glue.cpp:196-216) for GEMM results of the schedules that have no fused epilogue (the
 * decode bucket); same arithmetic as bfp8_gemm_block128_swiglu.  Any inter; 16-byte vector path when inter and both
 * leading dimensions are multiples of 8. */
int bfp8_silu_and_mul_bf16(const uint16_t* gate_up, int64_t ld_in, uint16_t* out, int64_t ld_out,
                           int64_t rows, int64_t inter, void* stream);

/* bfp8_silu_and_mul_bf16 followed by bfp8_quant_act_1x128_bf16 as one kernel: the values quantized are
 * bf16(silu(gate_up[r, c]) * gate_up[r, inter + c]) (silu_and_mul_bf16.c:16, rounded as that kernel stores them), the
 * quantization is block_fp8_oracle.py:25-28 (+ :31-34 with native_half) over groups of 128 columns of the [m, inter]
 * product.  Codes, scales and status exactly as the two calls would give them; the intermediate tensor never reaches
 * HBM.  This is the activation side of the down projection that follows a gate/up GEMM in the decode bucket. */
int bfp8_silu_quant_act_1x128_bf16(const uint16_t* gate_up, int64_t m, int64_t inter, int64_t ld_in,
                                   uint8_t* codes, int64_t ld_codes,
                                   float* scales, int64_t scale_stride_m, int64_t scale_stride_g,
                                   int native_half, uint32_t* status_dev, void* stream);

/* Sum of world_size per-rank slices in canonical rank order: dst[i] = ((s0[i] + s1[i]) + s2[i]) + ... in fp32,
 * rounded once (RNE) for bf16 data.  Replaces gk_rank_sum_bf16_v1 / gk_rank_sum_f32_v1
 * (csrc/tpc/generic_dense/rank_sum.c:4-42; glue csrc/host/generic_dense_glue.cpp:569-600): `gathered` holds the
 * slices back to back ([world_size * elems]), dst is [elems], both of `dtype` (BFP8_OUT_F32 / BFP8_OUT_BF16);
 * world_size 2..8 as there (BFP8_ERR_UNSUPPORTED otherwise). */
int bfp8_rank_sum(const void* gathered, void* dst, int64_t elems, int world_size, int dtype, void* stream);

/* The same sum over slices given by pointer (`slices` is a HOST array of world_size device pointers), which is
 * what the K-sharded GEMM uses: slice r may be memory of GPU r opened with bfp8_peer_open, so no gather precedes
 * the sum - the kernel reads every slice once through plain peer loads.  Optional bias: fp32, added after the
 * sum as bias[i % bias_period] (the slices then start at column 0 of a row of bias_period values). */
int bfp8_rank_sum_slices(const void* const* slices, void* dst, int64_t elems, int world_size, int dtype,
                         const float* bias, int64_t bias_period, void* stream);

/* Row-parallel (K-sharded) GEMM whose epilogue scatters the result: this rank's partial product
 * A[:, K_r] . W[:, K_r]^T is rounded to bf16 and every 128-row tile is stored - by the same bulk tensor store the
 * ordinary kernel uses, over NVLink where the destination is another GPU - into the receive area of the rank
 * that owns those rows, so the transfer runs under the remaining tiles' math.  recv is a HOST array of world_size
 * device pointers; recv[o] is rank o's receive area, bf16 [world_size][m / world_size][n] contiguous (peer
 * memory from bfp8_peer_open for o != rank), and this rank's rows [o R, (o + 1) R), R = m / world_size, land in
 * recv[o][rank].  After a bfp8_peer_barrier, recv[rank] is exactly the `gathered` operand of bfp8_rank_sum
 * (csrc/tpc/generic_dense/rank_sum.c:2: world_size contiguous slices).  Two shapes are taken, both with
 * n % 64 == 0: m % (128 * world_size) == 0 (large-tile schedule, bulk tensor stores; no workspace needed), and the
 * decode bucket m <= 128 with m % world_size == 0 (weight-streaming schedule, plain peer stores of each activation
 * row to its owner; needs a workspace of bfp8_gemm_block128_workspace_bytes(m, n, k) bytes, as bfp8_gemm_block128).
 * Anything else returns BFP8_ERR_UNSUPPORTED (use bfp8_gemm_block128 + bfp8_rank_sum_slices then).  No bias here -
 * add it in the sum.  No TMA load of this kernel touches peer memory and nothing is multicast. */
int bfp8_gemm_block128_push(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                            const uint8_t* w_codes, int64_t ldw, const float* w_scales,
                            void* const* recv, int rank, int world_size,
                            int64_t m, int64_t n, int64_t k,
                            void* workspace, size_t workspace_bytes, uint32_t* status_dev, void* stream);

/* Device memory that other processes on the same machine can map (one process per GPU).  These have no
 * counterpart in the reference, whose cross-device exchange lives in the external runtime
 * (csrc/tpc/generic_dense/rank_sum.c:2 only sees gathered data).
 *   bfp8_peer_alloc   cudaMalloc + zero fill on the current device (synchronous; set-up time only)
 *   bfp8_peer_export  64-byte handle of such an allocation, to be sent to the other ranks by any host channel
 *   bfp8_peer_open    map another rank's allocation into this process; the pointer is valid on the current device
 *   bfp8_peer_close / bfp8_peer_free   undo open / alloc */
int bfp8_peer_alloc(size_t bytes, void** ptr);
int bfp8_peer_free(void* ptr);
int bfp8_peer_export(void* ptr, uint8_t handle[64]);
int bfp8_peer_open(const uint8_t handle[64], void** ptr);
int bfp8_peer_close(void* ptr);

/* Stream-ordered barrier between the ranks' GPUs.  `flags` is a HOST array of world_size device pointers:
 * flags[r] is rank r's flag array (world_size uint32, zero at start, in bfp8_peer_alloc memory; flags[rank] is
 * this rank's own).  The kernel publishes `epoch` (use 1, 2, 3, ... on every rank alike) to every rank and waits
 * until every rank has published it; work enqueued on `stream` before the call is visible to the other ranks'
 * GPUs once their barrier returns.  The wait is bounded (wait_limit_cycles, 0 = about two seconds): on expiry
 * BFP8_STATUS_WAIT_TIMEOUT is raised in *status_dev and the kernel returns.  Each rank must run on its own GPU. */
int bfp8_peer_barrier(uint32_t* const* flags, int rank, int world_size, uint32_t epoch,
                      int64_t wait_limit_cycles, uint32_t* status_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif  /* BFP8_H_ */
