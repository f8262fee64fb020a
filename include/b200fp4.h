/* libb200fp4 -- C-ABI of the B200 (sm_100a) NVFP4 quantized-inference hot path.
 *
 * Every entry point takes plain device pointers and sizes, launches on the
 * given CUDA stream without synchronising the host, and returns 0 on success
 * or a positive status code (see B200FP4_* below); b200fp4_last_error() gives
 * the message of the calling thread's last failure.  The caller owns all
 * buffers.  Paths quoted in the comments are relative to the reference
 * project's root.
 */
#ifndef B200FP4_H_
#define B200FP4_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200FP4_OK 0
#define B200FP4_INVALID_ARGUMENT 1
#define B200FP4_UNSUPPORTED 2
#define B200FP4_CUDA_ERROR 3
#define B200FP4_DEVICE_TIMEOUT 4
#define B200FP4_NOT_INITIALISED 5

/* dtype codes of 16-bit activations */
#define B200FP4_FP16 0
#define B200FP4_BF16 1

/* scale-factor output layouts of the norm-quant kernels */
#define B200FP4_SF_ROW_MAJOR 0 /* [rows, hidden/16] bytes */
#define B200FP4_SF_SWIZZLED 1  /* 128x4 tiles: [ceil(rows/128)][ceil(hidden/64)][32][4][4] */
#define B200FP4_SF_BOTH 2      /* tiled into block_scale, row-major into block_scale_unswizzled */

const char* b200fp4_last_error(void);
int b200fp4_version(void);

/* RMSNorm * weight -> NVFP4 (e2m1 codes, two per byte with the even element in
 * the low nibble, plus one e4m3 scale factor per 16 elements).
 * Stands in for flashinfer's cute_dsl rmsnorm_fp4quant as the reference calls it:
 *   tests/python/test_flashinfer_norm_verbatim.py:134
 *   tools/perf/bench_flashinfer_norm.py:53-54
 * Arithmetic contract: tests/python/test_flashinfer_norm_verbatim.py:58-81.
 * x [rows, hidden] with x_row_stride elements between rows, weight [hidden],
 * y_fp4 [rows, hidden/2], global_scale = one f32 in device memory. */
int b200fp4_rmsnorm_fp4quant(const void* x, const void* weight, void* y_fp4, void* block_scale,
                             void* block_scale_unswizzled, const float* global_scale, float eps, int64_t rows,
                             int hidden, int64_t x_row_stride, int dtype, int sf_layout, void* stream);

/* residual <- x + residual (rounded to dtype, in place); RMSNorm of the sum *
 * weight -> NVFP4.  Stands in for flashinfer's cute_dsl add_rmsnorm_fp4quant:
 *   tests/python/test_flashinfer_norm_verbatim.py:155-164
 *   tools/perf/bench_flashinfer_norm.py:58-60
 * Arithmetic contract: tests/python/test_flashinfer_norm_verbatim.py:84-99. */
int b200fp4_add_rmsnorm_fp4quant(const void* x, void* residual, const void* weight, void* y_fp4,
                                 void* block_scale, void* block_scale_unswizzled, const float* global_scale,
                                 float eps, int64_t rows, int hidden, int64_t x_row_stride,
                                 int64_t residual_row_stride, int dtype, int sf_layout, void* stream);

/* NVFP4 block-scaled dense GEMM, C[l][m][n] = alpha * sum_k (A*SFA)[l][m][k] * (B*SFB)[l][n][k].
 * A [l][m][k/2] and B [l][n][k/2]: e2m1 codes, two per byte (lower k in the low nibble), K contiguous.
 * SFA / SFB: e4m3 bytes, one per 16 K-elements, in 128x4 tiles [l][ceil(rows/128)][ceil(k/64)][32][4][4]
 * (padding bytes zero).  C row-major, c_dtype 0 = fp16, 1 = bf16, 2 = f32; f32 accumulation.
 * alpha: one f32 in device memory, or NULL for 1.  tile_n: 0 = choose, 128 or 256.
 * Stands in for Sm120BlockScaledGemmKernel.__call__ and its kernel:
 *   third_party/cutlass/examples/python/CuTeDSL/cute/blackwell_geforce/kernel/blockscaled_gemm/
 *   dense_blockscaled_gemm_persistent_cooperative.py:281-439 (host), :443-1185 (device),
 *   alignment rule :1461-1511 (k % 32, n % 8, else "Invalid tensor alignment"). */
int b200fp4_nvfp4_gemm(const void* a, const void* b, const void* sfa, const void* sfb, void* c, const float* alpha,
                       int m, int n, int k, int l, int c_dtype, int tile_n, void* stream);

/* Router: softmax over `experts` logits per token, the top_k largest probabilities (lowest index
 * first among equals), optionally renormalised to sum 1.  logits f32 [tokens, experts] ->
 * ids i32 [tokens, top_k], weights f32 [tokens, top_k].
 * The reference op takes ids and weights as inputs and its harness draws them on the host
 * (tests/python/test_flashinfer_b12x_verbatim.py:142-143, tools/perf/bench_flashinfer_b12x.py:70-74);
 * this entry puts that step on the GPU. */
int b200fp4_topk_route(const float* logits, int* ids, float* weights, int tokens, int experts, int top_k,
                       int renormalize, void* stream);

/* Bytes of scratch that b200fp4_moe_fused needs for this problem size (0 on bad arguments). */
size_t b200fp4_moe_workspace_bytes(int64_t tokens, int hidden, int intermediate, int local_experts, int top_k);

/* Fused NVFP4 MoE: quantise tokens (NVFP4, in kernel), route by the given expert ids, FC1 [2I,H] per
 * expert, silu(gate)*up -> bf16 -> NVFP4, FC2 [H,I], times the routing weight, summed per token -> bf16.
 * Stands in for flashinfer's b12x_fused_moe as the reference calls it:
 *   tests/python/test_flashinfer_b12x_verbatim.py:99-116, tools/perf/bench_flashinfer_b12x.py:77-81
 * Arithmetic contract: tests/python/test_flashinfer_b12x_verbatim.py:28-65,209-219.
 * x bf16 [tokens, hidden]; w1 u8 [local_experts, 2I, hidden/2] (rows 0..I-1 = up, I..2I-1 = gate);
 * w2 u8 [local_experts, hidden, I/2]; w1_sf / w2_sf e4m3 bytes in 128x4 tiles
 * [local_experts][rows/128][K/64][32][4][4]; ids i32 and scales f32 [tokens, top_k]; alphas f32
 * [local_experts] or NULL; fc2_input_scale one f32 or NULL; out [tokens, hidden], bf16 (out_dtype 1 or 3) or
 * f32 (out_dtype 2, what expert-parallel ranks reduce across GPUs).  The k per-expert rows of a token are
 * always summed in f32 in slot order and rounded once; out_dtype 3 stores them as bf16 between FC2 and the
 * sum (half the bytes of the step's largest stream), 1 and 2 as f32.
 * Expert ids are global: those in [local_expert_offset, local_expert_offset + local_experts) are
 * computed, the others contribute nothing (expert parallelism).  accumulate != 0 adds into out.
 * workspace: 256-byte aligned device scratch of b200fp4_moe_workspace_bytes(...) bytes. */
int b200fp4_moe_fused(const void* x, const void* w1, const void* w1_sf, const void* w2, const void* w2_sf,
                      const int* token_selected_experts, const float* token_final_scales, const float* w1_alpha,
                      const float* w2_alpha, const float* fc2_input_scale, void* out, int64_t tokens, int hidden,
                      int intermediate, int local_experts, int top_k, int local_expert_offset, int accumulate,
                      int out_dtype, void* workspace, size_t workspace_bytes, void* stream);

/* The same fused MoE for callers that cannot allocate device memory (engines that forbid cudaMalloc after
 * start-up, plugins that only receive raw pointers, latency-critical loops).  It has no counterpart in the
 * reference; it exists only in this library.  Arguments as b200fp4_moe_fused, without the workspace: the
 * scratch is a fixed 32 MiB array inside the library's device image (held by every GPU that loads the
 * library until the process ends).  Problems whose b200fp4_moe_workspace_bytes(...) exceeds 32 MiB are
 * refused with B200FP4_UNSUPPORTED.  status_word: a caller-owned int in device memory, zeroed by the
 * caller, into which the kernels OR the bits described at b200fp4_device_status.
 * The first call on each device looks up the array's device address; make it before any stream capture.
 * All calls on a GPU share the array: calls whose kernels overlap on the same GPU race, serialise them. */
int b200fp4_moe_fused_noalloc(const void* x, const void* w1, const void* w1_sf, const void* w2, const void* w2_sf,
                              const int* token_selected_experts, const float* token_final_scales,
                              const float* w1_alpha, const float* w2_alpha, const float* fc2_input_scale, void* out,
                              int64_t tokens, int hidden, int intermediate, int local_experts, int top_k,
                              int local_expert_offset, int accumulate, int* status_word, void* stream);

/* Expert-parallel MoE over peer memory: one process per GPU, every rank owns tokens_local tokens and
 * local_experts consecutive experts (rank r: experts r*local_experts ...), and every rank holds a
 * buffer of b200fp4_moe_ep_buffer_bytes(...) bytes that all ranks can address (peer_buffers[i] is
 * rank i's buffer as seen from the calling process, e.g. CUDA IPC or symmetric memory; 256-byte
 * aligned).  One step = stage, <cross-rank barrier>, compute, <cross-rank barrier>, combine, all
 * stream-ordered; the barriers are the caller's (any stream-ordered barrier across the ranks).
 *   stage    quantise the rank's tokens once to NVFP4 and publish them with their expert ids;
 *   compute  pull the rows routed to local experts from their owners, FC1 / SwiGLU / FC2;
 *   combine  out[t] = bf16(sum_j scale[t,j] * row_j), rows read from the ranks that computed them.
 * Arguments as b200fp4_moe_fused (ids are global).  The reference is single-GPU and has no
 * counterpart; these entry points are the dispatch / combine of an expert-parallel deployment of
 * the same operator (tests/python/test_flashinfer_b12x_verbatim.py:99-116). */
size_t b200fp4_moe_ep_buffer_bytes(int64_t tokens_local, int hidden, int intermediate, int local_experts, int top_k,
                                   int world);
int b200fp4_moe_ep_stage(const void* x, const int* token_selected_experts, void* own_buffer, int64_t tokens_local,
                         int hidden, int intermediate, int local_experts, int top_k, int world, void* stream);
int b200fp4_moe_ep_compute(const void* const* peer_buffers, int rank, int world, const void* w1, const void* w1_sf,
                           const void* w2, const void* w2_sf, const float* w1_alpha, const float* w2_alpha,
                           const float* fc2_input_scale, int64_t tokens_local, int hidden, int intermediate,
                           int local_experts, int top_k, void* stream);
int b200fp4_moe_ep_combine(const void* const* peer_buffers, int rank, int world, const int* token_selected_experts,
                           const float* token_final_scales, void* out, int64_t tokens_local, int hidden,
                           int intermediate, int local_experts, int top_k, void* stream);

/* Kernels never trap: a device-side wait that exceeds its bound ORs a bit into a per-device
 * status word and the kernel returns.  This call synchronises the stream and copies the word
 * to *status_out (0 = healthy; 1/2/4 = GEMM producer / MMA / epilogue wait expired; 8 = a fused-MoE call with
 * at most 32 tokens named one expert more than 32 times: those rows are wrong), clearing
 * it when clear != 0.  No counterpart in the reference, whose kernels wait without bounds. */
int b200fp4_device_status(void* stream, int* status_out, int clear);

#ifdef __cplusplus
}
#endif
#endif /* B200FP4_H_ */
