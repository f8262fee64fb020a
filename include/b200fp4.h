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
 * alpha: one f32 in device memory, or NULL for 1.  tile_n: 0 = choose (by problem size), or force one of
 * 64 / 128 / 256 (output columns per single-CTA tile) or 512 (256 x 256 tiles on CTA pairs).
 * Stands in for Sm120BlockScaledGemmKernel.__call__ and its kernel:
 *   third_party/cutlass/examples/python/CuTeDSL/cute/blackwell_geforce/kernel/blockscaled_gemm/
 *   dense_blockscaled_gemm_persistent_cooperative.py:281-439 (host), :443-1185 (device),
 *   alignment rule :1461-1511 (k % 32, n % 8, else "Invalid tensor alignment"). */
int b200fp4_nvfp4_gemm(const void* a, const void* b, const void* sfa, const void* sfb, void* c, const float* alpha,
                       int m, int n, int k, int l, int c_dtype, int tile_n, void* stream);

/* The same GEMM with scratch memory for split-K.  Problems with few 128 x 256 output tiles and a long reduction
 * (M = 128 against an 8192 x 8192 weight matrix: a 40 MB weight stream for 32 tiles) leave most SMs idle; with a
 * workspace of b200fp4_nvfp4_gemm_workspace_bytes(m, n, k) bytes (0 = this shape does not split; f32, 16-byte aligned,
 * caller-owned) and tile_n = 0 the K tiles of every output tile are dealt to several CTAs and a second small kernel
 * sums their partial matrices in slice order, applies alpha and rounds once.  workspace = NULL behaves exactly as
 * b200fp4_nvfp4_gemm.  (Measured at M = 128, N = K = 8192: the split kernel takes the same 15 us as the unsplit
 * 64-wide tiles and the reduction adds 4, so nothing selects this by default.)  Same reference interface as above. */
size_t b200fp4_nvfp4_gemm_workspace_bytes(int m, int n, int k);
int b200fp4_nvfp4_gemm_ws(const void* a, const void* b, const void* sfa, const void* sfb, void* c, const float* alpha,
                          int m, int n, int k, int l, int c_dtype, int tile_n, void* workspace, size_t workspace_bytes,
                          void* stream);

/* MXFP4 flavour of the same GEMM (sf_vec_size 32 of the demo): e2m1 codes as above, one ue8m0 scale byte (2^(b-127))
 * per 32 K-elements, in the same 128x4 tiles ([l][ceil(rows/128)][ceil(k/128)][32][4][4]).  Single-CTA tiles only
 * (tile_n 0, 64, 128 or 256).  Stands in for the (Float4E2M1FN, Float4E2M1FN, Float8E8M0FNU, 32) configuration of
 *   .../blockscaled_gemm/blockscaled_gemm_dispatch.py:34-43 and dense_blockscaled_gemm_persistent_cooperative.py:60-68. */
int b200fp4_mxfp4_gemm(const void* a, const void* b, const void* sfa, const void* sfb, void* c, const float* alpha,
                       int m, int n, int k, int l, int c_dtype, int tile_n, void* stream);

/* MXFP8 flavour: A [l][m][k] and B [l][n][k] are 8-bit floats (e4m3, or e5m2 where a_e5m2 / b_e5m2 != 0), one ue8m0
 * scale byte per 32 K-elements in 128x4 tiles ([l][ceil(rows/128)][ceil(k/128)][32][4][4]); k a multiple of 16.
 * Single-CTA tiles only.  Stands in for the (Float8E4M3FN | Float8E5M2, ..., Float8E8M0FNU, 32) configurations of
 *   .../blockscaled_gemm/blockscaled_gemm_dispatch.py:34-43. */
int b200fp4_mxfp8_gemm(const void* a, const void* b, const void* sfa, const void* sfb, void* c, const float* alpha,
                       int m, int n, int k, int l, int c_dtype, int tile_n, int a_e5m2, int b_e5m2, void* stream);

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

/* b200fp4_moe_fused with the router inside: router_logits f32 [tokens, num_experts] -> softmax -> top_k ->
 * (renormalised) weights as b200fp4_topk_route computes them, fused into the first kernel of the front end
 * (one launch fewer, and the ids never leave the GPU).  The routing is written to
 * token_selected_experts_out / token_final_scales_out ([tokens, top_k]) for the caller.  Other arguments as
 * b200fp4_moe_fused.  The reference op takes ids and weights as inputs and its harness draws them
 * (tools/perf/bench_flashinfer_b12x.py:70-74); this entry is the same operator with that step on the GPU. */
int b200fp4_moe_fused_routed(const void* x, const float* router_logits, int num_experts, int renormalize,
                             const void* w1, const void* w1_sf, const void* w2, const void* w2_sf,
                             int* token_selected_experts_out, float* token_final_scales_out, const float* w1_alpha,
                             const float* w2_alpha, const float* fc2_input_scale, void* out, int64_t tokens,
                             int hidden, int intermediate, int local_experts, int top_k, int local_expert_offset,
                             int accumulate, int out_dtype, void* workspace, size_t workspace_bytes, void* stream);

/* The same fused MoE for callers that cannot allocate device memory (engines that forbid cudaMalloc after
 * start-up, plugins that only receive raw pointers, latency-critical loops).  It has no counterpart in the
 * reference; it exists only in this library.  Arguments as b200fp4_moe_fused, without the workspace and without
 * out_dtype: `out` is always bf16 [tokens, hidden] and the k per-expert rows of a token are kept in f32 between
 * FC2 and the weighted sum (what out_dtype 1 selects in b200fp4_moe_fused).  The
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
 * aligned; cleared once with b200fp4_moe_ep_reset).  One step = dispatch, compute, combine on every rank,
 * all stream-ordered; the kernels synchronise the ranks themselves with three signals per step (words in
 * the buffers that carry a step counter), so the caller provides no barrier:
 *   dispatch (route +) count the slots per expert and publish the counts [signal 0]; wait for the counts of
 *            all ranks; quantise the rank's tokens once to NVFP4 and store every (token, slot) row straight
 *            into the expert-major FC1 operand of the rank that owns the slot's expert [signal 1];
 *   compute  wait for the rows of all ranks; FC1 / SwiGLU / FC2, whose epilogue stores every output row
 *            (bf16) into the buffer of the rank that owns the token [signal 2];
 *   combine  wait for the rows of all ranks; out[t] = bf16(sum_j scale[t,j] * row_j) in f32, slot order.
 * All peer accesses are plain loads / stores of these kernels over NVLink.  Every wait is bounded by wait_ms
 * (0 < wait_ms <= 60000): on expiry the kernel ORs bit 16 into the device status word, marks the buffer as
 * aborted and returns; later kernels of the group then touch no peer memory until b200fp4_moe_ep_reset.
 * return_mode (the same value in all calls of a step, on all ranks): 0 = as above, one row per (token, slot)
 * travels home and the results are bit-identical to b200fp4_moe_fused; 1 = FC2 keeps its rows on the expert's
 * GPU, a second kernel sums them per (source rank, token) with the routing weights (f32, slot order, one bf16
 * rounding) and sends ONE row per (token, rank that serves some of its slots); the combine adds those rows in
 * rank order.  Fewer bytes cross NVLink (a token's top_k experts sit on at most `world` ranks); the sum is
 * grouped by rank, so results differ from mode 0 by bf16 roundings of the partial sums.  Mode 1 needs
 * token_final_scales at dispatch when ids are given.
 * Routing: either token_selected_experts (global ids) is given, or router_logits f32
 * [tokens_local, world*local_experts] and the dispatch routes on the GPU (then pass NULL ids / scales to the
 * combine, and fetch the routing with b200fp4_moe_ep_routing if it is wanted).
 * Arguments otherwise as b200fp4_moe_fused.  The reference is single-GPU and has no counterpart; these entry
 * points are the dispatch / combine all-to-all of an expert-parallel deployment of the same operator
 * (tests/python/test_flashinfer_b12x_verbatim.py:99-116). */
size_t b200fp4_moe_ep_buffer_bytes(int64_t tokens_local, int hidden, int intermediate, int local_experts, int top_k,
                                   int world);
/* Clears the signal words, counters and abort word of the rank's own buffer.  No step may be in flight on any
 * rank (host-side barrier before and after). */
int b200fp4_moe_ep_reset(void* own_buffer, int64_t tokens_local, int hidden, int intermediate, int local_experts,
                         int top_k, int world, void* stream);
int b200fp4_moe_ep_dispatch(const void* x, const int* token_selected_experts, const float* token_final_scales,
                            const float* router_logits, int renormalize, const void* const* peer_buffers, int rank,
                            int world, int64_t tokens_local, int hidden, int intermediate, int local_experts,
                            int top_k, int return_mode, double wait_ms, void* stream);
/* The two halves of the dispatch as separate calls (count + signal 0, then wait + place + signal 1; same
 * arguments).  A harness that emulates several ranks of a group on ONE GPU must issue all ranks' counts before
 * any rank's place, all places before any compute and all computes before any combine, on one stream: then
 * every wait is already satisfied when its kernel starts and no kernel ever waits for a later launch. */
int b200fp4_moe_ep_dispatch_count(const void* x, const int* token_selected_experts, const float* token_final_scales,
                                  const float* router_logits, int renormalize, const void* const* peer_buffers,
                                  int rank, int world, int64_t tokens_local, int hidden, int intermediate,
                                  int local_experts, int top_k, int return_mode, double wait_ms, void* stream);
int b200fp4_moe_ep_dispatch_place(const void* x, const int* token_selected_experts, const float* token_final_scales,
                                  const float* router_logits, int renormalize, const void* const* peer_buffers,
                                  int rank, int world, int64_t tokens_local, int hidden, int intermediate,
                                  int local_experts, int top_k, int return_mode, double wait_ms, void* stream);
int b200fp4_moe_ep_compute(const void* const* peer_buffers, int rank, int world, const void* w1, const void* w1_sf,
                           const void* w2, const void* w2_sf, const float* w1_alpha, const float* w2_alpha,
                           const float* fc2_input_scale, int64_t tokens_local, int hidden, int intermediate,
                           int local_experts, int top_k, int return_mode, double wait_ms, void* stream);
int b200fp4_moe_ep_combine(const void* const* peer_buffers, int rank, int world, const int* token_selected_experts,
                           const float* token_final_scales, void* out, int64_t tokens_local, int hidden,
                           int intermediate, int local_experts, int top_k, int return_mode, double wait_ms,
                           void* stream);
int b200fp4_moe_ep_routing(const void* own_buffer, int* ids_out, float* weights_out, int64_t tokens_local, int hidden,
                           int intermediate, int local_experts, int top_k, int world, void* stream);

/* Self-tests of the bounded waits; they fault nothing and leave nothing in flight.
 * b200fp4_selftest_peer_wait: on ONE GPU, waits for the signal of `world` ranks on a cleared buffer that nobody
 * signals; after wait_ms the kernel gives up, ORs bit 16 into the device status word and returns.
 * b200fp4_selftest_bounded_wait: one CTA waits, with the GEMM kernels' own wait routine and a limit of
 * limit_cycles, on an mbarrier on which nothing arrives; it gives up, ORs bit 2 into the device status word and
 * writes 1 to *gave_up (device memory).  Neither has a counterpart in the reference, whose kernels wait without
 * bounds (python/self_cutedsl/frontend/jit.py:237-242). */
int b200fp4_selftest_peer_wait(void* own_buffer, int world, double wait_ms, int64_t tokens_local, int hidden,
                               int intermediate, int local_experts, int top_k, void* stream);
int b200fp4_selftest_bounded_wait(long long limit_cycles, int* gave_up, void* stream);

/* Kernels never trap: a device-side wait that exceeds its bound ORs a bit into a per-device
 * status word and the kernel returns.  This call synchronises the stream and copies the word
 * to *status_out (0 = healthy; 1/2/4 = GEMM producer / MMA / epilogue wait expired; 8 = a few-row GEMM launch
 * met a row block with more rows than it loads (the MoE front end never builds such a block); 16 = a wait for
 * another rank of an expert-parallel group expired), clearing it when clear != 0.  No counterpart in the reference, whose kernels wait without bounds. */
int b200fp4_device_status(void* stream, int* status_out, int clear);

#ifdef __cplusplus
}
#endif
#endif /* B200FP4_H_ */
