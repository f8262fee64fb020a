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

/* Kernels never trap: a device-side wait that exceeds its bound ORs a bit into a per-device
 * status word and the kernel returns.  This call synchronises the stream and copies the word
 * to *status_out (0 = healthy; 1/2/4 = GEMM producer / MMA / epilogue wait expired), clearing
 * it when clear != 0.  No counterpart in the reference, whose kernels wait without bounds. */
int b200fp4_device_status(void* stream, int* status_out, int clear);

#ifdef __cplusplus
}
#endif
#endif /* B200FP4_H_ */
