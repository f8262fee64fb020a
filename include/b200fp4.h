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

#ifdef __cplusplus
}
#endif
#endif /* B200FP4_H_ */
