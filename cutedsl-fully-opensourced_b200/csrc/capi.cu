// C-ABI of libb200fp4: plain pointers and sizes in, status code out.  The
// declarations (with the reference interface each entry point stands in for)
// are in include/b200fp4.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/b200fp4.h"
#include "common.cuh"

namespace b200fp4 {

static thread_local char g_last_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return kOk;
  return fail(kCudaError, "%s: %s", what, cudaGetErrorString(e));
}

int norm_fp4quant_launch(const void* x, void* residual, const void* weight, void* y_fp4, void* block_scale,
                         void* block_scale_unswizzled, const float* global_scale, float eps, int64_t rows,
                         int hidden, int64_t x_row_stride, int64_t res_row_stride, int dtype, int sf_layout,
                         cudaStream_t stream);

int gemm_dense(const void* a, const void* b, const void* sfa, const void* sfb, void* c, const float* alpha, int m, int n,
               int k, int l, int c_dtype, int tile_n, void* workspace, size_t workspace_bytes, int sf_vec, int fmt8,
               cudaStream_t stream);
size_t gemm_workspace_bytes(int m, int n, int k);
int device_status_word(int** out);
int route_topk(const float* logits, int* ids, float* weights, int tokens, int experts, int top_k, int renormalize,
               cudaStream_t stream);
size_t moe_workspace_bytes(int64_t tokens, int hidden, int inter, int experts, int top_k);
int moe_fused(const void* x, const void* w1, const void* w1_sf, const void* w2, const void* w2_sf, int* ids,
              float* route_w, const float* logits, int route_experts, int renormalize, const float* w1_alpha,
              const float* w2_alpha, const float* fc2_input_scale, void* out, int64_t tokens, int hidden, int inter,
              int experts, int top_k, int expert_lo, int accumulate, int out_dtype, void* workspace,
              size_t workspace_bytes, int* status, cudaStream_t stream);
int bounded_wait_selftest(long long limit_cycles, int* gave_up_dev, cudaStream_t stream);

size_t moe_ep_buffer_bytes(int64_t tokens_local, int hidden, int inter, int experts_local, int top_k, int world);
int moe_ep_reset(void* own_buffer, int64_t tokens_local, int hidden, int inter, int experts_local, int top_k,
                 int world, cudaStream_t stream);
int moe_ep_dispatch(const void* x, const int* ids, const float* weights, const float* logits, int route_experts,
                    int renormalize, const void* const* peer_buffers, int rank, int world, int64_t tokens_local,
                    int hidden, int inter, int experts_local, int top_k, int return_mode, double wait_ms, int phases,
                    int* status, cudaStream_t stream);
int moe_ep_compute(const void* const* peer_buffers, int rank, int world, const void* w1, const void* w1_sf,
                   const void* w2, const void* w2_sf, const float* w1_alpha, const float* w2_alpha,
                   const float* fc2_input_scale, int64_t tokens_local, int hidden, int inter, int experts_local,
                   int top_k, int return_mode, double wait_ms, int* status, cudaStream_t stream);
int moe_ep_combine(const void* const* peer_buffers, int rank, int world, const int* ids, const float* weights,
                   void* out, int64_t tokens_local, int hidden, int inter, int experts_local, int top_k,
                   int return_mode, double wait_ms, int* status, cudaStream_t stream);
int moe_ep_routing(const void* own_buffer, int* ids_out, float* weights_out, int64_t tokens_local, int hidden,
                   int inter, int experts_local, int top_k, int world, cudaStream_t stream);
int moe_ep_wait_selftest(void* own_buffer, int world, double wait_ms, int64_t tokens_local, int hidden, int inter,
                         int experts_local, int top_k, int* status, cudaStream_t stream);

}  // namespace b200fp4

using namespace b200fp4;

extern "C" {

const char* b200fp4_last_error(void) { return g_last_error; }

int b200fp4_version(void) { return 1; }

int b200fp4_rmsnorm_fp4quant(const void* x, const void* weight, void* y_fp4, void* block_scale,
                             void* block_scale_unswizzled, const float* global_scale, float eps, int64_t rows,
                             int hidden, int64_t x_row_stride, int dtype, int sf_layout, void* stream) {
  return norm_fp4quant_launch(x, nullptr, weight, y_fp4, block_scale, block_scale_unswizzled, global_scale, eps,
                              rows, hidden, x_row_stride, 0, dtype, sf_layout, static_cast<cudaStream_t>(stream));
}

int b200fp4_add_rmsnorm_fp4quant(const void* x, void* residual, const void* weight, void* y_fp4,
                                 void* block_scale, void* block_scale_unswizzled, const float* global_scale,
                                 float eps, int64_t rows, int hidden, int64_t x_row_stride,
                                 int64_t residual_row_stride, int dtype, int sf_layout, void* stream) {
  if (residual == nullptr) return fail(kInvalidArgument, "residual is null");
  if (residual == x) return fail(kInvalidArgument, "input and residual must not alias");
  return norm_fp4quant_launch(x, residual, weight, y_fp4, block_scale, block_scale_unswizzled, global_scale, eps,
                              rows, hidden, x_row_stride, residual_row_stride, dtype, sf_layout,
                              static_cast<cudaStream_t>(stream));
}

int b200fp4_nvfp4_gemm(const void* a, const void* b, const void* sfa, const void* sfb, void* c, const float* alpha,
                       int m, int n, int k, int l, int c_dtype, int tile_n, void* stream) {
  return gemm_dense(a, b, sfa, sfb, c, alpha, m, n, k, l, c_dtype, tile_n, nullptr, 0, 16, -1, static_cast<cudaStream_t>(stream));
}

int b200fp4_mxfp4_gemm(const void* a, const void* b, const void* sfa, const void* sfb, void* c, const float* alpha,
                       int m, int n, int k, int l, int c_dtype, int tile_n, void* stream) {
  return gemm_dense(a, b, sfa, sfb, c, alpha, m, n, k, l, c_dtype, tile_n, nullptr, 0, 32, -1, static_cast<cudaStream_t>(stream));
}

int b200fp4_mxfp8_gemm(const void* a, const void* b, const void* sfa, const void* sfb, void* c, const float* alpha,
                       int m, int n, int k, int l, int c_dtype, int tile_n, int a_e5m2, int b_e5m2, void* stream) {
  return gemm_dense(a, b, sfa, sfb, c, alpha, m, n, k, l, c_dtype, tile_n, nullptr, 0, 32, (a_e5m2 ? 1 : 0) | (b_e5m2 ? 2 : 0),
                    static_cast<cudaStream_t>(stream));
}

size_t b200fp4_nvfp4_gemm_workspace_bytes(int m, int n, int k) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  return gemm_workspace_bytes(m, n, k);
}

int b200fp4_nvfp4_gemm_ws(const void* a, const void* b, const void* sfa, const void* sfb, void* c, const float* alpha,
                          int m, int n, int k, int l, int c_dtype, int tile_n, void* workspace, size_t workspace_bytes,
                          void* stream) {
  return gemm_dense(a, b, sfa, sfb, c, alpha, m, n, k, l, c_dtype, tile_n, workspace, workspace_bytes, 16, -1,
                    static_cast<cudaStream_t>(stream));
}

int b200fp4_topk_route(const float* logits, int* ids, float* weights, int tokens, int experts, int top_k,
                       int renormalize, void* stream) {
  return route_topk(logits, ids, weights, tokens, experts, top_k, renormalize, static_cast<cudaStream_t>(stream));
}

size_t b200fp4_moe_workspace_bytes(int64_t tokens, int hidden, int intermediate, int local_experts, int top_k) {
  if (tokens < 0 || hidden <= 0 || intermediate <= 0 || local_experts <= 0 || top_k <= 0) return 0;
  return moe_workspace_bytes(tokens, hidden, intermediate, local_experts, top_k);
}

int b200fp4_moe_fused(const void* x, const void* w1, const void* w1_sf, const void* w2, const void* w2_sf,
                      const int* token_selected_experts, const float* token_final_scales, const float* w1_alpha,
                      const float* w2_alpha, const float* fc2_input_scale, void* out, int64_t tokens, int hidden,
                      int intermediate, int local_experts, int top_k, int local_expert_offset, int accumulate,
                      int out_dtype, void* workspace, size_t workspace_bytes, void* stream) {
  int* status = nullptr;
  int rc = device_status_word(&status);
  if (rc) return rc;
  // ids and scales are inputs here: the routed variant below is the one that writes them
  return moe_fused(x, w1, w1_sf, w2, w2_sf, const_cast<int*>(token_selected_experts),
                   const_cast<float*>(token_final_scales), nullptr, 0, 0, w1_alpha, w2_alpha, fc2_input_scale, out,
                   tokens, hidden, intermediate, local_experts, top_k, local_expert_offset, accumulate, out_dtype,
                   workspace, workspace_bytes, status, static_cast<cudaStream_t>(stream));
}

int b200fp4_moe_fused_routed(const void* x, const float* router_logits, int num_experts, int renormalize,
                             const void* w1, const void* w1_sf, const void* w2, const void* w2_sf,
                             int* token_selected_experts_out, float* token_final_scales_out, const float* w1_alpha,
                             const float* w2_alpha, const float* fc2_input_scale, void* out, int64_t tokens,
                             int hidden, int intermediate, int local_experts, int top_k, int local_expert_offset,
                             int accumulate, int out_dtype, void* workspace, size_t workspace_bytes, void* stream) {
  if (router_logits == nullptr) return fail(kInvalidArgument, "router_logits is null");
  int* status = nullptr;
  int rc = device_status_word(&status);
  if (rc) return rc;
  return moe_fused(x, w1, w1_sf, w2, w2_sf, token_selected_experts_out, token_final_scales_out, router_logits,
                   num_experts, renormalize, w1_alpha, w2_alpha, fc2_input_scale, out, tokens, hidden, intermediate,
                   local_experts, top_k, local_expert_offset, accumulate, out_dtype, workspace, workspace_bytes, status,
                   static_cast<cudaStream_t>(stream));
}

size_t b200fp4_moe_ep_buffer_bytes(int64_t tokens_local, int hidden, int intermediate, int local_experts, int top_k,
                                   int world) {
  if (tokens_local < 0 || hidden <= 0 || intermediate <= 0 || local_experts <= 0 || top_k <= 0 || world <= 0) return 0;
  return moe_ep_buffer_bytes(tokens_local, hidden, intermediate, local_experts, top_k, world);
}

int b200fp4_moe_ep_reset(void* own_buffer, int64_t tokens_local, int hidden, int intermediate, int local_experts,
                         int top_k, int world, void* stream) {
  return moe_ep_reset(own_buffer, tokens_local, hidden, intermediate, local_experts, top_k, world,
                      static_cast<cudaStream_t>(stream));
}

static int ep_dispatch_phases(const void* x, const int* ids, const float* scales, const float* logits, int renormalize,
                              const void* const* peer_buffers, int rank, int world, int64_t tokens_local, int hidden,
                              int intermediate, int local_experts, int top_k, int return_mode, double wait_ms,
                              int phases, void* stream) {
  int* status = nullptr;
  int rc = device_status_word(&status);
  if (rc) return rc;
  return moe_ep_dispatch(x, ids, scales, logits, local_experts * world, renormalize, peer_buffers, rank, world,
                         tokens_local, hidden, intermediate, local_experts, top_k, return_mode, wait_ms, phases, status,
                         static_cast<cudaStream_t>(stream));
}

int b200fp4_moe_ep_dispatch(const void* x, const int* token_selected_experts, const float* token_final_scales,
                            const float* router_logits, int renormalize, const void* const* peer_buffers, int rank, int world,
                            int64_t tokens_local, int hidden, int intermediate, int local_experts, int top_k,
                            int return_mode, double wait_ms, void* stream) {
  return ep_dispatch_phases(x, token_selected_experts, token_final_scales, router_logits, renormalize, peer_buffers,
                            rank, world, tokens_local, hidden, intermediate, local_experts, top_k, return_mode, wait_ms,
                            3, stream);
}

int b200fp4_moe_ep_dispatch_count(const void* x, const int* token_selected_experts, const float* token_final_scales,
                                  const float* router_logits, int renormalize, const void* const* peer_buffers, int rank, int world,
                                  int64_t tokens_local, int hidden, int intermediate, int local_experts, int top_k,
                                  int return_mode, double wait_ms, void* stream) {
  return ep_dispatch_phases(x, token_selected_experts, token_final_scales, router_logits, renormalize, peer_buffers,
                            rank, world, tokens_local, hidden, intermediate, local_experts, top_k, return_mode, wait_ms,
                            1, stream);
}

int b200fp4_moe_ep_dispatch_place(const void* x, const int* token_selected_experts, const float* token_final_scales,
                                  const float* router_logits, int renormalize, const void* const* peer_buffers, int rank, int world,
                                  int64_t tokens_local, int hidden, int intermediate, int local_experts, int top_k,
                                  int return_mode, double wait_ms, void* stream) {
  return ep_dispatch_phases(x, token_selected_experts, token_final_scales, router_logits, renormalize, peer_buffers,
                            rank, world, tokens_local, hidden, intermediate, local_experts, top_k, return_mode, wait_ms,
                            2, stream);
}

int b200fp4_moe_ep_compute(const void* const* peer_buffers, int rank, int world, const void* w1, const void* w1_sf,
                           const void* w2, const void* w2_sf, const float* w1_alpha, const float* w2_alpha,
                           const float* fc2_input_scale, int64_t tokens_local, int hidden, int intermediate,
                           int local_experts, int top_k, int return_mode, double wait_ms, void* stream) {
  int* status = nullptr;
  int rc = device_status_word(&status);
  if (rc) return rc;
  return moe_ep_compute(peer_buffers, rank, world, w1, w1_sf, w2, w2_sf, w1_alpha, w2_alpha, fc2_input_scale,
                        tokens_local, hidden, intermediate, local_experts, top_k, return_mode, wait_ms, status,
                        static_cast<cudaStream_t>(stream));
}

int b200fp4_moe_ep_combine(const void* const* peer_buffers, int rank, int world, const int* token_selected_experts,
                           const float* token_final_scales, void* out, int64_t tokens_local, int hidden,
                           int intermediate, int local_experts, int top_k, int return_mode, double wait_ms,
                           void* stream) {
  int* status = nullptr;
  int rc = device_status_word(&status);
  if (rc) return rc;
  return moe_ep_combine(peer_buffers, rank, world, token_selected_experts, token_final_scales, out, tokens_local,
                        hidden, intermediate, local_experts, top_k, return_mode, wait_ms, status,
                        static_cast<cudaStream_t>(stream));
}

int b200fp4_moe_ep_routing(const void* own_buffer, int* ids_out, float* weights_out, int64_t tokens_local, int hidden,
                           int intermediate, int local_experts, int top_k, int world, void* stream) {
  return moe_ep_routing(own_buffer, ids_out, weights_out, tokens_local, hidden, intermediate, local_experts, top_k,
                        world, static_cast<cudaStream_t>(stream));
}

int b200fp4_selftest_peer_wait(void* own_buffer, int world, double wait_ms, int64_t tokens_local, int hidden,
                               int intermediate, int local_experts, int top_k, void* stream) {
  int* status = nullptr;
  int rc = device_status_word(&status);
  if (rc) return rc;
  return moe_ep_wait_selftest(own_buffer, world, wait_ms, tokens_local, hidden, intermediate, local_experts, top_k,
                              status, static_cast<cudaStream_t>(stream));
}

int b200fp4_selftest_bounded_wait(long long limit_cycles, int* gave_up, void* stream) {
  return bounded_wait_selftest(limit_cycles, gave_up, static_cast<cudaStream_t>(stream));
}

int b200fp4_device_status(void* stream, int* status_out, int clear) {
  if (status_out == nullptr) return fail(kInvalidArgument, "status_out is null");
  int* word = nullptr;
  int rc = device_status_word(&word);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_CUDA(cudaMemcpyAsync(status_out, word, sizeof(int), cudaMemcpyDeviceToHost, s));
  if (clear) B200_CUDA(cudaMemsetAsync(word, 0, sizeof(int), s));
  B200_CUDA(cudaStreamSynchronize(s));
  return kOk;
}

}  // extern "C"
