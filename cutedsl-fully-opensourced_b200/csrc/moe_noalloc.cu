// b200fp4_moe_fused_noalloc: the fused NVFP4 MoE for callers that are not allowed to allocate.
//
// Some users of this library run where device memory cannot be requested at call time: inside a
// serving engine that hands all of its HBM to a pool at start-up and forbids cudaMalloc afterwards,
// inside a plugin that is only given raw pointers by its host framework, or in a real-time loop where
// an allocation (an implicit device synchronisation) is not acceptable.  b200fp4_moe_fused asks such a
// caller for a scratch buffer it may have no way to produce.  This variant carries its own scratch:
// a fixed 32 MiB array in the library's device image.  Every GPU that loads the library holds those
// 32 MiB until the process exits; problems whose scratch need
// (b200fp4_moe_workspace_bytes) exceeds it are refused with B200FP4_UNSUPPORTED.
//
// The array's symbol is only a host-side handle here; the address the kernels use is obtained once per
// device with cudaGetSymbolAddress while that device is current.  That look-up happens on the first
// call made on a device, so make that first call outside of any stream capture.
//
// All calls on one GPU share the one array and it keeps whatever the previous call left in it; the parts
// that must start at zero are cleared on the stream at the start of every call.  Two calls whose kernels
// overlap on the same GPU (different streams) would race on the array: serialise them.
#include <mutex>

#include "../../include/b200fp4.h"
#include "common.cuh"

namespace b200fp4 {

size_t moe_workspace_bytes(int64_t tokens, int hidden, int inter, int experts, int top_k);
int moe_fused(const void* x, const void* w1, const void* w1_sf, const void* w2, const void* w2_sf, int* ids,
              float* route_w, const float* logits, int route_experts, int renormalize, const float* w1_alpha,
              const float* w2_alpha, const float* fc2_input_scale, void* out, int64_t tokens, int hidden, int inter,
              int experts, int top_k, int expert_lo, int accumulate, int out_dtype, void* workspace,
              size_t workspace_bytes, int* status, cudaStream_t stream);

namespace {

constexpr size_t kBuiltinScratchBytes = 32u << 20;          // 32 MiB per GPU
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];

std::mutex g_scratch_mutex;
void* g_scratch_addr[64] = {};                               // device address of the array, per device ordinal

// Device address of the built-in scratch on the current device (looked up once per device).
int builtin_scratch(void** out) {
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(kUnsupported, "device ordinal %d", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    B200_CUDA(cudaGetSymbolAddress(&p, g_builtin_scratch));
    if (p == nullptr) return fail(kCudaError, "cudaGetSymbolAddress returned a null address");
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return kOk;
}

}  // namespace
}  // namespace b200fp4

using namespace b200fp4;

extern "C" int b200fp4_moe_fused_noalloc(const void* x, const void* w1, const void* w1_sf, const void* w2,
                                         const void* w2_sf, const int* token_selected_experts,
                                         const float* token_final_scales, const float* w1_alpha,
                                         const float* w2_alpha, const float* fc2_input_scale, void* out,
                                         int64_t tokens, int hidden, int intermediate, int local_experts, int top_k,
                                         int local_expert_offset, int accumulate, int* status_word, void* stream) {
  if (status_word == nullptr) return fail(kInvalidArgument, "status_word is null");
  if (tokens < 0 || hidden <= 0 || intermediate <= 0 || local_experts <= 0 || top_k <= 0)
    return fail(kInvalidArgument,
                "tokens must not be negative; hidden, intermediate, local_experts and top_k must be positive");
  const size_t need = moe_workspace_bytes(tokens, hidden, intermediate, local_experts, top_k);
  if (need > kBuiltinScratchBytes)
    return fail(kUnsupported,
                "this problem needs %zu bytes of scratch but the built-in scratch of b200fp4_moe_fused_noalloc holds "
                "%zu; use b200fp4_moe_fused with your own workspace", need, kBuiltinScratchBytes);
  void* scratch = nullptr;
  int rc = builtin_scratch(&scratch);
  if (rc) return rc;
  return moe_fused(x, w1, w1_sf, w2, w2_sf, const_cast<int*>(token_selected_experts),
                   const_cast<float*>(token_final_scales), nullptr, 0, 0, w1_alpha, w2_alpha, fc2_input_scale, out, tokens, hidden, intermediate, local_experts, top_k, local_expert_offset,
                   accumulate, /*out_dtype=bf16*/ 1, scratch, kBuiltinScratchBytes, status_word,
                   static_cast<cudaStream_t>(stream));
}
