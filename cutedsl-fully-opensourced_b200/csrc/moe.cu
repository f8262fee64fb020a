// Fused NVFP4 MoE for sm_100a: the stages around the two grouped GEMMs.
//
// Stands in for flashinfer's b12x_fused_moe as the reference calls it
// (tests/python/test_flashinfer_b12x_verbatim.py:99-116); arithmetic contract is
// the reference's routed golden (same file, lines 28-65 and 209-219):
//
//   route (optional)   softmax over expert logits -> top-k -> renormalise
//   count / scan       rows per local expert; every expert's segment is padded to whole 128-row
//                      blocks so that a GEMM tile never straddles two experts
//   scatter + quant    each token is quantised ONCE to NVFP4 with the activation packer and its
//                      codes / scale bytes are written to the row of every (token, slot) pair
//   FC1 grouped GEMM   [up | gate] = Xq . W1[e]^T, epilogue silu(gate)*up -> bf16 -> NVFP4   (gemm.cu)
//   FC2 grouped GEMM   partial = Actq . W2[e]^T * w2_alpha[e]                               (gemm.cu)
//   combine            out[t] = bf16( sum_j weight[t,j] * partial[row(t,j)] ), f32, slot order
//
// All intermediate buffers live in a caller-provided workspace.
#include <algorithm>

#include "common.cuh"

namespace b200fp4 {

int gemm_moe_fc1(const void* xq, const void* xq_sf, const void* w1, const void* w1_sf, void* act_codes, void* act_sf,
                 const float* w1_alpha, const float* fc2_input_scale, const int* num_m_blocks_dev,
                 const int* m_block_expert, const int* m_block_rows, int max_m_blocks, int hidden, int inter,
                 int experts, int few_rows, int* status, cudaStream_t stream);
int gemm_moe_fc2(const void* act_codes, const void* act_sf, const void* w2, const void* w2_sf, void* partial,
                 int rows_bf16, const float* w2_alpha, const int* num_m_blocks_dev, const int* m_block_expert,
                 const int* m_block_rows, int max_m_blocks, int hidden, int inter, int experts, int few_rows,
                 int* status, cudaStream_t stream);

namespace {

constexpr int kRouteMaxPerLane = 32;       // experts <= 1024

// ---------------------------------------------------------------------------
// route: one warp per token; kPerLane = experts a lane holds (experts <= 32 * kPerLane)
// ---------------------------------------------------------------------------
template <int kPerLane>
__global__ void route_topk_kernel(const float* __restrict__ logits, int* __restrict__ ids, float* __restrict__ weights,
                                  int tokens, int experts, int top_k, int renormalize) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= tokens) return;
  const float* row = logits + static_cast<int64_t>(warp) * experts;
  float v[kPerLane];
  const int per_lane = (experts + 31) >> 5;
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int e = lane + 32 * i;
    v[i] = (i < per_lane && e < experts) ? row[e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    v[i] = (i < per_lane && lane + 32 * i < experts) ? expf(v[i] - mx) : -1.0f;   // -1 = absent / already taken
    if (v[i] > 0.0f) sum += v[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.0f / sum;
  float picked = 0.0f;
  float my_w = 0.0f;
  int my_id = 0;
  for (int j = 0; j < top_k; ++j) {
    // lane-local best (lowest index among equals), then the warp's best
    float best = -1.0f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      if (i < per_lane && v[i] > best) {
        best = v[i];
        best_e = lane + 32 * i;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kPerLane; ++i)
        if (i == (best_e >> 5)) v[i] = -1.0f;
    }
    const float prob = best * inv;
    picked += prob;
    if (lane == j) {
      my_w = prob;
      my_id = best_e;
    }
  }
  if (lane < top_k) {
    ids[static_cast<int64_t>(warp) * top_k + lane] = my_id;
    weights[static_cast<int64_t>(warp) * top_k + lane] = renormalize ? my_w / picked : my_w;
  }
}

// ---------------------------------------------------------------------------
// bookkeeping header at the start of the workspace
// ---------------------------------------------------------------------------
struct MoeHeader {           // all int32, contiguous
  int* counts;               // [experts]     rows routed to each local expert
  int* cursor;               // [experts]     next free row inside the expert's segment
  int* offsets;              // [experts + 1] first row of each expert's padded segment
  int* num_m_blocks;         // [1]
  int* m_block_expert;       // [max_m_blocks]
  int* m_block_rows;         // [max_m_blocks] rows of the block that hold data (the rest pads it to 128)
  int* slot_row;             // [tokens * top_k] row of every (token, slot), -1 if the expert is not local
};

// rows per local expert: a histogram per CTA in shared memory (experts <= 1024), then one global add per
// expert that the CTA saw
constexpr int kCountSlotsPerCta = 1024;
__global__ void moe_count_kernel(const int* __restrict__ ids, int n_slots, int expert_lo, int experts, int* counts) {
  __shared__ int s_hist[1024];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) s_hist[e] = 0;
  __syncthreads();
  const int first = blockIdx.x * kCountSlotsPerCta;
  const int last = min(n_slots, first + kCountSlotsPerCta);
  for (int i = first + threadIdx.x; i < last; i += blockDim.x) {
    const int e = ids[i] - expert_lo;
    if (e >= 0 && e < experts) atomicAdd(s_hist + e, 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x)
    if (s_hist[e] != 0) atomicAdd(counts + e, s_hist[e]);
}

// single CTA: padded exclusive scan over experts and the block -> expert table
__global__ void moe_scan_kernel(MoeHeader h, int experts, int max_m_blocks) {
  __shared__ int s_blocks[1024];
  const int t = threadIdx.x;
  int blocks = 0;
  if (t < experts) blocks = (h.counts[t] + 127) >> 7;
  s_blocks[t] = blocks;
  __syncthreads();
  // Hillis-Steele inclusive scan over up to 1024 experts
  for (int o = 1; o < 1024; o <<= 1) {
    const int add = t >= o ? s_blocks[t - o] : 0;
    __syncthreads();
    s_blocks[t] += add;
    __syncthreads();
  }
  const int incl = s_blocks[t];
  const int excl = incl - blocks;
  if (t < experts) {
    h.offsets[t] = excl * 128;
    h.cursor[t] = 0;
    const int count = h.counts[t];
    for (int b = 0; b < blocks; ++b) {
      if (excl + b < max_m_blocks) {
        h.m_block_expert[excl + b] = t;
        h.m_block_rows[excl + b] = min(128, count - 128 * b);
      }
    }
  }
  if (t == experts - 1) {
    h.offsets[experts] = incl * 128;
    *h.num_m_blocks = min(incl, max_m_blocks);
  }
}

// Few slots (<= 1024): count, scan and row assignment in one CTA -- one launch instead of a memset and three
// kernels, which is most of a decode step's bookkeeping time.  Rows of an expert go to its slots in slot order.
__global__ void __launch_bounds__(1024) moe_prepare_small_kernel(const int* __restrict__ ids, int n_slots, int expert_lo,
                                                                 MoeHeader h, int experts, int max_m_blocks,
                                                                 int max_rows) {
  __shared__ int s_count[1024];
  __shared__ int s_blocks[1024];
  __shared__ int s_offset[1024];
  __shared__ int s_expert[1024];
  const int t = threadIdx.x;
  s_count[t] = 0;
  int e = -1, rank_in_expert = 0;
  if (t < n_slots) {
    e = ids[t] - expert_lo;
    if (e < 0 || e >= experts) e = -1;
  }
  s_expert[t] = e;
  __syncthreads();
  // position of the slot among the slots of its expert, in slot order: count earlier slots with the same expert
  if (e >= 0) {
    atomicAdd(s_count + e, 1);
    for (int i = 0; i < t; ++i) rank_in_expert += s_expert[i] == e;
  }
  __syncthreads();
  const int count = t < experts ? s_count[t] : 0;
  const int blocks = (count + 127) >> 7;
  s_blocks[t] = blocks;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    const int add = t >= o ? s_blocks[t - o] : 0;
    __syncthreads();
    s_blocks[t] += add;
    __syncthreads();
  }
  const int incl = s_blocks[t];
  const int excl = incl - blocks;
  s_offset[t] = excl * 128;
  if (t < experts) {
    h.counts[t] = count;
    h.offsets[t] = excl * 128;
    h.cursor[t] = count;
    for (int b = 0; b < blocks; ++b) {
      if (excl + b < max_m_blocks) {
        h.m_block_expert[excl + b] = t;
        h.m_block_rows[excl + b] = min(128, count - 128 * b);
      }
    }
  }
  if (t == experts - 1) {
    h.offsets[experts] = incl * 128;
    *h.num_m_blocks = min(incl, max_m_blocks);
  }
  __syncthreads();
  if (t < n_slots) {
    int row = -1;
    if (e >= 0) {
      row = s_offset[e] + rank_in_expert;
      if (row >= max_rows) row = -1;
    }
    h.slot_row[t] = row;
  }
}

// CTA (token, part): quantise a share of the row's 16-element blocks and write it to the rows assigned above
template <int kThreads>
__global__ void __launch_bounds__(kThreads)
moe_scatter_quant_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ slot_row, uint8_t* xq,
                              uint8_t* xq_sf, int hidden, int top_k) {
  __shared__ int s_rows[64];
  const int token = blockIdx.x;
  if (threadIdx.x < top_k) s_rows[threadIdx.x] = slot_row[static_cast<int64_t>(token) * top_k + threadIdx.x];
  __syncthreads();
  const int nchunks = hidden >> 4;
  const int rk = (nchunks + 3) >> 2;
  for (int chunk = blockIdx.y * kThreads + threadIdx.x; chunk < nchunks; chunk += gridDim.y * kThreads) {
    const U32x8 raw = ld_stream_32B(x + static_cast<int64_t>(token) * hidden + chunk * 16);
    float v[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[2 * i] = Pair16<__nv_bfloat16>::lo(raw.v[i]);
      v[2 * i + 1] = Pair16<__nv_bfloat16>::hi(raw.v[i]);
    }
    uint32_t lo, hi, sfb;
    quantize_block16<true>(v, 1.0f, lo, hi, sfb);
    for (int j = 0; j < top_k; ++j) {
      const int row = s_rows[j];
      if (row < 0) continue;
      *reinterpret_cast<uint2*>(xq + static_cast<int64_t>(row) * (hidden >> 1) + chunk * 8) = make_uint2(lo, hi);
      xq_sf[sf_swizzled_offset(row, chunk, rk)] = static_cast<uint8_t>(sfb);
    }
  }
}

// one CTA per token: quantise the row once, then write it to the row of every local slot
template <int kThreads>
__global__ void __launch_bounds__(kThreads)
moe_scatter_quant_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids, MoeHeader h, uint8_t* xq,
                         uint8_t* xq_sf, int hidden, int top_k, int expert_lo, int experts, int max_rows) {
  __shared__ int s_rows[64];
  const int token = blockIdx.x;
  if (threadIdx.x < top_k) {
    const int e = ids[static_cast<int64_t>(token) * top_k + threadIdx.x] - expert_lo;
    int row = -1;
    if (e >= 0 && e < experts) {
      row = h.offsets[e] + atomicAdd(h.cursor + e, 1);
      if (row >= max_rows) row = -1;
    }
    s_rows[threadIdx.x] = row;
    h.slot_row[static_cast<int64_t>(token) * top_k + threadIdx.x] = row;
  }
  __syncthreads();
  const int nchunks = hidden >> 4;
  const int rk = (nchunks + 3) >> 2;
  for (int chunk = threadIdx.x; chunk < nchunks; chunk += kThreads) {
    const U32x8 raw = ld_stream_32B(x + static_cast<int64_t>(token) * hidden + chunk * 16);
    float v[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[2 * i] = Pair16<__nv_bfloat16>::lo(raw.v[i]);
      v[2 * i + 1] = Pair16<__nv_bfloat16>::hi(raw.v[i]);
    }
    uint32_t lo, hi, sfb;
    quantize_block16<true>(v, 1.0f, lo, hi, sfb);
    for (int j = 0; j < top_k; ++j) {
      const int row = s_rows[j];
      if (row < 0) continue;
      *reinterpret_cast<uint2*>(xq + static_cast<int64_t>(row) * (hidden >> 1) + chunk * 8) = make_uint2(lo, hi);
      xq_sf[sf_swizzled_offset(row, chunk, rk)] = static_cast<uint8_t>(sfb);
    }
  }
}

// four consecutive elements of a per-slot output row (f32 or bf16 storage) as f32
template <typename RowT>
__device__ __forceinline__ float4 load_row4(const RowT* p) {
  if constexpr (sizeof(RowT) == 4) {
    return *reinterpret_cast<const float4*>(p);
  } else {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    return make_float4(Pair16<__nv_bfloat16>::lo(u.x), Pair16<__nv_bfloat16>::hi(u.x), Pair16<__nv_bfloat16>::lo(u.y),
                       Pair16<__nv_bfloat16>::hi(u.y));
  }
}

// one CTA per token; every thread owns 4 output columns at a time
template <typename OutT, typename RowT>
__global__ void moe_combine_kernel(const RowT* __restrict__ partial, const int* __restrict__ slot_row,
                                   const float* __restrict__ weights, OutT* __restrict__ out, int hidden,
                                   int top_k, int accumulate) {
  __shared__ int s_rows[64];
  __shared__ float s_w[64];
  const int token = blockIdx.x;
  if (threadIdx.x < top_k) {
    s_rows[threadIdx.x] = slot_row[static_cast<int64_t>(token) * top_k + threadIdx.x];
    s_w[threadIdx.x] = weights[static_cast<int64_t>(token) * top_k + threadIdx.x];
  }
  __syncthreads();
  for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < top_k; ++j) {
      const int row = s_rows[j];
      if (row < 0) continue;
      const float4 pv = load_row4(partial + static_cast<int64_t>(row) * hidden + c);
      const float w = s_w[j];
      acc.x = __fadd_rn(acc.x, __fmul_rn(w, pv.x));
      acc.y = __fadd_rn(acc.y, __fmul_rn(w, pv.y));
      acc.z = __fadd_rn(acc.z, __fmul_rn(w, pv.z));
      acc.w = __fadd_rn(acc.w, __fmul_rn(w, pv.w));
    }
    OutT* o = out + static_cast<int64_t>(token) * hidden + c;
    if constexpr (sizeof(OutT) == 4) {
      if (accumulate) {
        const float4 prev = *reinterpret_cast<const float4*>(o);
        acc.x += prev.x;
        acc.y += prev.y;
        acc.z += prev.z;
        acc.w += prev.w;
      }
      *reinterpret_cast<float4*>(o) = acc;
    } else {
      if (accumulate) {
        acc.x += __bfloat162float(o[0]);
        acc.y += __bfloat162float(o[1]);
        acc.z += __bfloat162float(o[2]);
        acc.w += __bfloat162float(o[3]);
      }
      uint2 packed;
      packed.x = Pair16<__nv_bfloat16>::pack(acc.x, acc.y);
      packed.y = Pair16<__nv_bfloat16>::pack(acc.z, acc.w);
      *reinterpret_cast<uint2*>(o) = packed;
    }
  }
}

// The same for few tokens: CTA (token, column chunk), every thread owns 4 output columns and reads the k rows
// with independent loads (a decode step with one token is nothing but the latency of these reads; with thousands
// of tokens the plain kernel above is faster).
template <typename OutT, typename RowT>
__global__ void moe_combine_few_kernel(const RowT* __restrict__ partial, const int* __restrict__ slot_row,
                                   const float* __restrict__ weights, OutT* __restrict__ out, int hidden,
                                   int top_k, int accumulate) {
  __shared__ int s_rows[64];
  __shared__ float s_w[64];
  const int token = blockIdx.x;
  if (threadIdx.x < top_k) {
    s_rows[threadIdx.x] = slot_row[static_cast<int64_t>(token) * top_k + threadIdx.x];
    s_w[threadIdx.x] = weights[static_cast<int64_t>(token) * top_k + threadIdx.x];
  }
  __syncthreads();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (c >= hidden) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j0 = 0; j0 < top_k; j0 += 8) {
    float4 pv[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int row = j0 + u < top_k ? s_rows[j0 + u] : -1;
      pv[u] = row >= 0 ? load_row4(partial + static_cast<int64_t>(row) * hidden + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (j0 + u < top_k && s_rows[j0 + u] >= 0) {      // slot order, one product and one sum per slot
        const float w = s_w[j0 + u];
        acc.x = __fadd_rn(acc.x, __fmul_rn(w, pv[u].x));
        acc.y = __fadd_rn(acc.y, __fmul_rn(w, pv[u].y));
        acc.z = __fadd_rn(acc.z, __fmul_rn(w, pv[u].z));
        acc.w = __fadd_rn(acc.w, __fmul_rn(w, pv[u].w));
      }
    }
  }
  OutT* o = out + static_cast<int64_t>(token) * hidden + c;
  if constexpr (sizeof(OutT) == 4) {
    if (accumulate) {
      const float4 prev = *reinterpret_cast<const float4*>(o);
      acc.x += prev.x;
      acc.y += prev.y;
      acc.z += prev.z;
      acc.w += prev.w;
    }
    *reinterpret_cast<float4*>(o) = acc;
  } else {
    if (accumulate) {
      acc.x += __bfloat162float(o[0]);
      acc.y += __bfloat162float(o[1]);
      acc.z += __bfloat162float(o[2]);
      acc.w += __bfloat162float(o[3]);
    }
    uint2 packed;
    packed.x = Pair16<__nv_bfloat16>::pack(acc.x, acc.y);
    packed.y = Pair16<__nv_bfloat16>::pack(acc.z, acc.w);
    *reinterpret_cast<uint2*>(o) = packed;
  }
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct MoeWorkspace {
  MoeHeader h;
  uint8_t* xq;
  uint8_t* xq_sf;
  uint8_t* act;
  uint8_t* act_sf;
  float* partial;
  size_t header_bytes;     // counts .. slot_row
  size_t xq_sf_bytes;
  size_t total;
  int max_m_blocks;
};

MoeWorkspace carve(void* base, int64_t tokens, int hidden, int inter, int experts, int top_k) {
  MoeWorkspace w{};
  const int64_t slots = tokens * top_k;
  const int64_t blocks = std::min<int64_t>(experts, slots) + slots / 128;
  w.max_m_blocks = static_cast<int>(blocks);
  const int64_t rows = blocks * 128;
  uint8_t* p = static_cast<uint8_t*>(base);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    uint8_t* r = p == nullptr ? nullptr : p + off;
    off = align_up(off + bytes, 256);
    return r;
  };
  w.h.counts = reinterpret_cast<int*>(take(sizeof(int) * experts));
  w.h.cursor = reinterpret_cast<int*>(take(sizeof(int) * experts));
  w.h.offsets = reinterpret_cast<int*>(take(sizeof(int) * (experts + 1)));
  w.h.num_m_blocks = reinterpret_cast<int*>(take(sizeof(int)));
  w.h.m_block_expert = reinterpret_cast<int*>(take(sizeof(int) * blocks));
  w.h.m_block_rows = reinterpret_cast<int*>(take(sizeof(int) * blocks));
  w.h.slot_row = reinterpret_cast<int*>(take(sizeof(int) * slots));
  w.header_bytes = off;
  w.xq_sf_bytes = static_cast<size_t>(blocks) * ((hidden + 63) / 64) * 512;
  w.xq_sf = take(w.xq_sf_bytes);
  w.xq = take(static_cast<size_t>(rows) * (hidden / 2));
  w.act_sf = take(static_cast<size_t>(blocks) * ((inter + 63) / 64) * 512);
  w.act = take(static_cast<size_t>(rows) * (inter / 2));
  w.partial = reinterpret_cast<float*>(take(static_cast<size_t>(rows) * hidden * sizeof(float)));
  w.total = off;
  return w;
}

}  // namespace

int route_topk(const float* logits, int* ids, float* weights, int tokens, int experts, int top_k, int renormalize,
               cudaStream_t stream) {
  if (logits == nullptr || ids == nullptr || weights == nullptr) return fail(kInvalidArgument, "null pointer argument");
  if (tokens < 0 || experts < 1 || top_k < 1 || top_k > 32 || top_k > experts)
    return fail(kInvalidArgument, "tokens=%d experts=%d top_k=%d", tokens, experts, top_k);
  if (experts > 32 * kRouteMaxPerLane) return fail(kUnsupported, "experts=%d exceeds %d", experts, 32 * kRouteMaxPerLane);
  if (tokens == 0) return kOk;
  const int warps_per_cta = 4;
  const dim3 grid((tokens + warps_per_cta - 1) / warps_per_cta), block(32 * warps_per_cta);
  if (experts <= 64)
    route_topk_kernel<2><<<grid, block, 0, stream>>>(logits, ids, weights, tokens, experts, top_k, renormalize);
  else if (experts <= 128)
    route_topk_kernel<4><<<grid, block, 0, stream>>>(logits, ids, weights, tokens, experts, top_k, renormalize);
  else if (experts <= 256)
    route_topk_kernel<8><<<grid, block, 0, stream>>>(logits, ids, weights, tokens, experts, top_k, renormalize);
  else
    route_topk_kernel<kRouteMaxPerLane><<<grid, block, 0, stream>>>(logits, ids, weights, tokens, experts, top_k,
                                                                     renormalize);
  return check_cuda(cudaGetLastError(), "route_topk_kernel launch");
}

size_t moe_workspace_bytes(int64_t tokens, int hidden, int inter, int experts, int top_k) {
  return carve(nullptr, tokens, hidden, inter, experts, top_k).total;
}

// status: device word that the GEMM kernels OR failure bits into.
// experts = number of LOCAL experts (w1/w2/alphas hold exactly those); token_selected_experts holds global
// ids, of which [expert_lo, expert_lo + experts) are served here.  accumulate != 0 adds into `out`.
int moe_fused(const void* x, const void* w1, const void* w1_sf, const void* w2, const void* w2_sf, const int* ids,
              const float* route_w, const float* w1_alpha, const float* w2_alpha, const float* fc2_input_scale,
              void* out, int64_t tokens, int hidden, int inter, int experts, int top_k, int expert_lo,
              int accumulate, int out_dtype, void* workspace, size_t workspace_bytes, int* status,
              cudaStream_t stream) {
  if (out_dtype < 1 || out_dtype > 3)
    return fail(kUnsupported, "out_dtype code %d (1 bf16, 2 f32, 3 bf16 with bf16 per-slot rows)", out_dtype);
  const int rows_bf16 = out_dtype == 3;
  if (x == nullptr || w1 == nullptr || w1_sf == nullptr || w2 == nullptr || w2_sf == nullptr || ids == nullptr ||
      route_w == nullptr || out == nullptr || workspace == nullptr || status == nullptr)
    return fail(kInvalidArgument, "null pointer argument");
  if (tokens < 0 || top_k < 1 || top_k > 64 || experts < 1 || experts > 1024)
    return fail(kInvalidArgument, "tokens=%lld top_k=%d experts=%d", static_cast<long long>(tokens), top_k, experts);
  if (hidden % 64 != 0 || hidden < 64) return fail(kUnsupported, "hidden=%d must be a multiple of 64", hidden);
  if (inter % 128 != 0 || inter < 128) return fail(kUnsupported, "intermediate=%d must be a multiple of 128", inter);
  if ((reinterpret_cast<uintptr_t>(x) & 31) || (reinterpret_cast<uintptr_t>(workspace) & 255) ||
      ((reinterpret_cast<uintptr_t>(w1) | reinterpret_cast<uintptr_t>(w2) | reinterpret_cast<uintptr_t>(w1_sf) |
        reinterpret_cast<uintptr_t>(w2_sf)) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return fail(kInvalidArgument, "misaligned pointer (x 32 B, weights 16 B, workspace 256 B, out 16 B)");
  if (tokens * top_k > (1ll << 30)) return fail(kUnsupported, "too many routed rows");
  if (tokens == 0) return kOk;
  MoeWorkspace ws = carve(workspace, tokens, hidden, inter, experts, top_k);
  if (workspace_bytes < ws.total)
    return fail(kInvalidArgument, "workspace holds %zu bytes, %zu needed", workspace_bytes, ws.total);
  const int slots = static_cast<int>(tokens * top_k);
  const int max_rows = ws.max_m_blocks * 128;

  B200_CUDA(cudaMemsetAsync(ws.xq_sf, 0, ws.xq_sf_bytes, stream));      // rows that only pad a block read as zero
  if (slots <= 1024) {
    moe_prepare_small_kernel<<<1, 1024, 0, stream>>>(ids, slots, expert_lo, ws.h, experts, ws.max_m_blocks, max_rows);
    const int parts = std::max(1, std::min(8, (hidden / 16) / 128));
    moe_scatter_quant_rows_kernel<128><<<dim3(static_cast<unsigned>(tokens), parts), 128, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), ws.h.slot_row, ws.xq, ws.xq_sf, hidden, top_k);
  } else {
    B200_CUDA(cudaMemsetAsync(ws.h.counts, 0, sizeof(int) * experts, stream));
    moe_count_kernel<<<(slots + kCountSlotsPerCta - 1) / kCountSlotsPerCta, 256, 0, stream>>>(ids, slots, expert_lo,
                                                                                                experts, ws.h.counts);
    moe_scan_kernel<<<1, 1024, 0, stream>>>(ws.h, experts, ws.max_m_blocks);
    moe_scatter_quant_kernel<128><<<static_cast<unsigned>(tokens), 128, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), ids, ws.h, ws.xq, ws.xq_sf, hidden, top_k, expert_lo, experts, max_rows);
  }
  B200_CUDA(cudaGetLastError());
  // With at most 32 tokens no expert receives more than 32 rows (a token names an expert once, as top-k selection
  // does): the wide GEMM variants then keep 32 rows of A per stage and one more stage of weights in flight.  A
  // row block that breaks the assumption raises bit 8 of the device status word instead of passing unnoticed.
  const int few_rows = tokens <= 32;
  int rc = gemm_moe_fc1(ws.xq, ws.xq_sf, w1, w1_sf, ws.act, ws.act_sf, w1_alpha, fc2_input_scale, ws.h.num_m_blocks,
                        ws.h.m_block_expert, ws.h.m_block_rows, ws.max_m_blocks, hidden, inter, experts, few_rows,
                        status, stream);
  if (rc) return rc;
  rc = gemm_moe_fc2(ws.act, ws.act_sf, w2, w2_sf, ws.partial, rows_bf16, w2_alpha, ws.h.num_m_blocks, ws.h.m_block_expert,
                    ws.h.m_block_rows, ws.max_m_blocks, hidden, inter, experts, few_rows, status, stream);
  if (rc) return rc;
  const int threads = hidden / 4 >= 256 ? 256 : 128;
  if (tokens <= 256 && out_dtype == 3) {
    const dim3 cgrid(static_cast<unsigned>(tokens), (hidden / 4 + threads - 1) / threads);
    moe_combine_few_kernel<__nv_bfloat16, __nv_bfloat16><<<cgrid, threads, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(ws.partial), ws.h.slot_row, route_w, static_cast<__nv_bfloat16*>(out),
        hidden, top_k, accumulate);
  } else if (out_dtype == 2) {
    moe_combine_kernel<float, float><<<static_cast<unsigned>(tokens), threads, 0, stream>>>(
        ws.partial, ws.h.slot_row, route_w, static_cast<float*>(out), hidden, top_k, accumulate);
  } else if (rows_bf16) {
    moe_combine_kernel<__nv_bfloat16, __nv_bfloat16><<<static_cast<unsigned>(tokens), threads, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(ws.partial), ws.h.slot_row, route_w, static_cast<__nv_bfloat16*>(out),
        hidden, top_k, accumulate);
  } else {
    moe_combine_kernel<__nv_bfloat16, float><<<static_cast<unsigned>(tokens), threads, 0, stream>>>(
        ws.partial, ws.h.slot_row, route_w, static_cast<__nv_bfloat16*>(out), hidden, top_k, accumulate);
  }
  return check_cuda(cudaGetLastError(), "moe_combine_kernel launch");
}

}  // namespace b200fp4

// =============================================================================================
// Expert parallelism over peer memory.
//
// Every rank owns a slice of the token batch and a contiguous range of experts.  All ranks hold a
// buffer of identical layout that the others can address (peer pointers: NVLink loads, no
// multimem, no TMA from peer memory).  One step is three launches per rank, separated by two
// cross-rank barriers that the caller provides:
//
//   stage      quantise the local tokens ONCE to NVFP4 and publish codes, scale bytes and expert
//              ids in the own buffer                                                   -- barrier --
//   compute    count the slots of ALL ranks' tokens that hit local experts, lay the rows out,
//              pull the quantised rows over NVLink straight into the expert-major GEMM operand
//              (4.5 bits per element cross the wire instead of 16), FC1, FC2, then send every
//              output row home: whole 8 KB rows written into the buffer of the rank that owns the
//              token (coalesced peer stores; row-strided 32-byte stores from inside the GEMM
//              epilogue were measured 2x slower end to end)                            -- barrier --
//   combine    every rank sums the k rows that arrived for each of its tokens (local memory),
//              one bf16 rounding
//
// The reference has no multi-GPU path; this is the dispatch / combine all-to-all of an
// expert-parallel MoE written as kernels over peer memory.
// =============================================================================================
namespace b200fp4 {
namespace {

constexpr int kMaxPeers = 16;
struct PeerPtrs {
  uint8_t* p[kMaxPeers];
};

struct EpLayout {
  // published for peers: the rank's quantised tokens, and the landing zone of its tokens' output rows
  size_t tok_codes, tok_sf, tok_ids, recv;
  // private to the rank
  size_t partial, row_dst, counts, cursor, offsets, num_m_blocks, m_block_expert, m_block_rows, xq_sf, xq, act_sf, act;
  size_t xq_sf_bytes, total;
  int max_m_blocks;
};

EpLayout ep_layout(int64_t tokens_local, int hidden, int inter, int experts_local, int top_k, int world) {
  EpLayout L{};
  const int64_t slots = tokens_local * world * top_k;
  const int64_t blocks = std::min<int64_t>(experts_local, slots) + slots / 128;
  L.max_m_blocks = static_cast<int>(blocks);
  const int64_t rows = blocks * 128;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t r = off;
    off = align_up(off + bytes, 256);
    return r;
  };
  L.tok_codes = take(static_cast<size_t>(tokens_local) * (hidden / 2));
  L.tok_sf = take(static_cast<size_t>(tokens_local) * (hidden / 16));
  L.tok_ids = take(sizeof(int) * tokens_local * top_k);
  // per-slot output rows cross NVLink and are summed as bf16 rows (f32 accumulation in the combine)
  L.recv = take(static_cast<size_t>(tokens_local) * top_k * hidden * sizeof(__nv_bfloat16));
  L.partial = take(static_cast<size_t>(rows) * hidden * sizeof(__nv_bfloat16));
  L.row_dst = take(sizeof(void*) * rows);
  L.counts = take(sizeof(int) * experts_local);
  L.cursor = take(sizeof(int) * experts_local);
  L.offsets = take(sizeof(int) * (experts_local + 1));
  L.num_m_blocks = take(sizeof(int));
  L.m_block_expert = take(sizeof(int) * blocks);
  L.m_block_rows = take(sizeof(int) * blocks);
  L.xq_sf_bytes = static_cast<size_t>(blocks) * ((hidden + 63) / 64) * 512;
  L.xq_sf = take(L.xq_sf_bytes);
  L.xq = take(static_cast<size_t>(rows) * (hidden / 2));
  L.act_sf = take(static_cast<size_t>(blocks) * ((inter + 63) / 64) * 512);
  L.act = take(static_cast<size_t>(rows) * (inter / 2));
  L.total = off;
  return L;
}

// one CTA per local token: NVFP4 codes + row-major scale bytes + the token's expert ids
template <int kThreads>
__global__ void __launch_bounds__(kThreads)
ep_stage_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids, uint8_t* tok_codes, uint8_t* tok_sf,
                int* tok_ids, int hidden, int top_k) {
  const int token = blockIdx.x;
  if (threadIdx.x < top_k)
    tok_ids[static_cast<int64_t>(token) * top_k + threadIdx.x] = ids[static_cast<int64_t>(token) * top_k + threadIdx.x];
  const int nchunks = hidden >> 4;
  for (int chunk = threadIdx.x; chunk < nchunks; chunk += kThreads) {
    const U32x8 raw = ld_stream_32B(x + static_cast<int64_t>(token) * hidden + chunk * 16);
    uint64_t v2[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v2[i] = pair16_to_f32x2<__nv_bfloat16>(raw.v[i]);
    uint32_t lo, hi, sfb;
    quantize_block16<true>(v2, 1.0f, lo, hi, sfb);
    *reinterpret_cast<uint2*>(tok_codes + static_cast<int64_t>(token) * (hidden >> 1) + chunk * 8) = make_uint2(lo, hi);
    tok_sf[static_cast<int64_t>(token) * nchunks + chunk] = static_cast<uint8_t>(sfb);
  }
}

__global__ void ep_count_kernel(PeerPtrs peers, size_t tok_ids_off, int slots_per_rank, int world, int expert_lo,
                                int experts, int* counts) {
  __shared__ int s_hist[1024];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) s_hist[e] = 0;
  __syncthreads();
  const int total = slots_per_rank * world;
  const int first = blockIdx.x * kCountSlotsPerCta;
  const int last = min(total, first + kCountSlotsPerCta);
  for (int i = first + threadIdx.x; i < last; i += blockDim.x) {
    const int src = i / slots_per_rank;
    const int* ids = reinterpret_cast<const int*>(peers.p[src] + tok_ids_off);
    const int e = ids[i - src * slots_per_rank] - expert_lo;
    if (e >= 0 && e < experts) atomicAdd(s_hist + e, 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x)
    if (s_hist[e] != 0) atomicAdd(counts + e, s_hist[e]);
}

// one CTA per token of ANY rank: rows for its local slots, then the quantised row is pulled from its owner
template <int kThreads>
__global__ void __launch_bounds__(kThreads)
ep_gather_kernel(PeerPtrs peers, EpLayout L, MoeHeader h, __nv_bfloat16** row_dst, uint8_t* xq, uint8_t* xq_sf,
                 int tokens_local, int hidden, int top_k, int expert_lo, int experts, int max_rows) {
  __shared__ int s_rows[64];
  __shared__ int s_any;
  const int g = blockIdx.x;                        // global token index
  const int src = g / tokens_local;
  const int t = g - src * tokens_local;
  const uint8_t* peer = peers.p[src];
  if (threadIdx.x == 0) s_any = 0;
  __syncthreads();
  if (threadIdx.x < top_k) {
    const int e = reinterpret_cast<const int*>(peer + L.tok_ids)[static_cast<int64_t>(t) * top_k + threadIdx.x] - expert_lo;
    int row = -1;
    if (e >= 0 && e < experts) {
      row = h.offsets[e] + atomicAdd(h.cursor + e, 1);
      if (row >= max_rows) row = -1;
    }
    s_rows[threadIdx.x] = row;
    if (row >= 0) {
      s_any = 1;
      // the output row of this slot goes home: slot (t, j) of rank src
      row_dst[row] = reinterpret_cast<__nv_bfloat16*>(peers.p[src] + L.recv) +
                     (static_cast<int64_t>(t) * top_k + threadIdx.x) * hidden;
    }
  }
  __syncthreads();
  if (!s_any) return;
  const int nchunks = hidden >> 4;
  const int rk = (nchunks + 3) >> 2;
  const uint8_t* codes = peer + L.tok_codes + static_cast<int64_t>(t) * (hidden >> 1);
  const uint8_t* sf = peer + L.tok_sf + static_cast<int64_t>(t) * nchunks;
  for (int chunk = threadIdx.x; chunk < nchunks; chunk += kThreads) {
    const uint2 c = *reinterpret_cast<const uint2*>(codes + chunk * 8);
    const uint8_t s = sf[chunk];
    for (int j = 0; j < top_k; ++j) {
      const int row = s_rows[j];
      if (row < 0) continue;
      *reinterpret_cast<uint2*>(xq + static_cast<int64_t>(row) * (hidden >> 1) + chunk * 8) = c;
      xq_sf[sf_swizzled_offset(row, chunk, rk)] = s;
    }
  }
}

// one CTA per row of the expert-major output (bf16): copy it to the landing zone of the token's rank
__global__ void ep_return_rows_kernel(const __nv_bfloat16* __restrict__ partial,
                                      __nv_bfloat16* const* __restrict__ row_dst,
                                      const int* __restrict__ num_m_blocks, const int* __restrict__ m_block_rows,
                                      int hidden) {
  const int blk = blockIdx.x >> 7;
  const int r = blockIdx.x & 127;
  if (blk >= __ldg(num_m_blocks) || r >= __ldg(m_block_rows + blk)) return;
  const int64_t row = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(partial + row * hidden);
  uint4* dst = reinterpret_cast<uint4*>(row_dst[row]);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
}

// one CTA per local token: its k output rows have been delivered into this rank's own buffer
__global__ void ep_combine_kernel(const __nv_bfloat16* __restrict__ recv, const float* __restrict__ weights,
                                  __nv_bfloat16* __restrict__ out, int hidden, int top_k) {
  __shared__ float s_w[64];
  const int t = blockIdx.x;
  if (threadIdx.x < top_k) s_w[threadIdx.x] = weights[static_cast<int64_t>(t) * top_k + threadIdx.x];
  __syncthreads();
  const __nv_bfloat16* rows = recv + static_cast<int64_t>(t) * top_k * hidden;
  for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < top_k; ++j) {
      const float4 pv = load_row4(rows + static_cast<int64_t>(j) * hidden + c);
      const float w = s_w[j];
      acc.x = __fadd_rn(acc.x, __fmul_rn(w, pv.x));
      acc.y = __fadd_rn(acc.y, __fmul_rn(w, pv.y));
      acc.z = __fadd_rn(acc.z, __fmul_rn(w, pv.z));
      acc.w = __fadd_rn(acc.w, __fmul_rn(w, pv.w));
    }
    uint2 packed;
    packed.x = Pair16<__nv_bfloat16>::pack(acc.x, acc.y);
    packed.y = Pair16<__nv_bfloat16>::pack(acc.z, acc.w);
    *reinterpret_cast<uint2*>(out + static_cast<int64_t>(t) * hidden + c) = packed;
  }
}

// CTA (local token, column chunk): the token's k output rows have been delivered into this rank's own buffer
__global__ void ep_combine_few_kernel(const __nv_bfloat16* __restrict__ recv, const float* __restrict__ weights,
                                  __nv_bfloat16* __restrict__ out, int hidden, int top_k) {
  __shared__ float s_w[64];
  const int t = blockIdx.x;
  if (threadIdx.x < top_k) s_w[threadIdx.x] = weights[static_cast<int64_t>(t) * top_k + threadIdx.x];
  __syncthreads();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (c >= hidden) return;
  const __nv_bfloat16* rows = recv + static_cast<int64_t>(t) * top_k * hidden;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j0 = 0; j0 < top_k; j0 += 8) {
    float4 pv[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      pv[u] = j0 + u < top_k ? load_row4(rows + static_cast<int64_t>(j0 + u) * hidden + c) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (j0 + u < top_k) {
        const float w = s_w[j0 + u];
        acc.x = __fadd_rn(acc.x, __fmul_rn(w, pv[u].x));
        acc.y = __fadd_rn(acc.y, __fmul_rn(w, pv[u].y));
        acc.z = __fadd_rn(acc.z, __fmul_rn(w, pv[u].z));
        acc.w = __fadd_rn(acc.w, __fmul_rn(w, pv[u].w));
      }
    }
  }
  uint2 packed;
  packed.x = Pair16<__nv_bfloat16>::pack(acc.x, acc.y);
  packed.y = Pair16<__nv_bfloat16>::pack(acc.z, acc.w);
  *reinterpret_cast<uint2*>(out + static_cast<int64_t>(t) * hidden + c) = packed;
}

int ep_check(int64_t tokens_local, int hidden, int inter, int experts_local, int top_k, int world, int rank) {
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
    return fail(kInvalidArgument, "world=%d rank=%d (at most %d ranks)", world, rank, kMaxPeers);
  if (tokens_local < 0 || top_k < 1 || top_k > 64 || experts_local < 1 || experts_local > 1024)
    return fail(kInvalidArgument, "tokens=%lld top_k=%d experts=%d", static_cast<long long>(tokens_local), top_k,
                experts_local);
  if (hidden % 64 != 0 || hidden < 64) return fail(kUnsupported, "hidden=%d must be a multiple of 64", hidden);
  if (inter % 128 != 0 || inter < 128) return fail(kUnsupported, "intermediate=%d must be a multiple of 128", inter);
  if (tokens_local * world * top_k > (1ll << 30)) return fail(kUnsupported, "too many routed rows");
  return kOk;
}

int ep_peers(const void* const* peer_buffers, int world, PeerPtrs* out) {
  if (peer_buffers == nullptr) return fail(kInvalidArgument, "peer_buffers is null");
  for (int i = 0; i < kMaxPeers; ++i) out->p[i] = nullptr;
  for (int i = 0; i < world; ++i) {
    if (peer_buffers[i] == nullptr || (reinterpret_cast<uintptr_t>(peer_buffers[i]) & 255))
      return fail(kInvalidArgument, "peer buffer %d is null or not 256-byte aligned", i);
    out->p[i] = static_cast<uint8_t*>(const_cast<void*>(peer_buffers[i]));
  }
  return kOk;
}

}  // namespace

size_t moe_ep_buffer_bytes(int64_t tokens_local, int hidden, int inter, int experts_local, int top_k, int world) {
  return ep_layout(tokens_local, hidden, inter, experts_local, top_k, world).total;
}

int moe_ep_stage(const void* x, const int* ids, void* own_buffer, int64_t tokens_local, int hidden, int inter,
                 int experts_local, int top_k, int world, cudaStream_t stream) {
  int rc = ep_check(tokens_local, hidden, inter, experts_local, top_k, world, 0);
  if (rc) return rc;
  if (x == nullptr || ids == nullptr || own_buffer == nullptr) return fail(kInvalidArgument, "null pointer argument");
  if ((reinterpret_cast<uintptr_t>(x) & 31) || (reinterpret_cast<uintptr_t>(own_buffer) & 255))
    return fail(kInvalidArgument, "x must be 32-byte and the buffer 256-byte aligned");
  if (tokens_local == 0) return kOk;
  const EpLayout L = ep_layout(tokens_local, hidden, inter, experts_local, top_k, world);
  uint8_t* b = static_cast<uint8_t*>(own_buffer);
  ep_stage_kernel<128><<<static_cast<unsigned>(tokens_local), 128, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), ids, b + L.tok_codes, b + L.tok_sf, reinterpret_cast<int*>(b + L.tok_ids),
      hidden, top_k);
  return check_cuda(cudaGetLastError(), "ep_stage_kernel launch");
}

int moe_ep_compute(const void* const* peer_buffers, int rank, int world, const void* w1, const void* w1_sf,
                   const void* w2, const void* w2_sf, const float* w1_alpha, const float* w2_alpha,
                   const float* fc2_input_scale, int64_t tokens_local, int hidden, int inter, int experts_local,
                   int top_k, int* status, cudaStream_t stream) {
  int rc = ep_check(tokens_local, hidden, inter, experts_local, top_k, world, rank);
  if (rc) return rc;
  if (w1 == nullptr || w1_sf == nullptr || w2 == nullptr || w2_sf == nullptr || status == nullptr)
    return fail(kInvalidArgument, "null pointer argument");
  PeerPtrs peers;
  rc = ep_peers(peer_buffers, world, &peers);
  if (rc) return rc;
  if (tokens_local == 0) return kOk;
  const EpLayout L = ep_layout(tokens_local, hidden, inter, experts_local, top_k, world);
  uint8_t* b = peers.p[rank];
  MoeHeader h{};
  h.counts = reinterpret_cast<int*>(b + L.counts);
  h.cursor = reinterpret_cast<int*>(b + L.cursor);
  h.offsets = reinterpret_cast<int*>(b + L.offsets);
  h.num_m_blocks = reinterpret_cast<int*>(b + L.num_m_blocks);
  h.m_block_expert = reinterpret_cast<int*>(b + L.m_block_expert);
  h.m_block_rows = reinterpret_cast<int*>(b + L.m_block_rows);
  h.slot_row = nullptr;
  __nv_bfloat16** row_dst = reinterpret_cast<__nv_bfloat16**>(b + L.row_dst);
  const int expert_lo = rank * experts_local;
  const int slots_per_rank = static_cast<int>(tokens_local * top_k);
  const int total_slots = slots_per_rank * world;
  const int max_rows = L.max_m_blocks * 128;
  B200_CUDA(cudaMemsetAsync(h.counts, 0, sizeof(int) * experts_local, stream));
  B200_CUDA(cudaMemsetAsync(b + L.xq_sf, 0, L.xq_sf_bytes, stream));
  ep_count_kernel<<<(total_slots + kCountSlotsPerCta - 1) / kCountSlotsPerCta, 256, 0, stream>>>(
      peers, L.tok_ids, slots_per_rank, world, expert_lo, experts_local, h.counts);
  moe_scan_kernel<<<1, 1024, 0, stream>>>(h, experts_local, L.max_m_blocks);
  ep_gather_kernel<128><<<static_cast<unsigned>(tokens_local * world), 128, 0, stream>>>(
      peers, L, h, row_dst, b + L.xq, b + L.xq_sf, static_cast<int>(tokens_local), hidden, top_k, expert_lo,
      experts_local, max_rows);
  B200_CUDA(cudaGetLastError());
  const int few_rows = tokens_local * world <= 32;
  rc = gemm_moe_fc1(b + L.xq, b + L.xq_sf, w1, w1_sf, b + L.act, b + L.act_sf, w1_alpha, fc2_input_scale,
                    h.num_m_blocks, h.m_block_expert, h.m_block_rows, L.max_m_blocks, hidden, inter, experts_local,
                    few_rows, status, stream);
  if (rc) return rc;
  rc = gemm_moe_fc2(b + L.act, b + L.act_sf, w2, w2_sf, b + L.partial, /*rows_bf16=*/1, w2_alpha,
                    h.num_m_blocks, h.m_block_expert, h.m_block_rows, L.max_m_blocks, hidden, inter, experts_local,
                    few_rows, status, stream);
  if (rc) return rc;
  ep_return_rows_kernel<<<static_cast<unsigned>(max_rows), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(b + L.partial), row_dst, h.num_m_blocks, h.m_block_rows, hidden);
  return check_cuda(cudaGetLastError(), "ep_return_rows_kernel launch");
}

int moe_ep_combine(const void* const* peer_buffers, int rank, int world, const int* ids, const float* weights,
                   void* out, int64_t tokens_local, int hidden, int inter, int experts_local, int top_k,
                   cudaStream_t stream) {
  int rc = ep_check(tokens_local, hidden, inter, experts_local, top_k, world, rank);
  if (rc) return rc;
  if (ids == nullptr || weights == nullptr || out == nullptr) return fail(kInvalidArgument, "null pointer argument");
  PeerPtrs peers;
  rc = ep_peers(peer_buffers, world, &peers);
  if (rc) return rc;
  if (tokens_local == 0) return kOk;
  const EpLayout L = ep_layout(tokens_local, hidden, inter, experts_local, top_k, world);
  const int threads = hidden / 4 >= 256 ? 256 : 128;
  (void)ids;
  if (tokens_local <= 256) {
    ep_combine_few_kernel<<<dim3(static_cast<unsigned>(tokens_local), (hidden / 4 + threads - 1) / threads), threads, 0,
                            stream>>>(reinterpret_cast<const __nv_bfloat16*>(peers.p[rank] + L.recv), weights,
                                      static_cast<__nv_bfloat16*>(out), hidden, top_k);
  } else {
    ep_combine_kernel<<<static_cast<unsigned>(tokens_local), threads, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(peers.p[rank] + L.recv), weights, static_cast<__nv_bfloat16*>(out),
        hidden, top_k);
  }
  return check_cuda(cudaGetLastError(), "ep_combine_kernel launch");
}

}  // namespace b200fp4
