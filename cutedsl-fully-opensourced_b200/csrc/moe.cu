// Fused NVFP4 MoE for sm_100a: the stages around the two grouped GEMMs.
//
// Stands in for flashinfer's b12x_fused_moe as the reference calls it
// (tests/python/test_flashinfer_b12x_verbatim.py:99-116); arithmetic contract is
// the reference's routed golden (same file, lines 28-65 and 209-219):
//
//   route (optional)   softmax over expert logits -> top-k -> renormalise
//   count              (fused with the router when logits are given) rows per expert, and the position of
//                      every (token, slot) pair among the rows of its expert
//   quantise + place   every CTA rebuilds the padded row offsets from the counts (every expert's segment is
//                      padded to whole 128-row blocks so that a GEMM tile never straddles two experts);
//                      each token is quantised ONCE to NVFP4 with the activation packer and its codes /
//                      scale bytes are written to the row of every (token, slot) pair
//   FC1 grouped GEMM   [up | gate] = Xq . W1[e]^T, epilogue silu(gate)*up -> bf16 -> NVFP4   (gemm.cu)
//   FC2 grouped GEMM   partial = Actq . W2[e]^T * w2_alpha[e]                               (gemm.cu)
//   combine            out[t] = bf16( sum_j weight[t,j] * partial[row(t,j)] ), f32, slot order
//
// All intermediate buffers live in a caller-provided workspace.
#include <algorithm>

#include "gemm_kernel.cuh"

namespace b200fp4 {

int gemm_moe_fc1(const void* xq, const void* xq_sf, const void* w1, const void* w1_sf, void* act_codes, void* act_sf,
                 const float* w1_alpha, const float* fc2_input_scale, const int* num_m_blocks_dev,
                 const int* m_block_expert, const int* m_block_rows, int max_m_blocks, int hidden, int inter,
                 int experts, int few_rows, int* status, cudaStream_t stream, const PeerSync* peer = nullptr,
                 int sfa_row_pitch = 0);
int gemm_moe_fc2(const void* act_codes, const void* act_sf, const void* w2, const void* w2_sf, void* partial,
                 int rows_bf16, const float* w2_alpha, const int* num_m_blocks_dev, const int* m_block_expert,
                 const int* m_block_rows, int max_m_blocks, int hidden, int inter, int experts, int few_rows,
                 int* status, cudaStream_t stream);

int sm_count_of_current_device();

namespace {

constexpr int kRouteMaxPerLane = 32;       // experts <= 1024

// ---------------------------------------------------------------------------
// route: one warp per token; kPerLane = experts a lane holds (experts <= 32 * kPerLane)
// ---------------------------------------------------------------------------
// Lane j (< top_k) of the warp returns the j-th choice of the token whose logits start at `row`.
template <int kPerLane>
__device__ __forceinline__ void route_one_token(const float* __restrict__ row, int lane, int experts, int top_k,
                                                int renormalize, int& my_id, float& my_w) {
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
  my_w = 0.0f;
  my_id = 0;
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
  if (renormalize) my_w = my_w / picked;
}

template <int kPerLane>
__global__ void route_topk_kernel(const float* __restrict__ logits, int* __restrict__ ids, float* __restrict__ weights,
                                  int tokens, int experts, int top_k, int renormalize) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= tokens) return;
  int my_id;
  float my_w;
  route_one_token<kPerLane>(logits + static_cast<int64_t>(warp) * experts, lane, experts, top_k, renormalize, my_id, my_w);
  if (lane < top_k) {
    ids[static_cast<int64_t>(warp) * top_k + lane] = my_id;
    weights[static_cast<int64_t>(warp) * top_k + lane] = my_w;
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

// ---------------------------------------------------------------------------
// Front end shared by the single-GPU operator and the expert-parallel one.
//
// Experts are numbered 0 .. experts_total-1 and expert e lives on rank e / experts_local (single GPU: one
// rank).  Every rank owns a buffer of identical layout; peers.p[d] is rank d's buffer as mapped into this
// process (single GPU: the workspace).  Two kernels:
//
//   count   one warp per token: (route from logits, or take the given ids) and claim, per (token, slot), a
//           position among THIS rank's slots of the same expert; the last CTA publishes the rank's counts
//           to every rank and raises signal 0
//   place   wait for signal 0 of every rank; every CTA derives from the counts of all ranks where each
//           expert's rows start at its owner (segments padded to 128-row blocks) and where this rank's rows
//           start inside the segment; then quantises its tokens once and writes codes + scale bytes into the
//           row of every slot AT THE OWNER OF THE SLOT'S EXPERT (plain stores; over NVLink when the owner is
//           a peer: 4.5 bits per element cross the wire), plus the row's return address; the last CTA raises
//           signal 1.  CTA 0 also writes this rank's block tables for the grouped GEMMs.
//
// Signals are per (phase, source rank) words in the destination's buffer carrying a step counter; waits on
// them are bounded in time: on expiry the kernel sets kStatusPeerWaitExpired in the device status word and the
// abort word of the buffer, after which no kernel touches peer memory until the host resets the exchange.
// ---------------------------------------------------------------------------
struct Exchange {
  PeerPtrs peers;
  size_t flags, counts_all, xq, xq_sf, row_tag;      // offsets inside a rank's buffer (written by peers)
  // per-rank return (see the expert-parallel section): [source rank][slot] row at this rank (-1: not served
  // here) and routing weight of every (token, slot) of every rank; 0 = per-slot return, nothing is written
  size_t inv_row, inv_w;
  int rank, world, experts_local;
  int xq_sf_pitch;            // bytes between the rows of scale bytes of the FC1 operand (plain rows, see place)
  unsigned long long wait_ns;
};

// Threads 0..world-1 of the CTA wait for `phase` of their rank; returns false (to all threads) when a wait
// expired now or earlier in the step.  The first failure is recorded in the status word.
__device__ __forceinline__ bool wait_all_ranks(const Exchange& ex, int phase, int* ctrl, int* status, int* s_ok) {
  if (ex.world <= 1) return true;
  if (threadIdx.x == 0) *s_ok = 1;
  __syncthreads();
  if (threadIdx.x < ex.world && threadIdx.x != ex.rank) {
    const int epoch = *reinterpret_cast<volatile int*>(ctrl + kCtrlEpoch) + 1;
    const int* flags = reinterpret_cast<const int*>(ex.peers.p[ex.rank] + ex.flags) + phase * kMaxPeers;
    if (*reinterpret_cast<volatile int*>(ctrl + kCtrlAbort) != 0) {
      *s_ok = 0;
    } else if (!wait_flag(flags + threadIdx.x, epoch, ex.wait_ns)) {
      *s_ok = 0;
      atomicOr(status, kStatusPeerWaitExpired);
      atomicExch(ctrl + kCtrlAbort, 1);
    }
  }
  __syncthreads();
  return *s_ok != 0;
}
// Called by all threads at the end of a kernel whose CTAs wrote to peer memory: the last CTA to arrive raises
// `phase` at every peer.  `ticket` counts finished CTAs and is left at zero.
__device__ __forceinline__ void signal_when_all_ctas_done(const Exchange& ex, int phase, int* ctrl, int ticket, int* s_last) {
  if (ex.world <= 1) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    *s_last = atomicAdd(ctrl + ticket, 1) == static_cast<int>(gridDim.x * gridDim.y) - 1;
  }
  __syncthreads();
  if (!*s_last) return;
  if (threadIdx.x < ex.world && threadIdx.x != ex.rank &&
      *reinterpret_cast<volatile int*>(ctrl + kCtrlAbort) == 0) {
    __threadfence_system();
    const int epoch = *reinterpret_cast<volatile int*>(ctrl + kCtrlEpoch) + 1;
    st_release_sys(reinterpret_cast<int*>(ex.peers.p[threadIdx.x] + ex.flags) + phase * kMaxPeers + ex.rank, epoch);
  }
  if (threadIdx.x == 0) ctrl[ticket] = 0;
}

// count: one warp per token, up to 32 tokens per CTA (fewer when there are few tokens, so that the routing of a
// small batch still spreads over many SMs).  kPerLane > 0: route from logits (experts <= 32 * kPerLane)
// and write ids / weights; kPerLane == 0: ids are given.  Positions are claimed in two levels: a histogram of the
// CTA's slots in shared memory (position inside the CTA's share), then ONE global add per (CTA, expert) that the
// CTA saw -- thousands of same-address global atomics with a returned value are what made a flat version slow.
// Dynamic shared memory: 2 * experts_total ints.
constexpr int kCountTokensPerCta = 32;
// one warp per token where the router's registers allow 1024 threads (routing four tokens one after the other in
// a warp was measured at 19 us for 4096 tokens, twice the time of the routing itself)
__host__ __device__ constexpr int count_threads(int per_lane) { return per_lane <= 8 ? 1024 : 256; }
template <int kPerLane>
__global__ void __launch_bounds__(count_threads(kPerLane))
moe_count_kernel(const float* __restrict__ logits, int route_experts, int renormalize, const int* __restrict__ ids_in,
                 int* __restrict__ ids_out, float* __restrict__ weights_out, int tokens, int top_k, int expert_lo,
                 int experts_total, int* my_counts, int* __restrict__ slot_pos, int* ctrl, Exchange ex,
                 int tokens_per_cta) {
  const int kCountThreads = blockDim.x;
  extern __shared__ int s_dyn[];
  int* s_hist = s_dyn;
  int* s_base = s_dyn + experts_total;
  __shared__ int s_e[kCountTokensPerCta * 64];       // expert of every slot of the CTA (-1: not served here)
  __shared__ int s_p[kCountTokensPerCta * 64];       // its position among the CTA's slots of that expert
  __shared__ int s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int token0 = blockIdx.x * tokens_per_cta;
  const int n_tokens = min(tokens_per_cta, tokens - token0);
  for (int e = threadIdx.x; e < experts_total; e += kCountThreads) s_hist[e] = 0;
  __syncthreads();
  for (int lt = warp; lt < n_tokens; lt += kCountThreads >> 5) {
    const int token = token0 + lt;
    if constexpr (kPerLane > 0) {
      int my_id;
      float my_w;
      route_one_token<kPerLane>(logits + static_cast<int64_t>(token) * route_experts, lane, route_experts, top_k,
                                renormalize, my_id, my_w);
      if (lane < top_k) {
        const int64_t slot = static_cast<int64_t>(token) * top_k + lane;
        ids_out[slot] = my_id;
        weights_out[slot] = my_w;
        const int e = my_id - expert_lo;
        const bool ok = e >= 0 && e < experts_total;
        s_e[lt * top_k + lane] = ok ? e : -1;
        s_p[lt * top_k + lane] = ok ? atomicAdd(s_hist + e, 1) : 0;
      }
    } else {
      for (int j = lane; j < top_k; j += 32) {
        const int e = ids_in[static_cast<int64_t>(token) * top_k + j] - expert_lo;
        const bool ok = e >= 0 && e < experts_total;
        s_e[lt * top_k + j] = ok ? e : -1;
        s_p[lt * top_k + j] = ok ? atomicAdd(s_hist + e, 1) : 0;
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts_total; e += kCountThreads) {
    const int c = s_hist[e];
    s_base[e] = c != 0 ? atomicAdd(my_counts + e, c) : 0;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_tokens * top_k; i += kCountThreads) {
    const int e = s_e[i];
    slot_pos[static_cast<int64_t>(token0) * top_k + i] = e >= 0 ? s_base[e] + s_p[i] : -1;
  }
  // the last CTA hands the counts to every rank (and clears them for the next step)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = atomicAdd(ctrl + kCtrlTicketCount, 1) == static_cast<int>(gridDim.x) - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const bool live = *reinterpret_cast<volatile int*>(ctrl + kCtrlAbort) == 0;
  for (int e = threadIdx.x; e < experts_total; e += blockDim.x) {
    const int c = atomicExch(my_counts + e, 0);
    for (int d = 0; d < ex.world; ++d)
      if (d == ex.rank || live)
        reinterpret_cast<int*>(ex.peers.p[d] + ex.counts_all)[ex.rank * experts_total + e] = c;
  }
  __syncthreads();
  if (threadIdx.x < ex.world && threadIdx.x != ex.rank && live) {
    __threadfence_system();
    const int epoch = *reinterpret_cast<volatile int*>(ctrl + kCtrlEpoch) + 1;
    st_release_sys(reinterpret_cast<int*>(ex.peers.p[threadIdx.x] + ex.flags) + 0 * kMaxPeers + ex.rank, epoch);
  }
  if (threadIdx.x == 0) ctrl[kCtrlTicketCount] = 0;
}

// place: see the section comment.  rows_per_block: valid rows that a 128-row block may hold (128, or 32 for the
// few-row GEMM variants).  One warp per token at a time; a lane quantises groups of four adjacent 16-element
// blocks (128 bytes of the token in flight per lane) and writes, per slot, their 32 bytes of codes and their four
// scale bytes (adjacent in the 128x4 tiles) with one store each.  Dynamic shared memory: 3 * experts_total ints.
template <int kThreads>
__global__ void __launch_bounds__(kThreads)
moe_quant_place_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids,
                       const int* __restrict__ slot_pos, Exchange ex, int tokens, int hidden, int top_k,
                       int expert_lo, int experts_total, int max_m_blocks, int rows_per_block, int* slot_row,
                       int* num_m_blocks, int* m_block_expert, int* m_block_rows, int* ctrl, int* status,
                       const float* __restrict__ weights) {
  extern __shared__ int s_dyn[];
  int* s_base = s_dyn;                       // blocks before expert e (over all experts, in expert order)
  int* s_myoff = s_dyn + experts_total;      // rows of lower ranks inside expert e's segment
  int* s_tot = s_dyn + 2 * experts_total;    // rows of expert e over all ranks
  constexpr int kWarps = kThreads / 32;
  __shared__ int s_warp[kWarps];
  __shared__ int s_flag;
  __shared__ int s_rows[kWarps][64];
  __shared__ int s_dst[kWarps][64];
  if (!wait_all_ranks(ex, 0, ctrl, status, &s_flag)) return;

  const int rpb = rows_per_block;
  const int el = ex.experts_local;
  const int* counts = reinterpret_cast<const int*>(ex.peers.p[ex.rank] + ex.counts_all);
  const int per_thread = (experts_total + kThreads - 1) / kThreads;
  const int e0 = threadIdx.x * per_thread;
  int my_blocks = 0;
  for (int i = 0; i < per_thread; ++i) {
    const int e = e0 + i;
    if (e < experts_total) {
      int tot = 0, off = 0;
      for (int r = 0; r < ex.world; ++r) {
        const int c = __ldcg(counts + r * experts_total + e);
        if (r < ex.rank) off += c;
        tot += c;
      }
      s_tot[e] = tot;
      s_myoff[e] = off;
      my_blocks += (tot + rpb - 1) / rpb;
    }
  }
  // exclusive scan of my_blocks over the CTA's threads
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = my_blocks;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  int before = 0;
  for (int w = 0; w < warp; ++w) before += s_warp[w];
  int run = before + incl - my_blocks;
  for (int i = 0; i < per_thread; ++i) {
    const int e = e0 + i;
    if (e < experts_total) {
      s_base[e] = run;
      run += (s_tot[e] + rpb - 1) / rpb;
    }
  }
  __syncthreads();

  if (blockIdx.x == 0) {               // block tables of this rank's experts for the grouped GEMMs
    const int first = ex.rank * el;
    const int seg0 = s_base[first];
    for (int le = threadIdx.x; le < el; le += kThreads) {
      const int tot = s_tot[first + le];
      const int nb = (tot + rpb - 1) / rpb;
      const int b0 = s_base[first + le] - seg0;
      for (int b = 0; b < nb; ++b) {
        if (b0 + b < max_m_blocks) {
          m_block_expert[b0 + b] = le;
          m_block_rows[b0 + b] = min(rpb, tot - rpb * b);
        }
      }
    }
    if (threadIdx.x == 0) {
      const int last = first + el - 1;
      *num_m_blocks = min(s_base[last] - seg0 + (s_tot[last] + rpb - 1) / rpb, max_m_blocks);
    }
  }

  const int groups = hidden >> 6;            // groups of four 16-element blocks
  for (int token = blockIdx.x * kWarps + warp; token < tokens; token += gridDim.x * kWarps) {
    __syncwarp();
    for (int j = lane; j < top_k; j += 32) {
      const int64_t slot = static_cast<int64_t>(token) * top_k + j;
      const int e = ids[slot] - expert_lo;
      const int pos = slot_pos[slot];
      int row = -1, d = 0;
      if (e >= 0 && e < experts_total && pos >= 0) {
        d = e / el;
        const int r = s_myoff[e] + pos;
        row = (s_base[e] - s_base[d * el] + r / rpb) * 128 + r % rpb;
        if (row >= max_m_blocks * 128) row = -1;
        else reinterpret_cast<int*>(ex.peers.p[d] + ex.row_tag)[row] = (ex.rank << 24) | static_cast<int>(slot);
      }
      s_rows[warp][j] = row;
      s_dst[warp][j] = d;
      if (slot_row != nullptr) slot_row[slot] = row;
      if (ex.inv_row != 0) {
        // per-rank return: every rank learns which of its rows (if any) holds this slot, the owner also its weight
        const int64_t idx = static_cast<int64_t>(ex.rank) * tokens * top_k + slot;
        for (int q = 0; q < ex.world; ++q)
          reinterpret_cast<int*>(ex.peers.p[q] + ex.inv_row)[idx] = (q == d && row >= 0) ? row : -1;
        if (row >= 0) reinterpret_cast<float*>(ex.peers.p[d] + ex.inv_w)[idx] = weights[slot];
      }
    }
    __syncwarp();
    const __nv_bfloat16* xrow = x + static_cast<int64_t>(token) * hidden;
    for (int g = lane; g < groups; g += 32) {
      U32x8 raw[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) raw[c] = ld_stream_32B(xrow + g * 64 + c * 16);
      U32x8 codes;
      uint32_t quad = 0;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint64_t v2[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v2[i] = pair16_to_f32x2<__nv_bfloat16>(raw[c].v[i]);
        uint32_t sfb;
        quantize_block16<true>(v2, 1.0f, codes.v[2 * c], codes.v[2 * c + 1], sfb);
        quad |= (sfb & 0xffu) << (8 * c);
      }
      for (int j = 0; j < top_k; ++j) {
        const int row = s_rows[warp][j];
        if (row < 0) continue;
        uint8_t* base = ex.peers.p[s_dst[warp][j]];
        st_32B(base + ex.xq + static_cast<int64_t>(row) * (hidden >> 1) + g * 32, codes);
        // scale bytes as plain rows: a warp's 32 groups are 128 contiguous bytes (one write instead of 32 pieces
        // 512 bytes apart, which is what the 128x4 tiles would ask for; FC1 fetches these rows as they are)
        *reinterpret_cast<uint32_t*>(base + ex.xq_sf + static_cast<int64_t>(row) * ex.xq_sf_pitch + 4 * g) = quad;
      }
    }
  }
  signal_when_all_ctas_done(ex, 1, ctrl, kCtrlTicketPlace, &s_flag);
}

// Few slots (<= 1024): count, scan and row assignment in one CTA -- one launch instead of a memset and three
// kernels, which is most of a decode step's bookkeeping time.  Rows of an expert go to its slots in slot order.
// rows_per_block: valid rows that a 128-row block may hold.  128 normally; 32 for the few-row GEMM variants, which
// load only the first 32 rows of every block (an expert with more rows than that simply gets more blocks).
// kRoutePerLane > 0: the router runs here first (one warp per token, the CTA's 32 warps take the tokens in turn;
// experts per lane as in route_one_token) and writes its choice to ids / weights -- one launch fewer in a decode
// step.  0: the ids are inputs.
template <int kRoutePerLane>
__global__ void __launch_bounds__(1024)
moe_prepare_small_kernel(const float* __restrict__ logits, int route_experts, int renormalize, int top_k, int* ids,
                         float* weights, int n_slots, int expert_lo, MoeHeader h, int experts, int max_m_blocks,
                         int max_rows, int rows_per_block) {
  __shared__ int s_count[1024];
  __shared__ int s_blocks[1024];
  __shared__ int s_offset[1024];
  __shared__ int s_expert[1024];
  const int t = threadIdx.x;
  s_count[t] = 0;
  if constexpr (kRoutePerLane > 0) {
    const int lane = t & 31;
    for (int token = t >> 5; token * top_k < n_slots; token += 32) {
      int my_id;
      float my_w;
      route_one_token<kRoutePerLane>(logits + static_cast<int64_t>(token) * route_experts, lane, route_experts, top_k,
                                     renormalize, my_id, my_w);
      if (lane < top_k) {
        ids[token * top_k + lane] = my_id;
        weights[token * top_k + lane] = my_w;
        s_blocks[token * top_k + lane] = my_id;          // handed to the slot's thread below
      }
    }
    __syncthreads();
  }
  int e = -1, rank_in_expert = 0;
  if (t < n_slots) {
    e = (kRoutePerLane > 0 ? s_blocks[t] : ids[t]) - expert_lo;
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
  const int blocks = (count + rows_per_block - 1) / rows_per_block;
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
        h.m_block_rows[excl + b] = min(rows_per_block, count - rows_per_block * b);
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
      row = s_offset[e] + (rank_in_expert / rows_per_block) * 128 + rank_in_expert % rows_per_block;
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

// The same sum for bf16 rows and a bf16 output with 16-byte accesses: one CTA per token, a thread owns 8 columns and
// keeps the loads of four rows in flight.  Same arithmetic as moe_combine_kernel (f32, slot order, one product and
// one sum per slot, one rounding).
__global__ void moe_combine_bf16x8_kernel(const __nv_bfloat16* __restrict__ partial, const int* __restrict__ slot_row,
                                          const float* __restrict__ weights, __nv_bfloat16* __restrict__ out,
                                          int hidden, int top_k, int accumulate) {
  __shared__ int s_rows[64];
  __shared__ float s_w[64];
  const int token = blockIdx.x;
  if (threadIdx.x < top_k) {
    s_rows[threadIdx.x] = slot_row[static_cast<int64_t>(token) * top_k + threadIdx.x];
    s_w[threadIdx.x] = weights[static_cast<int64_t>(token) * top_k + threadIdx.x];
  }
  __syncthreads();
  for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j0 = 0; j0 < top_k; j0 += 4) {
      uint4 u[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int row = j0 + k < top_k ? s_rows[j0 + k] : -1;
        u[k] = row >= 0 ? *reinterpret_cast<const uint4*>(partial + static_cast<int64_t>(row) * hidden + c)
                        : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (j0 + k < top_k && s_rows[j0 + k] >= 0) {
          const float w = s_w[j0 + k];
          const uint32_t words[4] = {u[k].x, u[k].y, u[k].z, u[k].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            acc[2 * i] = __fadd_rn(acc[2 * i], __fmul_rn(w, Pair16<__nv_bfloat16>::lo(words[i])));
            acc[2 * i + 1] = __fadd_rn(acc[2 * i + 1], __fmul_rn(w, Pair16<__nv_bfloat16>::hi(words[i])));
          }
        }
      }
    }
    __nv_bfloat16* o = out + static_cast<int64_t>(token) * hidden + c;
    if (accumulate) {
      const uint4 prev = *reinterpret_cast<const uint4*>(o);
      const uint32_t words[4] = {prev.x, prev.y, prev.z, prev.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] += Pair16<__nv_bfloat16>::lo(words[i]);
        acc[2 * i + 1] += Pair16<__nv_bfloat16>::hi(words[i]);
      }
    }
    uint4 v;
    v.x = Pair16<__nv_bfloat16>::pack(acc[0], acc[1]);
    v.y = Pair16<__nv_bfloat16>::pack(acc[2], acc[3]);
    v.z = Pair16<__nv_bfloat16>::pack(acc[4], acc[5]);
    v.w = Pair16<__nv_bfloat16>::pack(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(o) = v;
  }
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// With at most 32 tokens (and few enough slots for the single-CTA bookkeeping kernel) the wide GEMM variants keep
// only 32 rows of A per stage, which buys another stage of weights in flight.  The bookkeeping then fills every
// 128-row block with at most 32 rows, so an expert that is named more than 32 times (ids may repeat inside a
// token: the reference's own bench draws them with replacement, tools/perf/bench_flashinfer_b12x.py:70-71)
// gets several blocks instead of wrong results.
inline bool moe_few_rows(int64_t tokens, int top_k) { return tokens <= 32 && tokens * top_k <= 1024; }

// Scale bytes of the FC1 operand.  The general front end writes them as plain rows, sf_row_pitch(hidden) bytes
// apart (a multiple of 16, as the tensor map wants); the few-slot front end writes 128x4 tiles.  The buffer fits
// either.  Rows that only pad a 128-row block are never written and never cleared: a row of the accumulator
// depends on its own row of A and of its scale bytes only, and rows without data are never read back.
inline int sf_row_pitch(int hidden) { return ((hidden / 16) + 15) / 16 * 16; }
inline size_t xq_sf_buffer_bytes(int64_t blocks, int hidden) {
  const size_t tiled = static_cast<size_t>(blocks) * ((hidden + 63) / 64) * 512;
  const size_t rows = static_cast<size_t>(blocks) * 128 * sf_row_pitch(hidden);
  return std::max(tiled, rows);
}

struct MoeWorkspace {
  MoeHeader h;
  int* ctrl;               // [kCtrlWords] + my_counts [experts] right behind it: cleared together at every call
  int* my_counts;
  int* counts_all;         // [experts]
  int* slot_pos;           // [slots]
  int* row_tag;            // [rows]
  uint8_t* xq;
  uint8_t* xq_sf;
  uint8_t* act;
  uint8_t* act_sf;
  float* partial;
  size_t clear_bytes;      // ctrl + my_counts
  size_t xq_sf_bytes;
  size_t total;
  int max_m_blocks;
};

MoeWorkspace carve(void* base, int64_t tokens, int hidden, int inter, int experts, int top_k) {
  MoeWorkspace w{};
  const int64_t slots = tokens * top_k;
  // few-row launches (see moe_fused) fill a block with at most 32 rows
  const int64_t blocks = std::min<int64_t>(experts, slots) + slots / (moe_few_rows(tokens, top_k) ? 32 : 128);
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
  w.ctrl = reinterpret_cast<int*>(take(sizeof(int) * (kCtrlWords + experts)));
  w.my_counts = w.ctrl == nullptr ? nullptr : w.ctrl + kCtrlWords;
  w.clear_bytes = sizeof(int) * (kCtrlWords + experts);
  w.counts_all = reinterpret_cast<int*>(take(sizeof(int) * experts));
  w.slot_pos = reinterpret_cast<int*>(take(sizeof(int) * slots));
  w.row_tag = reinterpret_cast<int*>(take(sizeof(int) * rows));
  w.xq_sf_bytes = xq_sf_buffer_bytes(blocks, hidden);
  w.xq_sf = take(w.xq_sf_bytes);
  w.xq = take(static_cast<size_t>(rows) * (hidden / 2));
  w.act_sf = take(static_cast<size_t>(blocks) * ((inter + 63) / 64) * 512);
  w.act = take(static_cast<size_t>(rows) * (inter / 2));
  w.partial = reinterpret_cast<float*>(take(static_cast<size_t>(rows) * hidden * sizeof(float)));
  w.total = off;
  return w;
}

// launch of the count kernel: routing from logits when `logits` is given (ids_out / weights_out receive the
// result), else the caller's ids
int launch_count(const float* logits, int route_experts, int renormalize, const int* ids_in, int* ids_out,
                 float* weights_out, int tokens, int top_k, int expert_lo, int experts_total, int* my_counts,
                 int* slot_pos, int* ctrl, const Exchange& ex, cudaStream_t stream) {
  const int tpc = tokens >= 4096 ? kCountTokensPerCta : (tokens >= 1024 ? 16 : 8);
  const dim3 grid((tokens + tpc - 1) / tpc);
  const size_t smem = sizeof(int) * 2 * experts_total;
#define B200_COUNT(PL)                                                                                             \
  moe_count_kernel<PL><<<grid, std::min(count_threads(PL), 32 * tpc), smem, stream>>>(                             \
      logits, route_experts, renormalize, ids_in, ids_out, weights_out, tokens, top_k, expert_lo, experts_total,    \
      my_counts, slot_pos, ctrl, ex, tpc)
  if (logits == nullptr) B200_COUNT(0);
  else if (route_experts <= 64) B200_COUNT(2);
  else if (route_experts <= 128) B200_COUNT(4);
  else if (route_experts <= 256) B200_COUNT(8);
  else B200_COUNT(kRouteMaxPerLane);
#undef B200_COUNT
  return check_cuda(cudaGetLastError(), "moe_count_kernel launch");
}

int launch_place(const void* x, const int* ids, const int* slot_pos, const Exchange& ex, int tokens, int hidden,
                 int top_k, int expert_lo, int experts_total, int max_m_blocks, int rows_per_block, int* slot_row,
                 int* num_m_blocks, int* m_block_expert, int* m_block_rows, int* ctrl, int* status,
                 cudaStream_t stream, const float* weights = nullptr) {
  // eight warps per CTA, one token per warp at a time; enough CTAs that every SM holds several
  const int grid = std::max(1, std::min((tokens + 7) / 8, 6 * sm_count_of_current_device()));
  const size_t smem = sizeof(int) * 3 * experts_total;
  moe_quant_place_kernel<256><<<grid, 256, smem, stream>>>(
      static_cast<const __nv_bfloat16*>(x), ids, slot_pos, ex, tokens, hidden, top_k, expert_lo, experts_total,
      max_m_blocks, rows_per_block, slot_row, num_m_blocks, m_block_expert, m_block_rows, ctrl, status, weights);
  return check_cuda(cudaGetLastError(), "moe_quant_place_kernel launch");
}

int route_check(int tokens, int experts, int top_k) {
  if (tokens < 0 || experts < 1 || top_k < 1 || top_k > 32 || top_k > experts)
    return fail(kInvalidArgument, "tokens=%d experts=%d top_k=%d", tokens, experts, top_k);
  if (experts > 32 * kRouteMaxPerLane) return fail(kUnsupported, "experts=%d exceeds %d", experts, 32 * kRouteMaxPerLane);
  return kOk;
}

}  // namespace

int route_topk(const float* logits, int* ids, float* weights, int tokens, int experts, int top_k, int renormalize,
               cudaStream_t stream) {
  if (logits == nullptr || ids == nullptr || weights == nullptr) return fail(kInvalidArgument, "null pointer argument");
  int rc = route_check(tokens, experts, top_k);
  if (rc) return rc;
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
// experts = number of LOCAL experts (w1/w2/alphas hold exactly those); the expert ids are global, of which
// [expert_lo, expert_lo + experts) are served here.  accumulate != 0 adds into `out`.
// Routing: either `ids` and `route_w` are inputs (logits == nullptr), or `logits` f32 [tokens, route_experts] is
// given and the router runs inside the front end, writing its choice to `ids` / `route_w` (then outputs).
int moe_fused(const void* x, const void* w1, const void* w1_sf, const void* w2, const void* w2_sf, int* ids,
              float* route_w, const float* logits, int route_experts, int renormalize, const float* w1_alpha,
              const float* w2_alpha, const float* fc2_input_scale, void* out, int64_t tokens, int hidden, int inter,
              int experts, int top_k, int expert_lo, int accumulate, int out_dtype, void* workspace,
              size_t workspace_bytes, int* status, cudaStream_t stream) {
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
  if (tokens * top_k > (1ll << 24)) return fail(kUnsupported, "too many routed rows (at most 2^24 slots)");
  if (logits != nullptr) {
    int rc = route_check(static_cast<int>(tokens), route_experts, top_k);
    if (rc) return rc;
  }
  if (tokens == 0) return kOk;
  MoeWorkspace ws = carve(workspace, tokens, hidden, inter, experts, top_k);
  if (workspace_bytes < ws.total)
    return fail(kInvalidArgument, "workspace holds %zu bytes, %zu needed", workspace_bytes, ws.total);
  const int slots = static_cast<int>(tokens * top_k);
  const int max_rows = ws.max_m_blocks * 128;
  const int few_rows = moe_few_rows(tokens, top_k);

  if (slots <= 1024) {
    B200_CUDA(cudaMemsetAsync(ws.xq_sf, 0, ws.xq_sf_bytes, stream));    // rows that only pad a block read as zero
    // few slots: one CTA counts, scans and assigns rows in slot order; quantisation splits a token's columns
    // over several CTAs (a decode step is mostly the latency of these small kernels)
#define B200_PREPARE(PL)                                                                                          \
  moe_prepare_small_kernel<PL><<<1, 1024, 0, stream>>>(logits, route_experts, renormalize, top_k, ids, route_w, slots, \
                                                       expert_lo, ws.h, experts, ws.max_m_blocks, max_rows,          \
                                                       few_rows ? 32 : 128)
    if (logits == nullptr) {
      B200_PREPARE(0);
    } else if (route_experts <= 64) {
      B200_PREPARE(2);
    } else if (route_experts <= 128) {
      B200_PREPARE(4);
    } else if (route_experts <= 256) {
      B200_PREPARE(8);
    } else {
      // more experts per lane than the 64 registers of a 1024-thread CTA hold: the router keeps its own launch
      int rc = route_topk(logits, ids, route_w, static_cast<int>(tokens), route_experts, top_k, renormalize, stream);
      if (rc) return rc;
      B200_PREPARE(0);
    }
#undef B200_PREPARE
    const int parts = std::max(1, std::min(8, (hidden / 16) / 128));
    moe_scatter_quant_rows_kernel<128><<<dim3(static_cast<unsigned>(tokens), parts), 128, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), ws.h.slot_row, ws.xq, ws.xq_sf, hidden, top_k);
  } else {
    // two launches for any number of tokens: (route +) count, then scan + quantise + place
    B200_CUDA(cudaMemsetAsync(ws.ctrl, 0, ws.clear_bytes, stream));
    Exchange ex{};
    uint8_t* base = static_cast<uint8_t*>(workspace);
    ex.peers.p[0] = base;
    ex.counts_all = reinterpret_cast<uint8_t*>(ws.counts_all) - base;
    ex.xq = ws.xq - base;
    ex.xq_sf = ws.xq_sf - base;
    ex.xq_sf_pitch = sf_row_pitch(hidden);
    ex.row_tag = reinterpret_cast<uint8_t*>(ws.row_tag) - base;
    ex.rank = 0;
    ex.world = 1;
    ex.experts_local = experts;
    int rc = launch_count(logits, route_experts, renormalize, ids, ids, route_w, static_cast<int>(tokens), top_k,
                          expert_lo, experts, ws.my_counts, ws.slot_pos, ws.ctrl, ex, stream);
    if (rc) return rc;
    rc = launch_place(x, ids, ws.slot_pos, ex, static_cast<int>(tokens), hidden, top_k, expert_lo, experts,
                      ws.max_m_blocks, 128, ws.h.slot_row, ws.h.num_m_blocks, ws.h.m_block_expert, ws.h.m_block_rows,
                      ws.ctrl, status, stream);
    if (rc) return rc;
  }
  B200_CUDA(cudaGetLastError());
  int rc = gemm_moe_fc1(ws.xq, ws.xq_sf, w1, w1_sf, ws.act, ws.act_sf, w1_alpha, fc2_input_scale, ws.h.num_m_blocks,
                        ws.h.m_block_expert, ws.h.m_block_rows, ws.max_m_blocks, hidden, inter, experts, few_rows,
                        status, stream, nullptr, slots <= 1024 ? 0 : sf_row_pitch(hidden));
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
    // hidden is a multiple of 64 (checked above): whole 16-byte pieces (32.8 -> 27.9 us at the prefill shape against
    // 8-byte accesses with one row in flight)
    const int t8 = hidden / 8 >= 256 ? 256 : 128;
    moe_combine_bf16x8_kernel<<<static_cast<unsigned>(tokens), t8, 0, stream>>>(
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
// buffer of identical layout that the others can address (peer pointers over NVLink: plain loads
// and stores of these kernels, no multimem, no TMA or bulk copy on peer memory).  One step per rank:
//
//   dispatch   count kernel (routing optional) -> signal 0 -> place kernel: waits for every rank's
//              counts, then quantises the rank's tokens ONCE to NVFP4 and writes every (token, slot)
//              row straight into the expert-major FC1 operand of the rank that owns the slot's
//              expert (4.5 bits per element cross the wire instead of 16) -> signal 1
//   compute    wait for signal 1 of every rank; FC1; FC2, whose epilogue stores every output row
//              (bf16) into the landing zone of the rank that owns the token while the remaining
//              tiles are still being computed; -> signal 2
//   combine    wait for signal 2 of every rank; sum the k rows of each local token in f32 in slot
//              order, one bf16 rounding
//
// Per-rank return (return_mode 1) changes the second half: the place kernel also hands every rank the row index
// (or -1) and the routing weight of every (token, slot) it serves; FC2 keeps its rows on this GPU; a pre-sum kernel
// adds the rows of every (source rank, token) with their weights and stores ONE row per pair into the owner's
// landing zone -> signal 2; the combine adds a token's rows (one per serving rank) in rank order.  Fewer bytes
// cross NVLink; the sum is grouped by rank, so its bf16 roundings differ from the single-GPU operator's.
//
// The signals carry a step counter, so the three of them also separate consecutive steps (a rank can
// only run ahead of a peer by less than one phase of the same kind); there is no other barrier.
// Every wait is bounded (Exchange::wait_ns).  The reference has no multi-GPU path; this is the
// dispatch / combine all-to-all of an expert-parallel MoE written as kernels over peer memory.
// =============================================================================================
namespace b200fp4 {

int gemm_moe_fc2_push(const void* act_codes, const void* act_sf, const void* w2, const void* w2_sf,
                      const int* row_tag, const PeerPtrs& peers, size_t recv_off, const int* abort_flag,
                      const float* w2_alpha, const int* num_m_blocks_dev, const int* m_block_expert,
                      const int* m_block_rows, int max_m_blocks, int hidden, int inter, int experts, int few_rows,
                      int* status, cudaStream_t stream, const PeerSync* peer);

namespace {

struct EpLayout {
  // written by peers
  size_t flags, counts_all, xq_sf, xq, row_tag, recv, inv_row, inv_w;
  // private to the rank
  size_t ctrl, my_counts, slot_pos, ids, weights, num_m_blocks, m_block_expert, m_block_rows, act_sf, act, partial;
  size_t xq_sf_bytes, total;
  int max_m_blocks, rows_per_block, xq_sf_pitch;
};

EpLayout ep_layout(int64_t tokens_local, int hidden, int inter, int experts_local, int top_k, int world) {
  EpLayout L{};
  const int64_t slots_local = tokens_local * top_k;
  const int64_t slots = slots_local * world;
  // the few-row GEMM variants when the whole batch has at most 32 tokens (decode): 32 rows per block
  L.rows_per_block = moe_few_rows(tokens_local * world, top_k) ? 32 : 128;
  const int64_t blocks = std::min<int64_t>(experts_local, slots) + slots / L.rows_per_block;
  L.max_m_blocks = static_cast<int>(blocks);
  const int64_t rows = blocks * 128;
  const int64_t experts_total = static_cast<int64_t>(experts_local) * world;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t r = off;
    off = align_up(off + bytes, 256);
    return r;
  };
  L.flags = take(sizeof(int) * kSignalPhases * kMaxPeers);
  L.counts_all = take(sizeof(int) * world * experts_total);
  L.xq_sf_pitch = sf_row_pitch(hidden);
  L.xq_sf_bytes = xq_sf_buffer_bytes(blocks, hidden);
  L.xq_sf = take(L.xq_sf_bytes);
  L.xq = take(static_cast<size_t>(rows) * (hidden / 2));
  L.row_tag = take(sizeof(int) * rows);
  // output rows cross NVLink as bf16 rows (f32 accumulation in the combine): one per slot, or one per (token,
  // rank that serves some of the token's slots)
  L.recv = take(static_cast<size_t>(std::max<int64_t>(slots_local, tokens_local * world)) * hidden *
                sizeof(__nv_bfloat16));
  L.inv_row = take(sizeof(int) * slots);
  L.inv_w = take(sizeof(float) * slots);
  L.ctrl = take(sizeof(int) * kCtrlWords);
  L.my_counts = take(sizeof(int) * experts_total);
  L.slot_pos = take(sizeof(int) * slots_local);
  L.ids = take(sizeof(int) * slots_local);
  L.weights = take(sizeof(float) * slots_local);
  L.num_m_blocks = take(sizeof(int));
  L.m_block_expert = take(sizeof(int) * blocks);
  L.m_block_rows = take(sizeof(int) * blocks);
  L.act_sf = take(static_cast<size_t>(blocks) * ((inter + 63) / 64) * 512);
  L.act = take(static_cast<size_t>(rows) * (inter / 2));
  // FC2's rows before they are summed per (source rank, token) (per-rank return only)
  L.partial = take(static_cast<size_t>(rows) * hidden * sizeof(__nv_bfloat16));
  L.total = off;
  return L;
}

// one warp: wait for `phase` of every rank (bounded).  When the wait fails (now or earlier in the step) the
// block count of the grouped GEMMs that follow is set to zero: their tables may not have been written.
__global__ void ep_wait_kernel(Exchange ex, int phase, int* ctrl, int* status, int* num_m_blocks) {
  __shared__ int s_ok;
  const bool ok = wait_all_ranks(ex, phase, ctrl, status, &s_ok);
  if (!ok && threadIdx.x == 0 && num_m_blocks != nullptr) *num_m_blocks = 0;
}

// Weighted sum of the k rows that arrived for each local token (this rank's own memory).  kFew: CTA (token,
// column chunk) with independent loads of the k rows; otherwise one CTA per token.  Slots whose expert id is
// outside [0, experts_total) were never computed and are skipped.  The last CTA closes the step.
template <bool kFew>
__global__ void ep_combine_kernel(const __nv_bfloat16* __restrict__ recv, const int* __restrict__ ids,
                                  const float* __restrict__ weights, __nv_bfloat16* __restrict__ out, int hidden,
                                  int top_k, int experts_total, Exchange ex, int* ctrl, int* status) {
  __shared__ float s_w[64];
  __shared__ int s_valid[64];
  __shared__ int s_flag;
  const bool ok = wait_all_ranks(ex, 2, ctrl, status, &s_flag);
  const int t = blockIdx.x;
  if (ok) {
    if (threadIdx.x < top_k) {
      const int id = ids[static_cast<int64_t>(t) * top_k + threadIdx.x];
      s_valid[threadIdx.x] = id >= 0 && id < experts_total;
      s_w[threadIdx.x] = weights[static_cast<int64_t>(t) * top_k + threadIdx.x];
    }
    __syncthreads();
    const __nv_bfloat16* rows = recv + static_cast<int64_t>(t) * top_k * hidden;
    if constexpr (kFew) {
      const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
      if (c < hidden) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j0 = 0; j0 < top_k; j0 += 8) {
          float4 pv[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            pv[u] = (j0 + u < top_k && s_valid[j0 + u]) ? load_row4(rows + static_cast<int64_t>(j0 + u) * hidden + c)
                                                        : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (j0 + u < top_k && s_valid[j0 + u]) {
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
    } else {
      for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < top_k; ++j) {
          if (!s_valid[j]) continue;
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
  }
  // the last CTA closes the step: the next step's kernels signal and wait for epoch + 1
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(ctrl + kCtrlTicketCombine, 1) == static_cast<int>(gridDim.x * gridDim.y) - 1) {
      ctrl[kCtrlTicketCombine] = 0;
      if (ok) atomicAdd(ctrl + kCtrlEpoch, 1);
    }
  }
}

// Per-rank return, expert side.  One warp per (source rank r, token t of r): the rows of this rank that hold slots
// of that token (inv_row, written by r's place kernel) are summed with their routing weights in f32 in slot order,
// rounded to bf16 once and stored as ONE row into r's landing zone at [t][this rank] -- over NVLink when r is a
// peer.  A token whose top_k experts sit on few ranks sends few rows home instead of top_k.  A lane owns eight
// 16-byte pieces of a 2048-element segment at a time, so eight loads per row are in flight.  Persistent grid: every
// CTA fences its remote stores once; the last one raises signal 2 at every rank.
__global__ void __launch_bounds__(256)
ep_presum_push_kernel(const __nv_bfloat16* __restrict__ partial, const int* __restrict__ inv_row,
                      const float* __restrict__ inv_w, Exchange ex, size_t recv_off, int tokens_local, int hidden,
                      int top_k, int* ctrl) {
  __shared__ int s_flag;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int pairs = tokens_local * ex.world;
  const bool live = *reinterpret_cast<volatile int*>(ctrl + kCtrlAbort) == 0;
  for (int pair = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; pair < pairs && live; pair += warps) {
    const int r = pair % ex.world;                     // neighbouring warps send to different ranks
    const int t = pair / ex.world;
    int row = -1;
    float w = 0.0f;
    if (lane < top_k) {
      const int64_t idx = (static_cast<int64_t>(r) * tokens_local + t) * top_k + lane;
      row = inv_row[idx];
      if (row >= 0) w = inv_w[idx];
    }
    const unsigned served = __ballot_sync(0xffffffffu, row >= 0);
    if (served == 0) continue;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(ex.peers.p[r] + recv_off) +
                         (static_cast<int64_t>(t) * ex.world + ex.rank) * hidden;
    for (int seg = 0; seg < hidden; seg += 2048) {
      float acc[8][8];
#pragma unroll
      for (int q = 0; q < 8; ++q)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[q][i] = 0.0f;
      for (unsigned m = served; m != 0; m &= m - 1) {  // slot order
        const int j = __ffs(m) - 1;
        const int rj = __shfl_sync(0xffffffffu, row, j);
        const float wj = __shfl_sync(0xffffffffu, w, j);
        const __nv_bfloat16* src = partial + static_cast<int64_t>(rj) * hidden + seg + lane * 8;
        uint4 u[8];
#pragma unroll
        for (int q = 0; q < 8; ++q)
          u[q] = seg + q * 256 + lane * 8 < hidden ? *reinterpret_cast<const uint4*>(src + q * 256)
                                                   : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const uint32_t words[4] = {u[q].x, u[q].y, u[q].z, u[q].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            acc[q][2 * i] = __fadd_rn(acc[q][2 * i], __fmul_rn(wj, Pair16<__nv_bfloat16>::lo(words[i])));
            acc[q][2 * i + 1] = __fadd_rn(acc[q][2 * i + 1], __fmul_rn(wj, Pair16<__nv_bfloat16>::hi(words[i])));
          }
        }
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const int c = seg + q * 256 + lane * 8;
        if (c < hidden) {
          uint4 o;
          o.x = Pair16<__nv_bfloat16>::pack(acc[q][0], acc[q][1]);
          o.y = Pair16<__nv_bfloat16>::pack(acc[q][2], acc[q][3]);
          o.z = Pair16<__nv_bfloat16>::pack(acc[q][4], acc[q][5]);
          o.w = Pair16<__nv_bfloat16>::pack(acc[q][6], acc[q][7]);
          *reinterpret_cast<uint4*>(dst + c) = o;
        }
      }
    }
  }
  signal_when_all_ctas_done(ex, 2, ctrl, kCtrlTicketGemm, &s_flag);
}

// Per-rank return, home side: out[t] = sum over the ranks that serve at least one valid slot of t, in rank
// order, of the row that rank sent (f32 accumulation, one bf16 rounding).  The last CTA closes the step.
__global__ void ep_combine_ranks_kernel(const __nv_bfloat16* __restrict__ recv, const int* __restrict__ ids,
                                        __nv_bfloat16* __restrict__ out, int hidden, int top_k, int experts_total,
                                        Exchange ex, int* ctrl, int* status) {
  __shared__ int s_serves[kMaxPeers];
  __shared__ int s_flag;
  const bool ok = wait_all_ranks(ex, 2, ctrl, status, &s_flag);
  const int t = blockIdx.x;
  if (ok) {
    if (threadIdx.x < kMaxPeers) s_serves[threadIdx.x] = 0;
    __syncthreads();
    if (threadIdx.x < top_k) {
      const int id = ids[static_cast<int64_t>(t) * top_k + threadIdx.x];
      if (id >= 0 && id < experts_total) s_serves[id / ex.experts_local] = 1;
    }
    __syncthreads();
    const __nv_bfloat16* rows = recv + static_cast<int64_t>(t) * ex.world * hidden;
    for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int d = 0; d < ex.world; ++d) {
        if (!s_serves[d]) continue;
        const uint4 u = *reinterpret_cast<const uint4*>(rows + static_cast<int64_t>(d) * hidden + c);
        const uint32_t words[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[2 * i] = __fadd_rn(acc[2 * i], Pair16<__nv_bfloat16>::lo(words[i]));
          acc[2 * i + 1] = __fadd_rn(acc[2 * i + 1], Pair16<__nv_bfloat16>::hi(words[i]));
        }
      }
      uint4 o;
      o.x = Pair16<__nv_bfloat16>::pack(acc[0], acc[1]);
      o.y = Pair16<__nv_bfloat16>::pack(acc[2], acc[3]);
      o.z = Pair16<__nv_bfloat16>::pack(acc[4], acc[5]);
      o.w = Pair16<__nv_bfloat16>::pack(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(out + static_cast<int64_t>(t) * hidden + c) = o;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(ctrl + kCtrlTicketCombine, 1) == static_cast<int>(gridDim.x) - 1) {
      ctrl[kCtrlTicketCombine] = 0;
      if (ok) atomicAdd(ctrl + kCtrlEpoch, 1);
    }
  }
}

int ep_check(int64_t tokens_local, int hidden, int inter, int experts_local, int top_k, int world, int rank) {
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
    return fail(kInvalidArgument, "world=%d rank=%d (at most %d ranks)", world, rank, kMaxPeers);
  if (tokens_local < 0 || top_k < 1 || top_k > 64 || experts_local < 1 ||
      static_cast<int64_t>(experts_local) * world > 1024)
    return fail(kInvalidArgument, "tokens=%lld top_k=%d experts=%d x %d ranks (at most 1024 experts in total)",
                static_cast<long long>(tokens_local), top_k, experts_local, world);
  if (hidden % 64 != 0 || hidden < 64) return fail(kUnsupported, "hidden=%d must be a multiple of 64", hidden);
  if (inter % 128 != 0 || inter < 128) return fail(kUnsupported, "intermediate=%d must be a multiple of 128", inter);
  if (tokens_local * top_k > (1ll << 24) || tokens_local * world * top_k > (1ll << 30))
    return fail(kUnsupported, "too many routed rows");
  return kOk;
}

// return_mode: 0 = FC2's epilogue sends one row per slot home; 1 = rows are summed per (source rank, token) on
// the expert's rank first and one row per (token, rank) travels
int ep_exchange(const void* const* peer_buffers, int rank, int world, int experts_local, const EpLayout& L,
                double wait_ms, Exchange* ex, int return_mode = 0) {
  if (return_mode != 0 && return_mode != 1) return fail(kInvalidArgument, "return_mode must be 0 or 1");
  if (peer_buffers == nullptr) return fail(kInvalidArgument, "peer_buffers is null");
  *ex = Exchange{};
  for (int i = 0; i < world; ++i) {
    if (peer_buffers[i] == nullptr || (reinterpret_cast<uintptr_t>(peer_buffers[i]) & 255))
      return fail(kInvalidArgument, "peer buffer %d is null or not 256-byte aligned", i);
    ex->peers.p[i] = static_cast<uint8_t*>(const_cast<void*>(peer_buffers[i]));
  }
  ex->flags = L.flags;
  ex->counts_all = L.counts_all;
  ex->xq = L.xq;
  ex->xq_sf = L.xq_sf;
  ex->xq_sf_pitch = L.xq_sf_pitch;
  ex->row_tag = L.row_tag;
  ex->inv_row = return_mode == 1 ? L.inv_row : 0;
  ex->inv_w = return_mode == 1 ? L.inv_w : 0;
  ex->rank = rank;
  ex->world = world;
  ex->experts_local = experts_local;
  if (!(wait_ms > 0.0) || wait_ms > 60000.0) return fail(kInvalidArgument, "wait_ms must be in (0, 60000]");
  ex->wait_ns = static_cast<unsigned long long>(wait_ms * 1e6);
  return kOk;
}

}  // namespace

size_t moe_ep_buffer_bytes(int64_t tokens_local, int hidden, int inter, int experts_local, int top_k, int world) {
  return ep_layout(tokens_local, hidden, inter, experts_local, top_k, world).total;
}

// Clears the signal words, counters and the abort word of the rank's own buffer.  Call it on every rank with a
// host-side barrier before and after (no step may be in flight anywhere), once after allocating the buffers and
// again to recover after a wait expired.
int moe_ep_reset(void* own_buffer, int64_t tokens_local, int hidden, int inter, int experts_local, int top_k,
                 int world, cudaStream_t stream) {
  int rc = ep_check(tokens_local, hidden, inter, experts_local, top_k, world, 0);
  if (rc) return rc;
  if (own_buffer == nullptr || (reinterpret_cast<uintptr_t>(own_buffer) & 255))
    return fail(kInvalidArgument, "own_buffer is null or not 256-byte aligned");
  const EpLayout L = ep_layout(tokens_local, hidden, inter, experts_local, top_k, world);
  uint8_t* b = static_cast<uint8_t*>(own_buffer);
  B200_CUDA(cudaMemsetAsync(b + L.flags, 0, sizeof(int) * kSignalPhases * kMaxPeers, stream));
  // control words, counters, routing and the block tables of the grouped GEMMs (zero blocks = nothing to do)
  B200_CUDA(cudaMemsetAsync(b + L.ctrl, 0, L.act_sf - L.ctrl, stream));
  return kOk;
}

// dispatch: (route +) count, publish counts, quantise and place the rows at the expert owners.
// logits == nullptr: ids (and weights, used by the combine) are the caller's; else they are computed here into
// the rank's buffer.  phases: bit 0 = the count kernel, bit 1 = the place kernel (the two are separate entry
// points as well so that a test can interleave the ranks of a group on one stream).
// return_mode 1 (per-rank return) also needs the routing weights here (`weights`, with ids; from the router
// otherwise): the place kernel hands them to the ranks that own the experts.
int moe_ep_dispatch(const void* x, const int* ids, const float* weights, const float* logits, int route_experts,
                    int renormalize, const void* const* peer_buffers, int rank, int world, int64_t tokens_local,
                    int hidden, int inter, int experts_local, int top_k, int return_mode, double wait_ms, int phases,
                    int* status, cudaStream_t stream) {
  int rc = ep_check(tokens_local, hidden, inter, experts_local, top_k, world, rank);
  if (rc) return rc;
  if (x == nullptr || (ids == nullptr && logits == nullptr) || status == nullptr)
    return fail(kInvalidArgument, "null pointer argument");
  if (return_mode == 1 && logits == nullptr && weights == nullptr)
    return fail(kInvalidArgument, "the per-rank return needs the routing weights at dispatch");
  if (reinterpret_cast<uintptr_t>(x) & 31) return fail(kInvalidArgument, "x must be 32-byte aligned");
  const int experts_total = experts_local * world;
  if (logits != nullptr) {
    rc = route_check(static_cast<int>(tokens_local), route_experts, top_k);
    if (rc) return rc;
    if (route_experts != experts_total)
      return fail(kInvalidArgument, "logits have %d columns but the group serves %d experts", route_experts, experts_total);
  }
  const EpLayout L = ep_layout(tokens_local, hidden, inter, experts_local, top_k, world);
  Exchange ex;
  rc = ep_exchange(peer_buffers, rank, world, experts_local, L, wait_ms, &ex, return_mode);
  if (rc) return rc;
  if (tokens_local == 0) return fail(kUnsupported, "every rank must hold at least one token");
  uint8_t* b = ex.peers.p[rank];
  int* ctrl = reinterpret_cast<int*>(b + L.ctrl);
  int* ids_buf = reinterpret_cast<int*>(b + L.ids);
  float* w_buf = reinterpret_cast<float*>(b + L.weights);
  if (phases & 1) {
    rc = launch_count(logits, route_experts, renormalize, ids, ids_buf, w_buf, static_cast<int>(tokens_local), top_k, 0,
                      experts_total, reinterpret_cast<int*>(b + L.my_counts), reinterpret_cast<int*>(b + L.slot_pos),
                      ctrl, ex, stream);
    if (rc) return rc;
  }
  if (phases & 2) {
    rc = launch_place(x, logits != nullptr ? ids_buf : ids, reinterpret_cast<int*>(b + L.slot_pos), ex,
                      static_cast<int>(tokens_local), hidden, top_k, 0, experts_total, L.max_m_blocks,
                      L.rows_per_block, nullptr, reinterpret_cast<int*>(b + L.num_m_blocks),
                      reinterpret_cast<int*>(b + L.m_block_expert), reinterpret_cast<int*>(b + L.m_block_rows), ctrl,
                      status, stream, logits != nullptr ? w_buf : weights);
    if (rc) return rc;
  }
  return kOk;
}

int moe_ep_compute(const void* const* peer_buffers, int rank, int world, const void* w1, const void* w1_sf,
                   const void* w2, const void* w2_sf, const float* w1_alpha, const float* w2_alpha,
                   const float* fc2_input_scale, int64_t tokens_local, int hidden, int inter, int experts_local,
                   int top_k, int return_mode, double wait_ms, int* status, cudaStream_t stream) {
  int rc = ep_check(tokens_local, hidden, inter, experts_local, top_k, world, rank);
  if (rc) return rc;
  if (w1 == nullptr || w1_sf == nullptr || w2 == nullptr || w2_sf == nullptr || status == nullptr)
    return fail(kInvalidArgument, "null pointer argument");
  const EpLayout L = ep_layout(tokens_local, hidden, inter, experts_local, top_k, world);
  Exchange ex;
  rc = ep_exchange(peer_buffers, rank, world, experts_local, L, wait_ms, &ex, return_mode);
  if (rc) return rc;
  uint8_t* b = ex.peers.p[rank];
  int* ctrl = reinterpret_cast<int*>(b + L.ctrl);
  const int* num_m_blocks = reinterpret_cast<const int*>(b + L.num_m_blocks);
  const int* m_block_expert = reinterpret_cast<const int*>(b + L.m_block_expert);
  const int* m_block_rows = reinterpret_cast<const int*>(b + L.m_block_rows);
  const int few_rows = L.rows_per_block == 32;
  // FC1 waits (inside the kernel, bounded) for the "rows placed" signal of every rank; FC2's last CTA raises
  // "output rows delivered" at every rank
  PeerSync sync{};
  sync.ctrl = ctrl;
  sync.wait_ns = ex.wait_ns;
  sync.rank = rank;
  sync.world = world;
  sync.flags_off = L.flags;
  sync.peers = ex.peers;
  PeerSync fc1_sync = sync;
  fc1_sync.wait_flags = reinterpret_cast<const int*>(b + L.flags) + 1 * kMaxPeers;
  PeerSync fc2_sync = sync;
  fc2_sync.signal_phase = 2;
  fc2_sync.ticket = kCtrlTicketGemm;
  rc = gemm_moe_fc1(b + L.xq, b + L.xq_sf, w1, w1_sf, b + L.act, b + L.act_sf, w1_alpha, fc2_input_scale, num_m_blocks,
                    m_block_expert, m_block_rows, L.max_m_blocks, hidden, inter, experts_local, few_rows, status, stream,
                    &fc1_sync, L.xq_sf_pitch);
  if (rc) return rc;
  if (return_mode == 1) {
    // FC2 keeps its rows on this GPU (TMA stores); a second kernel sums them per (source rank, token) and sends
    // one row per pair home
    rc = gemm_moe_fc2(b + L.act, b + L.act_sf, w2, w2_sf, b + L.partial, 1, w2_alpha, num_m_blocks, m_block_expert,
                      m_block_rows, L.max_m_blocks, hidden, inter, experts_local, few_rows, status, stream);
    if (rc) return rc;
    if (top_k > 32) return fail(kUnsupported, "the per-rank return serves top_k <= 32");
    // one warp per (source rank, token); two resident CTAs per SM (128 registers), one system-wide fence per CTA
    const int64_t pairs = tokens_local * world;
    const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>((pairs + 7) / 8, 2 * sm_count_of_current_device())));
    ep_presum_push_kernel<<<grid, 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(b + L.partial), reinterpret_cast<const int*>(b + L.inv_row),
        reinterpret_cast<const float*>(b + L.inv_w), ex, L.recv, static_cast<int>(tokens_local), hidden, top_k, ctrl);
    return check_cuda(cudaGetLastError(), "ep_presum_push_kernel launch");
  }
  return gemm_moe_fc2_push(b + L.act, b + L.act_sf, w2, w2_sf, reinterpret_cast<const int*>(b + L.row_tag), ex.peers,
                           L.recv, ctrl + kCtrlAbort, w2_alpha, num_m_blocks, m_block_expert, m_block_rows,
                           L.max_m_blocks, hidden, inter, experts_local, few_rows, status, stream, &fc2_sync);
}

// ids / weights: the routing of the local tokens; null = what the dispatch computed from logits
int moe_ep_combine(const void* const* peer_buffers, int rank, int world, const int* ids, const float* weights,
                   void* out, int64_t tokens_local, int hidden, int inter, int experts_local, int top_k,
                   int return_mode, double wait_ms, int* status, cudaStream_t stream) {
  int rc = ep_check(tokens_local, hidden, inter, experts_local, top_k, world, rank);
  if (rc) return rc;
  if (out == nullptr || status == nullptr || (ids == nullptr) != (weights == nullptr))
    return fail(kInvalidArgument, "null pointer argument (ids and weights are given together or not at all)");
  const EpLayout L = ep_layout(tokens_local, hidden, inter, experts_local, top_k, world);
  Exchange ex;
  rc = ep_exchange(peer_buffers, rank, world, experts_local, L, wait_ms, &ex, return_mode);
  if (rc) return rc;
  if (tokens_local == 0) return kOk;
  uint8_t* b = ex.peers.p[rank];
  int* ctrl = reinterpret_cast<int*>(b + L.ctrl);
  if (ids == nullptr) {
    ids = reinterpret_cast<const int*>(b + L.ids);
    weights = reinterpret_cast<const float*>(b + L.weights);
  }
  const __nv_bfloat16* recv = reinterpret_cast<const __nv_bfloat16*>(b + L.recv);
  const int threads = hidden / 4 >= 256 ? 256 : 128;
  const int experts_total = experts_local * world;
  if (return_mode == 1) {
    ep_combine_ranks_kernel<<<static_cast<unsigned>(tokens_local), hidden / 8 >= 256 ? 256 : 128, 0, stream>>>(
        recv, ids, static_cast<__nv_bfloat16*>(out), hidden, top_k, experts_total, ex, ctrl, status);
    return check_cuda(cudaGetLastError(), "ep_combine_ranks_kernel launch");
  }
  if (tokens_local <= 256) {
    ep_combine_kernel<true><<<dim3(static_cast<unsigned>(tokens_local), (hidden / 4 + threads - 1) / threads), threads, 0,
                              stream>>>(recv, ids, weights, static_cast<__nv_bfloat16*>(out), hidden, top_k,
                                        experts_total, ex, ctrl, status);
  } else {
    ep_combine_kernel<false><<<static_cast<unsigned>(tokens_local), threads, 0, stream>>>(
        recv, ids, weights, static_cast<__nv_bfloat16*>(out), hidden, top_k, experts_total, ex, ctrl, status);
  }
  return check_cuda(cudaGetLastError(), "ep_combine_kernel launch");
}

// Copies the routing that the dispatch computed from logits (ids i32, weights f32, [tokens_local, top_k]).
int moe_ep_routing(const void* own_buffer, int* ids_out, float* weights_out, int64_t tokens_local, int hidden,
                   int inter, int experts_local, int top_k, int world, cudaStream_t stream) {
  int rc = ep_check(tokens_local, hidden, inter, experts_local, top_k, world, 0);
  if (rc) return rc;
  if (own_buffer == nullptr || ids_out == nullptr || weights_out == nullptr)
    return fail(kInvalidArgument, "null pointer argument");
  const EpLayout L = ep_layout(tokens_local, hidden, inter, experts_local, top_k, world);
  const uint8_t* b = static_cast<const uint8_t*>(own_buffer);
  const size_t n = static_cast<size_t>(tokens_local) * top_k;
  B200_CUDA(cudaMemcpyAsync(ids_out, b + L.ids, n * sizeof(int), cudaMemcpyDeviceToDevice, stream));
  B200_CUDA(cudaMemcpyAsync(weights_out, b + L.weights, n * sizeof(float), cudaMemcpyDeviceToDevice, stream));
  return kOk;
}

// Self-test of the bounded cross-rank wait on ONE GPU: a wait for `world` ranks on a buffer whose signal words
// nobody writes.  The kernel gives up after wait_ms, sets kStatusPeerWaitExpired in the device status word and
// the abort word of the buffer, and returns; no peer memory is involved.
int moe_ep_wait_selftest(void* own_buffer, int world, double wait_ms, int64_t tokens_local, int hidden, int inter,
                         int experts_local, int top_k, int* status, cudaStream_t stream) {
  int rc = ep_check(tokens_local, hidden, inter, experts_local, top_k, world, 0);
  if (rc) return rc;
  if (own_buffer == nullptr || status == nullptr) return fail(kInvalidArgument, "null pointer argument");
  const EpLayout L = ep_layout(tokens_local, hidden, inter, experts_local, top_k, world);
  const void* bufs[kMaxPeers];
  for (int i = 0; i < world; ++i) bufs[i] = own_buffer;      // only this rank's words are ever read
  Exchange ex;
  rc = ep_exchange(bufs, 0, world, experts_local, L, wait_ms, &ex);
  if (rc) return rc;
  ep_wait_kernel<<<1, 32, 0, stream>>>(ex, 1, reinterpret_cast<int*>(static_cast<uint8_t*>(own_buffer) + L.ctrl), status,
                                       nullptr);
  return check_cuda(cudaGetLastError(), "ep_wait_kernel launch");
}

}  // namespace b200fp4
