// Fused RMSNorm / residual-add RMSNorm + NVFP4 quantisation for sm_100a.
//
// Replaces the flashinfer CuTe-DSL operators the reference runs verbatim
// (call sites tests/python/test_flashinfer_norm_verbatim.py:134,155-164); the
// arithmetic contract is the reference's torch golden (same file, lines 58-99).
//
// One pass over HBM: a row is read once (x, and residual for the add variant),
// kept in registers across the row reduction, and written once (residual, e2m1
// codes, e4m3 scale factors).  Each thread owns kVec adjacent 16-element scale
// blocks (one 256-bit load per block and tensor), so a block's amax, scale
// factor and code bytes never leave the thread; neighbouring lanes merge their
// scale bytes into one 32-bit store, which is contiguous both in the row-major
// and in the 128x4 tiled scale-factor layout.  The grid is persistent (a
// multiple of the SM count); every thread parks the f32 copy of its own slice
// of the weight vector in shared memory once and re-reads it per row.
#include <atomic>

#include "common.cuh"

namespace b200fp4 {
namespace {

constexpr int kMaxUnitsPerThread = 2;    // strided units per thread per row
constexpr int kMaxThreads = 512;

struct NormParams {
  const void* x;
  void* residual;           // in/out, null for plain rmsnorm
  const void* weight;
  uint8_t* y;               // [rows, hidden/2]
  uint8_t* sf_swizzled;     // 128x4 tiled, or null
  uint8_t* sf_rowmajor;     // [rows, hidden/16], or null
  const float* global_scale;
  float eps;
  int64_t rows;
  int hidden;
  int64_t x_row_stride;     // elements
  int64_t res_row_stride;   // elements
};

template <typename T>
__device__ __forceinline__ void unpack16(const U32x8& p, float (&f)[16]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    f[2 * i] = Pair16<T>::lo(p.v[i]);
    f[2 * i + 1] = Pair16<T>::hi(p.v[i]);
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// A "unit" is kVec adjacent 16-element chunks; thread t of a team handles units
// t, t+team, ... (kUnits of them).  kWarpRow: the team is one warp and a CTA
// works on one row per warp (hidden <= 512); otherwise the team is the CTA.
// kCap: upper bound of the block size of this instantiation; small blocks ask the compiler for a
// register budget that lets five of them share an SM.
// kPipe: the loads of the team's next row are issued as soon as the current row's registers have been consumed
// (before the row reduction), so DRAM requests stay in flight through the reduction, the quantisation and the
// stores; costs the 32 load registers per thread for the whole loop, hence fewer resident CTAs.
template <typename T, bool kAdd, int kVec, int kUnits, bool kWarpRow, int kCap, bool kPipe = false>
__global__ void __launch_bounds__(kCap, kPipe ? 3 : (kCap <= 256 ? 5 : 2)) norm_quant_kernel(const NormParams p) {
  extern __shared__ float4 wsm[];          // per-thread weight slices, f32
  __shared__ float red[2][kMaxThreads / 32];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  const int nchunks = p.hidden >> 4;
  const int team = kWarpRow ? 32 : blockDim.x;
  const int tid = kWarpRow ? lane : threadIdx.x;
  const int rk = (nchunks + 3) >> 2;
  const float gs = __ldg(p.global_scale);
  const float n_as_float = static_cast<float>(p.hidden);
  const T* __restrict__ xg = static_cast<const T*>(p.x);
  T* rg = static_cast<T*>(p.residual);
  const bool sf_row_vec = (nchunks & 3) == 0;                  // row-major SF rows are 4-byte aligned
  const bool y_vec16 = ((p.hidden >> 1) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.y) & 15) == 0;
  constexpr int kSlots = kUnits * kVec * 4;                    // float4 slots per thread
  float4* wmine = wsm + (kWarpRow ? warp * kSlots * 32 : 0) + tid;   // slot s lives at wmine[s * team]

#pragma unroll
  for (int u = 0; u < kUnits; ++u) {
#pragma unroll
    for (int v = 0; v < kVec; ++v) {
      const int chunk = (tid + u * team) * kVec + v;
      float wf[16];
      if (chunk < nchunks) {
        unpack16<T>(ld_stream_32B(static_cast<const T*>(p.weight) + chunk * 16), wf);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) wf[i] = 0.0f;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q)
        wmine[((u * kVec + v) * 4 + q) * team] = make_float4(wf[4 * q], wf[4 * q + 1], wf[4 * q + 2], wf[4 * q + 3]);
    }
  }
  // each thread only ever reads back its own slots: no barrier needed

  const int64_t row0 = kWarpRow ? static_cast<int64_t>(blockIdx.x) * nwarps + warp : blockIdx.x;
  const int64_t row_step = kWarpRow ? static_cast<int64_t>(gridDim.x) * nwarps : gridDim.x;
  int parity = 0;
  const uint32_t row_bytes = static_cast<uint32_t>(p.hidden) * 2u;
  // kPipe: raw rows travel in these registers from one iteration to the next
  U32x8 xnext[kPipe ? kUnits * kVec : 1], rnext[kPipe && kAdd ? kUnits * kVec : 1];
  auto load_row = [&](int64_t r) {
#pragma unroll
    for (int u = 0; u < kUnits; ++u) {
#pragma unroll
      for (int v = 0; v < kVec; ++v) {
        const int chunk = (tid + u * team) * kVec + v;
        if (chunk < nchunks) {
          xnext[u * kVec + v] = ld_stream_32B(xg + r * p.x_row_stride + chunk * 16);
          if constexpr (kAdd) rnext[u * kVec + v] = ld_32B(rg + r * p.res_row_stride + chunk * 16);
        }
      }
    }
  };
  if constexpr (kPipe) {
    if (row0 < p.rows) load_row(row0);
  }
  for (int64_t row = row0; row < p.rows; row += row_step, parity ^= 1) {
    // pull the row this team will work on next (kPipe: the one after it) into L2 while the current one is processed
    const int64_t ahead = row + (kPipe ? 2 : 1) * row_step;
    if (tid == 0 && ahead < p.rows) {
      prefetch_l2_bulk(xg + ahead * p.x_row_stride, row_bytes);
      if constexpr (kAdd) prefetch_l2_bulk(rg + ahead * p.res_row_stride, row_bytes);
    }
    // ---- phase 1: load, (add, round, write residual), sum of squares; all f32 math on register pairs
    // what phase 2 normalises, kept as packed 16-bit pairs so that few registers live across the row reduction
    uint32_t h[kUnits * kVec][8];
    uint64_t ssq2 = 0;                       // {0.0f, 0.0f}
#pragma unroll
    for (int u = 0; u < kUnits; ++u) {
#pragma unroll
      for (int v = 0; v < kVec; ++v) {
        const int c = u * kVec + v;
        const int chunk = (tid + u * team) * kVec + v;
        if (chunk < nchunks) {
          const U32x8 xv = kPipe ? xnext[c] : ld_stream_32B(xg + row * p.x_row_stride + chunk * 16);
          if constexpr (kAdd) {
            T* rptr = rg + row * p.res_row_stride + chunk * 16;
            const U32x8 rv = kPipe ? rnext[c] : ld_32B(rptr);
            U32x8 outv;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint64_t s2 = f32x2_add(pair16_to_f32x2<T>(xv.v[i]), pair16_to_f32x2<T>(rv.v[i]));
              ssq2 = f32x2_fma(s2, s2, ssq2);
              outv.v[i] = f32x2_to_pair16<T>(s2);
              h[c][i] = outv.v[i];                         // the normalised value is built from the ROUNDED residual
            }
            st_32B(rptr, outv);
          } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 w4 = wmine[(c * 4 + q) * team];
              const uint64_t x0 = pair16_to_f32x2<T>(xv.v[2 * q]);
              const uint64_t x1 = pair16_to_f32x2<T>(xv.v[2 * q + 1]);
              ssq2 = f32x2_fma(x0, x0, ssq2);
              ssq2 = f32x2_fma(x1, x1, ssq2);
              // x*w is rounded to the input type before the f32 scaling
              h[c][2 * q] = f32x2_to_pair16<T>(f32x2_mul(x0, f32x2_pack(w4.x, w4.y)));
              h[c][2 * q + 1] = f32x2_to_pair16<T>(f32x2_mul(x1, f32x2_pack(w4.z, w4.w)));
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) h[c][i] = 0;
        }
      }
    }
    float ssq = __fadd_rn(f32x2_lo(ssq2), f32x2_hi(ssq2));
    if constexpr (kPipe) {
      if (row + row_step < p.rows) load_row(row + row_step);      // in flight until the next iteration's phase 1
    }

    // ---- row reduction: lanes, then (CTA teams) warps through shared memory
    ssq = warp_sum(ssq);
    if constexpr (!kWarpRow) {
      if (lane == 0) red[parity][warp] = ssq;
      __syncthreads();
      ssq = warp_sum(lane < nwarps ? red[parity][lane] : 0.0f);
    }
    // 1/sqrt(mean + eps) with IEEE division and square root
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ssq, n_as_float), p.eps)));
    const uint64_t rstd2 = f32x2_pack(rstd, rstd);

    // ---- phase 2: scale, quantise, store
#pragma unroll
    for (int u = 0; u < kUnits; ++u) {
      uint32_t codes[kVec][2];
      uint32_t sfb[kVec];
      const int chunk0 = (tid + u * team) * kVec;
#pragma unroll
      for (int v = 0; v < kVec; ++v) {
        const int c = u * kVec + v;
        uint64_t val[8];
        if constexpr (kAdd) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float4 w4 = wmine[(c * 4 + q) * team];
            val[2 * q] = f32x2_mul(f32x2_mul(pair16_to_f32x2<T>(h[c][2 * q]), rstd2), f32x2_pack(w4.x, w4.y));
            val[2 * q + 1] =
                f32x2_mul(f32x2_mul(pair16_to_f32x2<T>(h[c][2 * q + 1]), rstd2), f32x2_pack(w4.z, w4.w));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) val[i] = f32x2_mul(pair16_to_f32x2<T>(h[c][i]), rstd2);
        }
        quantize_block16<false>(val, gs, codes[v][0], codes[v][1], sfb[v]);
        if (chunk0 + v >= nchunks) sfb[v] = 0;
      }
      // codes: kVec * 8 contiguous bytes per thread
      uint8_t* yrow = p.y + row * (p.hidden >> 1);
      if constexpr (kVec == 2) {
        if (chunk0 + 1 < nchunks) {
          if (y_vec16) {
            *reinterpret_cast<uint4*>(yrow + chunk0 * 8) =
                make_uint4(codes[0][0], codes[0][1], codes[1][0], codes[1][1]);
          } else {
            *reinterpret_cast<uint2*>(yrow + chunk0 * 8) = make_uint2(codes[0][0], codes[0][1]);
            *reinterpret_cast<uint2*>(yrow + chunk0 * 8 + 8) = make_uint2(codes[1][0], codes[1][1]);
          }
        } else if (chunk0 < nchunks) {
          *reinterpret_cast<uint2*>(yrow + chunk0 * 8) = make_uint2(codes[0][0], codes[0][1]);
        }
      } else {
        if (chunk0 < nchunks) *reinterpret_cast<uint2*>(yrow + chunk0 * 8) = make_uint2(codes[0][0], codes[0][1]);
      }
      // scale bytes: the lane whose first chunk is a multiple of 4 collects four K-blocks
      uint32_t quad;
      bool leader;
      if constexpr (kVec == 2) {
        const uint32_t pair = sfb[0] | (sfb[1] << 8);
        quad = pair | (__shfl_down_sync(0xffffffffu, pair, 1) << 16);
        leader = (lane & 1) == 0;
      } else {
        quad = sfb[0];
        quad |= __shfl_down_sync(0xffffffffu, sfb[0], 1) << 8;
        quad |= __shfl_down_sync(0xffffffffu, sfb[0], 2) << 16;
        quad |= __shfl_down_sync(0xffffffffu, sfb[0], 3) << 24;
        leader = (lane & 3) == 0;
      }
      if (leader && chunk0 < nchunks) {
        if (p.sf_swizzled != nullptr) {
          *reinterpret_cast<uint32_t*>(p.sf_swizzled + sf_swizzled_offset(row, chunk0, rk)) = quad;
        }
        if (p.sf_rowmajor != nullptr) {
          uint8_t* dst = p.sf_rowmajor + row * nchunks + chunk0;
          if (sf_row_vec) {
            *reinterpret_cast<uint32_t*>(dst) = quad;
          } else {
            for (int j = 0; j < 4 && chunk0 + j < nchunks; ++j) dst[j] = static_cast<uint8_t>(quad >> (8 * j));
          }
        }
      }
    }
  }
}

constexpr int kMaxDevices = 64;

int current_device_ordinal() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dev >= 0 && dev < kMaxDevices ? dev : 0;
}

// SM count, cached per device ordinal
int sm_count(int dev) {
  static std::atomic<int> cached[kMaxDevices];
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

template <typename T, bool kAdd, int kVec, int kUnits, bool kWarpRow, int kCap, bool kPipe = false>
int launch_one(const NormParams& p, int threads, cudaStream_t stream) {
  auto kern = norm_quant_kernel<T, kAdd, kVec, kUnits, kWarpRow, kCap, kPipe>;
  const size_t smem = static_cast<size_t>(kUnits) * kVec * 4 * sizeof(float4) * threads;
  // Shared-memory opt-in and occupancy are per device and per block size: queried once for each (this
  // instantiation, device, block size) and remembered -- the two driver calls cost more host time than the
  // launch of a small problem.  per_sm_cache holds (threads << 8 | resident CTAs), 0 = not yet known.
  static std::atomic<int> per_sm_cache[kMaxDevices];
  const int dev = current_device_ordinal();
  int per_sm = 0;
  const int cached = per_sm_cache[dev].load(std::memory_order_acquire);
  if (cached != 0 && (cached >> 8) == threads) {
    per_sm = cached & 0xff;
  } else {
    if (smem > 48 * 1024) {
      B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    }
    B200_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, smem));
    if (per_sm < 1) return fail(kUnsupported, "norm_quant_kernel does not fit on an SM (%zu bytes of shared memory)", smem);
    if (per_sm > 255) per_sm = 255;
    per_sm_cache[dev].store((threads << 8) | per_sm, std::memory_order_release);
  }
  // the residual-add variant is DRAM-bound with four resident CTAs per SM already; more of them only
  // lengthen the last wave (measured on B200: 70 us with 4, 74 us with 6 at [8192, 7168])
  if (kAdd && !kWarpRow && per_sm > 4) per_sm = 4;
  const int64_t rows_per_cta = kWarpRow ? threads / 32 : 1;
  const int64_t want = (p.rows + rows_per_cta - 1) / rows_per_cta;
  int64_t grid = static_cast<int64_t>(sm_count(dev)) * per_sm;
  if (grid > want) grid = want;
  kern<<<static_cast<unsigned>(grid), threads, smem, stream>>>(p);
  return check_cuda(cudaGetLastError(), "norm_quant_kernel launch");
}

template <typename T, bool kAdd>
int dispatch(const NormParams& p, cudaStream_t stream) {
  const int nchunks = p.hidden / 16;
  if (nchunks <= 32) return launch_one<T, kAdd, 1, 1, true, 128>(p, 128, stream);
  const int nunits = (nchunks + 1) / 2;                       // two adjacent chunks per unit
  const int units = (nunits + kMaxThreads - 1) / kMaxThreads;
  const int threads = (((nunits + units - 1) / units) + 31) / 32 * 32;
  switch (units) {
    case 1:
      // the residual-add variant keeps its next row's loads in flight in registers (three resident CTAs instead
      // of four: 71.2 -> 70.0 us at [8192, 7168]; with four pipelined CTAs 77 us); the plain variant, with half
      // the bytes per row, does better with more resident CTAs and the L2 prefetch alone
      if (kAdd && threads <= 256) return launch_one<T, kAdd, 2, 1, false, 256, kAdd>(p, threads, stream);
      return threads <= 256 ? launch_one<T, kAdd, 2, 1, false, 256>(p, threads, stream)
                            : launch_one<T, kAdd, 2, 1, false, kMaxThreads>(p, threads, stream);
    case 2: return launch_one<T, kAdd, 2, 2, false, kMaxThreads>(p, threads, stream);
    default: return fail(kUnsupported, "hidden=%d exceeds the supported maximum of %d", p.hidden,
                         32 * kMaxThreads * kMaxUnitsPerThread);
  }
}

}  // namespace

// sf_layout: 0 = row-major [rows, hidden/16], 1 = 128x4 tiled, 2 = both
// (tiled into block_scale, row-major into block_scale_unswizzled)
int norm_fp4quant_launch(const void* x, void* residual, const void* weight, void* y_fp4, void* block_scale,
                         void* block_scale_unswizzled, const float* global_scale, float eps, int64_t rows,
                         int hidden, int64_t x_row_stride, int64_t res_row_stride, int dtype, int sf_layout,
                         cudaStream_t stream) {
  if (x == nullptr || weight == nullptr || y_fp4 == nullptr || block_scale == nullptr || global_scale == nullptr)
    return fail(kInvalidArgument, "null pointer argument");
  if (rows < 0) return fail(kInvalidArgument, "rows=%lld is negative", static_cast<long long>(rows));
  if (hidden < 64 || hidden % 16 != 0)
    return fail(kInvalidArgument, "hidden=%d must be a multiple of 16 and at least 64", hidden);
  if (x_row_stride % 16 != 0 || (residual != nullptr && res_row_stride % 16 != 0))
    return fail(kInvalidArgument, "row strides must be multiples of 16 elements (32-byte rows)");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(weight)) & 31)
    return fail(kInvalidArgument, "input, residual and weight must be 32-byte aligned");
  if ((reinterpret_cast<uintptr_t>(y_fp4) & 7) || (reinterpret_cast<uintptr_t>(block_scale) & 3))
    return fail(kInvalidArgument, "y_fp4 must be 8-byte and block_scale 4-byte aligned");
  if (dtype != 0 && dtype != 1) return fail(kUnsupported, "dtype code %d (0 = fp16, 1 = bf16)", dtype);
  if (sf_layout < 0 || sf_layout > 2) return fail(kInvalidArgument, "sf_layout=%d", sf_layout);
  if (sf_layout == 2 && block_scale_unswizzled == nullptr)
    return fail(kInvalidArgument, "sf_layout=2 needs block_scale_unswizzled");
  if (rows == 0) return kOk;

  NormParams p{};
  p.x = x;
  p.residual = residual;
  p.weight = weight;
  p.y = static_cast<uint8_t*>(y_fp4);
  p.sf_swizzled = sf_layout >= 1 ? static_cast<uint8_t*>(block_scale) : nullptr;
  p.sf_rowmajor = sf_layout == 0 ? static_cast<uint8_t*>(block_scale)
                                 : (sf_layout == 2 ? static_cast<uint8_t*>(block_scale_unswizzled) : nullptr);
  p.global_scale = global_scale;
  p.eps = eps;
  p.rows = rows;
  p.hidden = hidden;
  p.x_row_stride = x_row_stride;
  p.res_row_stride = res_row_stride;

  const int nchunks = hidden / 16;
  if (p.sf_swizzled != nullptr && ((rows & 127) != 0 || (nchunks & 3) != 0)) {
    // rows / K-blocks that only pad a 128x4 tile must read as zero
    const size_t bytes = static_cast<size_t>((rows + 127) / 128) * ((nchunks + 3) / 4) * 512;
    B200_CUDA(cudaMemsetAsync(p.sf_swizzled, 0, bytes, stream));
  }
  const bool add = residual != nullptr;
  if (dtype == 1) return add ? dispatch<__nv_bfloat16, true>(p, stream) : dispatch<__nv_bfloat16, false>(p, stream);
  return add ? dispatch<__half, true>(p, stream) : dispatch<__half, false>(p, stream);
}

}  // namespace b200fp4
