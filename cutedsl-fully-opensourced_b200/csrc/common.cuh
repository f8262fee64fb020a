// Shared device helpers for the sm_100a NVFP4 kernels: error plumbing, wide
// global-memory accesses, scalar-format conversions and the 16-element NVFP4
// block quantiser whose rounding rules follow the reference's torch golden
// (tests/python/test_flashinfer_norm_verbatim.py:47-68 and, for the MoE
// activation packer, tests/python/test_flashinfer_b12x_verbatim.py:28-65).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200fp4 {

// ---------------------------------------------------------------------------
// host-side error reporting (defined in capi.cu)
// ---------------------------------------------------------------------------
enum Status : int {
  kOk = 0,
  kInvalidArgument = 1,
  kUnsupported = 2,
  kCudaError = 3,
  kDeviceTimeout = 4,
  kNotInitialised = 5,
};

int fail(int code, const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

#define B200_CUDA(call)                                         \
  do {                                                          \
    int _rc = ::b200fp4::check_cuda((call), #call);             \
    if (_rc) return _rc;                                        \
  } while (0)

// ---------------------------------------------------------------------------
// 32-byte global accesses (one instruction per 16 half-precision elements)
// ---------------------------------------------------------------------------
struct alignas(32) U32x8 {
  uint32_t v[8];
};

// read-only, streamed once: bypass L1 allocation
__device__ __forceinline__ U32x8 ld_stream_32B(const void* p) {
  U32x8 r;
  asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]),
                 "=r"(r.v[6]), "=r"(r.v[7])
               : "l"(p));
  return r;
}

// data that the same kernel writes back later (no .nc)
__device__ __forceinline__ U32x8 ld_32B(const void* p) {
  U32x8 r;
  asm volatile("ld.global.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]),
                 "=r"(r.v[6]), "=r"(r.v[7])
               : "l"(p)
               : "memory");
  return r;
}

__device__ __forceinline__ void st_32B(void* p, const U32x8& r) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(r.v[0]), "r"(r.v[1]),
               "r"(r.v[2]), "r"(r.v[3]), "r"(r.v[4]), "r"(r.v[5]), "r"(r.v[6]), "r"(r.v[7])
               : "memory");
}

// asynchronous L2 prefetch of a contiguous span (address and size multiples of 16 bytes)
__device__ __forceinline__ void prefetch_l2_bulk(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// ---------------------------------------------------------------------------
// 16-bit float pairs <-> f32
// ---------------------------------------------------------------------------
template <typename T>
struct Pair16;

template <>
struct Pair16<__nv_bfloat16> {
  static __device__ __forceinline__ float lo(uint32_t u) { return __uint_as_float(u << 16); }
  static __device__ __forceinline__ float hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
  // two f32 -> packed pair, round-to-nearest-even each
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    return r;
  }
};

template <>
struct Pair16<__half> {
  static __device__ __forceinline__ float lo(uint32_t u) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(u & 0xffffu)));
  }
  static __device__ __forceinline__ float hi(uint32_t u) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(u >> 16)));
  }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    return r;
  }
};

// both halves of a packed 16-bit pair as one f32x2 register pair (defined after f32x2_pack)
template <typename T>
__device__ __forceinline__ uint64_t pair16_to_f32x2(uint32_t u);

// ---------------------------------------------------------------------------
// packed f32x2 arithmetic (sm_100): two IEEE round-to-nearest f32 operations per instruction,
// operands are register pairs viewed as one 64-bit value {lo, hi}
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint64_t f32x2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ float f32x2_lo(uint64_t v) { return __uint_as_float(static_cast<uint32_t>(v)); }
__device__ __forceinline__ float f32x2_hi(uint64_t v) { return __uint_as_float(static_cast<uint32_t>(v >> 32)); }
__device__ __forceinline__ uint64_t f32x2_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f32x2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f32x2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

template <typename T>
__device__ __forceinline__ uint64_t pair16_to_f32x2(uint32_t u) {
  return f32x2_pack(Pair16<T>::lo(u), Pair16<T>::hi(u));
}
// f32x2 -> packed 16-bit pair, round-to-nearest-even each
template <typename T>
__device__ __forceinline__ uint32_t f32x2_to_pair16(uint64_t v) {
  return Pair16<T>::pack(f32x2_lo(v), f32x2_hi(v));
}

// ---------------------------------------------------------------------------
// e4m3 scale factors
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t e4m3_encode_rn(float x) {   // 0 <= x <= 448
  return static_cast<uint32_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ float e4m3_decode(uint32_t bits) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(bits & 0xffu), __NV_E4M3);
  return __half2float(__half(h));
}

// every non-zero code read as 2^(e-7) * (1 + m/8), exponent-0 codes included
__device__ __forceinline__ float e4m3_decode_implicit_one(uint32_t bits) {
  bits &= 0x7fu;
  return bits == 0 ? 0.0f : __uint_as_float((((bits >> 3) + 120u) << 23) | ((bits & 7u) << 20));
}

// ---------------------------------------------------------------------------
// e2m1 codes
// ---------------------------------------------------------------------------
// Exact code of q = t / s (s > 0): nearest grid value; a value half way
// between two grid points takes the smaller magnitude; a result of zero is +0.
// t > c*s  <=>  fl(t/s) > c  for every midpoint c, because c*s is exact in f32.
__device__ __forceinline__ uint32_t e2m1_code_exact(float t, float s) {
  const float mag = fabsf(t);
  uint32_t idx = (mag > 0.25f * s) + (mag > 0.75f * s) + (mag > 1.25f * s) + (mag > 1.75f * s) +
                 (mag > 2.5f * s) + (mag > 3.5f * s) + (mag > 5.0f * s);
  return (t < 0.0f && idx != 0) ? (idx | 8u) : idx;
}

// hardware round-to-nearest-even conversion of eight values; element i lands
// in nibble i (cvt's first source operand goes to the high nibble)
__device__ __forceinline__ uint32_t e2m1x8_hw(const float* u) {
  uint32_t r;
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3};\n"
      "}"
      : "=r"(r)
      : "f"(u[0]), "f"(u[1]), "f"(u[2]), "f"(u[3]), "f"(u[4]), "f"(u[5]), "f"(u[6]), "f"(u[7]));
  return r;
}

// -0 (code 8) -> +0 (code 0) in all eight nibbles
__device__ __forceinline__ uint32_t e2m1x8_drop_negative_zero(uint32_t x) {
  const uint32_t nonzero = ((x & 0x77777777u) + 0x77777777u) & 0x88888888u;
  return x & (0x77777777u | nonzero);
}

// a / 6 rounded to nearest, without the division routine: q = a*c, one exact
// residual and one correction with c = RN(1/6).  Checked against a/6.0f for
// every positive float whose quotient is a normal number; for denormal
// quotients (far below the smallest scale factor) it may be one ulp off,
// which the e4m3 rounding to zero hides.
__device__ __forceinline__ float div_by_6(float a) {
  const float c = 0.16666667163372039794921875f;
  const float q = __fmul_rn(a, c);
  return __fmaf_rn(__fmaf_rn(-6.0f, q, a), c, q);
}

__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// ---------------------------------------------------------------------------
// NVFP4 quantisation of one 16-element block held in registers
//   sf   = min((amax*gs)/6, 448) -> e4m3 (RN-even)
//   code = nearest_e2m1((v*gs) / sf_q), ties to the smaller magnitude
// The codes come from the hardware converter applied to two brackets of the
// quotient, v*k*(1+2^-19) and v*k*(1-2^-19) with k ~ gs/sf_q.  The exact
// quotient lies strictly between them, so when both brackets convert to the
// same eight codes that is the exact answer; the rare group where they differ
// (a value within 2^-18 of a midpoint, exact ties included) is redone with the
// division-free exact comparison above.
// kImplicitOne selects the MoE activation packer, which divides by the
// implicit-one reading of the scale byte instead of its true value.
// ---------------------------------------------------------------------------
// The arithmetic runs on the packed f32x2 instructions of sm_100 (two IEEE round-to-nearest f32
// operations per instruction): a block is eight register pairs.
template <bool kImplicitOne>
__device__ __forceinline__ void quantize_block16(const uint64_t (&v2)[8], float gs, uint32_t& codes_lo,
                                                 uint32_t& codes_hi, uint32_t& sf_bits) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(fmaxf(amax, fabsf(f32x2_lo(v2[i]))), fabsf(f32x2_hi(v2[i])));
  const float sf = fminf(div_by_6(__fmul_rn(amax, gs)), 448.0f);
  sf_bits = e4m3_encode_rn(sf);
  const float div = kImplicitOne ? e4m3_decode_implicit_one(sf_bits) : e4m3_decode(sf_bits);
  // k only has to be within a few ulp of gs/div: the brackets are 2^-19 wide
  const float k = div > 0.0f ? gs * rcp_approx(div) : 0.0f;
  const float k_hi = k * 1.0000019073486328125f;   // 1 + 2^-19
  const float k_lo = k * 0.9999980926513671875f;   // 1 - 2^-19
  const uint64_t k_hi2 = f32x2_pack(k_hi, k_hi);
  const uint64_t k_lo2 = f32x2_pack(k_lo, k_lo);
  uint32_t out[2];
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    float uh[8], ul[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint64_t h = f32x2_mul(v2[4 * g + i], k_hi2);
      const uint64_t l = f32x2_mul(v2[4 * g + i], k_lo2);
      uh[2 * i] = f32x2_lo(h);
      uh[2 * i + 1] = f32x2_hi(h);
      ul[2 * i] = f32x2_lo(l);
      ul[2 * i + 1] = f32x2_hi(l);
    }
    uint32_t ch = e2m1x8_hw(uh);
    const uint32_t cl = e2m1x8_hw(ul);
    if (ch != cl) {
      ch = 0;
      if (div > 0.0f) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ch |= e2m1_code_exact(__fmul_rn(f32x2_lo(v2[4 * g + i]), gs), div) << (8 * i);
          ch |= e2m1_code_exact(__fmul_rn(f32x2_hi(v2[4 * g + i]), gs), div) << (8 * i + 4);
        }
      }
    }
    out[g] = e2m1x8_drop_negative_zero(ch);
  }
  codes_lo = out[0];
  codes_hi = out[1];
}

// the same for sixteen scalars
template <bool kImplicitOne>
__device__ __forceinline__ void quantize_block16(const float (&v)[16], float gs, uint32_t& codes_lo,
                                                 uint32_t& codes_hi, uint32_t& sf_bits) {
  uint64_t v2[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v2[i] = f32x2_pack(v[2 * i], v[2 * i + 1]);
  quantize_block16<kImplicitOne>(v2, gs, codes_lo, codes_hi, sf_bits);
}

// exchange buffers of the ranks of an expert-parallel group, as mapped into this process
constexpr int kMaxPeers = 16;
struct PeerPtrs {
  uint8_t* p[kMaxPeers];
};

// ---------------------------------------------------------------------------
// cross-rank signalling of the expert-parallel kernels
// ---------------------------------------------------------------------------
enum CtrlWord : int {
  kCtrlEpoch = 0,            // completed steps; every kernel of a step signals / waits for epoch + 1
  kCtrlTicketCount = 1,      // CTAs of the count kernel that have finished
  kCtrlTicketPlace = 2,
  kCtrlTicketCombine = 3,
  kCtrlAbort = 4,            // a cross-rank wait expired
  kCtrlTicketGemm = 5,       // CTAs of the row-pushing FC2 that have finished
  kCtrlWords = 16,
};
constexpr int kStatusPeerWaitExpired = 16;
constexpr int kSignalPhases = 3;       // 0: counts published, 1: rows placed, 2: output rows delivered

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// wait until *flag has reached `epoch`; gives up after limit_ns
__device__ __forceinline__ bool wait_flag(const int* flag, int epoch, unsigned long long limit_ns) {
  if (ld_acquire_sys(flag) - epoch >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
    if (ld_acquire_sys(flag) - epoch >= 0) return true;
    if (globaltimer_ns() - t0 > limit_ns) return false;
    __nanosleep(64);
  }
}
// offset of scale factor (row m, K-block kb) in the 128x4 tiled layout with rk
// K-tiles per row tile (python/cutlass_compat/cutlass/utils/blockscaled_layout.py:37-42)
__device__ __host__ __forceinline__ int64_t sf_swizzled_offset(int64_t m, int kb, int rk) {
  return (m & 31) * 16 + ((m >> 5) & 3) * 4 + (kb & 3) + static_cast<int64_t>(kb >> 2) * 512 +
         (m >> 7) * static_cast<int64_t>(rk) * 512;
}

}  // namespace b200fp4
