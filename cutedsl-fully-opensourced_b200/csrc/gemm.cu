// Host side of the NVFP4 GEMM family: tensor-map construction, launch
// configuration and argument checks for the dense block-scaled GEMM and the
// two grouped GEMMs of the fused MoE.  The device code is in gemm_kernel.cuh.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "gemm2cta_kernel.cuh"
#include "gemm_kernel.cuh"

namespace b200fp4 {

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  });
  return fn;
}

// Tensor maps are pure functions of (base pointer, shape, box): encoding one costs a driver call of a few
// microseconds, which is most of the host time of a small GEMM.  They are memoised here and re-encoded only
// when a key has not been seen (the reference re-encodes when an operand's base pointer changes,
// python/self_cutedsl/frontend/jit.py:412-435).
struct MapKey {
  uint64_t kind, base, d0, d1, d2, box;
  bool operator==(const MapKey& o) const { return memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = 0x9e3779b97f4a7c15ull;
    const uint64_t v[6] = {k.kind, k.base, k.d0, k.d1, k.d2, k.box};
    for (uint64_t x : v) h = (h ^ x) * 0x100000001b3ull + (h >> 29);
    return static_cast<size_t>(h);
  }
};
std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;
constexpr size_t kMapCacheLimit = 8192;      // entries; the cache is dropped when it grows beyond this

bool cached_map(const MapKey& key, CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  auto it = g_map_cache.find(key);
  if (it == g_map_cache.end()) return false;
  *out = it->second;
  return true;
}
void remember_map(const MapKey& key, const CUtensorMap& map) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  if (g_map_cache.size() >= kMapCacheLimit) g_map_cache.clear();
  g_map_cache.emplace(key, map);
}

// K-major e2m1 operand viewed as bytes: [groups][rows][k/2], boxes of 128 rows x 128 bytes, 128-byte swizzle.
// (`k` counts e2m1 elements, two per byte; 8-bit operands pass twice their element count)
int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int k, int64_t groups, int box_rows = 128) {
  const MapKey key{1, reinterpret_cast<uint64_t>(base), static_cast<uint64_t>(rows), static_cast<uint64_t>(k),
                   static_cast<uint64_t>(groups), static_cast<uint64_t>(box_rows)};
  if (cached_map(key, map)) return kOk;
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return fail(kCudaError, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(k) / 2;
  cuuint64_t dims[3] = {row_bytes, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(groups)};
  cuuint64_t strides[2] = {row_bytes, row_bytes * static_cast<cuuint64_t>(rows)};
  cuuint32_t box[3] = {128, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t elem[3] = {1, 1, 1};
  const cuuint32_t rank = groups > 0 ? 3 : 2;
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, const_cast<void*>(base), dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(kCudaError, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  remember_map(key, *map);
  return kOk;
}

// Output matrix viewed as bytes: [rows][row_bytes] with `pitch_bytes` between rows; boxes of 32 rows x 128 bytes
// in the 128-byte swizzle (the layout the epilogue warps park their rows in).
int make_output_map(CUtensorMap* map, void* base, int64_t rows, int64_t row_bytes, int64_t pitch_bytes) {
  const MapKey key{2, reinterpret_cast<uint64_t>(base), static_cast<uint64_t>(rows), static_cast<uint64_t>(row_bytes),
                   static_cast<uint64_t>(pitch_bytes), 0};
  if (cached_map(key, map)) return kOk;
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return fail(kCudaError, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_bytes)};
  cuuint32_t box[2] = {128, 32};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(kCudaError, "cuTensorMapEncodeTiled (output) failed with CUresult %d", static_cast<int>(r));
  remember_map(key, *map);
  return kOk;
}

// Tiled scale-factor storage viewed as rows of 256 bytes; a box of 8 rows is the 2 KB slab of one
// 128-row tile and four 64-wide K tiles.  Rows past the end read as zero.
int make_sf_map(CUtensorMap* map, const void* base, int64_t total_bytes) {
  const MapKey key{3, reinterpret_cast<uint64_t>(base), static_cast<uint64_t>(total_bytes), 0, 0, 0};
  if (cached_map(key, map)) return kOk;
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return fail(kCudaError, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {256, static_cast<cuuint64_t>(total_bytes / 256)};
  cuuint64_t strides[1] = {256};
  cuuint32_t box[2] = {256, 8};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(kCudaError, "cuTensorMapEncodeTiled (scale factors) failed with CUresult %d", static_cast<int>(r));
  remember_map(key, *map);
  return kOk;
}

// Row-major scale factors of A: [rows][k / 16] bytes, `pitch` bytes between rows; boxes of 128 rows x 16 bytes (the
// scale bytes of one 256-wide K step).  Columns beyond k / 16 read as zero.
int make_sfa_rows_map(CUtensorMap* map, const void* base, int64_t rows, int k, int64_t pitch) {
  const MapKey key{4, reinterpret_cast<uint64_t>(base), static_cast<uint64_t>(rows), static_cast<uint64_t>(k),
                   static_cast<uint64_t>(pitch), 0};
  if (cached_map(key, map)) return kOk;
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return fail(kCudaError, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(k / 16), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch)};
  cuuint32_t box[2] = {16, 128};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(kCudaError, "cuTensorMapEncodeTiled (scale rows) failed with CUresult %d", static_cast<int>(r));
  remember_map(key, *map);
  return kOk;
}

std::mutex g_status_mutex;
int* g_status_word[64] = {};

}  // namespace

constexpr int kMaxDevices = 64;

int current_device_ordinal() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dev >= 0 && dev < kMaxDevices ? dev : 0;
}

// cached per device ordinal (attribute queries cost a driver call each)
int sm_count_of_current_device() {
  static std::atomic<int> cached[kMaxDevices];
  const int dev = current_device_ordinal();
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// The opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of a kernel: remember per
// device ordinal (and per kernel instantiation: one flag array per call site) that it has been set.
template <typename Kernel>
int configure_smem_once(std::atomic<bool>* done, Kernel kern, int bytes) {
  const int dev = current_device_ordinal();
  if (!done[dev].load(std::memory_order_acquire)) {
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    done[dev].store(true, std::memory_order_release);
  }
  return kOk;
}

// One int per device that kernels OR failure bits into (bounded waits that expired).
int device_status_word(int** out) {
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(kUnsupported, "device ordinal %d", dev);
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (g_status_word[dev] == nullptr) {
    B200_CUDA(cudaMalloc(&g_status_word[dev], sizeof(int)));
    B200_CUDA(cudaMemset(g_status_word[dev], 0, sizeof(int)));
  }
  *out = g_status_word[dev];
  return kOk;
}

// Self-test of the bounded wait: a CTA initialises an mbarrier on which nothing ever arrives and waits for it with
// the GEMM kernels' own wait routine and a short cycle limit.  The wait gives up, the abort flag goes up, the
// kernel ORs kStatusTimeoutMma into the status word and returns; no operand, no copy and no tensor memory is
// involved, so nothing is left in flight.
__global__ void bounded_wait_selftest_kernel(int* status, long long limit_cycles, int* gave_up) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    abort_flag = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();
  const bool ok = wait_bounded(ptx::smem_u32(&bar), 0u, &abort_flag, limit_cycles);
  if (!ok && threadIdx.x == 0) {
    atomicOr(status, kStatusTimeoutMma);
    *gave_up = abort_flag;
  }
}

int bounded_wait_selftest(long long limit_cycles, int* gave_up_dev, cudaStream_t stream) {
  if (gave_up_dev == nullptr) return fail(kInvalidArgument, "gave_up is null");
  if (limit_cycles < 1 || limit_cycles > 2000000000LL)
    return fail(kInvalidArgument, "limit_cycles must be in [1, 2e9]");
  int* status = nullptr;
  int rc = device_status_word(&status);
  if (rc) return rc;
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(status, limit_cycles, gave_up_dev);
  return check_cuda(cudaGetLastError(), "bounded_wait_selftest_kernel launch");
}

// tc: tensor map of the output for the variants whose tiles leave through TMA stores (others never touch it)
template <int kBlockN, bool kSwigluB, int kARows = 128, int kEpi = 0, typename Epilogue>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                const Epilogue& epi, int max_tiles, cudaStream_t stream) {
  auto kern = nvfp4_gemm_kernel<kBlockN, kSwigluB, Epilogue, kARows, kEpi>;
  constexpr SmemLayout L = smem_layout<kBlockN, kSwigluB, Epilogue::kOutBytes, kARows, Epilogue::kParkWide>();
  static std::atomic<bool> configured[kMaxDevices];      // per instantiation and device
  int rc_cfg = configure_smem_once(configured, kern, static_cast<int>(L.total));
  if (rc_cfg) return rc_cfg;
  int grid = sm_count_of_current_device();
  if (grid > max_tiles) grid = max_tiles;
  if (grid < 1) return kOk;
  kern<<<grid, gemm_threads(kBlockN, kSwigluB, kEpi), L.total, stream>>>(ta, tb, tc, p, epi);
  return check_cuda(cudaGetLastError(), "nvfp4_gemm_kernel launch");
}

// CTA-pair variant: 256 x 256 tiles on 2-CTA clusters
template <typename OutT>
int gemm_dense_pair(const void* a, const void* b, const void* sfa, const void* sfb, void* c, const float* alpha, int m,
                    int n, int k, cudaStream_t stream) {
  CUtensorMap ta, tb, tsa, tsb;
  int rc = make_operand_map(&ta, a, m, k, 0);
  if (rc) return rc;
  rc = make_operand_map(&tb, b, n, k, 1);
  if (rc) return rc;
  const int64_t rk = (k + 63) / 64;
  rc = make_sf_map(&tsa, sfa, static_cast<int64_t>((m + 127) / 128) * rk * 512);
  if (rc) return rc;
  rc = make_sf_map(&tsb, sfb, static_cast<int64_t>((n + 127) / 128) * rk * 512);
  if (rc) return rc;
  GemmParams p{};
  p.m_rows = m;
  p.n_cols = n;
  p.k = k;
  p.k_bytes = k / 2;
  p.rk = static_cast<int>(rk);
  p.num_k_tiles = (k + kBlockK - 1) / kBlockK;
  p.num_m_blocks = (m + 255) / 256;
  p.num_n_blocks = (n + 255) / 256;
  rc = device_status_word(&p.status);
  if (rc) return rc;
  EpilogueStore<OutT> epi{static_cast<OutT*>(c), n, alpha, 0};
  auto kern = nvfp4_gemm_pair_kernel<EpilogueStore<OutT>>;
  static std::atomic<bool> configured[kMaxDevices];
  rc = configure_smem_once(configured, kern, static_cast<int>(kPairSmemBytes));
  if (rc) return rc;
  int pairs = sm_count_of_current_device() / 2;
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  if (pairs > tiles) pairs = tiles;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kPairThreads, 1, 1);
  cfg.dynamicSmemBytes = kPairSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return check_cuda(cudaLaunchKernelEx(&cfg, kern, ta, tb, tsa, tsb, p, epi), "nvfp4_gemm_pair_kernel launch");
}

// ---------------------------------------------------------------------------
// split-K: few output tiles against a long weight stream (M = 128, N = K = 8192: 32 tiles of 128 x 256 for 148 SMs).
// The K tiles of every output tile are dealt to `splits` work items that run on different CTAs at the same time and
// write f32 partial matrices into a caller-provided workspace; this kernel sums them (slice order, so the result
// does not depend on timing), applies alpha and rounds once.
// ---------------------------------------------------------------------------
template <typename OutT>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, int64_t stride,
                                     const float* __restrict__ alpha, OutT* __restrict__ c, int64_t n4) {
  const float scale = alpha == nullptr ? 1.0f : __ldg(alpha);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float4 acc = *reinterpret_cast<const float4*>(partial + 4 * i);
    for (int s = 1; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(partial + s * stride + 4 * i);
      acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
    }
    acc.x *= scale, acc.y *= scale, acc.z *= scale, acc.w *= scale;
    if constexpr (sizeof(OutT) == 4) {
      *reinterpret_cast<float4*>(c + 4 * i) = acc;
    } else {
      uint2 packed;
      packed.x = Pair16<OutT>::pack(acc.x, acc.y);
      packed.y = Pair16<OutT>::pack(acc.z, acc.w);
      *reinterpret_cast<uint2*>(c + 4 * i) = packed;
    }
  }
}

// number of K slices for an m x n x k problem on 128 x 256 tiles (1 = no split)
int splitk_slices(int m, int n, int k) {
  const int sms = sm_count_of_current_device();
  const int64_t tiles = static_cast<int64_t>((m + 127) / 128) * ((n + 255) / 256);
  const int k_tiles = (k + kBlockK - 1) / kBlockK;
  if (n % 4 != 0 || tiles * 2 > sms || k_tiles < 8) return 1;
  int splits = static_cast<int>(std::min<int64_t>(sms / tiles, 8));
  splits = std::min(splits, k_tiles / 4);                         // at least four K steps per slice
  while (splits > 1 && (splits - 1) * ((k_tiles + splits - 1) / splits) >= k_tiles) --splits;   // no empty slice
  return std::max(splits, 1);
}

size_t gemm_workspace_bytes(int m, int n, int k) {
  const int splits = splitk_slices(m, n, k);
  return splits > 1 ? static_cast<size_t>(splits) * m * n * sizeof(float) : 0;
}

template <typename OutT>
int gemm_dense_splitk(const void* a, const void* b, const void* sfa, const void* sfb, void* c, const float* alpha, int m,
                      int n, int k, int splits, float* workspace, cudaStream_t stream) {
  CUtensorMap ta, tb;
  int rc = make_operand_map(&ta, a, m, k, 0);
  if (rc) return rc;
  rc = make_operand_map(&tb, b, n, k, 1);
  if (rc) return rc;
  GemmParams p{};
  p.sfa = static_cast<const uint8_t*>(sfa);
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.m_rows = m;
  p.n_cols = n;
  p.k = k;
  p.k_bytes = k / 2;
  p.rk = (k + 63) / 64;
  p.num_k_tiles = (k + kBlockK - 1) / kBlockK;
  p.b_row_tiles = (n + 127) / 128;
  p.num_m_blocks = (m + kBlockM - 1) / kBlockM;
  p.num_n_blocks = (n + 255) / 256;
  p.k_splits = splits;
  rc = device_status_word(&p.status);
  if (rc) return rc;
  EpilogueStore<float> epi{workspace, n, nullptr, 0, static_cast<int64_t>(m) * n};
  rc = launch_gemm<256, false>(ta, tb, CUtensorMap{}, p, epi, p.num_m_blocks * p.num_n_blocks * splits, stream);
  if (rc) return rc;
  const int64_t n4 = static_cast<int64_t>(m) * n / 4;
  const int grid = static_cast<int>(std::min<int64_t>((n4 + 255) / 256, 4 * sm_count_of_current_device()));
  splitk_reduce_kernel<OutT><<<grid, 256, 0, stream>>>(workspace, splits, static_cast<int64_t>(m) * n, alpha,
                                                        static_cast<OutT*>(c), n4);
  return check_cuda(cudaGetLastError(), "splitk_reduce_kernel launch");
}

// ---------------------------------------------------------------------------
// dense GEMM: C[l][m][n] = alpha * A[l][m][k] . B[l][n][k]^T
// ---------------------------------------------------------------------------
template <typename OutT>
int gemm_dense_typed(const void* a, const void* b, const void* sfa, const void* sfb, void* c, const float* alpha, int m,
                     int n, int k, int tile_n, int sf_vec, int fmt8, cudaStream_t stream) {
  // fmt8 < 0: e2m1 operands; else MXFP8 with operand formats a = fmt8 & 1, b = fmt8 >> 1 (0 e4m3, 1 e5m2)
  if (tile_n == 512) return gemm_dense_pair<OutT>(a, b, sfa, sfb, c, alpha, m, n, k, stream);
  CUtensorMap ta, tb;
  const int k_nibbles = fmt8 >= 0 ? 2 * k : k;           // operand maps count 4-bit units
  int rc = make_operand_map(&ta, a, m, k_nibbles, 0);
  if (rc) return rc;
  rc = make_operand_map(&tb, b, n, k_nibbles, 1, tile_n == 64 ? 64 : 128);
  if (rc) return rc;
  GemmParams p{};
  p.sfa = static_cast<const uint8_t*>(sfa);
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.m_rows = m;
  p.n_cols = n;
  p.k = k;
  p.k_bytes = fmt8 >= 0 ? k : k / 2;
  p.sf_block32 = fmt8 >= 0 ? 2 : (sf_vec == 32 ? 1 : 0);
  p.a_fmt8 = fmt8 >= 0 ? (fmt8 & 1) : 0;
  p.b_fmt8 = fmt8 >= 0 ? (fmt8 >> 1) : 0;
  p.rk = sf_vec == 32 ? (k + 127) / 128 : (k + 63) / 64;
  p.num_k_tiles = (p.k_bytes + 127) / 128;
  p.b_row_tiles = (n + 127) / 128;
  p.num_m_blocks = (m + kBlockM - 1) / kBlockM;
  rc = device_status_word(&p.status);
  if (rc) return rc;
  EpilogueStore<OutT> epi{static_cast<OutT*>(c), n, alpha, 0};
  CUtensorMap tc{};
  if (tile_n == 128) {
    rc = make_output_map(&tc, c, m, static_cast<int64_t>(n) * sizeof(OutT), static_cast<int64_t>(n) * sizeof(OutT));
    if (rc) return rc;
  }
  // few waves of tiles: walk row blocks first (measured 3-4 % faster at 4096^3 and M = 1024, 2 % slower at 8192^3)
  p.row_block_major = static_cast<int64_t>(p.num_m_blocks) * ((n + tile_n - 1) / tile_n) <= 8 * sm_count_of_current_device();
  if (tile_n == 256) {
    p.num_n_blocks = (n + 255) / 256;
    return launch_gemm<256, false>(ta, tb, tc, p, epi, p.num_m_blocks * p.num_n_blocks, stream);
  }
  if (tile_n == 64) {
    p.num_n_blocks = (n + 63) / 64;
    return launch_gemm<64, false>(ta, tb, tc, p, epi, p.num_m_blocks * p.num_n_blocks, stream);
  }
  p.num_n_blocks = (n + 127) / 128;
  return launch_gemm<128, false>(ta, tb, tc, p, epi, p.num_m_blocks * p.num_n_blocks, stream);
}

// workspace: optional f32 scratch of gemm_workspace_bytes(m, n, k) bytes; with it, problems with few output tiles
// and a long reduction run split-K (tile_n 0 only).  Without it they run unsplit.
// sf_vec: 16 = NVFP4 (e4m3 scale per 16 elements), 32 = MXFP4 (ue8m0 scale per 32 elements; single-CTA tiles only)
int gemm_dense(const void* a, const void* b, const void* sfa, const void* sfb, void* c, const float* alpha, int m, int n,
               int k, int l, int c_dtype, int tile_n, void* workspace, size_t workspace_bytes, int sf_vec, int fmt8,
               cudaStream_t stream) {
  if (sf_vec != 16 && sf_vec != 32) return fail(kUnsupported, "sf_vec=%d (16 = NVFP4, 32 = MXFP4 / MXFP8)", sf_vec);
  if (fmt8 >= 0 && (sf_vec != 32 || fmt8 > 3)) return fail(kUnsupported, "8-bit operands take ue8m0 scales per 32 elements");
  if (sf_vec == 32 && tile_n == 512) return fail(kUnsupported, "the MX flavours run on single-CTA tiles (tile_n 0, 64, 128, 256)");
  if (sf_vec == 32) workspace = nullptr;
  if (a == nullptr || b == nullptr || sfa == nullptr || sfb == nullptr || c == nullptr)
    return fail(kInvalidArgument, "null pointer argument");
  if (m <= 0 || n <= 0 || k <= 0 || l <= 0) return fail(kInvalidArgument, "m, n, k, l must be positive");
  // contiguous dimension of every tensor must cover whole 16-byte units (the reference's
  // is_valid_tensor_alignment rule): 32 e2m1 elements for A/B, 8 (16-bit) or 4 (f32) for C
  if (k % (fmt8 >= 0 ? 16 : 32) != 0)
    return fail(kInvalidArgument, "Invalid tensor alignment: k=%d is not a multiple of %d", k, fmt8 >= 0 ? 16 : 32);
  if (n % 8 != 0) return fail(kInvalidArgument, "Invalid tensor alignment: n=%d is not a multiple of 8", n);
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(sfa) |
       reinterpret_cast<uintptr_t>(sfb) | reinterpret_cast<uintptr_t>(c)) & 15)
    return fail(kInvalidArgument, "Invalid tensor alignment: pointers must be 16-byte aligned");
  if (c_dtype < 0 || c_dtype > 2) return fail(kUnsupported, "c_dtype code %d (0 fp16, 1 bf16, 2 f32)", c_dtype);
  if (tile_n != 0 && tile_n != 64 && tile_n != 128 && tile_n != 256 && tile_n != 512)
    return fail(kInvalidArgument, "tile_n must be 0, 64, 128, 256 or 512 (512 = 256 x 256 tiles on CTA pairs)");
  int splits = 1;
  if (tile_n == 0 && workspace != nullptr) {
    splits = splitk_slices(m, n, k);
    if (splits > 1 && (workspace_bytes < static_cast<size_t>(splits) * m * n * sizeof(float) ||
                       (reinterpret_cast<uintptr_t>(workspace) & 15)))
      return fail(kInvalidArgument, "split-K workspace must hold %zu bytes, 16-byte aligned",
                  static_cast<size_t>(splits) * m * n * sizeof(float));
  }
  if (tile_n == 0) {
    // wide tiles halve the operand traffic per flop; keep narrow ones while they are needed to fill the SMs
    const int sms = sm_count_of_current_device();
    const int64_t m_blocks = (m + 127) / 128;
    static const bool no_pairs = getenv("B200FP4_NO_PAIRS") != nullptr;
    // a full wave of 256 x 256 tiles on CTA pairs: each CTA fills 38 KB per K step instead of 54 KB
    if (!no_pairs && sf_vec == 16 && fmt8 < 0 && ((m + 255) / 256) * static_cast<int64_t>((n + 255) / 256) >= sms / 2 && k >= 1024) tile_n = 512;
    else if (m_blocks * ((n + 255) / 256) >= sms) tile_n = 256;
    else if (m_blocks * ((n + 127) / 128) >= sms) tile_n = 128;
    else tile_n = 64;            // few rows (weight streaming): narrow tiles put more SMs on the stream of B
  }
  const int64_t m_tiles = (m + 127) / 128, n_tiles = (n + 127) / 128, rk = sf_vec == 32 ? (k + 127) / 128 : (k + 63) / 64;
  const size_t c_elem = c_dtype == 2 ? 4 : 2;
  for (int i = 0; i < l; ++i) {
    const int64_t row_bytes = fmt8 >= 0 ? k : k / 2;
    const uint8_t* ai = static_cast<const uint8_t*>(a) + static_cast<int64_t>(i) * m * row_bytes;
    const uint8_t* bi = static_cast<const uint8_t*>(b) + static_cast<int64_t>(i) * n * row_bytes;
    const uint8_t* sfai = static_cast<const uint8_t*>(sfa) + i * m_tiles * rk * 512;
    const uint8_t* sfbi = static_cast<const uint8_t*>(sfb) + i * n_tiles * rk * 512;
    uint8_t* ci = static_cast<uint8_t*>(c) + static_cast<int64_t>(i) * m * n * c_elem;
    int rc;
    if (splits > 1) {
      float* ws = static_cast<float*>(workspace);
      if (c_dtype == 0) rc = gemm_dense_splitk<__half>(ai, bi, sfai, sfbi, ci, alpha, m, n, k, splits, ws, stream);
      else if (c_dtype == 1) rc = gemm_dense_splitk<__nv_bfloat16>(ai, bi, sfai, sfbi, ci, alpha, m, n, k, splits, ws, stream);
      else rc = gemm_dense_splitk<float>(ai, bi, sfai, sfbi, ci, alpha, m, n, k, splits, ws, stream);
      if (rc) return rc;
      continue;
    }
    if (c_dtype == 0) rc = gemm_dense_typed<__half>(ai, bi, sfai, sfbi, ci, alpha, m, n, k, tile_n, sf_vec, fmt8, stream);
    else if (c_dtype == 1) rc = gemm_dense_typed<__nv_bfloat16>(ai, bi, sfai, sfbi, ci, alpha, m, n, k, tile_n, sf_vec, fmt8, stream);
    else rc = gemm_dense_typed<float>(ai, bi, sfai, sfbi, ci, alpha, m, n, k, tile_n, sf_vec, fmt8, stream);
    if (rc) return rc;
  }
  return kOk;
}

// ---------------------------------------------------------------------------
// grouped GEMMs of the MoE (rows are expert-major, every 128-row block belongs to one expert)
// ---------------------------------------------------------------------------
// FC1: act = quant(bf16(silu(gate) * up)) with [up | gate] = Xq . W1[e]^T * w1_alpha[e]
int gemm_moe_fc1(const void* xq, const void* xq_sf, const void* w1, const void* w1_sf, void* act_codes, void* act_sf,
                 const float* w1_alpha, const float* fc2_input_scale, const int* num_m_blocks_dev,
                 const int* m_block_expert, const int* m_block_rows, int max_m_blocks, int hidden, int inter,
                 int experts, int few_rows, int* status, cudaStream_t stream, const PeerSync* peer,
                 int sfa_row_pitch) {
  // sfa_row_pitch: 0 = xq_sf holds 128x4 tiles; else plain rows of scale bytes with that pitch
  // few_rows: no row block holds more than 32 rows (the caller knows: at most 32 tokens) -> stages of 32 rows of A
  // Tile width: [up 128 | gate 128] tiles by default.  They have one accumulator, but the epilogue hands it back
  // as soon as it has read its columns (before the SwiGLU arithmetic), and they need half the MMA instructions
  // and 30 % fewer operand bytes per flop than [up 64 | gate 64] tiles with two accumulators (prefill step 256 us
  // with the narrow tiles, 233 with the wide ones).  B200FP4_FC1_TILE=128 selects the narrow variant.
  static const int forced_tile = [] {
    const char* e = getenv("B200FP4_FC1_TILE");
    return e != nullptr ? atoi(e) : 0;
  }();
  const bool narrow = forced_tile == 128;
  CUtensorMap ta, tb;
  const bool small_a = few_rows != 0 && !narrow;
  int rc = make_operand_map(&ta, xq, static_cast<int64_t>(max_m_blocks) * 128, hidden, 0, small_a ? 32 : 128);
  if (rc) return rc;
  rc = make_operand_map(&tb, w1, 2 * inter, hidden, experts, narrow ? 64 : 128);
  if (rc) return rc;
  GemmParams p{};
  p.sfa = static_cast<const uint8_t*>(xq_sf);
  p.sfb = static_cast<const uint8_t*>(w1_sf);
  p.m_rows = max_m_blocks * 128;
  p.n_cols = inter;
  p.k = hidden;
  p.k_bytes = hidden / 2;
  p.rk = (hidden + 63) / 64;
  p.num_k_tiles = (hidden + kBlockK - 1) / kBlockK;
  p.num_n_blocks = inter / 128;
  p.b_row_tiles = (2 * inter) / 128;
  p.gate_row_offset = inter;
  p.num_m_blocks_dev = num_m_blocks_dev;
  p.num_m_blocks = max_m_blocks;
  p.m_block_group = m_block_expert;
  p.num_groups = experts;
  p.m_block_rows = m_block_rows;
  p.status = status;
  p.row_block_major = 1;
  if (peer != nullptr) p.peer = *peer;
  CUtensorMap tsfa{};
  if (sfa_row_pitch != 0) {
    rc = make_sfa_rows_map(&tsfa, xq_sf, static_cast<int64_t>(max_m_blocks) * 128, hidden, sfa_row_pitch);
    if (rc) return rc;
    p.sfa_row_major = 1;
  }
  EpilogueSwiglu epi{static_cast<uint8_t*>(act_codes), static_cast<uint8_t*>(act_sf), w1_alpha, fc2_input_scale, inter};
  if (narrow) {
    p.num_n_blocks = inter / 64;
    return launch_gemm<128, true>(ta, tb, tsfa, p, epi, max_m_blocks * p.num_n_blocks, stream);
  }
  if (small_a) return launch_gemm<256, true, 32>(ta, tb, tsfa, p, epi, max_m_blocks * p.num_n_blocks, stream);
  // Sixteen epilogue warps: each reads its 32 up and 32 gate columns in one go and hands the (single) accumulator
  // back before any SwiGLU arithmetic, so the next tile's MMAs wait for a tensor-memory read only; with eight
  // warps half of the arithmetic ran before the release (FC1 of the prefill shape: 104 us with eight, 91 with
  // sixteen).  B200FP4_FC1_EPI=8 selects the eight-warp variant.
  static const bool epi8 = [] {
    const char* e = getenv("B200FP4_FC1_EPI");
    return e != nullptr && atoi(e) == 8;
  }();
  if (epi8) return launch_gemm<256, true>(ta, tb, tsfa, p, epi, max_m_blocks * p.num_n_blocks, stream);
  return launch_gemm<256, true, 128, 16>(ta, tb, tsfa, p, epi, max_m_blocks * p.num_n_blocks, stream);
}

// Epilogue warps of the 128-wide FC2 tiles (short reductions: three K steps per tile at the prefill shape, so the
// tile rate is set by how fast accumulators are drained).  B200FP4_FC2_EPI=4|8 overrides the default.
int fc2_epilogue_warps() {
  static const int n = [] {
    const char* e = getenv("B200FP4_FC2_EPI");
    const int v = e != nullptr ? atoi(e) : 0;
    return v == 4 || v == 8 ? v : 4;
  }();
  return n;
}

// B200FP4_FC2_WIDE=1 takes the 256-wide single-accumulator tiles for FC2 whatever the reduction length (experiment)
bool fc2_force_wide() {
  static const bool v = [] {
    const char* e = getenv("B200FP4_FC2_WIDE");
    return e != nullptr && atoi(e) != 0;
  }();
  return v;
}

// FC2: partial[row][h] = (Actq . W2[e]^T) * w2_alpha[e], stored as f32 or (rows_bf16) rounded to bf16.
// The kernel is sensitive to how its rows leave (an SM writes some 12-16 bytes per cycle when every lane stores to
// another row), so the 16-bit rows nearly halve its time and the combine's, and they leave through TMA stores.
template <typename RowT>
int gemm_moe_fc2_typed(const void* act_codes, const void* act_sf, const void* w2, const void* w2_sf, RowT* partial,
                       const float* w2_alpha, const int* num_m_blocks_dev, const int* m_block_expert,
                       const int* m_block_rows, int max_m_blocks, int hidden, int inter, int experts, int few_rows,
                       int* status, cudaStream_t stream) {
  CUtensorMap ta, tb;
  // Short reductions with 16-bit rows: 256-wide tiles whose rows leave through TMA stores (EpilogueStoreWide, three
  // stages).  FC2 of the prefill shape: 128-wide tiles with TMA stores 67 us, 256-wide with register stores 64,
  // 256-wide with TMA stores 53.  B200FP4_FC2_PARK=0 keeps the 128-wide tiles.
  static const bool park_allowed = [] {
    const char* e = getenv("B200FP4_FC2_PARK");
    return e == nullptr || atoi(e) != 0;
  }();
  const int k_tiles = (inter + kBlockK - 1) / kBlockK;
  const bool park = sizeof(RowT) == 2 && hidden % 256 == 0 && few_rows == 0 && k_tiles <= 4 && park_allowed;
  const bool wide = hidden % 256 == 0 && (k_tiles > 4 || fc2_force_wide() || park);
  const bool small_a = few_rows != 0 && wide;
  int rc = make_operand_map(&ta, act_codes, static_cast<int64_t>(max_m_blocks) * 128, inter, 0, small_a ? 32 : 128);
  if (rc) return rc;
  rc = make_operand_map(&tb, w2, hidden, inter, experts);
  if (rc) return rc;
  GemmParams p{};
  p.sfa = static_cast<const uint8_t*>(act_sf);
  p.sfb = static_cast<const uint8_t*>(w2_sf);
  p.m_rows = max_m_blocks * 128;
  p.n_cols = hidden;
  p.k = inter;
  p.k_bytes = inter / 2;
  p.rk = (inter + 63) / 64;
  p.num_k_tiles = (inter + kBlockK - 1) / kBlockK;
  p.b_row_tiles = (hidden + 127) / 128;
  p.num_m_blocks_dev = num_m_blocks_dev;
  p.num_m_blocks = max_m_blocks;
  p.m_block_group = m_block_expert;
  p.num_groups = experts;
  p.m_block_rows = m_block_rows;
  p.status = status;
  p.row_block_major = 1;
  EpilogueStore<RowT> epi{partial, hidden, w2_alpha, 1};
  CUtensorMap tc{};
  rc = make_output_map(&tc, partial, static_cast<int64_t>(max_m_blocks) * 128, static_cast<int64_t>(hidden) * sizeof(RowT),
                       static_cast<int64_t>(hidden) * sizeof(RowT));
  if (rc) return rc;
  // Short reductions (few K tiles) spend more time draining the accumulator than filling it; the
  // 128-wide tile has two accumulators, so its epilogue overlaps the next tile's MMAs.
  if (wide) {
    p.num_n_blocks = hidden / 256;
    if (small_a) return launch_gemm<256, false, 32>(ta, tb, tc, p, epi, max_m_blocks * p.num_n_blocks, stream);
    if constexpr (sizeof(RowT) == 2) {
      if (park) {
        EpilogueStoreWide wepi{w2_alpha};
        return launch_gemm<256, false>(ta, tb, tc, p, wepi, max_m_blocks * p.num_n_blocks, stream);
      }
    }
    return launch_gemm<256, false>(ta, tb, tc, p, epi, max_m_blocks * p.num_n_blocks, stream);
  }
  p.num_n_blocks = (hidden + 127) / 128;
  return launch_gemm<128, false>(ta, tb, tc, p, epi, max_m_blocks * p.num_n_blocks, stream);
}

// FC2 of the expert-parallel MoE: as gemm_moe_fc2 with bf16 rows, but every row is stored into the landing zone
// of the rank that owns its token (EpiloguePushRows) instead of a local buffer.
int gemm_moe_fc2_push(const void* act_codes, const void* act_sf, const void* w2, const void* w2_sf,
                      const int* row_tag, const PeerPtrs& peers, size_t recv_off, const int* abort_flag,
                      const float* w2_alpha, const int* num_m_blocks_dev, const int* m_block_expert,
                      const int* m_block_rows, int max_m_blocks, int hidden, int inter, int experts, int few_rows,
                      int* status, cudaStream_t stream, const PeerSync* peer) {
  CUtensorMap ta, tb;
  const bool wide = hidden % 256 == 0 && (inter + kBlockK - 1) / kBlockK > 4;
  const bool small_a = few_rows != 0 && wide;
  int rc = make_operand_map(&ta, act_codes, static_cast<int64_t>(max_m_blocks) * 128, inter, 0, small_a ? 32 : 128);
  if (rc) return rc;
  rc = make_operand_map(&tb, w2, hidden, inter, experts);
  if (rc) return rc;
  GemmParams p{};
  if (peer != nullptr) p.peer = *peer;
  p.sfa = static_cast<const uint8_t*>(act_sf);
  p.sfb = static_cast<const uint8_t*>(w2_sf);
  p.m_rows = max_m_blocks * 128;
  p.n_cols = hidden;
  p.k = inter;
  p.k_bytes = inter / 2;
  p.rk = (inter + 63) / 64;
  p.num_k_tiles = (inter + kBlockK - 1) / kBlockK;
  p.b_row_tiles = (hidden + 127) / 128;
  p.num_m_blocks_dev = num_m_blocks_dev;
  p.num_m_blocks = max_m_blocks;
  p.m_block_group = m_block_expert;
  p.num_groups = experts;
  p.m_block_rows = m_block_rows;
  p.status = status;
  p.row_block_major = 1;
  EpiloguePushRows epi{row_tag, peers, recv_off, hidden, w2_alpha, abort_flag};
  if (wide) {
    p.num_n_blocks = hidden / 256;
    if (small_a) return launch_gemm<256, false, 32>(ta, tb, CUtensorMap{}, p, epi, max_m_blocks * p.num_n_blocks, stream);
    return launch_gemm<256, false>(ta, tb, CUtensorMap{}, p, epi, max_m_blocks * p.num_n_blocks, stream);
  }
  p.num_n_blocks = (hidden + 127) / 128;
  if (fc2_epilogue_warps() == 8)
    return launch_gemm<128, false, 128, 8>(ta, tb, CUtensorMap{}, p, epi, max_m_blocks * p.num_n_blocks, stream);
  return launch_gemm<128, false>(ta, tb, CUtensorMap{}, p, epi, max_m_blocks * p.num_n_blocks, stream);
}

int gemm_moe_fc2(const void* act_codes, const void* act_sf, const void* w2, const void* w2_sf, void* partial,
                 int rows_bf16, const float* w2_alpha, const int* num_m_blocks_dev, const int* m_block_expert,
                 const int* m_block_rows, int max_m_blocks, int hidden, int inter, int experts, int few_rows,
                 int* status, cudaStream_t stream) {
  if (rows_bf16)
    return gemm_moe_fc2_typed(act_codes, act_sf, w2, w2_sf, static_cast<__nv_bfloat16*>(partial), w2_alpha,
                              num_m_blocks_dev, m_block_expert, m_block_rows, max_m_blocks, hidden, inter, experts,
                              few_rows, status, stream);
  return gemm_moe_fc2_typed(act_codes, act_sf, w2, w2_sf, static_cast<float*>(partial), w2_alpha, num_m_blocks_dev,
                            m_block_expert, m_block_rows, max_m_blocks, hidden, inter, experts, few_rows, status,
                            stream);
}

}  // namespace b200fp4

