// NVFP4 block-scaled GEMM mainloop for sm_100a, shared by the dense GEMM and
// the two grouped MoE GEMMs.
//
//   C[m, n] = sum_k (A[m,k] * SFA[m,k/16]) * (B[n,k] * SFB[n,k/16])
//
// A and B are e2m1, two per byte, K-major; SFA / SFB are e4m3 bytes in the
// 128x4 tiled layout.  The reference computes this with warp-level mma.sync on
// sm_120 (third_party/cutlass/examples/python/CuTeDSL/cute/blackwell_geforce/
// kernel/blockscaled_gemm/dense_blockscaled_gemm_persistent_cooperative.py:443-1185);
// here one CTA per SM runs a warp-specialised persistent loop:
//
//   warp 0  TMA producer: per 256-wide K tile, one tiled copy of A (128 rows x
//           128 bytes, 128-byte swizzle), one per 128-row piece of B, and plain
//           bulk copies of the scale-factor slabs (2 KB per 128 rows: four
//           512-byte 128x4 tiles are contiguous in the tiled layout)
//   warp 1  MMA issuer: per stage four tcgen05.mma kind::mxf4nvf4 (K = 64 each) accumulate into a TMEM
//           accumulator; tcgen05.commit releases the stage.  The whole warp walks the loop and an elected lane
//           issues, so that the operands stay in warp-wide registers (see the role below)
//   last 4 warps  scale-slab movers: shared memory -> registers -> tensor memory (tcgen05.st),
//           one set of slab columns per stage.  tcgen05.cp would do the same copy, but it runs
//           in the MMA pipe: twelve copies per stage cost a third of the kernel's time there
//   warps 2..  epilogue (4 warps for 128-wide tiles, 8 for 256-wide ones): tcgen05.ld the
//           accumulator (each warp its own 32-lane quarter; with 8 warps two warps share a
//           quarter and split the columns), apply the epilogue functor, store
//
// No cluster launch and no multicast anywhere.  Every wait is bounded: on
// expiry the kernel raises a flag in the status word and all roles leave.
#pragma once

#ifdef B200FP4_ACCT
#include <cstdio>
#endif
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace b200fp4 {

constexpr int kBlockM = 128;
constexpr int kBlockK = 256;                 // e2m1 elements per stage = 128 bytes per row
// two single-thread roles (TMA, MMA) + the epilogue warps: four for 128-wide tiles (the second
// accumulator hides the epilogue), eight for 256-wide tiles (one accumulator: drain it twice as fast)
// (the SwiGLU epilogue is arithmetic-heavy: eight warps at either width, sixteen on request)
__host__ __device__ constexpr int epilogue_warps(int block_n, bool swiglu = false, int forced = 0) {
  return forced != 0 ? forced : ((block_n == 256 || swiglu) ? 8 : 4);
}
// ... + four warps (one per 32-lane quarter of tensor memory) that move the scale slabs of every K
// tile from shared memory into tensor memory
__host__ __device__ constexpr int gemm_threads(int block_n, bool swiglu = false, int forced_epi_warps = 0) {
  return 64 + 32 * epilogue_warps(block_n, swiglu, forced_epi_warps) + 128;
}
constexpr uint32_t kTmemCols = 512;
constexpr long long kWaitLimitCycles = 4000000000LL;   // ~2 s at 2 GHz

enum GemmStatusBits : int {
  kStatusTimeoutProducer = 1,
  kStatusTimeoutMma = 2,
  kStatusTimeoutEpilogue = 4,
  kStatusRowsExceedTile = 8,    // a few-row launch met a row block with more rows than it loads
};

struct PeerSync {
  const int* wait_flags = nullptr;     // this rank's signal words of the phase to wait for, one per source rank
  int* ctrl = nullptr;                 // control words of the rank's exchange buffer (epoch, tickets, abort)
  unsigned long long wait_ns = 0;
  int rank = 0, world = 1;
  int signal_phase = -1;
  int ticket = 0;                      // control word that counts finished CTAs
  size_t flags_off = 0;                // offset of the signal words inside an exchange buffer
  PeerPtrs peers = {};
};

struct GemmParams {
  const uint8_t* sfa;          // tiled scale factors of A: [m_tiles][rk][512]
  const uint8_t* sfb;          // tiled scale factors of B: [groups][b_row_tiles][rk][512]
  int m_rows;                  // rows of A that exist (TMA zero-fills beyond); grouped: padded total
  int n_cols;                  // output columns per row
  int k;                       // reduction length in elements
  int rk;                      // ceil(k / 64): scale-factor K-tiles per row tile
  int num_k_tiles;             // ceil(k / 256)
  int num_n_blocks;
  int b_row_tiles;             // 128-row tiles of B per group (scale-factor addressing)
  int gate_row_offset;         // SwiGLU epilogue: first row of the gate half inside B
  // tile list: plain GEMM uses ceil(m_rows/128) row blocks of one group; the grouped GEMMs
  // read the number of row blocks and the group of every row block from device memory
  const int* num_m_blocks_dev; // null -> num_m_blocks
  int num_m_blocks;
  const int* m_block_group;    // null -> group 0
  int num_groups;              // groups of B (experts); group indices read from device memory are clamped to it
  const int* m_block_rows;     // null -> all 128 rows of a block hold data; else rows of the block that do
  int* status;                 // device status word (bits of GemmStatusBits)
  // Order of the tile list.  0: column block outermost (CTAs running together share a few column blocks of B
  // and sweep the rows of A).  1: row block outermost: the CTAs running together hold a few row blocks of A
  // and the column blocks of their groups -- for the grouped GEMMs that keeps an expert's weights and its
  // rows in L2 for exactly as long as they are needed.
  int row_block_major;
  // Scale factors of A as plain rows instead of 128x4 tiles: byte [row][k / 16] with sfa_row_pitch bytes between
  // rows, fetched per stage as a box of 128 rows x 16 bytes through the kernel's third tensor map (tmap_aux, which
  // is the output map in the variants that store through TMA -- never both).  The MoE front end writes them this
  // way: a row's scale bytes are then one contiguous run for the writer instead of 4-byte pieces 512 bytes apart.
  int sfa_row_major;
  // Split-K (dense GEMMs with few tiles, e.g. M = 128 against a large weight matrix): the K tiles of every output
  // tile are dealt to k_splits work items that run on different CTAs at the same time, so that all SMs pull on the
  // weight stream; item s of a tile hands its partial sums to the epilogue as "group" s (EpilogueStore adds
  // group * group_stride to the output pointer) and a small kernel sums the partial matrices afterwards.
  int k_splits;                // 0 or 1: off
  // Flavour of the block scaling.  0: NVFP4 (e2m1, e4m3 scale per 16 elements: four 512-byte scale tiles per stage).
  // 1: MXFP4 (e2m1, ue8m0 scale per 32 elements: a tile spans 128 K-elements, two per stage).  2: MXFP8 (8-bit
  // operands, 128 of them per 128-byte stage row, ue8m0 scale per 32: one tile per stage).  rk counts the tiles
  // along K of the flavour; every flavour feeds the tensor core 32 bytes of K per row and instruction.
  int sf_block32;
  int a_fmt8, b_fmt8;          // MXFP8: operand format codes (0 = e4m3, 1 = e5m2)
  int k_bytes;                 // bytes of K per operand row (k / 2 for e2m1, k for 8-bit operands)
  // Expert-parallel launches synchronise with the other ranks inside the kernel instead of through extra
  // launches.  peer.wait_flags != null: every CTA's producer thread waits (bounded) until the signal words of all
  // ranks have reached this step before it issues its first load -- the operand rows were written by peers.
  // peer.signal_phase >= 0: the last CTA to finish raises that signal at every peer (its epilogue stored rows
  // into their memory).
  PeerSync peer;
};

struct SmemLayout {
  int stages;
  uint32_t a_bytes, b_bytes, sfa_bytes, sfb_bytes, stage_bytes, total;
  uint32_t epi_stage_bytes;    // per epilogue warp: its 32 rows of the output tile, parked for a TMA store (0 = none)
};
constexpr uint32_t kBarrierBytes = 512;

// kOutBytes: element size of an output tile that leaves through shared memory and a TMA store (128-wide plain
// tiles only; 0 = the epilogue stores from registers)
// kARows: rows of A that a stage holds.  Below 128 (256-wide tiles of launches whose row blocks all hold that few
// rows: decode) the MMA still reads 128 rows -- the rest of its A operand is whatever follows in the stage, times
// scale factors that are zero for rows without data -- and the shared memory saved buys another stage of B.
// kParkWide: 256-wide plain tiles whose 16-bit rows leave through TMA stores as well: every epilogue warp parks one
// box of 32 rows x 64 columns at a time (two passes over its 128 columns); the parking space costs a stage
template <int kBlockN, bool kSwigluB = false, int kOutBytes = 0, int kARows = 128, bool kParkWide = false>
__host__ __device__ constexpr SmemLayout smem_layout() {
  SmemLayout s{};
  s.a_bytes = kARows * 128;
  s.b_bytes = kBlockN * 128;
  s.sfa_bytes = 2048;
  // whole 128-row slabs, also for 64-row pieces; the up and gate pieces of a SwiGLU tile sit in different slabs
  s.sfb_bytes = (kSwigluB ? 2 : (kBlockN >= 128 ? kBlockN / 128 : 1)) * 2048;
  s.stage_bytes = s.a_bytes + s.b_bytes + s.sfa_bytes + s.sfb_bytes;
  s.epi_stage_bytes = (kBlockN == 128 && !kSwigluB) ? 32u * 128u * kOutBytes : 0u;
  if (kBlockN == 256 && kParkWide) s.epi_stage_bytes = 2u * 4096u;      // per tensor-memory quarter: two warps, one box each
  s.stages = kBlockN == 256 ? (kARows <= 32 ? 5 : (kParkWide ? 3 : 4)) : (kBlockN == 128 ? (kSwigluB ? 5 : (kOutBytes == 0 ? 6 : (kOutBytes == 4 ? 4 : 5))) : 7);
  s.total = s.stages * s.stage_bytes + 1024 /*alignment slack*/ + kBarrierBytes +
            (s.epi_stage_bytes != 0 ? 1024 + 4 * s.epi_stage_bytes : 0);
  return s;
}

struct PipeState {
  int stage = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void advance(int n) {
    if (++stage == n) {
      stage = 0;
      phase ^= 1;
    }
  }
};

// Poll an mbarrier phase; gives up when another role raised the abort flag or the cycle budget ran out.
// kBackoffNs > 0: sleep between polls.  Warps that spin take issue slots from the warps on the critical
// path (MMA issuer, slab movers); roles that can afford some wake-up latency back off.
template <int kBackoffNs = 0>
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                             long long limit_cycles = kWaitLimitCycles) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t it = 1;; ++it) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if constexpr (kBackoffNs > 0) __nanosleep(kBackoffNs);
    if ((it & 255u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit_cycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// Cycle accounting of the MMA-issuing thread (builds with -DB200FP4_ACCT only; two CTAs print one line per launch):
// where its cycles go -- waiting for a free accumulator, for the operand tiles, for the scale slabs, or issuing.
// The issue of an MMA blocks while the tensor pipe's queue is full, so "issue" approaches the execution time of
// the MMAs when they run back to back.
#ifdef B200FP4_ACCT
struct MmaAcct {
  long long acc = 0, full = 0, first = 0, sf = 0, issue = 0, t = 0, begin = 0;
  int tiles = 0, ksteps = 0;
  __device__ __forceinline__ void start() { begin = t = clock64(); }
  __device__ __forceinline__ void mark(long long& bucket) {
    const long long now = clock64();
    bucket += now - t;
    t = now;
  }
  __device__ __forceinline__ void skip() { t = clock64(); }
};
#define B200_ACCT(x) x
#else
#define B200_ACCT(x)
#endif

// ----------------------------------------------------------------------------
// Epilogue functors.  operator() is called by the 128 epilogue threads once per
// tile; `row` is the accumulator row (TMEM lane) of the calling thread.
// load(c0, regs) fetches 32 accumulator columns starting at c0.
// ----------------------------------------------------------------------------
template <typename OutT>
struct EpilogueStore {
  OutT* c;
  int64_t ldc;                  // elements
  const float* alpha;           // one scale, or one per group (alpha_per_group); null = 1
  int alpha_per_group;
  int64_t group_stride = 0;     // elements between the outputs of consecutive groups (split-K partial matrices)

  static constexpr int kOutBytes = static_cast<int>(sizeof(OutT));
  static constexpr bool kUsesOutputMap = true;      // 128-wide tiles leave through TMA stores
  static constexpr bool kParkWide = false;

  // The warp parks its 32 rows of the tile in shared memory (boxes of 32 rows x 128 bytes in the 128-byte
  // swizzle of the tensor map) and one lane hands them to TMA stores: the accumulator is free as soon as it has
  // been read, and the rows leave as whole lines while the next tile is computed.  Stores from registers put
  // every lane on another output row, which an SM sustains at about 11 bytes per cycle only.
  // part / parts: with two warps per TMEM quarter each parks and stores half of the tile's boxes
  template <int kBlockN, typename Loader>
  __device__ __forceinline__ void tma_path(const GemmParams& p, int m_blk, int n_blk, int row, float scale,
                                           Loader&& load, uint8_t* stage, const CUtensorMap* cmap, int part,
                                           int parts) const {
    constexpr int kBoxCols = 128 / static_cast<int>(sizeof(OutT));     // columns in the 128 bytes of a box row
    constexpr int kBoxes = kBlockN / kBoxCols;
    const int lane = row & 31;
    const int b_first = part * (kBoxes / parts), b_last = b_first + kBoxes / parts;
    if (lane == 0) ptx::bulk_wait_group_read0();      // the previous tile's stores have read this memory
    __syncwarp();
#pragma unroll
    for (int b = 0; b < kBoxes; ++b) {
      if (b < b_first || b >= b_last) continue;
      uint8_t* box = stage + (b - b_first) * 4096 + lane * 128;
#pragma unroll
      for (int h = 0; h < kBoxCols / 32; ++h) {
        uint32_t r[32];
        load(b * kBoxCols + 32 * h, r);
        if constexpr (sizeof(OutT) == 4) {
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            uint4 v;
            v.x = __float_as_uint(__uint_as_float(r[4 * q]) * scale);
            v.y = __float_as_uint(__uint_as_float(r[4 * q + 1]) * scale);
            v.z = __float_as_uint(__uint_as_float(r[4 * q + 2]) * scale);
            v.w = __float_as_uint(__uint_as_float(r[4 * q + 3]) * scale);
            *reinterpret_cast<uint4*>(box + ((q ^ (lane & 7)) << 4)) = v;
          }
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v;
            v.x = Pair16<OutT>::pack(__uint_as_float(r[8 * q]) * scale, __uint_as_float(r[8 * q + 1]) * scale);
            v.y = Pair16<OutT>::pack(__uint_as_float(r[8 * q + 2]) * scale, __uint_as_float(r[8 * q + 3]) * scale);
            v.z = Pair16<OutT>::pack(__uint_as_float(r[8 * q + 4]) * scale, __uint_as_float(r[8 * q + 5]) * scale);
            v.w = Pair16<OutT>::pack(__uint_as_float(r[8 * q + 6]) * scale, __uint_as_float(r[8 * q + 7]) * scale);
            *reinterpret_cast<uint4*>(box + (((4 * h + q) ^ (lane & 7)) << 4)) = v;
          }
        }
      }
    }
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      const int y = m_blk * kBlockM + (row & ~31);
#pragma unroll
      for (int b = 0; b < kBoxes; ++b) {
        if (b < b_first || b >= b_last) continue;
        const int col = n_blk * kBlockN + b * kBoxCols;
        if (col < p.n_cols && y < p.m_rows)
          ptx::tma_store_2d(cmap, col * static_cast<int>(sizeof(OutT)), y, ptx::smem_u32(stage + (b - b_first) * 4096));
      }
      ptx::bulk_commit_group();
    }
  }

  // part / parts: which share of the tile's columns this warp drains (two warps per TMEM quarter when parts == 2)
  // stage / cmap: the warp's parking space and the tensor map of the output for the TMA-store variant, or null
  template <int kBlockN, typename Loader, typename Release>
  __device__ __forceinline__ void operator()(const GemmParams& p, int m_blk, int n_blk, int group, int row,
                                             int rows_valid, int part, int parts, Loader&& load, Release&& release,
                                             uint8_t* stage = nullptr, const CUtensorMap* cmap = nullptr) const {
    const float scale = alpha == nullptr ? 1.0f : __ldg(alpha + (alpha_per_group ? group : 0));
    if (stage != nullptr) {
      tma_path<kBlockN>(p, m_blk, n_blk, row, scale, load, stage, cmap, part, parts);
      release();
      return;
    }
    if constexpr (sizeof(OutT) == 2 && kBlockN == 256) {
      // One accumulator per CTA: its drain is what the next tile waits for.  A warp's 128 columns fit in 64
      // registers once packed to 16 bits, so read and pack everything first, hand the accumulator back, and
      // store afterwards (the stores of a tile take ten times longer than reading it).
      const int64_t grow = static_cast<int64_t>(m_blk) * kBlockM + row;
      const bool row_ok = grow < p.m_rows && row < rows_valid;
      OutT* crow = c + grow * ldc + static_cast<int64_t>(n_blk) * kBlockN;
      const int cols_left = p.n_cols - n_blk * kBlockN;
      const int span = kBlockN / parts;          // 128 with two warps per TMEM quarter
      uint32_t packed[64];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (32 * i < span) {
          uint32_t r[32];
          load(part * span + 32 * i, r);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            packed[16 * i + j] =
                Pair16<OutT>::pack(__uint_as_float(r[2 * j]) * scale, __uint_as_float(r[2 * j + 1]) * scale);
        }
      }
      release();
      if (!row_ok) return;
      const bool wide = (reinterpret_cast<uintptr_t>(crow) & 31) == 0 && (ldc & 15) == 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {              // 16 columns = 32 bytes per store
        const int c0 = part * span + 16 * i;
        if (16 * i >= span) break;
        U32x8 v;
#pragma unroll
        for (int j = 0; j < 8; ++j) v.v[j] = packed[8 * i + j];
        if (wide && c0 + 8 < cols_left) {
          st_32B(crow + c0, v);
        } else {
          if (c0 < cols_left) *reinterpret_cast<uint4*>(crow + c0) = make_uint4(v.v[0], v.v[1], v.v[2], v.v[3]);
          if (c0 + 8 < cols_left) *reinterpret_cast<uint4*>(crow + c0 + 8) = make_uint4(v.v[4], v.v[5], v.v[6], v.v[7]);
        }
      }
      return;
    }
    const int64_t grow = static_cast<int64_t>(m_blk) * kBlockM + row;
    const bool row_ok = grow < p.m_rows && row < rows_valid;
    OutT* crow = c + group * group_stride + grow * ldc + static_cast<int64_t>(n_blk) * kBlockN;
    const int cols_left = p.n_cols - n_blk * kBlockN;
    const int span = kBlockN / parts;
#pragma unroll 1
    for (int c0 = part * span; c0 < (part + 1) * span; c0 += 32) {
      uint32_t r[32];
      load(c0, r);                 // warp-collective: every lane takes part, stores are predicated
      if (!row_ok) continue;
      if constexpr (sizeof(OutT) == 4) {
        // 32-byte stores: every lane writes another row, so a store instruction costs one L1 wavefront per
        // lane whatever its width -- wider stores halve the wavefronts per tile
#pragma unroll
        for (int g = 0; g < 4; ++g) {          // 8 columns = 32 bytes per store; n_cols is a multiple of 8
          if (c0 + 8 * g < cols_left) {
            U32x8 v;
#pragma unroll
            for (int i = 0; i < 8; ++i) v.v[i] = __float_as_uint(__uint_as_float(r[8 * g + i]) * scale);
            if ((reinterpret_cast<uintptr_t>(crow) & 31) == 0) {
              st_32B(crow + c0 + 8 * g, v);
            } else {
              uint4* dst = reinterpret_cast<uint4*>(crow + c0 + 8 * g);
              dst[0] = make_uint4(v.v[0], v.v[1], v.v[2], v.v[3]);
              dst[1] = make_uint4(v.v[4], v.v[5], v.v[6], v.v[7]);
            }
          }
        }
      } else {
        const bool wide = (reinterpret_cast<uintptr_t>(crow) & 31) == 0 && (ldc & 15) == 0;
#pragma unroll
        for (int g = 0; g < 2; ++g) {          // 16 columns = 32 bytes per store when rows are 32-byte aligned
          U32x8 v;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            v.v[i] = Pair16<OutT>::pack(__uint_as_float(r[16 * g + 2 * i]) * scale,
                                        __uint_as_float(r[16 * g + 2 * i + 1]) * scale);
          if (wide && c0 + 16 * g + 8 < cols_left) {
            st_32B(crow + c0 + 16 * g, v);
          } else {
            if (c0 + 16 * g < cols_left)
              *reinterpret_cast<uint4*>(crow + c0 + 16 * g) = make_uint4(v.v[0], v.v[1], v.v[2], v.v[3]);
            if (c0 + 16 * g + 8 < cols_left)
              *reinterpret_cast<uint4*>(crow + c0 + 16 * g + 8) = make_uint4(v.v[4], v.v[5], v.v[6], v.v[7]);
          }
        }
      }
    }
    release();
  }
};

// 256-wide plain tiles with bf16 rows that leave through TMA stores (FC2 of the MoE with short reductions).  The
// tile has one accumulator, so what counts is how soon it is handed back: each of the eight epilogue warps owns 128
// columns of its 32 rows as two 32 x 64 boxes and has 4 KB of parking space: it reads and packs the first box into
// registers, reads the second straight into the parking space, releases the accumulator, stores the second box by
// TMA and, once that store has read the space, parks and stores the first.  Register stores of the same tile take
// 64 KB through lanes that each write another row (about 12 bytes per cycle and SM).
struct EpilogueStoreWide {
  static constexpr int kOutBytes = 2;
  static constexpr bool kUsesOutputMap = true;
  static constexpr bool kParkWide = true;
  const float* alpha;           // one scale per group, or null
  template <int kBlockN, typename Loader, typename Release>
  __device__ __forceinline__ void operator()(const GemmParams& p, int m_blk, int n_blk, int group, int row,
                                             int /*rows_valid*/, int part, int parts, Loader&& load, Release&& release,
                                             uint8_t* stage = nullptr, const CUtensorMap* cmap = nullptr) const {
    static_assert(kBlockN == 256, "wide parking serves 256-wide tiles");
    const float scale = alpha == nullptr ? 1.0f : __ldg(alpha + group);
    const int lane = row & 31;
    uint8_t* box = stage + lane * 128;
    const int y = m_blk * kBlockM + (row & ~31);
    const int b0 = part * (4 / parts);                 // first 64-column box of this warp (it owns two: parts == 2)
    auto pack8 = [&](const uint32_t (&r)[32], int q) {
      uint4 v;
      v.x = Pair16<__nv_bfloat16>::pack(__uint_as_float(r[8 * q]) * scale, __uint_as_float(r[8 * q + 1]) * scale);
      v.y = Pair16<__nv_bfloat16>::pack(__uint_as_float(r[8 * q + 2]) * scale, __uint_as_float(r[8 * q + 3]) * scale);
      v.z = Pair16<__nv_bfloat16>::pack(__uint_as_float(r[8 * q + 4]) * scale, __uint_as_float(r[8 * q + 5]) * scale);
      v.w = Pair16<__nv_bfloat16>::pack(__uint_as_float(r[8 * q + 6]) * scale, __uint_as_float(r[8 * q + 7]) * scale);
      return v;
    };
    auto store_box = [&](int b) {
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int col = n_blk * kBlockN + b * 64;
        if (col < p.n_cols && y < p.m_rows) ptx::tma_store_2d(cmap, col * 2, y, ptx::smem_u32(stage));
        ptx::bulk_commit_group();
      }
    };
    // the first box waits in registers while the second is read, so the accumulator goes back without any wait for a
    // store in between
    uint4 first[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t r[32];
      load(b0 * 64 + 32 * h, r);
#pragma unroll
      for (int q = 0; q < 4; ++q) first[4 * h + q] = pack8(r, q);
    }
    if (lane == 0) ptx::bulk_wait_group_read0();       // the previous tile's last store has read the box
    __syncwarp();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t r[32];
      load((b0 + 1) * 64 + 32 * h, r);
#pragma unroll
      for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(box + (((4 * h + q) ^ (lane & 7)) << 4)) = pack8(r, q);
    }
    release();                                         // the accumulator has been read
    store_box(b0 + 1);
    if (lane == 0) ptx::bulk_wait_group_read0();
    __syncwarp();
#pragma unroll
    for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(box + ((c ^ (lane & 7)) << 4)) = first[c];
    store_box(b0);
  }
};

// FC2 of the expert-parallel MoE: every output row goes straight to the GPU that owns its token.  `row_tag[r]`
// names the destination of expert-major row r as (rank << 24 | slot), slot = token * top_k + j at that rank; the
// row lands at recv[slot][0..hidden) (bf16) in that rank's exchange buffer.  All remote accesses are plain
// stores of this kernel over NVLink (no TMA, no bulk copy to peer memory).  128-wide tiles park the warp's 32
// rows in shared memory first so that every row leaves as 256 contiguous bytes (16 lanes x 16 bytes, two rows
// per store instruction); 256-wide tiles store 32 bytes per lane from registers.
struct EpiloguePushRows {
  static constexpr int kOutBytes = 2;
  static constexpr bool kUsesOutputMap = false;
  static constexpr bool kParkWide = false;
  const int* row_tag;           // [rows] destination of every expert-major row
  PeerPtrs peers;               // exchange buffer of every rank as mapped into this process
  size_t recv_off;              // offset of the landing zone inside an exchange buffer
  int hidden;                   // row length
  const float* alpha;           // per group, or null
  const int* abort_flag;        // non-zero: a cross-rank wait expired earlier in this step -> touch no peer memory

  __device__ __forceinline__ __nv_bfloat16* row_dst(int tag) const {
    return reinterpret_cast<__nv_bfloat16*>(peers.p[(tag >> 24) & (kMaxPeers - 1)] + recv_off) +
           static_cast<int64_t>(tag & 0xffffff) * hidden;
  }

  template <int kBlockN, typename Loader, typename Release>
  __device__ __forceinline__ void operator()(const GemmParams& p, int m_blk, int n_blk, int group, int row,
                                             int rows_valid, int part, int parts, Loader&& load, Release&& release,
                                             uint8_t* stage = nullptr, const CUtensorMap* /*cmap*/ = nullptr) const {
    const float scale = alpha == nullptr ? 1.0f : __ldg(alpha + group);
    const int lane = row & 31;
    const int64_t grow = static_cast<int64_t>(m_blk) * kBlockM + row;
    const bool live = __ldg(abort_flag) == 0;
    const int tag = (row < rows_valid && live) ? __ldg(row_tag + grow) : -1;
    if constexpr (kBlockN == 128) {
      // park: 2 boxes of 32 rows x 128 bytes, 16-byte chunks XOR-swizzled by the row (no bank conflicts either way);
      // with two warps per TMEM quarter (parts == 2) each warp parks and sends one box: 128 bytes per row
      const int b_first = part * (2 / parts), b_last = b_first + 2 / parts;
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        if (b < b_first || b >= b_last) continue;
        uint8_t* box = stage + (b - b_first) * 4096 + lane * 128;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          load(b * 64 + 32 * h, r);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v;
            v.x = Pair16<__nv_bfloat16>::pack(__uint_as_float(r[8 * q]) * scale, __uint_as_float(r[8 * q + 1]) * scale);
            v.y = Pair16<__nv_bfloat16>::pack(__uint_as_float(r[8 * q + 2]) * scale, __uint_as_float(r[8 * q + 3]) * scale);
            v.z = Pair16<__nv_bfloat16>::pack(__uint_as_float(r[8 * q + 4]) * scale, __uint_as_float(r[8 * q + 5]) * scale);
            v.w = Pair16<__nv_bfloat16>::pack(__uint_as_float(r[8 * q + 6]) * scale, __uint_as_float(r[8 * q + 7]) * scale);
            *reinterpret_cast<uint4*>(box + (((4 * h + q) ^ (lane & 7)) << 4)) = v;
          }
        }
      }
      release();                                   // the accumulator has been read
      __syncwarp();
      const int lanes_per_row = 16 / parts;        // 16-byte chunks of the warp's piece of a row (256 or 128 bytes)
      const int rows_per_store = 32 / lanes_per_row;
      const int col0 = n_blk * kBlockN + b_first * 64;
      const int c16 = lane % lanes_per_row;
      const bool col_ok = col0 + c16 * 8 < p.n_cols;
#pragma unroll 4
      for (int pr = 0; pr < 32 / rows_per_store; ++pr) {
        const int r = rows_per_store * pr + lane / lanes_per_row;
        const int t = __shfl_sync(0xffffffffu, tag, r);
        const uint4 v = *reinterpret_cast<const uint4*>(stage + (c16 >> 3) * 4096 + r * 128 + (((c16 & 7) ^ (r & 7)) << 4));
        if (t >= 0 && col_ok) *reinterpret_cast<uint4*>(row_dst(t) + col0 + c16 * 8) = v;
      }
      __syncwarp();                                // the parking space is free for the next tile
    } else {
      static_assert(kBlockN == 256, "rows are pushed from 128- or 256-wide tiles");
      const int span = kBlockN / parts;
      uint32_t packed[64];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (32 * i < span) {
          uint32_t r[32];
          load(part * span + 32 * i, r);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            packed[16 * i + j] =
                Pair16<__nv_bfloat16>::pack(__uint_as_float(r[2 * j]) * scale, __uint_as_float(r[2 * j + 1]) * scale);
        }
      }
      release();
      if (tag < 0) return;
      __nv_bfloat16* crow = row_dst(tag) + static_cast<int64_t>(n_blk) * kBlockN;
      const int cols_left = p.n_cols - n_blk * kBlockN;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c0 = part * span + 16 * i;
        if (16 * i >= span) break;
        if (c0 < cols_left) *reinterpret_cast<uint4*>(crow + c0) = make_uint4(packed[8 * i], packed[8 * i + 1], packed[8 * i + 2], packed[8 * i + 3]);
        if (c0 + 8 < cols_left) *reinterpret_cast<uint4*>(crow + c0 + 8) = make_uint4(packed[8 * i + 4], packed[8 * i + 5], packed[8 * i + 6], packed[8 * i + 7]);
      }
    }
  }
};

// FC1 of the MoE: the accumulator columns are [up j0..j0+h-1 | gate j0..j0+h-1], h = half the tile width;
// act = bf16(silu(gate) * up), re-quantised to NVFP4 with the MoE activation packer
// (tests/python/test_flashinfer_b12x_verbatim.py:214-218) and written as the A operand of FC2.
struct EpilogueSwiglu {
  static constexpr int kOutBytes = 0;     // stores from registers
  static constexpr bool kUsesOutputMap = false;
  static constexpr bool kParkWide = false;
  uint8_t* act_codes;           // [m_rows, inter/2]
  uint8_t* act_sf;              // tiled [m_tiles][rk2][512], rk2 = ceil(inter/64)
  const float* w1_alpha;        // per group
  const float* fc2_input_scale; // one f32 (global scale of the activation quantiser)
  int inter;                    // activation columns per row

  template <int kBlockN, typename Loader, typename Release>
  __device__ __forceinline__ void operator()(const GemmParams& p, int m_blk, int n_blk, int group, int row,
                                             int rows_valid, int part, int parts, Loader&& load, Release&& release,
                                             uint8_t* /*stage*/ = nullptr, const CUtensorMap* /*cmap*/ = nullptr) const {
    constexpr int kHalf = kBlockN / 2;
    static_assert(kHalf % 64 == 0, "the SwiGLU epilogue pairs two halves of whole 32-column groups per warp");
    const float a1 = w1_alpha == nullptr ? 1.0f : __ldg(w1_alpha + group);
    const float gs = fc2_input_scale == nullptr ? 1.0f : __ldg(fc2_input_scale);
    const int64_t grow = static_cast<int64_t>(m_blk) * kBlockM + row;
    const int j0 = n_blk * kHalf;
    const int rk2 = (inter + 63) >> 6;
    uint8_t* sf_tile = act_sf + static_cast<int64_t>(m_blk) * rk2 * 512 + (row & 31) * 16 + (row >> 5) * 4;
    const int span = kHalf / parts;
    // one 32-column group: silu(gate) * up -> bf16 -> NVFP4 (two 16-element blocks), codes and scale bytes out
    // The arithmetic runs on the packed f32x2 instructions where it can (scaling, 1 + e, the product, the bf16
    // round trip): every operation is the same IEEE f32 operation as in scalar form, two per instruction -- the
    // fewer instructions the epilogue issues, the less it holds up the warps that feed the tensor pipe.
    const uint64_t a1_2 = f32x2_pack(a1, a1);
    const uint64_t one_2 = f32x2_pack(1.0f, 1.0f);
    auto finish = [&](int c0, const uint32_t (&up)[32], const uint32_t (&gate)[32]) {
      if (j0 + c0 >= inter) return;
      uint32_t sfpair = 0;
      uint32_t codes[4];
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        uint64_t v2[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint64_t u2 = f32x2_mul(f32x2_pack(__uint_as_float(up[16 * b + 2 * i]), __uint_as_float(up[16 * b + 2 * i + 1])), a1_2);
          const uint64_t g2 = f32x2_mul(f32x2_pack(__uint_as_float(gate[16 * b + 2 * i]), __uint_as_float(gate[16 * b + 2 * i + 1])), a1_2);
          const float g0 = f32x2_lo(g2), g1 = f32x2_hi(g2);
          const uint64_t d2 = f32x2_add(one_2, f32x2_pack(__expf(-g0), __expf(-g1)));
          // silu in f32 (a few ulp; rounded to bf16 next)
          const uint64_t s2 = f32x2_pack(__fdividef(g0, f32x2_lo(d2)), __fdividef(g1, f32x2_hi(d2)));
          v2[i] = pair16_to_f32x2<__nv_bfloat16>(f32x2_to_pair16<__nv_bfloat16>(f32x2_mul(s2, u2)));
        }
        uint32_t sfb;
        quantize_block16<true>(v2, gs, codes[2 * b], codes[2 * b + 1], sfb);
        sfpair |= sfb << (8 * b);
      }
      *reinterpret_cast<uint4*>(act_codes + grow * (inter >> 1) + ((j0 + c0) >> 1)) =
          make_uint4(codes[0], codes[1], codes[2], codes[3]);
      const int kb = (j0 + c0) >> 4;          // even
      *reinterpret_cast<uint16_t*>(sf_tile + (kb & 3) + (kb >> 2) * 512) = static_cast<uint16_t>(sfpair);
    };
    // The accumulator is released after the warp's last read of it.  With sixteen warps (span = 32) that is
    // before any arithmetic.  With eight, reading the whole share first -- 128 registers -- to release early was
    // measured slower (116 against 103 us for FC1 of the prefill shape).
#pragma unroll 1
    for (int c0 = part * span; c0 < (part + 1) * span; c0 += 32) {
      uint32_t up[32], gate[32];
      load(c0, up);
      load(kHalf + c0, gate);
      if (c0 + 32 >= (part + 1) * span) release();      // last read of the accumulator: the arithmetic follows
      finish(c0, up, gate);
    }
  }
};

// ----------------------------------------------------------------------------
// kSwigluB: B tile = two pieces of kBlockN/2 rows (up rows, gate rows); otherwise consecutive 128-row pieces
// (one 64-row piece for 64-wide tiles).
// ----------------------------------------------------------------------------
// kEpi: number of epilogue warps (0 = the default of the tile shape)
template <int kBlockN, bool kSwigluB, typename Epilogue, int kARows = 128, int kEpi = 0>
__global__ void __launch_bounds__(gemm_threads(kBlockN, kSwigluB, kEpi), 1)
nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_aux, const GemmParams p, const Epilogue epi) {
  static_assert(kARows == 128 || (kBlockN == 256 && kARows == 32), "few-row stages exist for 256-wide tiles");
  constexpr SmemLayout L = smem_layout<kBlockN, kSwigluB, Epilogue::kOutBytes, kARows, Epilogue::kParkWide>();
  constexpr int kStages = L.stages;
  constexpr int kAccStages = kBlockN == 256 ? 1 : 2;
  constexpr int kBPieces = kSwigluB ? 2 : (kBlockN >= 128 ? kBlockN / 128 : 1);
  constexpr int kBPieceRows = kBlockN / kBPieces;               // rows per TMA box of B
  constexpr bool kHalfSlabPieces = kSwigluB && kBPieceRows == 64;   // two 64-row pieces: half a slab each
  constexpr int kEpiWarps = epilogue_warps(kBlockN, kSwigluB, kEpi);
  // slab columns per 64-wide K block: one per 32 rows of the tile (64-wide tiles keep their whole slab)
  constexpr uint32_t kSfbColsPerKb = kBlockN >= 128 ? kBlockN / 32 : 4;
  constexpr uint32_t kSfaCol = kAccStages * kBlockN;            // TMEM columns: accumulators first
  constexpr uint32_t kSfSetCols = 16 + 4 * kSfbColsPerKb;       // columns of one set of scale slabs (SFA + SFB)
  constexpr uint32_t kIdesc = ptx::idesc_mxf4nvf4(kBlockN);
  constexpr int kFirstSfWarp = 2 + kEpiWarps;
  static_assert(kSfaCol + kStages * kSfSetCols <= kTmemCols, "TMEM budget: one set of slab columns per stage");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kStages * L.stage_bytes;
  // barrier slots (8 bytes each): full[kStages], empty[kStages], acc_full[2], acc_empty[2]; then tmem ptr, abort flag
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto acc_full_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };
  auto acc_empty_bar = [&](int s) { return bar_base + 8u * (2 * kStages + 2 + s); };
  auto sf_full_bar = [&](int s) { return bar_base + 8u * (2 * kStages + 4 + s); };
  auto sf_loaded_bar = [&](int s) { return bar_base + 8u * (3 * kStages + 4 + s); };
  uint8_t* tail_gen = smem_gen + kStages * L.stage_bytes + 8 * (4 * kStages + 4);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(tail_gen);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail_gen + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
      ptx::mbar_init(sf_full_bar(s), 4);                 // one arrival per slab-mover warp
      ptx::mbar_init(sf_loaded_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(acc_full_bar(s), 1);
      ptx::mbar_init(acc_empty_bar(s), kEpiWarps);           // one arrival per epilogue warp
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
    if ((L.epi_stage_bytes != 0 && Epilogue::kUsesOutputMap) || p.sfa_row_major) ptx::prefetch_tensormap(&tmap_aux);
  }
  if (warp == 0) {
    __syncwarp();
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  // grouped launches read the number of row blocks from device memory; never trust it beyond the table size
  const int num_m_blocks =
      p.num_m_blocks_dev != nullptr ? max(0, min(__ldg(p.num_m_blocks_dev), p.num_m_blocks)) : p.num_m_blocks;
  const int num_out_tiles = num_m_blocks * p.num_n_blocks;
  const int splits = p.k_splits > 1 ? p.k_splits : 1;
  const int kt_per_split = (p.num_k_tiles + splits - 1) / splits;
  const int num_tiles = num_out_tiles * splits;               // work items: (output tile, K slice)
  auto tile_m = [&](int item) {
    const int tile = item % num_out_tiles;
    return p.row_block_major ? tile / p.num_n_blocks : tile % num_m_blocks;
  };
  auto tile_n = [&](int item) {
    const int tile = item % num_out_tiles;
    return p.row_block_major ? tile % p.num_n_blocks : tile / num_m_blocks;
  };
  auto tile_kt0 = [&](int item) { return (item / num_out_tiles) * kt_per_split; };
  auto tile_kt1 = [&](int item) { return min(p.num_k_tiles, (item / num_out_tiles + 1) * kt_per_split); };

  if (warp == 0) {
    // =============================== TMA producer ===============================
    if (lane == 0) {
      PipeState st;
      bool ok = true;
      if (p.peer.wait_flags != nullptr && p.peer.world > 1) {
        // rows of A come from the other ranks: wait for their "rows placed" signals (bounded)
        const int epoch = *reinterpret_cast<volatile int*>(p.peer.ctrl + kCtrlEpoch) + 1;
        ok = *reinterpret_cast<volatile int*>(p.peer.ctrl + kCtrlAbort) == 0;
        for (int r = 0; r < p.peer.world && ok; ++r) {
          if (r != p.peer.rank && !wait_flag(p.peer.wait_flags + r, epoch, p.peer.wait_ns)) {
            ok = false;
            atomicOr(p.status, kStatusPeerWaitExpired);
            atomicExch(p.peer.ctrl + kCtrlAbort, 1);
          }
        }
        if (!ok) *abort_flag = 1;          // the other roles leave at their next poll
        // peers wrote the rows with ordinary stores; the loads below go through the async proxy
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m_blk = tile_m(tile);
        const int n_blk = tile_n(tile);
        const int group =
            p.m_block_group != nullptr ? max(0, min(__ldg(p.m_block_group + m_blk), p.num_groups - 1)) : 0;
        int b_row[kBPieces];
        if constexpr (kSwigluB) {
          b_row[0] = n_blk * kBPieceRows;
          b_row[1] = p.gate_row_offset + n_blk * kBPieceRows;
        } else {
#pragma unroll
          for (int i = 0; i < kBPieces; ++i) b_row[i] = n_blk * kBlockN + kBPieceRows * i;
        }
        if (kARows < kBlockM && p.m_block_rows != nullptr && __ldg(p.m_block_rows + m_blk) > kARows)
          atomicOr(p.status, kStatusRowsExceedTile);      // results of this block are wrong: tell the host
        for (int kt = tile_kt0(tile), kt_end = tile_kt1(tile); kt < kt_end; ++kt) {
          if (!wait_bounded(empty_bar(st.stage), st.phase ^ 1u, abort_flag)) {
            atomicOr(p.status, kStatusTimeoutProducer);
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + st.stage * L.stage_bytes;
          const uint32_t sb = sa + L.a_bytes;
          const uint32_t ssfa = sb + L.b_bytes;
          const uint32_t ssfb = ssfa + L.sfa_bytes;
          const int tps = 4 >> p.sf_block32;                            // 512-byte scale tiles per stage: 4, 2 or 1
          const int k_sf_tiles = min(tps, p.rk - tps * kt);
          const uint32_t sf_bytes = static_cast<uint32_t>(k_sf_tiles) * 512u;
          // the scale slabs go first and report to their own barrier: the movers carry them into tensor
          // memory while the operand tiles are still on their way
          const uint32_t sbar = sf_loaded_bar(st.stage);
          if (p.sfa_row_major) {
            ptx::mbar_expect_tx(sbar, 2048u + sf_bytes * kBPieces);     // a box always delivers its full size
            ptx::tma_load_2d(ssfa, &tmap_aux, kt * 16, m_blk * kBlockM, sbar);
          } else {
            ptx::mbar_expect_tx(sbar, sf_bytes * (1 + kBPieces));
            ptx::bulk_load(ssfa, p.sfa + (static_cast<int64_t>(m_blk) * p.rk + tps * kt) * 512, sf_bytes, sbar);
          }
#pragma unroll
          for (int i = 0; i < kBPieces; ++i) {
            const int64_t tile_idx = static_cast<int64_t>(group) * p.b_row_tiles + (b_row[i] >> 7);
            ptx::bulk_load(ssfb + i * 2048, p.sfb + (tile_idx * p.rk + tps * kt) * 512, sf_bytes, sbar);
          }
          const uint32_t bar = full_bar(st.stage);
          ptx::mbar_expect_tx(bar, L.a_bytes + L.b_bytes);
          ptx::tma_load_2d(sa, &tmap_a, kt * 128, m_blk * kBlockM, bar);
#pragma unroll
          for (int i = 0; i < kBPieces; ++i) ptx::tma_load_3d(sb + i * kBPieceRows * 128, &tmap_b, kt * 128, b_row[i], group, bar);
          st.advance(kStages);
        }
      }
    }
  } else if (warp == 1) {
    // =============================== MMA issuer ===============================
    // The whole warp walks the loop and one elected lane issues: every operand of the MMAs (descriptors,
    // tensor-memory addresses) is then the same in all lanes, which lets the compiler keep them in the
    // warp-wide registers the instructions read.  Computed in one lane only they must be moved there before
    // every MMA, and a lone thread spends about 110 cycles per MMA on that instead of 55 to 65.
    {
      PipeState st;
      PipeState acc;
      bool ok = true;
      const uint64_t a_desc0 = ptx::smem_desc_sw128(smem_base);
      const uint64_t b_desc0 = ptx::smem_desc_sw128(smem_base + L.a_bytes);
      const int last_kblocks = ((p.k_bytes - (p.num_k_tiles - 1) * 128) + 31) >> 5;   // 32-byte steps of the last K tile
      B200_ACCT(MmaAcct acct; acct.start();)
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        B200_ACCT(acct.skip();)
        if (!wait_bounded(acc_empty_bar(acc.stage), acc.phase ^ 1u, abort_flag)) {
          if (lane == 0) atomicOr(p.status, kStatusTimeoutMma);
          break;
        }
        B200_ACCT(acct.mark(acct.acc); ++acct.tiles;)
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc.stage * kBlockN;
        // a 64-wide tile uses half of a 128-row slab of B scale factors: its row groups start at column 0 or 2
        // (the movers of a SwiGLU tile with 64-row pieces have already picked the right halves)
        const uint32_t sfb_shift = kBlockN >= 128 ? 0u : static_cast<uint32_t>((tile_n(tile) * kBlockN & 127) >> 5);
        const uint32_t sf_t0 = tmem_base + kSfaCol + 16 + sfb_shift;
        const int kt_first = tile_kt0(tile);
        for (int kt = kt_first, kt_end = tile_kt1(tile); kt < kt_end; ++kt) {
          // the slab movers have put this stage's scale factors into its set of TMEM columns (usually long
          // before the operands land), and the operand tiles are in shared memory
#ifdef B200FP4_ACCT
          acct.skip();
          wait_bounded(full_bar(st.stage), st.phase, abort_flag);
          if (kt == kt_first) {
            const long long before = acct.full;
            acct.mark(acct.full);
            acct.first += acct.full - before;
          } else {
            acct.mark(acct.full);
          }
          wait_bounded(sf_full_bar(st.stage), st.phase, abort_flag);
          acct.mark(acct.sf);
          ++acct.ksteps;
#endif
          if (!wait_bounded(sf_full_bar(st.stage), st.phase, abort_flag) ||
              !wait_bounded(full_bar(st.stage), st.phase, abort_flag)) {
            if (lane == 0) atomicOr(p.status, kStatusTimeoutMma);
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint64_t stage_off = static_cast<uint64_t>(st.stage * (L.stage_bytes >> 4));
          const uint64_t da = a_desc0 + stage_off, db = b_desc0 + stage_off;      // + 2 per 32 bytes of K
          const uint32_t sfb_t = sf_t0 + st.stage * kSfSetCols;
          const uint32_t sfa_t = tmem_base + kSfaCol + st.stage * kSfSetCols;
          const int kblocks = kt + 1 == p.num_k_tiles ? last_kblocks : 4;
          if (ptx::elect_one()) {
            if (p.sf_block32 == 2) {
              // one scale tile per stage; instruction kb reads byte kb of its columns
#pragma unroll
              for (int kb = 0; kb < 4; ++kb) {
                if (kb < kblocks)
                  ptx::mma_mxf8_block32(d_tmem, da + 2 * kb, db + 2 * kb,
                                        ptx::idesc_mxf8_block32(kBlockN, p.a_fmt8, p.b_fmt8, kb), sfa_t, sfb_t,
                                        (kt != kt_first || kb != 0) ? 1u : 0u);
              }
            } else if (p.sf_block32 == 1) {
              // a scale tile serves two instructions (bytes 0-1, then 2-3 of its columns)
#pragma unroll
              for (int kb = 0; kb < 4; ++kb) {
                if (kb < kblocks)
                  ptx::mma_mxf4_block32(d_tmem, da + 2 * kb, db + 2 * kb, ptx::idesc_mxf4_block32(kBlockN, (kb & 1) * 2),
                                        sfa_t + 4 * (kb >> 1), sfb_t + kSfbColsPerKb * (kb >> 1),
                                        (kt != kt_first || kb != 0) ? 1u : 0u);
              }
            } else {
              ptx::mma_mxf4nvf4(d_tmem, da, db, kIdesc, sfa_t, sfb_t, kt != kt_first ? 1u : 0u);
#pragma unroll
              for (int kb = 1; kb < 4; ++kb) {
                if (kb < kblocks)
                  ptx::mma_mxf4nvf4(d_tmem, da + 2 * kb, db + 2 * kb, kIdesc, sfa_t + 4 * kb, sfb_t + kSfbColsPerKb * kb, 1u);
              }
            }
            ptx::tc_commit(empty_bar(st.stage));        // stage reusable once these MMAs have read it
          }
          __syncwarp();
          B200_ACCT(acct.mark(acct.issue);)
          st.advance(kStages);
        }
        if (ok && ptx::elect_one()) ptx::tc_commit(acc_full_bar(acc.stage));
        __syncwarp();
        acc.advance(kAccStages);
      }
#ifdef B200FP4_ACCT
      if (lane == 0 && (blockIdx.x == 3 || blockIdx.x == 100))
        printf("acct cta %d tile_n %d swiglu %d epi_warps %d: tiles %d ksteps %d cycles %lld = accumulator wait %lld + "
               "operand wait %lld (first K step of a tile %lld) + slab wait %lld + issue %lld + other\n",
               blockIdx.x, kBlockN, kSwigluB ? 1 : 0, kEpiWarps, acct.tiles, acct.ksteps, clock64() - acct.begin, acct.acc,
               acct.full, acct.first, acct.sf, acct.issue);
#endif
    }
  } else if (warp >= kFirstSfWarp && warp < kFirstSfWarp + 4) {
    // =============================== scale-slab movers ===============================
    // Lane l of every quarter needs the 16 bytes of slab row l per 64-wide K block: 4 columns of SFA
    // (row groups 0-3 of the 128-row tile) and 4 per 128 rows of B.  All four warps write the same
    // values, each into its own 32 lanes: the MMA expects the slab replicated in every quarter.
    const int quarter = warp & 3;
    PipeState st;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      // 64-row pieces: rows (n_blk * 64) % 128 .. +63 of their slab = its row groups 0-1 or 2-3
      const bool upper_half = kHalfSlabPieces && (tile_n(tile) & 1) != 0;
      for (int kt = tile_kt0(tile), kt_end = tile_kt1(tile); kt < kt_end; ++kt) {
        if (!wait_bounded(sf_loaded_bar(st.stage), st.phase, abort_flag)) {
          if (lane == 0) atomicOr(p.status, kStatusTimeoutMma);
          ok = false;
          break;
        }
        const uint8_t* slab = smem_gen + st.stage * L.stage_bytes + L.a_bytes + L.b_bytes + lane * 16;
        const uint32_t t_sf = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kSfaCol + st.stage * kSfSetCols;
        uint32_t ra[16];
        if (p.sfa_row_major) {
          // stage holds [128 rows][16 bytes]: the words of row 32 c + lane are K blocks 0..3 of row group c
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 v = *reinterpret_cast<const uint4*>(slab + 512 * c);
            ra[c] = v.x, ra[4 + c] = v.y, ra[8 + c] = v.z, ra[12 + c] = v.w;
          }
        } else {
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            const uint4 v = *reinterpret_cast<const uint4*>(slab + 512 * kb);
            ra[4 * kb] = v.x, ra[4 * kb + 1] = v.y, ra[4 * kb + 2] = v.z, ra[4 * kb + 3] = v.w;
          }
        }
        ptx::tmem_st_32x16(t_sf, ra);
        const uint8_t* slab_b = slab + L.sfa_bytes;
        if constexpr (kHalfSlabPieces) {
          // columns per K block: [up rows 0-31, up rows 32-63, gate rows 0-31, gate rows 32-63] of the tile
          uint32_t rb[16];
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            const uint4 u = *reinterpret_cast<const uint4*>(slab_b + 512 * kb);
            const uint4 g = *reinterpret_cast<const uint4*>(slab_b + 2048 + 512 * kb);
            rb[4 * kb] = upper_half ? u.z : u.x, rb[4 * kb + 1] = upper_half ? u.w : u.y;
            rb[4 * kb + 2] = upper_half ? g.z : g.x, rb[4 * kb + 3] = upper_half ? g.w : g.y;
          }
          ptx::tmem_st_32x16(t_sf + 16, rb);
        } else if constexpr (kBPieces == 2) {
          uint32_t rb[32];
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const uint4 v = *reinterpret_cast<const uint4*>(slab_b + 2048 * i + 512 * kb);
              rb[8 * kb + 4 * i] = v.x, rb[8 * kb + 4 * i + 1] = v.y, rb[8 * kb + 4 * i + 2] = v.z,
                          rb[8 * kb + 4 * i + 3] = v.w;
            }
          }
          ptx::tmem_st_32x32(t_sf + 16, rb);
        } else {
          uint32_t rb[16];
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            const uint4 v = *reinterpret_cast<const uint4*>(slab_b + 512 * kb);
            rb[4 * kb] = v.x, rb[4 * kb + 1] = v.y, rb[4 * kb + 2] = v.z, rb[4 * kb + 3] = v.w;
          }
          ptx::tmem_st_32x16(t_sf + 16, rb);
        }
        ptx::tmem_st_wait();
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(sf_full_bar(st.stage));
        st.advance(kStages);
      }
    }
  } else if (warp >= 2 && warp < kFirstSfWarp) {
    // =============================== epilogue ===============================
    constexpr int kParts = kEpiWarps / 4;
    const int quarter = warp & 3;                      // TMEM lanes this warp may touch
    const int part = (warp - 2) >> 2;                  // which share of the columns (two warps per quarter)
    const int row = quarter * 32 + lane;
    PipeState acc;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int m_blk = tile_m(tile);
      const int n_blk = tile_n(tile);
      const int group =
          p.m_block_group != nullptr ? max(0, min(__ldg(p.m_block_group + m_blk), p.num_groups - 1))
                                     : (splits > 1 ? tile / num_out_tiles : 0);
      if (!wait_bounded<64>(acc_full_bar(acc.stage), acc.phase, abort_flag)) {
        if (lane == 0) atomicOr(p.status, kStatusTimeoutEpilogue);
        break;
      }
      ptx::tc_fence_after_sync();
      const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc.stage * kBlockN;
      const int rows_valid = p.m_block_rows != nullptr ? __ldg(p.m_block_rows + m_blk) : kBlockM;
      if (quarter * 32 < rows_valid) {                 // a warp whose 32 rows only pad the block has nothing to do
        // parking space of the TMA-store variant: 1024-byte aligned, one slice per epilogue warp
        uint8_t* stage = nullptr;
        if constexpr (L.epi_stage_bytes != 0) {
          // four slices of epi_stage_bytes per CTA; with two warps per TMEM quarter each takes half a slice
          const uint32_t off = ((kStages * L.stage_bytes + kBarrierBytes + 1023u) & ~1023u) +
                               (warp - 2) * (L.epi_stage_bytes / (kEpiWarps / 4));
          stage = smem_gen + off;
        }
        // the functor calls `release` once, as soon as it has read the accumulator for the last time: the MMAs
        // of the next tile may start while it is still converting and storing
        epi.template operator()<kBlockN>(p, m_blk, n_blk, group, row, rows_valid, part, kParts,
                                         [&](int c0, uint32_t (&r)[32]) {
                                           ptx::tmem_ld_32x32(t_acc + c0, r);
                                           ptx::tmem_ld_wait();
                                         },
                                         [&]() {        // called by all lanes of the warp together
                                           ptx::tc_fence_before_sync();
                                           __syncwarp();
                                           if (lane == 0) ptx::mbar_arrive(acc_empty_bar(acc.stage));
                                         },
                                         stage, &tmap_aux);
      } else {
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(acc_empty_bar(acc.stage));
      }
      acc.advance(kAccStages);
    }
    // the TMA stores of this warp's last tiles must have left shared memory and reached global memory
    if (L.epi_stage_bytes != 0 && lane == 0) ptx::bulk_wait_group0();
  }

  // ---- teardown: everybody meets, then the allocating warp frees tensor memory
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (p.peer.signal_phase >= 0 && p.peer.world > 1 && threadIdx.x == 32) {
    // this CTA's rows are on their way to the peers; the last CTA to get here tells every rank
    __threadfence_system();
    if (atomicAdd(p.peer.ctrl + p.peer.ticket, 1) == static_cast<int>(gridDim.x) - 1) {
      p.peer.ctrl[p.peer.ticket] = 0;
      if (*reinterpret_cast<volatile int*>(p.peer.ctrl + kCtrlAbort) == 0) {
        __threadfence_system();
        const int epoch = *reinterpret_cast<volatile int*>(p.peer.ctrl + kCtrlEpoch) + 1;
        for (int r = 0; r < p.peer.world; ++r)
          if (r != p.peer.rank)
            st_release_sys(reinterpret_cast<int*>(p.peer.peers.p[r] + p.peer.flags_off) +
                               p.peer.signal_phase * kMaxPeers + p.peer.rank, epoch);
      }
    }
  }
  if (warp == 0) {
    if (*abort_flag) {
      // a role gave up: let copies that are still in flight land before the CTA's memory is reused
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    __syncwarp();
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace b200fp4
