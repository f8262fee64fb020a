// NVFP4 block-scaled dense GEMM on CTA pairs (tcgen05 cta_group::2) for sm_100a.
//
// The single-CTA kernel (gemm_kernel.cuh) is bound by the bytes each SM pulls through its
// L2 port: a 128 x 256 tile needs 54 KB of operands per 256-wide K step.  Here two CTAs of a
// 2-CTA cluster share one 256 x 256 tile: each loads its own 128 rows of A, its own 128 of
// the 256 B rows and the scale factors, 38 KB per K step for the same flops per SM, and the
// even CTA issues 256-row MMAs that read B from both CTAs' shared memory.  Every CTA keeps
// its 128 x 256 half of the accumulator in its own tensor memory and drains it itself.
//
// Per CTA: warp 0 lane 0 = TMA producer (loads credit the full-barrier of the even CTA),
// warp 1 lane 0 of the even CTA = MMA issuer (tcgen05.commit with a CTA mask releases the
// stage in both CTAs), warps 2-9 = epilogue, warps 10-13 = scale-slab movers (shared memory ->
// tensor memory with tcgen05.st, each CTA for itself; they report to the even CTA).  No TMA multicast is used anywhere: every tile
// is fetched by the CTA that needs it.  All waits are bounded as in the single-CTA kernel.
//
// Measured at M = N = K = 8192 (cycle accounting of the MMA-issuing thread, -DB200FP4_ACCT): 720 cycles per K step
// against 875 for the single-CTA kernel with 128 x 256 tiles (512 would keep the tensor pipe busy).  40 % of the
// issuing thread's cycles go into issuing MMAs, 15 % into waiting for operand tiles and 26 % into waiting for
// scale slabs that reach tensor memory after the operands have landed.  Tried against that slab wait, without
// gain: a second group of mover warps (unchanged: one group keeps up); a slab ring of its own, twice as deep as
// the operand ring, with the slabs requested five K steps early and held in the movers' registers until the
// columns are free (slab wait down to 7 %, operand wait up to 45 %, 15 to 25 % slower overall); loading only A
// (42 % fewer bytes per stage: 7 % faster, so the kernel is not bound by the bytes an SM can take in); two groups
// of movers that each carry two of a stage's four K blocks and report to barriers of their own, the MMAs of
// blocks 2-3 issued after a second wait (the extra wait, fence and election in the issuing thread cost more than
// the shorter slab chain saves: 17 % slower).
#pragma once

#include "gemm_kernel.cuh"

namespace b200fp4 {


constexpr int kPairStages = 5;
constexpr uint32_t kPairStageBytes = 16384 + 16384 + 2048 + 4096;    // A, B half, SFA, SFB (both halves)
constexpr uint32_t kPairSmemBytes = kPairStages * kPairStageBytes + 1024 + 256;
constexpr int kPairThreads = 64 + 8 * 32 + 128;     // TMA, MMA, 8 epilogue warps, 4 scale-slab movers

template <typename Epilogue>
__global__ void __launch_bounds__(kPairThreads, 1)
nvfp4_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                       const GemmParams p, const Epilogue epi) {
  constexpr int kStages = kPairStages;
  constexpr int kBlockN = 256;
  constexpr uint32_t kSfaCol = 256;
  constexpr uint32_t kSfSetCols = 48;                    // 16 columns of SFA + 32 of SFB per stage
  static_assert(kSfaCol + kPairStages * kSfSetCols <= kTmemCols, "TMEM budget");
  constexpr uint32_t kIdesc = ptx::idesc_mxf4nvf4_m256(kBlockN);
  constexpr uint32_t kABytes = 16384, kBBytes = 16384, kSfaBytes = 2048;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kStages * kPairStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  const uint32_t acc_full_bar = bar_base + 8u * (2 * kStages);
  const uint32_t acc_empty_bar = bar_base + 8u * (2 * kStages + 1);
  auto sf_loaded_bar = [&](int s) { return bar_base + 8u * (2 * kStages + 2 + s); };   // own slabs have landed
  auto sf_full_bar = [&](int s) { return bar_base + 8u * (3 * kStages + 2 + s); };     // both CTAs' slabs are in TMEM
  uint8_t* tail_gen = smem_gen + kStages * kPairStageBytes + 8 * (4 * kStages + 2);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(tail_gen);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail_gen + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();          // 0 = even CTA (issues the MMAs), 1 = its peer
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);                    // the even CTA's expect_tx arrival (+ both CTAs' bytes)
      ptx::mbar_init(empty_bar(s), 1);                   // one commit per use, delivered to both CTAs
      ptx::mbar_init(sf_loaded_bar(s), 1);
      ptx::mbar_init(sf_full_bar(s), 8);                 // four mover warps in each CTA
    }
    ptx::mbar_init(acc_full_bar, 1);
    ptx::mbar_init(acc_empty_bar, 2 * 8);                // the epilogue warps of both CTAs
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
    ptx::prefetch_tensormap(&tmap_sfa);
    ptx::prefetch_tensormap(&tmap_sfb);
  }
  if (warp == 0) {
    __syncwarp();
    ptx::tmem2_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), kTmemCols);
    ptx::tmem2_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::cluster_sync();                                   // both CTAs' barriers exist before anyone signals them
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const int num_tiles = p.num_m_blocks * p.num_n_blocks; // num_m_blocks counts 256-row blocks here

  if (warp == 0) {
    // =============================== TMA producer (both CTAs) ===============================
    if (lane == 0) {
      PipeState st;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int m2 = tile % p.num_m_blocks;
        const int n_blk = tile / p.num_m_blocks;
        const int m_tile = 2 * m2 + static_cast<int>(rank);          // 128-row tile of A owned by this CTA
        for (int kt = 0; kt < p.num_k_tiles; ++kt) {
          if (!wait_bounded(empty_bar(st.stage), st.phase ^ 1u, abort_flag)) {
            atomicOr(p.status, kStatusTimeoutProducer);
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + st.stage * kPairStageBytes;
          const uint32_t sb = sa + kABytes;
          const uint32_t ssfa = sb + kBBytes;
          const uint32_t ssfb = ssfa + kSfaBytes;
          const uint32_t bar = full_bar(st.stage) & ptx::kPeerBitMask;   // always the even CTA's barrier
          // the scale slabs go first: this CTA's own mover warps (local barrier) carry them into tensor memory
          // while the operand tiles are still on their way
          const uint32_t sbar = sf_loaded_bar(st.stage);
          ptx::mbar_expect_tx(sbar, kSfaBytes + 4096);
          ptx::tma_load_2d(ssfa, &tmap_sfa, 0, (m_tile * p.rk + 4 * kt) * 2, sbar);
#pragma unroll
          for (int i = 0; i < 2; ++i)
            ptx::tma_load_2d(ssfb + i * 2048, &tmap_sfb, 0, ((n_blk * 2 + i) * p.rk + 4 * kt) * 2, sbar);
          if (rank == 0) ptx::mbar_expect_tx(full_bar(st.stage), 2 * (kABytes + kBBytes));
          ptx::tma2_load_2d(sa, &tmap_a, kt * 128, m_tile * 128, bar);
          ptx::tma2_load_3d(sb, &tmap_b, kt * 128, n_blk * 256 + static_cast<int>(rank) * 128, 0, bar);
          st.advance(kStages);
        }
      }
    }
  } else if (warp == 1) {
    // =============================== MMA issuer (even CTA only) ===============================
    // the whole warp walks the loop, an elected lane issues (see the single-CTA kernel)
    if (rank == 0) {
      PipeState st;
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint64_t a_desc0 = ptx::smem_desc_sw128(smem_base);
      const uint64_t b_desc0 = ptx::smem_desc_sw128(smem_base + kABytes);
      const int last_kblocks = ((p.k_bytes - (p.num_k_tiles - 1) * 128) + 31) >> 5;
      B200_ACCT(MmaAcct acct; acct.start();)
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        B200_ACCT(acct.skip();)
        if (!wait_bounded(acc_empty_bar, acc_phase ^ 1u, abort_flag)) {
          if (lane == 0) atomicOr(p.status, kStatusTimeoutMma);
          break;
        }
        B200_ACCT(acct.mark(acct.acc); ++acct.tiles;)
        ptx::tc_fence_after_sync();
        for (int kt = 0; kt < p.num_k_tiles; ++kt) {
#ifdef B200FP4_ACCT
          acct.skip();
          wait_bounded(full_bar(st.stage), st.phase, abort_flag);
          acct.mark(acct.full);
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
          const uint64_t stage_off = static_cast<uint64_t>(st.stage * (kPairStageBytes >> 4));
          const uint64_t da = a_desc0 + stage_off, db = b_desc0 + stage_off;
          const uint32_t sfa_t = tmem_base + kSfaCol + st.stage * kSfSetCols;
          const uint32_t sfb_t = sfa_t + 16;
          const int kblocks = kt + 1 == p.num_k_tiles ? last_kblocks : 4;
          if (ptx::elect_one()) {
            ptx::mma2_mxf4nvf4(tmem_base, da, db, kIdesc, sfa_t, sfb_t, kt != 0 ? 1u : 0u);
#pragma unroll
            for (int kb = 1; kb < 4; ++kb) {
              if (kb < kblocks)
                ptx::mma2_mxf4nvf4(tmem_base, da + 2 * kb, db + 2 * kb, kIdesc, sfa_t + 4 * kb, sfb_t + 8 * kb, 1u);
            }
            ptx::tc2_commit_mcast(empty_bar(st.stage), 3);      // frees the stage in both CTAs
          }
          __syncwarp();
          B200_ACCT(acct.mark(acct.issue);)
          st.advance(kStages);
        }
        if (ok && ptx::elect_one()) ptx::tc2_commit_mcast(acc_full_bar, 3);   // accumulators of both CTAs are complete
        __syncwarp();
        acc_phase ^= 1u;
      }
#ifdef B200FP4_ACCT
      if (lane == 0 && (pair == 3 || pair == 50))
        printf("acct pair %d: tiles %d ksteps %d cycles %lld = accumulator wait %lld + operand wait %lld + slab wait %lld + "
               "issue %lld + other\n",
               pair, acct.tiles, acct.ksteps, clock64() - acct.begin, acct.acc, acct.full, acct.sf, acct.issue);
#endif
    }
  } else if (warp >= 10) {
    // =============================== scale-slab movers (both CTAs) ===============================
    // (A second group of four mover warps taking every other K step changed nothing: the slabs are late because
    // the stage's bytes are, not because one group cannot keep up.)
    const int quarter = warp & 3;
    PipeState st;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      for (int kt = 0; kt < p.num_k_tiles; ++kt) {
        if (!wait_bounded(sf_loaded_bar(st.stage), st.phase, abort_flag)) {
          if (lane == 0) atomicOr(p.status, kStatusTimeoutMma);
          ok = false;
          break;
        }
        const uint8_t* slab = smem_gen + st.stage * kPairStageBytes + kABytes + kBBytes + lane * 16;
        const uint32_t t_sf = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kSfaCol + st.stage * kSfSetCols;
        uint32_t ra[16];
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
          const uint4 v = *reinterpret_cast<const uint4*>(slab + 512 * kb);
          ra[4 * kb] = v.x, ra[4 * kb + 1] = v.y, ra[4 * kb + 2] = v.z, ra[4 * kb + 3] = v.w;
        }
        ptx::tmem_st_32x16(t_sf, ra);
        uint32_t rb[32];
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const uint4 v = *reinterpret_cast<const uint4*>(slab + kSfaBytes + 2048 * i + 512 * kb);
            rb[8 * kb + 4 * i] = v.x, rb[8 * kb + 4 * i + 1] = v.y, rb[8 * kb + 4 * i + 2] = v.z,
                        rb[8 * kb + 4 * i + 3] = v.w;
          }
        }
        ptx::tmem_st_32x32(t_sf + 16, rb);
        ptx::tmem_st_wait();
        ptx::tc_fence_before_sync();
        __syncwarp();
        // The slabs are in tensor memory (tcgen05.wait::st returned) before the arrive is issued.  The odd CTA
        // signals with a relaxed arrive: one with cluster-scope release stalls its thread for 300 to 2000
        // cycles under load, and there is no memory write here for a release to order.
        if (lane == 0) {
          if (rank == 0) ptx::mbar_arrive(sf_full_bar(st.stage));
          else ptx::mbar_arrive_cluster_relaxed(sf_full_bar(st.stage) & ptx::kPeerBitMask);
        }
        st.advance(kStages);
      }
    }
  } else {
    // =============================== epilogue (both CTAs) ===============================
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    uint32_t acc_phase = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs) {
      const int m2 = tile % p.num_m_blocks;
      const int n_blk = tile / p.num_m_blocks;
      if (!wait_bounded<64>(acc_full_bar, acc_phase, abort_flag)) {
        if (lane == 0) atomicOr(p.status, kStatusTimeoutEpilogue);
        break;
      }
      ptx::tc_fence_after_sync();
      const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      epi.template operator()<kBlockN>(p, 2 * m2 + static_cast<int>(rank), n_blk, 0, row, kBlockM, part, 2,
                                       [&](int c0, uint32_t (&r)[32]) {
                                         ptx::tmem_ld_32x32(t_acc + c0, r);
                                         ptx::tmem_ld_wait();
                                       },
                                       [&]() {      // called once the warp has read its share of the accumulator
                                         ptx::tc_fence_before_sync();
                                         __syncwarp();
                                         if (lane == 0) {
                                           if (rank == 0) ptx::mbar_arrive(acc_empty_bar);
                                           else ptx::mbar_arrive_cluster_relaxed(acc_empty_bar & ptx::kPeerBitMask);   // tcgen05.wait::ld has returned
                                         }
                                       });
      acc_phase ^= 1u;
    }
  }

  // ---- teardown: nobody leaves while the peer may still signal this CTA or read its memory
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::cluster_sync();
  if (warp == 0) {
    if (*abort_flag) {
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    __syncwarp();
    ptx::tc_fence_after_sync();
    ptx::tmem2_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace b200fp4
