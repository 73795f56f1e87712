// CTA-pair version of the fused NF4 GEMM: two CTAs of a cluster (two SMs) compute one
// (BM_TILES x 256) x 256 output tile with tcgen05.mma.cta_group::2.
//
// Each CTA owns 128 of every 256 accumulator rows (in its own tensor memory) and HALF of the 256
// weight rows of the tile: it loads its own activation rows by TMA and dequantises only its 128
// quantisation blocks per stage; the pair's MMA (issued by the CTA of rank 0) reads the A rows and
// the B half out of both CTAs' shared memory. Compared with the single-CTA kernel this halves the
// decode work and the B-operand shared-memory traffic per FLOP, and the smaller B ring leaves room
// for a deeper activation ring. Nothing is multicast except tcgen05.commit's mbarrier arrive.
//
// Synchronisation between the two CTAs uses mbarriers only (every wait bounded): the rank-1 CTA's
// MMA warp relays "my stage s is loaded and dequantised" to the stage barrier of the rank-0 CTA with a
// remote arrive; rank 0 frees stages / publishes the accumulator to both CTAs with a multicast commit.
#include "nf4ll_gemm_shared.cuh"

namespace nf4ll {

template <int BM_TILES>
struct PairCfg {
  static constexpr int kStages = (BM_TILES == 2) ? 4 : 6;
  static constexpr int kDequantWarps = 8;                 // two teams of 128 threads on alternate stages, one block per thread
  static constexpr int kThreads = 32 * (4 + kDequantWarps);
  static constexpr int kABytes = BM_TILES * 128 * 128;    // per stage: this CTA's 128 rows x 64 fp16 per accumulator
  static constexpr int kBBytes = 128 * 128;               // per stage: this CTA's 128 dequantised blocks
  static constexpr int kNibBytes = 128 * 32;
  static constexpr int kAbsBytes = 128 * 4;
  static constexpr int kLoraLeftBytes = BM_TILES * 128 * 32;
  static constexpr int kLoraRightBytes = 128 * 32;
  static constexpr int kTmemCols = BM_TILES * 256;
  static constexpr int kRingBytes = kStages * (kABytes + kBBytes);
  static constexpr int kSmemBytes = 1024 + kStages * (kABytes + kBBytes + kNibBytes + kAbsBytes) + 1024 + 512;
  static_assert(kLoraLeftBytes + kLoraRightBytes <= kBBytes, "LoRA operands must fit one weight stage");
  static_assert(kRingBytes >= kFixSlots * 16384, "fix-up ring must fit the operand rings");
};

// --- cluster / cta_group::2 PTX ---------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// For single-thread roles waiting on something the OTHER CTA signals (a remote arrive, a multicast
// commit): poll without the hardware's suspended wait, whose wake-up on remote arrivals is slow.
__device__ __forceinline__ bool wait_cluster_or_abort(uint32_t bar, uint32_t parity, const Abort& ab, int code) {
  for (uint32_t i = 0; i < (kSpinLimit << 4); ++i) {
    if (mbar_test_wait_cluster(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *ab.flag) return false;
  }
  ab.raise(code);
  return false;
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrive on the barrier at the same shared-memory offset in BOTH CTAs once this thread's MMAs are done
__device__ __forceinline__ void tc_commit2(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(static_cast<uint16_t>(3)) : "memory");
}
__device__ __forceinline__ void tc_mma2_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int MODE, int BM_TILES>
__global__ void __launch_bounds__(PairCfg<BM_TILES>::kThreads, 1)
nf4_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_act, const __grid_constant__ CUtensorMap tmap_nib,
                     const __grid_constant__ CUtensorMap tmap_out, const GemmParams p) {
  using Cfg = PairCfg<BM_TILES>;
  constexpr int S = Cfg::kStages;
  constexpr int NDW = Cfg::kDequantWarps;
  constexpr int BN = 256;                       // tile columns of the pair; this CTA dequantises 128 of them

  pdl_wait();                  // everything below may read what the previous kernel on the stream wrote
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;                                   // [S][BM_TILES][128 rows][128 B]
  uint8_t* sB = sA + S * Cfg::kABytes;                  // [S][128 blocks][128 B]
  uint8_t* sNib = sB + S * Cfg::kBBytes;                // [S][128 blocks][32 B]
  uint8_t* sAbs = sNib + S * Cfg::kNibBytes;            // [S][128] fp32
  float* sCode2 = reinterpret_cast<float*>(sAbs + S * Cfg::kAbsBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sCode2) + 1024);
  uint8_t* sLL = sB + (S - 1) * Cfg::kBBytes;           // LoRA operands borrow the last weight-tile stage
  uint8_t* sLR = sLL + Cfg::kLoraLeftBytes;
  // [S] this CTA's stage is ready: activation boxes landed (producer arrive + bytes), blocks dequantised
  // (one arrive per warp of the stage's team) and, in rank 0, the relayed arrive of rank 1's own barrier
  uint64_t* full_a = bars;
  uint64_t* full_b = full_a;
  uint64_t* empty = bars + 2 * S;       // [S] the pair's MMAs on the stage are done (multicast commit)
  uint64_t* nib_full = bars + 3 * S;    // [S]
  uint64_t* nib_empty = bars + 4 * S;   // [S]
  uint64_t* lora_full = bars + 6 * S;
  uint64_t* acc_full = lora_full + 1;
  uint64_t* pre_full = lora_full + 2;
  uint64_t* pre_done = lora_full + 3;
  uint64_t* lora_done = lora_full + 4;
  uint64_t* fix_go = lora_full + 5;
  uint64_t* peer_lora = lora_full + 6;  // rank 0 only: rank 1's LoRA operands are staged
  uint64_t* peer_pre = lora_full + 7;   // rank 0 only: rank 1 has masked its half of the accumulator
  uint64_t* fx_full = lora_full + 8;
  uint64_t* fx_empty = fx_full + kFixSlots;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(fx_empty + kFixSlots);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = abort_flag + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();            // 0 issues the pair's MMAs
  const int tile_o = blockIdx.x >> 1, tile_m = blockIdx.y, split = blockIdx.z;
  const int tiles_o = gridDim.x >> 1;
  // accumulator mt of this CTA covers rows m0 + mt*256 .. +127 and all 256 tile columns
  const int64_t m0 = static_cast<int64_t>(tile_m) * (BM_TILES * 256) + rank * 128;
  const int64_t o0 = static_cast<int64_t>(tile_o) * BN;
  const int64_t oh = o0 + rank * 128;                 // first of the 128 weight rows / columns this CTA dequantises

  const int nkb_total = static_cast<int>(p.KC / 64);
  const int kb_begin = static_cast<int>(static_cast<int64_t>(nkb_total) * split / p.splits);
  const int kb_end = static_cast<int>(static_cast<int64_t>(nkb_total) * (split + 1) / p.splits);
  const int nkb = kb_end - kb_begin;
  const bool lora_here = p.has_lora && split == 0;
  const bool premask = lora_here && MODE == kBwd && p.mask != nullptr;

  const Abort ab{abort_flag, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(full_a + s), 1 + NDW / 2 + (rank == 0 ? 1 : 0));
      mbar_init(smem_u32(empty + s), 1);
      mbar_init(smem_u32(nib_full + s), 3);
      mbar_init(smem_u32(nib_empty + s), NDW / 2);
    }
    mbar_init(smem_u32(lora_full), NDW);
    mbar_init(smem_u32(acc_full), 1);
    mbar_init(smem_u32(pre_full), 1);
    mbar_init(smem_u32(pre_done), NDW);
    mbar_init(smem_u32(lora_done), 1);
    mbar_init(smem_u32(fix_go), 1);
    mbar_init(smem_u32(peer_lora), 1);
    mbar_init(smem_u32(peer_pre), 1);
    for (int i = 0; i < kFixSlots; ++i) {
      mbar_init(smem_u32(fx_full + i), 1);
      mbar_init(smem_u32(fx_empty + i), p.coop ? 4 : NDW);   // a slot is read by one warp group (shared reduction) or by all
    }
    *abort_flag = 0;
    *last_flag = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < 256) sCode2[threadIdx.x] = p.code2[threadIdx.x];
  if (warp == 1) {
    tmem_alloc2(smem_u32(tmem_slot), Cfg::kTmemCols);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncwarp();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers exist before anybody arrives remotely or multicasts
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ----------------------------------------------------------------------------- TMA producer (own rows, own half)
    if (lane == 0) {
      tma_prefetch_desc(&tmap_act);
      tma_prefetch_desc(&tmap_nib);
      int issued = 0;
      for (int i = 0; i < nkb; ++i, ++issued) {
        const int s = i % S;
        const uint32_t free_parity = ((i / S) & 1) ^ 1;
        const int kb = kb_begin + i;
        if (!wait_or_abort(smem_u32(nib_empty + s), free_parity, ab, 0x0102)) break;
        mbar_arrive_expect_tx(smem_u32(nib_full + s), Cfg::kNibBytes);
        if (MODE == kFwd) {
          tma_load_2d(smem_u32(sNib + s * Cfg::kNibBytes), &tmap_nib, kb * 32, static_cast<int>(oh), smem_u32(nib_full + s));
        } else {
          tma_load_2d(smem_u32(sNib + s * Cfg::kNibBytes), &tmap_nib, static_cast<int>(oh / 2), kb * 64, smem_u32(nib_full + s));
        }
        if (!wait_cluster_or_abort(smem_u32(empty + s), free_parity, ab, 0x0101)) break;
        mbar_arrive_expect_tx(smem_u32(full_a + s), Cfg::kABytes);
#pragma unroll
        for (int mt = 0; mt < BM_TILES; ++mt) {
          tma_load_2d(smem_u32(sA + s * Cfg::kABytes + mt * 16384), &tmap_act, kb * 64,
                      static_cast<int>(m0 + mt * 256), smem_u32(full_a + s));
        }
      }
      if (p.splits > 1 && !*abort_flag) {
        if (wait_or_abort(smem_u32(fix_go), 0, ab, 0x0104) && p.coop && !*abort_flag) {
          // shared reduction (see the single-CTA kernel): stream the other splits' partial sums of the boxes this CTA owns
          fence_proxy_async_all();
          constexpr int NB = BM_TILES * (BN / 32);
          // the boxes go to the warp groups in turn and every group has its own share of the ring's slots:
          // a slot is then always filled for, and drained by, the same group, in order
          constexpr int G = NDW / 4, SPG = kFixSlots / G;
          int cnt0 = 0, cnt1 = 0, mine = 0;
          bool fine = true;
          for (int b = split; fine && b < NB; b += p.splits) {
            const int mt = b / (BN / 32), cb = b % (BN / 32);
            const int64_t col0 = o0 + cb * 32;
            if (col0 >= p.NO) continue;
            const int grp = (mine++) % G;
            for (int sp = 0; sp < p.splits; ++sp) {
              if (sp == split) continue;
              const int nn = grp ? cnt1 : cnt0;
              const int slot = grp * SPG + nn % SPG;
              if (!wait_or_abort(smem_u32(fx_empty + slot), ((nn / SPG) & 1) ^ 1, ab, 0x0105)) { fine = false; break; }
              if (grp) ++cnt1; else ++cnt0;
              mbar_arrive_expect_tx(smem_u32(fx_full + slot), 16384);
              tma_load_2d(smem_u32(smem) + slot * 16384, &tmap_out, static_cast<int>(col0),
                          static_cast<int>(static_cast<int64_t>(sp) * p.m_pad + m0 + mt * 256), smem_u32(fx_full + slot));
            }
          }
        } else if (!p.coop && *last_flag) {
          fence_proxy_async_all();
          int n = 0;
          bool fine = true;
          for (int mt = 0; fine && mt < BM_TILES; ++mt) {
            for (int cb = 0; fine && cb < BN / 32; ++cb) {
              const int64_t col0 = o0 + cb * 32;
              if (col0 >= p.NO) break;
              for (int sp = 0; sp < p.splits; ++sp, ++n) {
                const int slot = n % kFixSlots;
                if (!wait_or_abort(smem_u32(fx_empty + slot), ((n / kFixSlots) & 1) ^ 1, ab, 0x0105)) { fine = false; break; }
                mbar_arrive_expect_tx(smem_u32(fx_full + slot), 16384);
                tma_load_2d(smem_u32(smem) + slot * 16384, &tmap_out, static_cast<int>(col0),
                            static_cast<int>(static_cast<int64_t>(sp) * p.m_pad + m0 + mt * 256), smem_u32(fx_full + slot));
              }
            }
          }
        }
      }
      if (*abort_flag) {
        for (int i = (issued > S ? issued - S : 0); i <= issued && i < nkb; ++i) {
          const uint32_t ph = (i / S) & 1;
          for (int spin = 0; spin < (1 << 16) && !mbar_try_wait(smem_u32(full_a + (i % S)), ph); ++spin) {}
          for (int spin = 0; spin < (1 << 16) && !mbar_try_wait(smem_u32(nib_full + (i % S)), ph); ++spin) {}
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank != 0) {
      // ----------------------------------------------------------------------------- rank 1: relay readiness to rank 0
      bool ok = true;
      if (lora_here) {
        ok = wait_or_abort(smem_u32(lora_full), 0, ab, 0x0211);
        if (ok) mbar_arrive_remote(map_to_cta(smem_u32(peer_lora), 0));
        if (ok && premask) {
          ok = wait_or_abort(smem_u32(pre_done), 0, ab, 0x0212);
          if (ok) mbar_arrive_remote(map_to_cta(smem_u32(peer_pre), 0));
        }
      }
      for (int i = 0; ok && i < nkb; ++i) {
        const int s = i % S;
        const uint32_t ph = (i / S) & 1;
        if (!wait_or_abort(smem_u32(full_a + s), ph, ab, 0x0213)) {
          ok = false;
          break;
        }
        mbar_arrive_remote(map_to_cta(smem_u32(full_a + s), 0));
      }
    } else if (lane == 0) {
      // ----------------------------------------------------------------------------- rank 0: the pair's MMA issuer
      constexpr uint32_t idesc_main = make_idesc_f16(256, BN, 0, MODE == kBwd ? 1 : 0);
      bool ok = true;
      if (lora_here) {
        ok = wait_or_abort(smem_u32(lora_full), 0, ab, 0x0201) && wait_cluster_or_abort(smem_u32(peer_lora), 0, ab, 0x0205);
        if (ok) {
          tc_fence_after();
          const uint64_t rdesc = make_smem_desc(smem_u32(sLR), 128, 256, kSwizzleNone);
#pragma unroll
          for (int mt = 0; mt < BM_TILES; ++mt) {
            const uint64_t ldesc = make_smem_desc(smem_u32(sLL + mt * 4096), 128, 256, kSwizzleNone);
            tc_mma2_f16(tmem_base + mt * BN, ldesc, rdesc, idesc_main, 0u);
          }
          tc_commit2(smem_u32(lora_done));
          if (premask) {
            tc_commit2(smem_u32(pre_full));
            ok = wait_or_abort(smem_u32(pre_done), 0, ab, 0x0202) && wait_cluster_or_abort(smem_u32(peer_pre), 0, ab, 0x0206);
            if (ok) tc_fence_after();
          }
        }
      }
      for (int i = 0; ok && i < nkb; ++i) {
        const int s = i % S;
        const uint32_t ph = (i / S) & 1;
        if (!wait_cluster_or_abort(smem_u32(full_a + s), ph, ab, 0x0203)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_base = smem_u32(sA + s * Cfg::kABytes);
        const uint32_t b_base = smem_u32(sB + s * Cfg::kBBytes);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          // each CTA supplies 128 of the 256 B rows: K-major 128 x 64 (forward), or two 64 x 64 MN-major sub-tiles
          const uint64_t bdesc = (MODE == kFwd)
                                     ? make_smem_desc(b_base + kk * 32, 16, 1024, kSwizzle128B)
                                     : make_smem_desc(b_base + kk * 2048, 8192, 1024, kSwizzle128B);
#pragma unroll
          for (int mt = 0; mt < BM_TILES; ++mt) {
            const uint64_t adesc = make_smem_desc(a_base + mt * 16384 + kk * 32, 16, 1024, kSwizzle128B);
            tc_mma2_f16(tmem_base + mt * BN, adesc, bdesc, idesc_main, (lora_here || i > 0 || kk > 0) ? 1u : 0u);
          }
        }
        tc_commit2(smem_u32(empty + s));
      }
      tc_commit2(smem_u32(acc_full));
      if (!ok) {
        for (int spin = 0; spin < (1 << 18) && !mbar_try_wait(smem_u32(acc_full), 0); ++spin) {}
      }
    }
  } else if (warp < 4) {
    // ----------------------------------------------------------------------------- absmax helper
    {
      constexpr int PER = 2;                       // 128 blocks over 64 helper threads
      const int t = threadIdx.x - 64;
      int64_t qb[PER], qstep;
#pragma unroll
      for (int e = 0; e < PER; ++e) {
        const int d = t + e * 64;
        if (MODE == kFwd) {
          int64_t n = oh + d;
          if (n >= p.N) n = p.N - 1;
          qb[e] = (n * p.K) / 64 + kb_begin;
        } else {
          const int j = d % 2, r = d / 2;
          int64_t kcol = oh + j * 64;
          if (kcol >= p.K) kcol = 0;
          qb[e] = ((static_cast<int64_t>(kb_begin) * 64 + r) * p.K + kcol) / 64;
        }
      }
      qstep = (MODE == kFwd) ? 1 : p.K;
      uint32_t qc[PER];
      float s2[PER], o2[PER];
#pragma unroll
      for (int e = 0; e < PER; ++e) {
        qc[e] = 0; s2[e] = 0.f; o2[e] = 0.f;
        if (nkb > 0) { qc[e] = __ldg(p.qabs + qb[e]); s2[e] = __ldg(p.scale2 + (qb[e] >> 8)); o2[e] = __ldg(p.offset2 + (qb[e] >> 8)); }
      }
      for (int i = 0; i < nkb; ++i) {
        const int s = i % S;
        uint32_t nq[PER];
        float ns2[PER], no2[PER];
#pragma unroll
        for (int e = 0; e < PER; ++e) {
          nq[e] = qc[e]; ns2[e] = s2[e]; no2[e] = o2[e];
          if (i + 1 < nkb) {
            const int64_t nb = qb[e] + qstep;
            nq[e] = __ldg(p.qabs + nb); ns2[e] = __ldg(p.scale2 + (nb >> 8)); no2[e] = __ldg(p.offset2 + (nb >> 8));
          }
        }
        if (!wait_or_abort(smem_u32(nib_empty + s), ((i / S) & 1) ^ 1, ab, 0x0401)) break;
        float* dst = reinterpret_cast<float*>(sAbs + s * Cfg::kAbsBytes);
#pragma unroll
        for (int e = 0; e < PER; ++e) dst[t + e * 64] = block_absmax(sCode2[qc[e]], s2[e], o2[e]);
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(nib_full + s));
#pragma unroll
        for (int e = 0; e < PER; ++e) { qc[e] = nq[e]; s2[e] = ns2[e]; o2[e] = no2[e]; qb[e] += qstep; }
      }
    }
  } else {
    // ----------------------------------------------------------------------------- dequant, then epilogue
    const int d = threadIdx.x - 128;      // 0..255: half a quantisation block per stage
    const int ew = warp - 4;
    const int q = warp & 3;
    bool ok = true;

    // --- LoRA operands: staged by these warps while the first weight codes are still on their way
    // (all loads issued before the first store: one trip to memory)
    if (lora_here) {
      constexpr int NT = NDW * 32;
      constexpr int LEFT = BM_TILES * 128 * 2;         // 16-byte chunks (8 fp16) of this CTA's left operand rows
      constexpr int RIGHT = 128 * 2;                   // this CTA's 128 rows of B[N,16] / 128 columns of A[16,K]
      constexpr int LPT = (LEFT + NT - 1) / NT, RPT = (RIGHT + NT - 1) / NT;
      float4 la[LPT], lb[LPT];
      uint4 rv[RPT];
#pragma unroll
      for (int e = 0; e < LPT; ++e) {
        const int c = d + e * NT, row = c >> 1, h = c & 1;
        const int mt = row >> 7, r = row & 127;
        const int64_t grow = m0 + mt * 256 + r;
        la[e] = make_float4(0.f, 0.f, 0.f, 0.f); lb[e] = la[e];
        if (c < LEFT && grow < p.M) {
          const float4* src = reinterpret_cast<const float4*>(p.lora_left + grow * 16 + h * 8);
          la[e] = __ldg(src); lb[e] = __ldg(src + 1);
        }
      }
#pragma unroll
      for (int e = 0; e < RPT; ++e) {
        const int c = d + e * NT;
        rv[e] = make_uint4(0, 0, 0, 0);
        if (MODE == kFwd) {
          const int row = c >> 1, h = c & 1;
          if (c < RIGHT && oh + row < p.NO) rv[e] = __ldg(reinterpret_cast<const uint4*>(p.lora_right + (oh + row) * 16 + h * 8));
        } else {
          const int j = c / 16, c8 = c % 16;
          if (c < RIGHT && oh + c8 * 8 < p.NO) rv[e] = __ldg(reinterpret_cast<const uint4*>(p.lora_right + j * p.K + oh + c8 * 8));
        }
      }
#pragma unroll
      for (int e = 0; e < LPT; ++e) {
        const int c = d + e * NT, row = c >> 1, h = c & 1;
        if (c < LEFT) {
          uint4 v;
          v.x = pack_half2_rn(la[e].x * p.left_scale, la[e].y * p.left_scale);
          v.y = pack_half2_rn(la[e].z * p.left_scale, la[e].w * p.left_scale);
          v.z = pack_half2_rn(lb[e].x * p.left_scale, lb[e].y * p.left_scale);
          v.w = pack_half2_rn(lb[e].z * p.left_scale, lb[e].w * p.left_scale);
          const int mt = row >> 7, r = row & 127;
          *reinterpret_cast<uint4*>(sLL + mt * 4096 + (r >> 3) * 256 + h * 128 + (r & 7) * 16) = v;
        }
      }
#pragma unroll
      for (int e = 0; e < RPT; ++e) {
        const int c = d + e * NT;
        if (c < RIGHT) {
          if (MODE == kFwd) {
            const int row = c >> 1, h = c & 1;
            *reinterpret_cast<uint4*>(sLR + (row >> 3) * 256 + h * 128 + (row & 7) * 16) = rv[e];
          } else {
            const int j = c / 16, c8 = c % 16;
            *reinterpret_cast<uint4*>(sLR + c8 * 256 + (j >> 3) * 128 + (j & 7) * 16) = rv[e];
          }
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(lora_full));
    }

    // --- dequantise: two teams of four warps take alternate stages, one block per thread (see the
    // single-CTA kernel for why the teams alternate)
    const int team = d >> 7, blk = d & 127;
    uint32_t nib_off, row_off;
    int key;
    if (MODE == kFwd) {
      nib_off = blk * 32;
      row_off = blk * 128;
      key = blk & 7;
    } else {
      const int j = blk % 2, r = blk / 2;
      nib_off = r * 64 + j * 32;
      row_off = j * 8192 + r * 128;
      key = r & 7;
    }
    const uint32_t nib_base = smem_u32(sNib) + nib_off, abs_base = smem_u32(sAbs) + blk * 4, b_base = smem_u32(sB) + row_off;
    auto dequant_stage = [&](int i) -> bool {
      const int s = i % S;
      const uint32_t ph = (i / S) & 1;
      if (!wait_or_abort(smem_u32(nib_full + s), ph, ab, 0x0304)) return false;
      const uint4 c0 = lds128(nib_base + s * Cfg::kNibBytes), c1 = lds128(nib_base + s * Cfg::kNibBytes + 16);
      const float absmax = lds_f32(abs_base + s * Cfg::kAbsBytes);
      if (!wait_or_abort(smem_u32(empty + s), ph ^ 1, ab, 0x0302)) return false;
      // the last stage holds the LoRA operands until the rank-16 MMAs have read them
      if (lora_here && i == S - 1 && !wait_or_abort(smem_u32(lora_done), 0, ab, 0x0305)) return false;
      dequant_block_to_smem(b_base + s * Cfg::kBBytes, key, c0, c1, absmax);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(full_b + s));
        mbar_arrive(smem_u32(nib_empty + s));
      }
      return true;
    };

    int i_next = team;
    if (premask) {
      // scale the LoRA product in the accumulator by keep_scale * mask before the base GEMM lands on it;
      // each team dequantises its first stage and the first mask bytes travel while the rank-16 MMAs run
      constexpr int kChunks = BM_TILES * (BN / 32);
      constexpr int kStep = NDW / 4;
      auto load_mask = [&](int u, uint4& a, uint4& b) {
        a = make_uint4(0, 0, 0, 0); b = a;
        if (u < kChunks) {
          const int mt = u / (BN / 32), c = u % (BN / 32);
          const int64_t row = m0 + mt * 256 + q * 32 + lane;
          const int64_t col0 = o0 + c * 32;
          if (row < p.M && col0 < p.NO) {
            const uint4* mp = reinterpret_cast<const uint4*>(p.mask + row * p.ld_mask + col0);
            a = __ldg(mp); b = __ldg(mp + 1);
          }
        }
      };
      uint4 ma, mb;
      load_mask(ew >> 2, ma, mb);
      if (i_next < nkb && i_next < S - 1) {
        ok = dequant_stage(i_next);
        i_next += 2;
      }
      if (ok) ok = wait_or_abort(smem_u32(pre_full), 0, ab, 0x0301);
      if (ok) {
        tc_fence_after();
        for (int u = ew >> 2; u < kChunks; u += kStep) {
          const int mt = u / (BN / 32), c = u % (BN / 32);
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + mt * BN + c * 32;
          uint32_t v[32];
          __syncwarp();
          tmem_ld32(taddr, v);
          uint4 na, nb;
          load_mask(u + kStep, na, nb);
          tmem_ld_wait();
          const uint32_t mk[8] = {ma.x, ma.y, ma.z, ma.w, mb.x, mb.y, mb.z, mb.w};
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const bool keep = ((mk[j >> 2] >> ((j & 3) * 8)) & 0xffu) != 0;
            v[j] = keep ? __float_as_uint(__uint_as_float(v[j]) * p.keep_scale) : 0u;
          }
          tmem_st32(taddr, v);
          ma = na; mb = nb;
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(pre_done));
      }
    }
    for (int i = i_next; ok && i < nkb; i += 2) ok = dequant_stage(i);

    // --- epilogue: tensor memory -> registers -> swizzled shared staging -> TMA store (see the single-CTA kernel)
    if (ok) ok = wait_or_abort(smem_u32(acc_full), 0, ab, 0x0303);
    const bool direct = (p.splits == 1);
    if (ok) {
      tc_fence_after();
      constexpr int G = NDW / 4;
      constexpr int HALVES = BN / 128;
      const int grp = ew >> 2;
      const int bar_id = 2 + grp;
      const uint32_t stage = smem_u32(smem) + grp * 32768;
      const int r_in = q * 32 + lane;
      const uint32_t row_addr = stage + r_in * 128;
      const int key2 = r_in & 7;
      const bool leader = (q == 0 && lane == 0);
      if (!direct && p.coop) {
        // shared reduction, first half (see the single-CTA kernel): boxes owned by other splits go to this split's slab
        constexpr int NB = BM_TILES * (BN / 32);
        constexpr int SB = 4;
        const uint32_t stage4 = smem_u32(smem) + grp * 65536;
        const uint32_t row_addr4 = stage4 + r_in * 128;
        int f = 0, pending = 0;
        uint32_t staged = 0;
        auto flush = [&]() {
          fence_proxy_async_smem();
          named_barrier(bar_id, 128);
          if (leader) {
            for (int k = 0; k < pending; ++k) {
              const int b = (staged >> (8 * k)) & 0xff;
              const int mt = b / (BN / 32), cb = b % (BN / 32);
              const int64_t col0 = o0 + cb * 32;
              if (col0 < p.NO)
                tma_store_2d(&tmap_out, stage4 + k * 16384, static_cast<int>(col0),
                             static_cast<int>(static_cast<int64_t>(split) * p.m_pad + m0 + mt * 256));
            }
            bulk_commit();
            bulk_wait_read_all();
          }
          named_barrier(bar_id, 128);
          pending = 0; staged = 0;
        };
#pragma unroll 1
        for (int b = 0; b < NB; ++b) {
          if (b % p.splits == split) continue;
          const int round = f / SB;
          ++f;
          if (round % G != grp) continue;
          const int mt = b / (BN / 32), cb = b % (BN / 32);
          uint32_t v[32];
          __syncwarp();
          tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + mt * BN + cb * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            sts128(row_addr4 + pending * 16384 + ((j ^ key2) << 4), make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
          staged |= static_cast<uint32_t>(b) << (8 * pending);
          if (++pending == SB) flush();
        }
        if (pending) flush();
      }
      // plain paths: the whole accumulator goes out as fp16 (no split) or as this split's fp32 slab
      const bool plain = direct || !p.coop;
      for (int u = grp; plain && u < BM_TILES * HALVES; u += G) {
        const int mt = u / HALVES, ch = u % HALVES;
        const uint32_t tacc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + mt * BN + ch * 128;
        const int row_g = static_cast<int>(m0 + mt * 256);
        const int64_t colh = o0 + ch * 128;
        if (direct) {
#pragma unroll 1
          for (int cb = 0; cb < 2; ++cb) {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              const int c = cb * 2 + hh;
              const int64_t col0 = colh + c * 32;
              uint32_t v[32];
              __syncwarp();
              tmem_ld32(tacc + c * 32, v);
              tmem_ld_wait();
#pragma unroll
              for (int g8 = 0; g8 < 4; ++g8) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[g8 * 8 + j]);
                if (MODE == kFwd && p.bias && col0 < p.NO) {
                  const uint4 bb = __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + g8 * 8));
                  const __half2* bh = reinterpret_cast<const __half2*>(&bb);
#pragma unroll
                  for (int j = 0; j < 4; ++j) { const float2 bf = __half22float2(bh[j]); f[2 * j] += bf.x; f[2 * j + 1] += bf.y; }
                }
                uint4 o;
                o.x = pack_half2_rn(f[0], f[1]); o.y = pack_half2_rn(f[2], f[3]);
                o.z = pack_half2_rn(f[4], f[5]); o.w = pack_half2_rn(f[6], f[7]);
                sts128(row_addr + cb * 16384 + (((hh * 4 + g8) ^ key2) << 4), o);
              }
            }
          }
          fence_proxy_async_smem();
          named_barrier(bar_id, 128);
          if (leader) {
            for (int cb = 0; cb < 2; ++cb) {
              const int64_t col0 = colh + cb * 64;
              if (col0 >= p.NO) break;
              if (MODE == kBwd && p.accumulate) tma_reduce_add_2d(&tmap_out, stage + cb * 16384, static_cast<int>(col0), row_g);
              else tma_store_2d(&tmap_out, stage + cb * 16384, static_cast<int>(col0), row_g);
            }
            bulk_commit();
            bulk_wait_read_all();
          }
          if (u + G < BM_TILES * HALVES) named_barrier(bar_id, 128);
        } else {
          const int slab_row = static_cast<int>(static_cast<int64_t>(split) * p.m_pad + m0 + mt * 256);
#pragma unroll 1
          for (int round = 0; round < 2; ++round) {
#pragma unroll 1
            for (int b2 = 0; b2 < 2; ++b2) {
              const int c = round * 2 + b2;
              uint32_t v[32];
              __syncwarp();
              tmem_ld32(tacc + c * 32, v);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 8; ++j)
                sts128(row_addr + b2 * 16384 + ((j ^ key2) << 4), make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
            }
            fence_proxy_async_smem();
            named_barrier(bar_id, 128);
            if (leader) {
              for (int b2 = 0; b2 < 2; ++b2) {
                const int64_t col0 = colh + (round * 2 + b2) * 32;
                if (col0 >= p.NO) break;
                tma_store_2d(&tmap_out, stage + b2 * 16384, static_cast<int>(col0), slab_row);
              }
              bulk_commit();
              bulk_wait_read_all();
            }
            named_barrier(bar_id, 128);
          }
        }
      }
      if (!direct && leader) {
        bulk_wait_all();
        fence_proxy_async_all();
        __threadfence();
      }
    }
    if (!direct && p.coop) {
      // shared reduction, second half (see the single-CTA kernel)
      __threadfence();
      named_barrier(1, NDW * 32);
      if (d == 0) {
        int* counter = p.counters + ((static_cast<int64_t>(tile_m) * tiles_o + tile_o) * 2 + rank);
        __threadfence();
        atomicAdd(counter, 1);
        bool seen = false;
        for (uint32_t i = 0; i < p.spin_limit; ++i) {
          if (ld_acquire_gpu(counter) >= p.splits) { seen = true; break; }
          if ((i & 255u) == 255u && *abort_flag) break;
          __nanosleep(32);
        }
        if (!seen) ab.raise(0x0306);
        __threadfence();
        mbar_arrive(smem_u32(fix_go));
      }
      named_barrier(1, NDW * 32);
      if (!*abort_flag) {
        constexpr int NB = BM_TILES * (BN / 32);
        constexpr int G = NDW / 4;
        const int grp = ew >> 2;
        const int r_in = q * 32 + lane;
        const uint32_t ring = smem_u32(smem);
        constexpr int SPG = kFixSlots / G;       // this group's share of the ring's slots
        int own = 0, mine = 0;
        bool fine = true;
#pragma unroll 1
        for (int b = split; fine && b < NB; b += p.splits) {
          const int mt = b / (BN / 32), cb = b % (BN / 32);
          const int64_t col0 = o0 + cb * 32;
          if (col0 >= p.NO) continue;
          if ((mine++) % G != grp) continue;
          uint32_t v[32];
          __syncwarp();
          tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + mt * BN + cb * 32, v);
          tmem_ld_wait();
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
          if (MODE == kFwd && p.bias) {
#pragma unroll
            for (int j8 = 0; j8 < 4; ++j8) {
              const uint4 bb = __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + j8 * 8));
              const __half2* bh = reinterpret_cast<const __half2*>(&bb);
#pragma unroll
              for (int j = 0; j < 4; ++j) { const float2 t2 = __half22float2(bh[j]); f[j8 * 8 + 2 * j] += t2.x; f[j8 * 8 + 2 * j + 1] += t2.y; }
            }
          }
          for (int k = 0; k < p.splits - 1; ++k) {
            const int nn = own++, slot = grp * SPG + nn % SPG;
            if (!wait_or_abort(smem_u32(fx_full + slot), (nn / SPG) & 1, ab, 0x0305)) { fine = false; break; }
            const uint32_t src = ring + slot * 16384 + r_in * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint4 w = lds128(src + ((j ^ (r_in & 7)) << 4));
              f[4 * j] += __uint_as_float(w.x); f[4 * j + 1] += __uint_as_float(w.y);
              f[4 * j + 2] += __uint_as_float(w.z); f[4 * j + 3] += __uint_as_float(w.w);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(fx_empty + slot));
          }
          const int64_t row = m0 + mt * 256 + r_in;
          if (fine && row < p.M) {
            __half* dst = p.out + row * p.ldo + col0;
#pragma unroll
            for (int j8 = 0; j8 < 4; ++j8) {
              float* g8 = f + j8 * 8;
              if (MODE == kBwd && p.accumulate) {
                const uint4 o = *reinterpret_cast<const uint4*>(dst + j8 * 8);
                const __half2* oh2 = reinterpret_cast<const __half2*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) { const float2 of = __half22float2(oh2[j]); g8[2 * j] += of.x; g8[2 * j + 1] += of.y; }
              }
              uint4 o;
              o.x = pack_half2_rn(g8[0], g8[1]); o.y = pack_half2_rn(g8[2], g8[3]);
              o.z = pack_half2_rn(g8[4], g8[5]); o.w = pack_half2_rn(g8[6], g8[7]);
              *reinterpret_cast<uint4*>(dst + j8 * 8) = o;
            }
          }
        }
      }
    } else if (!direct) {
      // split-K fix-up, per CTA: the last CTA (over the splits) that owns these rows of this tile adds the slabs up
      __threadfence();
      named_barrier(1, NDW * 32);
      int* counter = p.counters + ((static_cast<int64_t>(tile_m) * tiles_o + tile_o) * 2 + rank);
      if (d == 0) {
        const int prev = atomicAdd(counter, 1);
        if (prev == p.splits - 1) { *last_flag = 1; *counter = 0; }
        __threadfence();
        mbar_arrive(smem_u32(fix_go));
      }
      named_barrier(1, NDW * 32);
      if (*last_flag && !*abort_flag) {
        constexpr int PARTS = (NDW * 32) / 128;
        constexpr int CPT = 32 / PARTS;
        const int r_in = d & 127, part = d >> 7;
        const uint32_t ring = smem_u32(smem);
        int n = 0;
        bool fine = true;
        for (int mt = 0; fine && mt < BM_TILES; ++mt) {
          const int64_t row = m0 + mt * 256 + r_in;
          for (int cb = 0; fine && cb < BN / 32; ++cb) {
            const int64_t col = o0 + cb * 32 + part * CPT;
            if (o0 + cb * 32 >= p.NO) break;
            float f[CPT];
#pragma unroll
            for (int j = 0; j < CPT; ++j) f[j] = 0.f;
            if (MODE == kFwd && p.bias) {
#pragma unroll
              for (int j8 = 0; j8 < CPT / 8; ++j8) {
                const uint4 bb = __ldg(reinterpret_cast<const uint4*>(p.bias + col + j8 * 8));
                const __half2* bh = reinterpret_cast<const __half2*>(&bb);
#pragma unroll
                for (int j = 0; j < 4; ++j) { const float2 t2 = __half22float2(bh[j]); f[j8 * 8 + 2 * j] = t2.x; f[j8 * 8 + 2 * j + 1] = t2.y; }
              }
            }
            for (int sp = 0; sp < p.splits; ++sp, ++n) {
              const int slot = n % kFixSlots;
              if (!wait_or_abort(smem_u32(fx_full + slot), (n / kFixSlots) & 1, ab, 0x0305)) { fine = false; break; }
              const uint32_t src = ring + slot * 16384 + r_in * 128;
#pragma unroll
              for (int j = 0; j < CPT / 4; ++j) {
                const uint4 v = lds128(src + (((part * (CPT / 4) + j) ^ (r_in & 7)) << 4));
                f[4 * j] += __uint_as_float(v.x); f[4 * j + 1] += __uint_as_float(v.y);
                f[4 * j + 2] += __uint_as_float(v.z); f[4 * j + 3] += __uint_as_float(v.w);
              }
              __syncwarp();
              if (lane == 0) mbar_arrive(smem_u32(fx_empty + slot));
            }
            if (fine && row < p.M) {
              __half* dst = p.out + row * p.ldo + col;
#pragma unroll
              for (int j8 = 0; j8 < CPT / 8; ++j8) {
                float* g8 = f + j8 * 8;
                if (MODE == kBwd && p.accumulate) {
                  const uint4 o = *reinterpret_cast<const uint4*>(dst + j8 * 8);
                  const __half2* oh2 = reinterpret_cast<const __half2*>(&o);
#pragma unroll
                  for (int j = 0; j < 4; ++j) { const float2 of = __half22float2(oh2[j]); g8[2 * j] += of.x; g8[2 * j + 1] += of.y; }
                }
                uint4 o;
                o.x = pack_half2_rn(g8[0], g8[1]); o.y = pack_half2_rn(g8[2], g8[3]);
                o.z = pack_half2_rn(g8[4], g8[5]); o.w = pack_half2_rn(g8[6], g8[7]);
                *reinterpret_cast<uint4*>(dst + j8 * 8) = o;
              }
            }
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncwarp();
  __syncthreads();
  cluster_sync_all();        // neither CTA may free tensor memory or leave while the other still uses the pair's resources
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, Cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// launch (cluster of two CTAs along x)
// ---------------------------------------------------------------------------------------------
bool coop_grid_fits(int64_t ctas, int ctas_per_sm, int sms);

template <int MODE, int BM_TILES>
static int launch_pair_cfg(const CUtensorMap& map, const CUtensorMap& nib_map, const CUtensorMap& out_map, const GemmParams& p_in,
                           int64_t tiles_o, int64_t tiles_mp, int splits, int launch_splits, cudaStream_t stream) {
  using Cfg = PairCfg<BM_TILES>;
  auto kernel = nf4_gemm_pair_kernel<MODE, BM_TILES>;
  NF4LL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
  const dim3 grid(static_cast<unsigned>(2 * tiles_o), static_cast<unsigned>(tiles_mp), static_cast<unsigned>(launch_splits));
  GemmParams p = p_in;
  if (p.coop) {
    // the shared split reduction needs every cluster of the grid resident at once: ask the runtime
    PdlLaunch probe(dim3(grid.x, grid.y, static_cast<unsigned>(splits)), dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, 2, 1, false, false);
    probe.cfg.numAttrs = 1;            // the cluster dimension only
    int clusters = 0;
    NF4LL_CUDA(cudaOccupancyMaxActiveClusters(&clusters, kernel, &probe.cfg));
    if (static_cast<int64_t>(clusters) < static_cast<int64_t>(tiles_o) * tiles_mp * splits) p.coop = 0;
  }
  for (;;) {
    PdlLaunch lc(grid, dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, 2, 1, p.coop != 0);
    const cudaError_t err = cudaLaunchKernelEx(&lc.cfg, kernel, map, nib_map, out_map, p);
    if (err == cudaErrorCooperativeLaunchTooLarge && p.coop) {
      (void)cudaGetLastError();        // fall back to the last-CTA reduction (counters are already zero)
      p.coop = 0;
      continue;
    }
    NF4LL_CUDA(err);
    break;
  }
  NF4LL_CUDA(cudaGetLastError());
  return NF4LL_OK;
}

int launch_pair(int mode, int bm_tiles, const CUtensorMap& map, const CUtensorMap& nib_map, const CUtensorMap& out_map,
                const GemmParams& p, int64_t tiles_o, int64_t tiles_mp, int splits, int launch_splits, cudaStream_t stream) {
  if (mode == kFwd) {
    return bm_tiles == 2 ? launch_pair_cfg<kFwd, 2>(map, nib_map, out_map, p, tiles_o, tiles_mp, splits, launch_splits, stream)
                         : launch_pair_cfg<kFwd, 1>(map, nib_map, out_map, p, tiles_o, tiles_mp, splits, launch_splits, stream);
  }
  return bm_tiles == 2 ? launch_pair_cfg<kBwd, 2>(map, nib_map, out_map, p, tiles_o, tiles_mp, splits, launch_splits, stream)
                       : launch_pair_cfg<kBwd, 1>(map, nib_map, out_map, p, tiles_o, tiles_mp, splits, launch_splits, stream);
}

}  // namespace nf4ll
