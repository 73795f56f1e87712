// Fused NF4 linear for sm_100a: activations x on-the-fly dequantised NF4 weights on tcgen05 tensor
// cores, with the LoRA branch folded into the same accumulator.
//
//   forward   y[M,N]  = x[M,K] . W[N,K]^T + bias + (s.T)[M,16] . B[N,16]^T
//   backward  dx[M,K] = dy[M,N] . W[N,K]  + keep_scale * mask (.) ((s.U)[M,16] . A[16,K])
//
// Replaces the reference's dequant-into-workspace + cuBLAS GEMM + LoRA GEMMs + LoRA add
// (solution/fast_qwen.py:716-750, 943-947, 1037, 1080-1112, 1310-1377; solution/k_rope.py:39-58;
// solution/k_norm.py:64-71). No fp16 copy of W is ever written to global memory.
//
// One CTA computes a (BM_TILES*128) x BN output tile. Roles by warp:
//   warp 0        TMA producer: 128x64 fp16 activation boxes (128-byte swizzle) and the tile's packed
//                 4-bit codes (BN quantisation blocks x 32 bytes) into shared-memory rings; after a
//                 split contraction it streams other splits' partial sums back in
//   warp 1        allocates tensor memory; one lane issues every tcgen05.mma and commit
//   warps 2-3     recover the fp32 absmax of every block of each stage (code2[q] * scale2 + offset2)
//                 into shared memory
//   warps 4..     BN threads in two teams that take alternate stages, two 64-weight quantisation
//                 blocks per thread: 128-bit shared loads of codes, block table in registers, 8 x
//                 128-bit swizzled shared stores per block. Before that they stage the rank-16 LoRA
//                 operands (and, in the backward with dropout, scale the LoRA product in tensor
//                 memory by the keep-mask); afterwards they drain tensor memory (epilogue)
// Variants of the forward: several projections stacked along N with one LoRA branch per segment,
// and gate|up tiles (128 gate + 128 up columns) whose epilogue also writes silu(g) * u.
// The weight tile in shared memory is the same in both directions: rows of 64 consecutive weights of
// one W row (= one quantisation block, 128 bytes), 8 rows per 1024-byte swizzle atom. Forward reads
// it as a K-major B operand (contraction along the row), backward as an MN-major one (contraction
// across rows), so the same NF4 bytes serve W and W^T.
#include "nf4ll_gemm_shared.cuh"

namespace nf4ll {

template <int BM_TILES, int BN>
struct TileCfg {
  static constexpr int kStages = (BN == 256) ? 3 : 4;
  static constexpr int kDequantWarps = BN / 32;
  static constexpr int kThreads = 32 * (4 + kDequantWarps);
  static constexpr int kABytes = BM_TILES * 128 * 128;   // per stage: 128 rows x 64 fp16 per M tile
  static constexpr int kBBytes = BN * 128;               // per stage: BN dequantised quantisation blocks
  static constexpr int kNibBytes = BN * 32;              // per stage: their packed codes
  static constexpr int kAbsBytes = BN * 4;               // per stage: their fp32 absmax
  static constexpr int kLoraLeftBytes = BM_TILES * 128 * 32;
  static constexpr int kLoraRightBytes = BN * 32;
  static constexpr int kTmemCols = BM_TILES * BN;        // 128, 256 or 512: a power of two >= 32
  static constexpr int kSmemBytes = 1024 /* alignment slack */ + kStages * (kABytes + kBBytes + kNibBytes + kAbsBytes) +
                                    1024 /* code2 */ + 512 /* barriers */;
  // the LoRA operands are only read by the very first MMAs: they borrow the last weight-tile stage
  static_assert(kLoraLeftBytes + kLoraRightBytes <= kBBytes, "LoRA operands must fit one weight stage");
};

template <int MODE, int BM_TILES, int BN>
__global__ void __launch_bounds__(TileCfg<BM_TILES, BN>::kThreads, 1)
nf4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_act, const __grid_constant__ CUtensorMap tmap_nib,
                const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_out_u,
                const __grid_constant__ CUtensorMap tmap_out_h, const GemmParams p) {
  using Cfg = TileCfg<BM_TILES, BN>;
  constexpr int S = Cfg::kStages;
  constexpr int NDW = Cfg::kDequantWarps;

  pdl_wait();                  // everything below may read what the previous kernel on the stream wrote
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;                                   // [S][BM_TILES][128 rows][128 B]
  uint8_t* sB = sA + S * Cfg::kABytes;                  // [S][BN rows][128 B]
  uint8_t* sNib = sB + S * Cfg::kBBytes;                // [S][BN blocks][32 B] packed codes
  uint8_t* sAbs = sNib + S * Cfg::kNibBytes;            // [S][BN] fp32 absmax
  float* sCode2 = reinterpret_cast<float*>(sAbs + S * Cfg::kAbsBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sCode2) + 1024);
  uint8_t* sLL = sB + (S - 1) * Cfg::kBBytes;           // LoRA left operand  [BM_TILES][128 x 16] (borrows the last weight stage)
  uint8_t* sLR = sLL + Cfg::kLoraLeftBytes;             // LoRA right operand [BN x 16] or [16 x BN]
  // barrier slots
  // [S] stage ready for the tensor core: activation boxes landed (producer arrive + bytes) and the
  // weight tile dequantised (one arrive per warp of the stage's team); one barrier, one wait per stage
  uint64_t* full_a = bars;
  uint64_t* full_b = full_a;
  uint64_t* empty = bars + 2 * S;     // [S] MMAs that read the stage have completed
  uint64_t* nib_full = bars + 3 * S;  // [S] packed codes landed and absmax written
  uint64_t* nib_empty = bars + 4 * S; // [S] dequant warps have read codes and absmax
  uint64_t* lora_full = bars + 5 * S;
  uint64_t* acc_full = lora_full + 1;
  uint64_t* pre_full = lora_full + 2;
  uint64_t* pre_done = lora_full + 3;
  uint64_t* lora_done = lora_full + 4;
  uint64_t* fix_go = lora_full + 5;
  uint64_t* fx_full = lora_full + 6;              // [kFixSlots] split-K fix-up ring
  uint64_t* fx_empty = fx_full + kFixSlots;       // [kFixSlots]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(fx_empty + kFixSlots);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = abort_flag + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tile_o = blockIdx.x, tile_m = blockIdx.y, split = blockIdx.z;
  const int64_t m0 = static_cast<int64_t>(tile_m) * (BM_TILES * 128);
  // gate|up mode: the tile's 256 weight rows are 128 gate rows and the 128 up rows of the same columns
  constexpr bool kGuCapable = (MODE == kFwd && BM_TILES == 2 && BN == 256);
  const bool gu = kGuCapable && p.gu_inter > 0;
  const int64_t g0 = static_cast<int64_t>(tile_o) * 128;
  const int64_t o0 = gu ? g0 : static_cast<int64_t>(tile_o) * BN;
  // weight row behind tile row d
  auto wrow = [&](int d) -> int64_t { return (gu && d >= 128) ? p.gu_inter + g0 + (d - 128) : o0 + d; };

  // contraction range of this split, in 64-wide steps
  const int nkb_total = static_cast<int>(p.KC / 64);
  const int kb_begin = static_cast<int>(static_cast<int64_t>(nkb_total) * split / p.splits);
  const int kb_end = static_cast<int>(static_cast<int64_t>(nkb_total) * (split + 1) / p.splits);
  const int nkb = kb_end - kb_begin;
  // the LoRA branch of this tile: the projection's, or the one of the stacked segment the tile lies in
  const float* lora_left = p.lora_left;
  const __half* lora_right = p.lora_right;
  float left_scale = p.left_scale;
  bool has_lora = p.has_lora != 0;
  if (gu) {
    has_lora = p.seg_left[0] != nullptr || p.seg_left[1] != nullptr;
  } else if (p.n_seg > 0) {
    int sg = 0;
    for (int i = 1; i < p.n_seg; ++i) if (static_cast<int64_t>(tile_o) * BN >= p.seg_begin[i]) sg = i;
    lora_left = p.seg_left[sg]; lora_right = p.seg_right[sg]; left_scale = p.seg_scale[sg];
    has_lora = lora_left != nullptr;
  }
  const bool lora_here = has_lora && split == 0;
  const bool premask = lora_here && MODE == kBwd && p.mask != nullptr;

  const Abort ab{abort_flag, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(full_a + s), 1 + NDW / 2);    // producer + one of the two dequant teams per stage
      mbar_init(smem_u32(empty + s), 1);
      mbar_init(smem_u32(nib_full + s), 3);        // TMA expect_tx arrive + the two absmax warps
      mbar_init(smem_u32(nib_empty + s), NDW / 2);
    }
    mbar_init(smem_u32(lora_done), 1);
    mbar_init(smem_u32(fix_go), 1);
    for (int i = 0; i < kFixSlots; ++i) {
      mbar_init(smem_u32(fx_full + i), 1);
      mbar_init(smem_u32(fx_empty + i), p.coop ? 4 : NDW);   // a slot is read by one warp group (shared reduction) or by all
    }
    mbar_init(smem_u32(lora_full), NDW);
    mbar_init(smem_u32(acc_full), 1);
    mbar_init(smem_u32(pre_full), 1);
    mbar_init(smem_u32(pre_done), NDW);
    *abort_flag = 0;
    *last_flag = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < 256) sCode2[threadIdx.x] = p.code2[threadIdx.x];
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncwarp();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ----------------------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_act);
      tma_prefetch_desc(&tmap_nib);
      int issued = 0;
      for (int i = 0; i < nkb; ++i, ++issued) {
        const int s = i % S;
        const uint32_t free_parity = ((i / S) & 1) ^ 1;
        const int kb = kb_begin + i;
        // packed codes first (the dequant warps need them a whole stage before the MMA needs anything)
        if (!wait_or_abort(smem_u32(nib_empty + s), free_parity, ab, 0x0102)) break;
        mbar_arrive_expect_tx(smem_u32(nib_full + s), Cfg::kNibBytes);
        if (gu) {
          // two boxes of 128 weight rows: gate, then up
          tma_load_2d(smem_u32(sNib + s * Cfg::kNibBytes), &tmap_nib, kb * 32, static_cast<int>(g0), smem_u32(nib_full + s));
          tma_load_2d(smem_u32(sNib + s * Cfg::kNibBytes + 128 * 32), &tmap_nib, kb * 32, static_cast<int>(p.gu_inter + g0),
                      smem_u32(nib_full + s));
        } else if (MODE == kFwd) {
          tma_load_2d(smem_u32(sNib + s * Cfg::kNibBytes), &tmap_nib, kb * 32, static_cast<int>(o0), smem_u32(nib_full + s));
        } else {
          tma_load_2d(smem_u32(sNib + s * Cfg::kNibBytes), &tmap_nib, static_cast<int>(o0 / 2), kb * 64, smem_u32(nib_full + s));
        }
        if (!wait_or_abort(smem_u32(empty + s), free_parity, ab, 0x0101)) break;
        mbar_arrive_expect_tx(smem_u32(full_a + s), Cfg::kABytes);
#pragma unroll
        for (int mt = 0; mt < BM_TILES; ++mt) {
          tma_load_2d(smem_u32(sA + s * Cfg::kABytes + mt * 16384), &tmap_act, kb * 64,
                      static_cast<int>(m0 + mt * 128), smem_u32(full_a + s));
        }
      }
      if (p.splits > 1 && !*abort_flag) {
        // split-K: if this CTA turns out to be the last of its tile, stream all slabs back in
        if (wait_or_abort(smem_u32(fix_go), 0, ab, 0x0104) && p.coop && !*abort_flag) {
          // shared reduction: this CTA owns every splits-th box of the tile and streams the other
          // splits' partial sums of exactly those boxes back in
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
                          static_cast<int>(static_cast<int64_t>(sp) * p.m_pad + m0 + mt * 128), smem_u32(fx_full + slot));
            }
          }
        } else if (!p.coop && *last_flag) {
          fence_proxy_async_all();     // the other splits' slab writes were observed through ordinary loads / atomics
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
                            static_cast<int>(static_cast<int64_t>(sp) * p.m_pad + m0 + mt * 128), smem_u32(fx_full + slot));
              }
            }
          }
        }
      }
      if (*abort_flag) {
        // give copies still in flight a bounded chance to land before the CTA goes away
        for (int i = (issued > S ? issued - S : 0); i <= issued && i < nkb; ++i) {
          const uint32_t ph = (i / S) & 1;
          for (int spin = 0; spin < (1 << 16) && !mbar_try_wait(smem_u32(full_a + (i % S)), ph); ++spin) {}
          for (int spin = 0; spin < (1 << 16) && !mbar_try_wait(smem_u32(nib_full + (i % S)), ph); ++spin) {}
        }
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_main = make_idesc_f16(128, BN, 0, MODE == kBwd ? 1 : 0);
      bool ok = true;
      if (lora_here) {
        ok = wait_or_abort(smem_u32(lora_full), 0, ab, 0x0201);
        if (ok) {
          tc_fence_after();
          // rank-16 step: left [128 x 16] K-major, right K-major [BN x 16] (fwd) / MN-major [16 x BN] (bwd);
          // 8x(16 B) core matrices, 128 B between the two K halves, 256 B between 8-row (or 8-column) groups
          if (gu) {
            // two branches: gate columns from (T_gate, B_gate), up columns from (T_up, B_up), N = 128 each
            constexpr uint32_t idesc_half = make_idesc_f16(128, 128, 0, 0);
            const uint32_t right = smem_u32(sLL) + 2 * Cfg::kLoraLeftBytes;
#pragma unroll
            for (int mt = 0; mt < BM_TILES; ++mt) {
#pragma unroll
              for (int br = 0; br < 2; ++br) {
                const uint64_t ldesc = make_smem_desc(smem_u32(sLL) + br * Cfg::kLoraLeftBytes + mt * 4096, 128, 256, kSwizzleNone);
                const uint64_t rdesc = make_smem_desc(right + br * 4096, 128, 256, kSwizzleNone);
                tc_mma_f16(tmem_base + mt * BN + br * 128, ldesc, rdesc, idesc_half, 0u);
              }
            }
          } else {
            const uint64_t rdesc = make_smem_desc(smem_u32(sLR), 128, 256, kSwizzleNone);
#pragma unroll
            for (int mt = 0; mt < BM_TILES; ++mt) {
              const uint64_t ldesc = make_smem_desc(smem_u32(sLL + mt * 4096), 128, 256, kSwizzleNone);
              tc_mma_f16(tmem_base + mt * BN, ldesc, rdesc, idesc_main, 0u);
            }
          }
          tc_commit(smem_u32(lora_done));     // the borrowed weight stage may be overwritten after this
          if (premask) {
            tc_commit(smem_u32(pre_full));
            ok = wait_or_abort(smem_u32(pre_done), 0, ab, 0x0202);
            if (ok) tc_fence_after();
          }
        }
      }
      for (int i = 0; ok && i < nkb; ++i) {
        const int s = i % S;
        const uint32_t ph = (i / S) & 1;
        if (!wait_or_abort(smem_u32(full_a + s), ph, ab, 0x0203)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_base = smem_u32(sA + s * Cfg::kABytes);
        const uint32_t b_base = smem_u32(sB + s * Cfg::kBBytes);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {       // four K=16 steps per 64-wide stage
          const uint64_t bdesc = (MODE == kFwd)
                                     ? make_smem_desc(b_base + kk * 32, 16, 1024, kSwizzle128B)
                                     : make_smem_desc(b_base + kk * 2048, 8192, 1024, kSwizzle128B);
#pragma unroll
          for (int mt = 0; mt < BM_TILES; ++mt) {
            const uint64_t adesc = make_smem_desc(a_base + mt * 16384 + kk * 32, 16, 1024, kSwizzle128B);
            tc_mma_f16(tmem_base + mt * BN, adesc, bdesc, idesc_main, (lora_here || i > 0 || kk > 0) ? 1u : 0u);
          }
        }
        tc_commit(smem_u32(empty + s));     // frees the stage once these MMAs have read it
      }
      tc_commit(smem_u32(acc_full));
      if (!ok) {
        // make sure nothing is still running on the tensor core before tensor memory is freed
        for (int spin = 0; spin < (1 << 18) && !mbar_try_wait(smem_u32(acc_full), 0); ++spin) {}
      }
    }
  } else if (warp < 4) {
    // ----------------------------------------------------------------------------- absmax helper
    // absmax of the stage's BN quantisation blocks: code2[q] * scale2 + offset2, rounded separately
    {
      constexpr int PER = BN / 64;                 // blocks per helper thread
      const int t = threadIdx.x - 64;
      int64_t qb[PER], qstep;
#pragma unroll
      for (int e = 0; e < PER; ++e) {
        const int d = t + e * 64;
        if (MODE == kFwd) {
          int64_t n = wrow(d);
          if (n >= p.N) n = p.N - 1;               // tail rows: any valid block; their output is never stored
          qb[e] = (n * p.K) / 64 + kb_begin;
        } else {
          constexpr int SUB = BN / 64;
          const int j = d % SUB, r = d / SUB;
          int64_t kcol = o0 + j * 64;
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
        for (int e = 0; e < PER; ++e) {          // next stage's codes and scales, in flight during this stage
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
    const int d = threadIdx.x - 128;      // 0..BN-1: one quantisation block per stage
    const int ew = warp - 4;              // 0..NDW-1
    const int q = warp & 3;               // tensor-memory lane quarter this warp may read
    bool ok = true;

    // --- LoRA operands: staged by these warps while the first weight codes are still on their way.
    // All loads are issued before the first store, so the cost is one trip to memory.
    if (kGuCapable && gu && lora_here) {
      // gate|up: two left operands (T_gate, T_up: 256 rows x 16 each) and the tile's 128 rows of B_gate and
      // B_up; a branch without LoRA contributes zeros. Layout: [left gate | left up | right gate, right up].
      constexpr int NT = NDW * 32;
      constexpr int LEFT = 2 * BM_TILES * 128 * 2, RIGHT = 256 * 2;
      constexpr int LPT = LEFT / NT, RPT = RIGHT / NT;
      float4 la[LPT], lb[LPT];
      uint4 rv[RPT];
#pragma unroll
      for (int e = 0; e < LPT; ++e) {
        const int c = d + e * NT, br = c / (BM_TILES * 128 * 2), cc = c % (BM_TILES * 128 * 2), row = cc >> 1, h = cc & 1;
        la[e] = make_float4(0.f, 0.f, 0.f, 0.f); lb[e] = la[e];
        const float* left = p.seg_left[br];
        if (left && m0 + row < p.M) {
          const float4* src = reinterpret_cast<const float4*>(left + (m0 + row) * 16 + h * 8);
          la[e] = __ldg(src); lb[e] = __ldg(src + 1);
        }
      }
#pragma unroll
      for (int e = 0; e < RPT; ++e) {
        const int c = d + e * NT, row = c >> 1, h = c & 1, br = row >> 7, r = row & 127;
        rv[e] = make_uint4(0, 0, 0, 0);
        if (p.seg_left[br] && g0 + r < p.gu_inter)
          rv[e] = __ldg(reinterpret_cast<const uint4*>(p.seg_right[br] + (g0 + r) * 16 + h * 8));
      }
      uint8_t* sRight = sLL + 2 * Cfg::kLoraLeftBytes;
#pragma unroll
      for (int e = 0; e < LPT; ++e) {
        const int c = d + e * NT, br = c / (BM_TILES * 128 * 2), cc = c % (BM_TILES * 128 * 2), row = cc >> 1, h = cc & 1;
        const float sc = p.seg_scale[br];
        uint4 v;
        v.x = pack_half2_rn(la[e].x * sc, la[e].y * sc);
        v.y = pack_half2_rn(la[e].z * sc, la[e].w * sc);
        v.z = pack_half2_rn(lb[e].x * sc, lb[e].y * sc);
        v.w = pack_half2_rn(lb[e].z * sc, lb[e].w * sc);
        const int mt = row >> 7, r = row & 127;
        *reinterpret_cast<uint4*>(sLL + br * Cfg::kLoraLeftBytes + mt * 4096 + (r >> 3) * 256 + h * 128 + (r & 7) * 16) = v;
      }
#pragma unroll
      for (int e = 0; e < RPT; ++e) {
        const int c = d + e * NT, row = c >> 1, h = c & 1;
        *reinterpret_cast<uint4*>(sRight + (row >> 3) * 256 + h * 128 + (row & 7) * 16) = rv[e];
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(lora_full));
    } else if (lora_here) {
      constexpr int NT = NDW * 32;
      constexpr int LEFT = BM_TILES * 128 * 2;         // 16-byte chunks (8 fp16) of the left operand
      constexpr int RIGHT = BN * 2;
      constexpr int LPT = (LEFT + NT - 1) / NT, RPT = (RIGHT + NT - 1) / NT;
      float4 la[LPT], lb[LPT];
      uint4 rv[RPT];
      // left: rows m0.. of lora_left[M,16] (fp32), scaled and rounded to fp16 here
#pragma unroll
      for (int e = 0; e < LPT; ++e) {
        const int c = d + e * NT, row = c >> 1, h = c & 1;
        la[e] = make_float4(0.f, 0.f, 0.f, 0.f); lb[e] = la[e];
        if (c < LEFT && m0 + row < p.M) {
          const float4* src = reinterpret_cast<const float4*>(lora_left + (m0 + row) * 16 + h * 8);
          la[e] = __ldg(src); lb[e] = __ldg(src + 1);
        }
      }
#pragma unroll
      for (int e = 0; e < RPT; ++e) {
        const int c = d + e * NT;
        rv[e] = make_uint4(0, 0, 0, 0);
        if (MODE == kFwd) {
          const int row = c >> 1, h = c & 1;           // rows o0.. of B[N,16]
          if (c < RIGHT && o0 + row < p.NO) rv[e] = __ldg(reinterpret_cast<const uint4*>(lora_right + (o0 + row) * 16 + h * 8));
        } else {
          const int j = c / (BN / 8), c8 = c % (BN / 8);   // columns o0.. of A[16,K]
          if (c < RIGHT && o0 + c8 * 8 < p.NO) rv[e] = __ldg(reinterpret_cast<const uint4*>(lora_right + j * p.K + o0 + c8 * 8));
        }
      }
#pragma unroll
      for (int e = 0; e < LPT; ++e) {
        const int c = d + e * NT, row = c >> 1, h = c & 1;
        if (c < LEFT) {
          uint4 v;
          v.x = pack_half2_rn(la[e].x * left_scale, la[e].y * left_scale);
          v.y = pack_half2_rn(la[e].z * left_scale, la[e].w * left_scale);
          v.z = pack_half2_rn(lb[e].x * left_scale, lb[e].y * left_scale);
          v.w = pack_half2_rn(lb[e].z * left_scale, lb[e].w * left_scale);
          // chunk (row, h) -> (row/8)*256 + h*128 + (row%8)*16 inside the 128-row tile
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
            // chunk (8 columns c8, rank row j) -> c8*256 + (j/8)*128 + (j%8)*16
            const int j = c / (BN / 8), c8 = c % (BN / 8);
            *reinterpret_cast<uint4*>(sLR + c8 * 256 + (j >> 3) * 128 + (j & 7) * 16) = rv[e];
          }
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(lora_full));
    }

    // --- dequantise. The warps form two teams that take alternate stages, two blocks per thread, so
    // that one team's barrier round trips (wait, proxy fence, arrive) overlap the other team's decode
    // instead of leaving the integer pipe idle while all warps sit in the same wait.
    constexpr int TEAM = BN / 2;                       // threads per team = blocks per thread pair
    const int team = d / TEAM, tg = d % TEAM;
    uint32_t nib_off[2], row_off[2];                   // 32 bytes of codes / 128-byte output row inside a stage
    int key[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int blk = tg + h * TEAM;
      if (MODE == kFwd) {
        nib_off[h] = blk * 32;
        row_off[h] = blk * 128;
        key[h] = blk & 7;
      } else {
        constexpr int SUB = BN / 64;
        const int j = blk % SUB, r = blk / SUB;        // sub-tile (64 output columns) and row in the stage
        nib_off[h] = r * (BN / 2) + j * 32;
        row_off[h] = j * 8192 + r * 128;
        key[h] = r & 7;
      }
    }
    const uint32_t nib_base = smem_u32(sNib), abs_base = smem_u32(sAbs) + tg * 4, b_base = smem_u32(sB);
    auto dequant_stage = [&](int i) -> bool {
      const int s = i % S;
      const uint32_t ph = (i / S) & 1;
      if (!wait_or_abort(smem_u32(nib_full + s), ph, ab, 0x0304)) return false;
      uint4 c[2][2];
      float absmax[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        c[h][0] = lds128(nib_base + s * Cfg::kNibBytes + nib_off[h]);
        c[h][1] = lds128(nib_base + s * Cfg::kNibBytes + nib_off[h] + 16);
        absmax[h] = lds_f32(abs_base + s * Cfg::kAbsBytes + h * TEAM * 4);
      }
      if (!wait_or_abort(smem_u32(empty + s), ph ^ 1, ab, 0x0302)) return false;
      // the last stage holds the LoRA operands until the rank-16 MMAs have read them
      if (lora_here && i == S - 1 && !wait_or_abort(smem_u32(lora_done), 0, ab, 0x0305)) return false;
#pragma unroll
      for (int h = 0; h < 2; ++h)
        dequant_block_to_smem(b_base + s * Cfg::kBBytes + row_off[h], key[h], c[h][0], c[h][1], absmax[h]);
      fence_proxy_async_smem();      // generic-proxy stores -> visible to the tensor core's async proxy
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(full_b + s));
        mbar_arrive(smem_u32(nib_empty + s));      // codes and absmax of this stage are in registers / consumed
      }
      return true;
    };

    int i_next = team;
    if (premask) {
      // The LoRA product lands in the accumulator first and is scaled by keep_scale * mask in place, so
      // that the base GEMM then accumulates on top (dropout acts on the LoRA input only). While the
      // rank-16 MMAs run, each team already dequantises its first stage and the first mask bytes travel.
      constexpr int kChunks = BM_TILES * (BN / 32);
      constexpr int kStep = NDW / 4;
      auto load_mask = [&](int u, uint4& a, uint4& b) {
        a = make_uint4(0, 0, 0, 0); b = a;
        if (u < kChunks) {
          const int mt = u / (BN / 32), c = u % (BN / 32);
          const int64_t row = m0 + mt * 128 + q * 32 + lane;
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
          load_mask(u + kStep, na, nb);                // next chunk's mask travels during this chunk
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

    // --- epilogue: tensor memory -> registers -> swizzled shared staging -> TMA store.
    // The operand rings are idle once the accumulator is complete, so they serve as staging space:
    // each group of four warps (one per tensor-memory lane quarter) owns 64 KB of it and drains one
    // 128-row accumulator at a time in boxes of 128 rows x 128 bytes.
    if (ok) ok = wait_or_abort(smem_u32(acc_full), 0, ab, 0x0303);
    const bool direct = (p.splits == 1);
    if (ok) {
      tc_fence_after();
      constexpr int G = NDW / 4;                       // warp groups
      const int grp = ew >> 2;
      const int bar_id = 2 + grp;
      const uint32_t stage = smem_u32(smem) + grp * 65536;
      const int r_in = q * 32 + lane;                  // row inside the 128-row accumulator
      const uint32_t row_addr = stage + r_in * 128;
      const int key = r_in & 7;
      const bool leader = (q == 0 && lane == 0);
      if (kGuCapable && gu) {
        // gate|up: this warp group drains one 128-row accumulator: g (columns 0-127), u (128-255), and
        // h = silu(g) * u computed from the rounded fp16 values, as the stand-alone kernel would read them.
        // Staging: six boxes of 128 rows x 64 columns (g, g, u, u, h, h), one TMA store each.
        const uint32_t stage_gu = smem_u32(smem) + grp * 98304;
        const uint32_t row_gu = stage_gu + r_in * 128;
        const int mt = grp;
        const uint32_t tacc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + mt * BN;
#pragma unroll 1
        for (int jb = 0; jb < 2; ++jb) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int j = jb * 2 + half;
            uint32_t vg[32], vu[32];
            __syncwarp();
            tmem_ld32(tacc + j * 32, vg);
            tmem_ld32(tacc + 128 + j * 32, vu);
            tmem_ld_wait();
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {
              uint4 gq, uq;
              gq.x = pack_half2_rn(__uint_as_float(vg[g8 * 8 + 0]), __uint_as_float(vg[g8 * 8 + 1]));
              gq.y = pack_half2_rn(__uint_as_float(vg[g8 * 8 + 2]), __uint_as_float(vg[g8 * 8 + 3]));
              gq.z = pack_half2_rn(__uint_as_float(vg[g8 * 8 + 4]), __uint_as_float(vg[g8 * 8 + 5]));
              gq.w = pack_half2_rn(__uint_as_float(vg[g8 * 8 + 6]), __uint_as_float(vg[g8 * 8 + 7]));
              uq.x = pack_half2_rn(__uint_as_float(vu[g8 * 8 + 0]), __uint_as_float(vu[g8 * 8 + 1]));
              uq.y = pack_half2_rn(__uint_as_float(vu[g8 * 8 + 2]), __uint_as_float(vu[g8 * 8 + 3]));
              uq.z = pack_half2_rn(__uint_as_float(vu[g8 * 8 + 4]), __uint_as_float(vu[g8 * 8 + 5]));
              uq.w = pack_half2_rn(__uint_as_float(vu[g8 * 8 + 6]), __uint_as_float(vu[g8 * 8 + 7]));
              const uint4 hq = swiglu_fwd8(gq, uq);
              const uint32_t off = ((half * 4 + g8) ^ key) << 4;
              sts128(row_gu + (0 + jb) * 16384 + off, gq);
              sts128(row_gu + (2 + jb) * 16384 + off, uq);
              sts128(row_gu + (4 + jb) * 16384 + off, hq);
            }
          }
        }
        fence_proxy_async_smem();
        named_barrier(bar_id, 128);
        if (leader) {
          const int row_g = static_cast<int>(m0 + mt * 128);
          for (int jb = 0; jb < 2; ++jb) {
            const int64_t col0 = g0 + jb * 64;
            if (col0 >= p.gu_inter) break;
            tma_store_2d(&tmap_out, stage_gu + (0 + jb) * 16384, static_cast<int>(col0), row_g);
            tma_store_2d(&tmap_out_u, stage_gu + (2 + jb) * 16384, static_cast<int>(col0), row_g);
            tma_store_2d(&tmap_out_h, stage_gu + (4 + jb) * 16384, static_cast<int>(col0), row_g);
          }
          bulk_commit();
          bulk_wait_read_all();
        }
      } else if (!direct && p.coop) {
        // shared reduction, first half: every box of the tile that another split owns goes to this
        // split's slab as fp32, four boxes per staging round, rounds dealt to the warp groups in turn
        constexpr int NB = BM_TILES * (BN / 32);
        constexpr int SB = 4;
        int f = 0, pending = 0;
        uint32_t staged = 0;                         // box indices of the round, 8 bits each
        auto flush = [&]() {
          fence_proxy_async_smem();
          named_barrier(bar_id, 128);
          if (leader) {
            for (int k = 0; k < pending; ++k) {
              const int b = (staged >> (8 * k)) & 0xff;
              const int mt = b / (BN / 32), cb = b % (BN / 32);
              const int64_t col0 = o0 + cb * 32;
              if (col0 < p.NO)
                tma_store_2d(&tmap_out, stage + k * 16384, static_cast<int>(col0),
                             static_cast<int>(static_cast<int64_t>(split) * p.m_pad + m0 + mt * 128));
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
            sts128(row_addr + pending * 16384 + ((j ^ key) << 4), make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
          staged |= static_cast<uint32_t>(b) << (8 * pending);
          if (++pending == SB) flush();
        }
        if (pending) flush();
      }
      // plain paths: the whole accumulator goes out as fp16 (no split) or as this split's fp32 slab
      const bool plain = !gu && (direct || !p.coop);
      for (int mt = grp; plain && mt < BM_TILES; mt += G) {
        const uint32_t tacc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + mt * BN;
        const int row_g = static_cast<int>(m0 + mt * 128);
        if (direct) {
          // fp16 output: boxes of 64 columns
#pragma unroll 1
          for (int cb = 0; cb < BN / 64; ++cb) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const int c = cb * 2 + half;
              const int64_t col0 = o0 + c * 32;
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
                sts128(row_addr + cb * 16384 + (((half * 4 + g8) ^ key) << 4), o);
              }
            }
          }
          fence_proxy_async_smem();
          named_barrier(bar_id, 128);
          if (leader) {
            for (int cb = 0; cb < BN / 64; ++cb) {
              const int64_t col0 = o0 + cb * 64;
              if (col0 >= p.NO) break;
              // rows past M and columns past NO are clipped by the tensor map
              if (MODE == kBwd && p.accumulate) tma_reduce_add_2d(&tmap_out, stage + cb * 16384, static_cast<int>(col0), row_g);
              else tma_store_2d(&tmap_out, stage + cb * 16384, static_cast<int>(col0), row_g);
            }
            bulk_commit();
            bulk_wait_read_all();
          }
          if (mt + G < BM_TILES) named_barrier(bar_id, 128);      // staging is reused by the next accumulator
        } else {
          // fp32 partial sums into this split's slab: boxes of 32 columns, four per round
          const int slab_row = static_cast<int>(static_cast<int64_t>(split) * p.m_pad + m0 + mt * 128);
#pragma unroll 1
          for (int round = 0; round < BN / 128; ++round) {
#pragma unroll 1
            for (int b4 = 0; b4 < 4; ++b4) {
              const int c = round * 4 + b4;
              uint32_t v[32];
              __syncwarp();
              tmem_ld32(tacc + c * 32, v);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 8; ++j)
                sts128(row_addr + b4 * 16384 + ((j ^ key) << 4), make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
            }
            fence_proxy_async_smem();
            named_barrier(bar_id, 128);
            if (leader) {
              for (int b4 = 0; b4 < 4; ++b4) {
                const int64_t col0 = o0 + (round * 4 + b4) * 32;
                if (col0 >= p.NO) break;
                tma_store_2d(&tmap_out, stage + b4 * 16384, static_cast<int>(col0), slab_row);
              }
              bulk_commit();
              bulk_wait_read_all();
            }
            named_barrier(bar_id, 128);
          }
        }
      }
      if (!direct && leader) {
        // the slab must be complete and visible to other CTAs' ordinary loads before the tile counter moves
        bulk_wait_all();
        fence_proxy_async_all();
        __threadfence();
      }
    }
    if (!direct && p.coop) {
      // shared reduction, second half: once every split of this tile has published its slab, each
      // split finishes the boxes it owns: its own partial sums straight from tensor memory plus the
      // other splits' in ascending order (a fixed order: results do not depend on timing).
      __threadfence();
      named_barrier(1, NDW * 32);
      if (d == 0) {
        int* counter = p.counters + (static_cast<int64_t>(tile_m) * gridDim.x + tile_o);
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
        mbar_arrive(smem_u32(fix_go));       // warp 0 starts streaming the other splits' boxes
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
          const int64_t row = m0 + mt * 128 + r_in;
          if (fine && row < p.M) {
            __half* dst = p.out + row * p.ldo + col0;
#pragma unroll
            for (int j8 = 0; j8 < 4; ++j8) {
              float* g8 = f + j8 * 8;
              if (MODE == kBwd && p.accumulate) {
                const uint4 o = *reinterpret_cast<const uint4*>(dst + j8 * 8);
                const __half2* oh = reinterpret_cast<const __half2*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) { const float2 of = __half22float2(oh[j]); g8[2 * j] += of.x; g8[2 * j + 1] += of.y; }
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
      // split-K fix-up: the last CTA of this output tile to finish sums all slabs in split order
      // (deterministic) and writes the fp16 result. Every dequant thread takes both barriers, also
      // after a failed wait, so that nobody is left behind at a barrier.
      __threadfence();
      named_barrier(1, NDW * 32);
      int* counter = p.counters + (static_cast<int64_t>(tile_m) * gridDim.x + tile_o);
      if (d == 0) {
        const int prev = atomicAdd(counter, 1);
        if (prev == p.splits - 1) { *last_flag = 1; *counter = 0; }
        __threadfence();
        mbar_arrive(smem_u32(fix_go));       // tells warp 0 whether to stream the slabs back in
      }
      named_barrier(1, NDW * 32);
      if (*last_flag && !*abort_flag) {
        // Warp 0 streams every split's 128-row x 32-column fp32 box of this tile through a ring of
        // 16 KB shared-memory slots (TMA loads, several in flight); these threads add the boxes up in
        // split order, then round once to fp16. Thread = one row, CPT consecutive columns of the box.
        constexpr int PARTS = (NDW * 32) / 128;         // threads per box row
        constexpr int CPT = 32 / PARTS;                 // columns per thread
        const int r_in = d & 127, part = d >> 7;
        const uint32_t ring = smem_u32(smem);
        int n = 0;
        bool fine = true;
        for (int mt = 0; fine && mt < BM_TILES; ++mt) {
          const int64_t row = m0 + mt * 128 + r_in;
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
                  const __half2* oh = reinterpret_cast<const __half2*>(&o);
#pragma unroll
                  for (int j = 0; j < 4; ++j) { const float2 of = __half22float2(oh[j]); g8[2 * j] += of.x; g8[2 * j + 1] += of.y; }
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
  __syncwarp();          // single-lane roles (TMA producer, MMA issuer) rejoin their warps first
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int get_encode_fn(EncodeTiledFn* out) {
  static EncodeTiledFn cached = nullptr;   // written once with the same value by any thread
  if (!cached) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    NF4LL_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || !fn) {
      set_detail("cuTensorMapEncodeTiled not available from the driver");
      return NF4LL_ERR_CUDA;
    }
    cached = reinterpret_cast<EncodeTiledFn>(fn);
  }
  *out = cached;
  return NF4LL_OK;
}

// 2-D map over a row-major matrix [rows, cols] with leading dimension ld (elements): boxes of 128
// rows x 128 bytes (the swizzle span: 64 fp16 or 32 fp32 columns); loads zero-fill outside the
// matrix, stores are clipped to it.
static int make_tile_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, bool f32) {
  EncodeTiledFn enc = nullptr;
  if (int rc = get_encode_fn(&enc)) return rc;
  const int esz = f32 ? 4 : 2;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * esz};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / esz), 128};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_detail("cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld cols=%lld ld=%lld)", static_cast<int>(r),
               static_cast<long long>(rows), static_cast<long long>(cols), static_cast<long long>(ld));
    return NF4LL_ERR_CUDA;
  }
  return NF4LL_OK;
}

// 2-D map over the packed codes of W[N,K] seen as bytes [N, K/2]. Forward boxes: BN rows x 32 bytes
// (one quantisation block per row); backward boxes: 64 rows x BN/2 bytes. No swizzle, zero fill.
static int make_nib_map(CUtensorMap* map, const void* nib, int64_t N, int64_t K, int mode, int bn) {
  EncodeTiledFn enc = nullptr;
  if (int rc = get_encode_fn(&enc)) return rc;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K / 2), static_cast<cuuint64_t>(N)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K / 2)};
  const cuuint32_t box[2] = {mode == kFwd ? 32u : static_cast<cuuint32_t>(bn / 2), mode == kFwd ? static_cast<cuuint32_t>(bn) : 64u};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(nib), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_detail("cuTensorMapEncodeTiled (codes) failed with CUresult %d (N=%lld K=%lld)", static_cast<int>(r),
               static_cast<long long>(N), static_cast<long long>(K));
    return NF4LL_ERR_CUDA;
  }
  return NF4LL_OK;
}

struct Plan {
  int pair;                // 1: CTA-pair kernel (tcgen05 cta_group::2), tile (bm_tiles x 256) x 256 per pair
  int bm_tiles, bn, splits;
  int launch_splits;       // grid depth actually launched: `splits`, except under nf4ll_test_expire_wait
  int64_t tiles_m, tiles_o, m_pad;
  int64_t left_bytes, bt_bytes, counter_bytes, partial_bytes;
  int64_t total() const { return left_bytes + bt_bytes + counter_bytes + partial_bytes; }
};

// Tile shape / split count forced by a test (zeros: the built-in heuristic). flags bit 0: never use the
// cooperative (shared) split reduction.
struct Tune {
  int bm = 0, bn = 0, splits = 0, flags = 0;
  bool any() const { return bm || bn || splits; }
};
static thread_local Tune g_tune;
static thread_local uint32_t g_expire_polls = 0;      // nf4ll_test_expire_wait: one-shot
static thread_local cudaEvent_t g_ev_start = nullptr, g_ev_stop = nullptr;

// Record a measurement event on `stream`; inside a stream capture the record becomes a node of the graph that is
// executed (and timed) at every replay
static int record_event(cudaEvent_t ev, cudaStream_t stream) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  NF4LL_CUDA(cudaStreamIsCapturing(stream, &st));
  if (st == cudaStreamCaptureStatusActive) NF4LL_CUDA(cudaEventRecordWithFlags(ev, stream, cudaEventRecordExternal));
  else NF4LL_CUDA(cudaEventRecord(ev, stream));
  return NF4LL_OK;
}

static int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

static Plan make_plan(int mode, int64_t M, int64_t NO, int64_t KC, int r, int sms, const Tune& tune) {
  Plan pl;
  // CTA pairs whenever the output is wide enough for a 256-column tile and tall enough to fill the
  // pair's 256 accumulator rows; the single-CTA kernel serves narrow or short problems.
  // Measured on B200 (M = 2048, Qwen2.5-1.5B shapes): the pair is 8-10 % faster for backward-dX and a few
  // per cent slower for forward, whose single-CTA pipeline has less cross-CTA latency to hide.
  pl.pair = (mode == kBwd && NO > 128 && M > 128) ? 1 : 0;
  pl.bn = (NO % 256 == 0 || NO > 256) ? 256 : 128;
  if (NO <= 128) pl.bn = 128;
  pl.bm_tiles = (M > 128) ? 2 : 1;
  if (pl.pair) { pl.bn = 256; pl.bm_tiles = (M > 256) ? 2 : 1; }
  if (tune.bn == 512) { pl.pair = 1; pl.bn = 256; }          // testing hook: 512 asks for the pair kernel
  else if (tune.bn) { pl.pair = 0; pl.bn = tune.bn; if (!tune.bm) pl.bm_tiles = (M > 128) ? 2 : 1; }
  if (tune.bm) pl.bm_tiles = tune.bm;
  const int64_t bm = pl.bm_tiles * (pl.pair ? 256 : 128);       // rows per tile (per pair or per CTA)
  pl.tiles_m = (M + bm - 1) / bm;
  pl.tiles_o = (NO + pl.bn - 1) / pl.bn;
  pl.m_pad = pl.tiles_m * bm;
  const int64_t ctas = pl.tiles_m * pl.tiles_o * (pl.pair ? 2 : 1);
  const int64_t nkb = KC / 64;
  int splits = 1;
  if (ctas * 2 <= sms) {                        // less than half a wave: split the contraction
    splits = static_cast<int>(sms / ctas);
    const int64_t max_by_k = nkb / 4 > 0 ? nkb / 4 : 1;     // at least 4 stages per split
    if (splits > max_by_k) splits = static_cast<int>(max_by_k);
    if (splits > 16) splits = 16;
    if (splits < 1) splits = 1;
  }
  if (tune.splits) splits = tune.splits;
  if (splits > nkb) splits = static_cast<int>(nkb > 0 ? nkb : 1);
  pl.splits = splits;
  pl.launch_splits = splits;
  pl.left_bytes = r > 0 ? align256(M * r * 4) : 0;      // fp32 rank-16 projection when the caller does not keep it
  pl.bt_bytes = r > 0 ? align256(KC * r * 2) : 0;      // room for lora_B transposed (backward only uses it)
  pl.counter_bytes = splits > 1 ? align256(ctas * 4) : 0;      // one per CTA-owned block of output rows
  pl.partial_bytes = splits > 1 ? align256(static_cast<int64_t>(splits) * pl.m_pad * NO * 4) : 0;
  return pl;
}

static int device_sms(int* sms) {
  int dev = 0;
  NF4LL_CUDA(cudaGetDevice(&dev));
  // Planning only needs a stable number; without a device (host-only queries) assume a B200.
  if (cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || *sms <= 0) *sms = 148;
  return NF4LL_OK;
}

// Whether a cooperative grid of `ctas` CTAs can be resident at once, given how many CTAs of the kernel fit
// one SM and how many SMs the device offers.
bool coop_grid_fits(int64_t ctas, int ctas_per_sm, int sms) {
  return ctas_per_sm > 0 && sms > 0 && ctas <= static_cast<int64_t>(ctas_per_sm) * sms;
}

template <int MODE, int BM_TILES, int BN>
static int launch_cfg(const CUtensorMap& map, const CUtensorMap& nib_map, const CUtensorMap& out_map, const CUtensorMap& out_u,
                      const CUtensorMap& out_h, const GemmParams& p_in, const Plan& pl, cudaStream_t stream) {
  using Cfg = TileCfg<BM_TILES, BN>;
  auto kernel = nf4_gemm_kernel<MODE, BM_TILES, BN>;
  NF4LL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
  dim3 grid(static_cast<unsigned>(pl.tiles_o), static_cast<unsigned>(pl.tiles_m), static_cast<unsigned>(pl.launch_splits));
  GemmParams p = p_in;
  if (p.coop) {
    // split-K with a shared reduction: the splits of a tile wait for one another, which is only legal when
    // the whole grid is resident at once (cooperative launch). Ask the runtime how many CTAs of this kernel
    // an SM holds (fewer SMs or less shared memory may be usable than a bare B200 offers).
    int per_sm = 0, dev = 0, sms = 0;
    NF4LL_CUDA(cudaGetDevice(&dev));
    NF4LL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    NF4LL_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, Cfg::kThreads, Cfg::kSmemBytes));
    if (!coop_grid_fits(static_cast<int64_t>(grid.x) * grid.y * pl.splits, per_sm, sms)) p.coop = 0;
  }
  for (;;) {
    PdlLaunch lc(grid, dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, 0, 0, p.coop != 0);
    const cudaError_t err = cudaLaunchKernelEx(&lc.cfg, kernel, map, nib_map, out_map, out_u, out_h, p);
    if (err == cudaErrorCooperativeLaunchTooLarge && p.coop) {
      // the runtime disagrees after all: the last-CTA reduction needs no co-residency (counters are already zero)
      (void)cudaGetLastError();
      p.coop = 0;
      continue;
    }
    NF4LL_CUDA(err);
    break;
  }
  NF4LL_CUDA(cudaGetLastError());
  return NF4LL_OK;
}

template <int MODE>
static int launch(const CUtensorMap& map, const CUtensorMap& nib_map, const CUtensorMap& out_map, const GemmParams& p,
                  const Plan& pl, cudaStream_t stream) {
  // the two extra output maps are only read in the gate|up mode
  if (pl.bm_tiles == 2 && pl.bn == 256) return launch_cfg<MODE, 2, 256>(map, nib_map, out_map, out_map, out_map, p, pl, stream);
  if (pl.bm_tiles == 1 && pl.bn == 256) return launch_cfg<MODE, 1, 256>(map, nib_map, out_map, out_map, out_map, p, pl, stream);
  if (pl.bm_tiles == 2 && pl.bn == 128) return launch_cfg<MODE, 2, 128>(map, nib_map, out_map, out_map, out_map, p, pl, stream);
  return launch_cfg<MODE, 1, 128>(map, nib_map, out_map, out_map, out_map, p, pl, stream);
}

static int check_mat(const nf4ll_mat* W, const char* who) {
  if (!W || !W->nib || !W->qabs || !W->scale2 || !W->offset2 || !W->code2) {
    set_detail("%s: null weight pointer", who);
    return NF4LL_ERR_NULL;
  }
  if (W->N <= 0 || W->K <= 0 || W->K % 64 || W->N % 64 || (W->N * W->K) % 16384) {
    set_detail("%s: W[%lld,%lld]: N and K must be multiples of 64 and N*K of 16384", who, static_cast<long long>(W->N),
               static_cast<long long>(W->K));
    return NF4LL_ERR_SHAPE;
  }
  if (reinterpret_cast<uintptr_t>(W->nib) & 15) {
    set_detail("%s: nib must be 16-byte aligned", who);
    return NF4LL_ERR_ALIGN;
  }
  return NF4LL_OK;
}

static int check_act(const void* ptr, int64_t ld, int64_t cols, const char* who, const char* what) {
  if (!ptr) { set_detail("%s: %s is null", who, what); return NF4LL_ERR_NULL; }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ld % 8 || ld < cols) {
    set_detail("%s: %s must be 16-byte aligned with a leading dimension that is a multiple of 8 and >= %lld (got %lld)",
               who, what, static_cast<long long>(cols), static_cast<long long>(ld));
    return NF4LL_ERR_ALIGN;
  }
  return NF4LL_OK;
}

static int check_lora(const nf4ll_lora* l, const char* who, int64_t K) {
  if (!l) return NF4LL_OK;
  if (l->r != 16) { set_detail("%s: LoRA rank %d", who, l->r); return NF4LL_ERR_RANK; }
  if (!l->A || !l->B) { set_detail("%s: LoRA A/B null", who); return NF4LL_ERR_NULL; }
  if ((reinterpret_cast<uintptr_t>(l->A) & 15) || (reinterpret_cast<uintptr_t>(l->B) & 15) ||
      (reinterpret_cast<uintptr_t>(l->Bt) & 15)) {
    set_detail("%s: LoRA A/B must be 16-byte aligned", who);
    return NF4LL_ERR_ALIGN;
  }
  if (l->mask && ((reinterpret_cast<uintptr_t>(l->mask) & 15) || l->ld_mask % 16 || l->ld_mask < K)) {
    set_detail("%s: mask must be 16-byte aligned with ld_mask a multiple of 16 and >= K", who);
    return NF4LL_ERR_ALIGN;
  }
  return NF4LL_OK;
}

int lora_down_launch(const void* act, int64_t ldact, const uint8_t* mask, int64_t ld_mask, float keep_scale,
                     const void* R, float scale, int64_t M, int64_t C, void* t32, int* zero_ptr, int zero_words,
                     cudaStream_t stream);
int transpose_n16_launch(const void* B, void* Bt, int64_t N, cudaStream_t stream);
int launch_pair(int mode, int bm_tiles, const CUtensorMap& map, const CUtensorMap& nib_map, const CUtensorMap& out_map,
                const GemmParams& p, int64_t tiles_o, int64_t tiles_mp, int splits, int launch_splits, cudaStream_t stream);
int stream_forward_launch(const nf4ll_mat* W, const void* x, int64_t ldx, const void* bias, const float* t32,
                          const void* lora_b, float lora_scale, int64_t M, void* y, int64_t ldy, void* scratch,
                          bool counters_zeroed, int force_slices, cudaStream_t stream);
int64_t stream_workspace_bytes(int64_t N, int64_t K, int64_t M, int sms, int force_slices);
int swap_forward_launch(const nf4ll_mat* W, const void* x, int64_t ldx, const void* bias, const float* t32,
                        const void* lora_b, float lora_scale, int64_t M, void* y, int64_t ldy, void* scratch,
                        bool counters_zeroed, int force_slices, int32_t* status, cudaStream_t stream);
int64_t swap_workspace_bytes(int64_t N, int64_t K, int64_t M, int sms, int force_slices);
constexpr int64_t kStreamMaxRows = 16;     // at or below this many token rows the forward is a weight-streaming pass
constexpr int64_t kStreamCapRows = 64;     // the streaming kernel's own limit (reachable through the tuning hook)
constexpr int64_t kSwapMaxRows = 64;       // limit of the swapped-operand kernel (weights as the MMA's M operand)
// measured on B200 against the streaming kernel (two token tiles) and the 128-row tiles: the swapped-operand kernel
// wins from 9 rows up on weights of at least 2^24 elements, and up to 64 rows on weights of at least 2^26
constexpr int64_t kSwapMinRows = 9;
constexpr int64_t kSwapMidRows = 32;
constexpr int64_t kSwapMinWeights = int64_t(1) << 24;
constexpr int64_t kSwapBigWeights = int64_t(1) << 26;

// Which kernel computes a forward of M rows: the 256 x 256 / 128-row tile kernels (kTiles), the register-level
// weight-streaming kernel for decode-sized batches (kStream), or the swapped-operand tensor-core kernel for
// short batches of 9 to 64 rows against a large weight (kSwap). Bits 1 and 2 of the tuning flags force kStream /
// kSwap up to that kernel's limit.
enum : int { kTiles = 0, kStream = 1, kSwap = 2 };
static int forward_kind(int mode, int64_t M, int64_t N, int64_t K, bool stacked, const Tune& tune) {
  if (mode != kFwd || stacked) return kTiles;
  if (tune.flags & 2) return M <= kStreamCapRows ? kStream : kTiles;
  const bool swap_ok = M <= kSwapMaxRows && N * (K / 64) < (int64_t(1) << 31);      // the kernel indexes quantisation blocks with 32 bits
  if (tune.flags & 4) return swap_ok ? kSwap : kTiles;
  if (tune.any()) return kTiles;
  if (swap_ok && M >= kSwapMinRows && N * K >= (M <= kSwapMidRows ? kSwapMinWeights : kSwapBigWeights)) return kSwap;
  if (M <= kStreamMaxRows) return kStream;
  return kTiles;
}

static int64_t small_batch_scratch(int kind, int64_t N, int64_t K, int64_t M, int sms, int force_slices) {
  return kind == kStream ? stream_workspace_bytes(N, K, M, sms, force_slices) : swap_workspace_bytes(N, K, M, sms, force_slices);
}

// `segments` (forward only): the weight is several projections stacked along N, each with its own
// optional LoRA branch; `lora` / `side_out` are then unused.
static int run_gemm(int mode, const nf4ll_mat* W, const void* act, int64_t ldact, const void* bias,
                    const nf4ll_lora* lora, void* side_out, int64_t M, void* out, int64_t ldo, int accumulate,
                    void* workspace, int64_t workspace_bytes, int32_t* status, void* stream_v,
                    const nf4ll_segment* segments = nullptr, int n_segments = 0) {
  const char* who = segments ? "nf4ll_forward_multi" : (mode == kFwd ? "nf4ll_forward" : "nf4ll_backward_dx");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (int rc = check_mat(W, who)) return rc;
  if (M < 0) { set_detail("%s: M=%lld", who, static_cast<long long>(M)); return NF4LL_ERR_SHAPE; }
  if (M == 0) return NF4LL_OK;
  const int64_t NO = mode == kFwd ? W->N : W->K, KC = mode == kFwd ? W->K : W->N;
  if (int rc = check_act(act, ldact, KC, who, mode == kFwd ? "x" : "dy")) return rc;
  if (int rc = check_act(out, ldo, NO, who, mode == kFwd ? "y" : "dx")) return rc;
  if (int rc = check_lora(lora, who, W->K)) return rc;
  if (bias && (reinterpret_cast<uintptr_t>(bias) & 15)) { set_detail("%s: bias must be 16-byte aligned", who); return NF4LL_ERR_ALIGN; }
  if (M > (int64_t(1) << 30)) { set_detail("%s: M too large", who); return NF4LL_ERR_SHAPE; }
  if (int rc = require_sm100()) return rc;
  int sms = 148;
  if (int rc = device_sms(&sms)) return rc;
  bool narrow_tiles = false;       // a segment boundary that is not a multiple of 256 columns needs 128-column tiles
  if (segments) {
    if (n_segments < 1 || n_segments > kMaxSegments) { set_detail("%s: %d segments (1..%d)", who, n_segments, kMaxSegments); return NF4LL_ERR_SHAPE; }
    int64_t at = 0;
    for (int i = 0; i < n_segments; ++i) {
      if (segments[i].rows <= 0 || segments[i].rows % 128) {
        set_detail("%s: segment %d has %lld rows (multiples of 128)", who, i, static_cast<long long>(segments[i].rows));
        return NF4LL_ERR_SHAPE;
      }
      if (at % 256) narrow_tiles = true;
      at += segments[i].rows;
      if (int rc = check_lora(segments[i].lora, who, W->K)) return rc;
      if (segments[i].lora && !segments[i].t_out) { set_detail("%s: segment %d has LoRA but no t_out", who, i); return NF4LL_ERR_NULL; }
    }
    if (at != W->N) { set_detail("%s: segments cover %lld of %lld rows", who, static_cast<long long>(at), static_cast<long long>(W->N)); return NF4LL_ERR_SHAPE; }
  }
  Tune tune = g_tune;
  if (segments && (narrow_tiles || tune.bn == 512)) tune.bn = narrow_tiles ? 128 : 256;
  Plan pl = make_plan(mode, M, NO, KC, lora ? lora->r : 0, sms, tune);
  const int kind = forward_kind(mode, M, W->N, W->K, segments != nullptr, tune);
  const int force_slices = (tune.flags & 6) ? tune.splits : 0;
  const int64_t need = kind != kTiles ? pl.left_bytes + pl.bt_bytes + small_batch_scratch(kind, W->N, W->K, M, sms, force_slices)
                                      : pl.total();
  if (need > 0) {
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) || workspace_bytes < need) {
      set_detail("%s: needs a 256-byte aligned workspace of %lld bytes (got %lld)", who,
                 static_cast<long long>(need), static_cast<long long>(workspace_bytes));
      return NF4LL_ERR_WORKSPACE;
    }
  }
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  GemmParams p{};
  p.nib = W->nib; p.qabs = W->qabs; p.scale2 = W->scale2; p.offset2 = W->offset2; p.code2 = W->code2;
  p.N = W->N; p.K = W->K; p.M = M; p.NO = NO; p.KC = KC;
  p.out = static_cast<__half*>(out); p.ldo = ldo;
  p.bias = static_cast<const __half*>(bias);
  p.accumulate = accumulate;
  p.has_lora = lora != nullptr;
  p.splits = pl.splits; p.m_pad = pl.m_pad; p.status = status; p.spin_limit = kCoopSpinLimit;
  // one CTA per SM (shared memory): a split-K grid of at most `sms` CTAs is resident as a whole; the launch
  // itself re-checks this against the runtime's occupancy figure for the kernel it picks
  {
    const int64_t ctas = pl.tiles_o * pl.tiles_m * pl.splits * (pl.pair ? 2 : 1);
    p.coop = (pl.splits > 1 && coop_grid_fits(ctas, 1, sms) && !(tune.flags & 1)) ? 1 : 0;
  }
  const uint32_t expire = g_expire_polls;
  if (expire && p.coop && pl.splits > 1) {
    // test hook: launch one split short, so that every tile's counter stays below `splits` and each CTA's
    // bounded wait on it runs out after `expire` polls
    g_expire_polls = 0;
    pl.launch_splits = pl.splits - 1;
    p.spin_limit = expire;
  }
  int* counters = nullptr;
  int counter_words = 0;
  if (kind == kStream) {
    counters = reinterpret_cast<int*>(ws + pl.left_bytes + pl.bt_bytes);      // next-unit counter + one per 16 weight rows
    counter_words = static_cast<int>(1 + W->N / 16);
  } else if (kind == kSwap) {
    counters = reinterpret_cast<int*>(ws + pl.left_bytes + pl.bt_bytes);      // one per tile of 128 weight rows
    counter_words = static_cast<int>((W->N + 127) / 128);
  } else if (pl.splits > 1) {
    counters = reinterpret_cast<int*>(ws + pl.left_bytes + pl.bt_bytes);
    counter_words = static_cast<int>(pl.counter_bytes / sizeof(int));
  }
  if (segments) {
    int64_t at = 0;
    p.n_seg = n_segments;
    for (int i = 0; i < n_segments; ++i) {
      const nf4ll_lora* l = segments[i].lora;
      p.seg_begin[i] = at;
      if (l) {
        // the rank-16 projection of this segment: computed here unless the producer of x already wrote it
        if (!segments[i].t_ready)
          if (int rc = lora_down_launch(act, ldact, l->mask, l->ld_mask, l->keep_scale, l->A, 1.0f, M, W->K, segments[i].t_out,
                                        nullptr, 0, stream)) return rc;
        p.seg_left[i] = static_cast<const float*>(segments[i].t_out);
        p.seg_right[i] = static_cast<const __half*>(l->B) - at * 16;      // indexed by the fused output column
        p.seg_scale[i] = l->scale;
      }
      at += segments[i].rows;
    }
  }
  if (lora) {
    // rank-16 projection of the activation, fp32: T = drop(x).A^T (forward) or U = s.dy.B (backward);
    // it lands in the caller's t_out / u_out when given, else in the workspace. The same kernel
    // resets the split-K tile counters of the GEMM that follows it on the stream.
    float* left = side_out ? static_cast<float*>(side_out) : reinterpret_cast<float*>(ws);
    if (mode == kFwd) {
      if (int rc = lora_down_launch(act, ldact, lora->mask, lora->ld_mask, lora->keep_scale, lora->A, 1.0f, M, W->K, left,
                                    counters, counter_words, stream)) return rc;
      p.lora_right = static_cast<const __half*>(lora->B);
      p.left_scale = lora->scale;
    } else {
      const void* bt = lora->Bt;
      if (!bt) {
        void* tmp = ws + pl.left_bytes;
        if (int rc = transpose_n16_launch(lora->B, tmp, W->N, stream)) return rc;
        bt = tmp;
      }
      if (int rc = lora_down_launch(act, ldact, nullptr, 0, 1.0f, bt, lora->scale, M, W->N, left, counters, counter_words,
                                    stream)) return rc;
      p.lora_right = static_cast<const __half*>(lora->A);
      p.left_scale = 1.0f;
      p.mask = lora->mask; p.ld_mask = lora->ld_mask; p.keep_scale = lora->keep_scale;
    }
    p.lora_left = left;
  }
  // the measurement hook is one-shot: whichever kernel computes this call's product consumes it
  cudaEvent_t ev0 = g_ev_start, ev1 = g_ev_stop;
  g_ev_start = g_ev_stop = nullptr;
  if (kind != kTiles) {
    if (ev0) { if (int rce = record_event(ev0, stream)) return rce; }
    const float* t32 = lora ? p.lora_left : nullptr;
    const void* lb = lora ? lora->B : nullptr;
    const float ls = lora ? lora->scale : 0.f;
    const int rc = kind == kStream
                       ? stream_forward_launch(W, act, ldact, bias, t32, lb, ls, M, out, ldo, counters, lora != nullptr,
                                               force_slices, stream)
                       : swap_forward_launch(W, act, ldact, bias, t32, lb, ls, M, out, ldo, counters, lora != nullptr,
                                             force_slices, status, stream);
    if (rc == NF4LL_OK && ev1) { if (int rce = record_event(ev1, stream)) return rce; }
    return rc;
  }
  if (pl.splits > 1) {
    p.counters = counters;
    p.partial = reinterpret_cast<float*>(ws + pl.left_bytes + pl.bt_bytes + pl.counter_bytes);
    if (!lora) NF4LL_CUDA(cudaMemsetAsync(p.counters, 0, pl.counter_bytes, stream));
  }
  CUtensorMap map;
  if (int rc = make_tile_map(&map, act, M, KC, ldact, false)) return rc;
  CUtensorMap out_map;
  if (pl.splits == 1) {
    if (int rc = make_tile_map(&out_map, out, M, NO, ldo, false)) return rc;
  } else {
    if (int rc = make_tile_map(&out_map, p.partial, static_cast<int64_t>(pl.splits) * pl.m_pad, NO, NO, true)) return rc;
  }
  CUtensorMap nib_map;
  if (int rc = make_nib_map(&nib_map, W->nib, W->N, W->K, mode, pl.pair ? 128 : pl.bn)) return rc;
  if (ev0) { if (int rce = record_event(ev0, stream)) return rce; }
  const int rc = pl.pair ? launch_pair(mode, pl.bm_tiles, map, nib_map, out_map, p, pl.tiles_o, pl.tiles_m, pl.splits,
                                       pl.launch_splits, stream)
                 : (mode == kFwd ? launch<kFwd>(map, nib_map, out_map, p, pl, stream)
                                 : launch<kBwd>(map, nib_map, out_map, p, pl, stream));
  if (rc == NF4LL_OK && ev1) { if (int rce = record_event(ev1, stream)) return rce; }
  return rc;
}

// Rows [begin, begin + rows) of a weight as a weight of its own (same columns).
static nf4ll_mat sub_rows(const nf4ll_mat* W, int64_t begin, int64_t rows) {
  nf4ll_mat m = *W;
  const int64_t e0 = begin * W->K;
  m.nib = W->nib + e0 / 2;
  m.qabs = W->qabs + e0 / 64;
  m.scale2 = W->scale2 + e0 / 16384;
  m.offset2 = W->offset2 + e0 / 16384;
  m.N = rows;
  return m;
}

// gate|up forward with the gated-SiLU product in the epilogue
static int run_gate_up(const nf4ll_mat* W, const void* x, int64_t ldx, const nf4ll_lora* lora_gate, const nf4ll_lora* lora_up,
                       void* t_gate, void* t_up, int64_t M, void* g, int64_t ldg, void* u, int64_t ldu, void* h, int64_t ldh,
                       void* workspace, int64_t workspace_bytes, int32_t* status, void* stream_v) {
  const char* who = "nf4ll_forward_gate_up";
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (int rc = check_mat(W, who)) return rc;
  if (M < 0 || W->N % 2) { set_detail("%s: M=%lld, %lld stacked rows", who, (long long)M, (long long)W->N); return NF4LL_ERR_SHAPE; }
  if (M == 0) return NF4LL_OK;
  const int64_t I = W->N / 2;
  if ((I * W->K) % 16384) { set_detail("%s: each half must hold whole second-level blocks", who); return NF4LL_ERR_SHAPE; }
  if (int rc = check_act(x, ldx, W->K, who, "x")) return rc;
  if (int rc = check_act(g, ldg, I, who, "g")) return rc;
  if (int rc = check_act(u, ldu, I, who, "u")) return rc;
  if (int rc = check_act(h, ldh, I, who, "h")) return rc;
  if (int rc = check_lora(lora_gate, who, W->K)) return rc;
  if (int rc = check_lora(lora_up, who, W->K)) return rc;
  if ((lora_gate && !t_gate) || (lora_up && !t_up)) { set_detail("%s: a LoRA branch needs its t_out", who); return NF4LL_ERR_NULL; }
  if (int rc = require_sm100()) return rc;
  if (M <= 128 || I % 128 || g_tune.any()) {
    // short batches and odd widths: the two projections on their own, then the stand-alone gated product
    const nf4ll_mat wg = sub_rows(W, 0, I), wu = sub_rows(W, I, I);
    if (int rc = run_gemm(kFwd, &wg, x, ldx, nullptr, lora_gate, t_gate, M, g, ldg, 0, workspace, workspace_bytes, status, stream_v)) return rc;
    if (int rc = run_gemm(kFwd, &wu, x, ldx, nullptr, lora_up, t_up, M, u, ldu, 0, workspace, workspace_bytes, status, stream_v)) return rc;
    return nf4ll_swiglu_forward(g, ldg, u, ldu, h, ldh, M, I, stream_v);
  }
  GemmParams p{};
  p.nib = W->nib; p.qabs = W->qabs; p.scale2 = W->scale2; p.offset2 = W->offset2; p.code2 = W->code2;
  p.N = W->N; p.K = W->K; p.M = M; p.NO = W->N; p.KC = W->K;
  p.out = static_cast<__half*>(g); p.ldo = ldg;
  p.splits = 1; p.status = status; p.spin_limit = kCoopSpinLimit;
  p.gu_inter = I;
  const nf4ll_lora* br[2] = {lora_gate, lora_up};
  void* tout[2] = {t_gate, t_up};
  for (int i = 0; i < 2; ++i) {
    if (!br[i]) continue;
    if (int rc = lora_down_launch(x, ldx, br[i]->mask, br[i]->ld_mask, br[i]->keep_scale, br[i]->A, 1.0f, M, W->K, tout[i],
                                  nullptr, 0, stream)) return rc;
    p.seg_left[i] = static_cast<const float*>(tout[i]);
    p.seg_right[i] = static_cast<const __half*>(br[i]->B);
    p.seg_scale[i] = br[i]->scale;
  }
  p.has_lora = (lora_gate || lora_up) ? 1 : 0;
  Plan pl{};
  pl.bm_tiles = 2; pl.bn = 256; pl.splits = 1; pl.launch_splits = 1; pl.pair = 0;
  pl.tiles_o = I / 128;
  pl.tiles_m = (M + 255) / 256;
  CUtensorMap map, nib_map, mg, mu, mh;
  if (int rc = make_tile_map(&map, x, M, W->K, ldx, false)) return rc;
  if (int rc = make_nib_map(&nib_map, W->nib, W->N, W->K, kFwd, 128)) return rc;
  if (int rc = make_tile_map(&mg, g, M, I, ldg, false)) return rc;
  if (int rc = make_tile_map(&mu, u, M, I, ldu, false)) return rc;
  if (int rc = make_tile_map(&mh, h, M, I, ldh, false)) return rc;
  cudaEvent_t ev0 = g_ev_start, ev1 = g_ev_stop;
  g_ev_start = g_ev_stop = nullptr;
  if (ev0) { if (int rce = record_event(ev0, stream)) return rce; }
  const int rc = launch_cfg<kFwd, 2, 256>(map, nib_map, mg, mu, mh, p, pl, stream);
  if (rc == NF4LL_OK && ev1) { if (int rce = record_event(ev1, stream)) return rce; }
  return rc;
}

}  // namespace nf4ll

extern "C" int nf4ll_forward_gate_up(const nf4ll_mat* W, const void* x, int64_t ldx, const nf4ll_lora* lora_gate,
                                     const nf4ll_lora* lora_up, void* t_gate, void* t_up, int64_t M, void* g, int64_t ldg,
                                     void* u, int64_t ldu, void* h, int64_t ldh, void* workspace, int64_t workspace_bytes,
                                     int32_t* status, void* stream) {
  return nf4ll::run_gate_up(W, x, ldx, lora_gate, lora_up, t_gate, t_up, M, g, ldg, u, ldu, h, ldh, workspace, workspace_bytes,
                            status, stream);
}

namespace nf4ll {
static int sms_or_default() {
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) sms = v;
  }
  return sms;
}

// Scratch of the forward plan(s) a call may run for W[N,K]: the default tile width and, because a stack of
// projections whose boundaries are not multiples of 256 columns is planned with 128-column tiles, that one too.
static int64_t forward_need(int64_t M, int64_t N, int64_t K, int r, int sms, const Tune& tune) {
  const Plan base = make_plan(kFwd, M, N, K, r, sms, tune);
  int64_t need = base.total();
  // the small-batch kernels keep counters and partial sums in the workspace too; with the kernels forced by
  // the tuning flags a split count may be forced as well
  const int fs = tune.splits;
  if (M <= kStreamCapRows) {
    const int64_t st = base.left_bytes + base.bt_bytes + stream_workspace_bytes(N, K, M, sms, fs);
    if (st > need) need = st;
  }
  if (M <= kSwapMaxRows) {
    const int64_t st = base.left_bytes + base.bt_bytes + swap_workspace_bytes(N, K, M, sms, fs);
    if (st > need) need = st;
  }
  if (!tune.bn) {
    Tune narrow = tune;
    narrow.bn = 128;
    const int64_t n = make_plan(kFwd, M, N, K, r, sms, narrow).total();
    if (n > need) need = n;
  }
  return need;
}
}  // namespace nf4ll

extern "C" int64_t nf4ll_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t r) {
  return nf4ll_workspace_bytes_tuned(M, N, K, r, 0, 0, 0);
}

extern "C" int64_t nf4ll_workspace_bytes_tuned(int64_t M, int64_t N, int64_t K, int32_t r, int32_t bm_tiles, int32_t bn,
                                               int32_t splits) {
  using namespace nf4ll;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  Tune tune;
  tune.bm = (bm_tiles == 1 || bm_tiles == 2) ? bm_tiles : 0;
  tune.bn = (bn == 128 || bn == 256 || bn == 512) ? bn : 0;
  tune.splits = splits > 0 ? splits : 0;
  const int sms = sms_or_default();
  const int64_t f = forward_need(M, N, K, r, sms, tune), b = make_plan(kBwd, M, K, N, r, sms, tune).total();
  return f > b ? f : b;
}

extern "C" int nf4ll_forward(const nf4ll_mat* W, const void* x, int64_t ldx, const void* bias, const nf4ll_lora* lora,
                             void* t_out, int64_t M, void* y, int64_t ldy, void* workspace, int64_t workspace_bytes,
                             int32_t* status, void* stream) {
  return nf4ll::run_gemm(nf4ll::kFwd, W, x, ldx, bias, lora, t_out, M, y, ldy, 0, workspace, workspace_bytes, status, stream);
}

extern "C" int nf4ll_forward_multi(const nf4ll_mat* W, const void* x, int64_t ldx, const void* bias,
                                   const nf4ll_segment* segments, int32_t n_segments, int64_t M, void* y, int64_t ldy,
                                   void* workspace, int64_t workspace_bytes, int32_t* status, void* stream) {
  if (!segments) { nf4ll::set_detail("nf4ll_forward_multi: segments is null"); return NF4LL_ERR_NULL; }
  return nf4ll::run_gemm(nf4ll::kFwd, W, x, ldx, bias, nullptr, nullptr, M, y, ldy, 0, workspace, workspace_bytes, status, stream,
                         segments, n_segments);
}

extern "C" int nf4ll_backward_dx(const nf4ll_mat* W, const void* dy, int64_t lddy, const nf4ll_lora* lora, void* u_out,
                                 int64_t M, void* dx, int64_t lddx, int32_t accumulate, void* workspace,
                                 int64_t workspace_bytes, int32_t* status, void* stream) {
  return nf4ll::run_gemm(nf4ll::kBwd, W, dy, lddy, nullptr, lora, u_out, M, dx, lddx, accumulate, workspace,
                         workspace_bytes, status, stream);
}

// Testing / tuning hook (no counterpart in the reference): force the tile shape and the split count
// chosen by the calling thread's next calls; zeros restore the built-in heuristic.
extern "C" void nf4ll_tune_override(int32_t bm_tiles, int32_t bn, int32_t splits, int32_t flags) {
  nf4ll::g_tune.bm = (bm_tiles == 1 || bm_tiles == 2) ? bm_tiles : 0;
  nf4ll::g_tune.bn = (bn == 128 || bn == 256 || bn == 512) ? bn : 0;
  nf4ll::g_tune.splits = splits > 0 ? splits : 0;
  nf4ll::g_tune.flags = flags;
}

// Measurement hook (no counterpart in the reference): the calling thread's NEXT forward / backward-dX call
// records `start` immediately before and `stop` immediately after the kernel that computes its product
// on the call's stream (the rank-16 prologue kernel stays outside the pair). One-shot.
extern "C" void nf4ll_kernel_events(void* start, void* stop) {
  nf4ll::g_ev_start = static_cast<cudaEvent_t>(start);
  nf4ll::g_ev_stop = static_cast<cudaEvent_t>(stop);
}

// Failure-detection test hook (no counterpart in the reference). One-shot.
extern "C" void nf4ll_test_expire_wait(uint32_t polls) { nf4ll::g_expire_polls = polls; }

// ---------------------------------------------------------------------------------------------
// Forward without a caller-supplied workspace.
//
// Some callers cannot hand over scratch memory: a plugin host that forbids device allocations after
// start-up, an inference server whose memory pool is sealed once its budget is committed, or code
// that runs where cudaMalloc is illegal. For them the scratch of nf4ll_forward lives in a fixed
// array in this library's device image. The array exists once per GPU that loads the library (each
// such GPU gives up NF4LL_STATIC_SCRATCH_BYTES until the process exits), so its size is a
// compromise: it covers one benchmark configuration-0 forward (M = 2048 against a 1536 x 1536 weight with
// LoRA, including split-K partial sums) and nothing much larger.
//
// In host code the array's name is only a handle; the device address is asked from the runtime
// once per device (with that device current) and cached.
// ---------------------------------------------------------------------------------------------
namespace nf4ll {

static __device__ __align__(256) unsigned char g_static_scratch[NF4LL_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static void* g_static_scratch_addr[kMaxDevices];      // written once per device with the same value by any thread

static int static_scratch_for_current_device(void** out) {
  int dev = 0;
  NF4LL_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    set_detail("nf4ll_forward_static: device index %d is beyond the %d devices this entry point tracks", dev, kMaxDevices);
    return NF4LL_ERR_SHAPE;
  }
  void* ptr = __atomic_load_n(&g_static_scratch_addr[dev], __ATOMIC_ACQUIRE);
  if (!ptr) {
    NF4LL_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
    if (!ptr || (reinterpret_cast<uintptr_t>(ptr) & 255)) {
      set_detail("nf4ll_forward_static: runtime returned an unusable address for the built-in scratch");
      return NF4LL_ERR_CUDA;
    }
    __atomic_store_n(&g_static_scratch_addr[dev], ptr, __ATOMIC_RELEASE);
  }
  *out = ptr;
  return NF4LL_OK;
}

}  // namespace nf4ll

extern "C" int nf4ll_forward_static(const nf4ll_mat* W, const void* x, int64_t ldx, const void* bias,
                                    const nf4ll_lora* lora, void* t_out, int64_t M, void* y, int64_t ldy, int32_t* status,
                                    void* stream) {
  using namespace nf4ll;
  if (!W) { set_detail("nf4ll_forward_static: null weight"); return NF4LL_ERR_NULL; }
  if (M < 0 || W->N <= 0 || W->K <= 0) { set_detail("nf4ll_forward_static: bad shape"); return NF4LL_ERR_SHAPE; }
  // only the forward plan this call will run counts (nf4ll_workspace_bytes also covers the backward)
  const int64_t need = forward_need(M, W->N, W->K, lora ? lora->r : 0, sms_or_default(), g_tune);
  if (need > static_cast<int64_t>(NF4LL_STATIC_SCRATCH_BYTES)) {
    set_detail("nf4ll_forward_static: this problem needs %lld bytes of scratch, the built-in buffer holds %lld; "
               "use nf4ll_forward with a workspace of your own",
               static_cast<long long>(need), static_cast<long long>(NF4LL_STATIC_SCRATCH_BYTES));
    return NF4LL_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  if (int rc = static_scratch_for_current_device(&scratch)) return rc;
  // Whatever the previous call left in the buffer is harmless: the tile counters are cleared on the
  // stream before every launch that uses them, and every other byte is written before it is read.
  return run_gemm(kFwd, W, x, ldx, bias, lora, t_out, M, y, ldy, 0, scratch, NF4LL_STATIC_SCRATCH_BYTES, status, stream);
}

