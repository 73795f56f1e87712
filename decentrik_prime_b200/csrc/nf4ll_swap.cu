// Short-batch forward (up to 64 token rows) with the roles of the operands swapped: the WEIGHTS are the 128-row
// M operand of tcgen05.mma and the token rows its N operand (16, 32 or 64 columns), so no MMA row is padding and
// the kernel's cost is the stream of NF4 bytes, like the decode-sized kernel's. Replaces, for such batches, the
// same reference call sites as the big-tile kernel (solution/fast_qwen.py:947, 1037, 1080-1112).
//
//   y^T[128 weight rows, tokens] = W_tile[128, K-slice] . x^T          (fp32 in tensor memory)
//
// The dequantised weights never touch shared memory: a decode thread owns one weight row of the tile (= one
// tensor-memory lane), turns the 32 bytes of codes of a quantisation block into 64 fp16 values with 32 loads
// from a lane-replicated 256-entry table of half2 level pairs (one byte permute, one multiply-add and one
// conflict-free 4-byte shared load per two weights), scales them by the block's absmax and writes them with ONE
// tcgen05.st into the A-operand region of tensor memory; the MMA reads A from tensor memory and the token tile
// from shared memory.
//
// One persistent CTA per SM. Codes arrive in coarse stages of four quantisation blocks (one "group", K = 256): a
// TMA box of 128 rows x 128 bytes (whole 128-byte lines) plus the 8-bit absmax codes of those blocks (4 bytes
// per row, copied by the producer warp's 32 lanes with cp.async so that they travel with the codes and cost no
// thread a DRAM round trip). Five to eight stages are in flight per SM. Token tiles (TMA, 128-byte swizzle; they
// come out of L2) travel in a ring of their own, one group (four tiles) per slot.
//
// Sixteen decode warps form four teams (one warp per tensor-memory lane quarter each). A team takes a HALF group
// (two blocks, K = 128, 64 columns of A operand) at a time, the half groups going round the teams, so that four
// half groups are being decoded at once and each team's chain of latencies (wait, shared loads, table loads,
// tcgen05.st, fence, arrive) overlaps the others'. Tensor memory holds three groups of A operand.
// What an MMA-issuing thread does per group is kept to one wait, up to sixteen MMAs whose descriptors differ by
// immediates, and one commit: a group's A operand and its token tiles share one "full" barrier (eight warp
// arrivals + the TMA bytes) and one "empty" barrier (the commit), three groups deep. Measured on B200: ONE thread
// issues an MMA of 128 x N x 16 (N <= 128, A in tensor memory) every 70-90 clocks whatever N is, while the tensor
// pipe is busy for a fraction of that; the rate adds up over issuing threads (2 threads: 48 clocks per MMA, 4: 24).
// So TWO threads issue, one the MMAs of the first two blocks of every group, the other those of the last two,
// each into an accumulator of its own; the epilogue adds the two.
// Barrier discipline: an mbarrier wait names a phase by its parity only, so every waiter must meet every phase of a
// barrier in order. Even groups (decoded by teams 0-1) and odd groups (teams 2-3) therefore use barriers of their own: the "full" / "empty" pair of a group is indexed by its running count modulo 6 (slot x parity), while
// the storage it guards (tensor-memory columns, token tiles) is indexed modulo 3.
//
// The scale is applied in fp16 (weight = fp16(fp16(NF4[c]) * fp16(absmax))), which differs from the big-tile
// kernel's bit-exact fp16(NF4[c] * absmax) by a few 2^-11 relative roundings, inside the 1e-3 tolerance of the path.
//
// A unit of work = (tile of 128 weight rows) x (slice of the contraction); CTA c takes units c, c + grid, ...
// With more than one slice the units of a tile leave their partial sums in a slab of the workspace and the last
// one to arrive adds them up in slice order (a fixed order), adds bias and the LoRA term and stores fp16.
//
// Warp roles: 0 producer of codes (TMA) and absmax codes (cp.async), 1 tensor-memory allocation + MMA issue (first
// half of every group), 2 TMA producer of token tiles, 3..18 decode and then the epilogue, 19 MMA issue (second half). Every wait is bounded and reports through
// the status word.
#include "nf4ll_gemm_shared.cuh"

namespace nf4ll {

struct SwapParams {
  const uint8_t* qabs;
  const float* scale2;
  const float* offset2;
  const float* code2;
  int64_t N, K, M;
  __half* y;
  int64_t ldy;
  const __half* bias;
  const float* t32;        // [M,16] fp32 = drop(x) . A^T, or null (no LoRA)
  const __half* lora_b;    // [N,16]
  float lora_scale;
  int slices;              // slices of the contraction
  int groups_per_slice;    // groups of four quantisation blocks per slice
  int n_units;             // tiles * slices
  float* slab;             // [tiles][slices][NTOK][128] fp32 partial sums (slices > 1)
  int* counters;           // [tile]: arrivals (zero on entry)
  int32_t* status;
};

constexpr int kSwapThreads = 640;            // code producer, MMA issuer, token-tile producer, 16 decode warps, second MMA issuer
constexpr int kSwapIssuers = 2;              // MMA-issuing threads, each with its own accumulator
constexpr int kSwapIssuerWarp1 = 19;
constexpr int kSwapTeams = 4;
constexpr int kSwapDecodeWarps = 4 * kSwapTeams;
constexpr int kSwapFirstDecodeWarp = 3;
constexpr int kSwapAGrp = 3;                 // groups of A operand in tensor memory (128 columns each) = groups of token tiles in flight
constexpr int kSwapCodeBytes = 128 * 128;
constexpr int kSwapTableBytes = 256 * 128;

template <int NTOK>
struct SwapCfg {
  static constexpr int kXBytes = NTOK * 128;                       // one token tile: NTOK rows x 64 fp16
  static constexpr int kXGBytes = 4 * kXBytes;                     // the four token tiles of a group
  static constexpr int kXG = kSwapAGrp;                            // groups of token tiles in flight (they come from L2)
  // coarse stages in flight: codes of four blocks (16 KB) + their absmax codes. An EVEN number: a team reads the
  // groups of one parity only, and must meet every phase of a stage's barrier (a parity wait cannot skip one)
  // (a power of two, so that the stage and its phase are a mask and a shift of the running count)
  static constexpr int kCSt = NTOK == 64 ? 4 : 8;
  static constexpr int kAbsOff = kSwapCodeBytes;                   // absmax codes of the stage: [128 rows][4 blocks] bytes
  static constexpr int kStageBytes = kSwapCodeBytes + 1024;        // kept a multiple of 1024 for the swizzled codes
  static constexpr int kDCols = 64 * kSwapIssuers;                 // accumulator columns reserved: 64 per issuing thread
  static constexpr int kTmemCols = 512;                            // 2 accumulators + 3 x 128 A columns
  static constexpr int kSmemBytes = 1024 + kCSt * kStageBytes + kXG * kXGBytes + kSwapTableBytes + 1024 + 512;
  static_assert(kDCols + kSwapAGrp * 128 <= kTmemCols, "tensor memory budget");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

// 4-byte asynchronous copy global -> shared, and the arrive that fires on `bar` once all copies this
// thread has issued so far have landed (it counts as one of the barrier's expected arrivals)
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
// a wait for the threads on the kernel's critical path: polls without the slow path's bookkeeping until the limit
__device__ __forceinline__ bool swap_wait(uint32_t bar, uint32_t parity, const Abort& ab, int code) {
  if (mbar_test_wait(bar, parity)) return true;
  for (uint32_t i = 0; i < 16u; ++i)
    if (mbar_try_wait_hint(bar, parity, kParkNs)) return true;
  return wait_or_abort(bar, parity, ab, code);
}

// D[tmem] (+)= A[tmem] . B[smem]: the A operand (128 rows x 16 fp16, two per 32-bit column) comes from tensor memory
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ uint32_t lds_u32s(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// address of the table entry of byte I of `w` for this lane: one byte permute isolates the byte, one
// multiply-add (the other arithmetic pipe) scales it by the entry stride of 128 bytes and adds the lane's base
template <int I>
__device__ __forceinline__ uint32_t swap_entry(uint32_t w, uint32_t lane_base) {
  uint32_t addr;
  const uint32_t byte = prmt(w, 0u, 0x4440u | I);
  asm("mad.lo.u32 %0, %1, 128, %2;" : "=r"(addr) : "r"(byte), "r"(lane_base));
  return addr;
}

// eight weights of one word of codes (high nibble first), scaled by the block's absmax (both halves of `am2`)
__device__ __forceinline__ void swap_decode8(uint32_t w, uint32_t lane_base, uint32_t am2, uint32_t* out) {
  const __half2 a = *reinterpret_cast<const __half2*>(&am2);
  uint32_t h[4];
  h[0] = lds_u32s(swap_entry<0>(w, lane_base));
  h[1] = lds_u32s(swap_entry<1>(w, lane_base));
  h[2] = lds_u32s(swap_entry<2>(w, lane_base));
  h[3] = lds_u32s(swap_entry<3>(w, lane_base));
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&h[j]), a);
    out[j] = *reinterpret_cast<const uint32_t*>(&v);
  }
}

// 32 lanes x 16 consecutive 32-bit columns, registers -> tensor memory
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}

// 32 lanes x 16 consecutive fp32 columns
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

template <int NTOK>
__global__ void __launch_bounds__(kSwapThreads, 1)
nf4_swap_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_nib, const SwapParams p) {
  using Cfg = SwapCfg<NTOK>;
  // x, the weights and code2 may be read at once (what precedes this kernel on the stream is the rank-16
  // projection kernel, itself started only after all earlier work had finished, or a memset, which orders this
  // kernel after everything before it); the first write to global memory waits for the predecessor.
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kCSt = Cfg::kCSt;
  uint8_t* sStage = smem;                        // [kCSt] { codes [128 rows][128 B] (128-byte swizzle) | absmax codes [128 rows][4] }
  uint8_t* sX = sStage + kCSt * Cfg::kStageBytes;               // [kXG][4] token tiles [NTOK rows][128 B], 128-byte swizzle
  uint32_t* sTbl = reinterpret_cast<uint32_t*>(sX + Cfg::kXG * Cfg::kXGBytes);
  float* sCode2 = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(sTbl) + kSwapTableBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sCode2) + 1024);
  uint64_t* a_full = bars;                       // [kSwapAGrp] eight decode warps stored the group's A operand and its token tiles landed
  uint64_t* a_empty = a_full + 8;                // [kSwapAGrp] the MMAs that read the group (A operand and token tiles) have completed
  uint64_t* grp_full = a_empty + 8;              // [kCSt] codes and absmax codes landed
  uint64_t* grp_empty = grp_full + 8;            // [kCSt] the eight decode warps of the group's two half groups have read it
  uint64_t* drain = grp_empty + 8;               // [kSwapIssuers] used only when a wait has failed: the issuer's MMAs have all completed
  uint64_t* acc_full = drain + 2;
  uint64_t* acc_empty = acc_full + 1;            // the epilogue has read the accumulator (sixteen decode warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = abort_flag + 1;
  volatile int* stop_flag = abort_flag + 2;
  uint32_t* sLv = tmem_slot + 4;                 // 16 level bit patterns

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bpr = static_cast<int>(p.K / 64);
  const Abort ab{abort_flag, p.status};
  // unit u -> (tile, first block, number of blocks); every role walks the same sequence u = blockIdx.x, + gridDim.x, ...
  auto unit_range = [&](int u, int& tile, int& sl, int& blk_begin, int& nblk) {
    tile = u / p.slices;
    sl = u - tile * p.slices;
    blk_begin = sl * p.groups_per_slice * 4;
    int blk_end = blk_begin + p.groups_per_slice * 4;
    if (blk_end > bpr) blk_end = bpr;
    nblk = blk_end - blk_begin;                 // > 0 by construction of the slices
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2 * kSwapAGrp; ++s) {
      mbar_init(smem_u32(a_full + s), 8 + 1);          // the warps of the group's two half groups + the token tiles' TMA bytes
      mbar_init(smem_u32(a_empty + s), kSwapIssuers);  // one commit per issuing thread
    }
    for (int s = 0; s < kSwapIssuers; ++s) mbar_init(smem_u32(drain + s), 1);
    for (int s = 0; s < kCSt; ++s) {
      mbar_init(smem_u32(grp_full + s), 1 + 32);       // TMA bytes + the producer warp's 32 lanes (their absmax-code copies)
      mbar_init(smem_u32(grp_empty + s), 8);
    }
    mbar_init(smem_u32(acc_full), kSwapIssuers);
    mbar_init(smem_u32(acc_empty), kSwapDecodeWarps);
    *abort_flag = 0;
    *last_flag = 0;
    *stop_flag = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < 16) {
    constexpr float lv[16] = {NF4LL_LEVELS};
    float v = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) v = (static_cast<int>(threadIdx.x) == j) ? lv[j] : v;
    sLv[threadIdx.x] = __half_as_ushort(__float2half_rn(v));
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
  for (int idx = threadIdx.x; idx < 256 * 8; idx += kSwapThreads) {     // four lanes' copies of an entry per 16-byte store
    const int v = idx >> 3;                          // byte value: even element in the high nibble
    const uint32_t e = sLv[v >> 4] | (sLv[v & 15] << 16);
    reinterpret_cast<uint4*>(sTbl)[idx] = make_uint4(e, e, e, e);
  }
  __syncthreads();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kACol0 = Cfg::kDCols;

  if (warp == 0) {
    // ----------------------------------------------------------------------------- producer of codes and absmax codes
    // All 32 lanes walk the groups together: lane 0 issues the TMA box of the codes, every lane copies the
    // 4 absmax codes (one 32-bit word) of tile rows lane, lane + 32, lane + 64, lane + 96. A group's word of a row
    // is 4-byte aligned when the row length in blocks is a multiple of four; otherwise, and for a last group of
    // fewer than four blocks (its word would run past the row, for the last row past the array), the bytes are
    // fetched one by one.
    if (lane == 0) tma_prefetch_desc(&tmap_nib);
    const bool words_ok = (bpr & 3) == 0;
    int cg = 0;                                   // coarse stages issued so far, over all units
    bool ok = true;
    for (int u = blockIdx.x; ok && u < p.n_units; u += gridDim.x) {
      int tile, sl, blk_begin, nblk;
      unit_range(u, tile, sl, blk_begin, nblk);
      const int ngrp = (nblk + 3) / 4;
      int64_t qrow[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int64_t n = static_cast<int64_t>(tile) * 128 + lane + 32 * e;
        if (n >= p.N) n = p.N - 1;                 // tail rows: any valid row; their output is never stored
        qrow[e] = n * bpr + blk_begin;
      }
      for (int gidx = 0; gidx < ngrp; ++gidx, ++cg) {
        const int c = cg % kCSt;
        if (!wait_or_abort(smem_u32(grp_empty + c), ((cg / kCSt) & 1) ^ 1, ab, 0x0502)) { ok = false; break; }
        const uint32_t stage = smem_u32(sStage + c * Cfg::kStageBytes);
        const int nb = (nblk - gidx * 4 < 4) ? nblk - gidx * 4 : 4;
        if (lane == 0) {
          mbar_arrive_expect_tx(smem_u32(grp_full + c), kSwapCodeBytes);
          tma_load_2d(stage, &tmap_nib, (blk_begin + gidx * 4) * 32, tile * 128, smem_u32(grp_full + c));
        }
        if (words_ok && nb == 4) {
#pragma unroll
          for (int e = 0; e < 4; ++e) cp_async4(stage + Cfg::kAbsOff + (lane + 32 * e) * 4, p.qabs + qrow[e] + gidx * 4);
          cp_async_arrive(smem_u32(grp_full + c));
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint32_t w = 0;
            for (int j = 0; j < nb; ++j) w |= static_cast<uint32_t>(__ldg(p.qabs + qrow[e] + gidx * 4 + j)) << (8 * j);
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(stage + Cfg::kAbsOff + (lane + 32 * e) * 4), "r"(w) : "memory");
          }
          mbar_arrive(smem_u32(grp_full + c));
        }
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    if (lane == 0 && *abort_flag) {
      // give copies still in flight a bounded chance to land before the CTA goes away
      for (int k = (cg > kCSt ? cg - kCSt : 0); k < cg; ++k)
        for (int spin = 0; spin < (1 << 16) && !mbar_try_wait(smem_u32(grp_full + k % kCSt), (k / kCSt) & 1); ++spin) {}
    }
  } else if (warp == 1 || warp == kSwapIssuerWarp1) {
    // ----------------------------------------------------------------------------- MMA issuers
    // issuer mi takes blocks 2 mi and 2 mi + 1 of every group and accumulates them in its own columns
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(128, NTOK, 0, 0);
      const int mi = warp == 1 ? 0 : 1;
      const uint32_t d_tmem = tmem_base + mi * 64;
      bool ok = true;
      int cg = 0, ul = 0;
      for (int u = blockIdx.x; ok && u < p.n_units; u += gridDim.x, ++ul) {
        int tile, sl, blk_begin, nblk;
        unit_range(u, tile, sl, blk_begin, nblk);
        // the accumulator is free once the previous unit's epilogue has read it
        if (!wait_or_abort(smem_u32(acc_empty), (ul & 1) ^ 1, ab, 0x0507)) { ok = false; break; }
        tc_fence_after();
        const int ngrp = (nblk + 3) / 4;
        bool first = true;                         // this issuer's first MMA of the unit overwrites its accumulator
        for (int grp = 0; grp < ngrp; ++grp, ++cg) {
          const int gs = cg % kSwapAGrp;
          const int nb = (nblk - grp * 4 < 4) ? nblk - grp * 4 : 4;
          const int gb = cg % (2 * kSwapAGrp);        // the group's barrier pair
          if (!swap_wait(smem_u32(a_full + gb), (cg / (2 * kSwapAGrp)) & 1, ab, 0x0503)) { ok = false; break; }
          tc_fence_after();
          const uint64_t xdesc = make_smem_desc(smem_u32(sX + gs * Cfg::kXGBytes), 16, 1024, kSwizzle128B);
          const uint32_t a0 = tmem_base + kACol0 + gs * 128;
#pragma unroll
          for (int jj = 0; jj < 2; ++jj) {
            const int j = 2 * mi + jj;
            if (j < nb) {
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                tc_mma_f16_ts(d_tmem, a0 + j * 32 + kk * 8, xdesc + ((j * Cfg::kXBytes + kk * 32) >> 4), idesc,
                              (jj == 0 && kk == 0) ? (first ? 0u : 1u) : 1u);
            }
          }
          if (2 * mi < nb) first = false;
          tc_commit(smem_u32(a_empty + gb));
        }
        if (ok) tc_commit(smem_u32(acc_full));
      }
      if (!ok) {
        // make sure none of this thread's MMAs is still running before tensor memory is freed
        tc_commit(smem_u32(drain + mi));
        for (int spin = 0; spin < (1 << 18) && !mbar_try_wait(smem_u32(drain + mi), 0); ++spin) {}
      }
    }
  } else if (warp == 2) {
    // ----------------------------------------------------------------------------- token tiles
    if (lane == 0) {
      tma_prefetch_desc(&tmap_x);
      int cg = 0;
      bool ok = true;
      for (int u = blockIdx.x; ok && u < p.n_units; u += gridDim.x) {
        int tile, sl, blk_begin, nblk;
        unit_range(u, tile, sl, blk_begin, nblk);
        const int ngrp = (nblk + 3) / 4;
        for (int grp = 0; grp < ngrp; ++grp, ++cg) {
          const int xg = cg % Cfg::kXG;
          const int nb = (nblk - grp * 4 < 4) ? nblk - grp * 4 : 4;
          const int gb = cg % (2 * kSwapAGrp);
          if (cg >= kSwapAGrp &&
              !wait_or_abort(smem_u32(a_empty + (cg - kSwapAGrp) % (2 * kSwapAGrp)), ((cg - kSwapAGrp) / (2 * kSwapAGrp)) & 1, ab, 0x0501)) { ok = false; break; }
          mbar_arrive_expect_tx(smem_u32(a_full + gb), nb * Cfg::kXBytes);
          for (int j = 0; j < nb; ++j)
            tma_load_2d(smem_u32(sX + xg * Cfg::kXGBytes + j * Cfg::kXBytes), &tmap_x, (blk_begin + grp * 4 + j) * 64, 0, smem_u32(a_full + gb));
        }
      }
    }
  } else {
    // ----------------------------------------------------------------------------- decode, then epilogue
    const int q = warp & 3;                       // tensor-memory lane quarter
    const int team = (warp - kSwapFirstDecodeWarp) >> 2;
    const int r = q * 32 + lane;                  // weight row inside the tile = tensor-memory lane
    const uint32_t lane_base = smem_u32(sTbl) + lane * 4;
    const uint32_t row_off = r * 128;
    const int key = r & 7;
    const uint32_t tA = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + kACol0;
    const bool direct = p.slices == 1;
    bool ok = true;
    int cg = 0, ul = 0;
    int s_idx = -1;                               // index of the scale2 / offset2 pair held in registers
    float s2 = 0.f, o2 = 0.f;

    for (int u = blockIdx.x; u < p.n_units; u += gridDim.x, ++ul) {
      int tile, sl, blk_begin, nblk;
      unit_range(u, tile, sl, blk_begin, nblk);
      const int64_t n = static_cast<int64_t>(tile) * 128 + r;
      const bool row_ok = n < p.N;
      const int qrow = static_cast<int>((row_ok ? n : p.N - 1) * bpr) + blk_begin;   // block index of the row's first block of the slice (< 2^31: checked on the host)
      const int ngrp_unit = (nblk + 3) / 4;
      // teams 0, 1 take the first and the second half of the groups whose running count is even, teams 2, 3 those of
      // the odd ones: a team meets every phase of the barriers it waits on (a unit's last group may lack its second
      // half; the epilogue that follows orders everything of the unit before the team's next wait)
      const int half = team & 1;
      // first group of the unit with this team's parity; its running count split as 6 k6 + gb (gb = barrier pair, gb % 3 =
      // slot of tensor memory), kept up to date by additions inside the loop
      int grp = ((team >> 1) ^ cg) & 1;
      int k6 = (cg + grp) / (2 * kSwapAGrp), gb = (cg + grp) - k6 * (2 * kSwapAGrp);
      for (; grp < ngrp_unit; grp += 2, gb += 2) {
        if (gb >= 2 * kSwapAGrp) { gb -= 2 * kSwapAGrp; ++k6; }
        const int gcount = cg + grp;                           // running count of the group
        const int nb = (nblk - grp * 4 < 4) ? nblk - grp * 4 : 4;
        if (half * 2 >= nb) continue;
        const int hu = grp * 2 + half;                         // half group of the unit
        const int c = gcount & (kCSt - 1), gs = gb >= kSwapAGrp ? gb - kSwapAGrp : gb;
        const int nb2 = (nb - half * 2 < 2) ? 1 : 2;           // blocks in this half group
        if (ok && !swap_wait(smem_u32(grp_full + c), (gcount / kCSt) & 1, ab, 0x0504)) ok = false;
        uint4 c0 = make_uint4(0, 0, 0, 0), c1 = c0, c2 = c0, c3 = c0;
        uint32_t qa = 0;
        if (ok) {
          const uint32_t stage = smem_u32(sStage + c * Cfg::kStageBytes);
          const uint32_t src = stage + row_off;
          c0 = lds128(src + (((4 * half) ^ key) << 4));
          c1 = lds128(src + (((4 * half + 1) ^ key) << 4));
          if (nb2 == 2) {
            c2 = lds128(src + (((4 * half + 2) ^ key) << 4));
            c3 = lds128(src + (((4 * half + 3) ^ key) << 4));
          }
          asm volatile("ld.shared.u16 %0, [%1];" : "=r"(qa) : "r"(stage + Cfg::kAbsOff + r * 4 + half * 2) : "memory");
        }
        // the stage goes back as soon as this warp's codes are in registers: eight warps read a stage, or four
        // (arriving twice) when the unit's last group has one half group only
        __syncwarp();
        if (ok && lane == 0) {
          mbar_arrive(smem_u32(grp_empty + c));
          if (nb <= 2) mbar_arrive(smem_u32(grp_empty + c));
        }
        // absmax = code2[qabs] * scale2 + offset2, rounded separately (the scale pair changes every 256 blocks)
        uint32_t am2[2] = {0u, 0u};
        if (ok) {
          const int b0 = qrow + hu * 2;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int si = (b0 + j) >> 8;
            if (si != s_idx) { s_idx = si; s2 = __ldg(p.scale2 + si); o2 = __ldg(p.offset2 + si); }
            const __half2 a2 = __float2half2_rn(block_absmax(sCode2[(qa >> (8 * j)) & 0xffu], s2, o2));
            am2[j] = *reinterpret_cast<const uint32_t*>(&a2);
          }
        }
        // the group's columns of tensor memory are free once the MMAs of three groups ago have completed: that group's
        // barrier pair is (gb + 3) mod 6, its phase k6 or k6 - 1
        const bool lone = nb <= 2;                 // the unit's last group has this half group only
        if (ok && gcount >= kSwapAGrp) {
          const int pb = gb >= kSwapAGrp ? gb - kSwapAGrp : gb + kSwapAGrp;
          const int pk = gb >= kSwapAGrp ? k6 : k6 - 1;
          if (!swap_wait(smem_u32(a_empty + pb), pk & 1, ab, 0x0505)) ok = false;
        }
        if (ok) {
          // sixteen columns (32 weights) at a time: the thread holds its four words of codes and one batch of results
          uint32_t v[16];
          const uint32_t dst = tA + gs * 128 + half * 64;
          swap_decode8(c0.x, lane_base, am2[0], v + 0);  swap_decode8(c0.y, lane_base, am2[0], v + 4);
          swap_decode8(c0.z, lane_base, am2[0], v + 8);  swap_decode8(c0.w, lane_base, am2[0], v + 12);
          __syncwarp();
          tmem_st16(dst, v);
          swap_decode8(c1.x, lane_base, am2[0], v + 0);  swap_decode8(c1.y, lane_base, am2[0], v + 4);
          swap_decode8(c1.z, lane_base, am2[0], v + 8);  swap_decode8(c1.w, lane_base, am2[0], v + 12);
          tmem_st16(dst + 16, v);
          if (nb2 == 2) {
            swap_decode8(c2.x, lane_base, am2[1], v + 0);  swap_decode8(c2.y, lane_base, am2[1], v + 4);
            swap_decode8(c2.z, lane_base, am2[1], v + 8);  swap_decode8(c2.w, lane_base, am2[1], v + 12);
            tmem_st16(dst + 32, v);
            swap_decode8(c3.x, lane_base, am2[1], v + 0);  swap_decode8(c3.y, lane_base, am2[1], v + 4);
            swap_decode8(c3.z, lane_base, am2[1], v + 8);  swap_decode8(c3.w, lane_base, am2[1], v + 12);
            tmem_st16(dst + 48, v);
          }
          tmem_st_wait();
        }
        tc_fence_before();
        __syncwarp();
        if (ok && lane == 0) {
          mbar_arrive(smem_u32(a_full + gb));
          if (lone) mbar_arrive(smem_u32(a_full + gb));
        }
      }
      cg += ngrp_unit;

      // --- epilogue of the unit: lane = weight row, columns = tokens; team t takes token columns 16 t .. 16 t + 15
      if (ok) ok = wait_or_abort(smem_u32(acc_full), ul & 1, ab, 0x0506);
      pdl_wait();                                 // T and the cleared counters come from the kernel before this one
      float bias = 0.f, bs[16];
      auto load_row_terms = [&]() {
        if (p.bias && row_ok) bias = __half2float(p.bias[n]);
        if (p.t32 && row_ok) {
          float tmp[8];
          const uint4* bp = reinterpret_cast<const uint4*>(p.lora_b + n * 16);
          unpack8(__ldg(bp), tmp);
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) bs[jj] = tmp[jj] * p.lora_scale;
          unpack8(__ldg(bp + 1), tmp);
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) bs[8 + jj] = tmp[jj] * p.lora_scale;
        }
      };
      auto finish = [&](int tok, float v) {
        // bias, LoRA term, one rounding; 32 lanes store 32 consecutive output columns of one token row
        if (p.t32) {
          const float4* tr = reinterpret_cast<const float4*>(p.t32 + static_cast<int64_t>(tok) * 16);
          float l = 0.f;
#pragma unroll
          for (int j4 = 0; j4 < 4; ++j4) {
            const float4 tv = __ldcg(tr + j4);
            l = fmaf(tv.x, bs[4 * j4], l); l = fmaf(tv.y, bs[4 * j4 + 1], l);
            l = fmaf(tv.z, bs[4 * j4 + 2], l); l = fmaf(tv.w, bs[4 * j4 + 3], l);
          }
          v += l;
        }
        p.y[static_cast<int64_t>(tok) * p.ldy + n] = __float2half_rn(v + bias);
      };
      const bool has_cols = team * 16 < NTOK;
      if (ok) {
        tc_fence_after();
        uint32_t v[16];
        if (has_cols) {
          if (direct) load_row_terms();
          __syncwarp();
          // the accumulators of the two issuing threads (the second one unused by a unit of one or two blocks)
          const bool used0 = true, used1 = nblk > 2;
          uint32_t w[16];
          if (used0) tmem_ld16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + team * 16, v);
          if (used1) tmem_ld16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + 64 + team * 16, w);
          tmem_ld_wait();
#pragma unroll
          for (int jt = 0; jt < 16; ++jt)
            v[jt] = __float_as_uint((used0 ? __uint_as_float(v[jt]) : 0.f) + (used1 ? __uint_as_float(w[jt]) : 0.f));
        }
        // the accumulator is in registers: the next unit's MMAs may overwrite it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(acc_empty));
        if (has_cols) {
          if (direct) {
            if (row_ok) {
#pragma unroll
              for (int jt = 0; jt < 16; ++jt) {
                const int tok = team * 16 + jt;
                if (tok < p.M) finish(tok, __uint_as_float(v[jt]));
              }
            }
          } else {
            float* mine = p.slab + ((static_cast<int64_t>(tile) * p.slices + sl) * NTOK) * 128 + r;
#pragma unroll
            for (int jt = 0; jt < 16; ++jt) {
              const int tok = team * 16 + jt;
              if (tok < p.M) mine[static_cast<int64_t>(tok) * 128] = __uint_as_float(v[jt]);
            }
          }
        }
      } else {
        // a failed wait: still release the MMA issuer, which may be waiting for the accumulator to be read
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(acc_empty));
      }
      if (!direct) {
        // the unit of a tile that arrives last adds the partial sums up in slice order
        __threadfence();
        named_barrier(1, kSwapDecodeWarps * 32);
        if (threadIdx.x == kSwapFirstDecodeWarp * 32) {
          const int prev = atomicAdd(p.counters + tile, 1);
          *last_flag = (prev == p.slices - 1) ? 1 : 0;
          *stop_flag = *abort_flag;               // sampled once per unit, so that all decode warps leave together
          __threadfence();
        }
        named_barrier(1, kSwapDecodeWarps * 32);
        if (*last_flag && !*stop_flag) {
          load_row_terms();
          const float* all = p.slab + (static_cast<int64_t>(tile) * p.slices * NTOK) * 128 + r;
          const int tok_end = static_cast<int>(p.M < NTOK ? p.M : NTOK);
          for (int tok = team; tok < tok_end; tok += kSwapTeams) {
            float v = 0.f;
            for (int s2 = 0; s2 < p.slices; ++s2) v += __ldcg(all + (static_cast<int64_t>(s2) * NTOK + tok) * 128);
            if (row_ok) finish(tok, v);
          }
        }
        named_barrier(1, kSwapDecodeWarps * 32);  // last_flag is rewritten by the next unit
        if (*stop_flag) break;
      } else if (*abort_flag) {
        break;                                    // no barriers between the decode warps in this mode: each may leave on its own
      }
    }
  }

  // ------------------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncwarp();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*SwapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int swap_encode(CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t inner, uint64_t outer,
                       uint64_t stride_bytes, uint32_t box_inner, uint32_t box_outer, const char* what) {
  static SwapEncodeFn cached = nullptr;
  if (!cached) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    NF4LL_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || !fn) {
      set_detail("cuTensorMapEncodeTiled not available from the driver");
      return NF4LL_ERR_CUDA;
    }
    cached = reinterpret_cast<SwapEncodeFn>(fn);
  }
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {stride_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = cached(map, type, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_detail("cuTensorMapEncodeTiled (%s) failed with CUresult %d", what, static_cast<int>(r));
    return NF4LL_ERR_CUDA;
  }
  return NF4LL_OK;
}

static int swap_ntok(int64_t M) { return M <= 16 ? 16 : (M <= 32 ? 32 : 64); }

// Slices of the contraction for W[N,K] at `ntok` token columns. The persistent grid has one CTA per SM: the
// slice count is the one that minimises rounds x (work of a unit + a fixed cost per unit)
// + the traffic of the partial-sum slab, in whole groups of four quantisation blocks.
void swap_plan(int64_t N, int64_t K, int ntok, int sms, int force_slices, int* slices, int* groups_per_slice) {
  const int groups = static_cast<int>((K / 64 + 3) / 4);
  const int64_t tiles = (N + 127) / 128;
  const int64_t grid = sms;
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= groups && s <= 32; ++s) {
    const int per = (groups + s - 1) / s;
    if ((groups + per - 1) / per != s) continue;            // not a distinct split
    const int64_t units = tiles * s;
    const int64_t rounds = (units + grid - 1) / grid;
    // in units of "one group of four blocks of one tile": a unit costs its groups plus about four groups of fixed
    // overhead (pipeline fill and drain, epilogue: measured); a slab element costs 8 bytes of traffic against 16.9 KB
    // per tile-group, weighted twice (the exchange is latency-bound, not bandwidth-bound)
    const double slab = s > 1 ? 2.0 * static_cast<double>(units) * ntok * 128 * 8 / (128.0 * 256 * 0.516) / static_cast<double>(grid) : 0.0;
    const double cost = static_cast<double>(rounds) * (per + 4.0) + slab;
    if (cost < best_cost) { best_cost = cost; best = s; }
  }
  if (force_slices > 0) best = force_slices > groups ? groups : force_slices;
  const int per = (groups + best - 1) / best;
  *slices = (groups + per - 1) / per;
  *groups_per_slice = per;
}

int64_t swap_workspace_bytes(int64_t N, int64_t K, int64_t M, int sms, int force_slices) {
  int s = 1, per = 0;
  swap_plan(N, K, swap_ntok(M), sms, force_slices, &s, &per);
  const int64_t tiles = (N + 127) / 128;
  const int64_t counters = (tiles * 4 + 255) / 256 * 256;
  const int64_t slab = s > 1 ? tiles * s * swap_ntok(M) * 128 * 4 : 0;
  return counters + (slab + 255) / 256 * 256;
}

template <int NTOK>
static int swap_launch_cfg(const CUtensorMap& mx, const CUtensorMap& mn, const SwapParams& p, unsigned grid, cudaStream_t stream) {
  using Cfg = SwapCfg<NTOK>;
  auto kernel = nf4_swap_kernel<NTOK>;
  NF4LL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
  PdlLaunch lc(dim3(grid), dim3(kSwapThreads), Cfg::kSmemBytes, stream);
  NF4LL_CUDA(cudaLaunchKernelEx(&lc.cfg, kernel, mx, mn, p));
  return NF4LL_OK;
}

// `scratch`: the tile counters (cleared here unless `counters_zeroed`: the rank-16 projection kernel launched
// just before has then done it) followed, 256-byte aligned, by the slab.
int swap_forward_launch(const nf4ll_mat* W, const void* x, int64_t ldx, const void* bias, const float* t32,
                        const void* lora_b, float lora_scale, int64_t M, void* y, int64_t ldy, void* scratch,
                        bool counters_zeroed, int force_slices, int32_t* status, cudaStream_t stream) {
  int dev = 0, sms = 148;
  NF4LL_CUDA(cudaGetDevice(&dev));
  NF4LL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  SwapParams p{};
  p.qabs = W->qabs; p.scale2 = W->scale2; p.offset2 = W->offset2; p.code2 = W->code2;
  p.N = W->N; p.K = W->K; p.M = M;
  p.y = static_cast<__half*>(y); p.ldy = ldy;
  p.bias = static_cast<const __half*>(bias);
  p.t32 = t32; p.lora_b = static_cast<const __half*>(lora_b); p.lora_scale = lora_scale;
  p.status = status;
  const int ntok = swap_ntok(M);
  swap_plan(W->N, W->K, ntok, sms, force_slices, &p.slices, &p.groups_per_slice);
  const int64_t tiles = (W->N + 127) / 128;
  p.n_units = static_cast<int>(tiles * p.slices);
  const int64_t counter_bytes = (tiles * 4 + 255) / 256 * 256;
  p.counters = static_cast<int*>(scratch);
  p.slab = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + counter_bytes);
  if (p.slices > 1 && !counters_zeroed) NF4LL_CUDA(cudaMemsetAsync(p.counters, 0, tiles * 4, stream));
  CUtensorMap mx, mn;
  if (int rc = swap_encode(&mx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x, static_cast<uint64_t>(W->K), static_cast<uint64_t>(M),
                           static_cast<uint64_t>(ldx) * 2, 64, static_cast<uint32_t>(ntok), "token tile")) return rc;
  if (int rc = swap_encode(&mn, CU_TENSOR_MAP_DATA_TYPE_UINT8, W->nib, static_cast<uint64_t>(W->K / 2), static_cast<uint64_t>(W->N),
                           static_cast<uint64_t>(W->K / 2), 128, 128, "codes")) return rc;
  int64_t ctas = sms;
  if (ctas > p.n_units) ctas = p.n_units;
  const unsigned grid = static_cast<unsigned>(ctas);
  switch (ntok) {
    case 16: return swap_launch_cfg<16>(mx, mn, p, grid, stream);
    case 32: return swap_launch_cfg<32>(mx, mn, p, grid, stream);
    default: return swap_launch_cfg<64>(mx, mn, p, grid, stream);
  }
}

}  // namespace nf4ll
