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
//   warp 0        TMA producer: 128x64 fp16 activation boxes (128-byte swizzle) into a ring
//   warp 1        allocates tensor memory; one lane issues every tcgen05.mma and commit
//   warps 2-3     stage the two rank-16 LoRA operands in shared memory (canonical no-swizzle layout)
//   warps 4..     BN threads: each owns one 64-weight quantisation block per ring stage: 2 x 128-bit
//                 loads of codes, block table in registers, 8 x 128-bit swizzled shared stores;
//                 afterwards the same warps drain tensor memory (epilogue)
// The weight tile in shared memory is the same in both directions: rows of 64 consecutive weights of
// one W row (= one quantisation block, 128 bytes), 8 rows per 1024-byte swizzle atom. Forward reads
// it as a K-major B operand (contraction along the row), backward as an MN-major one (contraction
// across rows), so the same NF4 bytes serve W and W^T.
#include <cuda.h>

#include "nf4ll_common.cuh"

namespace nf4ll {

enum : int { kFwd = 0, kBwd = 1 };

struct GemmParams {
  const uint8_t* nib;
  const uint8_t* qabs;
  const float* scale2;
  const float* offset2;
  const float* code2;
  int64_t N, K;            // W[N,K]
  int64_t M;               // rows of the activation / output
  int64_t NO;              // output columns: N (forward) or K (backward)
  int64_t KC;              // contraction length: K (forward) or N (backward)
  __half* out;
  int64_t ldo;
  const __half* bias;      // forward only, may be null
  int accumulate;          // backward: out += result
  int has_lora;
  const __half* lora_left;   // [M,16] fp16: s.T (forward) or s.U (backward)
  const __half* lora_right;  // forward: B[N,16]; backward: A[16,K]
  const uint8_t* mask;       // backward only: keep-mask of the LoRA input [M, ld_mask], may be null
  int64_t ld_mask;
  float keep_scale;
  int splits;              // split of the contraction across blockIdx.z
  float* partial;          // [splits][M_pad][NO] fp32 when splits > 1
  int* counters;           // one per output tile when splits > 1 (zero on entry, zero on exit)
  int64_t m_pad;
  int32_t* status;
};

template <int BM_TILES, int BN>
struct TileCfg {
  static constexpr int kStages = (BM_TILES == 2 && BN == 256) ? 3 : 4;
  static constexpr int kDequantWarps = BN / 32;
  static constexpr int kThreads = 32 * (4 + kDequantWarps);
  static constexpr int kABytes = BM_TILES * 128 * 128;   // per stage: 128 rows x 64 fp16 per M tile
  static constexpr int kBBytes = BN * 128;               // per stage: BN quantisation blocks
  static constexpr int kLoraLeftBytes = BM_TILES * 128 * 32;
  static constexpr int kLoraRightBytes = BN * 32;
  static constexpr int kTmemCols = BM_TILES * BN;        // 128, 256 or 512: a power of two >= 32
  static constexpr int kSmemBytes = 1024 /* alignment slack */ + kStages * (kABytes + kBBytes) + kLoraLeftBytes +
                                    kLoraRightBytes + 1024 /* code2 */ + 256 /* barriers */;
};

struct Abort {
  volatile int* flag;
  int32_t* status;
  __device__ __forceinline__ void raise(int code) const {
    *flag = 1;
    if (status) atomicCAS(status, 0, code);
  }
};

__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, const Abort& ab, int code) {
  if (mbar_wait(bar, parity, ab.flag)) return true;
  ab.raise(code);
  return false;
}

// Decode one quantisation block (32 bytes of codes) into one 128-byte row of a 128B-swizzled tile.
__device__ __forceinline__ void dequant_block_to_smem(uint8_t* row_base, int key, uint4 c0, uint4 c1, float absmax) {
  const BlockTable t = make_block_table(absmax);
  const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    *reinterpret_cast<uint4*>(row_base + ((j ^ key) << 4)) = decode_word(t, w[j]);
  }
}

template <int MODE, int BM_TILES, int BN>
__global__ void __launch_bounds__(TileCfg<BM_TILES, BN>::kThreads, 1)
nf4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_act, const GemmParams p) {
  using Cfg = TileCfg<BM_TILES, BN>;
  constexpr int S = Cfg::kStages;
  constexpr int NDW = Cfg::kDequantWarps;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;                                   // [S][BM_TILES][128 rows][128 B]
  uint8_t* sB = sA + S * Cfg::kABytes;                  // [S][BN rows][128 B]
  uint8_t* sLL = sB + S * Cfg::kBBytes;                 // LoRA left operand  [BM_TILES][128 x 16]
  uint8_t* sLR = sLL + Cfg::kLoraLeftBytes;             // LoRA right operand [BN x 16] or [16 x BN]
  float* sCode2 = reinterpret_cast<float*>(sLR + Cfg::kLoraRightBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sCode2) + 1024);
  // barrier slots
  uint64_t* full_a = bars;            // [S] TMA bytes landed
  uint64_t* full_b = bars + S;        // [S] dequantised tile written (one arrive per dequant warp)
  uint64_t* empty = bars + 2 * S;     // [S] MMAs that read the stage have completed
  uint64_t* lora_full = bars + 3 * S;
  uint64_t* acc_full = lora_full + 1;
  uint64_t* pre_full = lora_full + 2;
  uint64_t* pre_done = lora_full + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(lora_full + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = abort_flag + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tile_o = blockIdx.x, tile_m = blockIdx.y, split = blockIdx.z;
  const int64_t m0 = static_cast<int64_t>(tile_m) * (BM_TILES * 128);
  const int64_t o0 = static_cast<int64_t>(tile_o) * BN;

  // contraction range of this split, in 64-wide steps
  const int nkb_total = static_cast<int>(p.KC / 64);
  const int kb_begin = static_cast<int>(static_cast<int64_t>(nkb_total) * split / p.splits);
  const int kb_end = static_cast<int>(static_cast<int64_t>(nkb_total) * (split + 1) / p.splits);
  const int nkb = kb_end - kb_begin;
  const bool lora_here = p.has_lora && split == 0;
  const bool premask = lora_here && MODE == kBwd && p.mask != nullptr;

  const Abort ab{abort_flag, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(full_a + s), 1);
      mbar_init(smem_u32(full_b + s), NDW);
      mbar_init(smem_u32(empty + s), 1);
    }
    mbar_init(smem_u32(lora_full), 2);
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
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ----------------------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_act);
      int issued = 0;
      for (int i = 0; i < nkb; ++i, ++issued) {
        const int s = i % S;
        if (!wait_or_abort(smem_u32(empty + s), ((i / S) & 1) ^ 1, ab, 0x0101)) break;
        mbar_arrive_expect_tx(smem_u32(full_a + s), Cfg::kABytes);
#pragma unroll
        for (int mt = 0; mt < BM_TILES; ++mt) {
          tma_load_2d(smem_u32(sA + s * Cfg::kABytes + mt * 16384), &tmap_act, (kb_begin + i) * 64,
                      static_cast<int>(m0 + mt * 128), smem_u32(full_a + s));
        }
      }
      if (*abort_flag) {
        // give copies still in flight a bounded chance to land before the CTA goes away
        for (int i = (issued > S ? issued - S : 0); i < issued; ++i) {
          const uint32_t bar = smem_u32(full_a + (i % S)), ph = (i / S) & 1;
          for (int spin = 0; spin < (1 << 16) && !mbar_try_wait(bar, ph); ++spin) {}
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
          const uint64_t rdesc = make_smem_desc(smem_u32(sLR), 128, 256, kSwizzleNone);
#pragma unroll
          for (int mt = 0; mt < BM_TILES; ++mt) {
            const uint64_t ldesc = make_smem_desc(smem_u32(sLL + mt * 4096), 128, 256, kSwizzleNone);
            tc_mma_f16(tmem_base + mt * BN, ldesc, rdesc, idesc_main, 0u);
          }
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
        if (!wait_or_abort(smem_u32(full_a + s), ph, ab, 0x0203) ||
            !wait_or_abort(smem_u32(full_b + s), ph, ab, 0x0204)) {
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
    // ----------------------------------------------------------------------------- LoRA operand staging
    if (lora_here) {
      const int t = threadIdx.x - 64;   // 0..63
      // left: rows m0.. of lora_left[M,16]; chunk (row, h) -> (row/8)*256 + h*128 + (row%8)*16
      for (int c = t; c < BM_TILES * 128 * 2; c += 64) {
        const int row = c >> 1, h = c & 1;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (m0 + row < p.M) v = __ldg(reinterpret_cast<const uint4*>(p.lora_left + (m0 + row) * 16 + h * 8));
        const int mt = row >> 7, r = row & 127;
        *reinterpret_cast<uint4*>(sLL + mt * 4096 + (r >> 3) * 256 + h * 128 + (r & 7) * 16) = v;
      }
      if (MODE == kFwd) {
        // right: rows o0.. of B[N,16], same chunk layout
        for (int c = t; c < BN * 2; c += 64) {
          const int row = c >> 1, h = c & 1;
          uint4 v = make_uint4(0, 0, 0, 0);
          if (o0 + row < p.NO) v = __ldg(reinterpret_cast<const uint4*>(p.lora_right + (o0 + row) * 16 + h * 8));
          *reinterpret_cast<uint4*>(sLR + (row >> 3) * 256 + h * 128 + (row & 7) * 16) = v;
        }
      } else {
        // right: columns o0.. of A[16,K]; chunk (8 columns c8, rank row j) -> c8*256 + (j/8)*128 + (j%8)*16
        for (int c = t; c < 16 * (BN / 8); c += 64) {
          const int j = c / (BN / 8), c8 = c % (BN / 8);
          uint4 v = make_uint4(0, 0, 0, 0);
          if (o0 + c8 * 8 < p.NO) v = __ldg(reinterpret_cast<const uint4*>(p.lora_right + j * p.K + o0 + c8 * 8));
          *reinterpret_cast<uint4*>(sLR + c8 * 256 + (j >> 3) * 128 + (j & 7) * 16) = v;
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(lora_full));
    }
  } else {
    // ----------------------------------------------------------------------------- dequant, then epilogue
    const int d = threadIdx.x - 128;      // 0..BN-1: one quantisation block per stage
    const int ew = warp - 4;              // 0..NDW-1
    const int q = warp & 3;               // tensor-memory lane quarter this warp may read
    bool ok = true;

    if (premask) {
      // The LoRA product is already in the accumulator: scale it by keep_scale * mask in place, so
      // that the base GEMM then accumulates on top (dropout acts on the LoRA input only).
      ok = wait_or_abort(smem_u32(pre_full), 0, ab, 0x0301);
      if (ok) {
        tc_fence_after();
        constexpr int kChunks = BM_TILES * (BN / 32);
        for (int u = ew >> 2; u < kChunks; u += NDW / 4) {
          const int mt = u / (BN / 32), c = u % (BN / 32);
          const int64_t row = m0 + mt * 128 + q * 32 + lane;
          const int64_t col0 = o0 + c * 32;
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + mt * BN + c * 32;
          uint32_t v[32];
          __syncwarp();
          tmem_ld32(taddr, v);
          tmem_ld_wait();
          uint32_t mk[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          if (row < p.M && col0 < p.NO) {
            const uint4* mp = reinterpret_cast<const uint4*>(p.mask + row * p.ld_mask + col0);
            const uint4 a = __ldg(mp), b = __ldg(mp + 1);
            mk[0] = a.x; mk[1] = a.y; mk[2] = a.z; mk[3] = a.w;
            mk[4] = b.x; mk[5] = b.y; mk[6] = b.z; mk[7] = b.w;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const bool keep = ((mk[j >> 2] >> ((j & 3) * 8)) & 0xffu) != 0;
            v[j] = keep ? __float_as_uint(__uint_as_float(v[j]) * p.keep_scale) : 0u;
          }
          tmem_st32(taddr, v);
          tmem_st_wait();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(pre_done));
      }
    }

    // --- dequantise one block per stage
    int64_t byte_off, qb, byte_step, qb_step;
    uint8_t* row_off_base;       // offset of this thread's 128-byte row inside a B stage
    int key;
    if (MODE == kFwd) {
      int64_t n = o0 + d;
      if (n >= p.N) n = p.N - 1;                       // tail rows decode valid memory; never stored
      const int64_t e = n * p.K + static_cast<int64_t>(kb_begin) * 64;
      byte_off = e >> 1; qb = e >> 6; byte_step = 32; qb_step = 1;
      row_off_base = sB + d * 128;
      key = d & 7;
    } else {
      constexpr int SUB = BN / 64;
      const int j = d % SUB, r = d / SUB;              // sub-tile (64 output columns) and row in the stage
      int64_t kcol = o0 + j * 64;
      if (kcol >= p.K) kcol = 0;
      const int64_t e = (static_cast<int64_t>(kb_begin) * 64 + r) * p.K + kcol;
      byte_off = e >> 1; qb = e >> 6; byte_step = 32 * p.K; qb_step = p.K;
      row_off_base = sB + j * 8192 + r * 128;
      key = r & 7;
    }
    uint4 c0 = make_uint4(0, 0, 0, 0), c1 = c0;
    uint32_t qcode = 0;
    float s2 = 0.f, o2 = 0.f;
    if (nkb > 0) {
      const uint4* src = reinterpret_cast<const uint4*>(p.nib + byte_off);
      c0 = __ldg(src); c1 = __ldg(src + 1);
      qcode = __ldg(p.qabs + qb); s2 = __ldg(p.scale2 + (qb >> 8)); o2 = __ldg(p.offset2 + (qb >> 8));
    }
    for (int i = 0; ok && i < nkb; ++i) {
      const int s = i % S;
      // prefetch the next block's codes and scales into registers (latency hidden by this block's decode)
      uint4 n0 = c0, n1 = c1;
      uint32_t nq = qcode;
      float ns2 = s2, no2 = o2;
      if (i + 1 < nkb) {
        const int64_t bo = byte_off + byte_step, nqb = qb + qb_step;
        const uint4* src = reinterpret_cast<const uint4*>(p.nib + bo);
        n0 = __ldg(src); n1 = __ldg(src + 1);
        nq = __ldg(p.qabs + nqb); ns2 = __ldg(p.scale2 + (nqb >> 8)); no2 = __ldg(p.offset2 + (nqb >> 8));
      }
      if (i + 4 < nkb) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p.nib + byte_off + 4 * byte_step));
      }
      if (!wait_or_abort(smem_u32(empty + s), ((i / S) & 1) ^ 1, ab, 0x0302)) { ok = false; break; }
      const float absmax = block_absmax(sCode2[qcode], s2, o2);
      dequant_block_to_smem(row_off_base + s * Cfg::kBBytes, key, c0, c1, absmax);
      fence_proxy_async_smem();      // generic-proxy stores -> visible to the tensor core's async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(full_b + s));
      c0 = n0; c1 = n1; qcode = nq; s2 = ns2; o2 = no2;
      byte_off += byte_step; qb += qb_step;
    }

    // --- epilogue: tensor memory -> registers -> global
    if (ok) ok = wait_or_abort(smem_u32(acc_full), 0, ab, 0x0303);
    const bool direct = (p.splits == 1);
    if (ok) {
      tc_fence_after();
      constexpr int kChunks = BM_TILES * (BN / 32);
      float* slab = direct ? nullptr : p.partial + static_cast<int64_t>(split) * p.m_pad * p.NO;
      for (int u = ew >> 2; u < kChunks; u += NDW / 4) {
        const int mt = u / (BN / 32), c = u % (BN / 32);
        const int64_t row = m0 + mt * 128 + q * 32 + lane;
        const int64_t col0 = o0 + c * 32;
        uint32_t v[32];
        __syncwarp();
        tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + mt * BN + c * 32, v);
        tmem_ld_wait();
        if (direct) {
          if (row < p.M && col0 < p.NO) {
            __half* dst = p.out + row * p.ldo + col0;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[g * 8 + j]);
              if (MODE == kFwd && p.bias) {
                const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + g * 8));
                const __half2* bh = reinterpret_cast<const __half2*>(&b);
#pragma unroll
                for (int j = 0; j < 4; ++j) { const float2 bf = __half22float2(bh[j]); f[2 * j] += bf.x; f[2 * j + 1] += bf.y; }
              }
              if (MODE == kBwd && p.accumulate) {
                const uint4 o = *reinterpret_cast<const uint4*>(dst + g * 8);
                const __half2* oh = reinterpret_cast<const __half2*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) { const float2 of = __half22float2(oh[j]); f[2 * j] += of.x; f[2 * j + 1] += of.y; }
              }
              uint4 o;
              o.x = pack_half2_rn(f[0], f[1]); o.y = pack_half2_rn(f[2], f[3]);
              o.z = pack_half2_rn(f[4], f[5]); o.w = pack_half2_rn(f[6], f[7]);
              *reinterpret_cast<uint4*>(dst + g * 8) = o;
            }
          }
        } else if (col0 < p.NO) {
          // rows beyond M still fit: the slab has m_pad rows
          float4* dst = reinterpret_cast<float4*>(slab + row * p.NO + col0);
#pragma unroll
          for (int g = 0; g < 8; ++g)
            dst[g] = make_float4(__uint_as_float(v[4 * g]), __uint_as_float(v[4 * g + 1]), __uint_as_float(v[4 * g + 2]),
                                 __uint_as_float(v[4 * g + 3]));
        }
      }
    }
    if (!direct) {
      // split-K fix-up: the last CTA of this output tile to finish sums all slabs in split order
      // (deterministic) and writes the fp16 result. Every dequant thread takes both barriers, also
      // after a failed wait, so that nobody is left behind at a barrier.
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"r"(NDW * 32) : "memory");
      int* counter = p.counters + (static_cast<int64_t>(tile_m) * gridDim.x + tile_o);
      if (d == 0) {
        const int prev = atomicAdd(counter, 1);
        if (prev == p.splits - 1) { *last_flag = 1; *counter = 0; }
        __threadfence();
      }
      asm volatile("bar.sync 1, %0;" ::"r"(NDW * 32) : "memory");
      if (*last_flag && !*abort_flag) {
        // thread d: 8 consecutive columns (c8 = d % (BN/8)), rows strided by NDW*32/(BN/8)
        constexpr int CPR = BN / 8;                    // 16-byte output chunks per tile row
        constexpr int RSTEP = (NDW * 32) / CPR;
        const int c8 = d % CPR;
        const int64_t col = o0 + c8 * 8;
        if (col < p.NO) {
          float bf[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          if (MODE == kFwd && p.bias) {
            const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.bias + col));
            const __half2* bh = reinterpret_cast<const __half2*>(&b);
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 t2 = __half22float2(bh[j]); bf[2 * j] = t2.x; bf[2 * j + 1] = t2.y; }
          }
          for (int r = d / CPR; r < BM_TILES * 128; r += RSTEP) {
            const int64_t row = m0 + r;
            if (row >= p.M) break;
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = bf[j];
            for (int sp = 0; sp < p.splits; ++sp) {
              const float4* src = reinterpret_cast<const float4*>(p.partial + (static_cast<int64_t>(sp) * p.m_pad + row) * p.NO + col);
              const float4 a = __ldcg(src), b = __ldcg(src + 1);
              f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
              f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
            }
            __half* dst = p.out + row * p.ldo + col;
            if (MODE == kBwd && p.accumulate) {
              const uint4 o = *reinterpret_cast<const uint4*>(dst);
              const __half2* oh = reinterpret_cast<const __half2*>(&o);
#pragma unroll
              for (int j = 0; j < 4; ++j) { const float2 of = __half22float2(oh[j]); f[2 * j] += of.x; f[2 * j + 1] += of.y; }
            }
            uint4 o;
            o.x = pack_half2_rn(f[0], f[1]); o.y = pack_half2_rn(f[2], f[3]);
            o.z = pack_half2_rn(f[4], f[5]); o.w = pack_half2_rn(f[6], f[7]);
            *reinterpret_cast<uint4*>(dst) = o;
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------------------- teardown
  tc_fence_before();
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

// 2-D map over a row-major fp16 matrix [rows, cols] with leading dimension ld: boxes of 64 columns
// (128 bytes, the swizzle span) x 128 rows, zero fill outside.
static int make_act_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld) {
  EncodeTiledFn enc;
  if (int rc = get_encode_fn(&enc)) return rc;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {64, 128};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_detail("cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld cols=%lld ld=%lld)", static_cast<int>(r),
               static_cast<long long>(rows), static_cast<long long>(cols), static_cast<long long>(ld));
    return NF4LL_ERR_CUDA;
  }
  return NF4LL_OK;
}

struct Plan {
  int bm_tiles, bn, splits;
  int64_t tiles_m, tiles_o, m_pad;
  int64_t left_bytes, bt_bytes, counter_bytes, partial_bytes;
  int64_t total() const { return left_bytes + bt_bytes + counter_bytes + partial_bytes; }
};

static thread_local int g_force_bm = 0, g_force_bn = 0, g_force_splits = 0;
static thread_local cudaEvent_t g_ev_start = nullptr, g_ev_stop = nullptr;

static int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

static Plan make_plan(int64_t M, int64_t NO, int64_t KC, int r, int sms) {
  Plan pl;
  pl.bn = (NO % 256 == 0 || NO > 256) ? 256 : 128;
  if (NO <= 128) pl.bn = 128;
  pl.bm_tiles = (M > 128) ? 2 : 1;
  if (g_force_bn) pl.bn = g_force_bn;
  if (g_force_bm) pl.bm_tiles = g_force_bm;
  const int64_t bm = pl.bm_tiles * 128;
  pl.tiles_m = (M + bm - 1) / bm;
  pl.tiles_o = (NO + pl.bn - 1) / pl.bn;
  pl.m_pad = pl.tiles_m * bm;
  const int64_t tiles = pl.tiles_m * pl.tiles_o;
  const int64_t nkb = KC / 64;
  int splits = 1;
  if (tiles * 2 <= sms) {                       // less than half a wave: split the contraction
    splits = static_cast<int>(sms / tiles);
    const int64_t max_by_k = nkb / 4 > 0 ? nkb / 4 : 1;     // at least 4 stages per split
    if (splits > max_by_k) splits = static_cast<int>(max_by_k);
    if (splits > 16) splits = 16;
    if (splits < 1) splits = 1;
  }
  if (g_force_splits) splits = g_force_splits;
  if (splits > nkb) splits = static_cast<int>(nkb > 0 ? nkb : 1);
  pl.splits = splits;
  pl.left_bytes = r > 0 ? align256(M * r * 2) : 0;
  pl.bt_bytes = r > 0 ? align256(KC * r * 2) : 0;      // room for lora_B transposed (backward only uses it)
  pl.counter_bytes = splits > 1 ? align256(tiles * 4) : 0;
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

template <int MODE, int BM_TILES, int BN>
static int launch_cfg(const CUtensorMap& map, const GemmParams& p, const Plan& pl, cudaStream_t stream) {
  using Cfg = TileCfg<BM_TILES, BN>;
  auto kernel = nf4_gemm_kernel<MODE, BM_TILES, BN>;
  NF4LL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
  dim3 grid(static_cast<unsigned>(pl.tiles_o), static_cast<unsigned>(pl.tiles_m), static_cast<unsigned>(pl.splits));
  kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(map, p);
  NF4LL_CUDA(cudaGetLastError());
  return NF4LL_OK;
}

template <int MODE>
static int launch(const CUtensorMap& map, const GemmParams& p, const Plan& pl, cudaStream_t stream) {
  if (pl.bm_tiles == 2 && pl.bn == 256) return launch_cfg<MODE, 2, 256>(map, p, pl, stream);
  if (pl.bm_tiles == 1 && pl.bn == 256) return launch_cfg<MODE, 1, 256>(map, p, pl, stream);
  if (pl.bm_tiles == 2 && pl.bn == 128) return launch_cfg<MODE, 2, 128>(map, p, pl, stream);
  return launch_cfg<MODE, 1, 128>(map, p, pl, stream);
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

static int check_lora(const nf4ll_lora* l, const char* who, bool need_mask_ld, int64_t K) {
  if (!l) return NF4LL_OK;
  if (l->r != 16) { set_detail("%s: LoRA rank %d", who, l->r); return NF4LL_ERR_RANK; }
  if (!l->A || !l->B) { set_detail("%s: LoRA A/B null", who); return NF4LL_ERR_NULL; }
  if ((reinterpret_cast<uintptr_t>(l->A) & 15) || (reinterpret_cast<uintptr_t>(l->B) & 15) ||
      (reinterpret_cast<uintptr_t>(l->Bt) & 15)) {
    set_detail("%s: LoRA A/B must be 16-byte aligned", who);
    return NF4LL_ERR_ALIGN;
  }
  if (l->mask && (need_mask_ld || true) && ((reinterpret_cast<uintptr_t>(l->mask) & 15) || l->ld_mask % 16 || l->ld_mask < K)) {
    set_detail("%s: mask must be 16-byte aligned with ld_mask a multiple of 16 and >= K", who);
    return NF4LL_ERR_ALIGN;
  }
  return NF4LL_OK;
}

int lora_down_launch(const void* act, int64_t ldact, const uint8_t* mask, int64_t ld_mask, float keep_scale,
                     const void* R, float t32_scale, float t16_scale, int64_t M, int64_t C, void* t32, void* t16,
                     cudaStream_t stream);
int transpose_n16_launch(const void* B, void* Bt, int64_t N, cudaStream_t stream);

static int run_gemm(int mode, const nf4ll_mat* W, const void* act, int64_t ldact, const void* bias,
                    const nf4ll_lora* lora, void* side_out, int64_t M, void* out, int64_t ldo, int accumulate,
                    void* workspace, int64_t workspace_bytes, int32_t* status, void* stream_v) {
  const char* who = mode == kFwd ? "nf4ll_forward" : "nf4ll_backward_dx";
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (int rc = check_mat(W, who)) return rc;
  if (M < 0) { set_detail("%s: M=%lld", who, static_cast<long long>(M)); return NF4LL_ERR_SHAPE; }
  if (M == 0) return NF4LL_OK;
  const int64_t NO = mode == kFwd ? W->N : W->K, KC = mode == kFwd ? W->K : W->N;
  if (int rc = check_act(act, ldact, KC, who, mode == kFwd ? "x" : "dy")) return rc;
  if (int rc = check_act(out, ldo, NO, who, mode == kFwd ? "y" : "dx")) return rc;
  if (int rc = check_lora(lora, who, mode == kBwd, W->K)) return rc;
  if (bias && (reinterpret_cast<uintptr_t>(bias) & 15)) { set_detail("%s: bias must be 16-byte aligned", who); return NF4LL_ERR_ALIGN; }
  if (M > (int64_t(1) << 30)) { set_detail("%s: M too large", who); return NF4LL_ERR_SHAPE; }
  if (int rc = require_sm100()) return rc;
  int sms = 148;
  if (int rc = device_sms(&sms)) return rc;
  const Plan pl = make_plan(M, NO, KC, lora ? lora->r : 0, sms);
  if (pl.total() > 0) {
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) || workspace_bytes < pl.total()) {
      set_detail("%s: needs a 256-byte aligned workspace of %lld bytes (got %lld)", who,
                 static_cast<long long>(pl.total()), static_cast<long long>(workspace_bytes));
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
  p.splits = pl.splits; p.m_pad = pl.m_pad; p.status = status;
  if (lora) {
    __half* left = reinterpret_cast<__half*>(ws);
    // rank-16 projection of the activation: T = drop(x).A^T (forward) or U = dy.B (backward)
    if (mode == kFwd) {
      if (int rc = lora_down_launch(act, ldact, lora->mask, lora->ld_mask, lora->keep_scale, lora->A, 1.0f, lora->scale,
                                    M, W->K, side_out, left, stream)) return rc;
      p.lora_right = static_cast<const __half*>(lora->B);
    } else {
      const void* bt = lora->Bt;
      if (!bt) {
        void* tmp = ws + pl.left_bytes;
        if (int rc = transpose_n16_launch(lora->B, tmp, W->N, stream)) return rc;
        bt = tmp;
      }
      // u = scale * dy.B: fp16 for the tensor core here, fp32 (side_out) for the dA kernel later
      if (int rc = lora_down_launch(act, ldact, nullptr, 0, 1.0f, bt, lora->scale, lora->scale, M, W->N, side_out, left,
                                    stream)) return rc;
      p.lora_right = static_cast<const __half*>(lora->A);
      p.mask = lora->mask; p.ld_mask = lora->ld_mask; p.keep_scale = lora->keep_scale;
    }
    p.lora_left = left;
  }
  if (pl.splits > 1) {
    p.counters = reinterpret_cast<int*>(ws + pl.left_bytes + pl.bt_bytes);
    p.partial = reinterpret_cast<float*>(ws + pl.left_bytes + pl.bt_bytes + pl.counter_bytes);
    NF4LL_CUDA(cudaMemsetAsync(p.counters, 0, pl.counter_bytes, stream));
  }
  CUtensorMap map;
  if (int rc = make_act_map(&map, act, M, KC, ldact)) return rc;
  cudaEvent_t ev0 = g_ev_start, ev1 = g_ev_stop;
  g_ev_start = g_ev_stop = nullptr;
  if (ev0) NF4LL_CUDA(cudaEventRecord(ev0, stream));
  const int rc = mode == kFwd ? launch<kFwd>(map, p, pl, stream) : launch<kBwd>(map, p, pl, stream);
  if (rc == NF4LL_OK && ev1) NF4LL_CUDA(cudaEventRecord(ev1, stream));
  return rc;
}

}  // namespace nf4ll

extern "C" int64_t nf4ll_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t r) {
  using namespace nf4ll;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  int sms = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) sms = v;
  }
  const int64_t f = make_plan(M, N, K, r, sms).total(), b = make_plan(M, K, N, r, sms).total();
  return f > b ? f : b;
}

extern "C" int nf4ll_forward(const nf4ll_mat* W, const void* x, int64_t ldx, const void* bias, const nf4ll_lora* lora,
                             void* t_out, int64_t M, void* y, int64_t ldy, void* workspace, int64_t workspace_bytes,
                             int32_t* status, void* stream) {
  return nf4ll::run_gemm(nf4ll::kFwd, W, x, ldx, bias, lora, t_out, M, y, ldy, 0, workspace, workspace_bytes, status, stream);
}

extern "C" int nf4ll_backward_dx(const nf4ll_mat* W, const void* dy, int64_t lddy, const nf4ll_lora* lora, void* u_out,
                                 int64_t M, void* dx, int64_t lddx, int32_t accumulate, void* workspace,
                                 int64_t workspace_bytes, int32_t* status, void* stream) {
  return nf4ll::run_gemm(nf4ll::kBwd, W, dy, lddy, nullptr, lora, u_out, M, dx, lddx, accumulate, workspace,
                         workspace_bytes, status, stream);
}

// Testing / tuning hook (no counterpart in the reference): force the tile shape and the split count
// chosen by the calling thread's next calls; zeros restore the built-in heuristic.
extern "C" void nf4ll_tune_override(int32_t bm_tiles, int32_t bn, int32_t splits) {
  nf4ll::g_force_bm = (bm_tiles == 1 || bm_tiles == 2) ? bm_tiles : 0;
  nf4ll::g_force_bn = (bn == 128 || bn == 256) ? bn : 0;
  nf4ll::g_force_splits = splits > 0 ? splits : 0;
}

// Measurement hook (no counterpart in the reference): the calling thread's NEXT nf4ll_forward /
// nf4ll_backward_dx records `start` immediately before and `stop` immediately after its tensor-core
// kernel on the call's stream (the rank-16 prologue kernel stays outside the pair). One-shot.
extern "C" void nf4ll_kernel_events(void* start, void* stop) {
  nf4ll::g_ev_start = static_cast<cudaEvent_t>(start);
  nf4ll::g_ev_stop = static_cast<cudaEvent_t>(stop);
}
