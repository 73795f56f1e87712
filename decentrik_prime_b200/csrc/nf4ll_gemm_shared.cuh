// Pieces shared by the single-CTA and the CTA-pair versions of the fused NF4 GEMM kernel.
#pragma once

#include <cuda.h>

#include "nf4ll_common.cuh"

namespace nf4ll {

enum : int { kFwd = 0, kBwd = 1 };

constexpr int kMaxSegments = 4;

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
  const float* lora_left;    // [M,16] fp32: T (forward) or s.U (backward)
  float left_scale;          // applied when the left operand is rounded to fp16: s (forward) or 1 (backward)
  const __half* lora_right;  // forward: B[N,16]; backward: A[16,K]
  const uint8_t* mask;       // backward only: keep-mask of the LoRA input [M, ld_mask], may be null
  int64_t ld_mask;
  float keep_scale;
  // forward over several projections stacked along N (Q|K|V, gate|up): per segment its own LoRA branch
  int n_seg;                          // 0: one projection, the fields above apply
  int64_t seg_begin[kMaxSegments];    // first output column of each segment, ascending, seg_begin[0] = 0
  const float* seg_left[kMaxSegments];     // [M,16] fp32 T of the segment, or null (no LoRA on it)
  const __half* seg_right[kMaxSegments];   // lora_B of the segment, offset so that it is indexed by the fused output column
  float seg_scale[kMaxSegments];
  // forward over gate|up with the gated-SiLU product in the epilogue: the weight is [2*gu_inter, K]
  // (gate rows, then up rows), a tile is 128 gate + 128 up columns, seg_* [0] / [1] hold the two LoRA
  // branches (lora_B not offset), and the three outputs g, u, h go through three tensor maps
  int64_t gu_inter;        // 0: not this mode
  int splits;              // split of the contraction across blockIdx.z
  float* partial;          // [splits][M_pad][NO] fp32 when splits > 1
  int* counters;           // one per output tile when splits > 1 (zero on entry, zero on exit)
  int64_t m_pad;
  int coop;                // split-K: every CTA of the grid is resident at once (cooperative launch), so the splits
                           // of a tile share its reduction instead of leaving it to the last one to finish
  int32_t* status;
  uint32_t spin_limit;     // polls of a tile counter (each followed by a short sleep) before a split gives up
};

constexpr uint32_t kCoopSpinLimit = 1u << 22;   // default for GemmParams::spin_limit
constexpr int kFixSlots = 8;     // 16 KB slots of the split-K fix-up ring (fits every tile shape's operand rings)

struct Abort {
  volatile int* flag;
  int32_t* status;
  __device__ __forceinline__ void raise(int code) const {
    *flag = 1;
    if (status) atomicCAS(status, 0, code);
  }
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, const Abort& ab, int code) {
  if (mbar_wait(bar, parity, ab.flag)) return true;
  ab.raise(code);
  return false;
}

__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

// Decode one quantisation block (32 bytes of codes) into one 128-byte row of a 128B-swizzled tile
// (row_addr: shared-memory address of the row; key: row index modulo 8).
__device__ __forceinline__ void dequant_block_to_smem(uint32_t row_addr, int key, const uint4& c0, const uint4& c1, float absmax) {
  const BlockTable t = make_block_table(absmax);
  const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) sts128(row_addr + ((j ^ key) << 4), decode_word(t, w[j]));
}

}  // namespace nf4ll
