// Small-batch forward (M <= 16 token rows): y[M,N] = x . W^T + bias + (s.T) . B^T, bound by the stream
// of NF4 bytes out of HBM, not by the tensor cores. Replaces, for decode-sized batches, the same
// reference call sites as the big-tile kernel (solution/fast_qwen.py:947, 1037, 1080-1112).
//
// Nothing is staged in shared memory: a warp owns 16 weight rows and a share of the contraction;
// each lane loads 8 bytes of codes per row and quantisation block straight into registers, turns
// them into fp16 with byte permutes against the 16 NF4 levels (a compile-time table, no per-block
// table build) in exactly the register layout mma.sync.m16n8k16 wants for its A operand, and the
// token rows are the B operand with the same column-to-slot assignment. The 64 weights of a block
// are accumulated on their own and folded into the running sum with that block's fp32 absmax, so
// the scale is applied once per block instead of once per weight:
//     y[m,n] = sum_blocks absmax[n,b] * sum_{k in b} x[m,k] * fp16(NF4[code[n,k]])
// This differs from the big-tile kernel's bit-exact fp16 weights by the rounding of
// NF4[c] * absmax to fp16 (relative 2^-12), inside the 1e-3 tolerance of the path.
#include "nf4ll_common.cuh"

namespace nf4ll {

__device__ __forceinline__ void mma16816_acc(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The 16 levels rounded to fp16, as byte planes for decode_word (same structure as a block table).
__device__ __forceinline__ BlockTable level_table() { return make_block_table(1.0f); }


struct StreamParams {
  const uint8_t* nib;
  const uint8_t* qabs;
  const float* scale2;
  const float* offset2;
  const float* code2;
  int64_t N, K;
  int64_t M;
  const __half* x;
  int64_t ldx;
  __half* y;
  int64_t ldy;
  const __half* bias;
  const float* t32;        // [M,16] fp32 = drop(x) . A^T, or null (no LoRA)
  const __half* lora_b;    // [N,16]
  float lora_scale;
};

// NT = number of 8-token tiles (1: M <= 8, 2: M <= 16). FULL4: the row holds a multiple of four
// quantisation blocks (every Qwen2.5 projection does), so the group-of-four loop needs no tail tests.
// kStreamWarps: warps per CTA that split the contraction (8; 16 for long rows under few CTAs, where eight
// warps per CTA would leave the SMs half empty).
template <int NT, bool FULL4, int kStreamWarps>
__global__ void __launch_bounds__(kStreamWarps * 32, NT == 1 ? 32 / kStreamWarps : (kStreamWarps == 8 ? 2 : 1))
nf4_stream_kernel(const StreamParams p) {
  // Launched as a programmatic dependent of the kernel before it. With a LoRA branch that kernel is the
  // rank-16 projection T = x . A^T, itself launched after everything earlier on the stream has
  // finished: x and the weights can be read at once and only the epilogue, which needs T, waits, so
  // the weight stream hides the projection. Without LoRA the predecessor may be x's producer: wait first.
  if (p.t32 == nullptr) pdl_wait();
  pdl_launch_dependents();
  __shared__ float s_code2[256];
  __shared__ float s_part[kStreamWarps][16][8 * NT + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  if (threadIdx.x < 256) s_code2[threadIdx.x] = p.code2[threadIdx.x];
  __syncthreads();

  const int64_t n0 = static_cast<int64_t>(blockIdx.x) * 16;
  const int64_t row0 = n0 + g, row1 = n0 + g + 8;          // N is a multiple of 64: always in range
  const int blocks_per_row = static_cast<int>(p.K / 64);
  const BlockTable lv = level_table();

  // running pointers of this lane: 8 bytes of codes per block and row, the absmax code of block b + t,
  // 32 bytes of each token row per block. Token rows past M read row 0: their sums are never stored.
  const int b_first = warp * 4;
  const uint8_t* w0 = p.nib + (row0 * p.K) / 2 + t * 8 + static_cast<int64_t>(b_first) * 32;
  const uint8_t* w1 = p.nib + (row1 * p.K) / 2 + t * 8 + static_cast<int64_t>(b_first) * 32;
  int64_t qa = (row0 * p.K) / 64 + b_first + t, qb = (row1 * p.K) / 64 + b_first + t;
  const __half* xr[NT];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    const int64_t tok = g + 8 * i;
    xr[i] = p.x + (tok < p.M ? tok : 0) * p.ldx + t * 16 + static_cast<int64_t>(b_first) * 64;
  }

  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // Blocks 4*warp .. 4*warp+3, then 32 further, ...: four at a time so that each lane recovers the
  // absmax of one of them (block b + t) for both of its rows and the quad shares them by shuffle.
  for (int b = b_first; b < blocks_per_row; b += kStreamWarps * 4) {
    const int nb = FULL4 ? 4 : ((blocks_per_row - b < 4) ? blocks_per_row - b : 4);
    uint2 c0[4], c1[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (FULL4 || u < nb) {
        c0[u] = __ldcs(reinterpret_cast<const uint2*>(w0 + u * 32));
        c1[u] = __ldcs(reinterpret_cast<const uint2*>(w1 + u * 32));
      } else {
        c0[u] = make_uint2(0, 0); c1[u] = make_uint2(0, 0);
      }
    }
    float am0 = 0.f, am1 = 0.f;
    if (FULL4 || t < nb) {
      am0 = block_absmax(s_code2[__ldg(p.qabs + qa)], __ldg(p.scale2 + (qa >> 8)), __ldg(p.offset2 + (qa >> 8)));
      am1 = block_absmax(s_code2[__ldg(p.qabs + qb)], __ldg(p.scale2 + (qb >> 8)), __ldg(p.offset2 + (qb >> 8)));
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float a0 = __shfl_sync(0xffffffffu, am0, (lane & ~3) | u);
      const float a1 = __shfl_sync(0xffffffffu, am1, (lane & ~3) | u);
      if (FULL4 || u < nb) {
        const uint4 lo0 = decode_word(lv, c0[u].x), hi0 = decode_word(lv, c0[u].y);   // row g:   k 16t..16t+7, +8..+15
        const uint4 lo1 = decode_word(lv, c1[u].x), hi1 = decode_word(lv, c1[u].y);   // row g+8
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          const uint4 xa = __ldg(reinterpret_cast<const uint4*>(xr[i] + u * 64));
          const uint4 xb = __ldg(reinterpret_cast<const uint4*>(xr[i] + u * 64 + 8));
          float blk[4] = {0.f, 0.f, 0.f, 0.f};
          mma16816_acc(blk, lo0.x, lo1.x, lo0.y, lo1.y, xa.x, xa.y);
          mma16816_acc(blk, lo0.z, lo1.z, lo0.w, lo1.w, xa.z, xa.w);
          mma16816_acc(blk, hi0.x, hi1.x, hi0.y, hi1.y, xb.x, xb.y);
          mma16816_acc(blk, hi0.z, hi1.z, hi0.w, hi1.w, xb.z, xb.w);
          acc[i][0] = fmaf(blk[0], a0, acc[i][0]);
          acc[i][1] = fmaf(blk[1], a0, acc[i][1]);
          acc[i][2] = fmaf(blk[2], a1, acc[i][2]);
          acc[i][3] = fmaf(blk[3], a1, acc[i][3]);
        }
      }
    }
    w0 += kStreamWarps * 4 * 32; w1 += kStreamWarps * 4 * 32;
    qa += kStreamWarps * 4; qb += kStreamWarps * 4;
#pragma unroll
    for (int i = 0; i < NT; ++i) xr[i] += kStreamWarps * 4 * 64;
  }

  // accumulator layout: acc[i][0..1] = (weight row g, tokens 8i + 2t, +1); acc[i][2..3] = row g + 8
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    s_part[warp][g][8 * i + 2 * t] = acc[i][0];
    s_part[warp][g][8 * i + 2 * t + 1] = acc[i][1];
    s_part[warp][g + 8][8 * i + 2 * t] = acc[i][2];
    s_part[warp][g + 8][8 * i + 2 * t + 1] = acc[i][3];
  }
  __syncthreads();
  if (p.t32 != nullptr) pdl_wait();              // T comes from the kernel this one was launched behind
  for (int idx = threadIdx.x; idx < 16 * 8 * NT; idx += kStreamWarps * 32) {
    const int r = idx & 15, tok = idx >> 4;      // consecutive threads -> consecutive output columns
    if (tok < p.M) {
      const int64_t n = n0 + r;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kStreamWarps; ++w) v += s_part[w][r][tok];
      if (p.bias) v += __half2float(p.bias[n]);
      if (p.t32) {
        const float* tr = p.t32 + tok * 16;
        const __half* br = p.lora_b + n * 16;
        float l = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) l = fmaf(tr[j], __half2float(br[j]), l);
        v = fmaf(l, p.lora_scale, v);
      }
      p.y[tok * p.ldy + n] = __float2half_rn(v);
    }
  }
}

int stream_forward_launch(const nf4ll_mat* W, const void* x, int64_t ldx, const void* bias, const float* t32,
                          const void* lora_b, float lora_scale, int64_t M, void* y, int64_t ldy, cudaStream_t stream) {
  StreamParams p{};
  p.nib = W->nib; p.qabs = W->qabs; p.scale2 = W->scale2; p.offset2 = W->offset2; p.code2 = W->code2;
  p.N = W->N; p.K = W->K; p.M = M;
  p.x = static_cast<const __half*>(x); p.ldx = ldx;
  p.y = static_cast<__half*>(y); p.ldy = ldy;
  p.bias = static_cast<const __half*>(bias);
  p.t32 = t32; p.lora_b = static_cast<const __half*>(lora_b); p.lora_scale = lora_scale;
  const unsigned grid = static_cast<unsigned>(W->N / 16);
  const bool full4 = (W->K % 256) == 0;
  const cudaStream_t st = stream;
  int dev = 0, sms = 148;
  NF4LL_CUDA(cudaGetDevice(&dev));
  NF4LL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  // few CTAs (narrow outputs) with long rows: sixteen warps per CTA keep the SMs occupied
  const bool wide = full4 && grid < 3u * static_cast<unsigned>(sms) && W->K / 64 >= 256;
  void (*kernel)(const StreamParams);
  if (wide) kernel = (M <= 8) ? nf4_stream_kernel<1, true, 16> : nf4_stream_kernel<2, true, 16>;
  else kernel = (M <= 8) ? (full4 ? nf4_stream_kernel<1, true, 8> : nf4_stream_kernel<1, false, 8>)
                         : (full4 ? nf4_stream_kernel<2, true, 8> : nf4_stream_kernel<2, false, 8>);
  PdlLaunch lc(dim3(grid), dim3(wide ? 512 : 256), 0, st);
  NF4LL_CUDA(cudaLaunchKernelEx(&lc.cfg, kernel, p));
  return NF4LL_OK;
}

}  // namespace nf4ll
