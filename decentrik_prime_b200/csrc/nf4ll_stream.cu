// Small-batch forward (a handful of token rows): y[M,N] = x . W^T + bias + (s.T) . B^T, bound by the stream
// of NF4 bytes out of HBM, not by the tensor cores. Replaces, for decode-sized batches, the same
// reference call sites as the big-tile kernel (solution/fast_qwen.py:947, 1037, 1080-1112).
//
// Work is cut into units of 16 weight rows x a slice of the contraction; a warp owns a unit at a time.
// The first unit of every warp is fixed by its position in the grid (so the weight stream starts before
// anything else on the stream has to be waited for), later units are handed out through a global counter,
// which keeps all SMs busy to the end whatever the shape. Per unit and quantisation block a lane loads 8
// bytes of codes of each of its two rows straight into registers and turns every BYTE (two 4-bit codes)
// into two fp16 levels with ONE shared-memory load from a 256-entry table of half2 pairs. The table is
// replicated per lane (entry stride 128 B = 32 lanes x 4 B, lane l reads bank l: no bank conflicts whatever
// the codes are), so a lookup costs one shift, one logic op and one conflict-free 4-byte LDS for two
// weights, against 21 integer operations per 8 weights for a byte-permute decode in registers. The levels
// land directly in the A-operand layout of mma.sync.m16n8k16; the token rows are the B operand with the same
// column-to-slot assignment. The 64 weights of a block are accumulated on their own and folded into the
// running sum with that block's fp32 absmax, so the scale is applied once per block:
//     y[m,n] = sum_blocks absmax[n,b] * sum_{k in b} x[m,k] * fp16(NF4[code[n,k]])
// This differs from the big-tile kernel's bit-exact fp16 weights by the rounding of NF4[c] * absmax to
// fp16 (relative 2^-12), inside the 1e-3 tolerance of the path.
//
// With the contraction cut into S > 1 slices, a unit writes its 16 x (8 NT) partial sums to a slab in the
// workspace and bumps its row group's counter; the warp that arrives last adds the S partial sums in slice
// order (a fixed order: results do not depend on timing), adds bias and the LoRA term and stores fp16.
#include "nf4ll_common.cuh"

namespace nf4ll {

__device__ __forceinline__ void mma16816_acc(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

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
  int slices;              // S: slices of the contraction
  int blocks_per_slice;    // quantisation blocks per slice (a multiple of 4, except that the last slice ends with the row)
  int n_units;             // (N / 16) * S
  float* slab;             // [N/16][S][8 NT tokens][16 rows] fp32 partial sums (S > 1)
  int* counters;           // [0]: next unit to hand out (beyond the statically assigned ones); [1 + row group]: arrivals
};

constexpr int kStreamWarps = 8;
constexpr int kTableBytes = 256 * 128;       // 256 byte values x 32 lanes x half2

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// byte offset into the table of the entry of byte `I` of `w` for this lane (lane_off = 4 * lane): entry
// stride 128 bytes, so bits 7..14 take the byte value and bits 2..6 the lane
template <int I>
__device__ __forceinline__ uint32_t entry_offset(uint32_t w, uint32_t lane_off) {
  const uint32_t shifted = (I == 0) ? (w << 7) : (w >> (8 * I - 7));
  return (shifted & 0x7F80u) | lane_off;
}

// the 8 weights of one 32-bit word of codes as four half2 registers (element order: high nibble first).
// `table` is the address of a static shared array: a link-time constant that folds into the load's offset.
__device__ __forceinline__ void decode8(uint32_t w, uint32_t table, uint32_t lane_off, uint32_t (&h)[4]) {
  h[0] = lds_u32(table + entry_offset<0>(w, lane_off));
  h[1] = lds_u32(table + entry_offset<1>(w, lane_off));
  h[2] = lds_u32(table + entry_offset<2>(w, lane_off));
  h[3] = lds_u32(table + entry_offset<3>(w, lane_off));
}

// NT = number of 8-token tiles (M <= 8 NT).
template <int NT>
__global__ void __launch_bounds__(kStreamWarps * 32, NT == 1 ? 3 : (NT == 2 ? 3 : (NT == 4 ? 2 : 1)))
nf4_stream_kernel(const StreamParams p) {
  // Launched as a programmatic dependent of the kernel before it (the rank-16 projection T = x . A^T when
  // there is a LoRA branch, which also clears this launch's counters): the table build and the first unit's
  // weight stream overlap that kernel; the first write to the workspace waits for it.
  pdl_launch_dependents();
  __shared__ __align__(128) uint32_t s_tbl[kTableBytes / 4];
  __shared__ float s_code2[256];
  __shared__ uint32_t s_lv[16];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const float code2_mine = threadIdx.x < 256 ? p.code2[threadIdx.x] : 0.f;     // in flight while the table is built
  {
    constexpr float lv[16] = {NF4LL_LEVELS};
    if (threadIdx.x < 16) {
      float v = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) v = (static_cast<int>(threadIdx.x) == j) ? lv[j] : v;
      s_lv[threadIdx.x] = __half_as_ushort(__float2half_rn(v));
    }
    __syncthreads();
    // four lanes' copies of an entry per 16-byte store
    for (int idx = threadIdx.x; idx < 256 * 8; idx += kStreamWarps * 32) {
      const int v = idx >> 3;                       // byte value: even element in the high nibble
      const uint32_t e = s_lv[v >> 4] | (s_lv[v & 15] << 16);
      reinterpret_cast<uint4*>(s_tbl)[idx] = make_uint4(e, e, e, e);
    }
  }
  // x, the weights and code2 may be read at once: what precedes this kernel on the stream is either the
  // rank-16 projection kernel, itself started only after all earlier work had finished, or the memset of the
  // counters, which orders this kernel after everything before it
  bool waited = false;
  if (threadIdx.x < 256) s_code2[threadIdx.x] = code2_mine;
  __syncthreads();

  const uint32_t table = smem_u32(s_tbl), lane_off = lane * 4;
  const int n_rg = static_cast<int>(p.N / 16);
  const int bpr = static_cast<int>(p.K / 64);       // quantisation blocks per weight row
  const int total_warps = gridDim.x * kStreamWarps;
  int unit = blockIdx.x * kStreamWarps + warp;

  while (unit < p.n_units) {
    // slice-major order: the warps resident at any time work on one slice of the contraction, i.e. on the
    // same few columns of x, which then stay in L1
    const int sl = unit / n_rg, rg = unit - sl * n_rg;
    const int64_t n0 = static_cast<int64_t>(rg) * 16;
    const int64_t row0 = n0 + g, row1 = n0 + g + 8;
    const int b_begin = sl * p.blocks_per_slice;
    int b_end = b_begin + p.blocks_per_slice;
    if (b_end > bpr) b_end = bpr;

    // running pointers of this lane: 8 bytes of codes per block and row, the absmax code of block b + t,
    // 32 bytes of each token row per block. Token rows past M read row 0: their sums are never stored.
    const uint8_t* w0 = p.nib + (row0 * p.K) / 2 + t * 8 + static_cast<int64_t>(b_begin) * 32;
    const uint8_t* w1 = p.nib + (row1 * p.K) / 2 + t * 8 + static_cast<int64_t>(b_begin) * 32;
    int64_t qa = (row0 * p.K) / 64 + b_begin + t, qb = (row1 * p.K) / 64 + b_begin + t;
    const __half* xr[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int64_t tok = g + 8 * i;
      xr[i] = p.x + (tok < p.M ? tok : 0) * p.ldx + t * 16 + static_cast<int64_t>(b_begin) * 64;
    }
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    // Four blocks at a time: each lane recovers the absmax of one of them (block b + t) for both of its rows
    // and the quad shares them by shuffle.
    for (int b = b_begin; b < b_end; b += 4) {
      const int nb = (b_end - b < 4) ? b_end - b : 4;
      uint2 c0[4], c1[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (u < nb) {
          c0[u] = __ldcs(reinterpret_cast<const uint2*>(w0 + u * 32));
          c1[u] = __ldcs(reinterpret_cast<const uint2*>(w1 + u * 32));
        } else {
          c0[u] = make_uint2(0, 0); c1[u] = make_uint2(0, 0);
        }
      }
      float am0 = 0.f, am1 = 0.f;
      if (t < nb) {
        am0 = block_absmax(s_code2[__ldg(p.qabs + qa)], __ldg(p.scale2 + (qa >> 8)), __ldg(p.offset2 + (qa >> 8)));
        am1 = block_absmax(s_code2[__ldg(p.qabs + qb)], __ldg(p.scale2 + (qb >> 8)), __ldg(p.offset2 + (qb >> 8)));
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float a0 = __shfl_sync(0xffffffffu, am0, (lane & ~3) | u);
        const float a1 = __shfl_sync(0xffffffffu, am1, (lane & ~3) | u);
        if (u < nb) {
          uint32_t lo0[4], hi0[4], lo1[4], hi1[4];
          decode8(c0[u].x, table, lane_off, lo0); decode8(c0[u].y, table, lane_off, hi0);     // row g:   k 16t..16t+7, +8..+15
          decode8(c1[u].x, table, lane_off, lo1); decode8(c1[u].y, table, lane_off, hi1);     // row g+8
#pragma unroll
          for (int i = 0; i < NT; ++i) {
            const uint4 xa = __ldg(reinterpret_cast<const uint4*>(xr[i] + u * 64));
            const uint4 xb = __ldg(reinterpret_cast<const uint4*>(xr[i] + u * 64 + 8));
            float blk[4] = {0.f, 0.f, 0.f, 0.f};
            mma16816_acc(blk, lo0[0], lo1[0], lo0[1], lo1[1], xa.x, xa.y);
            mma16816_acc(blk, lo0[2], lo1[2], lo0[3], lo1[3], xa.z, xa.w);
            mma16816_acc(blk, hi0[0], hi1[0], hi0[1], hi1[1], xb.x, xb.y);
            mma16816_acc(blk, hi0[2], hi1[2], hi0[3], hi1[3], xb.z, xb.w);
            acc[i][0] = fmaf(blk[0], a0, acc[i][0]);
            acc[i][1] = fmaf(blk[1], a0, acc[i][1]);
            acc[i][2] = fmaf(blk[2], a1, acc[i][2]);
            acc[i][3] = fmaf(blk[3], a1, acc[i][3]);
          }
        }
      }
      w0 += 4 * 32; w1 += 4 * 32;
      qa += 4; qb += 4;
#pragma unroll
      for (int i = 0; i < NT; ++i) xr[i] += 4 * 64;
    }

    // accumulator layout: acc[i][0..1] = (weight row g, tokens 8i + 2t, +1); acc[i][2..3] = row g + 8
    if (!waited) {
      pdl_wait();                 // T, and the zeroed counters, come from the kernel this one was launched behind
      waited = true;
    }
    bool finish = true;
    if (p.slices > 1) {
      float* mine = p.slab + ((static_cast<int64_t>(rg) * p.slices + sl) * (8 * NT)) * 16;
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        mine[(8 * i + 2 * t) * 16 + g] = acc[i][0];
        mine[(8 * i + 2 * t + 1) * 16 + g] = acc[i][1];
        mine[(8 * i + 2 * t) * 16 + g + 8] = acc[i][2];
        mine[(8 * i + 2 * t + 1) * 16 + g + 8] = acc[i][3];
      }
      __threadfence();
      __syncwarp();
      int prev = 0;
      if (lane == 0) prev = atomicAdd(p.counters + 1 + rg, 1);
      prev = __shfl_sync(0xffffffffu, prev, 0);
      finish = (prev == p.slices - 1);
      if (finish) {
        __threadfence();
        const float* all = p.slab + (static_cast<int64_t>(rg) * p.slices * (8 * NT)) * 16;
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
        for (int s2 = 0; s2 < p.slices; ++s2) {
          const float* part = all + static_cast<int64_t>(s2) * (8 * NT) * 16;
#pragma unroll
          for (int i = 0; i < NT; ++i) {
            acc[i][0] += __ldcg(part + (8 * i + 2 * t) * 16 + g);
            acc[i][1] += __ldcg(part + (8 * i + 2 * t + 1) * 16 + g);
            acc[i][2] += __ldcg(part + (8 * i + 2 * t) * 16 + g + 8);
            acc[i][3] += __ldcg(part + (8 * i + 2 * t + 1) * 16 + g + 8);
          }
        }
      }
    }
    if (finish) {
      // bias, LoRA term, one rounding to fp16
      float bias0 = 0.f, bias1 = 0.f;
      if (p.bias) { bias0 = __half2float(p.bias[row0]); bias1 = __half2float(p.bias[row1]); }
      float br0[16], br1[16];
      if (p.t32) {
        const uint4* b0p = reinterpret_cast<const uint4*>(p.lora_b + row0 * 16);
        const uint4* b1p = reinterpret_cast<const uint4*>(p.lora_b + row1 * 16);
        float tmp[8];
        unpack8(__ldg(b0p), tmp);
#pragma unroll
        for (int j = 0; j < 8; ++j) br0[j] = tmp[j] * p.lora_scale;
        unpack8(__ldg(b0p + 1), tmp);
#pragma unroll
        for (int j = 0; j < 8; ++j) br0[8 + j] = tmp[j] * p.lora_scale;
        unpack8(__ldg(b1p), tmp);
#pragma unroll
        for (int j = 0; j < 8; ++j) br1[j] = tmp[j] * p.lora_scale;
        unpack8(__ldg(b1p + 1), tmp);
#pragma unroll
        for (int j = 0; j < 8; ++j) br1[8 + j] = tmp[j] * p.lora_scale;
      }
#pragma unroll
      for (int i = 0; i < NT; ++i) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int64_t tok = 8 * i + 2 * t + e;
          if (tok < p.M) {
            float v0 = acc[i][e] + bias0, v1 = acc[i][2 + e] + bias1;
            if (p.t32) {
              const float4* tr = reinterpret_cast<const float4*>(p.t32 + tok * 16);
              float l0 = 0.f, l1 = 0.f;
#pragma unroll
              for (int j4 = 0; j4 < 4; ++j4) {
                const float4 tv = __ldcg(tr + j4);
                l0 = fmaf(tv.x, br0[4 * j4], l0); l0 = fmaf(tv.y, br0[4 * j4 + 1], l0);
                l0 = fmaf(tv.z, br0[4 * j4 + 2], l0); l0 = fmaf(tv.w, br0[4 * j4 + 3], l0);
                l1 = fmaf(tv.x, br1[4 * j4], l1); l1 = fmaf(tv.y, br1[4 * j4 + 1], l1);
                l1 = fmaf(tv.z, br1[4 * j4 + 2], l1); l1 = fmaf(tv.w, br1[4 * j4 + 3], l1);
              }
              v0 += l0; v1 += l1;
            }
            p.y[tok * p.ldy + row0] = __float2half_rn(v0);
            p.y[tok * p.ldy + row1] = __float2half_rn(v1);
          }
        }
      }
    }
    // next unit from the shared counter (the first `total_warps` units were assigned statically)
    int next = 0;
    if (lane == 0) next = total_warps + atomicAdd(p.counters, 1);
    unit = __shfl_sync(0xffffffffu, next, 0);
  }
}

// Units and slices for W[N,K] at M rows: aim at several units per resident warp so that the dynamic hand-out
// can balance the SMs, but never cut a row into slices shorter than 8 quantisation blocks.
void stream_plan(int64_t N, int64_t K, int64_t M, int sms, int force_slices, int* slices, int* blocks_per_slice) {
  const int bpr = static_cast<int>(K / 64);
  const int64_t row_groups = N / 16;
  int s = 1;
  const int64_t want = static_cast<int64_t>(sms) * 48;            // units to aim for
  if (row_groups < want) s = static_cast<int>((want + row_groups - 1) / row_groups);
  int max_s = bpr / 8;
  if (max_s < 1) max_s = 1;
  if (s > max_s) s = max_s;
  if (force_slices > 0) s = force_slices;
  int per = (bpr + s - 1) / s;
  per = (per + 3) / 4 * 4;                                        // whole groups of four blocks
  s = (bpr + per - 1) / per;
  *slices = s;
  *blocks_per_slice = per;
}

int64_t stream_workspace_bytes(int64_t N, int64_t K, int64_t M, int sms, int force_slices) {
  int s = 1, per = 0;
  stream_plan(N, K, M, sms, force_slices, &s, &per);
  const int nt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
  const int64_t counters = (1 + N / 16) * 4;
  const int64_t slab = s > 1 ? (N / 16) * s * (8 * nt) * 16 * 4 : 0;
  return (counters + 255) / 256 * 256 + (slab + 255) / 256 * 256;
}

// `scratch` holds the counters (zeroed here unless `counters_zeroed`: the rank-16 projection kernel launched just
// before has then done it) followed, 256-byte aligned, by the slab.
int stream_forward_launch(const nf4ll_mat* W, const void* x, int64_t ldx, const void* bias, const float* t32,
                          const void* lora_b, float lora_scale, int64_t M, void* y, int64_t ldy, void* scratch,
                          bool counters_zeroed, int force_slices, cudaStream_t stream) {
  int dev = 0, sms = 148;
  NF4LL_CUDA(cudaGetDevice(&dev));
  NF4LL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  StreamParams p{};
  p.nib = W->nib; p.qabs = W->qabs; p.scale2 = W->scale2; p.offset2 = W->offset2; p.code2 = W->code2;
  p.N = W->N; p.K = W->K; p.M = M;
  p.x = static_cast<const __half*>(x); p.ldx = ldx;
  p.y = static_cast<__half*>(y); p.ldy = ldy;
  p.bias = static_cast<const __half*>(bias);
  p.t32 = t32; p.lora_b = static_cast<const __half*>(lora_b); p.lora_scale = lora_scale;
  stream_plan(W->N, W->K, M, sms, force_slices, &p.slices, &p.blocks_per_slice);
  p.n_units = static_cast<int>(W->N / 16) * p.slices;
  const int64_t counter_bytes = ((1 + W->N / 16) * 4 + 255) / 256 * 256;
  p.counters = static_cast<int*>(scratch);
  p.slab = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + counter_bytes);
  if (!counters_zeroed) NF4LL_CUDA(cudaMemsetAsync(p.counters, 0, (1 + W->N / 16) * 4, stream));
  const int nt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
  void (*kernel)(const StreamParams) = nt == 1 ? nf4_stream_kernel<1> : (nt == 2 ? nf4_stream_kernel<2>
                                       : (nt == 4 ? nf4_stream_kernel<4> : nf4_stream_kernel<8>));
  const int smem = 0;
  int per_sm = 0;
  NF4LL_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kStreamWarps * 32, smem));
  if (per_sm < 1) per_sm = 1;
  int64_t grid = (p.n_units + kStreamWarps - 1) / kStreamWarps;
  if (grid > static_cast<int64_t>(sms) * per_sm) grid = static_cast<int64_t>(sms) * per_sm;
  PdlLaunch lc(dim3(static_cast<unsigned>(grid)), dim3(kStreamWarps * 32), smem, stream);
  NF4LL_CUDA(cudaLaunchKernelEx(&lc.cfg, kernel, p));
  return NF4LL_OK;
}

}  // namespace nf4ll
