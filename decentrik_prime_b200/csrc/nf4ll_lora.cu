// The skinny (rank-16) LoRA products around the fused linear, as small tensor-core GEMMs:
//   lora_down   t[M,16]  = drop(x)[M,C] . R^T,  R = lora_A [16,C]      (forward: T)
//                                               R = lora_B^T [16,C]    (backward: U = dy . B)
//   lora_grads  dA[16,K] (+)= u^T . drop(x),  dB[N,16] (+)= scale * dy^T . t
// Replaces solution/fast_qwen.py:943-944 and 1369-1374 of the reference. Accumulation is fp32 and
// t / u stay fp32 between the passes (split into fp16 hi + lo parts where they feed a tensor-core
// operand): the reference rounds them (and dA/dB) to fp16, which costs up to 0.08 absolute error on
// gradients of magnitude ~100.
//
// Both kernels are bandwidth-bound passes over x / dy (32 multiply-adds per fp16 element read), so
// they use warp-level mma.sync.m16n8k16 with operands loaded straight from global memory with
// 128-bit loads; there is nothing for TMA staging or tensor memory to win here.
#include "nf4ll_common.cuh"

namespace nf4ll {

// ---------------------------------------------------------------------------------------------
// Row reduction: t[M,16] = scale * drop(act)[M,C] . R^T with R [16,C] row-major fp16.
// One CTA = 8*RG rows x a range of the contraction, 8 warps; warp w takes the 32-column chunks
// w, w+8, ... of the range. Per chunk a lane issues RG 128-bit loads of act (rows g, g+8, ...) and
// two of R (rank rows g and g+8); a lane's 8 consecutive columns feed two MMAs with the SAME
// column-to-slot assignment on both operands, so no shuffle or shared-memory transpose is needed:
// out^T[16 ranks, 8 rows] = R[16, k] . act^T[k, 8 rows]. The warps' partial results are summed
// through shared memory. The contraction is split over grid.y so that every SM has loads in
// flight; how the parts of one row block meet depends on COMBINE:
//   kDownDirect   grid.y == 1, plain stores;
//   kDownCluster  the grid.y CTAs of a row block form one thread-block cluster (at most 8); after a
//                 cluster barrier rank 0 adds the others' partial sums out of their shared memory in
//                 rank order and stores: no zero-fill, no atomics, bit-reproducible;
//   kDownAtomic   more than 8 parts (few rows, long contraction): fp32 atomics into t, which the
//                 launcher zeroes first.
// `zero_words` 32-bit words at `zero_ptr` are cleared by CTA (0,0): the caller's next kernel (the
// split-K GEMM this product feeds) finds its tile counters reset without a separate memset.
// ---------------------------------------------------------------------------------------------
constexpr int kDownWarps = 8;
constexpr int kDownDirect = 0, kDownCluster = 1, kDownAtomic = 2;

__device__ __forceinline__ uint32_t down_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void down_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float down_peer_load(const float* local, uint32_t rank) {
  uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(local)), r;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(r) : "memory");
  return v;
}

template <int RG, int COMBINE, int NW>
__global__ void __launch_bounds__(NW * 32)
lora_down_kernel(const __half* __restrict__ act, int64_t ldact, const uint8_t* __restrict__ mask, int64_t ld_mask,
                 float keep_scale, const __half* __restrict__ R, float scale, int64_t M, int64_t C, int64_t c_per_cta,
                 float* __restrict__ t32, int* __restrict__ zero_ptr, int zero_words) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int ROWS = 8 * RG;
  __shared__ float part[NW][ROWS][17];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  if (blockIdx.x == 0 && blockIdx.y == 0) {
    for (int i = threadIdx.x; i < zero_words; i += NW * 32) zero_ptr[i] = 0;
  }
  const int64_t m0 = static_cast<int64_t>(blockIdx.x) * ROWS;
  const int64_t c_begin = static_cast<int64_t>(blockIdx.y) * c_per_cta;
  const int64_t c_end = (c_begin + c_per_cta < C) ? c_begin + c_per_cta : C;
  const __half* ap[RG];
  const uint8_t* mp[RG];
  bool ok[RG];
#pragma unroll
  for (int i = 0; i < RG; ++i) {
    const int64_t row = m0 + g + 8 * i;
    ok[i] = row < M;
    ap[i] = act + (ok[i] ? row : 0) * ldact;
    mp[i] = mask ? mask + (ok[i] ? row : 0) * ld_mask : nullptr;
  }
  const __half* r0p = R + static_cast<int64_t>(g) * C;
  const __half* r1p = R + static_cast<int64_t>(g + 8) * C;
  float c[RG][4];
#pragma unroll
  for (int i = 0; i < RG; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) c[i][j] = 0.f;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  // U chunks per trip, every load of the trip issued before the first use: the loop is bound by the
  // number of bytes a warp keeps in flight, not by arithmetic
  constexpr int U = (RG == 2) ? 4 : 2;
  for (int64_t k0 = c_begin + static_cast<int64_t>(warp) * 32 + t * 8; k0 < c_end; k0 += U * NW * 32) {
    uint4 x[U][RG], ra[U], rb[U];
    uint2 mk[U][RG];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t k = k0 + u * NW * 32;
      const bool in = k < c_end;
#pragma unroll
      for (int i = 0; i < RG; ++i) {
        x[u][i] = (in && ok[i]) ? __ldg(reinterpret_cast<const uint4*>(ap[i] + k)) : zero;
        mk[u][i] = (in && mask) ? __ldg(reinterpret_cast<const uint2*>(mp[i] + k)) : make_uint2(0, 0);
      }
      ra[u] = in ? __ldg(reinterpret_cast<const uint4*>(r0p + k)) : zero;
      rb[u] = in ? __ldg(reinterpret_cast<const uint4*>(r1p + k)) : zero;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (mask) {
#pragma unroll
        for (int i = 0; i < RG; ++i) x[u][i] = drop8(x[u][i], mk[u][i], keep_scale);
      }
      // columns k..k+3 -> MMA slots (2t, 2t+1, 2t+8, 2t+9) of the first MMA, k+4..k+7 of the second
#pragma unroll
      for (int i = 0; i < RG; ++i) {
        mma16816(c[i], ra[u].x, rb[u].x, ra[u].y, rb[u].y, x[u][i].x, x[u][i].y);
        mma16816(c[i], ra[u].z, rb[u].z, ra[u].w, rb[u].w, x[u][i].z, x[u][i].w);
      }
    }
  }
  // accumulator layout: c[.][0], c[.][1] = (rank g, rows 2t, 2t+1); c[.][2], c[.][3] = (rank g+8, same rows)
#pragma unroll
  for (int i = 0; i < RG; ++i) {
    part[warp][8 * i + 2 * t][g] = c[i][0];      part[warp][8 * i + 2 * t + 1][g] = c[i][1];
    part[warp][8 * i + 2 * t][g + 8] = c[i][2];  part[warp][8 * i + 2 * t + 1][g + 8] = c[i][3];
  }
  __syncthreads();
  if (COMBINE == kDownCluster) {
    // every CTA folds its warps' parts into part[0]; rank 0 then gathers the cluster's
    for (int idx = threadIdx.x; idx < ROWS * 16; idx += NW * 32) {
      const int row = idx >> 4, j = idx & 15;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) v += part[w][row][j];
      part[0][row][j] = v;                       // read and written by this thread only
    }
    down_cluster_sync();
    if (down_cluster_rank() == 0) {
      for (int idx = threadIdx.x; idx < ROWS * 16; idx += NW * 32) {
        const int row = idx >> 4, j = idx & 15;
        if (m0 + row < M) {
          float v = part[0][row][j];
          for (uint32_t r = 1; r < gridDim.y; ++r) v += down_peer_load(&part[0][row][j], r);
          t32[(m0 + row) * 16 + j] = v * scale;
        }
      }
    }
    down_cluster_sync();                         // peers keep their shared memory until rank 0 has read it
  } else {
    for (int idx = threadIdx.x; idx < ROWS * 16; idx += NW * 32) {
      const int row = idx >> 4, j = idx & 15;
      if (m0 + row < M) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) v += part[w][row][j];
        if (COMBINE == kDownAtomic) atomicAdd(t32 + (m0 + row) * 16 + j, v * scale);
        else t32[(m0 + row) * 16 + j] = v * scale;
      }
    }
  }
}

// t16 = fp16(scale * t32), for callers of the stand-alone projection that want the fp16 copy
__global__ void scale_to_half_kernel(const float* __restrict__ t32, __half* __restrict__ t16, float scale, int64_t n) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) t16[i] = __float2half_rn(t32[i] * scale);
}

// B[N,16] -> Bt[16,N] (fp16), for callers that do not keep a transposed shadow of lora_B.
__global__ void transpose_n16_kernel(const __half* __restrict__ B, __half* __restrict__ Bt, int64_t N) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < N * 16) {
    const int64_t n = i >> 4;
    const int j = static_cast<int>(i & 15);
    Bt[j * N + n] = B[i];
  }
}

int transpose_n16_launch(const void* B, void* Bt, int64_t N, cudaStream_t stream) {
  const int64_t total = N * 16;
  count_launch();
  transpose_n16_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      static_cast<const __half*>(B), static_cast<__half*>(Bt), N);
  NF4LL_CUDA(cudaGetLastError());
  return NF4LL_OK;
}

// R is [16,C] row-major. t32 (fp32 [M,16], required) = scale * (drop(act) . R^T). `zero_ptr` / `zero_words`:
// optional 32-bit words the kernel clears on the way (see the kernel).
int lora_down_launch(const void* act, int64_t ldact, const uint8_t* mask, int64_t ld_mask, float keep_scale,
                     const void* R, float scale, int64_t M, int64_t C, void* t32, int* zero_ptr, int zero_words,
                     cudaStream_t stream) {
  if (M == 0) {
    if (zero_words > 0) NF4LL_CUDA(cudaMemsetAsync(zero_ptr, 0, sizeof(int) * zero_words, stream));
    return NF4LL_OK;
  }
  int dev = 0, sms = 148;
  NF4LL_CUDA(cudaGetDevice(&dev));
  NF4LL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const __half* a = static_cast<const __half*>(act);
  const __half* r = static_cast<const __half*>(R);
  float* t = static_cast<float*>(t32);
  const int64_t groups16 = (M + 15) / 16;
  if (groups16 * 4 >= 3 * static_cast<int64_t>(sms)) {
    // enough rows for (nearly) one CTA per SM at 16 rows each: a CTA takes the whole contraction,
    // sixteen warps deep, and stores its rows directly
    PdlLaunch lc(dim3(static_cast<unsigned>(groups16), 1), dim3(16 * 32), 0, stream);
    NF4LL_CUDA(cudaLaunchKernelEx(&lc.cfg, lora_down_kernel<2, kDownDirect, 16>, a, ldact, mask, ld_mask, keep_scale, r, scale, M, C,
                                  C, t, zero_ptr, zero_words));
    return NF4LL_OK;
  }
  const int64_t row_groups = (M + 31) / 32;
  const int64_t units = (C + kDownWarps * 32 - 1) / (kDownWarps * 32);     // 256-column units
  int64_t ks = (2 * static_cast<int64_t>(sms)) / row_groups;     // at most two CTAs per SM: one wave, no tail
  if (ks > units) ks = units;
  if (ks < 1) ks = 1;
  // decode-sized batches are all latency: eight CTAs in one cluster (no zero-fill, no atomics) beat more CTAs + a memset
  if (ks > 8 && M * C <= (int64_t(1) << 21)) ks = 8;
  const int64_t c_per_cta = (units + ks - 1) / ks * (kDownWarps * 32);
  ks = (C + c_per_cta - 1) / c_per_cta;
  dim3 grid(static_cast<unsigned>(row_groups), static_cast<unsigned>(ks));
  if (ks == 1) {
    count_launch();
    lora_down_kernel<4, kDownDirect, kDownWarps><<<grid, kDownWarps * 32, 0, stream>>>(
        a, ldact, mask, ld_mask, keep_scale, r, scale, M, C, c_per_cta, t, zero_ptr, zero_words);
  } else if (ks <= 8) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = dim3(kDownWarps * 32); cfg.dynamicSmemBytes = 0; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = static_cast<unsigned>(ks); attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    count_launch();
    NF4LL_CUDA(cudaLaunchKernelEx(&cfg, lora_down_kernel<4, kDownCluster, kDownWarps>, a, ldact, mask, ld_mask, keep_scale, r,
                                  scale, M, C, c_per_cta, t, zero_ptr, zero_words));
  } else {
    NF4LL_CUDA(cudaMemsetAsync(t32, 0, sizeof(float) * 16 * M, stream));
    count_launch();
    lora_down_kernel<4, kDownAtomic, kDownWarps><<<grid, kDownWarps * 32, 0, stream>>>(
        a, ldact, mask, ld_mask, keep_scale, r, scale, M, C, c_per_cta, t, zero_ptr, zero_words);
  }
  NF4LL_CUDA(cudaGetLastError());
  return NF4LL_OK;
}

// ---------------------------------------------------------------------------------------------
// Column reduction: out[c][j] (+)= scale * sum_m drop(act)[m][c] * side[m][j]   (j < 16)
// as out^T[16, C] = side^T[16, M] . drop(act)[M, C]. One CTA = 64 columns x a range of rows, 4
// warps. The rows arrive in 64-row stages through a ring of shared-memory buffers filled by
// cp.async (act, mask and side as they lie in memory, two stages always in flight per CTA and
// several CTAs per SM: the kernel is a pass over act at memory speed). A stage is then prepared in
// place - dropout applied to the act tile, side transposed and split into fp16 hi + lo parts (two
// MMAs recover ~22 mantissa bits) - and warp w contracts rows 16w..16w+15 of it against all 64
// columns (ldmatrix.trans delivers the row-major act tile as the MMA's k-by-n operand). Row ranges
// of different CTAs are combined with fp32 atomics, so the summation order across ranges is not fixed.
// out index = j * ld_j + c * ld_c: dA[16,K] uses (K, 1), dB[N,16] uses (1, 16).
// ---------------------------------------------------------------------------------------------
constexpr int kGradThreads = 128;
constexpr int kGradCols = 64;
constexpr int kGradStage = 64;
constexpr int kGradRing = 3;
constexpr int kActStride = 72;     // halves per shared row: 144 B keeps ldmatrix rows on distinct banks
constexpr int kGradActBytes = kGradStage * kActStride * 2;
constexpr int kGradMaskBytes = kGradStage * kGradCols;
constexpr int kGradSideBytes = kGradStage * 16 * 4;
constexpr int kGradStageBytes = kGradActBytes + kGradMaskBytes + kGradSideBytes;
constexpr int kGradHiLoBytes = 2 * 16 * kActStride * 2;
constexpr int kGradSmemBytes = kGradRing * kGradStageBytes + kGradHiLoBytes;
static_assert(4 * 16 * (kGradCols + 1) * 4 <= kGradRing * kGradStageBytes, "the final reduction reuses the ring");

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// 16 bytes global -> shared, or 16 zero bytes when `valid` is false (src must still be an address)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One column reduction. A launch carries up to two of them (dA and dB of one projection): column
// tiles [0, tiles_first) of the grid belong to the first, the rest to the second.
struct GradProblem {
  const __half* act;
  int64_t ldact;
  const uint8_t* mask;
  int64_t ld_mask;
  float keep_scale;
  const float* side;
  float scale;
  int64_t C;
  int64_t rows_per_cta;
  float* out;
  int64_t ld_j, ld_c;
};

__global__ void __launch_bounds__(kGradThreads, 4)
lora_grad_kernel(const GradProblem first, const GradProblem second, int tiles_first, int64_t M) {
  pdl_wait();
  pdl_launch_dependents();
  const bool is_first = static_cast<int>(blockIdx.x) < tiles_first;
  const GradProblem& pb = is_first ? first : second;
  const __half* __restrict__ act = pb.act;
  const int64_t ldact = pb.ldact;
  const uint8_t* __restrict__ mask = pb.mask;
  const int64_t ld_mask = pb.ld_mask;
  const float keep_scale = pb.keep_scale;
  const float* __restrict__ side = pb.side;
  const float scale = pb.scale;
  const int64_t C = pb.C, rows_per_cta = pb.rows_per_cta;
  float* __restrict__ out = pb.out;
  const int64_t ld_j = pb.ld_j, ld_c = pb.ld_c;
  if (static_cast<int64_t>(blockIdx.y) * rows_per_cta >= M) return;      // this reduction has fewer row ranges than the other
  extern __shared__ __align__(16) uint8_t g_smem[];
  const uint32_t ring = smem_u32(g_smem);
  __half (*s_hi)[kActStride] = reinterpret_cast<__half (*)[kActStride]>(g_smem + kGradRing * kGradStageBytes);
  __half (*s_lo)[kActStride] = s_hi + 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t c0 = static_cast<int64_t>(is_first ? blockIdx.x : blockIdx.x - tiles_first) * kGradCols;
  const int64_t r_begin = static_cast<int64_t>(blockIdx.y) * rows_per_cta;
  const int64_t r_end = (r_begin + rows_per_cta < M) ? r_begin + rows_per_cta : M;
  float acc[8][4];
#pragma unroll
  for (int n = 0; n < 8; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;

  // one stage of loads: 64 rows x (128 B of act, 64 B of mask, 64 B of side), one commit group
  auto issue = [&](int64_t r0, int slot) {
    const uint32_t base = ring + slot * kGradStageBytes;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = threadIdx.x + i * kGradThreads;
      const int r = idx >> 3, ch = idx & 7;
      const int64_t row = r0 + r, col = c0 + ch * 8;
      const bool v = row < r_end && col < C;
      cp_async16(base + r * (kActStride * 2) + ch * 16, v ? act + row * ldact + col : act, v);
    }
    if (mask) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int idx = threadIdx.x + i * kGradThreads;
        const int r = idx >> 2, ch = idx & 3;
        const int64_t row = r0 + r, col = c0 + ch * 16;
        const bool v = row < r_end && col < C;
        cp_async16(base + kGradActBytes + r * kGradCols + ch * 16, v ? mask + row * ld_mask + col : mask, v);
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = threadIdx.x + i * kGradThreads;
      const int r = idx >> 2, ch = idx & 3;
      const bool v = r0 + r < r_end;
      cp_async16(base + kGradActBytes + kGradMaskBytes + r * 64 + ch * 16, v ? side + (r0 + r) * 16 + ch * 4 : side, v);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int s0 = 0; s0 < kGradRing - 1; ++s0) issue(r_begin + s0 * kGradStage, s0);
  int it = 0;
  for (int64_t r0 = r_begin; r0 < r_end; r0 += kGradStage, ++it) {
    issue(r0 + (kGradRing - 1) * kGradStage, (it + kGradRing - 1) % kGradRing);   // past the range: empty, zero-filled
    cp_async_wait<kGradRing - 1>();
    __syncthreads();
    uint8_t* st = g_smem + (it % kGradRing) * kGradStageBytes;
    if (mask) {
      // dropout in place: 64 rows x 8 chunks of 8 columns over 128 threads
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int idx = threadIdx.x + i * kGradThreads;
        const int r = idx >> 3, ch = idx & 7;
        uint4* ap = reinterpret_cast<uint4*>(st + r * (kActStride * 2) + ch * 16);
        const uint2 m = *reinterpret_cast<const uint2*>(st + kGradActBytes + r * kGradCols + ch * 8);
        *ap = drop8(*ap, m, keep_scale);
      }
    }
    // side transposed, split into hi + lo: 64 rows x 16 = 1024 values over 128 threads
    const float* sd = reinterpret_cast<const float*>(st + kGradActBytes + kGradMaskBytes);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = threadIdx.x + i * kGradThreads;
      const int r = idx >> 4, j = idx & 15;
      const float v = sd[idx];
      const __half hi = __float2half_rn(v);
      s_hi[j][r] = hi;
      s_lo[j][r] = __float2half_rn(v - __half2float(hi));
    }
    __syncthreads();
    const int kb = warp * 16;      // this warp's 16 rows of the stage
    const uint32_t ah0 = *reinterpret_cast<const uint32_t*>(&s_hi[g][kb + 2 * t]);
    const uint32_t ah1 = *reinterpret_cast<const uint32_t*>(&s_hi[g + 8][kb + 2 * t]);
    const uint32_t ah2 = *reinterpret_cast<const uint32_t*>(&s_hi[g][kb + 2 * t + 8]);
    const uint32_t ah3 = *reinterpret_cast<const uint32_t*>(&s_hi[g + 8][kb + 2 * t + 8]);
    const uint32_t al0 = *reinterpret_cast<const uint32_t*>(&s_lo[g][kb + 2 * t]);
    const uint32_t al1 = *reinterpret_cast<const uint32_t*>(&s_lo[g + 8][kb + 2 * t]);
    const uint32_t al2 = *reinterpret_cast<const uint32_t*>(&s_lo[g][kb + 2 * t + 8]);
    const uint32_t al3 = *reinterpret_cast<const uint32_t*>(&s_lo[g + 8][kb + 2 * t + 8]);
    const uint32_t act_base = ring + (it % kGradRing) * kGradStageBytes;
#pragma unroll
    for (int np = 0; np < 4; ++np) {     // pairs of 8-column tiles
      // matrices: (k 0-7, n 0-7), (k 8-15, n 0-7), (k 0-7, n 8-15), (k 8-15, n 8-15) of this pair
      const int mrow = kb + ((lane >> 3) & 1) * 8 + (lane & 7);
      const int mcol = np * 16 + (lane >> 4) * 8;
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(act_base + mrow * (kActStride * 2) + mcol * 2, b0, b1, b2, b3);
      mma16816(acc[2 * np], ah0, ah1, ah2, ah3, b0, b1);
      mma16816(acc[2 * np], al0, al1, al2, al3, b0, b1);
      mma16816(acc[2 * np + 1], ah0, ah1, ah2, ah3, b2, b3);
      mma16816(acc[2 * np + 1], al0, al1, al2, al3, b2, b3);
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();
  // combine the four warps' row slices (the ring is free now), then add into the output
  float (*s_red)[16][kGradCols + 1] = reinterpret_cast<float (*)[16][kGradCols + 1]>(g_smem);
#pragma unroll
  for (int n = 0; n < 8; ++n) {
    s_red[warp][g][n * 8 + 2 * t] = acc[n][0];
    s_red[warp][g][n * 8 + 2 * t + 1] = acc[n][1];
    s_red[warp][g + 8][n * 8 + 2 * t] = acc[n][2];
    s_red[warp][g + 8][n * 8 + 2 * t + 1] = acc[n][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 16 * kGradCols; idx += kGradThreads) {
    // dA (ld_c == 1): consecutive threads take consecutive columns; dB (ld_j == 1): consecutive ranks
    const int j = (ld_c == 1) ? idx / kGradCols : idx % 16;
    const int c = (ld_c == 1) ? idx % kGradCols : idx / 16;
    if (c0 + c < C) {
      const float v = s_red[0][j][c] + s_red[1][j][c] + s_red[2][j][c] + s_red[3][j][c];
      atomicAdd(out + j * ld_j + (c0 + c) * ld_c, v * scale);
    }
  }
}

struct GradPlan {
  int64_t col_tiles, msplit, rows_per;
};
static GradPlan grad_plan(int64_t M, int64_t C, int64_t sms, int64_t other_tiles) {
  GradPlan g;
  g.col_tiles = (C + kGradCols - 1) / kGradCols;
  const int64_t stages = (M + kGradStage - 1) / kGradStage;
  // three CTAs per SM (shared memory): one wave over both reductions of the launch, no tail
  int64_t msplit = (3 * sms + (g.col_tiles + other_tiles) - 1) / (g.col_tiles + other_tiles);
  if (msplit > stages) msplit = stages;
  if (msplit < 1) msplit = 1;
  g.rows_per = (stages + msplit - 1) / msplit * kGradStage;
  g.msplit = (M + g.rows_per - 1) / g.rows_per;
  return g;
}

// dA = u^T . drop(x) (u carries the LoRA scale, reference solution/fast_qwen.py:1370-1371) and / or
// dB = scale * dy^T . t (fast_qwen.py:1369), in one launch.
static int lora_grads_launch(const void* dy, int64_t lddy, const void* x, int64_t ldx, const uint8_t* mask, int64_t ld_mask,
                             float keep_scale, const void* t32, const void* u32, float scale, int64_t M, int64_t N, int64_t K,
                             void* dA, void* dB, cudaStream_t stream) {
  int dev = 0, sms = 148;
  NF4LL_CUDA(cudaGetDevice(&dev));
  NF4LL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  NF4LL_CUDA(cudaFuncSetAttribute(lora_grad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGradSmemBytes));
  const int64_t tiles_a = dA ? (K + kGradCols - 1) / kGradCols : 0;
  const int64_t tiles_b = dB ? (N + kGradCols - 1) / kGradCols : 0;
  GradProblem pa{}, pbb{};
  int64_t ms = 1;
  if (dA) {
    const GradPlan g = grad_plan(M, K, sms, tiles_b);
    pa = GradProblem{static_cast<const __half*>(x), ldx, mask, ld_mask, keep_scale, static_cast<const float*>(u32), 1.0f, K,
                     g.rows_per, static_cast<float*>(dA), K, 1};
    ms = g.msplit;
  }
  if (dB) {
    const GradPlan g = grad_plan(M, N, sms, tiles_a);
    pbb = GradProblem{static_cast<const __half*>(dy), lddy, nullptr, 0, 1.0f, static_cast<const float*>(t32), scale, N,
                      g.rows_per, static_cast<float*>(dB), 1, 16};
    if (g.msplit > ms) ms = g.msplit;
  }
  dim3 grid(static_cast<unsigned>(tiles_a + tiles_b), static_cast<unsigned>(ms));
  PdlLaunch lc(grid, dim3(kGradThreads), kGradSmemBytes, stream);
  NF4LL_CUDA(cudaLaunchKernelEx(&lc.cfg, lora_grad_kernel, pa, pbb, static_cast<int>(tiles_a), M));
  return NF4LL_OK;
}

}  // namespace nf4ll

extern "C" int nf4ll_lora_down(const void* x, int64_t ldx, const uint8_t* mask, int64_t ld_mask, float keep_scale,
                               const void* A, float scale, int32_t r, int64_t M, int64_t K, void* t32, void* t16,
                               void* stream) {
  using namespace nf4ll;
  if (r != 16) { set_detail("nf4ll_lora_down: rank %d", r); return NF4LL_ERR_RANK; }
  if (!x || !A) { set_detail("nf4ll_lora_down: null pointer"); return NF4LL_ERR_NULL; }
  if (M < 0 || K <= 0 || K % 8) { set_detail("nf4ll_lora_down: M=%lld K=%lld", (long long)M, (long long)K); return NF4LL_ERR_SHAPE; }
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(A) & 15) || ldx % 8 ||
      (mask && ((reinterpret_cast<uintptr_t>(mask) & 15) || ld_mask % 16))) {
    set_detail("nf4ll_lora_down: x/A 16-byte aligned, ldx multiple of 8, mask 16-byte aligned with ld_mask multiple of 16");
    return NF4LL_ERR_ALIGN;
  }
  if (int rc = require_sm100()) return rc;
  if (!t32) { set_detail("nf4ll_lora_down: t32 is required (t16 is optional)"); return NF4LL_ERR_NULL; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (int rc = lora_down_launch(x, ldx, mask, ld_mask, keep_scale, A, 1.0f, M, K, t32, nullptr, 0, st)) return rc;
  if (t16 && M > 0) {
    const int64_t n = M * 16;
    count_launch();
    scale_to_half_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(static_cast<const float*>(t32),
                                                                              static_cast<__half*>(t16), scale, n);
    NF4LL_CUDA(cudaGetLastError());
  }
  return NF4LL_OK;
}

extern "C" int nf4ll_lora_grads(const void* dy, int64_t lddy, const void* x, int64_t ldx, const uint8_t* mask,
                                int64_t ld_mask, float keep_scale, const void* t32, const void* u32, float scale,
                                int32_t r, int64_t M, int64_t N, int64_t K, void* dA, void* dB, int32_t accumulate,
                                void* stream_v) {
  using namespace nf4ll;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (r != 16) { set_detail("nf4ll_lora_grads: rank %d", r); return NF4LL_ERR_RANK; }
  if (M < 0 || N <= 0 || K <= 0 || (N % 8) || (K % 8)) {
    set_detail("nf4ll_lora_grads: M=%lld N=%lld K=%lld (N, K multiples of 8)", (long long)M, (long long)N, (long long)K);
    return NF4LL_ERR_SHAPE;
  }
  if (dA && (!x || !u32)) { set_detail("nf4ll_lora_grads: dA needs x and u"); return NF4LL_ERR_NULL; }
  if (dB && (!dy || !t32)) { set_detail("nf4ll_lora_grads: dB needs dy and t"); return NF4LL_ERR_NULL; }
  if ((dA && ((reinterpret_cast<uintptr_t>(x) & 15) || (ldx % 8))) || (dB && ((reinterpret_cast<uintptr_t>(dy) & 15) || (lddy % 8))) ||
      (dA && mask && ((reinterpret_cast<uintptr_t>(mask) & 15) || ld_mask % 16))) {
    set_detail("nf4ll_lora_grads: activations 16-byte aligned with leading dimensions multiples of 8; mask 16-byte aligned, ld_mask multiple of 16");
    return NF4LL_ERR_ALIGN;
  }
  if (int rc = require_sm100()) return rc;
  if (dA && !accumulate) NF4LL_CUDA(cudaMemsetAsync(dA, 0, sizeof(float) * 16 * K, stream));
  if (dB && !accumulate) NF4LL_CUDA(cudaMemsetAsync(dB, 0, sizeof(float) * 16 * N, stream));
  if (M > 0 && (dA || dB))
    if (int rc = lora_grads_launch(dy, lddy, x, ldx, mask, ld_mask, keep_scale, t32, u32, scale, M, N, K, dA, dB, stream)) return rc;
  return NF4LL_OK;
}
