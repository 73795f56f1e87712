// The skinny (rank-16) LoRA products around the fused linear:
//   lora_down   t[M,16]  = drop(x)[M,K] . A^T            (forward: T;  backward: U = dy . B)
//   lora_grads  dA[16,K] (+)= u^T . drop(x),  dB[N,16] (+)= scale * dy^T . t
// Replaces solution/fast_qwen.py:943-944 and 1369-1374 of the reference. All accumulation is fp32,
// and t / u are kept in fp32 between the passes: the reference rounds them (and dA/dB) to fp16,
// which costs up to 0.08 absolute error on gradients of magnitude ~100.
//
// These are bandwidth-bound streaming passes over x / dy (16 multiply-adds per element read).
#include "nf4ll_common.cuh"

namespace nf4ll {

// drop(x) for 8 packed fp16 values: fp16(x * keep_scale) where the mask byte is non-zero, else 0
// (reference solution/k_norm.py:49-53: scale in fp32, then one rounding to fp16).
__device__ __forceinline__ void load_dropped8(const __half* xp, const uint8_t* mp, float keep_scale, float (&f)[8]) {
  const uint4 raw = __ldg(reinterpret_cast<const uint4*>(xp));
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 v = __half22float2(h[j]);
    f[2 * j] = v.x;
    f[2 * j + 1] = v.y;
  }
  if (mp) {
    const uint2 m = __ldg(reinterpret_cast<const uint2*>(mp));
    const uint32_t mw[2] = {m.x, m.y};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool keep = ((mw[j >> 2] >> ((j & 3) * 8)) & 0xffu) != 0;
      f[j] = keep ? __half2float(__float2half_rn(f[j] * keep_scale)) : 0.0f;
    }
  }
}

constexpr int kDownWarps = 8;

// One warp per row. A_KMAJOR: A is [16, K] (lora_A); otherwise A is [K, 16] (lora_B read as dy's
// right factor). Lane l takes columns 8*(32*step + l) .. +7.
template <bool A_KMAJOR>
__global__ void __launch_bounds__(kDownWarps * 32)
lora_down_kernel(const __half* __restrict__ x, int64_t ldx, const uint8_t* __restrict__ mask, int64_t ld_mask,
                 float keep_scale, const __half* __restrict__ A, float scale, int64_t M, int64_t K,
                 float* __restrict__ t32, __half* __restrict__ t16) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kDownWarps + (threadIdx.x >> 5);
  if (row >= M) return;
  float acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = 0.f;
  const __half* xr = x + row * ldx;
  const uint8_t* mr = mask ? mask + row * ld_mask : nullptr;
  for (int64_t k = lane * 8; k < K; k += 256) {
    float f[8];
    load_dropped8(xr + k, mr ? mr + k : nullptr, keep_scale, f);
    if (A_KMAJOR) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(A + j * K + k));
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 a = __half22float2(h[i]);
          acc[j] = fmaf(f[2 * i], a.x, acc[j]);
          acc[j] = fmaf(f[2 * i + 1], a.y, acc[j]);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4* ap = reinterpret_cast<const uint4*>(A + (k + i) * 16);
        const uint4 r0 = __ldg(ap), r1 = __ldg(ap + 1);
        const __half2* h0 = reinterpret_cast<const __half2*>(&r0);
        const __half2* h1 = reinterpret_cast<const __half2*>(&r1);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = __half22float2(h0[j]), b = __half22float2(h1[j]);
          acc[2 * j] = fmaf(f[i], a.x, acc[2 * j]);
          acc[2 * j + 1] = fmaf(f[i], a.y, acc[2 * j + 1]);
          acc[8 + 2 * j] = fmaf(f[i], b.x, acc[8 + 2 * j]);
          acc[8 + 2 * j + 1] = fmaf(f[i], b.y, acc[8 + 2 * j + 1]);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], off);
  }
  if (lane < 16) {
    float v = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) v = (lane == j) ? acc[j] : v;
    if (t32) t32[row * 16 + lane] = A_KMAJOR ? v : v * scale;   // T unscaled; U carries the scale
    if (t16) t16[row * 16 + lane] = __float2half_rn(v * scale);
  }
}

int lora_down_launch(const void* x, int64_t ldx, const uint8_t* mask, int64_t ld_mask, float keep_scale, const void* A,
                     int a_kmajor, float scale, int64_t M, int64_t K, void* t32, void* t16, cudaStream_t stream) {
  if (M == 0) return NF4LL_OK;
  const unsigned blocks = static_cast<unsigned>((M + kDownWarps - 1) / kDownWarps);
  if (a_kmajor) {
    lora_down_kernel<true><<<blocks, kDownWarps * 32, 0, stream>>>(
        static_cast<const __half*>(x), ldx, mask, ld_mask, keep_scale, static_cast<const __half*>(A), scale, M, K,
        static_cast<float*>(t32), static_cast<__half*>(t16));
  } else {
    lora_down_kernel<false><<<blocks, kDownWarps * 32, 0, stream>>>(
        static_cast<const __half*>(x), ldx, mask, ld_mask, keep_scale, static_cast<const __half*>(A), scale, M, K,
        static_cast<float*>(t32), static_cast<__half*>(t16));
  }
  NF4LL_CUDA(cudaGetLastError());
  return NF4LL_OK;
}

// out[j, col] (+)= scale * sum_m side[m, j] * drop(act)[m, col]   for j < 16
// One CTA: 512 columns (2 per thread) x a chunk of kGradRows rows; partial sums are added to the
// output with fp32 atomics. out index = j * ld_j + col * ld_col, which covers dA[16,K] (ld_j = K,
// ld_col = 1) and dB[N,16] (ld_j = 1, ld_col = 16).
constexpr int kGradThreads = 256;
constexpr int kGradRows = 64;

__global__ void __launch_bounds__(kGradThreads)
lora_grad_kernel(const __half* __restrict__ act, int64_t ldact, const uint8_t* __restrict__ mask, int64_t ld_mask,
                 float keep_scale, const float* __restrict__ side, float scale, int64_t M, int64_t C,
                 float* __restrict__ out, int64_t ld_j, int64_t ld_col) {
  __shared__ float s_side[kGradRows][16];
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * kGradRows;
  const int rows = static_cast<int>(M - r0 < kGradRows ? M - r0 : kGradRows);
  for (int i = threadIdx.x; i < rows * 16; i += kGradThreads) s_side[i >> 4][i & 15] = side[r0 * 16 + i];
  __syncthreads();
  const int64_t col = (static_cast<int64_t>(blockIdx.x) * kGradThreads + threadIdx.x) * 2;
  if (col >= C) return;
  float a0[16], a1[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) a0[j] = a1[j] = 0.f;
  for (int r = 0; r < rows; ++r) {
    const __half2 h = *reinterpret_cast<const __half2*>(act + (r0 + r) * ldact + col);
    float2 v = __half22float2(h);
    if (mask) {
      const uint8_t* mp = mask + (r0 + r) * ld_mask + col;
      v.x = mp[0] ? __half2float(__float2half_rn(v.x * keep_scale)) : 0.f;
      v.y = mp[1] ? __half2float(__float2half_rn(v.y * keep_scale)) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float sj = s_side[r][j];
      a0[j] = fmaf(sj, v.x, a0[j]);
      a1[j] = fmaf(sj, v.y, a1[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    atomicAdd(out + j * ld_j + col * ld_col, a0[j] * scale);
    atomicAdd(out + j * ld_j + (col + 1) * ld_col, a1[j] * scale);
  }
}

}  // namespace nf4ll

extern "C" int nf4ll_lora_down(const void* x, int64_t ldx, const uint8_t* mask, int64_t ld_mask, float keep_scale,
                               const void* A, int32_t a_kmajor, float scale, int32_t r, int64_t M, int64_t K, void* t32,
                               void* t16, void* stream) {
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
  return lora_down_launch(x, ldx, mask, ld_mask, keep_scale, A, a_kmajor, scale, M, K, t32, t16, static_cast<cudaStream_t>(stream));
}

extern "C" int nf4ll_lora_grads(const void* dy, int64_t lddy, const void* x, int64_t ldx, const uint8_t* mask,
                                int64_t ld_mask, float keep_scale, const void* t32, const void* u32, float scale,
                                int32_t r, int64_t M, int64_t N, int64_t K, void* dA, void* dB, int32_t accumulate,
                                void* stream_v) {
  using namespace nf4ll;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (r != 16) { set_detail("nf4ll_lora_grads: rank %d", r); return NF4LL_ERR_RANK; }
  if (M < 0 || N <= 0 || K <= 0 || (N & 1) || (K & 1)) {
    set_detail("nf4ll_lora_grads: M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
    return NF4LL_ERR_SHAPE;
  }
  if (dA && (!x || !u32)) { set_detail("nf4ll_lora_grads: dA needs x and u"); return NF4LL_ERR_NULL; }
  if (dB && (!dy || !t32)) { set_detail("nf4ll_lora_grads: dB needs dy and t"); return NF4LL_ERR_NULL; }
  if ((dA && ((reinterpret_cast<uintptr_t>(x) & 3) || (ldx & 1))) || (dB && ((reinterpret_cast<uintptr_t>(dy) & 3) || (lddy & 1)))) {
    set_detail("nf4ll_lora_grads: activations must be 4-byte aligned with even leading dimensions");
    return NF4LL_ERR_ALIGN;
  }
  if (int rc = require_sm100()) return rc;
  const unsigned row_chunks = static_cast<unsigned>((M + kGradRows - 1) / kGradRows);
  if (dA) {
    if (!accumulate) NF4LL_CUDA(cudaMemsetAsync(dA, 0, sizeof(float) * 16 * K, stream));
    if (M > 0) {
      dim3 grid(static_cast<unsigned>((K / 2 + kGradThreads - 1) / kGradThreads), row_chunks);
      // dA = u^T . drop(x); u already carries the LoRA scale (reference solution/fast_qwen.py:1370-1371)
      lora_grad_kernel<<<grid, kGradThreads, 0, stream>>>(static_cast<const __half*>(x), ldx, mask, ld_mask, keep_scale,
                                                          static_cast<const float*>(u32), 1.0f, M, K,
                                                          static_cast<float*>(dA), K, 1);
      NF4LL_CUDA(cudaGetLastError());
    }
  }
  if (dB) {
    if (!accumulate) NF4LL_CUDA(cudaMemsetAsync(dB, 0, sizeof(float) * 16 * N, stream));
    if (M > 0) {
      dim3 grid(static_cast<unsigned>((N / 2 + kGradThreads - 1) / kGradThreads), row_chunks);
      // dB = scale * dy^T . t (reference solution/fast_qwen.py:1369)
      lora_grad_kernel<<<grid, kGradThreads, 0, stream>>>(static_cast<const __half*>(dy), lddy, nullptr, 0, 1.0f,
                                                          static_cast<const float*>(t32), scale, M, N,
                                                          static_cast<float*>(dB), 1, 16);
      NF4LL_CUDA(cudaGetLastError());
    }
  }
  return NF4LL_OK;
}
