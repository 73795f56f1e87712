// SiLU-gated product between the up and down projections, forward and backward, fp32 math on fp16
// tensors: the step that sits between two calls of the fused linear in an MLP block.
// Same arithmetic as the reference's gated_silu_fwd/bwd kernels (solution/k_mlp.py:21-47):
//   h      = fp16( g / (1 + exp(-g)) * u )
//   d up   = dh * silu(g),   d gate = (dh * u) * sig * (1 + g * (1 - sig))
// Bandwidth-bound: 8 fp16 per thread per 128-bit access, grid-stride over [M, I].
#include "nf4ll_common.cuh"

namespace nf4ll {

// Both kernels are one pass at memory speed: a thread takes two 16-byte chunks per trip, all loads
// of the trip issued before the arithmetic, so that every SM keeps enough bytes in flight.
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __half* __restrict__ g, int64_t ldg, const __half* __restrict__ u, int64_t ldu,
                  __half* __restrict__ h, int64_t ldh, int64_t M, int64_t chunks_per_row) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t total = M * chunks_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += 2 * stride) {
    const int64_t i2 = i + stride;
    const bool two = i2 < total;
    const int64_t row = i / chunks_per_row, col = (i - row * chunks_per_row) * 8;
    const int64_t row2 = two ? i2 / chunks_per_row : row, col2 = two ? (i2 - row2 * chunks_per_row) * 8 : col;
    const uint4 ga = __ldcs(reinterpret_cast<const uint4*>(g + row * ldg + col));
    const uint4 ua = __ldcs(reinterpret_cast<const uint4*>(u + row * ldu + col));
    const uint4 gb = __ldcs(reinterpret_cast<const uint4*>(g + row2 * ldg + col2));
    const uint4 ub = __ldcs(reinterpret_cast<const uint4*>(u + row2 * ldu + col2));
    *reinterpret_cast<uint4*>(h + row * ldh + col) = swiglu_fwd8(ga, ua);
    if (two) *reinterpret_cast<uint4*>(h + row2 * ldh + col2) = swiglu_fwd8(gb, ub);
  }
}

// dg / du may alias g / u (in-place, as the reference overwrites [gate | up]): a chunk is read in
// full before it is written, by the same thread.
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __half* g, int64_t ldg, const __half* u, int64_t ldu, const __half* __restrict__ dh, int64_t lddh,
                  __half* dg, int64_t lddg, __half* du, int64_t lddu, int64_t M, int64_t chunks_per_row) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t total = M * chunks_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += 2 * stride) {
    const int64_t i2 = i + stride;
    const bool two = i2 < total;
    const int64_t row = i / chunks_per_row, col = (i - row * chunks_per_row) * 8;
    const int64_t row2 = two ? i2 / chunks_per_row : row, col2 = two ? (i2 - row2 * chunks_per_row) * 8 : col;
    const uint4 ga = *reinterpret_cast<const uint4*>(g + row * ldg + col);
    const uint4 ua = *reinterpret_cast<const uint4*>(u + row * ldu + col);
    const uint4 da = __ldcs(reinterpret_cast<const uint4*>(dh + row * lddh + col));
    const uint4 gb = *reinterpret_cast<const uint4*>(g + row2 * ldg + col2);
    const uint4 ub = *reinterpret_cast<const uint4*>(u + row2 * ldu + col2);
    const uint4 db = __ldcs(reinterpret_cast<const uint4*>(dh + row2 * lddh + col2));
    uint4 og, ou;
    swiglu_bwd8(ga, ua, da, og, ou);
    *reinterpret_cast<uint4*>(dg + row * lddg + col) = og;
    *reinterpret_cast<uint4*>(du + row * lddu + col) = ou;
    if (two) {
      swiglu_bwd8(gb, ub, db, og, ou);
      *reinterpret_cast<uint4*>(dg + row2 * lddg + col2) = og;
      *reinterpret_cast<uint4*>(du + row2 * lddu + col2) = ou;
    }
  }
}

static int check_mat16(const void* p, int64_t ld, int64_t cols, const char* who, const char* what) {
  if (!p) { set_detail("%s: %s is null", who, what); return NF4LL_ERR_NULL; }
  if ((reinterpret_cast<uintptr_t>(p) & 15) || ld % 8 || ld < cols) {
    set_detail("%s: %s must be 16-byte aligned with a leading dimension multiple of 8 and >= the row length", who, what);
    return NF4LL_ERR_ALIGN;
  }
  return NF4LL_OK;
}

static int grid_for(int64_t total, unsigned* blocks) {
  int dev = 0, sms = 148;
  NF4LL_CUDA(cudaGetDevice(&dev));
  NF4LL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  int64_t b = (total + 511) / 512;              // two chunks per thread and trip
  const int64_t cap = static_cast<int64_t>(sms) * 8;
  *blocks = static_cast<unsigned>(b < cap ? b : cap);
  return NF4LL_OK;
}

}  // namespace nf4ll

extern "C" int nf4ll_swiglu_forward(const void* g, int64_t ldg, const void* u, int64_t ldu, void* h, int64_t ldh, int64_t M,
                                    int64_t I, void* stream) {
  using namespace nf4ll;
  if (M < 0 || I <= 0 || I % 8) { set_detail("nf4ll_swiglu_forward: M=%lld I=%lld", (long long)M, (long long)I); return NF4LL_ERR_SHAPE; }
  if (M == 0) return NF4LL_OK;
  if (int rc = check_mat16(g, ldg, I, "nf4ll_swiglu_forward", "g")) return rc;
  if (int rc = check_mat16(u, ldu, I, "nf4ll_swiglu_forward", "u")) return rc;
  if (int rc = check_mat16(h, ldh, I, "nf4ll_swiglu_forward", "h")) return rc;
  if (int rc = require_sm100()) return rc;
  unsigned blocks = 1;
  if (int rc = grid_for(M * (I / 8), &blocks)) return rc;
  PdlLaunch lc(dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream));
  NF4LL_CUDA(cudaLaunchKernelEx(&lc.cfg, swiglu_fwd_kernel, static_cast<const __half*>(g), ldg, static_cast<const __half*>(u), ldu,
                                static_cast<__half*>(h), ldh, M, I / 8));
  return NF4LL_OK;
}

extern "C" int nf4ll_swiglu_backward(const void* g, int64_t ldg, const void* u, int64_t ldu, const void* dh, int64_t lddh,
                                     void* dg, int64_t lddg, void* du, int64_t lddu, int64_t M, int64_t I, void* stream) {
  using namespace nf4ll;
  if (M < 0 || I <= 0 || I % 8) { set_detail("nf4ll_swiglu_backward: M=%lld I=%lld", (long long)M, (long long)I); return NF4LL_ERR_SHAPE; }
  if (M == 0) return NF4LL_OK;
  if (int rc = check_mat16(g, ldg, I, "nf4ll_swiglu_backward", "g")) return rc;
  if (int rc = check_mat16(u, ldu, I, "nf4ll_swiglu_backward", "u")) return rc;
  if (int rc = check_mat16(dh, lddh, I, "nf4ll_swiglu_backward", "dh")) return rc;
  if (int rc = check_mat16(dg, lddg, I, "nf4ll_swiglu_backward", "dg")) return rc;
  if (int rc = check_mat16(du, lddu, I, "nf4ll_swiglu_backward", "du")) return rc;
  if (int rc = require_sm100()) return rc;
  unsigned blocks = 1;
  if (int rc = grid_for(M * (I / 8), &blocks)) return rc;
  PdlLaunch lc(dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream));
  NF4LL_CUDA(cudaLaunchKernelEx(&lc.cfg, swiglu_bwd_kernel, static_cast<const __half*>(g), ldg, static_cast<const __half*>(u), ldu,
                                static_cast<const __half*>(dh), lddh, static_cast<__half*>(dg), lddg, static_cast<__half*>(du), lddu,
                                M, I / 8));
  return NF4LL_OK;
}
