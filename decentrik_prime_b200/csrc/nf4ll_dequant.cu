// Standalone NF4 -> fp16 dequantisation (the bit-exactness probe, and the launcher behind the
// k_nf4-compatible dequant_layer / dequant_range for callers that still want an fp16 workspace).
// Replaces the reference's nf4_layer_dequant_kernel (solution/k_nf4.py:40-57).
//
// Memory-bound: 0.516 B read + 2 B written per weight. One thread decodes half a quantisation
// block per step: one 128-bit load of 32 codes, coalesced across the warp, and four 128-bit
// stores. The 16 levels never touch memory: each thread builds the block's 16 fp16 products in
// registers and looks codes up with byte permutes.
#include "nf4ll_common.cuh"

namespace nf4ll {

constexpr int kDequantThreads = 256;

__global__ void __launch_bounds__(kDequantThreads)
dequant_kernel(const uint4* __restrict__ nib, const uint8_t* __restrict__ qabs,
               const float* __restrict__ scale2, const float* __restrict__ offset2,
               const float* __restrict__ code2, int64_t n_half_blocks, uint4* __restrict__ out) {
  __shared__ float s_code2[256];
  s_code2[threadIdx.x] = code2[threadIdx.x];
  __syncthreads();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kDequantThreads;
  for (int64_t h = static_cast<int64_t>(blockIdx.x) * kDequantThreads + threadIdx.x; h < n_half_blocks; h += stride) {
    const int64_t qb = h >> 1;
    const uint4 codes = __ldg(nib + h);
    const float absmax = block_absmax(s_code2[__ldg(qabs + qb)], __ldg(scale2 + (qb >> 8)), __ldg(offset2 + (qb >> 8)));
    const BlockTable t = make_block_table(absmax);
    uint4* dst = out + h * 4;
    dst[0] = decode_word(t, codes.x);
    dst[1] = decode_word(t, codes.y);
    dst[2] = decode_word(t, codes.z);
    dst[3] = decode_word(t, codes.w);
  }
}

}  // namespace nf4ll

extern "C" int nf4ll_dequant(const uint8_t* nib, const uint8_t* qabs, const float* scale2, const float* offset2,
                             const float* code2, int64_t n_qblocks, void* out_f16, void* stream) {
  using namespace nf4ll;
  if (n_qblocks == 0) return NF4LL_OK;
  if (!nib || !qabs || !scale2 || !offset2 || !code2 || !out_f16) {
    set_detail("nf4ll_dequant: null pointer");
    return NF4LL_ERR_NULL;
  }
  if (n_qblocks < 0) {
    set_detail("nf4ll_dequant: n_qblocks=%lld", static_cast<long long>(n_qblocks));
    return NF4LL_ERR_SHAPE;
  }
  if ((reinterpret_cast<uintptr_t>(nib) & 15) || (reinterpret_cast<uintptr_t>(out_f16) & 15) ||
      (reinterpret_cast<uintptr_t>(scale2) & 3) || (reinterpret_cast<uintptr_t>(offset2) & 3)) {
    set_detail("nf4ll_dequant: nib/out must be 16-byte aligned, scale2/offset2 4-byte aligned");
    return NF4LL_ERR_ALIGN;
  }
  if (int rc = require_sm100()) return rc;
  const int64_t n_half = n_qblocks * 2;
  int dev = 0, sms = 148;
  NF4LL_CUDA(cudaGetDevice(&dev));
  NF4LL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  int64_t blocks = (n_half + kDequantThreads - 1) / kDequantThreads;
  const int64_t cap = static_cast<int64_t>(sms) * 8;   // whole waves of 8 resident CTAs per SM
  if (blocks > cap) blocks = cap;
  count_launch();
  dequant_kernel<<<static_cast<unsigned>(blocks), kDequantThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(nib), qabs, scale2, offset2, code2, n_half, reinterpret_cast<uint4*>(out_f16));
  NF4LL_CUDA(cudaGetLastError());
  return NF4LL_OK;
}
