// Which mechanism streams a row-major byte matrix (27648 rows x 2560 B) from DRAM into shared memory fastest?
// Built and run by tests/micro/run.py.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <vector>
#include <algorithm>

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e), __FILE__, __LINE__); exit(1); } } while (0)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 22); ++i) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) { asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory"); }

// ------------------------------------------------------------------ TMA boxes of ROWS x 128 B, ST stages, one CTA per SM (or more)
// mode 0: tiled 2D boxes; mode 1: the matrix taken as pre-tiled (contiguous ROWS*128-byte blocks) and fetched with 1D bulk copies
template <int ST, int ROWS>
__global__ void __launch_bounds__(64) k_tma(const __grid_constant__ CUtensorMap tm, const uint8_t* src, int n_tiles, int n_groups, int mode, int* err) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) uint64_t full[ST], empty[ST];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~uintptr_t(1023));
  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; ++s) { mbar_init(smem_u32(full + s), 1); mbar_init(smem_u32(empty + s), 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int total = n_tiles * n_groups;
  if (threadIdx.x == 0) {
    int j = 0;
    for (int i = blockIdx.x; i < total; i += gridDim.x, ++j) {
      const int s = j % ST;
      if (!mbar_wait(smem_u32(empty + s), ((j / ST) & 1) ^ 1)) { *err = 1; return; }
      mbar_expect_tx(smem_u32(full + s), ROWS * 128);
      if (mode == 0) tma_load_2d(smem_u32(base + s * ROWS * 128), &tm, smem_u32(full + s), (i / n_tiles) * 128, (i % n_tiles) * ROWS);
      else bulk_load_1d(smem_u32(base + s * ROWS * 128), src + static_cast<int64_t>(i) * ROWS * 128, ROWS * 128, smem_u32(full + s));
    }
  } else if (threadIdx.x == 32) {
    int j = 0;
    for (int i = blockIdx.x; i < total; i += gridDim.x, ++j) {
      const int s = j % ST;
      if (!mbar_wait(smem_u32(full + s), (j / ST) & 1)) { *err = 2; return; }
      mbar_arrive(smem_u32(empty + s));
    }
  }
}

// ------------------------------------------------------------------ cp.async: LW loader warps fill stages of 128 rows x 128 B
template <int ST, int LW>
__global__ void __launch_bounds__(32 * LW + 32) k_cpasync(const uint8_t* __restrict__ src, int n_tiles, int n_groups, int rowbytes, int* err) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) uint64_t full[ST], empty[ST];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~uintptr_t(1023));
  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; ++s) { mbar_init(smem_u32(full + s), 32 * LW); mbar_init(smem_u32(empty + s), 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int total = n_tiles * n_groups;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < LW) {
    constexpr int ITER = 1024 / (32 * LW);            // 16-byte chunks per lane per stage
    // lane's first chunk: row warp*(128/LW) + lane/8, chunk lane%8; each iteration moves four rows down
    const int r0 = warp * (128 / LW) + (lane >> 3), ch = lane & 7;
    const uint32_t d0 = smem_u32(base) + r0 * 128 + ((ch ^ (r0 & 7)) << 4);
    int j = 0;
    for (int i = blockIdx.x; i < total; i += gridDim.x, ++j) {
      const int s = j % ST;
      if (!mbar_wait(smem_u32(empty + s), ((j / ST) & 1) ^ 1)) { *err = 1; break; }
      const uint8_t* g = src + (static_cast<int64_t>(i % n_tiles) * 128 + r0) * rowbytes + (i / n_tiles) * 128 + ch * 16;
      const uint32_t d = d0 + s * 16384;
#pragma unroll
      for (int it = 0; it < ITER; ++it)               // (r0 + 4 it) & 7 flips bit 2 of the swizzle key every iteration
        cp_async16((d + it * 512) ^ ((it & 1) << 6), g + static_cast<int64_t>(it) * 4 * rowbytes);
      cp_async_arrive(smem_u32(full + s));
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (lane == 0) {
    int j = 0;
    for (int i = blockIdx.x; i < total; i += gridDim.x, ++j) {
      const int s = j % ST;
      if (!mbar_wait(smem_u32(full + s), (j / ST) & 1)) { *err = 2; return; }
      mbar_arrive(smem_u32(empty + s));
    }
  }
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                             const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int main() {
  const int N = 27648, K = 5120, COPIES = 4, rowbytes = K / 2;
  const size_t nib_bytes = (size_t)N * rowbytes;
  std::vector<uint8_t*> nibs(COPIES);
  std::vector<uint8_t> h(nib_bytes);
  for (size_t i = 0; i < nib_bytes; ++i) h[i] = (uint8_t)(rand() & 0xff);
  for (int c = 0; c < COPIES; ++c) { CK(cudaMalloc(&nibs[c], nib_bytes)); CK(cudaMemcpy(nibs[c], h.data(), nib_bytes, cudaMemcpyHostToDevice)); }
  int* err; CK(cudaMalloc(&err, 4)); CK(cudaMemset(err, 0, 4));
  void* fn = nullptr; cudaDriverEntryPointQueryResult qres;
  CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
  EncodeFn encode = reinterpret_cast<EncodeFn>(fn);
  auto make_map = [&](void* p, int rows, CUtensorMapL2promotion promo) {
    CUtensorMap m; cuuint64_t dims[2] = {(cuuint64_t)rowbytes, (cuuint64_t)N}; cuuint64_t strides[1] = {(cuuint64_t)rowbytes};
    cuuint32_t box[2] = {128, (cuuint32_t)rows}; cuuint32_t el[2] = {1, 1};
    CUresult r = encode(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, p, dims, strides, box, el, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { printf("encode failed %d\n", (int)r); exit(1); }
    return m;
  };
  cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
  auto time_it = [&](const char* name, auto launch) {
    for (int c = 0; c < COPIES; ++c) launch(c);
    CK(cudaDeviceSynchronize());
    std::vector<float> ts;
    for (int r = 0; r < 10; ++r) {
      CK(cudaEventRecord(e0));
      for (int c = 0; c < COPIES; ++c) launch(c);
      CK(cudaEventRecord(e1)); CK(cudaEventSynchronize(e1));
      float ms; CK(cudaEventElapsedTime(&ms, e0, e1)); ts.push_back(ms / COPIES);
    }
    std::sort(ts.begin(), ts.end());
    int herr; CK(cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost));
    printf("%-72s %8.2f us  %8.1f GB/s%s\n", name, ts[ts.size() / 2] * 1e3, (double)nib_bytes / (ts[ts.size() / 2] * 1e-3) / 1e9, herr ? "  WAIT EXPIRED" : "");
    fflush(stdout);
    if (herr) exit(2);
  };
  char name[160];
  const int n_groups = rowbytes / 128;
#define TMA_CASE(ST, ROWS, CTAS, MODE, PROMO, PNAME)                                                                     \
  {                                                                                                                      \
    std::vector<CUtensorMap> maps; for (int c = 0; c < COPIES; ++c) maps.push_back(make_map(nibs[c], ROWS, PROMO));     \
    const int smem = ST * ROWS * 128 + 1024;                                                                             \
    CK(cudaFuncSetAttribute(k_tma<ST, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));                       \
    snprintf(name, sizeof name, "%s, %d stages of %d rows x 128 B (%d KB in flight/CTA), %d CTAs/SM, promo %s", MODE ? "bulk 1D (pre-tiled)" : "TMA 2D boxes", ST, ROWS, ST * ROWS / 8, CTAS, PNAME); \
    time_it(name, [&](int c) { k_tma<ST, ROWS><<<148 * CTAS, 64, smem>>>(maps[c], nibs[c], N / ROWS, n_groups, MODE, err); });                                \
  }
  TMA_CASE(4, 128, 1, 0, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "128B")
  TMA_CASE(8, 128, 1, 0, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "128B")
  TMA_CASE(12, 128, 1, 0, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "128B")
  TMA_CASE(8, 128, 1, 0, CU_TENSOR_MAP_L2_PROMOTION_NONE, "none")
  TMA_CASE(8, 128, 1, 0, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "256B")
  TMA_CASE(4, 128, 2, 0, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "128B")
  TMA_CASE(6, 128, 2, 0, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "128B")
  TMA_CASE(3, 128, 4, 0, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "128B")
  TMA_CASE(6, 256, 1, 0, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "128B")
  TMA_CASE(16, 64, 1, 0, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "128B")
  TMA_CASE(8, 128, 1, 1, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "-")
  TMA_CASE(12, 128, 1, 1, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "-")
  TMA_CASE(6, 128, 2, 1, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "-")
  TMA_CASE(3, 128, 4, 1, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "-")
#define CPA_CASE(ST, LW, CTAS)                                                                                           \
  {                                                                                                                      \
    const int smem = ST * 16384 + 1024;                                                                                  \
    CK(cudaFuncSetAttribute(k_cpasync<ST, LW>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));                     \
    snprintf(name, sizeof name, "cp.async 16 B, %d loader warps, %d stages of 16 KB, %d CTAs/SM", LW, ST, CTAS);          \
    time_it(name, [&](int c) { k_cpasync<ST, LW><<<148 * CTAS, 32 * LW + 32, smem>>>(nibs[c], N / 128, n_groups, rowbytes, err); }); \
  }
  CPA_CASE(8, 1, 1)
  CPA_CASE(8, 2, 1)
  CPA_CASE(8, 4, 1)
  CPA_CASE(8, 8, 1)
  CPA_CASE(12, 4, 1)
  CPA_CASE(12, 8, 1)
  CPA_CASE(4, 4, 1)
  CPA_CASE(6, 4, 2)
  CPA_CASE(3, 4, 4)
  CK(cudaDeviceSynchronize());
  printf("done\n");
  return 0;
}
