// How long does one thread take to issue / execute small-N tcgen05.mma instructions (A from tensor memory or shared memory)?
// Built and run by tests/micro/run.py.
#include "../../decentrik_prime_b200/csrc/nf4ll_gemm_shared.cuh"
#include <cstdio>
#include <vector>
using namespace nf4ll;
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e), __FILE__, __LINE__); exit(1); } } while (0)
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
template <int N, int MODE>   // MODE 0: A from tensor memory, 1: A from shared memory
__global__ void __launch_bounds__(128) k_mma(int count, int per_commit, long long* out) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  for (int i = threadIdx.x; i < 48 * 1024 / 4; i += 128) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); mbar_fence_init(); }
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&slot), 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  const uint32_t tm = slot;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = make_idesc_f16(128, N, 0, 0);
    const uint64_t bdesc0 = make_smem_desc(smem_u32(smem), 16, 1024, kSwizzle128B);
    const uint64_t adesc0 = make_smem_desc(smem_u32(smem) + 32768, 16, 1024, kSwizzle128B);
    int ph = 0;
    long long t0 = clock64(), t_issue = 0;
    for (int i = 0; i < count; i += per_commit) {
      long long a = clock64();
#pragma unroll 4
      for (int j = 0; j < per_commit; ++j) {
        if (MODE == 0) mma_ts(tm, tm + 256 + ((i + j) % 12) * 8, bdesc0 + 2 * (j & 3), idesc, 1u);
        else tc_mma_f16(tm, adesc0 + 2 * (j & 3), bdesc0 + 2 * (j & 3), idesc, 1u);
      }
      tc_commit(smem_u32(&bar));
      t_issue += clock64() - a;
      while (!mbar_try_wait(smem_u32(&bar), ph)) {}
      ph ^= 1;
    }
    long long t1 = clock64();
    if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t_issue; }
  }
  tc_fence_before(); __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tm, 512); }
}
template <int N, int MODE> void run(int per_commit, long long* out, const char* nm) {
  const int count = 960;
  CK(cudaFuncSetAttribute(k_mma<N, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
  for (int r = 0; r < 2; ++r) k_mma<N, MODE><<<148, 128, 64 * 1024>>>(count, per_commit, out);
  CK(cudaDeviceSynchronize());
  long long h[2]; CK(cudaMemcpy(h, out, 16, cudaMemcpyDeviceToHost));
  printf("%s N=%3d  %2d MMAs per commit+wait: %7.1f clk per MMA in all, %7.1f clk per MMA to issue (+ commit)\n", nm, N, per_commit, (double)h[0] / count, (double)h[1] / count);
}

// NI issuing threads (lane 0 of warps 0..NI-1), each with its own accumulator columns and barrier: does the MMA rate add up?
template <int N, int NI>
__global__ void __launch_bounds__(128) k_mma_multi(int count, int per_commit, long long* out) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar[4];
  __shared__ uint32_t slot;
  for (int i = threadIdx.x; i < 48 * 1024 / 4; i += 128) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&bar[i]), 1); mbar_fence_init(); }
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&slot), 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  const uint32_t tm = slot;
  const int w = threadIdx.x >> 5;
  long long t0 = clock64();
  if ((threadIdx.x & 31) == 0 && w < NI) {
    constexpr uint32_t idesc = make_idesc_f16(128, N, 0, 0);
    const uint64_t bdesc0 = make_smem_desc(smem_u32(smem) + w * 4096, 16, 1024, kSwizzle128B);
    int ph = 0;
    for (int i = 0; i < count; i += per_commit) {
#pragma unroll 4
      for (int j = 0; j < per_commit; ++j)
        mma_ts(tm + w * 64, tm + 256 + w * 64 + ((i + j) % 8) * 8, bdesc0 + 2 * (j & 3), idesc, 1u);
      tc_commit(smem_u32(&bar[w]));
      while (!mbar_try_wait(smem_u32(&bar[w]), ph)) {}
      ph ^= 1;
    }
  }
  __syncthreads();
  long long t1 = clock64();
  if (blockIdx.x == 0 && threadIdx.x == 0) out[0] = t1 - t0;
  tc_fence_before(); __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tm, 512); }
}
template <int N, int NI> void run_multi(int per_commit, long long* out) {
  const int count = 960;
  CK(cudaFuncSetAttribute(k_mma_multi<N, NI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
  for (int r = 0; r < 2; ++r) k_mma_multi<N, NI><<<148, 128, 64 * 1024>>>(count, per_commit, out);
  CK(cudaDeviceSynchronize());
  long long h[2]; CK(cudaMemcpy(h, out, 16, cudaMemcpyDeviceToHost));
  printf("A in tensor memory N=%3d, %d issuing threads x %d MMAs, %2d per commit: %7.1f clk per MMA per thread, %7.1f clk per MMA overall\n", N, NI, count, per_commit, (double)h[0] / count, (double)h[0] / count / NI);
}

int main() {
  long long* out; CK(cudaMalloc(&out, 64));
  for (int pc : {1, 16, 64}) {
    run<16, 0>(pc, out, "A in tensor memory"); run<64, 0>(pc, out, "A in tensor memory"); run<128, 0>(pc, out, "A in tensor memory"); run<256, 0>(pc, out, "A in tensor memory");
    run<16, 1>(pc, out, "A in shared memory"); run<64, 1>(pc, out, "A in shared memory"); run<256, 1>(pc, out, "A in shared memory");
  }
  for (int pc : {16}) { run_multi<16, 1>(pc, out); run_multi<16, 2>(pc, out); run_multi<16, 4>(pc, out); run_multi<64, 1>(pc, out); run_multi<64, 2>(pc, out); run_multi<64, 4>(pc, out); }
  printf("done\n");
  return 0;
}
