// Standalone micro-benchmark of weight-streaming variants (M = 1 token row), to find what limits the kernel.
// Built and run by tests/micro/run.py.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <vector>
#include <algorithm>

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e), __FILE__, __LINE__); exit(1); } } while (0)

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr)); return v; }
template <int I> __device__ __forceinline__ uint32_t eoff(uint32_t w, uint32_t lane_off) {
  const uint32_t s = (I == 0) ? (w << 7) : (w >> (8 * I - 7));
  return (s & 0x7F80u) | lane_off;
}
__device__ __forceinline__ void decode8(uint32_t w, uint32_t table, uint32_t lane_off, uint32_t (&h)[4]) {
  h[0] = lds_u32(table + eoff<0>(w, lane_off)); h[1] = lds_u32(table + eoff<1>(w, lane_off));
  h[2] = lds_u32(table + eoff<2>(w, lane_off)); h[3] = lds_u32(table + eoff<3>(w, lane_off));
}

struct P {
  const uint8_t* nib; const uint8_t* qabs; const __half* x; float* y;
  int N, K, slices, bps, n_units; int* counter; int mode; int order;
};
// mode 0: full; 1: loads only; 2: compute only (no global code loads); order 0: slice-major, 1: row-group-major
constexpr int W = 8;

template <int PREFETCH>
__global__ void __launch_bounds__(W * 32, 4) k_stream(const P p) {
  __shared__ __align__(128) uint32_t s_tbl[256 * 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  for (int idx = threadIdx.x; idx < 256 * 32; idx += W * 32) {
    const int v = idx >> 5;
    const __half a = __float2half(((v >> 4) - 7.5f) / 8.f), b = __float2half(((v & 15) - 7.5f) / 8.f);
    s_tbl[idx] = __half_as_ushort(a) | (uint32_t(__half_as_ushort(b)) << 16);
  }
  __syncthreads();
  const uint32_t table = (uint32_t)__cvta_generic_to_shared(s_tbl), lane_off = lane * 4;
  const int n_rg = p.N / 16, bpr = p.K / 64, total_warps = gridDim.x * W;
  int unit = blockIdx.x * W + warp;
  float sink = 0.f;
  while (unit < p.n_units) {
    int sl, rg;
    if (p.order == 0) { sl = unit / n_rg; rg = unit - sl * n_rg; } else { rg = unit / p.slices; sl = unit - rg * p.slices; }
    const int64_t row0 = (int64_t)rg * 16 + g, row1 = row0 + 8;
    const int b_begin = sl * p.bps, b_end = min(b_begin + p.bps, bpr);
    const uint8_t* w0 = p.nib + (row0 * p.K) / 2 + t * 8 + (int64_t)b_begin * 32;
    const uint8_t* w1 = p.nib + (row1 * p.K) / 2 + t * 8 + (int64_t)b_begin * 32;
    int64_t qa = (row0 * p.K) / 64 + b_begin + t, qb = (row1 * p.K) / 64 + b_begin + t;
    const __half* xr = p.x + t * 16 + (int64_t)b_begin * 64;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    uint2 c0[4], c1[4], n0[4], n1[4];
    auto load = [&](uint2 (&a)[4], uint2 (&b)[4], const uint8_t* pa, const uint8_t* pb) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (p.mode == 2) { a[u] = make_uint2(0x12345678u + u, 0x9abcdef0u); b[u] = make_uint2(0x0fedcba9u, 0x87654321u + u); }
        else { a[u] = __ldcs(reinterpret_cast<const uint2*>(pa + u * 32)); b[u] = __ldcs(reinterpret_cast<const uint2*>(pb + u * 32)); }
      }
    };
    if (PREFETCH) load(n0, n1, w0, w1);
    for (int b = b_begin; b < b_end; b += 4) {
      if (PREFETCH) {
#pragma unroll
        for (int u = 0; u < 4; ++u) { c0[u] = n0[u]; c1[u] = n1[u]; }
        if (b + 4 < b_end) load(n0, n1, w0 + 128, w1 + 128);
      } else {
        load(c0, c1, w0, w1);
      }
      float am0 = 1.f, am1 = 1.f;
      if (p.mode != 2) { am0 = (float)__ldg(p.qabs + qa) * (1.f / 256.f); am1 = (float)__ldg(p.qabs + qb) * (1.f / 256.f); }
      if (p.mode == 1) {
#pragma unroll
        for (int u = 0; u < 4; ++u) sink += __uint_as_float((c0[u].x ^ c0[u].y ^ c1[u].x ^ c1[u].y) & 0x3fffffff);
        sink += am0 + am1;
      } else {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float a0 = __shfl_sync(0xffffffffu, am0, (lane & ~3) | u), a1 = __shfl_sync(0xffffffffu, am1, (lane & ~3) | u);
          uint32_t lo0[4], hi0[4], lo1[4], hi1[4];
          decode8(c0[u].x, table, lane_off, lo0); decode8(c0[u].y, table, lane_off, hi0);
          decode8(c1[u].x, table, lane_off, lo1); decode8(c1[u].y, table, lane_off, hi1);
          const uint4 xa = __ldg(reinterpret_cast<const uint4*>(xr + u * 64)), xb = __ldg(reinterpret_cast<const uint4*>(xr + u * 64 + 8));
          float blk[4] = {0.f, 0.f, 0.f, 0.f};
          mma16816(blk, lo0[0], lo1[0], lo0[1], lo1[1], xa.x, xa.y);
          mma16816(blk, lo0[2], lo1[2], lo0[3], lo1[3], xa.z, xa.w);
          mma16816(blk, hi0[0], hi1[0], hi0[1], hi1[1], xb.x, xb.y);
          mma16816(blk, hi0[2], hi1[2], hi0[3], hi1[3], xb.z, xb.w);
          acc[0] = fmaf(blk[0], a0, acc[0]); acc[1] = fmaf(blk[1], a0, acc[1]);
          acc[2] = fmaf(blk[2], a1, acc[2]); acc[3] = fmaf(blk[3], a1, acc[3]);
        }
      }
      w0 += 128; w1 += 128; qa += 4; qb += 4; xr += 256;
    }
    sink += acc[0] + acc[1] + acc[2] + acc[3];
    int next = 0;
    if (lane == 0) next = total_warps + atomicAdd(p.counter, 1);
    unit = __shfl_sync(0xffffffffu, next, 0);
  }
  if (sink == 123.456f) p.y[threadIdx.x] = sink;
}

// plain streaming read of the same bytes: fully coalesced 16-byte loads, UNROLL loads in flight per thread
template <int UNROLL>
__global__ void __launch_bounds__(256) k_read(const uint4* __restrict__ src, int64_t n16, float* y) {
  uint32_t s = 0;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + (UNROLL - 1) * stride < n16; i += UNROLL * stride) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) v[u] = __ldcs(src + i + u * stride);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) s ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
  }
  if (s == 0x12345u) y[threadIdx.x] = 1.f;
}

// row-strided read: a warp reads `seg` contiguous bytes of each of 16 rows per step (the streaming kernel's pattern)
// with 16-byte loads: lane l reads row (l / (seg/16)) ... generalised: each lane 16 bytes, rows = 512 / seg per instruction
__global__ void __launch_bounds__(256) k_rows(const uint8_t* __restrict__ src, int N, int K, int seg, int iters_in_flight, float* y, int* counter) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int lanes_per_row = seg / 16, rows_per_instr = 32 / lanes_per_row;
  const int rowbytes = K / 2;
  const int chunks_per_row = rowbytes / seg;
  const int64_t n_units = (int64_t)(N / rows_per_instr) * chunks_per_row;      // unit: rows_per_instr rows x seg bytes
  const int total_warps = gridDim.x * 8;
  uint32_t s = 0;
  // static striding over units, 8 loads in flight per lane
  for (int64_t u0 = (int64_t)blockIdx.x * 8 + warp; u0 < n_units; u0 += (int64_t)total_warps * 8) {
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t u = u0 + (int64_t)j * total_warps;
      if (u < n_units) {
        const int64_t rgrp = u % (N / rows_per_instr), ch = u / (N / rows_per_instr);     // slice-major
        const int64_t row = rgrp * rows_per_instr + lane / lanes_per_row;
        v[j] = __ldcs(reinterpret_cast<const uint4*>(src + row * rowbytes + ch * seg + (lane % lanes_per_row) * 16));
      } else v[j] = make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s ^= v[j].x ^ v[j].y ^ v[j].z ^ v[j].w;
  }
  if (s == 0x12345u) y[threadIdx.x] = 1.f;
}

int main() {
  const int N = 27648, K = 5120, COPIES = 4;
  const size_t nib_bytes = (size_t)N * K / 2, q_bytes = (size_t)N * K / 64;
  std::vector<uint8_t*> nibs(COPIES), qs(COPIES);
  std::vector<uint8_t> h(nib_bytes);
  for (size_t i = 0; i < nib_bytes; ++i) h[i] = (uint8_t)(rand() & 0xff);
  for (int c = 0; c < COPIES; ++c) {
    CK(cudaMalloc(&nibs[c], nib_bytes)); CK(cudaMalloc(&qs[c], q_bytes));
    CK(cudaMemcpy(nibs[c], h.data(), nib_bytes, cudaMemcpyHostToDevice)); CK(cudaMemcpy(qs[c], h.data(), q_bytes, cudaMemcpyHostToDevice));
  }
  __half* x; float* y; int* counter;
  CK(cudaMalloc(&x, K * 2)); CK(cudaMemset(x, 0, K * 2)); CK(cudaMalloc(&y, 4096)); CK(cudaMalloc(&counter, 4));
  cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
  const double bytes = (double)nib_bytes + q_bytes;
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
    printf("%-60s %8.2f us  %8.1f GB/s\n", name, ts[ts.size() / 2] * 1e3, bytes / (ts[ts.size() / 2] * 1e-3) / 1e9);
    fflush(stdout);
  };
  char name[128];
  for (int unroll : {4, 8}) {
    for (int ctas : {148 * 4, 148 * 8, 148 * 16}) {
      snprintf(name, sizeof name, "plain read, 16 B loads, unroll %d, %d CTAs", unroll, ctas);
      time_it(name, [&](int c) {
        if (unroll == 4) k_read<4><<<ctas, 256>>>((const uint4*)nibs[c], nib_bytes / 16, y); else k_read<8><<<ctas, 256>>>((const uint4*)nibs[c], nib_bytes / 16, y);
      });
    }
  }
  for (int seg : {32, 64, 128, 256, 512}) {
    snprintf(name, sizeof name, "row-strided read, %d contiguous bytes per row per step", seg);
    time_it(name, [&](int c) { k_rows<<<148 * 8, 256>>>(nibs[c], N, K, seg, 8, y, counter); });
  }
  const int bpr = K / 64;
  for (int mode : {0, 1, 2}) for (int order : {0, 1}) for (int pre : {0, 1}) for (int S : {1, 2, 5, 10}) for (int ctas_per_sm : {4}) {
    P p{}; p.N = N; p.K = K; p.x = x; p.y = y; p.counter = counter; p.mode = mode; p.order = order;
    int per = (bpr + S - 1) / S; per = (per + 3) / 4 * 4; p.slices = (bpr + per - 1) / per; p.bps = per; p.n_units = (N / 16) * p.slices;
    int grid = std::min((p.n_units + W - 1) / W, 148 * ctas_per_sm);
    snprintf(name, sizeof name, "stream mode %d (0 full,1 loads,2 compute) order %d prefetch %d S %d", mode, order, pre, p.slices);
    time_it(name, [&](int c) {
      p.nib = nibs[c]; p.qabs = qs[c];
      CK(cudaMemsetAsync(counter, 0, 4));
      if (pre) k_stream<1><<<grid, W * 32>>>(p); else k_stream<0><<<grid, W * 32>>>(p);
    });
  }
  CK(cudaDeviceSynchronize());
  printf("done\n");
  return 0;
}
