// Fused residual add + RMSNorm producer of the NF4 + LoRA linear's inputs, and its backward.
//
// Forward (replaces the reference's rms_fwd_kernel, solution/k_norm.py:29-53, and the two LoRA-A GEMMs that
// read its xq / xv outputs, solution/fast_qwen.py:943-944; call sites fast_qwen.py:1021-1027):
//     x    = x_prev (fp32) [+ delta (fp16 GEMM output)]        residual stream, kept in fp32
//     rstd = rsqrt(mean(x^2) + eps)
//     y    = w * (x * rstd);   y16 = fp16(y)                    the A operand of the projections that follow
//     T_i  = fp16(keep_i ? y * keep_scale : 0) . A_i^T          for up to two LoRA branches (q and v), fp32 [M,16]
// The reference writes the dropped-out copies xq, xv ([M, D] fp16 each) and multiplies them by lora_A in
// separate GEMMs; here the rank-16 products are formed on the tensor cores while y is still in registers, so
// neither the copies nor a second pass over y exist, and the projections get their rank-16 operand ready-made.
//
// Backward (replaces rms_bwd_kernel, solution/k_norm.py:56-87, and the two GEMMs lqx = daq . A_q,
// lvx = dav . A_v that feed it, solution/fast_qwen.py:1376-1380):
//     dy   = fp16 grad * gscale + sum_i keep_i * keep_scale * (u_i . A_i)     u_i fp32 [M,16] = scale * d(out_i) . B_i
//     dx   = rstd * (w*dy - xhat * mean(w*dy*xhat)),  xhat = x * rstd
//     out  = dres + dx  (fp32)  and its fp16 copy
// The [M, D] LoRA input gradients of the reference never exist: the rank-16 factors are expanded per element.
//
// A CTA owns 16 (forward) or 8 (backward) token rows and the whole hidden dimension, sixteen warps deep; a
// lane's values stay in registers between the row reduction and the second phase, so every input is read once.
#include "nf4ll_common.cuh"

namespace nf4ll {

constexpr int kNormWarps = 16;

struct NormBranch {
  const __half* A;        // lora_A fp16 [16, D]; null = branch absent
  const uint8_t* mask;    // keep-mask [M, ld_mask] or null (no dropout)
  int64_t ld_mask;
  float keep_scale;
  float* t;               // forward: out fp32 [M,16]
  const float* u;         // backward: in fp32 [M,16]
};

__device__ __forceinline__ void load8_f32(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void store8_f32(float* p, const float (&v)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ bool keep_bit(const uint2& m, int j) {
  return (((j < 4 ? m.x : m.y) >> ((j & 3) * 8)) & 0xffu) != 0;
}

// RG row groups of 8 rows per CTA, CPW 32-column chunks per warp (D <= kNormWarps * 32 * CPW)
template <int RG, int CPW>
__global__ void __launch_bounds__(kNormWarps * 32)
rms_fwd_kernel(const float* __restrict__ x, const __half* __restrict__ delta, float* __restrict__ xout,
               const float* __restrict__ w, float eps, int64_t M, int64_t D, __half* __restrict__ y16, int64_t ldy,
               float* __restrict__ rstd_out, const NormBranch ba, const NormBranch bb) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int ROWS = 8 * RG;
  __shared__ float s_part[kNormWarps][ROWS];
  __shared__ float s_rstd[ROWS];
  __shared__ float s_t[kNormWarps][ROWS][17];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t m0 = static_cast<int64_t>(blockIdx.x) * ROWS;
  int64_t row[RG];
  bool ok[RG];
#pragma unroll
  for (int i = 0; i < RG; ++i) {
    row[i] = m0 + g + 8 * i;
    ok[i] = row[i] < M;
    if (!ok[i]) row[i] = 0;
  }
  // phase 1: load (x + delta), write the residual stream, sum of squares
  float xv[CPW][RG][8];
  float ss[RG];
#pragma unroll
  for (int i = 0; i < RG; ++i) ss[i] = 0.f;
#pragma unroll
  for (int c = 0; c < CPW; ++c) {
    const int64_t k = (static_cast<int64_t>(c) * kNormWarps + warp) * 32 + t * 8;
#pragma unroll
    for (int i = 0; i < RG; ++i) {
#pragma unroll
      for (int j = 0; j < 8; ++j) xv[c][i][j] = 0.f;
      if (k < D && ok[i]) {
        load8_f32(x + row[i] * D + k, xv[c][i]);
        if (delta) {
          float dv[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(delta + row[i] * D + k)), dv);
#pragma unroll
          for (int j = 0; j < 8; ++j) xv[c][i][j] += dv[j];
        }
        if (xout) store8_f32(xout + row[i] * D + k, xv[c][i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss[i] = fmaf(xv[c][i][j], xv[c][i][j], ss[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < RG; ++i) {
    ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], 1);
    ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], 2);
    if (t == 0) s_part[warp][g + 8 * i] = ss[i];
  }
  __syncthreads();
  if (threadIdx.x < ROWS) {
    float v = 0.f;
#pragma unroll
    for (int wq = 0; wq < kNormWarps; ++wq) v += s_part[wq][threadIdx.x];
    const float r = rsqrtf(v * (1.0f / static_cast<float>(D)) + eps);
    s_rstd[threadIdx.x] = r;
    if (m0 + threadIdx.x < M) rstd_out[m0 + threadIdx.x] = r;
  }
  __syncthreads();
  // phase 2: y, its fp16 copy, and the rank-16 products of the dropped-out copies
  float ca[RG][4], cb[RG][4];
#pragma unroll
  for (int i = 0; i < RG; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { ca[i][j] = 0.f; cb[i][j] = 0.f; }
#pragma unroll
  for (int c = 0; c < CPW; ++c) {
    const int64_t kc = (static_cast<int64_t>(c) * kNormWarps + warp) * 32;      // first column of the warp's chunk
    const int64_t k = kc + t * 8;
    // the MMAs below are warp-wide instructions: the whole warp takes part in a chunk that starts inside the
    // row, and lanes whose eight columns lie past its end (D need not be a multiple of 32) contribute zeros
    if (kc < D) {
      const bool in = k < D;
      float wv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) wv[j] = 0.f;
      if (in) load8_f32(w + k, wv);
      uint4 ra = make_uint4(0, 0, 0, 0), rb = ra, sa = ra, sb = ra;
      if (ba.A && in) { ra = __ldg(reinterpret_cast<const uint4*>(ba.A + static_cast<int64_t>(g) * D + k));
                        rb = __ldg(reinterpret_cast<const uint4*>(ba.A + static_cast<int64_t>(g + 8) * D + k)); }
      if (bb.A && in) { sa = __ldg(reinterpret_cast<const uint4*>(bb.A + static_cast<int64_t>(g) * D + k));
                        sb = __ldg(reinterpret_cast<const uint4*>(bb.A + static_cast<int64_t>(g + 8) * D + k)); }
#pragma unroll
      for (int i = 0; i < RG; ++i) {
        const float r = s_rstd[g + 8 * i];
        const bool live = in && ok[i];
        float y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = wv[j] * (xv[c][i][j] * r);
        if (y16 && live) *reinterpret_cast<uint4*>(y16 + row[i] * ldy + k) = pack8(y);
        if (ba.A) {
          float d[8];
          const uint2 m = (ba.mask && live) ? __ldg(reinterpret_cast<const uint2*>(ba.mask + row[i] * ba.ld_mask + k)) : make_uint2(0, 0);
#pragma unroll
          for (int j = 0; j < 8; ++j) d[j] = live ? (ba.mask ? (keep_bit(m, j) ? y[j] * ba.keep_scale : 0.f) : y[j]) : 0.f;
          const uint4 q = pack8(d);
          mma16816(ca[i], ra.x, rb.x, ra.y, rb.y, q.x, q.y);
          mma16816(ca[i], ra.z, rb.z, ra.w, rb.w, q.z, q.w);
        }
        if (bb.A) {
          float d[8];
          const uint2 m = (bb.mask && live) ? __ldg(reinterpret_cast<const uint2*>(bb.mask + row[i] * bb.ld_mask + k)) : make_uint2(0, 0);
#pragma unroll
          for (int j = 0; j < 8; ++j) d[j] = live ? (bb.mask ? (keep_bit(m, j) ? y[j] * bb.keep_scale : 0.f) : y[j]) : 0.f;
          const uint4 q = pack8(d);
          mma16816(cb[i], sa.x, sb.x, sa.y, sb.y, q.x, q.y);
          mma16816(cb[i], sa.z, sb.z, sa.w, sb.w, q.z, q.w);
        }
      }
    }
  }
  // accumulator layout: c[.][0], c[.][1] = (rank g, rows 2t, 2t+1); c[.][2], c[.][3] = (rank g+8, same rows)
#pragma unroll
  for (int br = 0; br < 2; ++br) {
    const NormBranch& b = br ? bb : ba;
    if (!b.A) continue;               // uniform over the CTA
    __syncthreads();
#pragma unroll
    for (int i = 0; i < RG; ++i) {
      const float* c = br ? cb[i] : ca[i];
      s_t[warp][8 * i + 2 * t][g] = c[0];      s_t[warp][8 * i + 2 * t + 1][g] = c[1];
      s_t[warp][8 * i + 2 * t][g + 8] = c[2];  s_t[warp][8 * i + 2 * t + 1][g + 8] = c[3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < ROWS * 16; idx += kNormWarps * 32) {
      const int rr = idx >> 4, j = idx & 15;
      if (m0 + rr < M) {
        float v = 0.f;
#pragma unroll
        for (int wq = 0; wq < kNormWarps; ++wq) v += s_t[wq][rr][j];
        b.t[(m0 + rr) * 16 + j] = v;
      }
    }
  }
}

// 8 rows per CTA
template <int CPW>
__global__ void __launch_bounds__(kNormWarps * 32)
rms_bwd_kernel(const __half* __restrict__ dy16, int64_t lddy, float gscale, const float* __restrict__ x,
               const __half* __restrict__ delta, const float* __restrict__ w, const float* __restrict__ rstd,
               const float* dres, float* out, __half* __restrict__ out16, int64_t M, int64_t D,
               const NormBranch ba, const NormBranch bb) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float s_part[kNormWarps][8];
  __shared__ float s_c[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t m0 = static_cast<int64_t>(blockIdx.x) * 8;
  const bool ok = m0 + g < M;
  const int64_t row = ok ? m0 + g : 0;
  const float r = __ldg(rstd + row);
  float ua[16], ub[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) { ua[j] = 0.f; ub[j] = 0.f; }
  if (ba.A) {
#pragma unroll
    for (int j4 = 0; j4 < 4; ++j4) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(ba.u + row * 16) + j4);
      ua[4 * j4] = v.x * ba.keep_scale; ua[4 * j4 + 1] = v.y * ba.keep_scale; ua[4 * j4 + 2] = v.z * ba.keep_scale; ua[4 * j4 + 3] = v.w * ba.keep_scale;
    }
  }
  if (bb.A) {
#pragma unroll
    for (int j4 = 0; j4 < 4; ++j4) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(bb.u + row * 16) + j4);
      ub[4 * j4] = v.x * bb.keep_scale; ub[4 * j4 + 1] = v.y * bb.keep_scale; ub[4 * j4 + 2] = v.z * bb.keep_scale; ub[4 * j4 + 3] = v.w * bb.keep_scale;
    }
  }
  float gv[CPW][8];
  float cs = 0.f;
#pragma unroll
  for (int c = 0; c < CPW; ++c) {
    const int64_t k = (static_cast<int64_t>(c) * kNormWarps + warp) * 32 + t * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) gv[c][j] = 0.f;
    if (k < D && ok) {
      float dy[8], xr[8], wv[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(dy16 + row * lddy + k)), dy);
#pragma unroll
      for (int j = 0; j < 8; ++j) dy[j] *= gscale;
#pragma unroll
      for (int br = 0; br < 2; ++br) {
        const NormBranch& b = br ? bb : ba;
        if (!b.A) continue;
        const float* u = br ? ub : ua;
        float l[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) l[j] = 0.f;
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
          float av[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(b.A + static_cast<int64_t>(jj) * D + k)), av);
#pragma unroll
          for (int j = 0; j < 8; ++j) l[j] = fmaf(u[jj], av[j], l[j]);
        }
        if (b.mask) {
          const uint2 m = __ldg(reinterpret_cast<const uint2*>(b.mask + row * b.ld_mask + k));
#pragma unroll
          for (int j = 0; j < 8; ++j) dy[j] += keep_bit(m, j) ? l[j] : 0.f;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) dy[j] += l[j];
        }
      }
      load8_f32(x + row * D + k, xr);
      if (delta) {
        float dv[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(delta + row * D + k)), dv);
#pragma unroll
        for (int j = 0; j < 8; ++j) xr[j] += dv[j];
      }
      load8_f32(w + k, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        gv[c][j] = dy[j] * wv[j];
        cs = fmaf(gv[c][j], xr[j] * r, cs);
      }
    }
  }
  cs += __shfl_xor_sync(0xffffffffu, cs, 1);
  cs += __shfl_xor_sync(0xffffffffu, cs, 2);
  if (t == 0) s_part[warp][g] = cs;
  __syncthreads();
  if (threadIdx.x < 8) {
    float v = 0.f;
#pragma unroll
    for (int wq = 0; wq < kNormWarps; ++wq) v += s_part[wq][threadIdx.x];
    s_c[threadIdx.x] = v * (1.0f / static_cast<float>(D));
  }
  __syncthreads();
  const float cm = s_c[g];
#pragma unroll
  for (int c = 0; c < CPW; ++c) {
    const int64_t k = (static_cast<int64_t>(c) * kNormWarps + warp) * 32 + t * 8;
    if (k < D && ok) {
      float xr[8], o[8];
      load8_f32(x + row * D + k, xr);          // second read of x: from L1 / L2
      if (delta) {
        float dv[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(delta + row * D + k)), dv);
#pragma unroll
        for (int j = 0; j < 8; ++j) xr[j] += dv[j];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (gv[c][j] - (xr[j] * r) * cm) * r;
      if (dres) {
        float dv[8];
        load8_f32(dres + row * D + k, dv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += dv[j];
      }
      store8_f32(out + row * D + k, o);
      if (out16) *reinterpret_cast<uint4*>(out16 + row * D + k) = pack8(o);
    }
  }
}

static int check_branch(const nf4ll_lora* l, const void* side, const char* who, int64_t D, NormBranch* out, bool forward) {
  *out = NormBranch{};
  if (!l) return NF4LL_OK;
  if (l->r != 16) { set_detail("%s: LoRA rank %d", who, l->r); return NF4LL_ERR_RANK; }
  if (!l->A || !side) { set_detail("%s: a LoRA branch needs lora_A and its [M,16] %s", who, forward ? "output t" : "input u"); return NF4LL_ERR_NULL; }
  if ((reinterpret_cast<uintptr_t>(l->A) & 15) || (reinterpret_cast<uintptr_t>(side) & 15)) { set_detail("%s: LoRA operands must be 16-byte aligned", who); return NF4LL_ERR_ALIGN; }
  if (l->mask && ((reinterpret_cast<uintptr_t>(l->mask) & 7) || l->ld_mask % 8 || l->ld_mask < D)) {
    set_detail("%s: mask must be 8-byte aligned with ld_mask a multiple of 8 and >= D", who);
    return NF4LL_ERR_ALIGN;
  }
  out->A = static_cast<const __half*>(l->A);
  out->mask = l->mask; out->ld_mask = l->ld_mask; out->keep_scale = l->mask ? l->keep_scale : 1.0f;
  if (forward) out->t = static_cast<float*>(const_cast<void*>(side)); else out->u = static_cast<const float*>(side);
  return NF4LL_OK;
}

static int check_norm_shape(const char* who, int64_t M, int64_t D) {
  if (M < 0 || D <= 0 || D % 8 || D > kNormWarps * 32 * 8) {
    set_detail("%s: M=%lld, D=%lld (D a multiple of 8, at most %d)", who, static_cast<long long>(M), static_cast<long long>(D), kNormWarps * 32 * 8);
    return NF4LL_ERR_SHAPE;
  }
  return NF4LL_OK;
}

}  // namespace nf4ll

extern "C" int nf4ll_rms_forward(const float* x, const void* delta16, float* xout, const float* w, float eps, int64_t M,
                                 int64_t D, void* y16, int64_t ldy, float* rstd, const nf4ll_lora* lora_a, void* t_a,
                                 const nf4ll_lora* lora_b, void* t_b, void* stream) {
  using namespace nf4ll;
  const char* who = "nf4ll_rms_forward";
  if (int rc = check_norm_shape(who, M, D)) return rc;
  if (M == 0) return NF4LL_OK;
  if (!x || !w || !rstd) { set_detail("%s: x, w and rstd are required", who); return NF4LL_ERR_NULL; }
  for (const void* p : {static_cast<const void*>(x), delta16, static_cast<const void*>(xout), static_cast<const void*>(w), static_cast<const void*>(y16)})
    if (reinterpret_cast<uintptr_t>(p) & 15) { set_detail("%s: pointers must be 16-byte aligned", who); return NF4LL_ERR_ALIGN; }
  if (y16 && (ldy % 8 || ldy < D)) { set_detail("%s: ldy must be a multiple of 8 and >= D", who); return NF4LL_ERR_ALIGN; }
  NormBranch ba, bb;
  if (int rc = check_branch(lora_a, t_a, who, D, &ba, true)) return rc;
  if (int rc = check_branch(lora_b, t_b, who, D, &bb, true)) return rc;
  if (int rc = require_sm100()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int cpw = static_cast<int>((D + kNormWarps * 32 - 1) / (kNormWarps * 32));
  const __half* dl = static_cast<const __half*>(delta16);
  __half* y = static_cast<__half*>(y16);
  if (cpw <= 4) {
    PdlLaunch lc(dim3(static_cast<unsigned>((M + 15) / 16)), dim3(kNormWarps * 32), 0, st);
    NF4LL_CUDA(cudaLaunchKernelEx(&lc.cfg, rms_fwd_kernel<2, 4>, x, dl, xout, w, eps, M, D, y, ldy, rstd, ba, bb));
  } else {
    PdlLaunch lc(dim3(static_cast<unsigned>((M + 7) / 8)), dim3(kNormWarps * 32), 0, st);
    NF4LL_CUDA(cudaLaunchKernelEx(&lc.cfg, rms_fwd_kernel<1, 8>, x, dl, xout, w, eps, M, D, y, ldy, rstd, ba, bb));
  }
  return NF4LL_OK;
}

extern "C" int nf4ll_rms_backward(const void* dy16, int64_t lddy, float gscale, const float* x, const void* delta16,
                                  const float* w, const float* rstd, const float* dres, float* out, void* out16, int64_t M,
                                  int64_t D, const nf4ll_lora* lora_a, const void* u_a, const nf4ll_lora* lora_b,
                                  const void* u_b, void* stream) {
  using namespace nf4ll;
  const char* who = "nf4ll_rms_backward";
  if (int rc = check_norm_shape(who, M, D)) return rc;
  if (M == 0) return NF4LL_OK;
  if (!dy16 || !x || !w || !rstd || !out) { set_detail("%s: dy, x, w, rstd and out are required", who); return NF4LL_ERR_NULL; }
  for (const void* p : {dy16, static_cast<const void*>(x), delta16, static_cast<const void*>(w), static_cast<const void*>(dres),
                        static_cast<const void*>(out), static_cast<const void*>(out16)})
    if (reinterpret_cast<uintptr_t>(p) & 15) { set_detail("%s: pointers must be 16-byte aligned", who); return NF4LL_ERR_ALIGN; }
  if (lddy % 8 || lddy < D) { set_detail("%s: lddy must be a multiple of 8 and >= D", who); return NF4LL_ERR_ALIGN; }
  NormBranch ba, bb;
  if (int rc = check_branch(lora_a, u_a, who, D, &ba, false)) return rc;
  if (int rc = check_branch(lora_b, u_b, who, D, &bb, false)) return rc;
  if (int rc = require_sm100()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int cpw = static_cast<int>((D + kNormWarps * 32 - 1) / (kNormWarps * 32));
  PdlLaunch lc(dim3(static_cast<unsigned>((M + 7) / 8)), dim3(kNormWarps * 32), 0, st);
  const __half* dyp = static_cast<const __half*>(dy16);
  const __half* dl = static_cast<const __half*>(delta16);
  __half* o16 = static_cast<__half*>(out16);
  if (cpw <= 4) {
    NF4LL_CUDA(cudaLaunchKernelEx(&lc.cfg, rms_bwd_kernel<4>, dyp, lddy, gscale, x, dl, w, rstd, dres, out, o16, M, D, ba, bb));
  } else {
    NF4LL_CUDA(cudaLaunchKernelEx(&lc.cfg, rms_bwd_kernel<8>, dyp, lddy, gscale, x, dl, w, rstd, dres, out, o16, M, D, ba, bb));
  }
  return NF4LL_OK;
}
