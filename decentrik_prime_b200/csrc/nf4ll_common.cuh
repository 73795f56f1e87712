// Shared device helpers: the NF4 decode (bit-exact with the reference's arithmetic), and thin
// wrappers over the sm_100a PTX this library uses (mbarrier, TMA, tcgen05, proxy fences).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "nf4ll.h"

namespace nf4ll {

// Launch configuration with the attributes this library uses: programmatic dependent launch (only
// for kernels that call pdl_wait() first thing), an optional thread-block cluster, an optional
// cooperative launch (whole grid resident at once; not combined with the programmatic attribute).
void count_launch();   // definition in nf4ll_api.cu: one more kernel launched by the calling thread

struct PdlLaunch {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[3];
  PdlLaunch(dim3 grid, dim3 block, size_t smem, cudaStream_t stream, unsigned cluster_x = 0, unsigned cluster_y = 0,
            bool cooperative = false, bool counted = true) {
    cfg = cudaLaunchConfig_t{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    int n = 0;
    if (cluster_x || cluster_y) {
      attr[n].id = cudaLaunchAttributeClusterDimension;
      attr[n].val.clusterDim.x = cluster_x ? cluster_x : 1;
      attr[n].val.clusterDim.y = cluster_y ? cluster_y : 1;
      attr[n].val.clusterDim.z = 1;
      ++n;
    }
    if (cooperative) {
      attr[n].id = cudaLaunchAttributeCooperative;
      attr[n].val.cooperative = 1;
      ++n;
    } else {
      attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[n].val.programmaticStreamSerializationAllowed = 1;
      ++n;
    }
    cfg.attrs = attr; cfg.numAttrs = n;
    if (counted) count_launch();       // a configuration built only to query occupancy is not a launch
  }
};


// ---------------------------------------------------------------------------------------------
// Host-side error plumbing (definitions in nf4ll_api.cu)
// ---------------------------------------------------------------------------------------------
void set_detail(const char* fmt, ...);
int cuda_fail(cudaError_t err, const char* what);
int require_sm100();   // NF4LL_OK or NF4LL_ERR_ARCH for the current device

#define NF4LL_CUDA(expr)                                              \
  do {                                                                \
    cudaError_t e__ = (expr);                                         \
    if (e__ != cudaSuccess) return ::nf4ll::cuda_fail(e__, #expr);    \
  } while (0)

// ---------------------------------------------------------------------------------------------
// NF4 decode
// ---------------------------------------------------------------------------------------------
// The 16 NF4 levels, fp32 (reference solution/k_nf4.py:29-34).
#define NF4LL_LEVELS                                                                          \
  -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,                   \
      -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,              \
      0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f, \
      0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f

// absmax of one quantisation block: code2[q] * scale2 + offset2, the product and the sum rounded
// separately (reference solution/k_nf4.py:19-21, 47-49; its launcher disables FMA fusion, 180).
__device__ __forceinline__ float block_absmax(float code, float scale2, float offset2) {
  return __fadd_rn(__fmul_rn(code, scale2), offset2);
}

// The 16 possible fp16 values of one quantisation block, fp16(NF4[c] * absmax) for c = 0..15, held
// as eight byte-plane registers so that four 4-bit codes can be looked up at once with byte
// permutes: lo[j] has the low bytes of entries 4j..4j+3, hi[j] their high bytes.
struct BlockTable {
  uint32_t lo[4];
  uint32_t hi[4];
};

__device__ __forceinline__ uint32_t pack_half2_rn(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);   // a -> low half, b -> high half, each round-to-nearest-even
  return *reinterpret_cast<uint32_t*>(&h);
}

// Raw byte permute. Unlike __byte_perm, which first clears bit 3 of every selector nibble (one more
// logic instruction per call), this hands the selector to the hardware as it is: bit 3 of a nibble
// would ask for sign replication, so callers keep it clear themselves.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

__device__ __forceinline__ BlockTable make_block_table(float absmax) {
  constexpr float lv[16] = {NF4LL_LEVELS};
  BlockTable t;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    // fp32 product rounded once, then rounded to fp16 (reference solution/k_nf4.py:53-54)
    uint32_t p0 = pack_half2_rn(__fmul_rn(lv[4 * j + 0], absmax), __fmul_rn(lv[4 * j + 1], absmax));
    uint32_t p1 = pack_half2_rn(__fmul_rn(lv[4 * j + 2], absmax), __fmul_rn(lv[4 * j + 3], absmax));
    t.lo[j] = __byte_perm(p0, p1, 0x6420);
    t.hi[j] = __byte_perm(p0, p1, 0x7531);
  }
  return t;
}

// Decode one 32-bit word of packed codes (bytes b0..b3 = elements 0..7, the even element of each
// byte in its high nibble) into 8 fp16 values, returned as four half2 registers in element order.
__device__ __forceinline__ uint4 decode_word(const BlockTable& t, uint32_t w) {
  // every selector nibble below stays within 0..7 (bit 3 clear), as the raw permute requires; only the
  // low 16 bits of a selector are read, so the shifted copies may carry anything above them
  const uint32_t sel = w & 0x77777777u;                                // low 3 bits of every code
  const uint32_t pick = ((w >> 1) & 0x44444444u) | 0x32103210u;        // byte i from the upper table if bit 3
  uint4 out;
  {
    const uint32_t la = prmt(t.lo[0], t.lo[1], sel), lb = prmt(t.lo[2], t.lo[3], sel);
    const uint32_t ha = prmt(t.hi[0], t.hi[1], sel), hb = prmt(t.hi[2], t.hi[3], sel);
    const uint32_t lo = prmt(la, lb, pick), hi = prmt(ha, hb, pick);
    // nibble order in the low 16 bits: e1, e0, e3, e2 -> (e0, e1) and (e2, e3)
    out.x = prmt(lo, hi, 0x4051u);
    out.y = prmt(lo, hi, 0x6273u);
  }
  {
    const uint32_t sel2 = sel >> 16, pick2 = pick >> 16;
    const uint32_t la = prmt(t.lo[0], t.lo[1], sel2), lb = prmt(t.lo[2], t.lo[3], sel2);
    const uint32_t ha = prmt(t.hi[0], t.hi[1], sel2), hb = prmt(t.hi[2], t.hi[3], sel2);
    const uint32_t lo = prmt(la, lb, pick2), hi = prmt(ha, hb, pick2);
    out.z = prmt(lo, hi, 0x4051u);
    out.w = prmt(lo, hi, 0x6273u);
  }
  return out;
}

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch. A kernel launched through PdlLaunch may be set up on the SMs
// while the kernel before it on the stream is still finishing; pdl_wait() blocks until that kernel
// has completed and its writes are visible, and must come before the first access to global
// memory. pdl_launch_dependents() lets the NEXT kernel's blocks start as soon as every block of this
// one has called it (or exited). Both are no-ops for an ordinary launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// try_wait with a suspend-time hint (nanoseconds): the hardware parks the thread until the phase completes or the
// time is up, so a long wait costs a handful of instructions instead of a polling loop's issue slots
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Every wait on an mbarrier is bounded twice over: after kSpinLimit failed polls (each poll parks the thread
// for at most kParkNs) or after kWaitLimitNs of wall time, whichever comes first,
// the waiter gives up, and the kernel reports it through the status word instead of hanging the GPU. `abort_flag` (shared memory) makes all other waiters of
// the CTA give up quickly too.
// The first polls use the non-blocking test_wait: try_wait costs a few hundred cycles even when the
// phase is already complete, which is the common case on the MMA issuer's and the decoders'
// critical paths; try_wait (which lets the hardware park the thread) only takes over for long waits.
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr uint32_t kFastPolls = 32;
constexpr uint64_t kWaitLimitNs = 1000000000ull;      // and never longer than one second of wall time
constexpr uint32_t kParkNs = 20000;                    // one parked poll: at most 20 us, so an abort is seen quickly

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kFastPolls; ++i) {
    if (mbar_test_wait(bar, parity)) return true;
  }
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait_hint(bar, parity, kParkNs)) return true;
    if (*abort_flag) return false;
    if (global_timer_ns() - t0 > kWaitLimitNs) break;
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// TMA stores: shared -> global, tracked by the issuing thread's bulk async-group.
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(tmap), "r"(src), "r"(x), "r"(y) : "memory");
}
// element-wise add into global memory (done at the L2, in the tensor map's element type)
__device__ __forceinline__ void tma_reduce_add_2d(const void* tmap, uint32_t src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(tmap), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all committed groups have finished READING shared memory (it may be overwritten)
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all committed groups have completed, writes included
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
// bar.sync is an ALIGNED barrier: every lane of a warp has to execute it together. Code that lets one
// elected lane do extra work first (issue a TMA store, wait for it) must therefore reconverge
// explicitly, or the other lanes' early arrival releases the barrier before the elected lane is done.
__device__ __forceinline__ void named_barrier(int id, int threads) {
  __syncwarp();
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// --- tensor memory -----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {                               // whole warp
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {    // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier once every tcgen05 operation this thread issued so far has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] . B[smem], fp16 inputs, fp32 accumulate; one thread issues.
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread t of the warp gets lane (base lane + t).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
        "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// --- descriptors -------------------------------------------------------------------------------
// Shared-memory matrix descriptor of tcgen05.mma: start address, leading and stride byte offsets
// (all in 16-byte units), descriptor version 1, swizzle mode in bits 61-63.
constexpr uint64_t kSwizzleNone = 0, kSwizzle128B = 2;

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint64_t swizzle) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16) |
         (static_cast<uint64_t>(sbo_bytes >> 4) << 32) | (1ull << 46) | (swizzle << 61);
}

// Instruction descriptor for kind::f16 with fp16 A and B and an fp32 accumulator.
// a_mn / b_mn: 0 = the operand is K-major in shared memory, 1 = MN-major.
__host__ __device__ constexpr uint32_t make_idesc_f16(int m, int n, int a_mn, int b_mn) {
  return (1u << 4) | (static_cast<uint32_t>(a_mn) << 15) | (static_cast<uint32_t>(b_mn) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------
// Warp-level pieces shared by the rank-16 LoRA kernels
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// drop(x) on 8 packed fp16 values: fp16(x * keep_scale) where the mask byte is non-zero, else 0
// (reference solution/k_norm.py:49-53: scale in fp32, then one rounding to fp16).
__device__ __forceinline__ uint4 drop8(uint4 raw, uint2 m, float keep_scale) {
  uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  const uint32_t mw[2] = {m.x, m.y};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
    const bool k0 = ((mw[j >> 1] >> ((2 * j & 3) * 8)) & 0xffu) != 0;
    const bool k1 = ((mw[j >> 1] >> (((2 * j + 1) & 3) * 8)) & 0xffu) != 0;
    w[j] = pack_half2_rn(k0 ? v.x * keep_scale : 0.f, k1 ? v.y * keep_scale : 0.f);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---------------------------------------------------------------------------------------------
// Gated SiLU on 8 packed fp16 values (fp32 math), shared by the stand-alone kernels and the fused
// gate|up epilogue
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 v = __half22float2(h[j]);
    f[2 * j] = v.x;
    f[2 * j + 1] = v.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_half2_rn(f[0], f[1]), pack_half2_rn(f[2], f[3]), pack_half2_rn(f[4], f[5]),
                    pack_half2_rn(f[6], f[7]));
}

// sigmoid through the special-function unit: ex2.approx and rcp.approx, a few ulp of fp32 - far inside
// the fp16 rounding of the results
__device__ __forceinline__ float fast_sigmoid(float a) { return __fdividef(1.0f, 1.0f + __expf(-a)); }

__device__ __forceinline__ uint4 swiglu_fwd8(const uint4& gv, const uint4& uv) {
  float a[8], b[8], o[8];
  unpack8(gv, a); unpack8(uv, b);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = a[j] * fast_sigmoid(a[j]) * b[j];
  return pack8(o);
}

__device__ __forceinline__ void swiglu_bwd8(const uint4& gv, const uint4& uv, const uint4& dv, uint4& og4, uint4& ou4) {
  float a[8], b[8], d[8], og[8], ou[8];
  unpack8(gv, a); unpack8(uv, b); unpack8(dv, d);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float sig = fast_sigmoid(a[j]);
    ou[j] = d[j] * (a[j] * sig);
    og[j] = (d[j] * b[j]) * sig * (1.0f + a[j] * (1.0f - sig));
  }
  og4 = pack8(og); ou4 = pack8(ou);
}

}  // namespace nf4ll
