/* nf4ll: NF4-quantised frozen linear layer with a fused LoRA branch, for NVIDIA B200 (sm_100a).
 *
 * C ABI of libnf4ll.so. Every pointer is a DEVICE pointer unless a comment says otherwise; the
 * caller owns every buffer. The library allocates nothing, keeps no caller pointer after a call
 * returns and has no global mutable state besides thread-local settings (error detail, test hooks)
 * and the cached address of its built-in scratch (nf4ll_forward_static), so it may be called
 * from several host threads and streams at once. Calls only enqueue work on `stream`
 * (a cudaStream_t passed as void*); nothing synchronises unless a comment says so.
 *
 * Return value: 0, or a negative nf4ll_status code. Codes -10..-19 are caller mistakes (what the
 * reference reports as ValueError), the others are device or driver failures.
 *
 * The weight format is the reference's (solution/k_nf4.py:16-21, 64-95): for W[N,K] row-major,
 * element e = n*K + k sits in byte e/2 (even element in the HIGH nibble) and dequantises to
 *   fp16( NF4[nibble] * absmax[e/64] ),  absmax[b] = code2[qabs[b]] * scale2[b/256] + offset2[b/256]
 * with the product and the sum rounded separately in fp32 and the final product rounded to
 * nearest-even fp16.
 */
#ifndef NF4LL_H_
#define NF4LL_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NF4LL_VERSION 1

enum nf4ll_status {
  NF4LL_OK = 0,
  NF4LL_ERR_NULL = -10,        /* a required pointer is NULL */
  NF4LL_ERR_SHAPE = -11,       /* a size is not supported (see each call) */
  NF4LL_ERR_ALIGN = -12,       /* a pointer or leading dimension breaks an alignment rule */
  NF4LL_ERR_RANK = -13,        /* LoRA rank other than 16 */
  NF4LL_ERR_WORKSPACE = -14,   /* workspace missing or smaller than nf4ll_workspace_bytes() */
  NF4LL_ERR_ARCH = -20,        /* current device is not compute capability 10.x */
  NF4LL_ERR_CUDA = -21,        /* a CUDA runtime / driver call failed (detail string has it) */
  NF4LL_ERR_DEVICE_WAIT = -22  /* a bounded wait inside a kernel ran out (from nf4ll_read_status) */
};

/* One NF4 weight W[N,K]: sub-views of a PackedLayer's four sections (reference
 * solution/k_nf4.py:64-95, PackedLayer / section_views) plus the 256-entry second-level code
 * table, which the reference passes to every launcher (solution/k_nf4.py:176-205, `code2`).
 * nib must be 16-byte aligned; N*K must be a multiple of 16384 and K a multiple of 64. */
typedef struct nf4ll_mat {
  const uint8_t* nib;     /* N*K/2 bytes  */
  const uint8_t* qabs;    /* N*K/64 bytes */
  const float* scale2;    /* N*K/16384    */
  const float* offset2;   /* N*K/16384    */
  const float* code2;     /* 256          */
  int64_t N, K;
} nf4ll_mat;

/* The LoRA branch of one linear: fp16 shadows of lora_A [r,K] and lora_B [N,r] (reference
 * solution/fast_qwen.py:452, 686-692), scale = alpha/r (fast_qwen.py:93, 225), and the dropout
 * keep-mask of the LoRA input (uint8 [M,K], non-zero = keep; reference solution/k_norm.py:10-11,
 * 49-53) with keep_scale = 1/float32(1-p) (fast_qwen.py:370). mask may be NULL (no dropout). */
typedef struct nf4ll_lora {
  const void* A;          /* __half [r,K] row-major */
  const void* B;          /* __half [N,r] row-major */
  int32_t r;              /* must be 16 */
  float scale;
  const uint8_t* mask;    /* [M, ld_mask] or NULL */
  int64_t ld_mask;
  float keep_scale;
  const void* Bt;         /* optional __half [r,N]: lora_B transposed, read by nf4ll_backward_dx; when NULL
                             the call transposes B into its workspace first */
} nf4ll_lora;

int nf4ll_version(void);

/* Static description of a status code. */
const char* nf4ll_error_string(int code);

/* What exactly failed in the calling thread's last failing call ("" if nothing). Thread-local. */
const char* nf4ll_last_error_detail(void);

/* Standalone dequantisation of n_qblocks blocks of 64 weights into fp16.
 * Replaces the reference's nf4_layer_dequant_kernel and its launcher dequant_tensors
 * (solution/k_nf4.py:40-57, 176-181); the NF4 level table is a compile-time constant here.
 * nib and out must be 16-byte aligned. scale2/offset2 are indexed from the first block given, so a
 * sub-range must start on a multiple of 256 blocks (the reference's dequant_range guarantees 1024). */
int nf4ll_dequant(const uint8_t* nib, const uint8_t* qabs, const float* scale2, const float* offset2,
                  const float* code2, int64_t n_qblocks, void* out_f16, void* stream);

/* Bytes of scratch that nf4ll_forward / nf4ll_backward_dx need for M rows against W[N,K] with LoRA
 * rank r (0 = no LoRA). The scratch holds the fp32 rank-r projection feeding the fused LoRA step, split-K
 * partial sums and tile counters. Always a multiple of 256; the workspace must be 256-byte aligned. */
int64_t nf4ll_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t r);

/* The same figure for calls made under nf4ll_tune_override(bm_tiles, bn, splits, ...): a forced split
 * count or tile shape changes the scratch a call needs. nf4ll_workspace_bytes itself never depends on
 * the calling thread's override. Testing hook; no counterpart in the reference. */
int64_t nf4ll_workspace_bytes_tuned(int64_t M, int64_t N, int64_t K, int32_t r, int32_t bm_tiles, int32_t bn,
                                    int32_t splits);

/* Forward:  y[M,N] = x[M,K] . W^T (+ bias) + scale * (drop(x) . A^T) . B^T,  drop(x) = fp16(x * mask * keep_scale)
 * in ONE pass over the NF4 bytes: tiles of W are dequantised into shared memory and fed to
 * tcgen05 MMAs (fp32 accumulation in tensor memory); bias and the LoRA term are added to the fp32
 * accumulator before the single rounding to fp16.
 * Replaces, per projection, the reference's dequant into the fp16 workspace + cuBLAS GEMM + LoRA
 * GEMMs + LoRA add: solution/fast_qwen.py:716-750 (_ws_load/_ws_use), 943-947, 1037, 1080-1098,
 * 1112 and solution/k_rope.py:39-45, 56-58.
 * x [M,ldx] fp16, y [M,ldy] fp16, bias fp16 [N] or NULL, lora NULL = no LoRA branch.
 * t_out: optional fp32 [M,16] = drop(x) . A^T (unscaled), kept for nf4ll_lora_grads.
 * ldx, ldy multiples of 8; x, y 16-byte aligned. status: optional device int32, set non-zero if a
 * bounded wait in the kernel expires (never reset by the library). */
int nf4ll_forward(const nf4ll_mat* W, const void* x, int64_t ldx, const void* bias,
                  const nf4ll_lora* lora, void* t_out, int64_t M, void* y, int64_t ldy,
                  void* workspace, int64_t workspace_bytes, int32_t* status, void* stream);

/* Size of the scratch buffer built into the library for nf4ll_forward_static. */
#define NF4LL_STATIC_SCRATCH_BYTES (40 * 1024 * 1024)

/* Forward over several projections that share x and lie row after row in one weight matrix, as the
 * reference's packed layer stores Q|K|V and gate|up (solution/k_nf4.py:7-10, 61) and as its fused
 * W_qkv GEMM uses them (solution/fast_qwen.py:405-413, 947; gate and up: 1080-1098): one launch
 * instead of one per projection, x read once per tile row.
 *   y[:, segment i] = x . W_i^T (+ bias over all N columns) + scale_i * (drop_i(x) . A_i^T) . B_i^T
 * W describes the stacked matrix (N = sum of the segments' rows); every segment's row count is a
 * multiple of 128; a segment with a LoRA branch must give t_out (fp32 [M,r], written by the call: the
 * backward needs it anyway). At most 4 segments. Workspace: nf4ll_workspace_bytes(M, N, K, 0).
 * The backward of such a group needs no entry point of its own: dX = [dY_1 | dY_2 | ...] . W is one
 * nf4ll_backward_dx on the stacked matrix for the base term (LoRA terms per projection). */
typedef struct {
  int64_t rows;             /* output columns (= weight rows) of this projection */
  const nf4ll_lora* lora;   /* its LoRA branch, or NULL */
  void* t_out;              /* fp32 [M,r] = drop(x) . A^T of this projection; required with lora */
  int32_t t_ready;          /* non-zero: t_out already holds that product (nf4ll_rms_forward wrote it while
                               producing x): the call reads it instead of computing it */
} nf4ll_segment;
int nf4ll_forward_multi(const nf4ll_mat* W, const void* x, int64_t ldx, const void* bias,
                        const nf4ll_segment* segments, int32_t n_segments, int64_t M, void* y, int64_t ldy,
                        void* workspace, int64_t workspace_bytes, int32_t* status, void* stream);

/* gate|up forward with the gated-SiLU product in the epilogue. W is gate_proj and up_proj stacked
 * ([2I, K], gate rows first: how the reference's packed layer stores them, solution/k_nf4.py:7-10, 61).
 * One launch computes
 *   g = x . Wg^T + LoRA_gate,   u = x . Wu^T + LoRA_up,   h = fp16(silu(g) * u)
 * where a tile holds 128 gate and the matching 128 up columns, so the product is formed from the
 * accumulators on their way out (from g and u as rounded to fp16: h is bit-identical to
 * nf4ll_swiglu_forward on the stored g, u). Replaces the two GEMMs and the gated_silu kernel of
 * solution/fast_qwen.py:1080-1108 (k_mlp.py:21-29). g and u are still written: the backward needs them.
 * A LoRA branch needs its t_out (fp32 [M,r]). I must be a multiple of 8 (of 128 for the fused path;
 * other widths, batches of at most 128 rows and calls under nf4ll_tune_override run the two
 * projections and the stand-alone product instead). Workspace: nf4ll_workspace_bytes(M, I, K, r). */
int nf4ll_forward_gate_up(const nf4ll_mat* W, const void* x, int64_t ldx, const nf4ll_lora* lora_gate,
                          const nf4ll_lora* lora_up, void* t_gate, void* t_up, int64_t M, void* g, int64_t ldg,
                          void* u, int64_t ldu, void* h, int64_t ldh, void* workspace, int64_t workspace_bytes,
                          int32_t* status, void* stream);

/* nf4ll_forward for callers that can neither allocate device memory nor pass a workspace - a plugin
 * host that bans allocations after start-up, a server whose memory pool is already sealed. It has no
 * counterpart in the reference. Same arguments and results as nf4ll_forward minus the workspace:
 * scratch comes from a fixed NF4LL_STATIC_SCRATCH_BYTES array inside the library's device image
 * (every GPU that loads the library holds that much until the process exits). Problems whose
 * nf4ll_workspace_bytes() exceeds it are refused with NF4LL_ERR_WORKSPACE; one config-0 forward
 * (M = 2048, 1536 x 1536, LoRA) fits. The call itself performs no allocation. The first call on
 * each device looks the array's device address up (that device must be current) and should happen
 * before any stream capture starts. All calls on a device share the one buffer, which keeps
 * whatever the last call wrote: the library clears the parts that must start at zero, but two calls
 * that overlap in time on the GPU (different streams) race on it - serialise them. */
int nf4ll_forward_static(const nf4ll_mat* W, const void* x, int64_t ldx, const void* bias,
                         const nf4ll_lora* lora, void* t_out, int64_t M, void* y, int64_t ldy,
                         int32_t* status, void* stream);

/* Backward-dX:  dx[M,K] (+)= dy[M,N] . W + keep_scale * mask (.) ((scale * dy . B) . A)
 * reading the same NF4 bytes (the contraction runs over N; no fp16 W and no W^T is materialised).
 * Replaces solution/fast_qwen.py:1310, 1320-1327, 1333-1338, 1350, 1364 (cuBLAS NN GEMMs on the
 * workspace), 1370/1373 (`daq`, `dav`), 1376-1377 (`lqx`, `lvx`) and the masked add in
 * solution/k_norm.py:64-71. accumulate != 0 adds to the existing dx (gate + up, q + k + v).
 * u_out: optional fp32 [M,16] = scale * dy . B, kept for nf4ll_lora_grads. */
int nf4ll_backward_dx(const nf4ll_mat* W, const void* dy, int64_t lddy, const nf4ll_lora* lora,
                      void* u_out, int64_t M, void* dx, int64_t lddx, int32_t accumulate,
                      void* workspace, int64_t workspace_bytes, int32_t* status, void* stream);

/* Rank-r projection on its own:  t32[M,r] = drop(x)[M,K] . A^T  and  t16 = fp16(scale * t32), with A
 * [r,K] row-major fp16 (lora_A; or lora_B transposed, to get dy . B). A small tensor-core GEMM that
 * streams x once. Replaces solution/fast_qwen.py:943-944 and 1370/1373. t32 is required, t16 optional.
 * K a multiple of 8; mask, when given, 16-byte aligned with ld_mask a multiple of 16. */
int nf4ll_lora_down(const void* x, int64_t ldx, const uint8_t* mask, int64_t ld_mask,
                    float keep_scale, const void* A, float scale, int32_t r,
                    int64_t M, int64_t K, void* t32, void* t16, void* stream);

/* LoRA gradients, fp32:  dA[r,K] (+)= u^T . drop(x),   dB[N,r] (+)= scale * dy^T . t
 * with t, u the fp32 [M,r] outputs of nf4ll_forward / nf4ll_backward_dx. fp32 t/u and fp32
 * accumulation keep dA/dB within 2e-2 of an fp32 reference, which the reference's fp16 GEMM outputs
 * (solution/fast_qwen.py:1369-1374) do not. dA, dB may point into a flat all-reduce bucket.
 * Either of dA/dB may be NULL to skip it. */
int nf4ll_lora_grads(const void* dy, int64_t lddy, const void* x, int64_t ldx, const uint8_t* mask,
                     int64_t ld_mask, float keep_scale, const void* t32, const void* u32,
                     float scale, int32_t r, int64_t M, int64_t N, int64_t K,
                     void* dA, void* dB, int32_t accumulate, void* stream);

/* Fused residual add + RMSNorm that PRODUCES the inputs of the projections which follow it:
 *   xs = x (+ delta16);  rstd = rsqrt(mean(xs^2) + eps);  y = w * (xs * rstd);  y16 = fp16(y)
 *   t_i = fp16(keep_i ? y * keep_scale_i : 0) . A_i^T      for up to two LoRA branches (q and v), fp32 [M,16]
 * Replaces the reference's rms_fwd_kernel (solution/k_norm.py:29-53; call sites solution/fast_qwen.py:1021-1027)
 * and the LoRA-A GEMMs on its dropped-out outputs xq / xv (fast_qwen.py:943-944): those [M,D] copies are never
 * written; hand t_i to nf4ll_forward_multi through nf4ll_segment.t_out with t_ready = 1.
 * x fp32 [M,D] (the residual stream), delta16 optional fp16 [M,D] added first, xout optional fp32 [M,D]
 * receiving xs (may be x itself), w fp32 [D], y16 optional fp16 [M,ldy], rstd fp32 [M].
 * lora_a / lora_b: NULL or a branch of which A [16,D], mask, ld_mask and keep_scale are read (mask 8-byte
 * aligned, ld_mask a multiple of 8); t_a / t_b receive the products. D a multiple of 8, at most 4096. */
int nf4ll_rms_forward(const float* x, const void* delta16, float* xout, const float* w, float eps, int64_t M,
                      int64_t D, void* y16, int64_t ldy, float* rstd, const nf4ll_lora* lora_a, void* t_a,
                      const nf4ll_lora* lora_b, void* t_b, void* stream);

/* Backward of that norm with the LoRA branches' input gradients folded in:
 *   dy = fp16 grad * gscale + sum_i keep_i * keep_scale_i * (u_i . A_i),   u_i fp32 [M,16] = scale_i * d(out_i) . B_i
 *   dx = rstd * (w*dy - xhat * mean(w*dy*xhat)),  xhat = xs * rstd;   out = dx (+ dres);  out16 = fp16(out)
 * Replaces rms_bwd_kernel (solution/k_norm.py:56-87) and the GEMMs lqx = daq . A_q, lvx = dav . A_v that feed it
 * (solution/fast_qwen.py:1376-1380): the rank-16 factors are expanded per element inside the kernel, so the
 * projections' backward-dX may run without its LoRA branch (one launch for the stacked Q|K|V matrix).
 * dy16 fp16 [M,lddy]; x, delta16 as in the forward (xs is recomputed); dres optional fp32 [M,D], may alias out;
 * out fp32 [M,D]; out16 optional fp16 [M,D]. u_a / u_b: the products nf4ll_lora_down gives for lora_B transposed. */
int nf4ll_rms_backward(const void* dy16, int64_t lddy, float gscale, const float* x, const void* delta16,
                       const float* w, const float* rstd, const float* dres, float* out, void* out16, int64_t M,
                       int64_t D, const nf4ll_lora* lora_a, const void* u_a, const nf4ll_lora* lora_b,
                       const void* u_b, void* stream);

/* SiLU-gated product between the up and down projections, fp32 math on fp16 matrices [M,I]:
 *   h = fp16(silu(g) * u);   backward: du = dh * silu(g), dg = (dh * u) * sig * (1 + g * (1 - sig)).
 * Same arithmetic as the reference's gated_silu_fwd/bwd kernels (solution/k_mlp.py:21-47), which is
 * the step between two calls of this library in an MLP block. dg / du may alias g / u.
 * I a multiple of 8; pointers 16-byte aligned; leading dimensions multiples of 8. */
int nf4ll_swiglu_forward(const void* g, int64_t ldg, const void* u, int64_t ldu, void* h, int64_t ldh,
                         int64_t M, int64_t I, void* stream);
int nf4ll_swiglu_backward(const void* g, int64_t ldg, const void* u, int64_t ldu, const void* dh,
                          int64_t lddh, void* dg, int64_t lddg, void* du, int64_t lddu, int64_t M,
                          int64_t I, void* stream);

/* Synchronise `stream`, copy the device status word to the host and return NF4LL_OK or
 * NF4LL_ERR_DEVICE_WAIT (detail string carries the raw word). */
int nf4ll_read_status(const int32_t* status, void* stream);

/* Testing and tuning hook; no counterpart in the reference. Forces the tile shape (bm_tiles 1|2 =
 * 128|256 rows, bn 128|256 columns, bn 512 = the CTA-pair kernel) and the split count of the contraction
 * for the calling thread's next nf4ll_forward / nf4ll_backward_dx calls; zeros restore the built-in
 * heuristic. flags bit 0: never use the cooperative split reduction (the splits of a tile then leave the
 * sum to whichever of them finishes last), e.g. under a profiler that replays kernels one at a time.
 * flags bit 1: run a forward of at most 64 rows on the register-level weight-streaming kernel (default: up to
 * 16 rows); flags bit 2: run a forward of at most 64 rows on the swapped-operand tensor-core kernel (default:
 * 9 to 32 rows against weights of at least 2^24 elements, 33 to 64 rows against at least 2^26). With bit 1 or 2, `splits` forces that kernel's
 * number of slices of the contraction. Size the workspace of such calls with nf4ll_workspace_bytes_tuned. */
void nf4ll_tune_override(int32_t bm_tiles, int32_t bn, int32_t splits, int32_t flags);

/* Measurement hook; no counterpart in the reference. The calling thread's NEXT nf4ll_forward /
 * nf4ll_backward_dx / nf4ll_forward_gate_up records the CUDA events `start` / `stop` (cudaEvent_t as
 * void*) right before / after the kernel that computes its product on the call's stream, leaving the
 * small rank-16 prologue kernel outside the pair. One-shot: the pair is forgotten after that call. On a stream
 * that is being captured the records become nodes of the graph (recorded, and timeable, at every replay). */
void nf4ll_kernel_events(void* start, void* stop);

/* Measurement hook; no counterpart in the reference. Number of kernels the calling thread has launched
 * through this library so far (memsets and event records are not kernels). Benchmarks take the difference
 * across one step to report how many of the library's kernels a step consists of. */
int64_t nf4ll_launch_count(void);

/* Failure-detection test hook; no counterpart in the reference. The calling thread's NEXT call whose
 * contraction is split with the cooperative reduction is launched one split short and with a limit of
 * `polls` polls (instead of 2^22) on the wait for a tile's other splits. Nothing ever completes those
 * tiles' counters, so every CTA's wait runs out: each one records NF4LL_ERR_DEVICE_WAIT's cause in the
 * status word, releases its tensor memory and returns; the call's output is undefined, the context stays
 * usable and later calls are unaffected (the tile counters are cleared before every use). One-shot;
 * ignored by calls that do not split cooperatively. */
void nf4ll_test_expire_wait(uint32_t polls);

#ifdef __cplusplus
}
#endif
#endif /* NF4LL_H_ */
