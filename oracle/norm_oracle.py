"""CPU oracle for the fused residual add + RMSNorm producer and its backward. TEST INFRASTRUCTURE, NOT A
PRODUCT PATH (only tests/ and the checker legs of bench.py / __graft_entry__ may import it).

A NumPy restatement of the reference's two Triton kernels, operation for operation in fp32:

* forward   solution/k_norm.py:29-53 (`rms_fwd_kernel`): x = x_prev (+ delta); rstd = rsqrt(mean(x^2) + eps);
            y = w * (x * rstd); y16 = fp16(y); xq16 = fp16(keep_q ? y * keep_scale : 0), same for v.
* backward  solution/k_norm.py:56-87 (`rms_bwd_kernel`): dy = fp16 grad * gscale (+ masked, scaled LoRA input
            grads lq, lv); dx = rstd * (w*dy - xhat * mean(w*dy*xhat)) (+ dres); fp16 copy of the result.

Parity pin: tests/golden/norm_golden.npz holds inputs and outputs of the reference's own kernels executed under
the reference's NumPy emulator (tests/golden/make_norm_golden.py); tests/test_oracle_golden.py holds these
functions to them.

What the CUDA kernels add on top (rank-16 products formed inside the kernels instead of [M, D] round trips):
  T  = xq16 . A^T           (reference solution/fast_qwen.py:943-944 on the kernel's xq / xv outputs)
  lq = u . A                (reference solution/fast_qwen.py:1376-1377, there rounded to fp16; here unrounded)
"""

import numpy as np

f32 = np.float32


def rms_forward_ref(x, w, eps, delta=None, mq=None, mv=None, keep_scale=1.0):
    """dict(xout fp32, rstd fp32, y16 fp16, xq16 / xv16 fp16 when the masks are given)."""
    x = np.asarray(x, dtype=f32)
    if delta is not None:
        x = x + np.asarray(delta, dtype=np.float16).astype(f32)
    d = x.shape[1]
    ms = np.sum(x * x, axis=1, dtype=f32) * f32(1.0 / d)
    r = (f32(1.0) / np.sqrt(ms + f32(eps))).astype(f32)
    y = np.asarray(w, dtype=f32)[None, :] * (x * r[:, None])
    out = {"xout": x, "rstd": r, "y32": y, "y16": y.astype(np.float16)}
    for name, m in (("xq16", mq), ("xv16", mv)):
        if m is not None:
            out[name] = np.where(np.asarray(m) != 0, y * f32(keep_scale), f32(0.0)).astype(np.float16)
    return out


def rms_backward_ref(dy16, gscale, x, w, rstd, delta=None, dres=None, lq=None, lv=None, mq=None, mv=None,
                     keep_scale=1.0):
    """(out fp32, out16 fp16). lq / lv: the LoRA-A input gradients [M, D] in any float dtype (the reference
    passes fp16 GEMM outputs); they are used in fp32, as the kernel does after its cast."""
    dy = np.asarray(dy16, dtype=np.float16).astype(f32) * f32(gscale)
    for l, m in ((lq, mq), (lv, mv)):
        if l is not None:
            dy = dy + np.where(np.asarray(m) != 0, np.asarray(l).astype(f32) * f32(keep_scale), f32(0.0))
    x = np.asarray(x, dtype=f32)
    if delta is not None:
        x = x + np.asarray(delta, dtype=np.float16).astype(f32)
    d = x.shape[1]
    r = np.asarray(rstd, dtype=f32)
    xh = x * r[:, None]
    g = dy * np.asarray(w, dtype=f32)[None, :]
    c = np.sum(g * xh, axis=1, dtype=f32) * f32(1.0 / d)
    dx = (g - xh * c[:, None]) * r[:, None]
    if dres is not None:
        dx = dx + np.asarray(dres, dtype=f32)
    dx = dx.astype(f32)
    return dx, dx.astype(np.float16)
