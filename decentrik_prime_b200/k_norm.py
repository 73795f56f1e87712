"""Fused residual add + RMSNorm around the NF4 + LoRA projections: same role, argument names and meaning as the
reference's solution/k_norm.py (`rms_forward`, `rms_backward`), so a layer loop written against that module reads
the same here. The kernels are hand-written sm_100a CUDA behind the C ABI (include/nf4ll.h); there is no Triton
and no CPU fallback.

Where the reference's forward writes the dropped-out copies xq / xv ([M, D] fp16) for the LoRA-A GEMMs that
follow (solution/fast_qwen.py:943-944), this one takes the lora_A shadows (`aq`, `av`) and writes the rank-16
products tq / tv ([M, 16] fp32) directly: hand them to linear.forward_multi as ready-made. Where the reference's
backward takes the [M, D] LoRA input gradients lq / lv (solution/fast_qwen.py:1376-1380), this one takes the
rank-16 factors uq / uv ([M, 16] fp32 = scale * d(out) . lora_B) with `aq`, `av` and expands them per element.
"""

import ctypes

import torch

from . import _lib


def _branch(A16, mask, keep_scale):
    if A16 is None:
        return None, None
    if A16.dtype != torch.float16 or not A16.is_contiguous() or A16.shape[0] != 16:
        raise ValueError("lora_A shadow must be contiguous fp16 [16, D]")
    if mask is not None and (mask.dtype not in (torch.uint8, torch.bool) or mask.stride(-1) != 1):
        raise ValueError("mask must be uint8/bool with unit inner stride")
    s = _lib.LoraArgs(A16.data_ptr(), 0, 16, 1.0, 0 if mask is None else mask.data_ptr(),
                      0 if mask is None else mask.stride(0), float(keep_scale), 0)
    return s, ctypes.byref(s)


def _f32(t, shape, what):
    if t.dtype != torch.float32 or tuple(t.shape) != tuple(shape) or not t.is_contiguous() or not t.is_cuda:
        raise ValueError(f"{what} must be a contiguous CUDA fp32 tensor {tuple(shape)}")


def rms_forward(x, w, y, rstd, eps, *, delta=None, xout=None, aq=None, av=None, tq=None, tv=None, mq=None, mv=None,
                keep_scale=1.0):
    """x fp32 [n, d] (+ delta fp16) -> xout fp32 (optional), y fp16 (optional, may be a column slice), rstd fp32 [n],
    tq / tv fp32 [n, 16] = fp16(dropout_{q,v}(norm output)) . {aq, av}^T. Reference: solution/k_norm.py:99-115."""
    n, d = x.shape
    _f32(x, (n, d), "x")
    _f32(w, (d,), "w")
    _f32(rstd, (n,), "rstd")
    if xout is not None:
        _f32(xout, (n, d), "xout")
    if delta is not None and (delta.dtype != torch.float16 or tuple(delta.shape) != (n, d) or not delta.is_contiguous()):
        raise ValueError("delta must be contiguous fp16 [n, d]")
    if y is not None and (y.dtype != torch.float16 or tuple(y.shape) != (n, d) or y.stride(1) != 1):
        raise ValueError("y must be fp16 [n, d] with unit inner stride")
    for A, t, m, name in ((aq, tq, mq, "q"), (av, tv, mv, "v")):
        if (A is None) != (t is None):
            raise ValueError(f"the {name} branch needs both its lora_A shadow and its [n, 16] output")
        if t is not None:
            _f32(t, (n, 16), f"t{name}")
        if m is not None and A is None:
            raise ValueError("a dropout mask without its LoRA branch has no meaning")
    ka, ra = _branch(aq, mq, keep_scale)
    kb, rb = _branch(av, mv, keep_scale)
    _lib.check(_lib.lib().nf4ll_rms_forward(
        x.data_ptr(), None if delta is None else delta.data_ptr(), None if xout is None else xout.data_ptr(), w.data_ptr(),
        float(eps), n, d, None if y is None else y.data_ptr(), 0 if y is None else y.stride(0), rstd.data_ptr(),
        ra, None if tq is None else tq.data_ptr(), rb, None if tv is None else tv.data_ptr(), _lib.current_stream(x.device)))
    del ka, kb


def rms_backward(dy16, gscale, x, w, rstd, out, *, dres=None, uq=None, uv=None, aq=None, av=None, mq=None, mv=None,
                 keep_scale=1.0, out16=None, delta=None):
    """out (fp32, may alias dres) = dres + d(norm input); out16 = its fp16 copy. dy16 is the fp16 gradient of the
    norm output from the projections' backward-dX (run WITHOUT their LoRA branch); uq / uv with aq / av and the
    keep-masks add the LoRA branches' input gradients. Reference: solution/k_norm.py:118-131."""
    n, d = x.shape
    _f32(x, (n, d), "x")
    _f32(w, (d,), "w")
    _f32(rstd, (n,), "rstd")
    _f32(out, (n, d), "out")
    if dres is not None:
        _f32(dres, (n, d), "dres")
    if dy16.dtype != torch.float16 or tuple(dy16.shape) != (n, d) or dy16.stride(1) != 1:
        raise ValueError("dy16 must be fp16 [n, d] with unit inner stride")
    if out16 is not None and (out16.dtype != torch.float16 or tuple(out16.shape) != (n, d) or not out16.is_contiguous()):
        raise ValueError("out16 must be contiguous fp16 [n, d]")
    for A, u, name in ((aq, uq, "q"), (av, uv, "v")):
        if (A is None) != (u is None):
            raise ValueError(f"the {name} branch needs both its lora_A shadow and its [n, 16] factor")
        if u is not None:
            _f32(u, (n, 16), f"u{name}")
    ka, ra = _branch(aq, mq, keep_scale)
    kb, rb = _branch(av, mv, keep_scale)
    g = float(gscale.item()) if isinstance(gscale, torch.Tensor) else float(gscale)
    _lib.check(_lib.lib().nf4ll_rms_backward(
        dy16.data_ptr(), dy16.stride(0), g, x.data_ptr(), None if delta is None else delta.data_ptr(), w.data_ptr(),
        rstd.data_ptr(), None if dres is None else dres.data_ptr(), out.data_ptr(), None if out16 is None else out16.data_ptr(),
        n, d, ra, None if uq is None else uq.data_ptr(), rb, None if uv is None else uv.data_ptr(), _lib.current_stream(x.device)))
    del ka, kb
