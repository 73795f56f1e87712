"""CPU oracle for the NF4 + LoRA linear path. TEST INFRASTRUCTURE, NOT A PRODUCT PATH.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this module; the
package decentrik_prime_b200 never does (its kernels fail loudly without the CUDA library).

A restatement, in NumPy / CPU PyTorch, of the reference's arithmetic for the path:

* dequantisation   - solution/k_nf4.py:16-21 (format), 40-57 (kernel); the NumPy statement of the
                     same semantics in dev/test_emu.py:49-55.
* forward          - solution/fast_qwen.py:943-947 (LoRA GEMMs, base addmm), solution/k_norm.py:46-53
                     (dropout on the LoRA input, then the fp16 cast), solution/k_rope.py:39-45, 56-58
                     (LoRA add with the scale), solution/fast_qwen.py:93, 370 (scale, keep_scale).
* backward         - solution/fast_qwen.py:1310-1377 (dX GEMMs, dA/dB, LoRA dX terms),
                     solution/k_norm.py:64-71 (masked add of the LoRA dX term).

Parity pin: `dequant_ref` is checked bit-for-bit against the reference's own kernel body executed
under the reference's NumPy emulator (tests/golden/make_golden.py generated the committed vectors
by importing solution/k_nf4.py and dev/tl_emu.py). The quantise direction belongs to bitsandbytes,
which is absent: it is not restated here (parity unpinned for that direction; the generator in
decentrik_prime_b200/quantize.py only has to emit valid bytes). The GEMM + LoRA stage has no golden
vectors in the reference (it is pinned there only end to end on a real model): for it the contract
is the tolerance against O1 below.

Two variants:
  O1 `lora_linear_o1`  fp32/fp64-accumulated, unrounded rank-16 intermediates: the grading oracle
                       (max-abs-err <= 2e-2, rel-L2 <= 1e-3).
  O2 `lora_linear_o2`  mirrors every fp16 rounding the reference makes (fp16 GEMM outputs, fp16
                       T/U, fp16 dA/dB before the fp32 cast): what the reference itself computes,
                       and the CPU path that bench.py times.
"""

import numpy as np
import torch

# The 16 NF4 levels (reference solution/k_nf4.py:29-34).
NF4_LEVELS = np.array([
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
    -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
    0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
    0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0], dtype=np.float32)


def absmax_ref(qabs, scale2, offset2, code2):
    """fp32 absmax of every quantisation block: code2[q] * scale2 + offset2, product and sum
    rounded separately (reference solution/k_nf4.py:47-49, launched with fp fusion off, 180)."""
    qabs = np.asarray(qabs, dtype=np.uint8).reshape(-1)
    g = np.arange(qabs.size) // 256
    prod = (np.asarray(code2, dtype=np.float32)[qabs] * np.asarray(scale2, dtype=np.float32)[g]).astype(np.float32)
    return (prod + np.asarray(offset2, dtype=np.float32)[g]).astype(np.float32)


def dequant_ref(packed, qabs, scale2, offset2, code2):
    """NF4 -> fp16, bit-exact restatement (reference solution/k_nf4.py:50-57, dev/test_emu.py:49-55):
    even element from the high nibble, fp32 product rounded to nearest-even fp16."""
    packed = np.asarray(packed, dtype=np.uint8).reshape(-1)
    absmax = absmax_ref(qabs, scale2, offset2, code2)
    per_byte = np.repeat(absmax, 32)
    out = np.empty(packed.size * 2, dtype=np.float16)
    out[0::2] = (NF4_LEVELS[packed >> 4] * per_byte).astype(np.float32).astype(np.float16)
    out[1::2] = (NF4_LEVELS[packed & 15] * per_byte).astype(np.float32).astype(np.float16)
    return out


def dequant_weight(layer, name, code2):
    """fp16 torch matrix [rows, cols] of one weight of a PackedLayer-like object (CPU tensors or
    anything with .cpu())."""
    pk, qa, s2, o2, rows, cols = layer.weight(name)
    w = dequant_ref(pk.cpu().numpy(), qa.cpu().numpy(), s2.cpu().numpy(), o2.cpu().numpy(),
                    code2.cpu().numpy())
    return torch.from_numpy(w).reshape(rows, cols)


def drop_ref(x16, mask, keep_scale):
    """LoRA input after dropout: fp16(x * keep_scale) where kept, 0 elsewhere (reference
    solution/k_norm.py:49-53; there x is the fp32 norm output, here the op's fp16 input)."""
    if mask is None:
        return x16
    return torch.where(mask.bool(), x16.float() * np.float32(keep_scale), torch.zeros((), dtype=torch.float32)).half()


def lora_linear_o1(w16, x16, dy16=None, bias16=None, A16=None, B16=None, scale=1.0, mask=None,
                   keep_scale=1.0, dtype=torch.float64):
    """Grading oracle: everything accumulated in `dtype` (fp64 by default), intermediates unrounded.
    Returns a dict with y (and dx, dA, dB, t, u when dy16 is given); y/dx are NOT rounded to fp16."""
    W = w16.to(dtype)
    X = x16.to(dtype)
    out = {}
    y = X @ W.t()
    if bias16 is not None:
        y = y + bias16.to(dtype)
    lora = A16 is not None
    if lora:
        A, B = A16.to(dtype), B16.to(dtype)
        xd = drop_ref(x16, mask, keep_scale).to(dtype)
        t = xd @ A.t()
        y = y + scale * (t @ B.t())
        out["t"] = t
    out["y"] = y
    if dy16 is not None:
        G = dy16.to(dtype)
        dx = G @ W
        if lora:
            u = scale * (G @ B)
            lx = u @ A
            if mask is not None:
                lx = lx * mask.to(dtype) * float(np.float32(keep_scale))
            dx = dx + lx
            out["u"] = u
            out["dA"] = u.t() @ xd
            out["dB"] = scale * (G.t() @ t)
        out["dx"] = dx
    return out


def lora_linear_o2(w16, x16, dy16=None, bias16=None, A16=None, B16=None, scale=1.0, mask=None,
                   keep_scale=1.0, mm_dtype=torch.float32):
    """Reference semantics: every GEMM output rounded to fp16 where the reference's is
    (solution/fast_qwen.py:943-947, 1369-1377; k_rope.py:39-45; k_norm.py:64-71). GEMMs run in
    `mm_dtype` on the CPU (fp32 accumulate, like cuBLAS) and are rounded afterwards."""
    def mm16(a, b):
        return (a.to(mm_dtype) @ b.to(mm_dtype)).half()

    out = {}
    lora = A16 is not None
    if bias16 is not None:
        y16 = (x16.to(mm_dtype) @ w16.to(mm_dtype).t() + bias16.to(mm_dtype)).half()   # addmm
    else:
        y16 = mm16(x16, w16.t())
    if lora:
        xd = drop_ref(x16, mask, keep_scale)
        t16 = mm16(xd, A16.t())
        l16 = mm16(t16, B16.t())
        y16 = (y16.float() + np.float32(scale) * l16.float()).half()
        out["t"] = t16
    out["y"] = y16
    if dy16 is not None:
        dx16 = mm16(dy16, w16)
        if lora:
            dB = mm16(dy16.t(), t16).float() * np.float32(scale)
            u16 = (mm16(dy16, B16).float() * np.float32(scale)).half()     # fp16 mul_
            dA = mm16(u16.t(), xd).float()
            lx16 = mm16(u16, A16)
            lx = lx16.float()
            if mask is not None:
                lx = torch.where(mask.bool(), lx * np.float32(keep_scale), torch.zeros(()))
            out.update(u=u16, dA=dA, dB=dB)
            out["dx"] = (dx16.float() + lx)          # summed in fp32 inside the norm backward
        else:
            out["dx"] = dx16.float()
    return out


def errors(got, ref):
    """(max-abs-err, rel-L2) of `got` against `ref`, both computed in fp64."""
    g, r = got.detach().cpu().double(), ref.detach().cpu().double()
    diff = (g - r)
    return diff.abs().max().item(), (diff.norm() / r.norm().clamp_min(1e-300)).item()
