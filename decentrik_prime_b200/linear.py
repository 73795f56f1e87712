"""The NF4 + LoRA linear as Python calls: raw forward / backward_dx / lora_grads for a hand-written
backward (the reference's model is one autograd node with its own backward,
solution/fast_qwen.py:1527-1543) and `nf4_lora_linear`, a torch.autograd.Function for ordinary
modules. All compute happens in libnf4ll.so (include/nf4ll.h); PyTorch only owns the memory and
the streams. Tensors must be CUDA tensors: nothing here runs on the CPU.

Call-site mapping to the reference (solution/fast_qwen.py):
  forward      <- _ws_use + torch.mm/addmm on the fp16 workspace (947, 1037, 1080-1098, 1112) and the
                  LoRA GEMMs + add (943-946; k_rope.py:39-45, 56-58)
  backward_dx  <- torch.mm(dy, W) (1310, 1320-1327, 1350, 1364), `daq`/`lqx` (1370-1377) and the
                  masked add in k_norm.py:64-71
  lora_grads   <- d_bq / d_aq / d_bv / d_av (1369-1374)
"""

import contextlib
import ctypes
import threading

import torch

from . import _lib
from .k_nf4 import PackedLayer

RANK = 16


class Nf4Weight:
    """One NF4 weight W[N, K] on the GPU: views into a PackedLayer's sections plus the shared
    second-level code table."""

    def __init__(self, packed, qabs, scale2, offset2, code2, rows, cols):
        for t in (packed, qabs, scale2, offset2, code2):
            if not t.is_cuda:
                raise ValueError("NF4 weights must live on the GPU")
        if code2.dtype != torch.float32 or code2.numel() != 256:
            raise ValueError("code2 must be 256 fp32 entries")
        self.packed, self.qabs, self.scale2, self.offset2, self.code2 = packed, qabs, scale2, offset2, code2
        self.N, self.K = int(rows), int(cols)
        self.device = packed.device
        self._c = _lib.Nf4Mat(packed.data_ptr(), qabs.data_ptr(), scale2.data_ptr(), offset2.data_ptr(),
                              code2.data_ptr(), self.N, self.K)

    @classmethod
    def from_layer(cls, layer: PackedLayer, name, code2):
        return cls(*layer.weight(name)[:4], code2, *layer.weight(name)[4:])

    @classmethod
    def from_layer_group(cls, layer: PackedLayer, names, code2):
        """Several consecutive weights of a layer as one stacked matrix (for forward_multi); the rows
        of each are kept in `.rows_each`."""
        packed, qabs, scale2, offset2, rows, cols, rows_each = layer.weight_group(names)
        w = cls(packed, qabs, scale2, offset2, code2, rows, cols)
        w.rows_each = list(rows_each)
        return w

    @property
    def nbytes(self):
        """Algorithmic bytes of the weight stream: nibbles + absmax codes + scale2 + offset2."""
        n = self.N * self.K
        return n // 2 + n // 64 + 2 * 4 * (n // 16384)


class _DeviceState(threading.local):
    def __init__(self):
        self.ws = {}
        self.status = {}
        self.tune = (0, 0, 0)


_state = _DeviceState()


def _workspace_need(M, N, K, r):
    if any(_state.tune):
        return _lib.lib().nf4ll_workspace_bytes_tuned(M, N, K, r, *_state.tune)
    return _lib.lib().nf4ll_workspace_bytes(M, N, K, r)


@contextlib.contextmanager
def tune_override(bm_tiles=0, bn=0, splits=0, flags=0):
    """Testing / tuning hook: force the tile shape (bm_tiles 1|2, bn 128|256, 512 = CTA-pair kernel) and the
    split count for this thread's calls inside the block; flags bit 0 keeps split contractions off the
    cooperative reduction. Workspaces allocated inside the block are sized for the forced plan."""
    h = _lib.lib()
    h.nf4ll_tune_override(bm_tiles, bn, splits, flags)
    _state.tune = (bm_tiles, bn, splits)
    try:
        yield
    finally:
        h.nf4ll_tune_override(0, 0, 0, 0)
        _state.tune = (0, 0, 0)


def _workspace(device, nbytes):
    """Per-thread, per-device scratch that grows on demand (the library never allocates). Calls on
    different streams of the same thread must not overlap while sharing it; pass `workspace=` to
    forward / backward_dx to use separate buffers."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _state.ws.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _state.ws[key] = ws
    return ws


def status_word(device):
    """The device status word kernels write when a bounded wait expires (zero = healthy)."""
    st = _state.status.get(device.index)
    if st is None:
        st = torch.zeros(1, dtype=torch.int32, device=device)
        _state.status[device.index] = st
    return st


def check_status(device=None):
    """Synchronise the current stream and raise if any kernel reported an expired wait."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    st = status_word(device)
    _lib.check(_lib.lib().nf4ll_read_status(st.data_ptr(), _lib.current_stream(device)))


def _lora_struct(lora, mask, keep_scale):
    if lora is None:
        return None, None
    A16, B16, scale = lora[:3]
    Bt = lora[3] if len(lora) > 3 else None
    if Bt is not None and (Bt.dtype != torch.float16 or not Bt.is_contiguous() or Bt.shape != (A16.shape[0], B16.shape[0])):
        raise ValueError("transposed lora_B shadow must be contiguous fp16 [16, N]")
    if A16.dtype != torch.float16 or B16.dtype != torch.float16:
        raise ValueError("LoRA shadows must be fp16")
    if not (A16.is_contiguous() and B16.is_contiguous()):
        raise ValueError("LoRA A/B must be contiguous")
    if mask is not None:
        if mask.dtype not in (torch.uint8, torch.bool) or mask.stride(-1) != 1:
            raise ValueError("mask must be uint8/bool with unit inner stride")
    s = _lib.LoraArgs(A16.data_ptr(), B16.data_ptr(), int(A16.shape[0]), float(scale),
                      0 if mask is None else mask.data_ptr(), 0 if mask is None else mask.stride(0),
                      float(keep_scale), 0 if Bt is None else Bt.data_ptr())
    return s, ctypes.byref(s)


def _check_act(t, cols, what):
    if t.dtype != torch.float16 or t.dim() != 2 or t.shape[1] != cols or t.stride(1) != 1 or not t.is_cuda:
        raise ValueError(f"{what} must be a CUDA fp16 matrix [M, {cols}] with unit inner stride")


def forward(w: Nf4Weight, x, bias=None, lora=None, mask=None, keep_scale=1.0, out=None, want_t=False,
            workspace=None):
    """y = x . W^T (+ bias) + scale * (drop(x) . A^T) . B^T. `lora` = (A16 [16,K], B16 [N,16], scale) or
    (A16, B16, scale, B16t [16,N]) when the caller keeps a transposed shadow of lora_B for the backward.
    Returns (y, t) with t = drop(x) . A^T in fp32 [M,16] when want_t, else None."""
    _check_act(x, w.K, "x")
    M = x.shape[0]
    y = torch.empty(M, w.N, dtype=torch.float16, device=x.device) if out is None else out
    _check_act(y, w.N, "out")
    if mask is not None and lora is None:
        raise ValueError("a dropout mask without a LoRA branch has no meaning")
    keep, ref = _lora_struct(lora, mask, keep_scale)
    t = torch.empty(M, RANK, dtype=torch.float32, device=x.device) if (want_t and lora is not None) else None
    h = _lib.lib()
    ws = _workspace(x.device, _workspace_need(M, w.N, w.K, RANK if lora is not None else 0)) if workspace is None else workspace
    _lib.check(h.nf4ll_forward(ctypes.byref(w._c), x.data_ptr(), x.stride(0),
                               None if bias is None else bias.data_ptr(), ref,
                               None if t is None else t.data_ptr(), M, y.data_ptr(), y.stride(0),
                               ws.data_ptr(), ws.numel(), status_word(x.device).data_ptr(),
                               _lib.current_stream(x.device)))
    del keep
    return y, t


def forward_multi(w: Nf4Weight, x, segments, bias=None, out=None, workspace=None):
    """One launch for several projections that share x and are stacked row-wise in `w` (Q|K|V,
    gate|up; the reference's fused W_qkv GEMM, solution/fast_qwen.py:405-413, 947).
    `segments`: one (rows, lora, mask, keep_scale) per projection, lora as in forward() or None; a fifth element,
    when given, is the projection's ready-made rank-16 product t fp32 [M,16] (k_norm.rms_forward wrote it while
    producing x), which the call then reads instead of computing.
    Returns (y [M, sum rows], [t per segment or None])."""
    _check_act(x, w.K, "x")
    M = x.shape[0]
    y = torch.empty(M, w.N, dtype=torch.float16, device=x.device) if out is None else out
    _check_act(y, w.N, "out")
    keep, ts = [], []
    arr = (_lib.Segment * len(segments))()
    for i, seg in enumerate(segments):
        rows, lora, mask, keep_scale = seg[:4]
        given = seg[4] if len(seg) > 4 else None
        if mask is not None and lora is None:
            raise ValueError("a dropout mask without a LoRA branch has no meaning")
        if given is not None and (lora is None or given.dtype != torch.float32 or tuple(given.shape) != (M, RANK)
                                  or not given.is_contiguous()):
            raise ValueError("a ready-made rank-16 product must be contiguous fp32 [M, 16] and needs its LoRA branch")
        s, ref = _lora_struct(lora, mask, keep_scale)
        t = given if given is not None else (torch.empty(M, RANK, dtype=torch.float32, device=x.device) if lora is not None else None)
        keep.append(s)
        ts.append(t)
        arr[i].rows = int(rows)
        arr[i].lora = ctypes.pointer(s) if s is not None else None
        arr[i].t_out = None if t is None else t.data_ptr()
        arr[i].t_ready = 1 if given is not None else 0
    h = _lib.lib()
    ws = _workspace(x.device, _workspace_need(M, w.N, w.K, 0)) if workspace is None else workspace
    _lib.check(h.nf4ll_forward_multi(ctypes.byref(w._c), x.data_ptr(), x.stride(0),
                                     None if bias is None else bias.data_ptr(), arr, len(segments), M,
                                     y.data_ptr(), y.stride(0), ws.data_ptr(), ws.numel(),
                                     status_word(x.device).data_ptr(), _lib.current_stream(x.device)))
    del keep
    return y, ts


def forward_gate_up(w: Nf4Weight, x, lora_gate=None, mask_gate=None, lora_up=None, mask_up=None, keep_scale=1.0,
                    workspace=None):
    """(g, u, h, t_gate, t_up) of an MLP's first half in one launch: `w` is gate_proj and up_proj stacked
    ([2I, K], Nf4Weight.from_layer_group), h = silu(g) * u is formed in the kernel's epilogue (reference:
    two GEMMs + gated_silu, solution/fast_qwen.py:1080-1108). g and u are views of one [M, 2I] buffer."""
    _check_act(x, w.K, "x")
    M, I = x.shape[0], w.N // 2
    gu = torch.empty(M, 2 * I, dtype=torch.float16, device=x.device)
    g, u = gu[:, :I], gu[:, I:]
    h = torch.empty(M, I, dtype=torch.float16, device=x.device)
    sg, rg = _lora_struct(lora_gate, mask_gate, keep_scale)
    su, ru = _lora_struct(lora_up, mask_up, keep_scale)
    tg = torch.empty(M, RANK, dtype=torch.float32, device=x.device) if lora_gate is not None else None
    tu = torch.empty(M, RANK, dtype=torch.float32, device=x.device) if lora_up is not None else None
    r = RANK if (lora_gate is not None or lora_up is not None) else 0
    ws = _workspace(x.device, _workspace_need(M, I, w.K, r)) if workspace is None else workspace
    _lib.check(_lib.lib().nf4ll_forward_gate_up(ctypes.byref(w._c), x.data_ptr(), x.stride(0), rg, ru,
                                                None if tg is None else tg.data_ptr(), None if tu is None else tu.data_ptr(),
                                                M, g.data_ptr(), g.stride(0), u.data_ptr(), u.stride(0), h.data_ptr(),
                                                h.stride(0), ws.data_ptr(), ws.numel(), status_word(x.device).data_ptr(),
                                                _lib.current_stream(x.device)))
    del sg, su
    return g, u, h, tg, tu


def backward_dx(w: Nf4Weight, dy, lora=None, mask=None, keep_scale=1.0, out=None, accumulate=False,
                want_u=False, workspace=None):
    """dx (+)= dy . W + keep_scale * mask (.) ((scale * dy . B) . A). Returns (dx, u) with
    u = scale * dy . B in fp32 [M,16] when want_u, else None."""
    _check_act(dy, w.N, "dy")
    M = dy.shape[0]
    if out is None:
        if accumulate:
            raise ValueError("accumulate needs an existing dx")
        out = torch.empty(M, w.K, dtype=torch.float16, device=dy.device)
    _check_act(out, w.K, "dx")
    keep, ref = _lora_struct(lora, mask, keep_scale)
    u = torch.empty(M, RANK, dtype=torch.float32, device=dy.device) if (want_u and lora is not None) else None
    h = _lib.lib()
    ws = _workspace(dy.device, _workspace_need(M, w.N, w.K, RANK if lora is not None else 0)) if workspace is None else workspace
    _lib.check(h.nf4ll_backward_dx(ctypes.byref(w._c), dy.data_ptr(), dy.stride(0), ref,
                                   None if u is None else u.data_ptr(), M, out.data_ptr(), out.stride(0),
                                   1 if accumulate else 0, ws.data_ptr(), ws.numel(),
                                   status_word(dy.device).data_ptr(), _lib.current_stream(dy.device)))
    del keep
    return out, u


def lora_grads(dy, x, t, u, scale, mask=None, keep_scale=1.0, dA=None, dB=None, accumulate=False):
    """dA[16,K] (+)= u^T . drop(x), dB[N,16] (+)= scale * dy^T . t, both fp32. dA / dB may be views
    into a flat gradient bucket; missing ones are allocated (zero-initialised by the call)."""
    M, K = x.shape
    N = dy.shape[1]
    _check_act(x, K, "x")
    _check_act(dy, N, "dy")
    if dA is None:
        dA = torch.empty(RANK, K, dtype=torch.float32, device=x.device)
        accumulate_a = False
    else:
        accumulate_a = accumulate
    if dB is None:
        dB = torch.empty(N, RANK, dtype=torch.float32, device=x.device)
        accumulate_b = False
    else:
        accumulate_b = accumulate
    for g in (dA, dB):
        if g.dtype != torch.float32 or not g.is_contiguous():
            raise ValueError("dA/dB must be contiguous fp32")
    h = _lib.lib()
    stream = _lib.current_stream(x.device)
    args = (dy.data_ptr(), dy.stride(0), x.data_ptr(), x.stride(0),
            None if mask is None else mask.data_ptr(), 0 if mask is None else mask.stride(0),
            float(keep_scale), t.data_ptr(), u.data_ptr(), float(scale), RANK, M, N, K)
    if accumulate_a == accumulate_b:
        _lib.check(h.nf4ll_lora_grads(*args, dA.data_ptr(), dB.data_ptr(), int(accumulate_a), stream))
    else:
        _lib.check(h.nf4ll_lora_grads(*args, dA.data_ptr(), None, int(accumulate_a), stream))
        _lib.check(h.nf4ll_lora_grads(*args, None, dB.data_ptr(), int(accumulate_b), stream))
    return dA, dB


def lora_u(dy, B16t, scale):
    """u fp32 [M,16] = scale * dy . B, the rank-16 factor of the LoRA branch's backward (reference
    solution/fast_qwen.py:1370, 1373 `daq`, `dav`), from the transposed fp16 shadow B16t [16, N]."""
    M, N = dy.shape
    _check_act(dy, N, "dy")
    if B16t.dtype != torch.float16 or tuple(B16t.shape) != (RANK, N) or not B16t.is_contiguous():
        raise ValueError("lora_B transposed shadow must be contiguous fp16 [16, N]")
    u = torch.empty(M, RANK, dtype=torch.float32, device=dy.device)
    _lib.check(_lib.lib().nf4ll_lora_down(dy.data_ptr(), dy.stride(0), None, 0, 1.0, B16t.data_ptr(), 1.0, RANK, M, N,
                                          u.data_ptr(), None, _lib.current_stream(dy.device)))
    return u.mul_(scale)


class _Nf4LoraLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, A, B, w, bias, scale, mask, keep_scale):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        lora = None
        if A is not None:
            lora = (A.detach().half().contiguous(), B.detach().half().contiguous(), scale)
        m2 = None if mask is None else mask.reshape(-1, mask.shape[-1])
        y, t = forward(w, x2, bias=bias, lora=lora, mask=m2, keep_scale=keep_scale, want_t=lora is not None)
        ctx.w, ctx.lora, ctx.mask, ctx.keep_scale, ctx.lead = w, lora, m2, keep_scale, lead
        ctx.save_for_backward(x2, t)
        ctx.need_x = x.requires_grad
        return y.reshape(*lead, w.N)

    @staticmethod
    def backward(ctx, dy):
        x2, t = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(1) != 1:
            dy2 = dy2.contiguous()
        dx, u = backward_dx(ctx.w, dy2, lora=ctx.lora, mask=ctx.mask, keep_scale=ctx.keep_scale,
                            want_u=ctx.lora is not None)
        dA = dB = None
        if ctx.lora is not None:
            dA, dB = lora_grads(dy2, x2, t, u, ctx.lora[2], mask=ctx.mask, keep_scale=ctx.keep_scale)
        return dx.reshape(*ctx.lead, ctx.w.K), dA, dB, None, None, None, None, None


def nf4_lora_linear(x, w: Nf4Weight, bias=None, lora=None, mask=None, keep_scale=1.0):
    """Differentiable y = NF4Linear(x) + LoRA(x). `lora` = (A fp32 [16,K], B fp32 [N,16], scale) with
    A and B ordinary parameters: they receive fp32 gradients; W is frozen (no dW)."""
    A, B, scale = (None, None, 1.0) if lora is None else lora
    return _Nf4LoraLinearFn.apply(x, A, B, w, bias, scale, mask, keep_scale)


def swiglu_forward(g, u, out=None):
    """h = fp16(silu(g) * u) in fp32 math (reference solution/k_mlp.py:21-29)."""
    M, I = g.shape
    _check_act(g, I, "g")
    _check_act(u, I, "u")
    h = torch.empty(M, I, dtype=torch.float16, device=g.device) if out is None else out
    _check_act(h, I, "h")
    _lib.check(_lib.lib().nf4ll_swiglu_forward(g.data_ptr(), g.stride(0), u.data_ptr(), u.stride(0), h.data_ptr(),
                                               h.stride(0), M, I, _lib.current_stream(g.device)))
    return h


def swiglu_backward(g, u, dh, inplace=True):
    """(dg, du) from dh; with inplace=True they overwrite g and u, as the reference overwrites its
    fused [gate | up] buffer (solution/k_mlp.py:32-47)."""
    M, I = g.shape
    for t, name in ((g, "g"), (u, "u"), (dh, "dh")):
        _check_act(t, I, name)
    dg = g if inplace else torch.empty_like(g)
    du = u if inplace else torch.empty_like(u)
    _lib.check(_lib.lib().nf4ll_swiglu_backward(g.data_ptr(), g.stride(0), u.data_ptr(), u.stride(0), dh.data_ptr(),
                                                dh.stride(0), dg.data_ptr(), dg.stride(0), du.data_ptr(), du.stride(0),
                                                M, I, _lib.current_stream(g.device)))
    return dg, du
