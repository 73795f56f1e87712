"""Projections and blocks built from the fused NF4 + LoRA linear, with a hand-written backward in
the style of the reference's layer loop (solution/fast_qwen.py:1017-1123 forward, 1232-1384
backward): activations are saved explicitly, dX flows through `backward_dx`, and the LoRA
gradients land, in fp32, in views of one flat bucket that a data-parallel run all-reduces once per
step (the reference returns them as a flat list, fast_qwen.py:1383, 1543).
"""

import math

import torch
import torch.nn.functional as F

from . import k_nf4, linear, quantize


class GradBucket:
    """One flat fp32 buffer for every LoRA gradient of a model; projections own views of it."""

    def __init__(self, numel, device):
        self.flat = torch.zeros(numel, dtype=torch.float32, device=device)
        self._at = 0

    def take(self, *shape):
        n = math.prod(shape)
        view = self.flat[self._at:self._at + n].view(*shape)
        self._at += n
        return view

    def zero_(self):
        self.flat.zero_()

    def all_reduce(self, group=None):
        """Sum over data-parallel ranks: the only exchange step of the path."""
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(self.flat, group=group)
        return self.flat


def lora_grad_numel(n_out, n_in, rank=linear.RANK):
    return rank * n_in + n_out * rank


class Projection:
    """One q/k/v/o/gate/up/down projection: frozen NF4 weight, optional fp16 bias, optional LoRA
    (fp32 master A [16,K], B [N,16] with fp16 shadows refreshed by `refresh16`, as the reference's
    `_refresh_lora16`, solution/fast_qwen.py:686-692)."""

    def __init__(self, weight: linear.Nf4Weight, bias=None, lora=False, alpha=32.0, bucket=None, seed=0,
                 b_std=0.01, lora_init=None):
        """`lora_init` = (A fp32 [16,K], B fp32 [N,16], scale): the masters of an existing adapter (they are
        used as they are, on the weight's device); otherwise `lora=True` draws seeded ones."""
        self.w, self.bias = weight, bias
        self.has_lora = bool(lora) or lora_init is not None
        self.scale = alpha / linear.RANK
        dev = weight.device
        if self.has_lora:
            if lora_init is not None:
                A, B, self.scale = lora_init
                if tuple(A.shape) != (linear.RANK, weight.K) or tuple(B.shape) != (weight.N, linear.RANK):
                    raise ValueError(f"LoRA factors {tuple(A.shape)}, {tuple(B.shape)} do not fit W[{weight.N},{weight.K}] at rank 16")
                self.A, self.B = A.detach().to(dev, torch.float32), B.detach().to(dev, torch.float32)
            else:
                gen = torch.Generator().manual_seed(seed)
                bound = 1.0 / math.sqrt(weight.K)          # kaiming_uniform(a=sqrt(5)), PEFT's lora_A init
                self.A = ((torch.rand(linear.RANK, weight.K, generator=gen) * 2 - 1) * bound).to(dev)
                self.B = (torch.randn(weight.N, linear.RANK, generator=gen) * b_std).to(dev)
            self.A16 = torch.empty_like(self.A, dtype=torch.float16)
            self.B16 = torch.empty_like(self.B, dtype=torch.float16)
            self.B16t = torch.empty(linear.RANK, weight.N, dtype=torch.float16, device=dev)
            self.refresh16()
            if bucket is not None:
                self.dA, self.dB = bucket.take(linear.RANK, weight.K), bucket.take(weight.N, linear.RANK)
            else:
                self.dA = torch.zeros(linear.RANK, weight.K, dtype=torch.float32, device=dev)
                self.dB = torch.zeros(weight.N, linear.RANK, dtype=torch.float32, device=dev)
        self._saved = None

    def refresh16(self):
        self.A16.copy_(self.A)
        self.B16.copy_(self.B)
        self.B16t.copy_(self.B.t())

    @property
    def lora(self):
        return (self.A16, self.B16, self.scale, self.B16t) if self.has_lora else None

    def flops(self, M):
        """Algorithmic FLOPs of forward + backward-dX (+ dA, dB): 4MNK + 6Mr(N+K)."""
        f = 4 * M * self.w.N * self.w.K
        if self.has_lora:
            f += 6 * M * linear.RANK * (self.w.N + self.w.K)
        return f

    def forward(self, x, mask=None, keep_scale=1.0, out=None, save=True):
        y, t = linear.forward(self.w, x, bias=self.bias, lora=self.lora, mask=mask if self.has_lora else None,
                              keep_scale=keep_scale, out=out, want_t=self.has_lora and save)
        if save:
            self._saved = (x, mask if self.has_lora else None, keep_scale, t)
        return y

    def backward(self, dy, out=None, accumulate=False, need_dx=True, accumulate_grads=False, grad_stream=None, pending=None):
        """dx (optionally accumulated into `out`) and, with LoRA, dA/dB into this projection's views.
        `grad_stream`: issue the dA/dB kernel there (after everything queued so far on the current stream), so
        that it runs beside the GEMMs that follow: nothing downstream of it in the backward reads dA/dB. The
        caller joins the stream again before the gradients are used and keeps `pending` (the tensors the side
        kernel reads) alive until then."""
        x, mask, keep_scale, t = self._saved
        dx = None
        u = None
        if need_dx:
            dx, u = linear.backward_dx(self.w, dy, lora=self.lora, mask=mask, keep_scale=keep_scale, out=out,
                                       accumulate=accumulate, want_u=self.has_lora)
        elif self.has_lora:
            # layer 0 of the reference needs no d(input), only LoRA gradients (fast_qwen.py:1363-1364)
            u = torch.empty(dy.shape[0], linear.RANK, dtype=torch.float32, device=dy.device)
            from . import _lib
            _lib.check(_lib.lib().nf4ll_lora_down(dy.data_ptr(), dy.stride(0), None, 0, 1.0, self.B16t.data_ptr(),
                                                  1.0, linear.RANK, dy.shape[0], self.w.N, u.data_ptr(), None,
                                                  _lib.current_stream(dy.device)))
            u.mul_(self.scale)
        if self.has_lora:
            if grad_stream is None:
                linear.lora_grads(dy, x, t, u, self.scale, mask=mask, keep_scale=keep_scale, dA=self.dA, dB=self.dB,
                                  accumulate=accumulate_grads)
            else:
                grad_stream.wait_stream(torch.cuda.current_stream(dy.device))
                with torch.cuda.stream(grad_stream):
                    linear.lora_grads(dy, x, t, u, self.scale, mask=mask, keep_scale=keep_scale, dA=self.dA, dB=self.dB,
                                      accumulate=accumulate_grads)
                if pending is not None:
                    pending.extend((dy, x, t, u, mask))
        self._saved = None
        return dx


def make_projection(n_out, n_in, seed, device, lora=False, bias=False, bucket=None, code2=None):
    """A projection with a seeded synthetic NF4 weight ~ N(0, 0.02) (benchmark configuration 0 construction)."""
    lin = quantize.random_nf4_weight(n_out, n_in, seed=seed, device=device, code2=code2)
    layer, c2 = k_nf4.repack_layer({"w": lin}, torch.device(device), names=("w",))
    w = linear.Nf4Weight.from_layer(layer, "w", c2)
    w._layer = layer          # keep the flat buffer alive
    b = None
    if bias:
        gen = torch.Generator().manual_seed(seed + 1)
        b = (torch.randn(n_out, generator=gen) * 0.1).half().to(device)
    return Projection(w, bias=b, lora=lora, bucket=bucket, seed=seed + 2)


class MlpBlock:
    """gate/up/down of one decoder layer with LoRA on every projection (benchmark configuration 1). The
    SiLU-gated product between up and down is either the library's fused kernel pair (the
    counterpart of the reference's gated_silu kernels) or plain PyTorch ops (fused_glue=False)."""

    def __init__(self, hidden, inter, seed, device, lora=True, bucket=None, fused_glue=True):
        self.hidden, self.inter = hidden, inter
        # fused_glue: the gated product comes out of the gate|up kernel's epilogue (short batches: the
        # library's stand-alone kernel, the counterpart of reference k_mlp.py); False: plain PyTorch ops
        self.fused_glue = fused_glue
        grad_lo = bucket._at if bucket is not None else 0
        # the three weights in one packed layer, gate and up row after row as in the reference's layout
        names = ("gate_proj", "up_proj", "down_proj")
        shapes = {"gate_proj": (inter, hidden), "up_proj": (inter, hidden), "down_proj": (hidden, inter)}
        lin = {n: quantize.random_nf4_weight(*shapes[n], seed=seed * 10 + 1 + i, device=device) for i, n in enumerate(names)}
        self.layer, self.code2 = k_nf4.repack_layer(lin, torch.device(device), names=names)
        pj = [Projection(linear.Nf4Weight.from_layer(self.layer, n, self.code2), lora=lora, bucket=bucket,
                         seed=seed * 10 + 3 + i) for i, n in enumerate(names)]
        self.gate, self.up, self.down = pj
        self.w_gu = linear.Nf4Weight.from_layer_group(self.layer, ("gate_proj", "up_proj"), self.code2)
        self.projections = (self.gate, self.up, self.down)
        # with a bucket the block's gradients are one contiguous slice: cleared by one fill per backward
        self._grad_slice = bucket.flat[grad_lo:bucket._at] if (bucket is not None and lora) else None
        self._saved = None
        self.grad_stream = None
        self._pending = []

    def use_grad_stream(self, stream=None):
        """Run the three dA/dB kernels of a backward on a side stream, beside the dX GEMMs (they are bound by
        HBM latency, the GEMMs by the tensor and shared-memory pipes); `backward` joins the stream before it
        returns. Works eagerly and under CUDA-graph capture (the fork and the join are captured as edges)."""
        self.grad_stream = stream if stream is not None else torch.cuda.Stream(self.gate.w.device)
        return self

    @staticmethod
    def grad_numel(hidden, inter):
        return 2 * lora_grad_numel(inter, hidden) + lora_grad_numel(hidden, inter)

    def flops(self, M):
        return sum(p.flops(M) for p in self.projections)

    def forward(self, x, masks=(None, None, None), keep_scale=1.0, out=None):
        """y = down(silu(gate(x)) * up(x)); `out` (optional) receives y."""
        if self.fused_glue:
            g, u, h, tg, tu = linear.forward_gate_up(self.w_gu, x, self.gate.lora, masks[0] if self.gate.has_lora else None,
                                                     self.up.lora, masks[1] if self.up.has_lora else None, keep_scale)
            self.gate._saved = (x, masks[0] if self.gate.has_lora else None, keep_scale, tg)
            self.up._saved = (x, masks[1] if self.up.has_lora else None, keep_scale, tu)
            y = self.down.forward(h, masks[2], keep_scale, out=out)
            self._saved = (g, u)
            return y
        g = self.gate.forward(x, masks[0], keep_scale)
        u = self.up.forward(x, masks[1], keep_scale)
        h = F.silu(g.float()).mul_(u.float()).half()
        y = self.down.forward(h, masks[2], keep_scale, out=out)
        self._saved = (g, u)
        return y

    def backward(self, dy, need_dx=True, accumulate_grads=False, out=None):
        """d(input) of the block (into `out` when given) and the LoRA gradients of its three projections."""
        g, u = self._saved
        if self._grad_slice is not None and not accumulate_grads:
            self._grad_slice.zero_()
            accumulate_grads = True
        gs, pend = self.grad_stream, self._pending
        dh = self.down.backward(dy, accumulate_grads=accumulate_grads, grad_stream=gs, pending=pend)
        if self.fused_glue:
            dg, du = linear.swiglu_backward(g, u, dh, inplace=True)
        else:
            gf = g.float()
            sig = torch.sigmoid(gf)
            dhf = dh.float()
            du = (dhf * gf * sig).half()
            dg = (dhf * u.float() * sig * (1.0 + gf * (1.0 - sig))).half()
        dx = self.gate.backward(dg, out=out, need_dx=need_dx, accumulate_grads=accumulate_grads, grad_stream=gs, pending=pend)
        # d(input) of gate and up are summed into one buffer: the second launch adds its fp32 result to the
        # fp16 values the first one stored and rounds again (two roundings, like the reference's fp16 add,
        # solution/fast_qwen.py:1320-1323)
        dx = self.up.backward(du, out=dx, accumulate=need_dx, need_dx=need_dx, accumulate_grads=accumulate_grads,
                              grad_stream=gs, pending=pend)
        if gs is not None:
            torch.cuda.current_stream(dy.device).wait_stream(gs)
            pend.clear()
        self._saved = None
        return dx
