"""All seven projections of every decoder layer, packed the way the reference packs them, driven
through the fused NF4 + LoRA linear: the projection stack of benchmark configurations 2 and 3.

Per layer the 4-bit weights q, k, v, o, gate, up, down live in one flat PackedLayer buffer
(k_nf4.repack_layer, same order and segment table as reference solution/k_nf4.py:126-173), so Q|K|V
and gate|up are contiguous and the three attention projections write into column slices of one
[M, hidden + 2*kv] buffer through the kernels' leading-dimension argument, as the reference's fused
W_qkv GEMM does (solution/fast_qwen.py:405-413, 947). LoRA (r=16) sits on the projections named in
`lora_on` (the task: q_proj and v_proj, solution/fast_qwen.py:93-99).

Only the projections are this library's business. What sits between them in a transformer
(normalisation, rotary embedding, attention, residuals) is stood in for by the cheapest
differentiable PyTorch glue that keeps every projection's input and gradient non-trivial:

    a   = q;  a[:, :kv] += k;  a[:, kv:2kv] += v        (stand-in for attention)
    h1  = x + o_proj(a)
    x'  = h1 + down_proj(silu(gate_proj(h1)) * up_proj(h1))

The backward is written by hand like the reference's (solution/fast_qwen.py:1232-1384): dX of
projections that share an input are accumulated in-kernel, LoRA gradients land in one flat bucket.
Token rows are a packed varlen batch: M = sum of the sequence lengths (fast_qwen.py:803-876); the
projections never need the sequence boundaries.
"""

import torch

from . import blocks, k_nf4, linear, quantize


def pack_lengths(batch, lo, hi, seed):
    """Seeded sequence lengths, uniform in [lo, hi], and their packed row count."""
    gen = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (batch,), generator=gen)
    return lens.tolist(), int(lens.sum())


class DecoderLayerProjections:
    def __init__(self, hidden, inter, kv, seed, device, lora_on=("q_proj", "v_proj"), bucket=None, bias_qkv=True):
        self.hidden, self.inter, self.kv = hidden, inter, kv
        shapes = {"q_proj": (hidden, hidden), "k_proj": (kv, hidden), "v_proj": (kv, hidden), "o_proj": (hidden, hidden),
                  "gate_proj": (inter, hidden), "up_proj": (inter, hidden), "down_proj": (hidden, inter)}
        linears = {name: quantize.random_nf4_weight(*shapes[name], seed=seed * 16 + i, device=device)
                   for i, name in enumerate(k_nf4.LAYER_WEIGHTS)}
        self.layer, self.code2 = k_nf4.repack_layer(linears, torch.device(device))
        self.proj = {}
        grad_lo = bucket._at if bucket is not None else 0
        gen = torch.Generator().manual_seed(seed * 16 + 9)
        for i, name in enumerate(k_nf4.LAYER_WEIGHTS):
            w = linear.Nf4Weight.from_layer(self.layer, name, self.code2)
            bias = None
            if bias_qkv and name in ("q_proj", "k_proj", "v_proj"):      # Qwen2 has biases on q, k, v only
                bias = (torch.randn(shapes[name][0], generator=gen) * 0.1).half().to(device)
            self.proj[name] = blocks.Projection(w, bias=bias, lora=name in lora_on, bucket=bucket, seed=seed * 16 + 10 + i)
        # Q|K|V and gate|up lie row after row in the packed layer: one stacked matrix and one launch each
        self.w_qkv = linear.Nf4Weight.from_layer_group(self.layer, ("q_proj", "k_proj", "v_proj"), self.code2)
        self.w_gu = linear.Nf4Weight.from_layer_group(self.layer, ("gate_proj", "up_proj"), self.code2)
        self.bias_qkv = torch.cat([self.proj[n].bias for n in ("q_proj", "k_proj", "v_proj")]) if bias_qkv else None
        self.fused_groups = all(r % 128 == 0 for r in self.w_qkv.rows_each + self.w_gu.rows_each)
        # backward of a stacked group as ONE launch (reference solution/fast_qwen.py:1338, 1364): gate|up when
        # neither carries LoRA; K|V when only v does (its lora_B zero-padded over the k rows, so that
        # [dk | dv] . B_pad = dv . B_v and the one dropout mask of the launch is v's)
        P = self.proj
        self.gu_one_backward = not (P["gate_proj"].has_lora or P["up_proj"].has_lora)
        self.kv_one_backward = P["v_proj"].has_lora and not P["k_proj"].has_lora
        if self.kv_one_backward:
            self.w_kv = linear.Nf4Weight.from_layer_group(self.layer, ("k_proj", "v_proj"), self.code2)
            pv = P["v_proj"]
            self._Bv_pad = torch.zeros(2 * kv, linear.RANK, dtype=torch.float16, device=device)
            self._Bvt_pad = torch.zeros(linear.RANK, 2 * kv, dtype=torch.float16, device=device)
            self._pad_src = pv
            self.refresh16()
        # with a bucket the layer's gradients are one contiguous slice: cleared by one fill per backward
        self._grad_slice = bucket.flat[grad_lo:bucket._at] if bucket is not None and bucket._at > grad_lo else None
        self._saved = None

    def refresh16(self):
        """Refresh every fp16 LoRA shadow from its fp32 master (after an optimiser step)."""
        for p in self.proj.values():
            if p.has_lora:
                p.refresh16()
        if self.kv_one_backward:
            self._Bv_pad[self.kv:].copy_(self._pad_src.B16)
            self._Bvt_pad[:, self.kv:].copy_(self._pad_src.B16t)

    def grad_numel(self, lora_on):
        return sum(blocks.lora_grad_numel(self.proj[n].w.N, self.proj[n].w.K) for n in lora_on)

    def flops(self, M):
        return sum(p.flops(M) for p in self.proj.values())

    def forward(self, x, masks, keep_scale):
        """x [M, hidden] fp16; masks: dict projection name -> uint8 keep-mask [M, K] for the LoRA ones."""
        P, H, KV, M = self.proj, self.hidden, self.kv, x.shape[0]
        qkv = torch.empty(M, H + 2 * KV, dtype=torch.float16, device=x.device)
        if self.fused_groups:
            self._forward_group(self.w_qkv, ("q_proj", "k_proj", "v_proj"), x, masks, keep_scale, self.bias_qkv, qkv)
        else:
            P["q_proj"].forward(x, masks.get("q_proj"), keep_scale, out=qkv[:, :H])
            P["k_proj"].forward(x, masks.get("k_proj"), keep_scale, out=qkv[:, H:H + KV])
            P["v_proj"].forward(x, masks.get("v_proj"), keep_scale, out=qkv[:, H + KV:])
        a = qkv[:, :H].clone()
        a[:, :KV] += qkv[:, H:H + KV]
        a[:, KV:2 * KV] += qkv[:, H + KV:]
        h1 = x + P["o_proj"].forward(a, masks.get("o_proj"), keep_scale)
        if self.fused_groups:
            # gate, up and the gated product in one launch
            pg, pu = P["gate_proj"], P["up_proj"]
            mg = masks.get("gate_proj") if pg.has_lora else None
            mu = masks.get("up_proj") if pu.has_lora else None
            g, u, h, tg, tu = linear.forward_gate_up(self.w_gu, h1, pg.lora, mg, pu.lora, mu, keep_scale)
            pg._saved = (h1, mg, keep_scale, tg)
            pu._saved = (h1, mu, keep_scale, tu)
        else:
            g = P["gate_proj"].forward(h1, masks.get("gate_proj"), keep_scale)
            u = P["up_proj"].forward(h1, masks.get("up_proj"), keep_scale)
            h = linear.swiglu_forward(g, u)
        out = h1 + P["down_proj"].forward(h, masks.get("down_proj"), keep_scale)
        self._saved = (g, u)
        return out

    def _forward_group(self, w, names, x, masks, keep_scale, bias, out):
        """One launch for projections that share x; each keeps its own saved state for the backward."""
        segs = []
        for n in names:
            pj = self.proj[n]
            segs.append((pj.w.N, pj.lora, masks.get(n) if pj.has_lora else None, keep_scale))
        _, ts = linear.forward_multi(w, x, segs, bias=bias, out=out)
        for n, t in zip(names, ts):
            pj = self.proj[n]
            pj._saved = (x, masks.get(n) if pj.has_lora else None, keep_scale, t)

    def backward(self, dout, need_dx=True, accumulate_grads=False):
        P, H, KV = self.proj, self.hidden, self.kv
        g, u = self._saved
        if self._grad_slice is not None and not accumulate_grads:
            self._grad_slice.zero_()
            accumulate_grads = True
        ag = accumulate_grads
        dh = P["down_proj"].backward(dout, accumulate_grads=ag)
        dg, du = linear.swiglu_backward(g, u, dh, inplace=True)
        gu = g._base
        if self.gu_one_backward and gu is not None and gu.shape == (g.shape[0], 2 * self.inter):
            # [dg | du] . W_gu: one launch, one rounding of the sum
            dh1, _ = linear.backward_dx(self.w_gu, gu)
            P["gate_proj"]._saved = P["up_proj"]._saved = None
        else:
            dh1 = P["gate_proj"].backward(dg, accumulate_grads=ag)
            dh1 = P["up_proj"].backward(du, out=dh1, accumulate=True, accumulate_grads=ag)
        dh1 += dout                                            # residual around the MLP
        da = P["o_proj"].backward(dh1, accumulate_grads=ag)
        dqkv = torch.empty(da.shape[0], H + 2 * KV, dtype=torch.float16, device=da.device)
        dqkv[:, :H] = da
        dqkv[:, H:H + KV] = da[:, :KV]
        dqkv[:, H + KV:] = da[:, KV:2 * KV]
        dx = None
        if need_dx:
            dx = P["q_proj"].backward(dqkv[:, :H], accumulate_grads=ag)
            if self.kv_one_backward:
                pv = P["v_proj"]
                xv, mask_v, ks_v, t_v = pv._saved
                lora_kv = (pv.A16, self._Bv_pad, pv.scale, self._Bvt_pad)
                dx, u_v = linear.backward_dx(self.w_kv, dqkv[:, H:], lora=lora_kv, mask=mask_v, keep_scale=ks_v, out=dx,
                                             accumulate=True, want_u=True)
                linear.lora_grads(dqkv[:, H + KV:], xv, t_v, u_v, pv.scale, mask=mask_v, keep_scale=ks_v, dA=pv.dA, dB=pv.dB,
                                  accumulate=ag)
                pv._saved = P["k_proj"]._saved = None
            else:
                dx = P["k_proj"].backward(dqkv[:, H:H + KV], out=dx, accumulate=True, accumulate_grads=ag)
                dx = P["v_proj"].backward(dqkv[:, H + KV:], out=dx, accumulate=True, accumulate_grads=ag)
            dx += dh1                                          # residual around the attention stand-in
        else:
            # the first layer needs no d(input), only its LoRA gradients (solution/fast_qwen.py:1363-1364)
            for name, sl in (("q_proj", slice(0, H)), ("k_proj", slice(H, H + KV)), ("v_proj", slice(H + KV, H + 2 * KV))):
                P[name].backward(dqkv[:, sl], need_dx=False, accumulate_grads=ag)
        self._saved = None
        return dx


class ProjectionStack:
    """n_layers DecoderLayerProjections with one LoRA gradient bucket (all-reduced once per step under DP)."""

    def __init__(self, hidden, inter, kv, n_layers, device, seed=0, lora_on=("q_proj", "v_proj"), distinct_layers=None):
        self.hidden, self.inter, self.kv, self.n_layers, self.lora_on = hidden, inter, kv, n_layers, tuple(lora_on)
        per_layer = sum(blocks.lora_grad_numel(*{"q_proj": (hidden, hidden), "k_proj": (kv, hidden), "v_proj": (kv, hidden),
                                                 "o_proj": (hidden, hidden), "gate_proj": (inter, hidden),
                                                 "up_proj": (inter, hidden), "down_proj": (hidden, inter)}[n])
                        for n in self.lora_on)
        # `distinct_layers` < n_layers reuses weight sets round-robin (benchmarks of very deep stacks on a
        # budget of set-up time); each backward then overwrites the gradients of the layer object it runs on
        n_distinct = n_layers if distinct_layers is None else min(distinct_layers, n_layers)
        self.bucket = blocks.GradBucket(per_layer * n_distinct, device)
        self._distinct = [DecoderLayerProjections(hidden, inter, kv, seed * 1000 + i, device, self.lora_on, self.bucket)
                          for i in range(n_distinct)]
        self.layers = [self._distinct[i % n_distinct] for i in range(n_layers)]
        # saved activations live in the layer objects: a reused object cannot appear twice in one forward pass
        self._shared = n_distinct < n_layers

    def flops(self, M):
        return sum(layer.flops(M) for layer in self.layers)

    def step(self, x, dy, masks_per_layer, keep_scale, need_input_grad=False, sync=None):
        """Forward through all layers, then backward-dX through all layers. With shared weight sets
        each layer runs forward+backward in turn instead (activation memory of one layer). The first
        layer's d(input) is only computed on request (the reference skips it: nothing below needs it).
        `sync` (a dp.GradSync with one slot per distinct layer): each layer's slice of the gradient bucket is
        all-reduced on the side stream as soon as its backward has been queued, under the remaining backward."""
        n_distinct = len(self._distinct)

        def backward(i, d, need_dx):
            layer = self.layers[i]
            if sync is not None:
                sync.wait_slot(i % n_distinct)          # the slice's previous exchange must be over before it is cleared
            out = layer.backward(d, need_dx=need_dx)
            if sync is not None and layer._grad_slice is not None:
                sync.launch(i % n_distinct, layer._grad_slice)
            return out

        if self._shared:
            dx = None
            for i, layer in enumerate(self.layers):
                out = layer.forward(x, masks_per_layer[i % len(masks_per_layer)], keep_scale)
                dx = backward(i, dy, True)
            return out, dx
        acts = [x]
        for i, layer in enumerate(self.layers):
            acts.append(layer.forward(acts[-1], masks_per_layer[i], keep_scale))
        d = dy
        for i in reversed(range(self.n_layers)):
            d = backward(i, d, i > 0 or need_input_grad)
        return acts[-1], d
