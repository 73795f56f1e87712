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
    def __init__(self, hidden, inter, kv, seed, device, lora_on=("q_proj", "v_proj"), bucket=None, bias_qkv=True, parts=None):
        """Seeded synthetic weights by default. `parts` (interop.layer_parts of a real model's decoder layer)
        supplies them instead: {"layer": PackedLayer, "code2", "bias": {name: fp16}, "lora": {name: (A, B, scale)}}."""
        self.hidden, self.inter, self.kv = hidden, inter, kv
        shapes = {"q_proj": (hidden, hidden), "k_proj": (kv, hidden), "v_proj": (kv, hidden), "o_proj": (hidden, hidden),
                  "gate_proj": (inter, hidden), "up_proj": (inter, hidden), "down_proj": (hidden, inter)}
        if parts is None:
            linears = {name: quantize.random_nf4_weight(*shapes[name], seed=seed * 16 + i, device=device)
                       for i, name in enumerate(k_nf4.LAYER_WEIGHTS)}
            self.layer, self.code2 = k_nf4.repack_layer(linears, torch.device(device))
            given_bias, given_lora = None, None
        else:
            self.layer, self.code2 = parts["layer"], parts["code2"]
            for name in k_nf4.LAYER_WEIGHTS:
                if tuple(self.layer.segments[name][1:]) != shapes[name]:
                    raise ValueError(f"{name}: {self.layer.segments[name][1:]} does not match the stack's shapes {shapes[name]}")
            given_bias, given_lora = parts.get("bias", {}), parts.get("lora", {})
            lora_on = tuple(given_lora)
            bias_qkv = all(n in given_bias for n in ("q_proj", "k_proj", "v_proj"))
        self.proj = {}
        grad_lo = bucket._at if bucket is not None else 0
        gen = torch.Generator().manual_seed(seed * 16 + 9)
        for i, name in enumerate(k_nf4.LAYER_WEIGHTS):
            w = linear.Nf4Weight.from_layer(self.layer, name, self.code2)
            bias = None
            if given_bias is not None:
                bias = given_bias.get(name)
            elif bias_qkv and name in ("q_proj", "k_proj", "v_proj"):      # Qwen2 has biases on q, k, v only
                bias = (torch.randn(shapes[name][0], generator=gen) * 0.1).half().to(device)
            self.proj[name] = blocks.Projection(w, bias=bias, lora=name in lora_on, bucket=bucket, seed=seed * 16 + 10 + i,
                                                lora_init=None if given_lora is None else given_lora.get(name))
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

    def __init__(self, hidden, inter, kv, n_layers, device, seed=0, lora_on=("q_proj", "v_proj"), distinct_layers=None,
                 layer_parts=None):
        """`layer_parts`: one interop.layer_parts dict per layer of a real model (the weights are then not
        synthetic, n_layers = len(layer_parts) and every layer must carry LoRA on the same projections)."""
        if layer_parts is not None:
            n_layers, distinct_layers = len(layer_parts), None
            lora_on = tuple(layer_parts[0].get("lora", {}))
            if any(tuple(p.get("lora", {})) != lora_on for p in layer_parts):
                raise ValueError("every layer must carry LoRA on the same projections")
        self.hidden, self.inter, self.kv, self.n_layers, self.lora_on = hidden, inter, kv, n_layers, tuple(lora_on)
        per_layer = sum(blocks.lora_grad_numel(*{"q_proj": (hidden, hidden), "k_proj": (kv, hidden), "v_proj": (kv, hidden),
                                                 "o_proj": (hidden, hidden), "gate_proj": (inter, hidden),
                                                 "up_proj": (inter, hidden), "down_proj": (hidden, inter)}[n])
                        for n in self.lora_on)
        # `distinct_layers` < n_layers reuses weight sets round-robin (benchmarks of very deep stacks on a
        # budget of set-up time); each backward then overwrites the gradients of the layer object it runs on
        n_distinct = n_layers if distinct_layers is None else min(distinct_layers, n_layers)
        self.bucket = blocks.GradBucket(per_layer * n_distinct, device)
        self._distinct = [DecoderLayerProjections(hidden, inter, kv, seed * 1000 + i, device, self.lora_on, self.bucket,
                                                  parts=None if layer_parts is None else layer_parts[i])
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


class PackedAttention:
    """Rotary embedding + causal grouped-query attention over packed varlen rows, forward and backward, through
    PyTorch's own kernels (scaled_dot_product_attention per sequence, autograd for the backward). Attention is not
    on this library's path (the reference has kernels of its own for it, solution/k_rope.py, k_attn.py); this is
    the glue that makes the layer runner a real Qwen2 decoder layer. Rotary embedding as in Qwen2: the two halves
    of a head rotate against each other, positions restart at every sequence."""

    def __init__(self, n_heads, n_kv_heads, head_dim, theta=1.0e6):
        self.nh, self.nkv, self.hd, self.theta = n_heads, n_kv_heads, head_dim, theta
        self._tables = {}

    def _cos_sin(self, seq_lens, device):
        key = (tuple(seq_lens), str(device))
        if key not in self._tables:
            pos = torch.cat([torch.arange(n, dtype=torch.float32) for n in seq_lens]).to(device)
            inv = self.theta ** (-torch.arange(0, self.hd, 2, dtype=torch.float32, device=device) / self.hd)
            ang = pos[:, None] * inv[None, :]
            emb = torch.cat([ang, ang], dim=1)
            self._tables = {key: (emb.cos()[:, None, :], emb.sin()[:, None, :])}
        return self._tables[key]

    @staticmethod
    def _rotate(x, cos, sin):
        half = x.shape[-1] // 2
        rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
        return (x.float() * cos + rot.float() * sin).to(x.dtype)

    def forward(self, qkv, seq_lens):
        """qkv fp16 [M, (nh + 2 nkv) hd] -> (a fp16 [M, nh hd], state for backward)."""
        import torch.nn.functional as F
        H, KV = self.nh * self.hd, self.nkv * self.hd
        if sum(seq_lens) != qkv.shape[0]:
            raise ValueError(f"sequence lengths {seq_lens} do not add up to {qkv.shape[0]} rows")
        leaf = qkv.detach().requires_grad_(True)
        cos, sin = self._cos_sin(seq_lens, qkv.device)
        with torch.enable_grad():
            q = self._rotate(leaf[:, :H].view(-1, self.nh, self.hd), cos, sin)
            k = self._rotate(leaf[:, H:H + KV].view(-1, self.nkv, self.hd), cos, sin)
            v = leaf[:, H + KV:].view(-1, self.nkv, self.hd)
            outs, at = [], 0
            for n in seq_lens:
                sl = slice(at, at + n)
                o = F.scaled_dot_product_attention(q[sl].transpose(0, 1)[None], k[sl].transpose(0, 1)[None],
                                                   v[sl].transpose(0, 1)[None], is_causal=True, enable_gqa=self.nkv != self.nh)
                outs.append(o[0].transpose(0, 1).reshape(n, H))
                at += n
            a = torch.cat(outs, dim=0)
        return a.detach(), (leaf, a)

    @staticmethod
    def backward(state, da):
        leaf, a = state
        (dqkv,) = torch.autograd.grad(a, leaf, da)
        return dqkv


class NormedDecoderLayer:
    """The projections of one decoder layer between REAL fused residual + RMSNorm kernels, driven the way the
    reference drives its layer loop (solution/fast_qwen.py:1017-1123 forward, 1232-1384 backward): an fp32 residual
    stream, each norm adding the fp16 output of the GEMM before it (`delta`), norm 1 producing y16 AND the rank-16
    LoRA products of q and v, one stacked launch for Q|K|V forward and ONE for its backward (the LoRA input
    gradients are folded into norm 1's backward, as in solution/k_norm.py:64-71), one for gate|up each way.
    Attention itself (RoPE, softmax) is not on this path: with `attention` (a PackedAttention) and the batch's
    sequence lengths it runs through PyTorch's kernels, otherwise the stand-in of DecoderLayerProjections is used.

        forward(x32, delta16)  -> (x32', delta16')     with x_next = x32' + delta16'
        backward(dres32, d16)  -> (dres32', d16')      gradients w.r.t. x_next in, w.r.t. this layer's input out
    """

    def __init__(self, base: DecoderLayerProjections, eps=1e-6, norm_weights=None, seed=0, attention=None):
        from . import k_norm
        self.k_norm = k_norm
        self.base, self.eps, self.attention = base, eps, attention
        if attention is not None and (attention.nh * attention.hd != base.hidden or attention.nkv * attention.hd != base.kv):
            raise ValueError("attention head layout does not match the projection widths")
        dev = base.layer.flat.device
        if norm_weights is None:
            gen = torch.Generator().manual_seed(seed * 16 + 15)
            norm_weights = tuple((torch.rand(base.hidden, generator=gen) + 0.5).to(dev) for _ in range(2))
        self.w_in, self.w_post = (w.to(dev, torch.float32).contiguous() for w in norm_weights[:2])
        P = base.proj
        if not (P["q_proj"].has_lora and P["v_proj"].has_lora) or any(P[n].has_lora for n in ("k_proj", "o_proj", "gate_proj", "up_proj", "down_proj")):
            raise ValueError("the normed layer implements the task's adapter: LoRA on q_proj and v_proj only")
        if not base.fused_groups:
            raise ValueError("projection widths must be multiples of 128")
        self._saved = None

    def forward(self, x32, delta16, masks, keep_scale, seq_lens=None):
        b, kn, P = self.base, self.k_norm, self.base.proj
        M, H, KV = x32.shape[0], b.hidden, b.kv
        dev = x32.device
        f32 = dict(dtype=torch.float32, device=dev)
        y1 = torch.empty(M, H, dtype=torch.float16, device=dev)
        x1 = torch.empty(M, H, **f32) if delta16 is not None else x32
        rstd1, tq, tv = torch.empty(M, **f32), torch.empty(M, 16, **f32), torch.empty(M, 16, **f32)
        mq, mv = masks.get("q_proj"), masks.get("v_proj")
        kn.rms_forward(x32, self.w_in, y1, rstd1, self.eps, delta=delta16, xout=x1 if delta16 is not None else None,
                       aq=P["q_proj"].A16, av=P["v_proj"].A16, tq=tq, tv=tv, mq=mq, mv=mv, keep_scale=keep_scale)
        qkv = torch.empty(M, H + 2 * KV, dtype=torch.float16, device=dev)
        linear.forward_multi(b.w_qkv, y1, [(H, P["q_proj"].lora, mq, keep_scale, tq), (KV, None, None, 1.0),
                                           (KV, P["v_proj"].lora, mv, keep_scale, tv)], bias=b.bias_qkv, out=qkv)
        att = None
        if self.attention is not None and seq_lens is not None:
            a, att = self.attention.forward(qkv, seq_lens)
        else:
            a = qkv[:, :H].clone()                             # attention stand-in (see DecoderLayerProjections)
            a[:, :KV] += qkv[:, H:H + KV]
            a[:, KV:2 * KV] += qkv[:, H + KV:]
        o, _ = linear.forward(P["o_proj"].w, a)
        y2 = torch.empty(M, H, dtype=torch.float16, device=dev)
        x2, rstd2 = torch.empty(M, H, **f32), torch.empty(M, **f32)
        kn.rms_forward(x1, self.w_post, y2, rstd2, self.eps, delta=o, xout=x2)
        g, u, h, _, _ = linear.forward_gate_up(b.w_gu, y2)
        dn, _ = linear.forward(P["down_proj"].w, h)
        self._saved = (x1, rstd1, y1, tq, tv, mq, mv, keep_scale, att, o, rstd2, g, u, h)
        return x2, dn

    def backward(self, dres, d16, need_dx=True):
        """dres fp32 / d16 fp16: gradient w.r.t. x_next = x2 + dn (the fp16 copy feeds the GEMM, as the reference's
        autocast copy does). Returns the same pair for this layer's input, or (None, None) when need_dx is False
        (the first layer: only its LoRA gradients are wanted, solution/fast_qwen.py:1363-1364)."""
        b, kn, P = self.base, self.k_norm, self.base.proj
        x1, rstd1, y1, tq, tv, mq, mv, ks, att, o, rstd2, g, u, h = self._saved
        H, KV, M = b.hidden, b.kv, dres.shape[0]
        dev = dres.device
        if b._grad_slice is not None:
            b._grad_slice.zero_()
        dh, _ = linear.backward_dx(P["down_proj"].w, d16)
        linear.swiglu_backward(g, u, dh, inplace=True)
        dy2, _ = linear.backward_dx(b.w_gu, g._base)           # [dg | du] . W_gu in one launch
        dres2 = torch.empty_like(dres)
        do16 = torch.empty(M, H, dtype=torch.float16, device=dev)
        # norm 2's input is x1 + o: recomputed inside the kernel from the two saved tensors
        kn.rms_backward(dy2, 1.0, x1, self.w_post, rstd2, dres2, dres=dres, out16=do16, delta=o)
        da, _ = linear.backward_dx(P["o_proj"].w, do16)
        if att is not None:
            dqkv = PackedAttention.backward(att, da)
        else:
            dqkv = torch.empty(M, H + 2 * KV, dtype=torch.float16, device=dev)
            dqkv[:, :H] = da
            dqkv[:, H:H + KV] = da[:, :KV]
            dqkv[:, H + KV:] = da[:, KV:2 * KV]
        pq, pv = P["q_proj"], P["v_proj"]
        uq = linear.lora_u(dqkv[:, :H], pq.B16t, pq.scale)
        uv = linear.lora_u(dqkv[:, H + KV:], pv.B16t, pv.scale)
        linear.lora_grads(dqkv[:, :H], y1, tq, uq, pq.scale, mask=mq, keep_scale=ks, dA=pq.dA, dB=pq.dB, accumulate=True)
        linear.lora_grads(dqkv[:, H + KV:], y1, tv, uv, pv.scale, mask=mv, keep_scale=ks, dA=pv.dA, dB=pv.dB, accumulate=True)
        self._saved = None
        if not need_dx:
            return None, None
        dy1, _ = linear.backward_dx(b.w_qkv, dqkv)             # base term of q, k and v in one launch, no LoRA branch
        out = torch.empty_like(dres)
        out16 = torch.empty(M, H, dtype=torch.float16, device=dev)
        kn.rms_backward(dy1, 1.0, x1, self.w_in, rstd1, out, dres=dres2, uq=uq, uv=uv, aq=pq.A16, av=pv.A16, mq=mq, mv=mv,
                        keep_scale=ks, out16=out16)
        return out, out16


class NormedStack:
    """n_layers NormedDecoderLayers over one LoRA gradient bucket: `run_step` is the whole forward and the
    hand-written backward of the decoder stack (embedding, attention proper and the LM head are outside the path)."""

    def __init__(self, hidden, inter, kv, n_layers, device, seed=0, eps=1e-6, layer_parts=None, n_heads=None, rope_theta=1.0e6):
        """`n_heads`: run real rotary + causal grouped-query attention (PackedAttention; head_dim = hidden / n_heads,
        kv / head_dim key-value heads) between the projections when `run_step` / `apply` get the sequence lengths."""
        self.stack = ProjectionStack(hidden, inter, kv, n_layers, device, seed=seed, layer_parts=layer_parts)
        norms = [None] * self.stack.n_layers if layer_parts is None else [p.get("norm") for p in layer_parts]
        self.attention = None
        if n_heads is not None:
            hd = hidden // n_heads
            self.attention = PackedAttention(n_heads, kv // hd, hd, rope_theta)
        self.layers = [NormedDecoderLayer(l, eps if nw is None else nw[2], nw, seed=seed * 1000 + i, attention=self.attention)
                       for i, (l, nw) in enumerate(zip(self.stack.layers, norms))]
        self.bucket = self.stack.bucket

    def flops(self, M):
        return self.stack.flops(M)

    def forward(self, x32, masks_per_layer, keep_scale, seq_lens=None):
        x, delta = x32, None
        for layer, masks in zip(self.layers, masks_per_layer):
            x, delta = layer.forward(x, delta, masks, keep_scale, seq_lens)
        return x + delta.float()

    def backward(self, dres, need_input_grad=False):
        d, d16 = dres, dres.half()
        for i in reversed(range(len(self.layers))):
            d, d16 = self.layers[i].backward(d, d16, need_dx=i > 0 or need_input_grad)
        return d

    def run_step(self, x32, dres, masks_per_layer, keep_scale, seq_lens=None):
        """x32 fp32 [M, hidden]: the embedded tokens; dres fp32: the gradient of the loss w.r.t. the stack's output.
        Returns (output fp32 = residual stream after the last layer, gradient w.r.t. layer 1's input or None)."""
        out = self.forward(x32, masks_per_layer, keep_scale, seq_lens)
        return out, self.backward(dres)

    def lora_masters(self):
        """The fp32 LoRA masters of every distinct layer, in the order `apply` returns their gradients."""
        return [t for l in self.stack._distinct for n in ("q_proj", "v_proj") for t in (l.proj[n].A, l.proj[n].B)]

    def apply(self, x32, masks_per_layer, keep_scale, seq_lens=None):
        """The whole decoder stack as ONE autograd node (the counterpart of the reference's fused runner,
        solution/fast_qwen.py:1527-1548): the output carries a grad_fn whose backward is the hand-written one and
        hands PyTorch the gradients of the LoRA masters (`lora_masters()`, which must be leaf tensors that require
        grad for an optimiser to see them) and, if x32 requires grad, of the input."""
        if self.stack._shared:
            raise ValueError("a stack that reuses weight sets cannot keep the activations of a whole forward pass")
        return _StackStep.apply(self, x32, masks_per_layer, keep_scale, seq_lens, *self.lora_masters())


class _StackStep(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ns, x32, masks_per_layer, keep_scale, seq_lens, *masters):
        for l in ns.stack._distinct:
            l.refresh16()                                      # fp16 shadows follow the masters (fast_qwen.py:686-692)
        ctx.ns, ctx.need_dx = ns, x32.requires_grad
        return ns.forward(x32.detach(), masks_per_layer, keep_scale, seq_lens)

    @staticmethod
    def backward(ctx, dout):
        ns = ctx.ns
        dx = ns.backward(dout.contiguous().float(), need_input_grad=ctx.need_dx)
        grads = [g for l in ns.stack._distinct for n in ("q_proj", "v_proj") for g in (l.proj[n].dA, l.proj[n].dB)]
        return (None, dx if ctx.need_dx else None, None, None, None, *grads)
