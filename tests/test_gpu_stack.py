"""The projection stack (benchmark configuration 2 in miniature): two decoder layers of seven NF4 projections
each, LoRA on q and v, a packed varlen batch, forward and hand-written backward, against the same
computation done projection by projection with the CPU oracle and the same fp16 glue."""

import pytest
import torch
import torch.nn.functional as F

from decentrik_prime_b200 import k_nf4, linear, stack
from oracle import nf4_oracle

pytestmark = pytest.mark.gpu


def oracle_layer(layer, x, dout, masks, keep_scale, need_dx):
    """CPU statement of DecoderLayerProjections.forward/backward with oracle linears (fp64 inside each
    projection, fp16 tensors between them, like the device path)."""
    H, KV = layer.hidden, layer.kv
    W = {n: nf4_oracle.dequant_weight(layer.layer, n, layer.code2) for n in k_nf4.LAYER_WEIGHTS}

    def lin(name, inp, grad=None):
        p = layer.proj[name]
        A16 = p.A16.cpu() if p.has_lora else None
        B16 = p.B16.cpu() if p.has_lora else None
        m = masks.get(name) if p.has_lora else None
        return nf4_oracle.lora_linear_o1(W[name], inp, grad, None if p.bias is None else p.bias.cpu(), A16, B16, p.scale,
                                         None if m is None else m.cpu(), keep_scale if m is not None else 1.0)

    q, k, v = (lin(n, x)["y"].half() for n in ("q_proj", "k_proj", "v_proj"))
    a = q.clone(); a[:, :KV] += k; a[:, KV:2 * KV] += v
    h1 = x + lin("o_proj", a)["y"].half()
    g, u = lin("gate_proj", h1)["y"].half(), lin("up_proj", h1)["y"].half()
    h = (F.silu(g.float()) * u.float()).half()
    out = h1 + lin("down_proj", h)["y"].half()
    grads = {}
    dh = lin("down_proj", h, dout)["dx"].half()
    gf, sig = g.float(), torch.sigmoid(g.float())
    du = (dh.float() * gf * sig).half()
    dg = ((dh.float() * u.float()) * sig * (1 + gf * (1 - sig))).half()
    dh1 = (lin("gate_proj", h1, dg)["dx"] + lin("up_proj", h1, du)["dx"]).half() + dout
    da = lin("o_proj", a, dh1)["dx"].half()
    rq, rk, rv = lin("q_proj", x, da), lin("k_proj", x, da[:, :KV].contiguous()), lin("v_proj", x, da[:, KV:2 * KV].contiguous())
    for n, r in (("q_proj", rq), ("v_proj", rv)):
        grads[n] = (r["dA"], r["dB"])
    dx = (rq["dx"] + rk["dx"] + rv["dx"]).half() + dh1 if need_dx else None
    return out, dx, grads


def test_two_layer_stack_matches_oracle():
    dev = torch.device("cuda")
    lens, M = stack.pack_lengths(4, 20, 60, seed=3)
    assert M == sum(lens) and len(lens) == 4
    st = stack.ProjectionStack(256, 512, 128, n_layers=2, device=dev, seed=5)
    gen = torch.Generator().manual_seed(11)
    x = torch.randn(M, 256, generator=gen).half()
    dy = (torch.randn(M, 256, generator=gen) * 0.5).half()
    keep_scale = 1.0 / float(torch.tensor(0.95, dtype=torch.float32))
    masks = [{n: (torch.rand(M, 256, generator=gen) >= 0.05).to(torch.uint8) for n in ("q_proj", "v_proj")} for _ in range(2)]
    dev_masks = [{n: m.to(dev) for n, m in layer.items()} for layer in masks]
    out, dx = st.step(x.to(dev), dy.to(dev), dev_masks, keep_scale, need_input_grad=True)
    linear.check_status()
    # oracle: forward through both layers, backward in reverse
    acts = [x]
    for i in range(2):
        o, _, _ = oracle_layer(st.layers[i], acts[-1], torch.zeros(M, 256, dtype=torch.float16), masks[i], keep_scale, False)
        acts.append(o)
    d = dy
    ref_grads = [None, None]
    for i in (1, 0):
        _, dxi, ref_grads[i] = oracle_layer(st.layers[i], acts[i], d, masks[i], keep_scale, True)
        d = dxi
    err, rel = nf4_oracle.errors(out, acts[-1].float())
    assert rel <= 2e-3, (err, rel)
    err, rel = nf4_oracle.errors(dx, d.float())       # layer 0's d(input), computed because it was asked for
    assert rel <= 3e-3, (err, rel)
    for i in range(2):
        for n in ("q_proj", "v_proj"):
            p = st.layers[i].proj[n]
            for got, ref in ((p.dA, ref_grads[i][n][0]), (p.dB, ref_grads[i][n][1])):
                err, rel = nf4_oracle.errors(got, ref)
                assert rel <= 5e-3, (i, n, err, rel)


def test_stack_flops_per_token():
    """Algorithmic FLOPs per token per layer of the Qwen2.5-1.5B and 7B shapes: 4*N*K per projection
    (forward + backward-dX) plus the LoRA terms on q and v."""
    base_15b = 4 * (1536 * 1536 * 2 + 256 * 1536 * 2 + 8960 * 1536 * 3)
    assert base_15b == 187_170_816            # 187.17 MFLOP per token per layer
    base_7b = 4 * (3584 * 3584 * 2 + 512 * 3584 * 2 + 18944 * 3584 * 3)
    assert base_7b == 932_184_064             # 932.18 MFLOP per token per layer


def test_stack_from_a_quantised_peft_model_and_adapter_save(tmp_path):
    """interop.model_parts on a bitsandbytes/PEFT-shaped module tree -> ProjectionStack(layer_parts=...) runs the
    real weights and LoRA factors (one layer against the oracle), and the trained factors leave as a PEFT adapter."""
    from decentrik_prime_b200 import interop
    from tests.test_interop import H, KV, I, fake_model
    dev = torch.device("cuda")
    parts = interop.model_parts(fake_model(2), dev)
    st = stack.ProjectionStack(H, I, KV, 0, dev, layer_parts=parts)
    assert st.n_layers == 2 and st.lora_on == ("q_proj", "v_proj")
    M = 150
    gen = torch.Generator().manual_seed(4)
    x = torch.randn(M, H, generator=gen).half()
    dy = (torch.randn(M, H, generator=gen) * 0.5).half()
    ks = 1.0 / float(torch.tensor(0.95, dtype=torch.float32))
    masks = [{n: (torch.rand(M, H, generator=gen) >= 0.05).to(torch.uint8) for n in ("q_proj", "v_proj")} for _ in range(2)]
    layer = st.layers[0]
    out = layer.forward(x.to(dev), {n: m.to(dev) for n, m in masks[0].items()}, ks)
    dx = layer.backward(dy.to(dev), need_dx=True)
    linear.check_status()
    ref_out, ref_dx, ref_grads = oracle_layer(layer, x, dy, masks[0], ks, True)
    err, rel = nf4_oracle.errors(out, ref_out.float())
    assert rel <= 2e-3, (err, rel)
    err, rel = nf4_oracle.errors(dx, ref_dx.float())
    assert rel <= 3e-3, (err, rel)
    for n in ("q_proj", "v_proj"):
        for got, ref in ((layer.proj[n].dA, ref_grads[n][0]), (layer.proj[n].dB, ref_grads[n][1])):
            err, rel = nf4_oracle.errors(got, ref)
            assert rel <= 5e-3, (n, err, rel)
    interop.save_adapter(tmp_path / "adapter", interop.stack_adapter(st))
    header = interop.adapter_header(tmp_path / "adapter")
    assert len(header) == 8 and header["base_model.model.model.layers.1.self_attn.q_proj.lora_A.weight"] == ["F32", [16, H]]


def _normed_oracle_forward(nl, x32, delta16, masks, ks):
    """CPU statement of NormedDecoderLayer.forward: norm_oracle for the norms, fp64 products rounded to fp16 where
    the device stores fp16."""
    import numpy as np
    from oracle import norm_oracle
    b = nl.base
    H, KV = b.hidden, b.kv
    W = {n: nf4_oracle.dequant_weight(b.layer, n, b.code2).double() for n in k_nf4.LAYER_WEIGHTS}
    P = b.proj
    n1 = norm_oracle.rms_forward_ref(x32.numpy(), nl.w_in.cpu().numpy(), nl.eps, delta=None if delta16 is None else delta16.numpy(),
                                     mq=masks["q_proj"].numpy(), mv=masks["v_proj"].numpy(), keep_scale=ks)
    y1 = torch.from_numpy(n1["y16"])
    cols = []
    t = {}
    for n, key in (("q_proj", "xq16"), ("k_proj", None), ("v_proj", "xv16")):
        y = y1.double() @ W[n].t() + P[n].bias.cpu().double()
        if key:
            t[n] = torch.from_numpy(n1[key]).double() @ P[n].A16.cpu().double().t()
            y = y + P[n].scale * (t[n] @ P[n].B16.cpu().double().t())
        cols.append(y.half())
    q, k, v = cols
    a = q.clone(); a[:, :KV] += k; a[:, KV:2 * KV] += v
    o = (a.double() @ W["o_proj"].t()).half()
    x1 = torch.from_numpy(n1["xout"])
    n2 = norm_oracle.rms_forward_ref(x1.numpy(), nl.w_post.cpu().numpy(), nl.eps, delta=o.numpy())
    y2 = torch.from_numpy(n2["y16"])
    g = (y2.double() @ W["gate_proj"].t()).half()
    u = (y2.double() @ W["up_proj"].t()).half()
    h = (F.silu(g.float()) * u.float()).half()
    dn = (h.double() @ W["down_proj"].t()).half()
    saved = dict(W=W, x1=x1, y1=y1, t=t, a=a, o=o, rstd1=n1["rstd"], rstd2=n2["rstd"], g=g, u=u, h=h, masks=masks, ks=ks)
    return torch.from_numpy(n2["xout"]), dn, saved


def _normed_oracle_backward(nl, s, dres, d16, need_dx):
    from oracle import norm_oracle
    b, P, W = nl.base, nl.base.proj, s["W"]
    H, KV = b.hidden, b.kv
    dh = (d16.double() @ W["down_proj"]).half()
    gf, sig = s["g"].float(), torch.sigmoid(s["g"].float())
    du = (dh.float() * gf * sig).half()
    dg = ((dh.float() * s["u"].float()) * sig * (1 + gf * (1 - sig))).half()
    dy2 = (dg.double() @ W["gate_proj"] + du.double() @ W["up_proj"]).half()
    dres2, do16 = norm_oracle.rms_backward_ref(dy2.numpy(), 1.0, s["x1"].numpy(), nl.w_post.cpu().numpy(), s["rstd2"],
                                               delta=s["o"].numpy(), dres=dres.numpy())
    da = (torch.from_numpy(do16).double() @ W["o_proj"]).half()
    dq, dk, dv = da, da[:, :KV], da[:, KV:2 * KV]
    grads, lx = {}, {}
    for n, dyn in (("q_proj", dq), ("v_proj", dv)):
        p = P[n]
        u = p.scale * (dyn.double() @ p.B16.cpu().double())
        xd = nf4_oracle.drop_ref(s["y1"], s["masks"][n], s["ks"]).double()
        grads[n] = (u.t() @ xd, p.scale * (dyn.double().t() @ s["t"][n]))
        lx[n] = (u @ p.A16.cpu().double()).numpy()
    if not need_dx:
        return None, None, grads
    dy1 = (dq.double() @ W["q_proj"] + dk.double() @ W["k_proj"] + dv.double() @ W["v_proj"]).half()
    out, out16 = norm_oracle.rms_backward_ref(dy1.numpy(), 1.0, s["x1"].numpy(), nl.w_in.cpu().numpy(), s["rstd1"], dres=dres2,
                                              lq=lx["q_proj"], lv=lx["v_proj"], mq=s["masks"]["q_proj"].numpy(),
                                              mv=s["masks"]["v_proj"].numpy(), keep_scale=s["ks"])
    return torch.from_numpy(out), torch.from_numpy(out16), grads


def test_normed_stack_matches_oracle():
    """Two decoder layers with the real fused residual + RMSNorm kernels either side of the projections: forward,
    hand-written backward (stacked Q|K|V and gate|up backward launches, LoRA input gradients folded into the norm
    backward) and LoRA gradients against the CPU oracle of the same computation."""
    dev = torch.device("cuda")
    H, I, KV, M = 256, 512, 128, 150
    ns = stack.NormedStack(H, I, KV, 2, dev, seed=9)
    gen = torch.Generator().manual_seed(21)
    x32 = torch.randn(M, H, generator=gen)
    dres = torch.randn(M, H, generator=gen) * 0.5
    ks = 1.0 / float(torch.tensor(0.95, dtype=torch.float32))
    masks = [{n: (torch.rand(M, H, generator=gen) >= 0.05).to(torch.uint8) for n in ("q_proj", "v_proj")} for _ in range(2)]
    out, d = ns.run_step(x32.to(dev), dres.to(dev), [{n: m.to(dev) for n, m in ms.items()} for ms in masks], ks)
    linear.check_status()
    x, delta, saved = x32, None, []
    for nl, ms in zip(ns.layers, masks):
        x, delta, s = _normed_oracle_forward(nl, x, delta, ms, ks)
        saved.append(s)
    err, rel = nf4_oracle.errors(out, x + delta.float())
    assert rel <= 2e-3, (err, rel)
    g_d, g_16 = dres, dres.half()
    ref_grads = [None, None]
    for i in (1, 0):
        g_d, g_16, ref_grads[i] = _normed_oracle_backward(ns.layers[i], saved[i], g_d, g_16, need_dx=i > 0)
    assert d is None and g_d is None          # the first layer's d(input) is not computed
    for i in range(2):
        for n in ("q_proj", "v_proj"):
            p = ns.layers[i].base.proj[n]
            for got, ref in ((p.dA, ref_grads[i][n][0]), (p.dB, ref_grads[i][n][1])):
                err, rel = nf4_oracle.errors(got, ref)
                assert rel <= 5e-3, (i, n, err, rel)
    # the gradient that reaches layer 0 from layer 1, checked through layer 1 alone
    nl = ns.layers[1]
    x_in, delta_in = (saved[0]["x1"] * 0 + _normed_oracle_forward(ns.layers[0], x32, None, masks[0], ks)[0],
                      _normed_oracle_forward(ns.layers[0], x32, None, masks[0], ks)[1])
    nl.forward(x_in.to(dev), delta_in.to(dev), {n: m.to(dev) for n, m in masks[1].items()}, ks)
    got, got16 = nl.backward(dres.to(dev), dres.half().to(dev), need_dx=True)
    linear.check_status()
    want, want16, _ = _normed_oracle_backward(nl, saved[1], dres, dres.half(), True)
    err, rel = nf4_oracle.errors(got, want)
    assert rel <= 3e-3, (err, rel)
    err, rel = nf4_oracle.errors(got16, want16.float())
    assert rel <= 3e-3, (err, rel)


def _reference_decoder_stack(ns, x32, masks, ks, seq_lens, theta):
    """The same decoder stack in plain PyTorch (fp64 on the CPU, autograd for the backward): dequantised weights
    from the oracle, the fp16 LoRA shadows as leaves, explicit rotary embedding and causal softmax attention with
    grouped key-value heads. Returns (output, leaves) with leaves[i][name] = (A, B)."""
    dt = torch.float64
    att = ns.attention
    nh, nkv, hd = att.nh, att.nkv, att.hd
    pos = torch.cat([torch.arange(n, dtype=dt) for n in seq_lens])
    inv = theta ** (-torch.arange(0, hd, 2, dtype=dt) / hd)
    ang = pos[:, None] * inv[None, :]
    cos, sin = torch.cat([ang, ang], 1).cos()[:, None, :], torch.cat([ang, ang], 1).sin()[:, None, :]

    def rot(t):
        half = hd // 2
        return t * cos + torch.cat([-t[..., half:], t[..., :half]], -1) * sin

    def rms(t, w, eps):
        return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * w

    x, leaves = x32.to(dt), []
    for nl, ms in zip(ns.layers, masks):
        b, P = nl.base, nl.base.proj
        H, KV = b.hidden, b.kv
        W = {n: nf4_oracle.dequant_weight(b.layer, n, b.code2).to(dt) for n in k_nf4.LAYER_WEIGHTS}
        lv = {n: (P[n].A16.cpu().to(dt).requires_grad_(True), P[n].B16.cpu().to(dt).requires_grad_(True)) for n in ("q_proj", "v_proj")}
        leaves.append(lv)
        y1 = rms(x, nl.w_in.cpu().to(dt), nl.eps)
        bias = b.bias_qkv.cpu().to(dt)
        outs = []
        for n, sl in (("q_proj", slice(0, H)), ("k_proj", slice(H, H + KV)), ("v_proj", slice(H + KV, H + 2 * KV))):
            o = y1 @ W[n].t() + bias[sl]
            if n in lv:
                A, B = lv[n]
                o = o + P[n].scale * ((y1 * ms[n].to(dt) * ks) @ A.t()) @ B.t()
            outs.append(o)
        q, k, v = rot(outs[0].view(-1, nh, hd)), rot(outs[1].view(-1, nkv, hd)), outs[2].view(-1, nkv, hd)
        rows, at = [], 0
        for n in seq_lens:
            qs, ks_, vs = q[at:at + n], k[at:at + n].repeat_interleave(nh // nkv, 1), v[at:at + n].repeat_interleave(nh // nkv, 1)
            sc = torch.einsum("ihd,jhd->hij", qs, ks_) / hd ** 0.5
            sc = sc.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool), 1), float("-inf"))
            rows.append(torch.einsum("hij,jhd->ihd", sc.softmax(-1), vs).reshape(n, H))
            at += n
        x = x + torch.cat(rows) @ W["o_proj"].t()
        y2 = rms(x, nl.w_post.cpu().to(dt), nl.eps)
        h = F.silu(y2 @ W["gate_proj"].t()) * (y2 @ W["up_proj"].t())
        x = x + h @ W["down_proj"].t()
    return x, leaves


def test_decoder_stack_with_attention_is_one_autograd_node():
    """NormedStack with real rotary + causal grouped-query attention between the projections, called as ONE autograd
    node: output, LoRA gradients (through the masters' .grad) and the input gradient against a plain PyTorch fp64
    model of the same two layers. Tolerances cover the path's fp16 rounding points (activations between kernels)."""
    dev = torch.device("cuda")
    H, I, KV, NH = 256, 512, 128, 4
    seq_lens = [70, 130]
    M = sum(seq_lens)
    ns = stack.NormedStack(H, I, KV, 2, dev, seed=11, n_heads=NH, rope_theta=1.0e4)
    gen = torch.Generator().manual_seed(5)
    x32 = torch.randn(M, H, generator=gen)
    dres = torch.randn(M, H, generator=gen) * 0.5
    ks = 1.0 / float(torch.tensor(0.95, dtype=torch.float32))
    masks = [{n: (torch.rand(M, H, generator=gen) >= 0.05).to(torch.uint8) for n in ("q_proj", "v_proj")} for _ in range(2)]
    masters = ns.lora_masters()
    for t in masters:
        t.requires_grad_(True)
    xin = x32.to(dev).requires_grad_(True)
    out = ns.apply(xin, [{n: m.to(dev) for n, m in ms.items()} for ms in masks], ks, seq_lens)
    assert out.grad_fn is not None
    (out * dres.to(dev)).sum().backward()
    linear.check_status()

    xr = x32.to(torch.float64).requires_grad_(True)
    ref, leaves = _reference_decoder_stack(ns, xr, masks, ks, seq_lens, 1.0e4)
    (ref * dres.to(torch.float64)).sum().backward()
    err, rel = nf4_oracle.errors(out.detach(), ref.detach())
    assert rel <= 3e-3, (err, rel)
    err, rel = nf4_oracle.errors(xin.grad, xr.grad)
    assert rel <= 1e-2, (err, rel)
    it = iter(masters)
    for i in range(2):
        for n in ("q_proj", "v_proj"):
            for ref_leaf in leaves[i][n]:
                got = next(it).grad
                err, rel = nf4_oracle.errors(got, ref_leaf.grad)
                assert rel <= 1e-2, (i, n, err, rel)
