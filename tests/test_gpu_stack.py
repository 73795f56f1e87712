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
