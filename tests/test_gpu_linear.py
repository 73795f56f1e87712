"""Fused NF4 + LoRA linear (forward, backward-dX, dA/dB) through the C ABI against the CPU oracle
on identical seeded inputs. Tolerance (the task statement): max-abs-err <= 2e-2 and rel-L2 <= 1e-3
against the fp32/fp64-accumulated oracle O1; dequantised weights bit-exact."""

import pytest
import torch

from decentrik_prime_b200 import _lib, linear
from oracle import nf4_oracle
from tests.problem import make_problem, oracle_weight, to_device

pytestmark = pytest.mark.gpu
MAX_ABS, REL_L2 = 2e-2, 1e-3


def assert_close(name, got, ref):
    err, rel = nf4_oracle.errors(got, ref)
    assert err <= MAX_ABS and rel <= REL_L2, f"{name}: max-abs {err:.3e} rel-L2 {rel:.3e}"


def run_case(N, K, M, lora=True, dropout=0.05, bias=False, force=(0, 0, 0), seed=0, padded=False):
    pr = make_problem(N, K, M, seed=seed, lora=lora, dropout=dropout if lora else 0.0, bias=bias)
    w16 = oracle_weight(pr)
    ref = nf4_oracle.lora_linear_o1(w16, pr.x, pr.dy, pr.bias, pr.A16, pr.B16, pr.scale, pr.mask, pr.keep_scale)
    d = to_device(pr)
    x, dy = d.x, d.dy
    if padded:          # leading dimensions larger than the row: column slices of wider tensors
        x = torch.cat([d.x, torch.full((M, 64), 7.0, dtype=torch.float16, device="cuda")], 1)[:, :K]
        dy = torch.cat([d.dy, torch.full((M, 8), 7.0, dtype=torch.float16, device="cuda")], 1)[:, :N]
    with linear.tune_override(*force):
        y, t = linear.forward(d.w, x, bias=d.bias, lora=d.lora, mask=d.mask, keep_scale=d.keep_scale, want_t=True)
        dx, u = linear.backward_dx(d.w, dy, lora=d.lora, mask=d.mask, keep_scale=d.keep_scale, want_u=True)
        linear.check_status()
    assert_close("y", y, ref["y"])
    assert_close("dx", dx, ref["dx"])
    if lora:
        assert_close("t", t, ref["t"])
        assert_close("u", u, ref["u"])
        dA, dB = linear.lora_grads(dy, x, t, u, pr.scale, mask=d.mask, keep_scale=d.keep_scale)
        assert_close("dA", dA, ref["dA"])
        assert_close("dB", dB, ref["dB"])
    return pr, d, ref


@pytest.mark.parametrize("M", [1, 8, 63, 64, 65, 127, 128, 129, 300])
def test_ragged_rows(M):
    run_case(256, 256, M, seed=M)


@pytest.mark.parametrize("N,K", [(256, 128), (128, 128), (384, 128), (128, 384)])
def test_toy_layer_shapes(N, K):
    """The shapes of the reference's GPU test layer (solution/test_kernels.py:48-49)."""
    run_case(N, K, 200, bias=True, seed=N + K)


def test_no_lora_no_bias():
    run_case(256, 512, 150, lora=False)


def test_lora_without_dropout():
    run_case(256, 256, 256, dropout=0.0, bias=True)


def test_leading_dimensions():
    run_case(256, 256, 130, padded=True, bias=True)


@pytest.mark.parametrize("force", [(1, 128, 1), (2, 128, 1), (1, 256, 1), (2, 256, 1), (1, 128, 3), (2, 256, 2), (2, 256, 4),
                                   (1, 512, 1), (2, 512, 1), (1, 512, 2), (2, 512, 3)])
def test_every_tile_shape_and_split(force):
    """force = (M tiles per CTA, tile columns, splits of the contraction); 512 columns = the CTA-pair kernel."""
    run_case(512, 768, 300, bias=True, force=force, seed=sum(force))


@pytest.mark.parametrize("force", [(1, 128, 2), (1, 512, 2)])
def test_split_contraction_on_a_grid_larger_than_one_wave(force):
    """When all CTAs of a split grid fit the GPU at once the splits of a tile share the final reduction
    (cooperative launch); a larger grid falls back to "the last CTA of a tile adds the partial sums up".
    384 / 192 CTAs here: the fall-back, for the single-CTA and the CTA-pair kernel."""
    run_case(1536, 1536, 2048, bias=True, force=force, seed=5 + force[1])


@pytest.mark.parametrize("M", [200, 1300])
def test_stacked_projections_in_one_launch_match_separate_calls(M):
    """nf4ll_forward_multi on Q|K|V of a packed layer (LoRA on q and v, bias on all, k narrower than a
    256-column tile) and on gate|up equals the three / two single-projection calls."""
    from decentrik_prime_b200 import k_nf4, quantize
    H, KV, I = 512, 128, 1024
    shapes = {"q_proj": (H, H), "k_proj": (KV, H), "v_proj": (KV, H), "o_proj": (H, H),
              "gate_proj": (I, H), "up_proj": (I, H), "down_proj": (H, I)}
    lin = {n: quantize.random_nf4_weight(*shapes[n], seed=40 + i, device="cuda") for i, n in enumerate(k_nf4.LAYER_WEIGHTS)}
    layer, code2 = k_nf4.repack_layer(lin, torch.device("cuda"))
    gen = torch.Generator().manual_seed(M)
    x = torch.randn(M, H, generator=gen).half().cuda()
    ks = float(1.0 / torch.tensor(0.95, dtype=torch.float32))
    def lora(n):
        A = (torch.randn(16, H, generator=gen) * 0.05).half().cuda()
        B = (torch.randn(n, 16, generator=gen) * 0.05).half().cuda()
        return (A, B, 2.0)
    def mask():
        return (torch.rand(M, H, generator=gen) >= 0.05).to(torch.uint8).cuda()
    for names, with_lora in ((("q_proj", "k_proj", "v_proj"), (True, False, True)), (("gate_proj", "up_proj"), (True, True))):
        ws = [linear.Nf4Weight.from_layer(layer, n, code2) for n in names]
        bias = [(torch.randn(w.N, generator=gen) * 0.1).half().cuda() for w in ws]
        loras = [lora(w.N) if on else None for w, on in zip(ws, with_lora)]
        masks = [mask() if on else None for on in with_lora]
        ref_y, ref_t = [], []
        for w, b, l, m in zip(ws, bias, loras, masks):
            y, t = linear.forward(w, x, bias=b, lora=l, mask=m, keep_scale=ks, want_t=True)
            ref_y.append(y); ref_t.append(t)
        wg = linear.Nf4Weight.from_layer_group(layer, names, code2)
        y, ts = linear.forward_multi(wg, x, [(w.N, l, m, ks) for w, l, m in zip(ws, loras, masks)], bias=torch.cat(bias))
        linear.check_status()
        assert_close("stacked y", y, torch.cat(ref_y, 1).double())
        for t, rt in zip(ts, ref_t):
            assert (t is None) == (rt is None)
            if t is not None:
                assert_close("stacked t", t, rt.double())
    with pytest.raises(ValueError):
        linear.forward_multi(wg, x, [(wg.N - 64, None, None, 1.0), (64, None, None, 1.0)])


@pytest.mark.parametrize("M,lora_up,I", [(300, True, 896), (1100, False, 896), (100, True, 896), (300, True, 960)])
def test_gate_up_forward_with_the_gated_product_in_its_epilogue(M, lora_up, I):
    """nf4ll_forward_gate_up against the two single-projection forwards and the stand-alone gated-SiLU
    kernel: g, u within the GEMM tolerance, h bit-identical to the stand-alone kernel applied to the
    stored g, u; M = 100 (short batch) and I = 960 (not a multiple of 128) take the composite path."""
    from decentrik_prime_b200 import k_nf4, quantize
    H = 512
    names = ("gate_proj", "up_proj")
    lin = {n: quantize.random_nf4_weight(I, H, seed=80 + i, device="cuda") for i, n in enumerate(names)}
    layer, code2 = k_nf4.repack_layer(lin, torch.device("cuda"), names=names)
    gen = torch.Generator().manual_seed(M)
    x = torch.randn(M, H, generator=gen).half().cuda()
    ks = float(1.0 / torch.tensor(0.95, dtype=torch.float32))
    def lora():
        return ((torch.randn(16, H, generator=gen) * 0.05).half().cuda(), (torch.randn(I, 16, generator=gen) * 0.05).half().cuda(), 2.0)
    def mask():
        return (torch.rand(M, H, generator=gen) >= 0.05).to(torch.uint8).cuda()
    lg, mg = lora(), mask()
    lu, mu = (lora(), mask()) if lora_up else (None, None)
    wg, wu = (linear.Nf4Weight.from_layer(layer, n, code2) for n in names)
    g0, tg0 = linear.forward(wg, x, lora=lg, mask=mg, keep_scale=ks, want_t=True)
    u0, tu0 = linear.forward(wu, x, lora=lu, mask=mu, keep_scale=ks, want_t=True)
    w = linear.Nf4Weight.from_layer_group(layer, names, code2)
    g, u, h, tg, tu = linear.forward_gate_up(w, x, lg, mg, lu, mu, ks)
    linear.check_status()
    assert_close("g", g, g0.double())
    assert_close("u", u, u0.double())
    assert_close("t_gate", tg, tg0.double())
    assert (tu is None) == (tu0 is None)
    assert torch.equal(h, linear.swiglu_forward(g.contiguous(), u.contiguous()))


def test_config0_q_proj():
    """benchmark configuration 0: W [1536,1536], X [2048,1536], LoRA r=16 alpha=32, dropout 0.05."""
    run_case(1536, 1536, 2048)


def test_accumulate_dx_and_grads():
    """dx of two projections sharing an input summed in-kernel (gate + up), LoRA grads accumulated."""
    pr1, d1, ref1 = run_case(256, 256, 200, seed=11)
    pr2 = make_problem(384, 256, 200, seed=12)
    w2 = oracle_weight(pr2)
    ref2 = nf4_oracle.lora_linear_o1(w2, pr2.x, pr2.dy, None, pr2.A16, pr2.B16, pr2.scale, pr2.mask, pr2.keep_scale)
    d2 = to_device(pr2)
    dx, _ = linear.backward_dx(d1.w, d1.dy, lora=d1.lora, mask=d1.mask, keep_scale=d1.keep_scale)
    dx, _ = linear.backward_dx(d2.w, d2.dy, lora=d2.lora, mask=d2.mask, keep_scale=d2.keep_scale, out=dx, accumulate=True)
    linear.check_status()
    assert_close("dx1+dx2", dx, ref1["dx"] + ref2["dx"])
    _, t = linear.forward(d1.w, d1.x, lora=d1.lora, mask=d1.mask, keep_scale=d1.keep_scale, want_t=True)
    _, u = linear.backward_dx(d1.w, d1.dy, lora=d1.lora, mask=d1.mask, keep_scale=d1.keep_scale, want_u=True)
    dA, dB = linear.lora_grads(d1.dy, d1.x, t, u, pr1.scale, mask=d1.mask, keep_scale=d1.keep_scale)
    linear.lora_grads(d1.dy, d1.x, t, u, pr1.scale, mask=d1.mask, keep_scale=d1.keep_scale, dA=dA, dB=dB, accumulate=True)
    assert_close("2dA", dA, 2 * ref1["dA"])
    assert_close("2dB", dB, 2 * ref1["dB"])


def test_autograd_function_matches_raw_calls():
    pr = make_problem(256, 256, 96, seed=21)
    w16 = oracle_weight(pr)
    ref = nf4_oracle.lora_linear_o1(w16, pr.x, pr.dy, None, pr.A16, pr.B16, pr.scale, pr.mask, pr.keep_scale)
    d = to_device(pr)
    x = d.x.reshape(2, 48, 256).clone().requires_grad_(True)
    A = pr.A16.float().cuda().requires_grad_(True)     # fp32 masters whose fp16 shadows equal the oracle's
    B = pr.B16.float().cuda().requires_grad_(True)
    y = linear.nf4_lora_linear(x, d.w, lora=(A, B, pr.scale), mask=d.mask.reshape(2, 48, 256), keep_scale=d.keep_scale)
    y.backward(d.dy.reshape(2, 48, 256))
    assert_close("y", y.reshape(96, 256), ref["y"])
    assert_close("dx", x.grad.reshape(96, 256), ref["dx"])
    assert A.grad.dtype == torch.float32 and B.grad.dtype == torch.float32
    assert_close("dA", A.grad, ref["dA"])
    assert_close("dB", B.grad, ref["dB"])


def test_full_size_linearity_property():
    """At a full-size shape (1.5B gate_proj, M=2048) the oracle is too slow to run in full, so use
    properties of the map: a sampled set of output rows equals the oracle on those rows, and
    forward(x1 + x2) = forward(x1) + forward(x2) within fp16 rounding (no bias, no dropout)."""
    N, K, M = 8960, 1536, 2048
    pr = make_problem(N, K, M, seed=31, lora=True, dropout=0.05)
    d = to_device(pr)
    y, _ = linear.forward(d.w, d.x, lora=d.lora, mask=d.mask, keep_scale=d.keep_scale)
    dx, _ = linear.backward_dx(d.w, d.dy, lora=d.lora, mask=d.mask, keep_scale=d.keep_scale)
    linear.check_status()
    rows = torch.tensor([0, 1, 127, 128, 255, 256, 1000, 2047])
    w16 = oracle_weight(pr)
    ref = nf4_oracle.lora_linear_o1(w16, pr.x[rows], pr.dy[rows], None, pr.A16, pr.B16, pr.scale, pr.mask[rows], pr.keep_scale)
    assert_close("y rows", y[rows.cuda()], ref["y"])
    assert_close("dx rows", dx[rows.cuda()], ref["dx"])
    x2 = torch.randn(M, K, generator=torch.Generator().manual_seed(5)).half().cuda()
    ya, _ = linear.forward(d.w, d.x, lora=d.lora)
    yb, _ = linear.forward(d.w, x2, lora=d.lora)
    yab, _ = linear.forward(d.w, (d.x.float() + x2.float()).half(), lora=d.lora)
    err, rel = nf4_oracle.errors(yab, ya.float() + yb.float())
    assert rel <= 2e-3, (err, rel)


def test_rejects_bad_arguments():
    pr = make_problem(256, 256, 16, seed=41)
    d = to_device(pr)
    with pytest.raises(ValueError):
        linear.forward(d.w, d.x[:, :128])
    with pytest.raises(ValueError):
        linear.forward(d.w, d.x.float())
    with pytest.raises(ValueError):
        linear.forward(d.w, d.x.cpu())
    with pytest.raises(ValueError):
        linear.forward(d.w, d.x, lora=(d.A16[:8], d.B16[:, :8].contiguous(), 2.0))      # rank 8
    with pytest.raises(ValueError):
        linear.forward(d.w, d.x, workspace=torch.empty(16, dtype=torch.uint8, device="cuda"), lora=d.lora)


def test_swiglu_kernels_match_fp32_reference():
    """The gated-SiLU glue between up and down against a plain PyTorch fp32 statement of the
    reference's arithmetic (solution/k_mlp.py:21-47); fp16 outputs, so tolerance is one fp16 ulp."""
    gen = torch.Generator().manual_seed(3)
    M, I = 77, 8960
    g = (torch.randn(M, I, generator=gen) * 2).half().cuda()
    u = torch.randn(M, I, generator=gen).half().cuda()
    dh = torch.randn(M, I, generator=gen).half().cuda()
    h = linear.swiglu_forward(g, u)
    gf, uf, df = g.float(), u.float(), dh.float()
    sig = torch.sigmoid(gf)
    torch.testing.assert_close(h.float(), (gf * sig * uf).half().float(), atol=2e-3, rtol=2e-3)
    dg, du = linear.swiglu_backward(g, u, dh, inplace=False)
    torch.testing.assert_close(du.float(), (df * gf * sig).half().float(), atol=2e-3, rtol=2e-3)
    torch.testing.assert_close(dg.float(), (df * uf * sig * (1 + gf * (1 - sig))).half().float(), atol=2e-3, rtol=2e-3)
    g2, u2 = g.clone(), u.clone()
    linear.swiglu_backward(g2, u2, dh, inplace=True)
    assert torch.equal(g2, dg) and torch.equal(u2, du)


def test_mlp_block_fused_glue_matches_pytorch_glue():
    from decentrik_prime_b200 import blocks
    outs = []
    for fused in (True, False):
        blk = blocks.MlpBlock(256, 512, seed=9, device=torch.device("cuda"), fused_glue=fused)
        gen = torch.Generator().manual_seed(1)
        x = torch.randn(200, 256, generator=gen).half().cuda()
        dy = torch.randn(200, 256, generator=gen).half().cuda()
        masks = [(torch.rand(200, k, generator=gen) >= 0.05).to(torch.uint8).cuda() for k in (256, 256, 512)]
        y = blk.forward(x, masks, 1.0 / 0.95)
        dx = blk.backward(dy)
        outs.append((y.float(), dx.float(), blk.down.dA.clone(), blk.gate.dB.clone()))
    linear.check_status()
    for a, b in zip(*outs):
        err, rel = nf4_oracle.errors(a, b)
        assert rel <= 2e-3, (err, rel)


def test_block_step_replays_from_a_cuda_graph():
    """Every launch of a block step (cluster, cooperative and programmatic-dependent launches included)
    can be captured into a CUDA graph; the replay gives the eager results bit for bit (the gradient
    reductions use atomics, so gradients are compared with a tolerance)."""
    from decentrik_prime_b200 import blocks
    dev = torch.device("cuda")
    bucket = blocks.GradBucket(blocks.MlpBlock.grad_numel(1536, 1024), dev)
    blk = blocks.MlpBlock(1536, 1024, seed=21, device=dev, bucket=bucket)     # down_proj: 1536-wide output, split contraction
    gen = torch.Generator().manual_seed(2)
    M = 2048
    x = torch.randn(M, 1536, generator=gen).half().cuda()
    dy = torch.randn(M, 1536, generator=gen).half().cuda()
    masks = [(torch.rand(M, k, generator=gen) >= 0.05).to(torch.uint8).cuda() for k in (1536, 1536, 1024)]
    ks = 1.0 / 0.95
    for _ in range(2):
        y0 = blk.forward(x, masks, ks)
        dx0 = blk.backward(dy)
    g0 = bucket.flat.clone()
    y0, dx0 = y0.clone(), dx0.clone()
    side = torch.cuda.Stream(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            y1 = blk.forward(x, masks, ks)
            dx1 = blk.backward(dy)
    torch.cuda.synchronize()
    for _ in range(3):
        graph.replay()
    linear.check_status()
    assert torch.equal(y1, y0) and torch.equal(dx1, dx0)
    err, rel = nf4_oracle.errors(bucket.flat, g0.double())
    assert rel <= 1e-5, (err, rel)


def test_block_gradients_on_a_side_stream_match_the_single_stream_step():
    """The dA/dB kernels issued on a side stream (forked after the dX launch of their projection, joined at
    the end of the backward) give what the single-stream step gives, eagerly and from a captured graph."""
    from decentrik_prime_b200 import blocks
    dev = torch.device("cuda")
    bucket = blocks.GradBucket(blocks.MlpBlock.grad_numel(1536, 1024), dev)
    blk = blocks.MlpBlock(1536, 1024, seed=23, device=dev, bucket=bucket)
    gen = torch.Generator().manual_seed(4)
    M = 1024
    x = torch.randn(M, 1536, generator=gen).half().cuda()
    dy = torch.randn(M, 1536, generator=gen).half().cuda()
    masks = [(torch.rand(M, k, generator=gen) >= 0.05).to(torch.uint8).cuda() for k in (1536, 1536, 1024)]
    ks = 1.0 / 0.95
    y0 = blk.forward(x, masks, ks)
    dx0 = blk.backward(dy).clone()
    g0 = bucket.flat.clone()
    blk.use_grad_stream()
    for _ in range(2):
        blk.forward(x, masks, ks)
        dx1 = blk.backward(dy)
    torch.cuda.synchronize()
    assert torch.equal(dx1, dx0)
    err, rel = nf4_oracle.errors(bucket.flat, g0.double())
    assert rel <= 1e-5, (err, rel)
    side = torch.cuda.Stream(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            blk.forward(x, masks, ks)
            dx2 = blk.backward(dy)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    linear.check_status()
    assert torch.equal(dx2, dx0)
    err, rel = nf4_oracle.errors(bucket.flat, g0.double())
    assert rel <= 1e-5, (err, rel)


def test_split_contraction_is_stable_under_back_to_back_launches():
    """The split-contraction path (partial sums through scratch, the splits of a tile share the final
    reduction) must give the same bits on every launch: 100 forwards queued back to back without host
    syncs, each compared with the single-pass result. Guards the ordering between the elected lane that
    issues the TMA stores of the partial sums and the barrier that lets its warp-mates reuse the staging,
    and the hand-over of partial sums between the CTAs of a tile."""
    pr = make_problem(1536, 1536, 2048, seed=61, lora=False, bias=True)
    d = to_device(pr)
    with linear.tune_override(splits=1):
        y0, _ = linear.forward(d.w, d.x, bias=d.bias)
    outs = [linear.forward(d.w, d.x, bias=d.bias)[0] for _ in range(100)]
    linear.check_status()
    assert all(torch.equal(o, outs[0]) for o in outs), "split-K results differ between launches"
    err, rel = nf4_oracle.errors(outs[0], y0.float())
    assert err <= 2e-3 and rel <= 1e-4, (err, rel)      # same sums, only the fp32 addition order differs
    # with LoRA too: at this batch size the rank-16 projection is computed without atomics
    pl = make_problem(1536, 1536, 2048, seed=62, lora=True, dropout=0.05)
    dl = to_device(pl)
    outs = [linear.forward(dl.w, dl.x, lora=dl.lora, mask=dl.mask, keep_scale=dl.keep_scale)[0] for _ in range(50)]
    dxs = [linear.backward_dx(dl.w, dl.dy, lora=dl.lora, mask=dl.mask, keep_scale=dl.keep_scale)[0] for _ in range(50)]
    linear.check_status()
    assert all(torch.equal(o, outs[0]) for o in outs), "forward with LoRA differs between launches"
    assert all(torch.equal(o, dxs[0]) for o in dxs), "backward-dX with LoRA differs between launches"
