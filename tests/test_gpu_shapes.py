"""Parity of the fused NF4 + LoRA linear at the benchmark's full shapes (configurations 1, 3 and 4)
and of every variant of the small-batch weight-streaming kernels, through the C ABI against the CPU
oracle O1 (fp64). Weights are quantised on the GPU from a seeded CPU draw; the oracle dequantises the
same packed bytes on the CPU. Where the full fp64 product would take minutes, sampled token rows (all
output columns) or sampled weight rows (all tokens) are compared instead; the rank-16 quantities
t, u, dA and dB are always compared in full. Tolerance: max-abs-err <= 2e-2 and rel-L2 <= 1e-3."""

import ctypes

import numpy as np
import pytest
import torch

from decentrik_prime_b200 import _lib, k_nf4, linear, quantize
from oracle import nf4_oracle
from tests.problem import make_problem, oracle_weight, to_device

pytestmark = pytest.mark.gpu
MAX_ABS, REL_L2 = 2e-2, 1e-3


def assert_close(name, got, ref):
    err, rel = nf4_oracle.errors(got, ref)
    assert err <= MAX_ABS and rel <= REL_L2, f"{name}: max-abs {err:.3e} rel-L2 {rel:.3e}"


def oracle_rows(layer, name, code2, rows):
    """fp16 rows `rows` of one weight of a packed layer, dequantised on the CPU (every row is a whole
    number of quantisation blocks because the column count is a multiple of 64)."""
    pk, qa, s2, o2, n_rows, cols = layer.weight(name)
    bpr = cols // 64
    out = torch.empty(len(rows), cols, dtype=torch.float16)
    pk, qa, s2, o2, c2 = (t.cpu().numpy() for t in (pk, qa, s2, o2, code2))
    for i, r in enumerate(rows):
        b0 = r * bpr
        g = np.arange(b0, b0 + bpr) // 256         # second-level block of each quantisation block
        prod = (c2[qa[b0:b0 + bpr]] * s2[g]).astype(np.float32)
        am = (prod + o2[g]).astype(np.float32)
        by = pk[b0 * 32:(b0 + bpr) * 32]
        per_byte = np.repeat(am, 32)
        row = np.empty(cols, dtype=np.float16)
        row[0::2] = (nf4_oracle.NF4_LEVELS[by >> 4] * per_byte).astype(np.float32).astype(np.float16)
        row[1::2] = (nf4_oracle.NF4_LEVELS[by & 15] * per_byte).astype(np.float32).astype(np.float16)
        out[i] = torch.from_numpy(row)
    return out


def test_oracle_rows_helper_matches_full_dequant():
    pr = make_problem(256, 384, 4, seed=1)
    rows = [0, 5, 255]
    assert torch.equal(oracle_rows(pr.layer, "w", pr.code2, rows), oracle_weight(pr)[rows])


# ----------------------------------------------------------------------------------------------
# small-batch forward: every variant the launcher can pick
# ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("N,K", [(256, 256), (256, 384), (256, 128), (128, 640)])
@pytest.mark.parametrize("M", [1, 7, 8, 9, 16, 17, 33, 64])
def test_small_batch_forward_variants(N, K, M):
    """Token tiles of 8 (M <= 8) and 16 (M <= 16), rows that are and are not a multiple of four
    quantisation blocks (K = 384, 128, 640), with and without bias / LoRA / dropout."""
    for lora, bias in ((True, True), (False, False)):
        pr = make_problem(N, K, M, seed=1000 + N + K + M, lora=lora, dropout=0.05 if lora else 0.0, bias=bias)
        ref = nf4_oracle.lora_linear_o1(oracle_weight(pr), pr.x, None, pr.bias, pr.A16, pr.B16, pr.scale, pr.mask, pr.keep_scale)
        d = to_device(pr)
        y, t = linear.forward(d.w, d.x, bias=d.bias, lora=d.lora, mask=d.mask, keep_scale=d.keep_scale, want_t=lora)
        linear.check_status()
        assert_close(f"y lora={lora}", y, ref["y"])
        if lora:
            assert_close("t", t, ref["t"])


@pytest.mark.parametrize("N,K", [(256, 256), (192, 256), (256, 384), (640, 1024), (4096, 512), (256, 320), (512, 2112)])
@pytest.mark.parametrize("M", [1, 16, 17, 33, 64])
def test_swapped_operand_kernel_variants(N, K, M):
    """The swapped-operand tensor-core kernel (weights as the MMA's 128-row operand, 16 / 32 / 64 token columns),
    forced through the tuning hook: one and several slices of the contraction, tiles with fewer than 128 weight
    rows (N = 192), last groups of one and two quantisation blocks (K = 320, 2112, 384),
    row lengths that are not a multiple of four blocks (K = 384, 320: absmax codes fetched byte by byte)."""
    pr = make_problem(N, K, M, seed=3000 + N + K + M, lora=True, dropout=0.05, bias=True)
    ref = nf4_oracle.lora_linear_o1(oracle_weight(pr), pr.x, None, pr.bias, pr.A16, pr.B16, pr.scale, pr.mask, pr.keep_scale)
    d = to_device(pr)
    ws = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
    for slices in (0, 1, 2, 3):
        with linear.tune_override(splits=slices, flags=4):
            y, t = linear.forward(d.w, d.x, bias=d.bias, lora=d.lora, mask=d.mask, keep_scale=d.keep_scale, workspace=ws, want_t=True)
        linear.check_status()
        assert_close(f"y slices={slices}", y, ref["y"])
        assert_close("t", t, ref["t"])
    # no LoRA, no bias: the epilogue's plain path
    pr = make_problem(N, K, M, seed=3100 + N + K + M, lora=False, dropout=0.0)
    ref = nf4_oracle.lora_linear_o1(oracle_weight(pr), pr.x, None, None, None, None, 1.0, None, 1.0)
    d = to_device(pr)
    with linear.tune_override(flags=4):
        y, _ = linear.forward(d.w, d.x, workspace=ws)
    linear.check_status()
    assert_close("y plain", y, ref["y"])


@pytest.mark.parametrize("M", [17, 32, 33, 64])
def test_streaming_kernel_forced_up_to_64_rows(M):
    """The register-level weight-streaming kernel with four and eight token tiles (17..64 rows), which the
    default dispatch never picks: forced through the tuning hook."""
    for N, K in ((256, 256), (256, 384)):
        pr = make_problem(N, K, M, seed=3200 + N + K + M, lora=True, dropout=0.05, bias=True)
        ref = nf4_oracle.lora_linear_o1(oracle_weight(pr), pr.x, None, pr.bias, pr.A16, pr.B16, pr.scale, pr.mask, pr.keep_scale)
        d = to_device(pr)
        ws = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
        for slices in (0, 2):
            with linear.tune_override(splits=slices, flags=2):
                y, _ = linear.forward(d.w, d.x, bias=d.bias, lora=d.lora, mask=d.mask, keep_scale=d.keep_scale, workspace=ws)
            linear.check_status()
            assert_close(f"y slices={slices}", y, ref["y"])


CONFIG4_SHAPES = {"q/o": (5120, 5120), "gate/up": (27648, 5120), "down": (5120, 27648)}


@pytest.mark.parametrize("which", list(CONFIG4_SHAPES))
def test_config4_weight_stream_shapes(which):
    """Benchmark configuration 4 (Qwen2.5-32B shapes, forward only, LoRA r=16 fused) at M in {1, 8, 16, 64}:
    y on 96 sampled output columns (weight rows) for every token."""
    N, K = CONFIG4_SHAPES[which]
    pr = make_problem(N, K, 64, seed=4000 + N % 97, lora=True, dropout=0.0, bias=True, device="cuda")
    gen = torch.Generator().manual_seed(N + K)
    cols = sorted(set([0, 1, 15, 16, 127, 128, 255, 256, N - 129, N - 128, N - 17, N - 16, N - 1] +
                      torch.randint(0, N, (83,), generator=gen).tolist()))
    w_rows = oracle_rows(pr.layer, "w", pr.code2, cols)
    d = to_device(pr)
    for M in (1, 8, 16, 64):
        x = pr.x[:M].contiguous()
        ref = nf4_oracle.lora_linear_o1(w_rows, x, None, pr.bias[cols], pr.A16, pr.B16[cols], pr.scale, None, 1.0)
        y, t = linear.forward(d.w, d.x[:M].contiguous(), bias=d.bias, lora=d.lora, want_t=True)
        linear.check_status()
        assert_close(f"{which} M={M} y", y[:, cols], ref["y"])
        assert_close(f"{which} M={M} t", t, ref["t"])
        # the whole output must be finite and of plausible size (no tile left unwritten)
        assert torch.isfinite(y).all()
        assert float(y.float().abs().max()) < 50.0


@pytest.mark.parametrize("N,K", [(18944, 3584), (3584, 18944), (3584, 3584)])
def test_short_batches_on_7b_shapes(N, K):
    """Every batch size class of the default dispatch (streaming kernel, swapped-operand kernel with 16 / 32 / 64
    token columns, 128-row tiles) at the Qwen2.5-7B shapes, whose rows are 56 and 296 quantisation blocks long
    (14 and 74 groups of four): M in {1, 8, 9, 16, 24, 33, 64, 65} with LoRA, dropout and bias; y on sampled output
    columns for every token, t in full."""
    pr = make_problem(N, K, 65, seed=4500 + N % 89, lora=True, dropout=0.05, bias=True, device="cuda")
    gen = torch.Generator().manual_seed(N * 3 + K)
    cols = sorted(set([0, 1, 127, 128, N - 128, N - 1] + torch.randint(0, N, (58,), generator=gen).tolist()))
    w_rows = oracle_rows(pr.layer, "w", pr.code2, cols)
    d = to_device(pr)
    for M in (1, 8, 9, 16, 24, 33, 64, 65):
        ref = nf4_oracle.lora_linear_o1(w_rows, pr.x[:M], None, pr.bias[cols], pr.A16, pr.B16[cols], pr.scale, pr.mask[:M], pr.keep_scale)
        y, t = linear.forward(d.w, d.x[:M].contiguous(), bias=d.bias, lora=d.lora, mask=d.mask[:M].contiguous(),
                              keep_scale=d.keep_scale, want_t=True)
        linear.check_status()
        assert_close(f"M={M} y", y[:, cols], ref["y"])
        assert_close(f"M={M} t", t, ref["t"])
        assert torch.isfinite(y).all()


# ----------------------------------------------------------------------------------------------
# training shapes: configuration 3 (Qwen2.5-7B) and configuration 1 (Qwen2.5-1.5B MLP), M = 2048
# ----------------------------------------------------------------------------------------------
ROWS = [0, 1, 127, 128, 255, 256, 511, 1000, 1023, 1024, 2046, 2047]


def full_shape_case(N, K, M, lora, dropout, bias, seed):
    pr = make_problem(N, K, M, seed=seed, lora=lora, dropout=dropout if lora else 0.0, bias=bias, device="cuda")
    w16 = oracle_weight(pr)
    d = to_device(pr)
    y, t = linear.forward(d.w, d.x, bias=d.bias, lora=d.lora, mask=d.mask, keep_scale=d.keep_scale, want_t=lora)
    dx, u = linear.backward_dx(d.w, d.dy, lora=d.lora, mask=d.mask, keep_scale=d.keep_scale, want_u=lora)
    linear.check_status()
    rows = torch.tensor(ROWS)
    m_rows = None if pr.mask is None else pr.mask[rows]
    ref = nf4_oracle.lora_linear_o1(w16, pr.x[rows], pr.dy[rows], pr.bias, pr.A16, pr.B16, pr.scale, m_rows, pr.keep_scale)
    assert_close("y rows", y[rows.cuda()], ref["y"])
    assert_close("dx rows", dx[rows.cuda()], ref["dx"])
    assert torch.isfinite(y).all() and torch.isfinite(dx).all()
    if lora:
        # rank-16 quantities in full, fp64 on the CPU: cheap because one factor is 16 wide
        xd = nf4_oracle.drop_ref(pr.x, pr.mask, pr.keep_scale).double()
        t_ref = xd @ pr.A16.double().t()
        u_ref = pr.scale * (pr.dy.double() @ pr.B16.double())
        assert_close("t", t, t_ref)
        assert_close("u", u, u_ref)
        dA, dB = linear.lora_grads(d.dy, d.x, t, u, pr.scale, mask=d.mask, keep_scale=d.keep_scale)
        assert_close("dA", dA, u_ref.t() @ xd)
        assert_close("dB", dB, pr.scale * (pr.dy.double().t() @ t_ref))


@pytest.mark.parametrize("name,N,K,lora", [("q", 3584, 3584, True), ("v", 512, 3584, True), ("gate", 18944, 3584, False),
                                           ("down", 3584, 18944, False)])
def test_config3_shapes(name, N, K, lora):
    full_shape_case(N, K, 2048, lora=lora, dropout=0.05, bias=name in ("q", "v"), seed=300 + N % 89)


@pytest.mark.parametrize("name,N,K", [("gate", 8960, 1536), ("down", 1536, 8960)])
def test_config1_shapes(name, N, K):
    """LoRA + dropout on every projection; down_proj's backward runs the in-accumulator mask pass on 280 tiles."""
    full_shape_case(N, K, 2048, lora=True, dropout=0.05, bias=False, seed=100 + N % 89)


# ----------------------------------------------------------------------------------------------
# stacked launches directly against the oracle
# ----------------------------------------------------------------------------------------------
def _packed_layer(H, KV, I, seed):
    shapes = {"q_proj": (H, H), "k_proj": (KV, H), "v_proj": (KV, H), "o_proj": (H, H),
              "gate_proj": (I, H), "up_proj": (I, H), "down_proj": (H, I)}
    lin = {n: quantize.random_nf4_weight(*shapes[n], seed=seed + i, device="cuda") for i, n in enumerate(k_nf4.LAYER_WEIGHTS)}
    return k_nf4.repack_layer(lin, torch.device("cuda"))


@pytest.mark.parametrize("M", [200, 1300])
def test_stacked_forward_against_oracle(M):
    """nf4ll_forward_multi on Q|K|V (LoRA on q and v, bias everywhere) and nf4ll_forward_gate_up (g, u and
    h = silu(g) * u) against the fp64 oracle of each projection."""
    H, KV, I = 512, 128, 1024
    layer, code2 = _packed_layer(H, KV, I, seed=140)
    gen = torch.Generator().manual_seed(M)
    x = torch.randn(M, H, generator=gen).half()
    ks = float(1.0 / torch.tensor(0.95, dtype=torch.float32))

    def lora(n):
        return ((torch.randn(16, H, generator=gen) * 0.05).half(), (torch.randn(n, 16, generator=gen) * 0.05).half(), 2.0)

    def mask():
        return (torch.rand(M, H, generator=gen) >= 0.05).to(torch.uint8)

    def dev(l):
        return None if l is None else (l[0].cuda(), l[1].cuda(), l[2])

    names = ("q_proj", "k_proj", "v_proj")
    rows = [layer.segments[n][1] for n in names]
    bias = [(torch.randn(r, generator=gen) * 0.1).half() for r in rows]
    loras = [lora(rows[0]), None, lora(rows[2])]
    masks = [mask(), None, mask()]
    wg = linear.Nf4Weight.from_layer_group(layer, names, code2)
    y, ts = linear.forward_multi(wg, x.cuda(), [(r, dev(l), None if m is None else m.cuda(), ks) for r, l, m in zip(rows, loras, masks)],
                                 bias=torch.cat(bias).cuda())
    linear.check_status()
    at = 0
    for n, r, b, l, m, t in zip(names, rows, bias, loras, masks, ts):
        w16 = nf4_oracle.dequant_weight(layer, n, code2)
        A, B, s = (None, None, 1.0) if l is None else l
        ref = nf4_oracle.lora_linear_o1(w16, x, None, b, A, B, s, m, ks if m is not None else 1.0)
        assert_close(f"{n} y", y[:, at:at + r], ref["y"])
        if l is not None:
            assert_close(f"{n} t", t, ref["t"])
        at += r

    lg, lu, mg, mu = lora(I), lora(I), mask(), mask()
    w = linear.Nf4Weight.from_layer_group(layer, ("gate_proj", "up_proj"), code2)
    g, u, h, tg, tu = linear.forward_gate_up(w, x.cuda(), dev(lg), mg.cuda(), dev(lu), mu.cuda(), ks)
    linear.check_status()
    rg = nf4_oracle.lora_linear_o1(nf4_oracle.dequant_weight(layer, "gate_proj", code2), x, None, None, lg[0], lg[1], 2.0, mg, ks)
    ru = nf4_oracle.lora_linear_o1(nf4_oracle.dequant_weight(layer, "up_proj", code2), x, None, None, lu[0], lu[1], 2.0, mu, ks)
    assert_close("g", g, rg["y"])
    assert_close("u", u, ru["y"])
    assert_close("t_gate", tg, rg["t"])
    assert_close("t_up", tu, ru["t"])
    g16, u16 = rg["y"].half().double(), ru["y"].half().double()
    assert_close("h", h, g16 * torch.sigmoid(g16) * u16)
