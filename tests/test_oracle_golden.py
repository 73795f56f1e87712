"""The CPU oracle's dequantisation against vectors produced by the reference's own kernel
(tests/golden/make_golden.py ran solution/k_nf4.py:nf4_layer_dequant_kernel under dev/tl_emu.py)."""

import hashlib
import os

import numpy as np
import pytest
import torch

from oracle import nf4_oracle
from tests.golden import make_golden


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_levels_match_reference(golden):
    assert np.array_equal(golden["nf4_levels"], nf4_oracle.NF4_LEVELS)
    from decentrik_prime_b200.k_nf4 import NF4_CODE
    assert np.array_equal(np.array(NF4_CODE, dtype=np.float32), golden["nf4_levels"])


def test_emu3_bit_exact(golden):
    out = nf4_oracle.dequant_ref(golden["emu3_packed"], golden["emu3_qabs"], golden["emu3_scale2"],
                                 golden["emu3_offset2"], golden["emu3_code2"])
    assert out.dtype == np.float16
    assert np.array_equal(out.view(np.uint16), golden["emu3_out"].view(np.uint16))


def test_emu3_prefix_and_range(golden):
    p, q, s2, o2, c2 = (golden["emu3_" + k] for k in ("packed", "qabs", "scale2", "offset2", "code2"))
    pre = nf4_oracle.dequant_ref(p[:512 * 32], q[:512], s2[:2], o2[:2], c2)
    assert sha(pre) == str(golden["emu3_prefix_sha"])
    assert np.array_equal(pre, golden["emu3_out"][:512 * 64])
    rng = nf4_oracle.dequant_ref(p[256 * 32:768 * 32], q[256:768], s2[1:3], o2[1:3], c2)
    assert sha(rng) == str(golden["emu3_range_sha"])
    assert np.array_equal(rng, golden["emu3_out"][256 * 64:768 * 64])


def test_exhaustive_codes(golden):
    out = nf4_oracle.dequant_ref(*make_golden.exhaustive_inputs())
    assert sha(out) == str(golden["exhaustive_sha"])
    assert np.array_equal(out[::97], golden["exhaustive_sample"])


def test_toy_layer(golden):
    layer, code2 = make_golden.toy_layer()
    assert sha(layer.flat.numpy()) == str(golden["toy_flat_sha"]), "the synthetic quantiser drifted"
    out = nf4_oracle.dequant_ref(layer.packed.numpy(), layer.qabs.numpy(), layer.scale2.numpy(),
                                 layer.offset2.numpy(), code2.numpy())
    assert sha(out) == str(golden["toy_out_sha"])
    assert np.array_equal(out[::251], golden["toy_out_sample"])
    # per-weight views agree with the flat dequantisation
    for name, (start, rows, cols) in layer.segments.items():
        w = nf4_oracle.dequant_weight(layer, name, code2)
        assert w.shape == (rows, cols)
        assert torch.equal(w.reshape(-1), torch.from_numpy(out[start:start + rows * cols]))


def test_quantiser_round_trip_is_close():
    """Not a parity claim (the quantise direction is bitsandbytes'): only that the generator emits
    sensible bytes, i.e. dequantised weights approximate the originals like 4-bit NF4 should."""
    from decentrik_prime_b200 import k_nf4, quantize
    gen = torch.Generator().manual_seed(5)
    w = (torch.randn(256, 128, generator=gen) * 0.02).half()
    lin = quantize.FakeLinear4bit(quantize.quantize_nf4(w))
    layer, code2 = k_nf4.repack_layer({"w": lin}, torch.device("cpu"), names=("w",))
    back = nf4_oracle.dequant_weight(layer, "w", code2)
    rel = ((back.float() - w.float()).norm() / w.float().norm()).item()
    assert rel < 0.12, rel


# ------------------------------------------------------------------------------------------------
# RMSNorm producer / backward oracle against the reference's own kernels (run under its emulator)
# ------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def norm_golden():
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "norm_golden.npz"))


@pytest.mark.parametrize("tag", ["a", "b"])
def test_norm_oracle_matches_reference_kernels(norm_golden, tag):
    from oracle import norm_oracle
    g = {k[2:]: norm_golden[k] for k in norm_golden.files if k.startswith(tag + "_")}
    ks, eps = float(g["ks"]), float(g["eps"])
    fwd = norm_oracle.rms_forward_ref(g["x"], g["w"], eps, delta=g["delta"], mq=g["mq"], mv=g["mv"], keep_scale=ks)
    assert np.array_equal(fwd["xout"], g["xout"])
    np.testing.assert_allclose(fwd["rstd"], g["rstd"], rtol=3e-7, atol=0)
    # fp16 outputs: identical up to a last-place flip where the fp32 row sum was added up in another order
    for name, ref in (("y16", g["y"]), ("xq16", g["xq"]), ("xv16", g["xv"])):
        diff = np.abs(fwd[name].astype(np.float64) - ref.astype(np.float64))
        assert (diff <= np.spacing(np.abs(ref)).astype(np.float64)).all(), name
        assert (diff > 0).mean() < 1e-2, name
    plain = norm_oracle.rms_forward_ref(g["x"], g["w"], eps)
    np.testing.assert_allclose(plain["rstd"], g["rstd_nodelta"], rtol=3e-7, atol=0)
    out, out16 = norm_oracle.rms_backward_ref(g["dy16"], float(g["gscale"][0]), g["x"], g["w"], g["rstd"], delta=g["delta"],
                                              dres=g["dres"], lq=g["lq"], lv=g["lv"], mq=g["mq"], mv=g["mv"], keep_scale=ks)
    np.testing.assert_allclose(out, g["bwd_out"], rtol=2e-5, atol=2e-6)
    assert np.abs(out16.astype(np.float64) - g["bwd_out16"].astype(np.float64)).max() <= 4e-3
    out, out16 = norm_oracle.rms_backward_ref(g["dy16"], float(g["gscale"][0]), g["xout"], g["w"], g["rstd"])
    np.testing.assert_allclose(out, g["bwd_plain"], rtol=2e-5, atol=2e-6)
