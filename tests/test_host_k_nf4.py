"""Host-side format logic (decentrik_prime_b200/k_nf4.py) against the reference's rules
(solution/k_nf4.py:81-173, 190-205; solution/test_kernels.py:72-84)."""

import pytest
import torch

from decentrik_prime_b200 import k_nf4, quantize
from tests.golden import make_golden


def test_section_layout_alignment():
    for nq in (256, 1024, 3840, 731136):
        offs, total = k_nf4.section_layout(nq)
        assert all(o % 64 == 0 for o in offs) and total % 64 == 0
        assert offs[0] == 0 and offs[1] >= nq * 32 and offs[2] >= offs[1] + nq
        assert total >= offs[3] + 4 * (nq // 256)


def test_repack_layer_segments_and_views():
    layer, code2 = make_golden.toy_layer()
    at = 0
    for name in k_nf4.LAYER_WEIGHTS:
        rows, cols = make_golden.TOY_SHAPES[name]
        assert layer.segments[name] == (at, rows, cols)
        at += rows * cols
    assert layer.numel == at and layer.n_qblocks == at // 64
    assert layer.packed.numel() == at // 2 and layer.qabs.numel() == at // 64
    assert layer.scale2.dtype == torch.float32 and layer.scale2.numel() == at // 16384
    assert code2.dtype == torch.float32 and code2.numel() == 256
    # q|k|v and gate|up are contiguous (fused-matrix views, reference solution/k_nf4.py:7-10)
    assert layer.segments["k_proj"][0] == layer.segments["q_proj"][0] + 256 * 128


def test_repack_points_modules_at_views():
    lin = {n: quantize.random_nf4_weight(*make_golden.TOY_SHAPES[n], seed=i)
           for i, n in enumerate(k_nf4.LAYER_WEIGHTS)}
    before = {n: lin[n].weight.data.clone() for n in lin}
    layer, _ = k_nf4.repack_layer(lin, torch.device("cpu"))
    for n in lin:
        assert torch.equal(lin[n].weight.data, before[n])
        assert lin[n].weight.data.data_ptr() == layer.weight(n)[0].data_ptr()


def test_repack_rejects_other_formats():
    good = quantize.random_nf4_weight(128, 128, seed=3)
    for field, value in (("quant_type", "fp4"), ("blocksize", 128), ("nested", False)):
        bad = quantize.random_nf4_weight(128, 128, seed=3)
        setattr(bad.weight.quant_state, field, value)
        with pytest.raises(ValueError):
            k_nf4.repack_layer({"w": bad}, torch.device("cpu"), names=("w",))
    other = quantize.random_nf4_weight(128, 128, seed=4, code2=torch.linspace(-0.9, 0.9, 256))
    with pytest.raises(ValueError, match="code tables differ"):
        k_nf4.repack_layer({"a": good, "b": other}, torch.device("cpu"), names=("a", "b"))
    with pytest.raises(ValueError, match="whole absmax blocks"):
        quantize.quantize_nf4(torch.zeros(100, 64, dtype=torch.float16))


def test_dequant_range_alignment_errors():
    layer, code2 = make_golden.toy_layer()
    out = torch.empty(layer.numel, dtype=torch.float16)
    with pytest.raises(ValueError, match="not aligned"):
        k_nf4.dequant_range(layer, 256, layer.n_qblocks, code2, None, out)
    with pytest.raises(ValueError, match="destination not aligned"):
        k_nf4.dequant_range(layer, 0, 1024, code2, None, out, dst=64)
    with pytest.raises(ValueError, match="nf4 table"):
        k_nf4.dequant_layer(layer, code2, torch.zeros(16), out)
    with pytest.raises(ValueError, match="GPU"):        # CPU tensors: no CPU fallback exists
        k_nf4.dequant_layer(layer, code2, None, out)
