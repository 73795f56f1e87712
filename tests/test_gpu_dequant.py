"""Standalone dequantisation kernel against the reference's golden vectors and the oracle, through
the k_nf4-compatible launchers (what solution/test_kernels.py:41-84 checks against bitsandbytes)."""

import hashlib

import numpy as np
import pytest
import torch

from decentrik_prime_b200 import k_nf4
from oracle import nf4_oracle
from tests.golden import make_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def gpu_dequant(packed, qabs, scale2, offset2, code2, nq=None):
    t = [torch.from_numpy(np.ascontiguousarray(a)).to(DEV) for a in (packed, qabs, scale2, offset2, code2)]
    nq = qabs.size if nq is None else nq
    out = torch.zeros(nq * 64, dtype=torch.float16, device=DEV)
    k_nf4.dequant_tensors(*t[:4], nq, t[4], None, out)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_emu3_bit_exact_and_ranges(golden):
    p, q, s2, o2, c2 = (golden["emu3_" + k] for k in ("packed", "qabs", "scale2", "offset2", "code2"))
    out = gpu_dequant(p, q, s2, o2, c2)
    assert np.array_equal(out.view(np.uint16), golden["emu3_out"].view(np.uint16))
    assert sha(gpu_dequant(p[:512 * 32], q[:512], s2[:2], o2[:2], c2)) == str(golden["emu3_prefix_sha"])
    assert sha(gpu_dequant(p[256 * 32:768 * 32], q[256:768], s2[1:3], o2[1:3], c2)) == str(golden["emu3_range_sha"])


def test_exhaustive_codes(golden):
    out = gpu_dequant(*make_golden.exhaustive_inputs())
    assert sha(out) == str(golden["exhaustive_sha"])


def test_toy_layer_and_split_ranges(golden):
    cpu_layer, code2 = make_golden.toy_layer()
    flat = cpu_layer.flat.to(DEV)
    layer = k_nf4.PackedLayer(flat, cpu_layer.offsets, cpu_layer.n_qblocks, cpu_layer.segments)
    code2 = code2.to(DEV)
    nf4 = torch.tensor(k_nf4.NF4_CODE, dtype=torch.float32, device=DEV)
    out = torch.empty(layer.numel, dtype=torch.float16, device=DEV)
    k_nf4.dequant_layer(layer, code2, nf4, out)
    assert sha(out.cpu().numpy()) == str(golden["toy_out_sha"])
    # split dequantisation, the second part on a side stream (solution/test_kernels.py:72-84)
    split = k_nf4.RANGE_ALIGN
    assert layer.n_qblocks > split
    out3 = torch.zeros_like(out)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        k_nf4.dequant_range(layer, split, layer.n_qblocks, code2, nf4, out3)
    torch.cuda.current_stream().wait_stream(side)
    assert not out3[:split * 64].any(), "range dequant wrote outside its range"
    k_nf4.dequant_range(layer, 0, split, code2, nf4, out3)
    assert torch.equal(out3, out), "split dequant differs from the whole-layer dequant"
    with pytest.raises(ValueError):
        k_nf4.dequant_range(layer, 256, layer.n_qblocks, code2, nf4, out3)
    # a range into a shared region (dst offset), as the reference's gate/up/down turn-taking uses
    shared = torch.zeros(split * 64 * 2, dtype=torch.float16, device=DEV)
    k_nf4.dequant_range(layer, split, 2 * split, code2, nf4, shared, dst=0)
    assert torch.equal(shared[:split * 64], out[split * 64:2 * split * 64])
    assert not shared[split * 64:].any()


def test_large_random_against_oracle():
    """Full-size check (a 1.5B gate_proj's worth of blocks) through a size-independent property:
    the kernel equals the oracle on a strided sample and the whole output hashes identically when
    the same bytes are dequantised as two halves."""
    rng = np.random.default_rng(7)
    nq = 8960 * 1536 // 64
    p = rng.integers(0, 256, nq * 32, dtype=np.uint8)
    q = rng.integers(0, 256, nq, dtype=np.uint8)
    c2 = np.linspace(-1, 1, 256, dtype=np.float32)
    s2 = rng.uniform(0.001, 0.02, nq // 256).astype(np.float32)
    o2 = np.full(nq // 256, 0.02, dtype=np.float32)
    out = gpu_dequant(p, q, s2, o2, c2)
    ref = nf4_oracle.dequant_ref(p, q, s2, o2, c2)
    assert np.array_equal(out.view(np.uint16), ref.view(np.uint16))
    half = (nq // 2) // 1024 * 1024
    a = gpu_dequant(p[:half * 32], q[:half], s2[:half // 256], o2[:half // 256], c2)
    b = gpu_dequant(p[half * 32:], q[half:], s2[half // 256:], o2[half // 256:], c2)
    assert np.array_equal(np.concatenate([a, b]).view(np.uint16), out.view(np.uint16))
