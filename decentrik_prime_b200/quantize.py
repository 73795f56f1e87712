"""Synthetic NF4 double-quantiser: fp16 weights -> the byte format the kernels read.

The reference never quantises itself: bitsandbytes does it at model-load time, and that package
(and its source) is not available here. This quantiser is therefore this repository's own: it
produces *valid inputs* in the reference's format (solution/k_nf4.py:16-21) for tests and
benchmarks; it is not claimed to reproduce bitsandbytes' code choice bit for bit. Only the
dequantise direction has a parity contract, and both the kernels and the checker consume the same
bytes produced here.

    absmax[b]   = max |w| over block b of 64 weights (fp32)
    code        = index of the NF4 level nearest to w / absmax[b]
    offset      = mean(absmax)
    scale2[g]   = max |absmax - offset| over group g of 256 blocks
    qabs[b]     = index of the code2 entry nearest to (absmax[b] - offset) / scale2[b // 256]

`code2` is an input of the format (any sorted 256-entry fp32 table in [-1, 1]); the default is the
linear table the reference's own benchmark uses (dev/bench_kernels.py:203).
"""

from types import SimpleNamespace

import torch

from .k_nf4 import NF4_CODE, QBLOCK, QBLOCKS2


def default_code2(device="cpu"):
    return torch.linspace(-1.0, 1.0, 256, dtype=torch.float32, device=device)


def _nearest_index(values, table):
    """Index of the nearest entry of the sorted 1-D `table` for every element of `values`."""
    mids = (table[1:] + table[:-1]) * 0.5
    return torch.bucketize(values, mids)


class Quantized4bit:
    """Stands in for a bitsandbytes Params4bit: `.data` holds the packed bytes [n/2, 1] and
    `.quant_state` the nested state, with the attribute names k_nf4.repack_layer reads."""

    def __init__(self, data, quant_state):
        self.data = data
        self.quant_state = quant_state


class FakeLinear4bit:
    def __init__(self, weight):
        self.weight = weight


def quantize_nf4(w, code2=None, chunk_blocks=1 << 20):
    """Quantise an fp16 matrix `w` [rows, cols] (rows*cols a multiple of 16384) on its own device."""
    if w.dtype != torch.float16 or w.dim() != 2:
        raise ValueError("expected a 2-D fp16 weight")
    n = w.numel()
    if n % (QBLOCK * QBLOCKS2):
        raise ValueError(f"{n} weights do not fill whole absmax blocks")
    dev = w.device
    code2 = default_code2(dev) if code2 is None else code2.to(dev, torch.float32)
    levels = torch.tensor(NF4_CODE, dtype=torch.float32, device=dev)
    nb = n // QBLOCK
    flat = w.reshape(nb, QBLOCK)
    absmax = torch.empty(nb, dtype=torch.float32, device=dev)
    packed = torch.empty(nb, QBLOCK // 2, dtype=torch.uint8, device=dev)
    for b0 in range(0, nb, chunk_blocks):
        blk = flat[b0:b0 + chunk_blocks].float()
        am = blk.abs().amax(dim=1)
        absmax[b0:b0 + chunk_blocks] = am
        norm = blk / am.clamp_min(1e-30)[:, None]
        codes = _nearest_index(norm, levels).to(torch.uint8)
        packed[b0:b0 + chunk_blocks] = (codes[:, 0::2] << 4) | codes[:, 1::2]
    offset = absmax.mean()
    centred = (absmax - offset).reshape(nb // QBLOCKS2, QBLOCKS2)
    scale2 = centred.abs().amax(dim=1).clamp_min(1e-30)
    qabs = _nearest_index(centred / scale2[:, None], code2).to(torch.uint8).reshape(nb)
    state2 = SimpleNamespace(absmax=scale2.contiguous(), code=code2, blocksize=QBLOCKS2)
    state = SimpleNamespace(quant_type="nf4", blocksize=QBLOCK, nested=True, state2=state2,
                            absmax=qabs, offset=offset.reshape(()), dtype=torch.float16,
                            shape=torch.Size(w.shape))
    return Quantized4bit(packed.reshape(-1, 1), state)


def random_nf4_weight(rows, cols, seed, device="cpu", std=0.02, code2=None):
    """A seeded fp16 weight ~ N(0, std) drawn on the CPU generator (identical on every box),
    quantised on `device`. Returns a FakeLinear4bit ready for k_nf4.repack_layer."""
    gen = torch.Generator().manual_seed(seed)
    chunks, left = [], rows * cols
    while left:                      # bounded host memory for the largest shapes
        take = min(left, 1 << 24)
        chunks.append((torch.randn(take, generator=gen) * std).half().to(device))
        left -= take
    w = torch.cat(chunks).reshape(rows, cols)
    return FakeLinear4bit(quantize_nf4(w, code2))
