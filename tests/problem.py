"""Seeded synthetic problems for the NF4 + LoRA linear, built the way benchmark configuration 0 describes:
fp16 weight ~ N(0, 0.02) quantised to NF4 (block 64, double-quantised absmax), fp16 activations
~ N(0, 1), LoRA r=16 / alpha=32 with kaiming-uniform A and B ~ N(0, 0.01), dropout p=0.05 with the
keep-mask drawn from the seed, keep_scale = 1 / float32(1 - p)."""

import math

import numpy as np
import torch

from decentrik_prime_b200 import k_nf4, quantize


class Problem:
    pass


def keep_scale_for(p):
    return 1.0 / float(torch.tensor(1.0 - p, dtype=torch.float32))   # reference solution/fast_qwen.py:370


def make_problem(N, K, M, seed=0, lora=True, dropout=0.05, bias=False, device="cpu", w_std=0.02, ld_pad=0):
    gen = torch.Generator().manual_seed(seed)
    pr = Problem()
    pr.N, pr.K, pr.M = N, K, M
    lin = quantize.random_nf4_weight(N, K, seed=seed * 7919 + 13, device=device, std=w_std)
    pr.layer, pr.code2 = k_nf4.repack_layer({"w": lin}, torch.device(device), names=("w",))
    pr.x = torch.randn(M, K, generator=gen).half()
    pr.dy = torch.randn(M, N, generator=gen).half()
    pr.bias = (torch.randn(N, generator=gen) * 0.1).half() if bias else None
    pr.scale, pr.A, pr.B, pr.mask, pr.keep_scale = 1.0, None, None, None, 1.0
    if lora:
        bound = 1.0 / math.sqrt(K)                 # kaiming_uniform(a=sqrt(5)) on [16, K]
        pr.A = ((torch.rand(16, K, generator=gen) * 2 - 1) * bound)
        pr.B = torch.randn(N, 16, generator=gen) * 0.01
        pr.scale = 32.0 / 16.0
        if dropout:
            pr.mask = (torch.rand(M, K, generator=gen) >= dropout).to(torch.uint8)
            pr.keep_scale = keep_scale_for(dropout)
    pr.A16 = None if pr.A is None else pr.A.half()
    pr.B16 = None if pr.B is None else pr.B.half()
    return pr


def oracle_weight(pr):
    from oracle import nf4_oracle
    return nf4_oracle.dequant_weight(pr.layer, "w", pr.code2)


def to_device(pr, dev="cuda"):
    """Device copies of the operands (the packed layer is re-homed on the device too)."""
    from decentrik_prime_b200.linear import Nf4Weight
    d = Problem()
    flat = pr.layer.flat.to(dev)
    d.layer = k_nf4.PackedLayer(flat, pr.layer.offsets, pr.layer.n_qblocks, pr.layer.segments)
    d.code2 = pr.code2.to(dev)
    d.w = Nf4Weight.from_layer(d.layer, "w", d.code2)
    for name in ("x", "dy", "bias", "A16", "B16", "mask"):
        v = getattr(pr, name)
        setattr(d, name, None if v is None else v.to(dev))
    d.lora = None if pr.A16 is None else (d.A16, d.B16, pr.scale)
    d.keep_scale = pr.keep_scale
    return d
