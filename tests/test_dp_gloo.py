"""Row-sharded data parallelism on CPU ranks (gloo, world_size 2): each rank works on its own block
of token rows, the LoRA gradients are summed through the flat bucket, and the result equals the
full-batch gradients. The per-rank arithmetic is the oracle's (no GPU here); what is under test is
the sharding rule and the bucket all-reduce, i.e. the N > 1 host logic of bench.py and blocks.py."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from decentrik_prime_b200 import blocks, dp
from oracle import nf4_oracle
from tests.problem import make_problem, oracle_weight


def test_shard_rows_covers_everything_once():
    for n, world in ((2048, 1), (2048, 2), (16384, 8), (1213, 4), (100, 8), (129, 2)):
        spans = [dp.shard_rows(n, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        for (a, b), (c, d) in zip(spans, spans[1:]):
            assert b == c and a <= b
        assert all(a % 128 == 0 for a, _ in spans)
    with pytest.raises(ValueError):
        dp.shard_rows(10, 2, 2)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pr = make_problem(256, 128, 512, seed=9, lora=True, dropout=0.05)
        w16 = oracle_weight(pr)
        lo, hi = dp.shard_rows(pr.M, world, rank)
        ref = nf4_oracle.lora_linear_o1(w16, pr.x[lo:hi], pr.dy[lo:hi], None, pr.A16, pr.B16, pr.scale,
                                        pr.mask[lo:hi], pr.keep_scale, dtype=torch.float32)
        bucket = blocks.GradBucket(blocks.lora_grad_numel(pr.N, pr.K), "cpu")
        dA, dB = bucket.take(16, pr.K), bucket.take(pr.N, 16)
        dA.copy_(ref["dA"]); dB.copy_(ref["dB"])
        bucket.all_reduce()
        if rank == 0:
            full = nf4_oracle.lora_linear_o1(w16, pr.x, pr.dy, None, pr.A16, pr.B16, pr.scale, pr.mask, pr.keep_scale)
            out["dA"] = nf4_oracle.errors(dA, full["dA"])
            out["dB"] = nf4_oracle.errors(dB, full["dB"])
            # forward rows are independent: a rank's block equals the same rows of the full batch
            out["y"] = nf4_oracle.errors(ref["y"], full["y"][lo:hi])
    finally:
        dist.destroy_process_group()


def test_two_rank_gradient_bucket_matches_full_batch():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
        res = dict(out)
    for name in ("dA", "dB", "y"):
        err, rel = res[name]
        assert rel < 1e-5, (name, err, rel)
