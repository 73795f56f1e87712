#!/usr/bin/env python
"""Benchmark of the NF4 + LoRA linear hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (`config.workload` = "qwen2.5-1.5b-mlp-block-M2048"): the gate, up (1536 -> 8960) and
down (8960 -> 1536) projections of one Qwen2.5-1.5B decoder layer, NF4 weights (block 64,
double-quantised absmax) drawn N(0, 0.02) from a seed, LoRA r=16 / alpha=32 with dropout p=0.05 on
every projection, M = 2048 packed token rows per GPU, forward + backward-dX + dA/dB, frozen base
(no dW). The SiLU-gated product between up and down is PyTorch. One step = one forward and one
backward of the block. Metric: algorithmic TFLOP/s, FLOPs = sum over projections of
4*M*N*K + 6*M*16*(N+K) (dequantisation, bias, dropout and epilogues count as zero).

With N > 1 (torchrun, one rank per GPU) token rows are data-parallel: each rank runs the same block
on its own 2048 rows (weak scaling), NF4 weights replicated, and the fp32 LoRA-gradient bucket is
all-reduced with NCCL every step inside the timed region.

`--impl reference` times the reference's own CPU arithmetic for the same block (oracle O2: dequant
into fp16, fp32-accumulated GEMMs rounded to fp16 where the reference rounds) on the host cores.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN, INTER, M_ROWS, P_DROP = 1536, 8960, 2048, 0.05
WORKLOAD = "qwen2.5-1.5b-mlp-block-M2048"
METRIC = "nf4_lora_linear_fwd_bwd_tflops_M2048"
N_WEIGHT_SETS, N_INPUT_SETS = 8, 4
NCU_DRAM_BYTES_PER_LAUNCH = 53.0e6
ROOFLINE_EVERY = 9      # timed steps whose tensor-core launches are bracketed by events: every ninth (9 and the 8 weight sets are coprime)


def block_flops(M):
    r = 16
    per = lambda n, k: 4 * M * n * k + 6 * M * r * (n + k)
    return 2 * per(INTER, HIDDEN) + per(HIDDEN, INTER)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"tflops_burst": p["bf16_tflops"], "tflops_sustained": p["bf16_tflops_sustained"],
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"tflops_burst": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference's arithmetic on the host cores (test/measurement infrastructure only)
# ------------------------------------------------------------------------------------------------
def cpu_block_step(parts, x, dy, masks, keep_scale):
    """One forward + backward of the block on the CPU with the reference's roundings; dequantises
    each weight from its NF4 bytes first, as the reference does before every GEMM."""
    import torch
    import torch.nn.functional as F
    from oracle import nf4_oracle

    def deq(part):
        layer, code2, _, _ = part
        return nf4_oracle.dequant_weight(layer, "w", code2)

    outs = []
    wg, wu = deq(parts[0]), deq(parts[1])
    og = nf4_oracle.lora_linear_o2(wg, x, None, None, parts[0][2], parts[0][3], 2.0, masks[0], keep_scale)
    ou = nf4_oracle.lora_linear_o2(wu, x, None, None, parts[1][2], parts[1][3], 2.0, masks[1], keep_scale)
    g, u = og["y"], ou["y"]
    h = (F.silu(g.float()) * u.float()).half()
    wd = deq(parts[2])
    od = nf4_oracle.lora_linear_o2(wd, h, dy, None, parts[2][2], parts[2][3], 2.0, masks[2], keep_scale)
    dh = od["dx"].half()
    gf = g.float()
    sig = torch.sigmoid(gf)
    du = (dh.float() * gf * sig).half()
    dg = (dh.float() * u.float() * sig * (1 + gf * (1 - sig))).half()
    bg = nf4_oracle.lora_linear_o2(wg, x, dg, None, parts[0][2], parts[0][3], 2.0, masks[0], keep_scale)
    bu = nf4_oracle.lora_linear_o2(wu, x, du, None, parts[1][2], parts[1][3], 2.0, masks[1], keep_scale)
    dx = (bg["dx"] + bu["dx"]).half()
    outs.append(dx)
    return od["y"], dx


def cpu_problem(M, seed=0):
    import math
    import torch
    from decentrik_prime_b200 import k_nf4, quantize
    gen = torch.Generator().manual_seed(seed)
    parts = []
    for i, (n, k) in enumerate(((INTER, HIDDEN), (INTER, HIDDEN), (HIDDEN, INTER))):
        lin = quantize.random_nf4_weight(n, k, seed=seed * 10 + i + 1)
        layer, code2 = k_nf4.repack_layer({"w": lin}, torch.device("cpu"), names=("w",))
        A = (((torch.rand(16, k, generator=gen) * 2 - 1) / math.sqrt(k))).half()
        B = (torch.randn(n, 16, generator=gen) * 0.01).half()
        parts.append((layer, code2, A, B))
    x = torch.randn(M, HIDDEN, generator=gen).half()
    dy = torch.randn(M, HIDDEN, generator=gen).half()
    masks = [(torch.rand(M, k, generator=gen) >= P_DROP).to(torch.uint8) for k in (HIDDEN, HIDDEN, INTER)]
    keep_scale = 1.0 / float(torch.tensor(1.0 - P_DROP, dtype=torch.float32))
    return parts, x, dy, masks, keep_scale


def time_cpu(M, steps, warmup):
    import torch
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    prob = cpu_problem(M)
    for _ in range(warmup):
        cpu_block_step(*prob)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_block_step(*prob)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return block_flops(M) / dt / 1e12, dt, cores


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    M = 256
    tf, dt, cores = time_cpu(M, max(args.steps, 1), max(min(args.warmup, 1), 0))
    sample = f"same block, M={M} of {M_ROWS} rows per step, dequantisation of all three weights included"
    line = {"impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows_per_gpu": M_ROWS, "hidden": HIDDEN, "intermediate": INTER,
                       "lora_rank": 16, "dropout": P_DROP},
            "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            text, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            text, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for row in text.strip().splitlines():
            f = [c.strip() for c in row.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            # under load = the upper half of the samples (the sampler also sees idle time around the region)
            busy = sorted(sm)[len(sm) // 2:]
            out.update(sm_mhz=statistics.median(busy), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    from decentrik_prime_b200 import _lib, blocks, dp, linear

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the NF4 kernels have no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    h = _lib.lib()
    M = M_ROWS
    keep_scale = 1.0 / float(torch.tensor(1.0 - P_DROP, dtype=torch.float32))

    # replicated weights: several distinct layers so that consecutive steps stream different NF4 bytes
    bucket = blocks.GradBucket(N_WEIGHT_SETS * blocks.MlpBlock.grad_numel(HIDDEN, INTER), dev)
    layers = [blocks.MlpBlock(HIDDEN, INTER, seed=100 + i, device=dev, lora=True, bucket=bucket) for i in range(N_WEIGHT_SETS)]
    per_layer = blocks.MlpBlock.grad_numel(HIDDEN, INTER)
    gen = torch.Generator().manual_seed(1234 + rank)       # every rank has its own rows
    host_x = [torch.randn(M, HIDDEN, generator=gen).half().pin_memory() for _ in range(N_INPUT_SETS)]
    host_dy = [torch.randn(M, HIDDEN, generator=gen).half().pin_memory() for _ in range(N_INPUT_SETS)]
    dev_x = [t.to(dev) for t in host_x]
    dev_dy = [t.to(dev) for t in host_dy]
    gdev = torch.Generator(device=dev).manual_seed(77 + rank)
    mask_sets = [[(torch.rand(M, k, device=dev, generator=gdev) >= P_DROP).to(torch.uint8) for k in (HIDDEN, HIDDEN, INTER)]
                 for _ in range(N_INPUT_SETS)]
    flops = block_flops(M)

    ev_pairs = []      # (start, stop, flops) of tensor-core kernels inside the timed region

    graphs = {}        # (weight set, id of x) -> (CUDAGraph, outputs): whole steps captured once, replayed afterwards

    def step(i, x, dy, masks, timed=False):
        blk = layers[i % N_WEIGHT_SETS]
        hooked = timed and i % ROOFLINE_EVERY == 0
        if timed:
            # every ROOFLINE_EVERY-th timed step has its tensor-core launches bracketed by events: the
            # event records cost ~3 % of a step, so the other steps run without them
            _hook_block(blk, ev_pairs if hooked else None, M)
        slot = i % N_WEIGHT_SETS
        if sync is not None:
            sync.wait_slot(slot)          # this layer's gradients of 8 steps ago have been exchanged
        g = None if hooked else graphs.get((slot, x.data_ptr()))
        if g is not None:
            g[0].replay()                 # the same launches, issued by the GPU front end instead of Python
            y, dx = g[1]
        else:
            y = blk.forward(x, masks, keep_scale)
            dx = blk.backward(dy)
        if sync is not None:
            # the exchange runs on a side stream under the next step's compute
            sync.launch(slot, bucket.flat[slot * per_layer:(slot + 1) * per_layer])
        return y, dx

    def capture_steps(xs, dys):
        """One CUDA graph per (weight set, input set) pair the loops below use: the step's launches are
        fixed, so the ~0.5 ms of Python per step need not race the GPU. Falls back to eager on failure."""
        if args.no_graphs:
            return
        side = torch.cuda.Stream(dev)
        try:
            with torch.cuda.stream(side):
                for i in range(N_WEIGHT_SETS):
                    x, dy, masks = xs[i % len(xs)], dys[i % len(dys)], mask_sets[i % N_INPUT_SETS]
                    blk = layers[i % N_WEIGHT_SETS]
                    blk._ev_sink = None
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        y = blk.forward(x, masks, keep_scale)
                        dx = blk.backward(dy)
                    graphs[(i, x.data_ptr())] = (g, (y, dx))
            torch.cuda.synchronize()
        except Exception as exc:      # capture is an optimisation, never a requirement
            graphs.clear()
            torch.cuda.synchronize()
            print(f"[bench] CUDA graph capture failed ({type(exc).__name__}: {exc}); running eagerly", file=sys.stderr)

    sync = dp.GradSync(dev, N_WEIGHT_SETS) if world > 1 else None

    def barrier():
        if sync is not None:
            sync.wait_all()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------- device-resident throughput ("value")
    for i in range(args.warmup):
        step(i, dev_x[i % N_INPUT_SETS], dev_dy[i % N_INPUT_SETS], mask_sets[i % N_INPUT_SETS])
    barrier()
    linear.check_status(dev)
    capture_steps(dev_x, dev_dy)
    _fill_event_pool(6 * args.steps + 6)
    torch.cuda.synchronize()
    sampler = ClockSampler(local) if rank == 0 else None
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    if args.profile_leg == "step":
        torch.cuda.profiler.start()      # `ncu --profile-from-start off` captures the timed region only
    t0.record()
    for i in range(args.steps):
        step(i, dev_x[i % N_INPUT_SETS], dev_dy[i % N_INPUT_SETS], mask_sets[i % N_INPUT_SETS], timed=True)
    if sync is not None:
        sync.wait_all()                   # the last exchanges are inside the timed region
    t1.record()
    barrier()
    if args.profile_leg == "step":
        torch.cuda.profiler.stop()
    ms = t0.elapsed_time(t1)
    clocks = sampler.stop() if sampler else None
    linear.check_status(dev)
    for blk in layers:
        blk._ev_sink = None
    kern_ms = sum(a.elapsed_time(b) for a, b, _ in ev_pairs)
    kern_flops = sum(f for _, _, f in ev_pairs)
    n_kern = len(ev_pairs)

    # ---------------- end to end through the public API with host buffers ("e2e")
    # x and dy start in pinned host memory every step; y, dx and the LoRA gradients are read back.
    copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    main = torch.cuda.current_stream(dev)
    slots = 2
    in_x = [torch.empty(M, HIDDEN, dtype=torch.float16, device=dev) for _ in range(slots)]
    in_dy = [torch.empty(M, HIDDEN, dtype=torch.float16, device=dev) for _ in range(slots)]
    out_y = [torch.empty(M, HIDDEN, dtype=torch.float16).pin_memory() for _ in range(slots)]
    out_dx = [torch.empty(M, HIDDEN, dtype=torch.float16).pin_memory() for _ in range(slots)]
    out_g = [torch.empty(per_layer, dtype=torch.float32).pin_memory() for _ in range(slots)]
    ev_in = [torch.cuda.Event() for _ in range(slots)]
    ev_done = [torch.cuda.Event() for _ in range(slots)]
    ev_free = [torch.cuda.Event() for _ in range(slots)]
    ev_out = [torch.cuda.Event() for _ in range(slots)]
    h2d = 2 * M * HIDDEN * 2
    d2h = 2 * M * HIDDEN * 2 + per_layer * 4

    def e2e_loop(n):
        for s in range(slots):
            ev_free[s].record(main)
            ev_out[s].record(copy_out)
        for i in range(n):
            s = i % slots
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(ev_free[s])              # compute of step i-2 has consumed the slot
                in_x[s].copy_(host_x[i % N_INPUT_SETS], non_blocking=True)
                in_dy[s].copy_(host_dy[i % N_INPUT_SETS], non_blocking=True)
                ev_in[s].record(copy_in)
            main.wait_event(ev_in[s])
            main.wait_event(ev_out[s])                      # results of step i-2 have left the device
            y, dx = step(i, in_x[s], in_dy[s], mask_sets[i % N_INPUT_SETS])
            ev_free[s].record(main)
            ev_done[s].record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(ev_done[s])
                if sync is not None and sync.done[i % N_WEIGHT_SETS] is not None:
                    copy_out.wait_event(sync.done[i % N_WEIGHT_SETS])    # the gradients leave the device summed
                out_y[s].copy_(y, non_blocking=True)
                out_dx[s].copy_(dx, non_blocking=True)
                lo = (i % N_WEIGHT_SETS) * per_layer
                out_g[s].copy_(bucket.flat[lo:lo + per_layer], non_blocking=True)
                ev_out[s].record(copy_out)
                y.record_stream(copy_out); dx.record_stream(copy_out)
        main.wait_stream(copy_out)

    capture_steps(in_x, in_dy)
    e2e_loop(max(args.warmup, 1))
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_loop(args.steps)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)

    # ---------------- max over ranks
    if world > 1:
        t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
    if rank == 0:
        pk = peaks()
        value = world * flops * args.steps / (ms * 1e-3) / 1e12
        e2e_val = world * flops * args.steps / (e2e_ms * 1e-3) / 1e12
        achieved = kern_flops / (kern_ms * 1e-3) / 1e12 if kern_ms > 0 else None
        # the tensor-core kernels run back to back inside a long step: the sustained peak applies
        peak = pk["tflops_sustained"]
        line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": {"workload": WORKLOAD, "rows_per_gpu": M, "hidden": HIDDEN, "intermediate": INTER,
                           "lora_rank": 16, "dropout": P_DROP, "parallelism": f"dp{world}",
                           "tokens_per_s": world * M * args.steps / (ms * 1e-3),
                           "l2": f"inputs larger than L2: {N_WEIGHT_SETS} weight sets and {N_INPUT_SETS} input sets rotate; "
                                 "one step touches > 300 MB of activations",
                           "launch": ("cuda graphs: one captured step per weight set, replayed; every ninth timed step "
                                      "of the value loop issued eagerly with event hooks") if graphs
                           else "eager: every launch issued from python"},
                "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                             "frac": (achieved / peak) if achieved else None,
                             # DRAM bytes per tensor-core launch (read + written), mean over the five launches of a
                             # step, from the ncu capture summarised in profiles/nf4_gemm_kernels_mlp_block_M2048.md
                             "traffic": NCU_DRAM_BYTES_PER_LAUNCH, "traffic_unit": "bytes per launch (ncu, one step)",
                             "peak_source": pk["source"] + " sustained bf16",
                             "frac_of_burst": (achieved / pk["tflops_burst"]) if achieved else None,
                             "kernel": "nf4_gemm_kernel (forward and backward-dX launches)",
                             "launches_timed": n_kern, "avg_launch_us": kern_ms * 1e3 / max(n_kern, 1)},
                "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": e2e_ms / args.steps},
                "gpu_launches": 15 * args.steps, "clocks": clocks}
        if world == 1 and not args.no_stream:
            if args.profile_leg == "stream":
                torch.cuda.profiler.start()
            line["weight_stream"] = {"unit": "GB/s of NF4 bytes", "peak_gbs": pk["hbm_gbs"], "peak_source": pk["source"],
                                     "cases": weight_stream_numbers(dev, pk["hbm_gbs"])}
            if args.profile_leg == "stream":
                torch.cuda.profiler.stop()
        if world == 1 and not args.no_cpu:
            tf, dt, cores = time_cpu(128, 2, 1)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": "same block with M=128 of 2048 rows, 2 steps after 1 warm-up, "
                                              "dequantisation of all three weights included"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_stack(args):
    """Secondary workloads (not the default line): the full projection stack of benchmark
    configuration 2 (`--workload stack1.5b`: 28 layers, 4 packed sequences of 64..512 tokens, one GPU) and
    configuration 3 (`--workload stack7b`: Qwen2.5-7B shapes, M = 16384 packed rows split by rows over the
    ranks = strong scaling, LoRA gradients all-reduced once per step). Only projections and the
    minimal glue of decentrik_prime_b200/stack.py run; FLOPs are the projections' algorithmic FLOPs."""
    import torch
    import torch.distributed as dist
    from decentrik_prime_b200 import dp, linear, stack

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.workload == "stack1.5b":
        hidden, inter, kv, layers, distinct = 1536, 8960, 256, 28, 28
        lens, M_total = stack.pack_lengths(4, 64, 512, seed=2)
        note = f"4 sequences of lengths {lens}"
    else:
        hidden, inter, kv, layers, distinct = 3584, 18944, 512, 28, 2
        lens, M_total = stack.pack_lengths(32, 256, 512, seed=3)
        M_total = 16384          # the configuration's fixed packed row count
        note = "32 sequences packed to 16384 rows; 2 distinct weight sets reused over 28 layers"
    lo, hi = dp.shard_rows(M_total, world, rank)
    M = hi - lo
    st = stack.ProjectionStack(hidden, inter, kv, layers, dev, seed=7, distinct_layers=distinct)
    gen = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(M, hidden, generator=gen).half().to(dev)
    dy = (torch.randn(M, hidden, generator=gen) * 0.1).half().to(dev)
    gdev = torch.Generator(device=dev).manual_seed(5 + rank)
    n_mask_sets = min(distinct, 4)
    masks = [{n: (torch.rand(M, hidden, device=dev, generator=gdev) >= P_DROP).to(torch.uint8) for n in ("q_proj", "v_proj")}
             for _ in range(n_mask_sets)]
    masks = [masks[i % n_mask_sets] for i in range(layers)]
    keep_scale = 1.0 / float(torch.tensor(1.0 - P_DROP, dtype=torch.float32))

    graph = [None]

    def step():
        if graph[0] is not None:
            graph[0].replay()
        else:
            st.step(x, dy, masks, keep_scale)
        if world > 1:
            dist.all_reduce(st.bucket.flat)

    def capture():
        """The ~1000 launches of a stack step as one CUDA graph: issued from Python they cost more host time
        than GPU time at the small configuration. Falls back to eager on failure."""
        if args.no_graphs:
            return
        side = torch.cuda.Stream(dev)
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(g, stream=side):
                    st.step(x, dy, masks, keep_scale)
            torch.cuda.synchronize()
            graph[0] = g
        except Exception as exc:
            graph[0] = None
            torch.cuda.synchronize()
            print(f"[bench] CUDA graph capture failed ({type(exc).__name__}: {exc}); running eagerly", file=sys.stderr)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    steps, warmup = min(args.steps, 20), min(max(args.warmup, 3), 5)
    for _ in range(warmup):
        step()
    barrier()
    linear.check_status(dev)
    capture()
    step()
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        step()
    t1.record()
    barrier()
    ms = t0.elapsed_time(t1)
    linear.check_status(dev)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
        fl = torch.tensor([float(st.flops(M))], dtype=torch.float64, device=dev)
        dist.all_reduce(fl)
        flops = fl.item()
    else:
        flops = float(st.flops(M))
    if rank == 0:
        line = {"metric": "nf4_lora_projection_stack_tokens_per_s", "value": M_total * steps / (ms * 1e-3), "unit": "tokens/s",
                "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True,
                "scaling": "strong" if args.workload == "stack7b" else "weak", "vs_baseline": None, "dtype": "f16",
                "data": "synthetic",
                "config": {"workload": args.workload, "rows": M_total, "rows_per_gpu": M, "layers": layers, "hidden": hidden,
                           "intermediate": inter, "kv": kv, "lora": "r=16 on q_proj, v_proj", "note": note,
                           "tflops": flops * steps / (ms * 1e-3) / 1e12, "parallelism": f"dp{world}",
                           "launch": "cuda graph of the whole step, replayed" if graph[0] is not None else "eager"}}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def weight_stream_numbers(dev, peak_gbs):
    """Secondary metric of the path: NF4 bytes streamed per second by the forward at decode-sized
    batches (benchmark configuration 4: Qwen2.5-32B shapes, LoRA r=16 fused, M in {1, 8, 64}). Distinct weight
    copies larger than L2 (126 MB) rotate inside one CUDA graph so that every launch reads its NF4
    bytes from HBM; the figure is algorithmic bytes (0.516 B per weight) over the median replay time."""
    import statistics
    import torch
    from decentrik_prime_b200 import blocks, linear
    out = []
    for name, n, k, copies in (("q/o 5120x5120", 5120, 5120, 20), ("gate/up 27648x5120", 27648, 5120, 4),
                               ("down 5120x27648", 5120, 27648, 4)):
        ps = [blocks.make_projection(n, k, seed=900 + i, device=dev, lora=True) for i in range(copies)]
        nbytes = ps[0].w.nbytes
        for M in (1, 8, 64):
            x = torch.randn(M, k, device=dev).half()
            ys = [torch.empty(M, n, device=dev, dtype=torch.float16) for _ in ps]
            side = torch.cuda.Stream(dev)
            with torch.cuda.stream(side):
                for p_, y_ in zip(ps, ys):
                    linear.forward(p_.w, x, lora=p_.lora, out=y_)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for p_, y_ in zip(ps, ys):
                        linear.forward(p_.w, x, lora=p_.lora, out=y_)
                times = []
                for _ in range(20):
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(side); graph.replay(); b.record(side)
                    torch.cuda.synchronize()
                    times.append(a.elapsed_time(b) * 1e-3 / copies)
            t = statistics.median(times)
            out.append({"shape": name, "M": M, "us": t * 1e6, "gbs": nbytes / t / 1e9,
                        "frac_of_measured_hbm": nbytes / t / 1e9 / peak_gbs})
            del graph
        del ps
        torch.cuda.empty_cache()
    return out


_event_pool = []


def _fill_event_pool(n):
    """Timing events are created (and their handles materialised by a first record) before the timed
    region, so that arming the kernel hook costs one ctypes call per launch."""
    import torch
    while len(_event_pool) < n:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); b.record()
        _event_pool.append((a, b))


def _hook_block(blk, ev_pairs, M):
    """Arrange for the six tensor-core launches of this block step to be bracketed by CUDA events.
    The library records a one-shot event pair around its next GEMM kernel, so each projection call
    is wrapped to arm the hook right before it."""
    import torch
    from decentrik_prime_b200 import _lib, linear
    h = _lib.lib()
    if getattr(blk, "_hooked", False) or ev_pairs is None:
        blk._ev_sink = ev_pairs
        return
    blk._hooked, blk._ev_sink = True, ev_pairs

    def arm(proj, n_out):
        if blk._ev_sink is None:
            return
        a, b = _event_pool.pop()
        h.nf4ll_kernel_events(a.cuda_event, b.cuda_event)
        blk._ev_sink.append((a, b, 2 * M * proj.w.N * proj.w.K + 2 * M * 16 * n_out))

    if getattr(blk, "fused_glue", False):
        # gate and up run as ONE tensor-core launch (gated product in its epilogue): arm the hook once for both
        blk_fwd = blk.forward

        def blk_fwd_hook(*a, _f=blk_fwd, **k):
            if blk._ev_sink is not None:
                ea, eb = _event_pool.pop()
                h.nf4ll_kernel_events(ea.cuda_event, eb.cuda_event)
                blk._ev_sink.append((ea, eb, sum(2 * M * pj.w.N * pj.w.K + 2 * M * 16 * pj.w.N for pj in (blk.gate, blk.up))))
            return _f(*a, **k)

        blk.forward = blk_fwd_hook

    for proj in blk.projections:
        fwd, bwd = proj.forward, proj.backward

        def fwd_hook(*a, _p=proj, _f=fwd, **k):
            arm(_p, _p.w.N)
            return _f(*a, **k)

        def bwd_hook(*a, _p=proj, _f=bwd, **k):
            arm(_p, _p.w.K)
            return _f(*a, **k)

        proj.forward, proj.backward = fwd_hook, bwd_hook


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-stream", action="store_true", help="skip the small-batch weight-stream numbers")
    ap.add_argument("--no-graphs", action="store_true", help="issue every step from Python instead of replaying CUDA graphs")
    ap.add_argument("--profile-leg", default="step", choices=("step", "stream"),
                    help="which leg cudaProfilerStart/Stop brackets (for `ncu --profile-from-start off`): the timed "
                         "steps, or the small-batch weight-stream measurements")
    ap.add_argument("--workload", default="mlp", choices=("mlp", "stack1.5b", "stack7b"),
                    help="mlp = the default bench line (benchmark configuration 1); stack* = configs 2 / 3")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload != "mlp":
        run_stack(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
