#!/usr/bin/env python
"""Benchmark of the NF4 + LoRA linear hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (`config.workload` = "qwen2.5-1.5b-mlp-block-M2048"): the gate, up (1536 -> 8960) and
down (8960 -> 1536) projections of one Qwen2.5-1.5B decoder layer, NF4 weights (block 64,
double-quantised absmax) drawn N(0, 0.02) from a seed, LoRA r=16 / alpha=32 with dropout p=0.05 on
every projection, M = 2048 packed token rows per GPU, forward + backward-dX + dA/dB, frozen base
(no dW). The SiLU-gated product between up and down runs in the library's kernels. One step = one
forward and one backward of the block. Metric: algorithmic TFLOP/s, FLOPs = sum over projections of
4*M*N*K + 6*M*16*(N+K) (dequantisation, bias, dropout and epilogues count as zero).

With N > 1 (torchrun, one rank per GPU) token rows are data-parallel: each rank runs the same block
on its own 2048 rows (weak scaling), NF4 weights replicated, and the fp32 LoRA-gradient bucket is
all-reduced with NCCL every step inside the timed region.

Besides the headline numbers the line carries, at N = 1, benchmark configuration 0 (one q_proj linear),
configuration 2 (the 1.5B projection stack) and configuration 4 (small-batch weight streaming, with a
roofline object of its own), and at every N configuration 3 (Qwen2.5-7B shapes, 16384 packed rows split by
rows over the ranks: strong scaling, LoRA gradients all-reduced per layer under the backward).

`--impl reference` times the reference's own CPU arithmetic for the same block at the same M = 2048
(oracle O2: dequant into fp16, fp32-accumulated GEMMs rounded to fp16 where the reference rounds) on
all host cores; it runs as many of the requested steps as fit a time budget of about 100 s.
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
# mean DRAM bytes (read + written) per tensor-core launch of a step, from an ncu capture of one step (not a
# measurement of this run); reported with that label
NCU_DRAM_BYTES_PER_LAUNCH = 53.0e6
CPU_BUDGET_S = 100.0
# timed steps whose tensor-core launches are bracketed by events: every 49th (49 and the 8 weight sets are coprime). Such a
# step is issued from Python instead of replayed from its graph, which costs host time (0.5 ms here, 2 ms on a slow
# host core): rare enough that the timed region stays GPU-bound wherever it runs
ROOFLINE_EVERY = 49
ROOFLINE_FIRST = 7     # the first instrumented step: not the first of the timed region


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


def time_cpu(M, steps, warmup, budget_s=CPU_BUDGET_S):
    """(TFLOP/s, seconds per step, cores, timed steps): at most `steps` timed steps, fewer when the time
    budget runs out first (every step is the whole block at M rows, dequantisation included)."""
    import torch
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    prob = cpu_problem(M)
    t_start = time.perf_counter()
    for _ in range(warmup):
        cpu_block_step(*prob)
    done, t0 = 0, time.perf_counter()
    while done < max(steps, 1):
        cpu_block_step(*prob)
        done += 1
        if time.perf_counter() - t_start > budget_s:
            break
    dt = (time.perf_counter() - t0) / done
    return block_flops(M) / dt / 1e12, dt, cores, done


def block_config(world):
    """The same dictionary in both arms (the driver compares them)."""
    return {"workload": WORKLOAD, "rows_per_gpu": M_ROWS, "hidden": HIDDEN, "intermediate": INTER,
            "lora_rank": 16, "dropout": P_DROP, "parallelism": f"dp{world}",
            "l2": f"inputs larger than L2: {N_WEIGHT_SETS} weight sets and {N_INPUT_SETS} input sets rotate; "
                  "one step touches > 300 MB of activations"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tf, dt, cores, done = time_cpu(M_ROWS, args.steps, 1 if args.warmup > 0 else 0)
    sample = (f"the same block at the same M={M_ROWS} rows, dequantisation of all three weights included in every step; "
              f"{done} of the {args.steps} requested steps timed (time budget {CPU_BUDGET_S:.0f} s)")
    line = {"impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "steps_timed": done, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": block_config(args.gpus),
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
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20"],
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
        _limit_nccl_ctas()
        dist.init_process_group("nccl", device_id=dev)
    h = _lib.lib()
    M = M_ROWS
    keep_scale = 1.0 / float(torch.tensor(1.0 - P_DROP, dtype=torch.float32))
    sampler = ClockSampler(local) if rank == 0 else None      # runs from before the warm-up to the end of the e2e leg

    # replicated weights: several distinct layers so that consecutive steps stream different NF4 bytes
    bucket = blocks.GradBucket(N_WEIGHT_SETS * blocks.MlpBlock.grad_numel(HIDDEN, INTER), dev)
    layers = [blocks.MlpBlock(HIDDEN, INTER, seed=100 + i, device=dev, lora=True, bucket=bucket) for i in range(N_WEIGHT_SETS)]
    per_layer = blocks.MlpBlock.grad_numel(HIDDEN, INTER)
    if args.no_coop:
        h.nf4ll_tune_override(0, 0, 0, 1)
    if not args.no_grad_stream:
        # the dA/dB kernels of a backward run on a side stream beside the dX GEMMs (forked and joined inside the step)
        grad_stream = torch.cuda.Stream(dev)
        for blk in layers:
            blk.use_grad_stream(grad_stream)
    gen = torch.Generator().manual_seed(1234 + rank)       # every rank has its own rows
    # x and dy of a step lie back to back in one pinned buffer: one host-to-device copy per step
    host_in = [torch.randn(2, M, HIDDEN, generator=gen).half().pin_memory() for _ in range(N_INPUT_SETS)]
    dev_in = [t.to(dev) for t in host_in]
    gdev = torch.Generator(device=dev).manual_seed(77 + rank)
    mask_sets = [[(torch.rand(M, k, device=dev, generator=gdev) >= P_DROP).to(torch.uint8) for k in (HIDDEN, HIDDEN, INTER)]
                 for _ in range(N_INPUT_SETS)]
    flops = block_flops(M)

    ev_pairs = []      # (start, stop, flops) of tensor-core kernels inside the timed region
    graphs = {}        # (weight set, id of the input buffer) -> CUDAGraph: whole steps captured once, replayed afterwards
    hooked_graphs = {}     # the same key -> (CUDAGraph with event-record nodes around the tensor-core launches, its event pairs)
    hooked_graphs_made = [False]
    kept_graphs = []
    launches_per_step = [None]

    def run_block(blk, inp, masks, out):
        """One forward + backward of a block through the public API; y and dx land in `out` ([2, M, HIDDEN])."""
        y = blk.forward(inp[0], masks, keep_scale, out=out[0])
        dx = blk.backward(inp[1], out=out[1])
        return y, dx

    def step(i, inp, masks, out, timed=False):
        blk = layers[i % N_WEIGHT_SETS]
        hooked = (timed and args.steps > ROOFLINE_FIRST and i % ROOFLINE_EVERY == ROOFLINE_FIRST) or timed == "hooked"
        if timed:
            # every ROOFLINE_EVERY-th timed step has its tensor-core launches bracketed by events: the
            # event records cost ~3 % of a step, so the other steps run without them
            _hook_block(blk, ev_pairs if hooked else None, M)
        slot = i % N_WEIGHT_SETS
        if sync is not None:
            sync.wait_slot(slot)          # this layer's gradients of 8 steps ago have been exchanged
        g = None if hooked else graphs.get((slot, inp.data_ptr()))
        hg = hooked_graphs.pop((slot, inp.data_ptr()), None) if hooked and timed is True else None
        if hg is not None:
            # an instrumented copy of the step's graph: the event records are nodes of the graph, so the step costs the
            # host what any replay costs; each copy is replayed once, its events then hold this step's launch times
            hg[0].replay()
            ev_pairs.extend(hg[1])
            kept_graphs.append(hg[0])
        elif g is not None:
            g.replay()                    # the same launches, issued by the GPU front end instead of Python
        elif hooked and timed is True and hooked_graphs_made[0]:
            graphs[(slot, inp.data_ptr())].replay()      # all instrumented copies are used up: an ordinary step
        else:
            run_block(blk, inp, masks, out)
        if sync is not None:
            # the exchange runs on a side stream under the next step's compute
            sync.launch(slot, bucket.flat[slot * per_layer:(slot + 1) * per_layer])

    def capture_steps(inputs, outs, instrumented=False):
        """One CUDA graph per (weight set, input buffer) pair the loops below use: the step's launches are
        fixed, so the ~0.5 ms of Python per step need not race the GPU. Falls back to eager on failure."""
        if args.no_graphs:
            return
        side = torch.cuda.Stream(dev)
        try:
            with torch.cuda.stream(side):
                for i in range(N_WEIGHT_SETS):
                    inp, out, masks = inputs[i % len(inputs)], outs[i % len(outs)], mask_sets[i % N_INPUT_SETS]
                    blk = layers[i % N_WEIGHT_SETS]
                    blk._ev_sink = None
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        run_block(blk, inp, masks, out)
                    graphs[(i, inp.data_ptr())] = g
                    if instrumented:
                        mine = []
                        _hook_block(blk, mine, M)
                        hg = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(hg, stream=side):
                            run_block(blk, inp, masks, out)
                        blk._ev_sink = None
                        hooked_graphs[(i, inp.data_ptr())] = (hg, mine)
                hooked_graphs_made[0] = bool(hooked_graphs)
                # a graph's first launch uploads it to the device: done here, outside every timed region
                for g in graphs.values():
                    g.replay()
                for hg, _ in hooked_graphs.values():
                    hg.replay()
            torch.cuda.synchronize()
        except Exception as exc:      # capture is an optimisation, never a requirement
            graphs.clear()
            hooked_graphs.clear()
            hooked_graphs_made[0] = False
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
    dev_out = [torch.empty(2, M, HIDDEN, dtype=torch.float16, device=dev) for _ in range(N_INPUT_SETS)]
    for i in range(max(args.warmup, 3)):
        if i == 1:
            n0 = h.nf4ll_launch_count()
        step(i, dev_in[i % N_INPUT_SETS], mask_sets[i % N_INPUT_SETS], dev_out[i % N_INPUT_SETS])
        if i == 1:
            # kernels of the library in one step, counted by the library itself (+1: the gradient fill is PyTorch's)
            launches_per_step[0] = int(h.nf4ll_launch_count() - n0) + 1
    barrier()
    linear.check_status(dev)
    _fill_event_pool(6 * N_WEIGHT_SETS + 6 * (args.steps // ROOFLINE_EVERY + 4) + 12)
    capture_steps(dev_in, dev_out, instrumented=True)
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    if args.profile_leg == "step":
        torch.cuda.profiler.start()      # `ncu --profile-from-start off` captures the timed region only
    t0.record()
    for i in range(args.steps):
        step(i, dev_in[i % N_INPUT_SETS], mask_sets[i % N_INPUT_SETS], dev_out[i % N_INPUT_SETS], timed=True)
    if sync is not None:
        sync.wait_all()                   # the last exchanges are inside the timed region
    t1.record()
    barrier()
    if args.profile_leg == "step":
        torch.cuda.profiler.stop()
    ms = t0.elapsed_time(t1)
    linear.check_status(dev)
    events_where = "inside the timed region"
    if not ev_pairs:
        # too few timed steps to hide an eagerly issued one behind queued work: the tensor-core launches are timed in
        # two extra steps right after the region instead (same inputs, same weights)
        for i in range(2):
            step(i, dev_in[i % N_INPUT_SETS], mask_sets[i % N_INPUT_SETS], dev_out[i % N_INPUT_SETS], timed="hooked")
        barrier()
        events_where = "two extra steps right after the timed region (fewer than 8 timed steps)"
    for blk in layers:
        blk._ev_sink = None
    kern_ms = sum(a.elapsed_time(b) for a, b, _ in ev_pairs)
    kern_flops = sum(f for _, _, f in ev_pairs)
    n_kern = len(ev_pairs)

    # ---------------- end to end through the public API with host buffers ("e2e")
    # Per step: ONE copy in (x | dy, pinned host -> device) and ONE copy out (y | dx | LoRA gradients, device ->
    # pinned host), on two copy streams, double-buffered around the compute stream.
    copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    main = torch.cuda.current_stream(dev)
    slots = 2
    act_elems = 2 * M * HIDDEN
    in_buf = [torch.empty(2, M, HIDDEN, dtype=torch.float16, device=dev) for _ in range(slots)]
    # outputs and gradients share one device buffer (fp16 words; the fp32 gradients take two each)
    out_words = act_elems + 2 * per_layer
    out_dev = [torch.empty(out_words, dtype=torch.float16, device=dev) for _ in range(slots)]
    out_act = [o[:act_elems].view(2, M, HIDDEN) for o in out_dev]
    out_grad = [o[act_elems:].view(torch.float32) for o in out_dev]
    out_host = [torch.empty(out_words, dtype=torch.float16).pin_memory() for _ in range(slots)]
    ev_in = [torch.cuda.Event() for _ in range(slots)]
    ev_done = [torch.cuda.Event() for _ in range(slots)]
    ev_free = [torch.cuda.Event() for _ in range(slots)]
    ev_out = [torch.cuda.Event() for _ in range(slots)]
    h2d = act_elems * 2
    d2h = out_words * 2

    def e2e_loop(n, compute=True):
        for s in range(slots):
            ev_free[s].record(main)
            ev_out[s].record(copy_out)
        for i in range(n):
            s = i % slots
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(ev_free[s])              # compute of step i-2 has consumed the slot
                in_buf[s].copy_(host_in[i % N_INPUT_SETS], non_blocking=True)
                ev_in[s].record(copy_in)
            main.wait_event(ev_in[s])
            main.wait_event(ev_out[s])                      # results of step i-2 have left the device
            if compute:
                step(i, in_buf[s], mask_sets[i % N_INPUT_SETS], out_act[s])
                if sync is not None and sync.done[i % N_WEIGHT_SETS] is not None:
                    main.wait_event(sync.done[i % N_WEIGHT_SETS])       # the gradients leave the device summed
                lo = (i % N_WEIGHT_SETS) * per_layer
                out_grad[s].copy_(bucket.flat[lo:lo + per_layer], non_blocking=True)
            ev_free[s].record(main)
            ev_done[s].record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(ev_done[s])
                out_host[s].copy_(out_dev[s], non_blocking=True)
                ev_out[s].record(copy_out)
        main.wait_stream(copy_out)

    capture_steps(in_buf, out_act)
    e2e_loop(max(args.warmup, 3))
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_loop(args.steps)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    linear.check_status(dev)
    # the host-side ceiling of that loop: the same copies on the same streams with no compute between them
    e2e_loop(3, compute=False)
    barrier()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    e2e_loop(args.steps, compute=False)
    c1.record()
    barrier()
    copy_ms = c0.elapsed_time(c1)
    clocks = sampler.stop() if sampler else None

    # ---------------- configuration 3 on every N (strong scaling), the other configurations at N = 1
    extra = {}
    if not args.no_extras:
        del graphs, layers, dev_in, in_buf, out_dev
        torch.cuda.empty_cache()
        extra["config3_stack7b"] = stack_numbers("stack7b", dev, world, rank, args)
        if world == 1:
            extra["config0_q_proj"] = config0_numbers(dev)
            extra["config2_stack1.5b"] = stack_numbers("stack1.5b", dev, world, rank, args)
            extra["config2_decoder_stack"] = decoder_stack_numbers(dev, args)

    # ---------------- max over ranks
    if world > 1:
        t = torch.tensor([ms, e2e_ms, copy_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, copy_ms = t.tolist()
    if rank == 0:
        pk = peaks()
        value = world * flops * args.steps / (ms * 1e-3) / 1e12
        e2e_val = world * flops * args.steps / (e2e_ms * 1e-3) / 1e12
        achieved = kern_flops / (kern_ms * 1e-3) / 1e12 if kern_ms > 0 else None
        # a timed region of under a second runs at boost clocks: the burst figure is the peak to compare with;
        # a longer one settles under the power cap, where the sustained figure applies
        burst = ms < 1000.0
        peak = pk["tflops_burst"] if burst else pk["tflops_sustained"]
        line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": block_config(world),
                "tokens_per_s": world * M * args.steps / (ms * 1e-3),
                "launch": ("cuda graphs: one captured step per weight set, replayed; every 49th timed step of the value "
                           "loop (eight at most) replays a copy of its graph with event-record nodes around the "
                           "tensor-core launches") if not args.no_graphs
                else "eager: every launch issued from python",
                "grad_stream": not args.no_grad_stream,
                "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                             "frac": (achieved / peak) if achieved else None,
                             "peak_source": pk["source"] + (" burst bf16 (timed region under 1 s)" if burst
                                                            else " sustained bf16 (timed region over 1 s)"),
                             "frac_of_burst": (achieved / pk["tflops_burst"]) if achieved else None,
                             "frac_of_sustained": (achieved / pk["tflops_sustained"]) if achieved else None,
                             "traffic": NCU_DRAM_BYTES_PER_LAUNCH,
                             "traffic_source": "ncu capture of one step (mean DRAM bytes read + written per tensor-core launch), "
                                               "not a measurement of this run",
                             # NF4 bytes of the six weight passes of a step + every activation matrix a launch reads or
                             # writes (x, g, u, h | h, y | dy, dh | dg, dx | du, dx read + written), over the five launches
                             "algorithmic_bytes_per_launch": (6 * INTER * HIDDEN * 0.516113
                                                              + 2 * M * (6 * HIDDEN + 7 * INTER)) / 5,
                             "kernel": "nf4_gemm_kernel / nf4_gemm_pair_kernel (forward and backward-dX launches)",
                             "events": events_where,
                             "launches_timed": n_kern, "avg_launch_us": kern_ms * 1e3 / max(n_kern, 1)},
                "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": e2e_ms / args.steps, "copies_per_step": 2,
                        "copy_only_ms_per_step": copy_ms / args.steps,
                        "copy_only_gbs_per_gpu": (h2d + d2h) * args.steps / (copy_ms * 1e-3) / 1e9,
                        "note": "copy_only = the same two copies per step on the same streams with no compute: the host-side "
                                "ceiling of this loop at this N"},
                "gpu_launches": (launches_per_step[0] or 0) * args.steps, "gpu_launches_per_step": launches_per_step[0],
                "nccl_max_ctas": os.environ.get("NCCL_MAX_CTAS") if world > 1 else None,
                "clocks": clocks}
        line.update(extra)
        if world == 1 and not args.no_stream:
            if args.profile_leg == "stream":
                torch.cuda.profiler.start()
            cases = weight_stream_numbers(dev, pk["hbm_gbs"], args.stream_case)
            if args.profile_leg == "stream":
                torch.cuda.profiler.stop()
            others = [c for c in cases if c["M"] not in (1, 8, 64)]
            cases = [c for c in cases if c["M"] in (1, 8, 64)] or cases
            line["weight_stream"] = {"unit": "GB/s of NF4 bytes", "peak_gbs": pk["hbm_gbs"], "peak_source": pk["source"],
                                     "cases": cases, "other_batch_sizes": others}
            best = max(cases, key=lambda c: c["gbs"])
            worst = min(cases, key=lambda c: c["gbs"])
            line["roofline_weight_stream"] = {
                "bound": "hbm", "achieved": best["gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": best["gbs"] / pk["hbm_gbs"],
                "case": f"{best['shape']} M={best['M']}", "worst": worst["gbs"], "worst_case": f"{worst['shape']} M={worst['M']}",
                "worst_frac": worst["gbs"] / pk["hbm_gbs"], "peak_source": pk["source"] + " copy bandwidth",
                "algorithmic_bytes": "0.516113 B per weight: nibbles + absmax codes + scale2 + offset2",
                "traffic": None, "traffic_source": "see the ncu summary of the streaming kernel (DRAM bytes read = algorithmic bytes)"}
        if world == 1 and not args.no_cpu:
            tf, dt, cores, done = time_cpu(M_ROWS, 3, 1, budget_s=30.0)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": f"the same block at the same M={M_ROWS} rows, {done} steps after 1 warm-up, "
                                              "dequantisation of all three weights included"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _limit_nccl_ctas():
    """The gradient all-reduce runs on a side stream under the next step's compute. Three of a step's five
    tensor-core launches are cooperative split-K grids of 144 CTAs (one per SM, 148 SMs): they start only when
    their whole grid can be resident, i.e. when at most 4 SMs are busy elsewhere. NCCL's default of up to 32 CTAs
    for a collective would make each of them wait for the all-reduce to finish; four CTAs move the 2 MB bucket
    slice of a step in far less than a step. Set before the communicator is created; a value from the environment wins."""
    os.environ.setdefault("NCCL_MAX_CTAS", "4")
    os.environ.setdefault("NCCL_MIN_CTAS", "1")


def config0_numbers(dev):
    """Benchmark configuration 0 on the GPU: one q_proj linear 1536 x 1536 at M = 2048 with LoRA and dropout,
    forward + backward-dX + dA/dB; 48 output tiles on 148 SMs, so the plan splits the contraction. Several
    weight copies rotate inside one CUDA graph; algorithmic FLOPs 4MNK + 6Mr(N+K)."""
    import torch
    from decentrik_prime_b200 import blocks, linear
    N = K = 1536
    M = M_ROWS
    copies = 24
    ps = [blocks.make_projection(N, K, seed=500 + i, device=dev, lora=True) for i in range(copies)]
    gen = torch.Generator().manual_seed(9)
    x = torch.randn(M, K, generator=gen).half().to(dev)
    dy = torch.randn(M, N, generator=gen).half().to(dev)
    mask = (torch.rand(M, K, generator=gen) >= P_DROP).to(torch.uint8).to(dev)
    ks = 1.0 / float(torch.tensor(1.0 - P_DROP, dtype=torch.float32))

    def run():
        for p_ in ps:
            p_.forward(x, mask, ks)
            p_.backward(dy, accumulate_grads=False)

    side = torch.cuda.Stream(dev)
    with torch.cuda.stream(side):
        run()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            run()
        times = []
        for _ in range(10):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(side); graph.replay(); b.record(side)
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e-3 / copies)
    linear.check_status(dev)
    t = statistics.median(times)
    fl = ps[0].flops(M)
    return {"workload": "q_proj 1536x1536, M=2048, LoRA r=16 + dropout, fwd + bwd-dX + dA/dB", "us": t * 1e6,
            "tflops": fl / t / 1e12, "gflop": fl / 1e9, "weight_copies": copies}


def stack_numbers(workload, dev, world, rank, args):
    """Benchmark configurations 2 (`stack1.5b`: 28 layers of Qwen2.5-1.5B shapes, 4 packed sequences of 64..512
    tokens, one GPU) and 3 (`stack7b`: Qwen2.5-7B shapes, 16384 packed rows split by rows over the ranks =
    strong scaling; each layer's LoRA gradients all-reduced on a side stream under the remaining backward).
    All seven projections of every layer run; what lies between them is decentrik_prime_b200/stack.py's glue.
    Returns tokens/s and the projections' algorithmic TFLOP/s (max over ranks)."""
    import torch
    import torch.distributed as dist
    from decentrik_prime_b200 import dp, linear, stack

    if workload == "stack1.5b":
        hidden, inter, kv, layers, distinct = 1536, 8960, 256, 28, 8
        lens, M_total = stack.pack_lengths(4, 64, 512, seed=2)
        note = f"4 sequences of lengths {lens}; 8 distinct weight sets (193 MB of NF4 bytes) reused over 28 layers"
    else:
        hidden, inter, kv, layers, distinct = 3584, 18944, 512, 28, 2
        M_total = 16384
        note = "32 sequences packed to 16384 rows; 2 distinct weight sets (240 MB of NF4 bytes) reused over 28 layers"
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
    sync = dp.GradSync(dev, distinct) if world > 1 else None
    graph = [None]

    def step():
        if graph[0] is not None:
            graph[0].replay()
        else:
            st.step(x, dy, masks, keep_scale, sync=sync)
        if sync is not None:
            sync.wait_all()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    steps, warmup = min(args.steps, 10), 3
    for _ in range(warmup):
        step()
    barrier()
    linear.check_status(dev)
    if world == 1 and not args.no_graphs:
        # the ~1000 launches of a stack step as one CUDA graph (one GPU: no collective inside)
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
    flops = float(st.flops(M))
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
        fl = torch.tensor([flops], dtype=torch.float64, device=dev)
        dist.all_reduce(fl)
        flops = fl.item()
    del st, graph
    torch.cuda.empty_cache()
    return {"workload": workload, "rows": M_total, "rows_per_gpu": M, "layers": layers, "hidden": hidden, "intermediate": inter,
            "kv": kv, "lora": "r=16 on q_proj, v_proj", "scaling": "strong" if workload == "stack7b" else "single GPU",
            "tokens_per_s": M_total * steps / (ms * 1e-3), "tflops": flops * steps / (ms * 1e-3) / 1e12,
            "ms_per_step": ms / steps, "steps": steps, "warmup": warmup, "note": note,
            "launch": "cuda graph of the whole step, replayed" if world == 1 and not args.no_graphs else
                      "eager, per-layer gradient all-reduce on a side stream"}


def run_stack(args):
    """`--workload stack1.5b | stack7b`: the projection-stack configurations as a line of their own."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        _limit_nccl_ctas()
        dist.init_process_group("nccl", device_id=dev)
    res = stack_numbers(args.workload, dev, world, rank, args)
    if rank == 0:
        line = {"metric": "nf4_lora_projection_stack_tokens_per_s", "value": res["tokens_per_s"], "unit": "tokens/s",
                "n_gpus": world, "steps": res["steps"], "warmup": res["warmup"], "ms_per_step": res["ms_per_step"],
                "higher_is_better": True, "scaling": "strong" if args.workload == "stack7b" else "weak", "vs_baseline": None,
                "dtype": "f16", "data": "synthetic", "config": res}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def decoder_stack_numbers(dev, args):
    """Benchmark configuration 2 as a real model step: 28 Qwen2.5-1.5B decoder layers (RMSNorm + residual kernels
    of this library, Q|K|V / O / gate|up / down through the fused NF4 + LoRA linear, rotary embedding and causal
    grouped-query attention through PyTorch's kernels), the same 4 packed sequences, forward and the hand-written
    backward called as one autograd node. 28 distinct weight sets; issued eagerly."""
    import torch
    from decentrik_prime_b200 import linear, stack
    hidden, inter, kv, layers, heads = 1536, 8960, 256, 28, 12
    lens, M = stack.pack_lengths(4, 64, 512, seed=2)
    ns = stack.NormedStack(hidden, inter, kv, layers, dev, seed=7, n_heads=heads)
    for t in ns.lora_masters():
        t.requires_grad_(True)
    gen = torch.Generator().manual_seed(100)
    x = torch.randn(M, hidden, generator=gen).to(dev)
    dres = (torch.randn(M, hidden, generator=gen) * 0.1).to(dev)
    gdev = torch.Generator(device=dev).manual_seed(5)
    mask_sets = [{n: (torch.rand(M, hidden, device=dev, generator=gdev) >= P_DROP).to(torch.uint8) for n in ("q_proj", "v_proj")}
                 for _ in range(4)]
    masks = [mask_sets[i % 4] for i in range(layers)]
    keep_scale = 1.0 / float(torch.tensor(1.0 - P_DROP, dtype=torch.float32))

    def step():
        out = ns.apply(x, masks, keep_scale, lens)
        out.backward(dres)
        for t in ns.lora_masters():
            t.grad = None

    steps, warmup = min(args.steps, 10), 3
    side = torch.cuda.Stream(dev)
    graph = None
    with torch.cuda.stream(side):
        for _ in range(warmup):
            step()
        torch.cuda.synchronize()
        linear.check_status(dev)
        if not args.no_graphs:
            # forward and backward (the autograd engine included) of the whole stack as one CUDA graph
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    step()
                torch.cuda.synchronize()
                graph.replay()
                torch.cuda.synchronize()
            except Exception as exc:
                graph = None
                torch.cuda.synchronize()
                print(f"[bench] CUDA graph capture of the decoder stack failed ({type(exc).__name__}: {exc}); running eagerly", file=sys.stderr)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(side)
        for _ in range(steps):
            if graph is not None:
                graph.replay()
            else:
                step()
        t1.record(side)
        torch.cuda.synchronize()
    ms = t0.elapsed_time(t1)
    linear.check_status(dev)
    res = {"workload": "decoder stack 1.5b: norms + projections + rotary/causal attention, one autograd node",
           "rows": M, "layers": layers, "heads": heads, "kv_heads": 2, "lengths": lens,
           "tokens_per_s": M * steps / (ms * 1e-3), "projection_tflops": float(ns.flops(M)) * steps / (ms * 1e-3) / 1e12,
           "ms_per_step": ms / steps, "steps": steps, "warmup": warmup,
           "launch": ("cuda graph of the whole step, replayed" if graph is not None else "eager") +
                     "; attention through torch.nn.functional.scaled_dot_product_attention per sequence"}
    del ns, graph
    torch.cuda.empty_cache()
    return res


def weight_stream_numbers(dev, peak_gbs, only=None, rows=(1, 8, 64, 16, 32)):
    """Secondary metric of the path: NF4 bytes streamed per second by the forward at decode-sized
    batches (benchmark configuration 4: Qwen2.5-32B shapes, LoRA r=16 fused, M in {1, 8, 64}). Distinct weight
    copies larger than L2 (126 MB) rotate inside one CUDA graph so that every launch reads its NF4
    bytes from HBM; the figure is algorithmic bytes (0.516 B per weight) over the median replay time.
    `only` = "<shape prefix>:<M>" (e.g. "gate:64") restricts the leg to one case, for a profiler capture.
    `rows`: the benchmark's M in {1, 8, 64} first, then the batch sizes in between (reported separately)."""
    import statistics
    import torch
    from decentrik_prime_b200 import blocks, linear
    out = []
    for name, n, k, copies in (("q/o 5120x5120", 5120, 5120, 20), ("gate/up 27648x5120", 27648, 5120, 4),
                               ("down 5120x27648", 5120, 27648, 4)):
        if only and not name.startswith(only.split(":")[0]):
            continue
        ps = [blocks.make_projection(n, k, seed=900 + i, device=dev, lora=True) for i in range(copies)]
        nbytes = ps[0].w.nbytes
        for M in rows:
            if only and int(only.split(":")[1]) != M:
                continue
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
    ap.add_argument("--no-extras", action="store_true", help="skip benchmark configurations 0, 2 and 3")
    ap.add_argument("--no-graphs", action="store_true", help="issue every step from Python instead of replaying CUDA graphs")
    ap.add_argument("--no-grad-stream", action="store_true", help="issue the LoRA gradient kernels on the step's own stream instead of a side stream")
    ap.add_argument("--no-coop", action="store_true",
                    help="keep split contractions off the cooperative reduction (tuning flag bit 0): for a profiler that "
                         "replays kernels one at a time; the kernel choice is otherwise unchanged")
    ap.add_argument("--profile-leg", default="step", choices=("step", "stream"),
                    help="which leg cudaProfilerStart/Stop brackets (for `ncu --profile-from-start off`): the timed "
                         "steps, or the small-batch weight-stream measurements")
    ap.add_argument("--stream-case", default=None,
                    help='run one case of the weight-stream leg only, "<shape prefix>:<M>", e.g. "gate:64" (profiler captures)')
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
