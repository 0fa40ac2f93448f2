#!/usr/bin/env python
"""MoE-layer throughput benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl reference]

One "step" is one pass of the whole MoE block (router -> routed NVFP4 experts -> shared expert ->
combine) over one batch of synthetic tokens.  At N = 1 the workload is the decode configuration
(T = 64 tokens, hidden 2048, 256 resident NVFP4 experts, top-8, one bf16 shared expert).  The step
cycles through several independently seeded layers and batches so that successive steps touch
different expert bytes (a layer's banks are 455 MB, larger than the 126 MB L2).

Rank 0 prints ONE JSON line.  `value` is tokens/s with inputs resident in HBM, timed with CUDA
events; `e2e` is the same metric through the public call with HOST buffers (pinned host x copied in,
the block run, the result copied out, every step, inside the timed region); `roofline` is the
dominant kernel's algorithmic bytes over its own CUDA-event time (per-kernel profile pass);
`cpu_baseline` is the CPU restatement of the reference's host path timed on this box's cores.

--impl reference times the reference's CPU algorithm (the C restatement under oracle/: the Rust
reference cannot be compiled in this image) on the same workload, bounded to a sample per step.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN, INTER, EXPERTS, TOP_K, SHARED = 2048, 512, 256, 8, 512
EXPERT_BYTES = 1775616                      # six bank rows of one expert
GATE_UP_BYTES = 1048576 + 131072 + 2048     # packed + scales + globals of gate_up
DOWN_BYTES = 524288 + 65536 + 4096
METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=0, help="tokens per step (default: 64 at N=1)")
    ap.add_argument("--layers", type=int, default=4, help="independent layers cycled through")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--sweep", action="store_true", help="also report T = 1, 8, 512, 2048")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ep-chunks", type=int, default=2,
                    help="N > 1: expert ranges per owner that are exchanged and computed one after the other, so that "
                         "exchanges run under compute; 1 = the plain schedule")
    ap.add_argument("--ep-exchange", default="p2p", choices=["p2p", "nccl"],
                    help="N > 1: dispatch / return by this library's kernels over peer memory, or by NCCL all-to-all")
    ap.add_argument("--ep-comm-sms", type=int, default=16, help="N > 1: SMs left to the exchange kernels when overlapping")
    ap.add_argument("--zipf", type=float, default=None,
                    help="add a per-expert Zipf(alpha) popularity bias to the router logits (skewed expert counts)")
    ap.add_argument("--stack", action="store_true",
                    help="N = 1: one step = a pass through --layers MoE blocks with a residual add between them "
                         "(the 40-layer stack of the benchmark configs: --layers 40 --stack)")
    ap.add_argument("--path", default="auto", choices=["auto", "gemv", "grouped", "scalar"],
                    help="routed-expert kernels: auto = decode kernels up to 256 tokens, tcgen05 grouped GEMM above")
    return ap.parse_args()


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "which": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "which": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except Exception:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------ CPU reference arm / baseline

def host_layer_for_cpu(seed: int):
    pkg = importlib.import_module("ferrum-torrens_b200")
    from oracle import oracle as o
    lay = pkg.synth.make_layer(seed)
    banks = o.HostBanks(*lay.banks, slots=EXPERTS, gu_rows=2 * INTER, gu_cols=HIDDEN, dn_rows=HIDDEN, dn_cols=INTER)
    ol = o.Layer(HIDDEN, INTER, EXPERTS, TOP_K, SHARED, lay.gate_w, lay.sh_gate_up, lay.sh_down, lay.sh_gate, banks)
    return pkg, o, lay, ol


def time_cpu(tokens_sample: int, steps: int, warmup: int, seed: int = 2024):
    """tokens/s of the CPU restatement of the reference's host path, all host threads."""
    pkg, o, lay, ol = host_layer_for_cpu(seed)
    # every core this process may run on: a launcher's OMP_NUM_THREADS=1 (torchrun sets it) must not shrink
    # the CPU arm to one thread
    try:
        threads = len(os.sched_getaffinity(0))
    except AttributeError:
        threads = os.cpu_count() or 1
    threads = max(threads, o.max_threads())
    times = []
    for i in range(warmup + steps):
        x = pkg.synth.bf16_bits_to_f32(pkg.synth.make_x(seed + i, tokens_sample, HIDDEN))
        t0 = time.perf_counter()
        o.moe_block(ol, x, threads=threads)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    return tokens_sample * len(times) / sum(times), threads, sum(times) / len(times)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tokens = args.tokens or 64
    sample = min(tokens, 16)
    steps, warmup = max(1, min(args.steps, 8)), max(1, min(args.warmup, 2))
    tps, threads, sec = time_cpu(sample, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"decode T={tokens}, hidden {HIDDEN}, {EXPERTS} NVFP4 experts top-{TOP_K}, shared {SHARED}",
                   "sample": f"{sample} tokens per step"},
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{sample} tokens of the T={tokens} batch per step, whole block, "
                                   f"{steps} steps; C restatement of the reference's host path (the Rust "
                                   f"reference cannot be compiled in this image)"},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ------------------------------------------------------------------ B200 arm

def run_b200(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    import __graft_entry__ as ge
    if rank == 0:
        ge.build()
    if world > 1:
        dist.barrier()
    pkg = importlib.import_module("ferrum-torrens_b200")

    if world > 1:
        return run_ep(args, pkg, dev, world, rank, local)

    T = args.tokens or 64
    path = {"auto": 0, "gemv": 1, "grouped": 2, "scalar": 3}[args.path]
    nlayers = max(1, args.layers)
    moe = pkg.B200MoE(local, pkg.ExpertShapes(HIDDEN, INTER), EXPERTS * nlayers, experts=EXPERTS, layers=nlayers,
                      top_k=TOP_K, shared_inter=SHARED, max_tokens=max(T, 64))
    dense, xs = [], []
    # a stack feeds every block's output back into the residual stream: row globals 2^-6 / 2^-10 keep it O(1)
    gbits = (0x2400, 0x1400) if args.stack else (0x3C00, 0x3C00)
    for l in range(nlayers):
        pkg.synth.fill_banks_on_device(moe, l, seed=1000 + 17 * rank + l, slot0=l * EXPERTS, global_bits=gbits)
        dense.append(pkg.synth.device_dense_weights(2000 + 17 * rank + l, dev, zipf_alpha=args.zipf))
        xs.append(pkg.synth.device_x(3000 + 17 * rank + l, T, HIDDEN, dev, biased=args.zipf is not None))
    if args.stack and world == 1:
        return run_stack(args, pkg, moe, dense, xs[0], dev, T, nlayers, path)
    out = torch.empty((T, HIDDEN), dtype=torch.bfloat16, device=dev)
    ids = torch.empty((T, TOP_K), dtype=torch.int32, device=dev)
    wts = torch.empty((T, TOP_K), dtype=torch.float32, device=dev)

    def step(i, x=None, o=None):
        l = i % nlayers
        g, su, sd, sg = dense[l]
        moe.moe_block(l, xs[l] if x is None else x, g, su, sd, sg, out if o is None else o, ids_out=ids, weights_out=wts,
                      path=path)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for i in range(warmup):
            fn(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(warmup + i)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    W, K = max(3, args.warmup), max(1, args.steps)
    # one checked step before anything is timed: a kernel that gave up a bounded wait fails here
    step(0)
    moe.sync_status()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = moe.kernel_launches()
    total_ms = timed(step, K, W)
    launches = (moe.kernel_launches() - l0) * K // (K + W)
    value = world * T * K / (total_ms * 1e-3)

    # end to end: every step's activations come from pinned host memory and its result goes back to pinned host
    # memory.  The copies run on a copy stream with two staging buffers each way, so the H2D of step i + 1 and the
    # D2H of step i overlap the compute of a neighbouring step, as a serving loop would run them.
    x_host = [x.cpu().pin_memory() for x in xs]
    x_stage = [torch.empty_like(xs[0]) for _ in range(2)]
    out_dev = [torch.empty_like(out) for _ in range(2)]
    out_host = [torch.empty((T, HIDDEN), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    copy_s = torch.cuda.Stream()
    ev_h2d = [torch.cuda.Event() for _ in range(2)]
    ev_comp = [torch.cuda.Event() for _ in range(2)]
    ev_d2h = [torch.cuda.Event() for _ in range(2)]
    primed = [False]

    def step_e2e(i):
        cur = torch.cuda.current_stream()
        b = i & 1
        if not primed[0]:                      # the first step's input
            with torch.cuda.stream(copy_s):
                x_stage[b].copy_(x_host[i % nlayers], non_blocking=True)
                ev_h2d[b].record(copy_s)
            for e in ev_comp + ev_d2h:
                e.record(cur)
            primed[0] = True
        cur.wait_event(ev_h2d[b])              # this step's input has arrived
        cur.wait_event(ev_d2h[b])              # the result buffer's previous content has left
        step(i, x=x_stage[b], o=out_dev[b])
        ev_comp[b].record(cur)
        with torch.cuda.stream(copy_s):
            copy_s.wait_event(ev_comp[b ^ 1])  # the other input buffer was read by the previous step
            x_stage[b ^ 1].copy_(x_host[(i + 1) % nlayers], non_blocking=True)
            ev_h2d[b ^ 1].record(copy_s)
            copy_s.wait_event(ev_comp[b])
            out_host[b].copy_(out_dev[b], non_blocking=True)
            ev_d2h[b].record(copy_s)

    def timed_e2e():
        for i in range(W):
            step_e2e(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(K):
            step_e2e(W + i)
        torch.cuda.current_stream().wait_event(ev_d2h[(W + K - 1) & 1])    # the last result has reached the host buffer
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    e2e_ms = timed_e2e()

    # the same without any overlap: copy in, block, copy out on one stream
    def step_serial(i):
        x_stage[0].copy_(x_host[i % nlayers], non_blocking=True)
        step(i, x=x_stage[0], o=out_dev[0])
        out_host[0].copy_(out_dev[0], non_blocking=True)

    serial_ms = timed(step_serial, K, W)
    e2e = {"value": world * T * K / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": T * HIDDEN * 2,
           "d2h_bytes_per_step": T * HIDDEN * 2,
           "how": "pinned host buffers; H2D of step i + 1 and D2H of step i on a copy stream (two staging buffers each "
                  "way) under the compute of the neighbouring step",
           "serial_value": world * T * K / (serial_ms * 1e-3)}

    # per-kernel profile pass (CUDA events around every launch) for the roofline of the dominant kernel.
    # The routed half runs alone here (serving call with the router's ids), so that the shared expert,
    # which the whole block overlaps on a second stream, does not share the SMs with the timed kernels.
    routed = []
    for l in range(nlayers):
        step(l)
        torch.cuda.synchronize()
        routed.append((ids.clone(), wts.clone()))
    uniq = [int(torch.unique(i).numel()) for i, _ in routed]
    reqs = [pkg.MoEDeviceRequest(l, HIDDEN, INTER, TOP_K, xs[l], routed[l][0], routed[l][1]) for l in range(nlayers)]
    for i in range(W):
        moe.grouped_moe_staged(reqs[i % nlayers], out, path=path)
    moe.profile(True)
    for i in range(K):
        moe.grouped_moe_staged(reqs[i % nlayers], out, path=path)
    prof = moe.profile_read()
    moe.profile(False)
    # the router and shared-expert kernels, each alone on the stream
    moe.profile(True)
    for i in range(K):
        g, su, sd, sg = dense[i % nlayers]
        moe.router(xs[i % nlayers], g)
        moe.shared_expert(xs[i % nlayers], su, sd, sg)
    prof.update(moe.profile_read())
    moe.profile(False)
    U = sum(uniq) / len(uniq)
    pk = peaks()
    gate_kind = "expert_gate_up" if "expert_gate_up" in prof else "grouped_gate_up"
    g_ms, g_n = prof[gate_kind]
    kernels = {k: {"us_per_launch": ms / n * 1e3, "launches": n} for k, (ms, n) in prof.items()}
    if gate_kind == "expert_gate_up":
        # decode kernels: bound by the HBM stream of the routed experts' weights
        gu_bytes = U * GATE_UP_BYTES + T * HIDDEN * 2
        # DRAM traffic per algorithmic byte of this kernel, from one ncu capture of it
        # (dram__bytes_read + dram__bytes_write over one launch at T = 64)
        NCU_TRAFFIC_RATIO = 1.042
        achieved = gu_bytes / (g_ms / g_n * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": gate_kind, "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / pk["hbm_gbs"], "peak_source": pk["which"], "frac_of_nominal_8000": achieved / 8000.0,
                    "traffic": NCU_TRAFFIC_RATIO * gu_bytes, "distinct_experts": U, "bytes_per_launch": gu_bytes,
                    "us_per_launch": g_ms / g_n * 1e3, "kernels": kernels}
    else:
        # tcgen05 grouped GEMM: useful flops of the routes (padding of ragged groups not counted)
        flops = T * TOP_K * 2.0 * HIDDEN * (2 * INTER)
        achieved = flops / (g_ms / g_n * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": gate_kind, "achieved": achieved, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": achieved / pk["bf16_tflops"], "peak_source": pk["which"] + " (burst; sustained %.0f)" % pk["bf16_tflops_sustained"],
                    "traffic": None, "distinct_experts": U, "flops_per_launch": flops, "us_per_launch": g_ms / g_n * 1e3,
                    "kernels": kernels}
        if "grouped_down" in prof:
            d_ms, d_n = prof["grouped_down"]
            dn = T * TOP_K * 2.0 * INTER * HIDDEN / (d_ms / d_n * 1e-3) / 1e12
            roofline["down"] = {"achieved": dn, "frac": dn / pk["bf16_tflops"]}
    if "expert_down" in prof:
        d_ms, d_n = prof["expert_down"]
        dn = (U * DOWN_BYTES) / (d_ms / d_n * 1e-3) / 1e9
        roofline["down"] = {"achieved": dn, "frac": dn / pk["hbm_gbs"]}
        both = (U * EXPERT_BYTES) / ((g_ms / g_n + d_ms / d_n) * 1e-3) / 1e9
        roofline["expert_weights_gbs"] = both

    # the sampler ran through the timed steps, the end-to-end steps and the per-kernel passes (all GPU-busy)
    clocks = sampler.stop() if rank == 0 else None

    # the same steps replayed from one captured CUDA graph (one block per layer in the graph): what an engine
    # that captures its decode step gets; reported beside the eager numbers, not instead of them
    graph_info = None
    if world == 1:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            cg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cg, stream=side):
                for l in range(nlayers):
                    step(l)
            reps = max(1, K // nlayers)
            g_ms = timed(lambda i: cg.replay(), reps, 3)
            moe.sync_status()
            graph_info = {"layers_per_graph": nlayers, "replays": reps, "us_per_layer_step": g_ms / (reps * nlayers) * 1e3,
                          "tokens_per_s": T * reps * nlayers / (g_ms * 1e-3)}
        except Exception as exc:      # a failed capture must not lose the eager line
            graph_info = {"error": str(exc)[:200]}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 activations x NVFP4 (e2m1 + e4m3 block scales) weights, f32 accumulate", "data": "synthetic",
        "config": {"workload": f"{'decode' if T <= 256 else 'prefill'} T={T} tokens/step, hidden {HIDDEN}, {EXPERTS} resident NVFP4 experts top-{TOP_K}, "
                               f"bf16 shared expert {SHARED}, {'uniform' if args.zipf is None else f'Zipf({args.zipf})-skewed'} routing",
                   "l2": f"inputs larger than L2: {nlayers} independently seeded layers "
                         f"({nlayers * EXPERTS * EXPERT_BYTES / 1e6:.0f} MB of banks) cycled step by step",
                   "timed_region": "whole block (router, routed experts, shared expert, combine), CUDA events"},
        "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline, "clocks": clocks, "graph_replay": graph_info,
    }

    if args.sweep and world == 1:
        sweep = {}
        for t in (1, 8, 512, 2048):
            if t > moe.max_tokens:
                continue
            xt = [pkg.synth.device_x(4000 + l, t, HIDDEN, dev) for l in range(nlayers)]
            o2 = torch.empty((t, HIDDEN), dtype=torch.bfloat16, device=dev)

            def st(i, t=t, xt=xt, o2=o2):
                l = i % nlayers
                g, su, sd, sg = dense[l]
                moe.moe_block(l, xt[l], g, su, sd, sg, o2)
            ms = timed(st, K, W)
            sweep[f"T={t}"] = {"tokens_per_s": t * K / (ms * 1e-3), "us_per_step": ms / K * 1e3}
        line["sweep"] = sweep

    if rank == 0 and not args.no_cpu_baseline:
        sample = min(T, 16)
        tps, threads, sec = time_cpu(sample, 3, 1)
        line["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": f"{sample} tokens of the same block per step, 3 steps, all host threads; "
                                          f"C restatement of the reference's host path"}
    if rank == 0:
        print(json.dumps(line))
    moe.close()
    if world > 1:
        dist.destroy_process_group()


def run_stack(args, pkg, moe, dense, x0, dev, T, nlayers, path):
    """One step = a pass through `nlayers` MoE blocks, x <- x + block(x) between them (the 40-layer stack of the
    benchmark configs).  Prints one JSON line: tokens/s through the whole stack, eager and from one CUDA graph."""
    import torch
    out = torch.empty((T, HIDDEN), dtype=torch.bfloat16, device=dev)
    xa, xb = torch.empty_like(x0), torch.empty_like(x0)

    def stack_pass(i=0):
        xa.copy_(x0)
        cur, nxt = xa, xb
        for l in range(nlayers):
            g, su, sd, sg = dense[l]
            moe.moe_block(l, cur, g, su, sd, sg, out, path=path)
            torch.add(cur, out, out=nxt)
            cur, nxt = nxt, cur
        return cur

    def timed(fn, steps, warmup):
        for i in range(warmup):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    W, K = max(3, args.warmup), max(1, args.steps)
    last = stack_pass()
    moe.sync_status()
    finite = bool(torch.isfinite(last.float()).all())
    rms = float(last.float().pow(2).mean().sqrt())
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    ms = timed(stack_pass, K, W)
    clocks = sampler.stop()
    graph = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        cg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cg, stream=side):
            stack_pass()
        g_ms = timed(lambda i: cg.replay(), K, 3)
        moe.sync_status()
        graph = {"ms_per_pass": g_ms / K, "tokens_per_s": T * K / (g_ms * 1e-3)}
    except Exception as exc:
        graph = {"error": str(exc)[:200]}
    print(json.dumps({
        "metric": METRIC, "value": T * K / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 activations x NVFP4 (e2m1 + e4m3 block scales) weights, f32 accumulate", "data": "synthetic",
        "config": {"workload": f"{nlayers}-layer MoE-only stack, T={T}, residual add between the blocks, "
                               f"{nlayers * EXPERTS * EXPERT_BYTES / 1e9:.1f} GB of expert banks, independent seeds per layer; "
                               "one step = one pass through all layers; value = tokens/s through the whole stack",
                   "l2": "every layer's banks are read once per pass (banks far larger than L2)",
                   "residual_rms_after_last_layer": rms, "finite": finite},
        "layer_steps_per_s": nlayers * K / (ms * 1e-3), "us_per_layer": ms / K / nlayers * 1e3,
        "graph_replay": graph, "clocks": clocks,
    }))
    moe.close()


def run_ep(args, pkg, dev, world, rank, local):
    """N > 1: the expert-parallel layer (256 experts split over the ranks, T = 8192 tokens per GPU,
    dispatch / combine by NCCL all-to-all).  Weak scaling: per-GPU tokens are fixed."""
    import torch
    import torch.distributed as dist
    ep = importlib.import_module("ferrum-torrens_b200.ep")

    T = args.tokens or 8192
    nlayers = min(max(1, args.layers), 2)
    per = EXPERTS // world
    be = ep.LibBackend(local, rank, world, pkg.ExpertShapes(HIDDEN, INTER), experts=EXPERTS, layers=nlayers,
                       top_k=TOP_K, shared_inter=SHARED, max_tokens=T, comm_sms=args.ep_comm_sms if (args.ep_chunks > 1 and args.ep_exchange == "nccl") else 0)
    dense, xs = [], []
    for l in range(nlayers):
        pkg.synth.fill_banks_on_device(be.owner, l, seed=1000 + 977 * rank + l, experts=per, slot0=l * per,
                                       expert0=rank * per)
        dense.append(pkg.synth.device_dense_weights(2000 + l, dev, zipf_alpha=args.zipf))   # replicated: same seed on every rank
        xs.append(pkg.synth.device_x(3000 + 17 * rank + l, T, HIDDEN, dev, biased=args.zipf is not None))
    out = torch.empty((T, HIDDEN), dtype=torch.bfloat16, device=dev)
    layer = ep.ExpertParallelMoE(be, world)

    chunks = max(1, args.ep_chunks)
    p2p = args.ep_exchange == "p2p"
    exchange_note = None
    if p2p:
        # symmetric memory must come up on every rank, else every rank takes the NCCL exchange
        ok = torch.ones((1,), device=dev)
        try:
            be.enable_peer_exchange()
        except Exception as exc:
            ok.zero_()
            exchange_note = f"peer exchange unavailable ({str(exc)[:120]}); NCCL all-to-all used"
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok.item()) == 0.0:
            p2p = False
            exchange_note = exchange_note or "peer exchange unavailable on another rank; NCCL all-to-all used"

    def step(i, record=None, x=None, o=None):
        l = i % nlayers
        g, su, sd, sg = dense[l]
        xin, dst = (xs[l] if x is None else x), (out if o is None else o)
        if p2p:
            layer.forward_p2p(l, xin, g, su, sd, sg, dst, record=record)
        elif record is None and chunks > 1:
            layer.forward_overlapped(l, xin, g, su, sd, sg, dst, chunks=chunks)
        else:
            layer.forward(l, xin, g, su, sd, sg, dst, record=record)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    W, K = max(3, args.warmup), max(1, args.steps)
    step(0)
    be.front.sync_status()
    be.owner.sync_status()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for i in range(W):
        step(i)
    barrier()
    l0 = be.front.kernel_launches() + be.owner.kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        step(W + i)
    e1.record()
    barrier()
    launches = be.front.kernel_launches() + be.owner.kernel_launches() - l0
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    total_ms = float(ms.item())
    clocks = sampler.stop() if rank == 0 else None

    # end to end: pinned host activations in, the result out, every step; the copies run on a copy stream with two
    # staging buffers each way, so they overlap the neighbouring steps' compute as in a serving loop
    x_host = [x.cpu().pin_memory() for x in xs]
    x_stage = [torch.empty_like(xs[0]) for _ in range(2)]
    out_dev = [torch.empty_like(out) for _ in range(2)]
    out_host = [torch.empty((T, HIDDEN), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    copy_s = torch.cuda.Stream()
    ev_h2d = [torch.cuda.Event() for _ in range(2)]
    ev_comp = [torch.cuda.Event() for _ in range(2)]
    ev_d2h = [torch.cuda.Event() for _ in range(2)]
    primed = [False]

    def step_e2e(i):
        cur = torch.cuda.current_stream()
        b = i & 1
        if not primed[0]:
            with torch.cuda.stream(copy_s):
                x_stage[b].copy_(x_host[i % nlayers], non_blocking=True)
                ev_h2d[b].record(copy_s)
            for e in ev_comp + ev_d2h:
                e.record(cur)
            primed[0] = True
        cur.wait_event(ev_h2d[b])
        cur.wait_event(ev_d2h[b])
        step(i, x=x_stage[b], o=out_dev[b])
        ev_comp[b].record(cur)
        with torch.cuda.stream(copy_s):
            copy_s.wait_event(ev_comp[b ^ 1])
            x_stage[b ^ 1].copy_(x_host[(i + 1) % nlayers], non_blocking=True)
            ev_h2d[b ^ 1].record(copy_s)
            copy_s.wait_event(ev_comp[b])
            out_host[b].copy_(out_dev[b], non_blocking=True)
            ev_d2h[b].record(copy_s)

    for i in range(2):
        step_e2e(i)
    barrier()
    e0.record()
    for i in range(K):
        step_e2e(2 + i)
    torch.cuda.current_stream().wait_event(ev_d2h[(2 + K - 1) & 1])
    e1.record()
    barrier()
    ms2 = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
    e2e = {"value": world * T * K / (float(ms2.item()) * 1e-3), "unit": UNIT, "h2d_bytes_per_step": T * HIDDEN * 2,
           "d2h_bytes_per_step": T * HIDDEN * 2}

    # phase breakdown of a few steps: time between the marks, median over steps, max over ranks
    names = ["packed", "dispatched", "computed", "returned", "combined"]
    reps = max(3, min(K, 7))
    samples = torch.zeros((reps, len(names)), device=dev)
    for i in range(reps):
        evs = {}
        start = torch.cuda.Event(enable_timing=True)
        start.record()

        def rec(name):
            evs[name] = torch.cuda.Event(enable_timing=True)
            evs[name].record()
        step(W + i, record=rec)
        torch.cuda.synchronize()
        prev = start
        for j, n in enumerate(names):
            samples[i, j] = prev.elapsed_time(evs[n])
            prev = evs[n]
    acc = samples.median(dim=0).values
    dist.all_reduce(acc, op=dist.ReduceOp.MAX)
    phases = {n: float(v) for n, v in zip(["router_shared_pack_ms", "dispatch_a2a_ms", "experts_ms", "return_a2a_ms",
                                           "combine_ms"], acc.tolist())}
    # roofline of the dominant kernel (the owner's grouped gate_up GEMM): CUDA events around every launch
    be.owner.profile(True)
    for i in range(3):
        step(W + i)
    oprof = be.owner.profile_read()
    be.owner.profile(False)
    recv_routes = float(sum(layer.last_counts[1]))
    roofline = None
    if "grouped_gate_up" in oprof:
        pk = peaks()
        g_ms, g_n = oprof["grouped_gate_up"]
        flops = recv_routes * 2.0 * HIDDEN * (2 * INTER)
        ach = flops / (g_ms / g_n * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": "grouped_gate_up (owner side, rank 0)", "achieved": ach, "peak": pk["bf16_tflops"],
                    "unit": "TFLOP/s", "frac": ach / pk["bf16_tflops"], "peak_source": pk["which"], "traffic": None,
                    "routes_received": recv_routes, "us_per_launch": g_ms / g_n * 1e3,
                    "kernels": {k: {"us_per_launch": ms / n * 1e3, "launches": n} for k, (ms, n) in oprof.items()}}
    sent = torch.tensor([sum(layer.last_counts[0]) - layer.last_counts[0][rank]], device=dev, dtype=torch.float32)
    dist.all_reduce(sent, op=dist.ReduceOp.MAX)
    if rank == 0:
        line = {
            "metric": METRIC, "value": world * T * K / (total_ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 activations x NVFP4 (e2m1 + e4m3 block scales) weights, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": f"expert-parallel layer, T={T} tokens per GPU, {EXPERTS} experts split {per} per GPU, "
                                   f"top-{TOP_K}, {'uniform' if args.zipf is None else f'Zipf({args.zipf})-skewed'} routing, " +
                                   ("dispatch / return by peer-memory kernels over NVLink" if p2p else
                                    f"NCCL all-to-all dispatch/combine, {chunks} overlapped expert range(s) per owner"),
                       "l2": f"inputs larger than L2: {nlayers} layers cycled, {T * TOP_K} routes x 4 KB rows per step",
                       "timed_region": "whole block incl. both all-to-alls, CUDA events, max over ranks"},
            "gpu_launches": int(launches), "clocks": clocks,
            "ep": {"exchange_note": exchange_note,"phases_of": "one step, marks after each phase" if p2p else "one step of the plain schedule (every phase waits for the one before)",
                   "phases_ms_max_over_ranks": phases, "unpipelined_ms_per_step": sum(phases.values()),
                   "exchange_ms_unpipelined": phases["dispatch_a2a_ms"] + phases["return_a2a_ms"],
                   "max_routes_sent_off_rank": float(sent.item()),
                   "nvlink_bytes_each_way_per_gpu": float(sent.item()) * HIDDEN * 2},
            "e2e": e2e, "roofline": roofline,
        }
        print(json.dumps(line))
    be.close()
    dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
