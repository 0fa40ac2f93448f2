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
UNIT_S = UNIT
DTYPE = "bf16 activations x NVFP4 (e2m1 + e4m3 block scales) weights, f32 accumulate"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=0, help="tokens per step (default: 64 at N=1)")
    ap.add_argument("--layers", type=int, default=4, help="independent layers cycled through")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--lm-head", action="store_true",
                    help="N = 1: only the dense NVFP4 GEMV of the lm_head (248320 x 2048), one and eight rows")
    ap.add_argument("--no-sweep", action="store_true",
                    help="N = 1: leave out the other batch sizes (T = 1, 8, 512, 2048) and the 40-layer stack that the "
                         "default line carries beside the T = 64 headline")
    ap.add_argument("--stack-layers", type=int, default=40, help="layers of the stack reported by the default line")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ep-chunks", type=int, default=2,
                    help="N > 1: expert ranges per owner that are exchanged and computed one after the other, so that "
                         "exchanges run under compute; 1 = the plain schedule")
    ap.add_argument("--ep-exchange", default="p2p", choices=["p2p", "nccl"],
                    help="N > 1: dispatch / return by this library's kernels over peer memory, or by NCCL all-to-all")
    ap.add_argument("--ep-unsorted", action="store_true",
                    help="N > 1, peer-memory exchange: dispatch bf16 rows in receive order (the owner sorts and gathers) "
                         "instead of storing them straight into the owner's sorted f16 activation matrix")
    ap.add_argument("--ep-separate-return", action="store_true",
                    help="N > 1, peer-memory exchange: return the rows by a kernel of its own instead of the owner's down GEMM")
    ap.add_argument("--ep-micro", type=int, default=1,
                    help="N > 1, peer-memory exchange: micro-batches per step (dispatch of one under the experts of the one before)")
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
    ep = args.gpus > 1
    tokens = args.tokens or (8192 if ep else 64)
    sample = min(tokens, 16)
    steps, warmup = max(1, min(args.steps, 8)), max(1, min(args.warmup, 2))
    tps, threads, sec = time_cpu(sample, steps, warmup)
    workload = (f"expert-parallel layer, T={tokens} tokens per GPU on {args.gpus} GPUs" if ep else f"decode T={tokens}") + \
        f", hidden {HIDDEN}, {EXPERTS} NVFP4 experts top-{TOP_K}, shared {SHARED}"
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "sample": f"{sample} tokens per step",
                   "sample_reason": "the CPU path costs the same per (token, route) whatever the batch size or the number "
                                    "of GPUs it is compared with, about 5 ms per token on 16 cores: the whole batch for the "
                                    "requested steps would take minutes, so a step is a 16-token sample of the batch and "
                                    "steps / warm-up are capped at 8 / 2; tokens/s is unaffected by the cut"},
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
        import datetime
        # a rank that fails before a collective must not leave the others inside it for long
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))

    import __graft_entry__ as ge
    if rank == 0:
        ge.build()
    if world > 1:
        dist.barrier()
    pkg = importlib.import_module("ferrum-torrens_b200")

    if world > 1:
        return run_ep(args, pkg, dev, world, rank, local)

    if args.lm_head:
        moe = pkg.B200MoE(local, pkg.ExpertShapes(HIDDEN, INTER), 1, experts=EXPERTS, layers=1, top_k=TOP_K, shared_inter=0,
                          max_tokens=64)
        print(json.dumps({"lm_head": measure_lm_head(torch, moe, dev, peaks(), max(1, args.steps), max(3, args.warmup))}))
        moe.close()
        return
    return run_single(args, pkg, dev, local)


L2_BYTES = 126e6


def timed_steps(torch, fn, steps, warmup):
    """CUDA-event time of `steps` calls of fn(i) after `warmup` untimed ones, synchronised on both sides (ms)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    return float(e0.elapsed_time(e1))


class Workload:
    """One batch size of the whole block on one adapter: `nl` independently seeded layers cycled step by step."""

    def __init__(self, pkg, moe, dense, dev, T, nl, biased, path):
        import torch
        self.torch, self.pkg, self.moe, self.dense, self.T, self.nl, self.path = torch, pkg, moe, dense, T, nl, path
        self.xs = [pkg.synth.device_x(3000 + l, T, HIDDEN, dev, biased=biased) for l in range(nl)]
        self.out = torch.empty((T, HIDDEN), dtype=torch.bfloat16, device=dev)
        self.ids = torch.empty((T, TOP_K), dtype=torch.int32, device=dev)
        self.wts = torch.empty((T, TOP_K), dtype=torch.float32, device=dev)

    def step(self, i, x=None, o=None):
        l = i % self.nl
        g, su, sd, sg = self.dense[l]
        self.moe.moe_block(l, self.xs[l] if x is None else x, g, su, sd, sg, self.out if o is None else o,
                           ids_out=self.ids, weights_out=self.wts, path=self.path)

    def time_block(self, K, W):
        self.step(0)
        self.moe.sync_status()      # a kernel that gave up a bounded wait fails here, before anything is timed
        l0 = self.moe.kernel_launches()
        ms = timed_steps(self.torch, self.step, K, W)
        launches = (self.moe.kernel_launches() - l0) * K // (K + W)
        return ms, launches

    def profile(self, K, W):
        """Per-kernel CUDA-event pass.  The routed half runs alone (serving call with the router's ids), so that
        the shared expert, which the whole block overlaps on a second stream, does not share the SMs with the
        timed kernels; router and shared expert are then timed each alone.  Returns (kernels, mean distinct
        experts per step)."""
        torch, moe, pkg = self.torch, self.moe, self.pkg
        routed = []
        for l in range(self.nl):
            self.step(l)
            torch.cuda.synchronize()
            routed.append((self.ids.clone(), self.wts.clone()))
        uniq = [int(torch.unique(i).numel()) for i, _ in routed]
        reqs = [pkg.MoEDeviceRequest(l, HIDDEN, INTER, TOP_K, self.xs[l], routed[l][0], routed[l][1]) for l in range(self.nl)]
        for i in range(W):
            moe.grouped_moe_staged(reqs[i % self.nl], self.out, path=self.path)
        moe.profile(True)
        for i in range(K):
            moe.grouped_moe_staged(reqs[i % self.nl], self.out, path=self.path)
        prof = moe.profile_read()
        moe.profile(False)
        moe.profile(True)
        for i in range(K):
            g, su, sd, sg = self.dense[i % self.nl]
            moe.router(self.xs[i % self.nl], g)
            moe.shared_expert(self.xs[i % self.nl], su, sd, sg)
        prof.update(moe.profile_read())
        moe.profile(False)
        return prof, sum(uniq) / len(uniq)


def roofline_of(prof, U, T, nl, pk):
    """`roofline` object of the dominant routed-expert kernel from a per-kernel profile."""
    gate_kind = "expert_gate_up" if "expert_gate_up" in prof else "grouped_gate_up"
    g_ms, g_n = prof[gate_kind]
    us = g_ms / g_n * 1e3
    kernels = {k: {"us_per_launch": ms / n * 1e3, "launches": n} for k, (ms, n) in prof.items()}
    if gate_kind == "expert_gate_up":
        # decode kernels: bound by the stream of the routed experts' weights
        gu_bytes = U * GATE_UP_BYTES + T * HIDDEN * 2
        achieved = gu_bytes / (us * 1e-6) / 1e9
        touched = nl * U * EXPERT_BYTES
        resident = touched < 2 * L2_BYTES
        r = {"bound": "L2 (the cycled experts fit the 126 MB L2)" if resident else "hbm", "kernel": gate_kind,
             "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
             "peak_source": pk["which"], "frac_of_nominal_8000": achieved / 8000.0,
             "traffic": None,
             "traffic_source": "not captured in this run; profiles/expert_ldg_T64.md holds the ncu capture of this "
                               "kernel (dram bytes read + written against the algorithmic bytes of the same launch: 1.04x)",
             "distinct_experts": U, "bytes_per_launch": gu_bytes, "us_per_launch": us,
             "expert_bytes_touched_per_cycle": touched, "l2_resident": resident, "kernels": kernels}
        if "expert_down" in prof:
            d_ms, d_n = prof["expert_down"]
            dn = (U * DOWN_BYTES) / (d_ms / d_n * 1e-3) / 1e9
            r["down"] = {"achieved": dn, "frac": dn / pk["hbm_gbs"], "us_per_launch": d_ms / d_n * 1e3}
            r["expert_weights_gbs"] = (U * EXPERT_BYTES) / ((g_ms / g_n + d_ms / d_n) * 1e-3) / 1e9
        return r
    # tcgen05 grouped GEMM: useful flops of the routes (padding of ragged groups not counted)
    flops = T * TOP_K * 2.0 * HIDDEN * (2 * INTER)
    achieved = flops / (us * 1e-6) / 1e12
    r = {"bound": "tensor", "kernel": gate_kind, "achieved": achieved, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
         "frac": achieved / pk["bf16_tflops"],
         "peak_source": pk["which"] + " (burst; sustained %.0f)" % pk["bf16_tflops_sustained"], "traffic": None,
         "distinct_experts": U, "flops_per_launch": flops, "us_per_launch": us,
         "weight_stream_gbs": U * GATE_UP_BYTES / (us * 1e-6) / 1e9, "kernels": kernels}
    if "grouped_down" in prof:
        d_ms, d_n = prof["grouped_down"]
        dn = T * TOP_K * 2.0 * INTER * HIDDEN / (d_ms / d_n * 1e-3) / 1e12
        r["down"] = {"achieved": dn, "frac": dn / pk["bf16_tflops"], "us_per_launch": d_ms / d_n * 1e3}
    return r


def stack_pass_fn(torch, moe, dense, x0, nlayers, path):
    """One pass through `nlayers` MoE blocks with a bf16 residual add between them."""
    T = x0.shape[0]
    out = torch.empty((T, HIDDEN), dtype=torch.bfloat16, device=x0.device)
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
    return stack_pass


def measure_stack(torch, moe, dense, x0, nlayers, path, K, W):
    """tokens/s through the whole stack, eager and replayed from one CUDA graph."""
    T = x0.shape[0]
    fn = stack_pass_fn(torch, moe, dense, x0, nlayers, path)
    last = fn()
    moe.sync_status()
    finite = bool(torch.isfinite(last.float()).all())
    rms = float(last.float().pow(2).mean().sqrt())
    ms = timed_steps(torch, fn, K, W)
    res = {"layers": nlayers, "tokens": T, "ms_per_pass": ms / K, "tokens_per_s": T * K / (ms * 1e-3),
           "us_per_layer": ms / K / nlayers * 1e3, "residual_rms_after_last_layer": rms, "finite": finite,
           "expert_bank_gb": nlayers * EXPERTS * EXPERT_BYTES / 1e9}
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        cg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cg, stream=side):
            fn()
        g_ms = timed_steps(torch, lambda i: cg.replay(), K, 3)
        moe.sync_status()
        res["graph_replay"] = {"ms_per_pass": g_ms / K, "tokens_per_s": T * K / (g_ms * 1e-3)}
    except Exception as exc:
        res["graph_replay"] = {"error": str(exc)[:200]}
    return res


def measure_lm_head(torch, moe, dev, pk, K, W):
    """The neighbour of the layer at the end of the model: the dense NVFP4 GEMV of `lm_head` (K-major bank, vocabulary
    248320 x hidden 2048), one and eight rows.  HBM-bound: 286.6 MB of bank per call, larger than L2."""
    N, Kd = 248320, HIDDEN
    g = torch.Generator(device=dev).manual_seed(4242)
    packed = torch.randint(-2**31, 2**31 - 1, (Kd // 8, N), generator=g, device=dev, dtype=torch.int64).to(torch.int32)
    # e4m3 scale bytes 0x28..0x47 (2^-2 .. 1.75): no NaN, no overflow of the f16 product
    scale = torch.randint(0x28, 0x48, (Kd // 16, N), generator=g, device=dev, dtype=torch.int32).to(torch.uint8)
    glob = torch.full((N,), 0x3C00, dtype=torch.int16, device=dev)
    bank_bytes = packed.numel() * 4 + scale.numel() + glob.numel() * 2
    out = {"workload": f"dense NVFP4 GEMV (lm_head), N={N} K={Kd}, K-major bank of {bank_bytes / 1e6:.1f} MB (larger than L2)",
           "peak_GBps": pk["hbm_gbs"], "peak_source": pk["which"]}
    for m in (1, 8):
        a = torch.randn((m, Kd), generator=g, device=dev).to(torch.bfloat16)
        c = torch.empty((m, N), dtype=torch.float32, device=dev)
        ms = timed_steps(torch, lambda i: moe.dense_gemv(a, packed, scale, glob, c), K, W)
        moe.sync_status()
        us = ms / K * 1e3
        algo = bank_bytes + m * Kd * 2 + m * N * 4
        out[f"M={m}"] = {"us_per_call": us, "algorithmic_bytes": algo, "achieved_GBps": algo / (us * 1e-6) / 1e9,
                         "frac": algo / (us * 1e-6) / 1e9 / pk["hbm_gbs"]}
    del packed, scale, c
    torch.cuda.empty_cache()
    return out


def run_single(args, pkg, dev, local):
    import torch
    T = args.tokens or 64
    path = {"auto": 0, "gemv": 1, "grouped": 2, "scalar": 3}[args.path]
    cycle = max(1, args.layers)
    # the default line also carries the other batch sizes of the metric (T = 1, 8, 512, 2048) and the 40-layer
    # stack; a run asked for one particular workload (--tokens / --zipf / --path / --stack) reports only that
    default_line = not (args.tokens or args.zipf is not None or args.path != "auto" or args.stack) and not args.no_sweep
    # --stack --layers N runs a stack of N layers; the default line keeps --stack-layers layers resident
    total_layers = max(cycle, args.stack_layers) if default_line else cycle
    max_tokens = max(T, 64, 2048 if default_line else 0)
    moe = pkg.B200MoE(local, pkg.ExpertShapes(HIDDEN, INTER), EXPERTS * total_layers, experts=EXPERTS, layers=total_layers,
                      top_k=TOP_K, shared_inter=SHARED, max_tokens=max_tokens)
    G_SMALL = (0x2400, 0x1400)    # f16 row globals 2^-6 / 2^-10: a stack's residual stream stays O(1)
    G_ONE = (0x3C00, 0x3C00)      # 1.0, the benchmark configs' global scale
    for l in range(total_layers):
        pkg.synth.fill_banks_on_device(moe, l, seed=1000 + l, slot0=l * EXPERTS, global_bits=G_SMALL if args.stack else G_ONE)
    dense = [pkg.synth.device_dense_weights(2000 + l, dev, zipf_alpha=args.zipf) for l in range(total_layers)]
    W, K = max(3, args.warmup), max(1, args.steps)
    pk = peaks()

    if args.stack:
        x0 = pkg.synth.device_x(3000, T, HIDDEN, dev, biased=args.zipf is not None)
        sampler = ClockSampler(local)
        sampler.start()
        st = measure_stack(torch, moe, dense, x0, total_layers, path, K, W)
        clocks = sampler.stop()
        print(json.dumps({
            "metric": METRIC, "value": st["tokens_per_s"], "unit": UNIT_S, "n_gpus": 1, "steps": K, "warmup": W,
            "ms_per_step": st["ms_per_pass"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": DTYPE, "data": "synthetic",
            "config": {"workload": f"{total_layers}-layer MoE-only stack, T={T}, residual add between the blocks, "
                                   f"{st['expert_bank_gb']:.1f} GB of expert banks, independent seeds per layer; "
                                   "one step = one pass through all layers; value = tokens/s through the whole stack",
                       "l2": "every layer's banks are read once per pass (banks far larger than L2)"},
            "stack": st, "clocks": clocks}))
        moe.close()
        return

    sampler = ClockSampler(local)
    sampler.start()
    wl = Workload(pkg, moe, dense, dev, T, cycle, args.zipf is not None, path)
    total_ms, launches = wl.time_block(K, W)
    value = T * K / (total_ms * 1e-3)
    step, xs, out = wl.step, wl.xs, wl.out
    nlayers = cycle

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

    for i in range(W):
        step_e2e(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        step_e2e(W + i)
    torch.cuda.current_stream().wait_event(ev_d2h[(W + K - 1) & 1])    # the last result has reached the host buffer
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = float(e0.elapsed_time(e1))

    # the same without any overlap: copy in, block, copy out on one stream
    def step_serial(i):
        x_stage[0].copy_(x_host[i % nlayers], non_blocking=True)
        step(i, x=x_stage[0], o=out_dev[0])
        out_host[0].copy_(out_dev[0], non_blocking=True)

    serial_ms = timed_steps(torch, step_serial, K, W)
    e2e = {"value": T * K / (e2e_ms * 1e-3), "unit": UNIT_S, "h2d_bytes_per_step": T * HIDDEN * 2,
           "d2h_bytes_per_step": T * HIDDEN * 2,
           "how": "pinned host buffers; H2D of step i + 1 and D2H of step i on a copy stream (two staging buffers each "
                  "way) under the compute of the neighbouring step",
           "serial_value": T * K / (serial_ms * 1e-3)}

    prof, U = wl.profile(K, W)
    roofline = roofline_of(prof, U, T, nlayers, pk)

    # the same steps replayed from one captured CUDA graph (one block per layer in the graph): what an engine
    # that captures its decode step gets; reported beside the eager numbers, not instead of them
    graph_info = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        cg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cg, stream=side):
            for l in range(nlayers):
                step(l)
        reps = max(1, K // nlayers)
        g_ms = timed_steps(torch, lambda i: cg.replay(), reps, 3)
        moe.sync_status()
        graph_info = {"layers_per_graph": nlayers, "replays": reps, "us_per_layer_step": g_ms / (reps * nlayers) * 1e3,
                      "tokens_per_s": T * reps * nlayers / (g_ms * 1e-3)}
    except Exception as exc:      # a failed capture must not lose the eager line
        graph_info = {"error": str(exc)[:200]}

    routing = "uniform" if args.zipf is None else f"Zipf({args.zipf})-skewed"
    line = {
        "metric": METRIC, "value": value, "unit": UNIT_S, "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": DTYPE, "data": "synthetic",
        "config": {"workload": f"{'decode' if T <= 256 else 'prefill'} T={T} tokens/step, hidden {HIDDEN}, {EXPERTS} resident NVFP4 "
                               f"experts top-{TOP_K}, bf16 shared expert {SHARED}, {routing} routing",
                   "l2": f"inputs larger than L2: {nlayers} independently seeded layers cycled step by step, "
                         f"{nlayers * U * EXPERT_BYTES / 1e6:.0f} MB of routed expert bytes touched per cycle (L2 is 126 MB)",
                   "timed_region": "whole block (router, routed experts, shared expert, combine), CUDA events"},
        "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline, "graph_replay": graph_info,
    }

    if default_line:
        # the other batch sizes the metric is quoted on.  Decode sizes cycle every resident layer so that the few
        # experts a step touches are not served from L2; prefill sizes route with the Zipf(1.1) bias of config 3.
        sweep = {}
        dense_zipf = [pkg.synth.device_dense_weights(2000 + l, dev, zipf_alpha=1.1) for l in range(cycle)]
        for t, zipf in ((1, None), (8, None), (512, 1.1), (2048, 1.1)):
            nl = total_layers if zipf is None else cycle
            w2 = Workload(pkg, moe, dense if zipf is None else dense_zipf, dev, t, nl, zipf is not None, 0)
            k2 = K if t <= 64 else max(8, K // 2)
            ms, _ = w2.time_block(k2, W)
            entry = {"tokens_per_s": t * k2 / (ms * 1e-3), "ms_per_step": ms / k2, "layers_cycled": nl,
                     "routing": "uniform" if zipf is None else f"Zipf({zipf}) bias through the router"}
            p2, u2 = w2.profile(k2, W)
            entry["roofline"] = roofline_of(p2, u2, t, nl, pk)
            if t == 1:
                try:
                    side = torch.cuda.Stream()
                    side.wait_stream(torch.cuda.current_stream())
                    cg = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(cg, stream=side):
                        for l in range(nl):
                            w2.step(l)
                    g_ms = timed_steps(torch, lambda i: cg.replay(), 3, 2)
                    moe.sync_status()
                    entry["graph_replay_us_per_step"] = g_ms / (3 * nl) * 1e3
                except Exception as exc:
                    entry["graph_replay_us_per_step"] = str(exc)[:120]
            sweep[f"T={t}"] = entry
            del w2
        line["sweep"] = sweep
        # config 4: the 40-layer stack (row globals 2^-6 / 2^-10 so that the residual stream stays O(1))
        pkg.synth.set_global_bits_on_device(moe, 0, EXPERTS * total_layers, G_SMALL)
        stack = {}
        for t in (1, 2048):
            x0 = pkg.synth.device_x(3500 + t, t, HIDDEN, dev)
            stack[f"T={t}"] = measure_stack(torch, moe, dense, x0, total_layers, 0, max(4, K // 4), 3)
        line["stack40"] = stack
        pkg.synth.set_global_bits_on_device(moe, 0, EXPERTS * total_layers, G_ONE)

    if default_line:
        line["lm_head"] = measure_lm_head(torch, moe, dev, pk, K, W)

    # the sampler ran through every timed region above (all GPU-busy)
    line["clocks"] = sampler.stop()
    if not args.no_cpu_baseline:
        sample = min(T, 16)
        tps, threads, sec = time_cpu(sample, 3, 1)
        line["cpu_baseline"] = {"value": tps, "unit": UNIT_S, "cores": threads, "kind": "port",
                                "sample": f"{sample} tokens of the same block per step, 3 steps, all host threads; "
                                          f"C restatement of the reference's host path"}
    print(json.dumps(line))
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
                       top_k=TOP_K, shared_inter=SHARED, max_tokens=T, comm_sms=args.ep_comm_sms if ((args.ep_chunks > 1 and args.ep_exchange == "nccl") or
                                                    (args.ep_micro > 1 and args.ep_exchange == "p2p")) else 0)
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

    micro = max(1, args.ep_micro)

    def step(i, record=None, x=None, o=None):
        l = i % nlayers
        g, su, sd, sg = dense[l]
        xin, dst = (xs[l] if x is None else x), (out if o is None else o)
        if p2p:
            if not args.ep_unsorted and micro == 1 and not args.ep_separate_return:
                return layer.forward_p2p_sorted(l, xin, g, su, sd, sg, dst, record=record)
            # the phase breakdown (record set) runs the step as one batch, every phase after the one before
            return layer.forward_p2p(l, xin, g, su, sd, sg, dst, record=record, micro=1 if record else micro,
                                     fused_return=not args.ep_separate_return)
        if record is None and chunks > 1:
            return layer.forward_overlapped(l, xin, g, su, sd, sg, dst, chunks=chunks)
        return layer.forward(l, xin, g, su, sd, sg, dst, record=record)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    W, K = max(3, args.warmup), max(1, args.steps)
    ep_ids, _ = step(0)
    be.front.sync_status()
    be.owner.sync_status()

    # Before anything is timed: (1) the expert-parallel result of rank 0's first 256 tokens against one adapter on
    # this GPU that holds all 256 experts (the banks are regenerated from every owner's seed), and (2) the same
    # 8192-token block on that one GPU alone, so that the N-GPU figure has a same-workload one-GPU reference.
    parity = {"checked": False}
    single_tps = None
    if rank == 0:
        solo = pkg.B200MoE(local, pkg.ExpertShapes(HIDDEN, INTER), EXPERTS * nlayers, experts=EXPERTS, layers=nlayers,
                           top_k=TOP_K, shared_inter=SHARED, max_tokens=T)
        for l in range(nlayers):
            for r in range(world):
                pkg.synth.fill_banks_on_device(solo, l, seed=1000 + 977 * r + l, experts=per, slot0=l * EXPERTS + r * per,
                                               expert0=r * per)
        n_chk = min(256, T)
        want = torch.empty((n_chk, HIDDEN), dtype=torch.bfloat16, device=dev)
        want_ids = torch.empty((n_chk, TOP_K), dtype=torch.int32, device=dev)
        g, su, sd, sg = dense[0]
        solo.moe_block(0, xs[0][:n_chk].contiguous(), g, su, sd, sg, want, ids_out=want_ids)
        solo.sync_status()
        got = out[:n_chk].float()
        rel = float((got - want.float()).norm() / want.float().norm())
        parity = {"checked": True, "tokens": n_chk, "ids_equal": bool(torch.equal(ep_ids[:n_chk], want_ids)),
                  "parity_rel_l2": rel, "bar_rel_l2": 1e-2,
                  "against": "one adapter on rank 0's GPU holding all experts, same seeded banks and inputs"}
        o1 = torch.empty((T, HIDDEN), dtype=torch.bfloat16, device=dev)

        def solo_step(i):
            l = i % nlayers
            g, su, sd, sg = dense[l]
            solo.moe_block(l, xs[l], g, su, sd, sg, o1)
        ms1 = timed_steps(torch, solo_step, max(4, K // 2), 3)
        solo.sync_status()
        single_tps = T * max(4, K // 2) / (ms1 * 1e-3)
        solo.close()
        del solo, o1
        torch.cuda.empty_cache()
    bad = torch.zeros((1,), device=dev)
    if rank == 0 and not (parity["ids_equal"] and parity["parity_rel_l2"] <= 1e-2):
        bad.fill_(1.0)
    dist.all_reduce(bad, op=dist.ReduceOp.MAX)
    if float(bad.item()) != 0.0:
        if rank == 0:
            print(json.dumps({"error": "expert-parallel parity check failed", "ep": parity}))
        be.close()
        dist.destroy_process_group()
        raise SystemExit(3)

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
        # three profiled steps; a step that cuts the owner's experts into ranges (or micro-batches) launches the
        # GEMM once per range, each on its share of the routes
        launches_per_step = max(1.0, g_n / 3.0)
        flops = recv_routes / launches_per_step * 2.0 * HIDDEN * (2 * INTER)
        ach = flops / (g_ms / g_n * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": "grouped_gate_up (owner side, rank 0)", "achieved": ach, "peak": pk["bf16_tflops"],
                    "unit": "TFLOP/s", "frac": ach / pk["bf16_tflops"], "peak_source": pk["which"], "traffic": None,
                    "routes_received": recv_routes, "gemm_launches_per_step": launches_per_step,
                    "us_per_launch": g_ms / g_n * 1e3,
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
                                   (("rows dispatched by a peer-memory kernel straight into the owner's sorted f16 activation matrix (no permutation "
                                     "build or gather on the owner), " if not args.ep_unsorted and micro == 1 and not args.ep_separate_return
                                     else "dispatch by a peer-memory kernel in receive order, ") + f"return by {'the down GEMM itself' if not args.ep_separate_return else 'a kernel reading the GEMM rows in place'} "
                                    f"(plain peer stores over NVLink), {micro} micro-batch(es) "
                                    f"per step (dispatch of one under the experts of the one before, {args.ep_comm_sms if micro > 1 else 0} SMs "
                                    f"left to the exchange)" if p2p else
                                    f"NCCL all-to-all dispatch/combine, {chunks} overlapped expert range(s) per owner"),
                       "l2": f"inputs larger than L2: {nlayers} layers cycled, {T * TOP_K} routes x 4 KB rows per step",
                       "timed_region": "whole block incl. both all-to-alls, CUDA events, max over ranks"},
            "gpu_launches": int(launches), "clocks": clocks,
            "ep": {"parity": parity, "parity_rel_l2": parity.get("parity_rel_l2"), "ids_equal": parity.get("ids_equal"),
                   "single_gpu_same_block_tokens_per_s": single_tps,
                   "efficiency_vs_1gpu": (world * T * K / (total_ms * 1e-3) / world / single_tps) if single_tps else None,
                   "efficiency_note": "tokens/s per GPU of this run over tokens/s of the same 8192-token block on one GPU "
                                      "with all 256 experts resident (rank 0, measured in this run before the timed steps)",
                   "exchange_note": exchange_note,"phases_of": "one step run as ONE batch, marks after each phase" if p2p else "one step of the plain schedule (every phase waits for the one before)",
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
