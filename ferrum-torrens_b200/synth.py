"""Seeded synthetic MoE layers with the shapes and value distributions of the benchmark configs.

* activations x [T, hidden]: N(0, 1) rounded to bf16;
* router weight [experts, hidden]: N(0, 0.02) -> bf16.  An optional per-expert popularity bias
  (Zipf with exponent alpha over a random ranking) is carried in hidden column 0 of the router
  weight, and the activations then hold 1.0 in column 0, so the skew goes through the real
  router: logit[t, e] = bias[e] + sum_{k>0} x[t,k] w[e,k];
* every expert: gate_up packed [2I, H/2] and down packed [H, I/2] uniform random bytes (uniform
  E2M1 codes), block scales 2^u with u ~ U[-6, 0] rounded to the nearest e4m3 code, f16 row
  globals 1.0 (0x3c00);
* shared expert gate_up [2*SI, H], down [H, SI], shared gate [1, H]: N(0, 0.02) -> bf16.

numpy builds host layers for the parity tests; `fill_banks_on_device` draws the same
distributions with torch directly into an adapter's banks for the large benchmark workloads.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

_E4M3_POS = None


def _e4m3_table():
    """(values, codes) of the positive finite e4m3fn codes, ascending."""
    global _E4M3_POS
    if _E4M3_POS is None:
        codes = np.arange(1, 0x7F, dtype=np.int32)
        exp, man = codes >> 3, codes & 7
        vals = np.where(exp == 0, man * 2.0 ** -9, (1 + man / 8.0) * np.exp2(exp - 7.0))
        _E4M3_POS = (vals.astype(np.float64), codes.astype(np.uint8))
    return _E4M3_POS


def nearest_e4m3(v: np.ndarray) -> np.ndarray:
    """Nearest positive e4m3fn code of each value (ties to the lower code)."""
    vals, codes = _e4m3_table()
    mid = (vals[1:] + vals[:-1]) / 2
    return codes[np.searchsorted(mid, v.astype(np.float64), side="left")]


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def zipf_bias(rng: np.random.Generator, experts: int, alpha: float) -> np.ndarray:
    """log of a Zipf(alpha) popularity over a random ranking of the experts."""
    rank = rng.permutation(experts) + 1
    return (-alpha * np.log(rank)).astype(np.float32)


@dataclass
class HostLayer:
    hidden: int
    inter: int
    experts: int
    top_k: int
    shared_inter: int
    gate_w: np.ndarray      # [E, H] bf16 bits
    sh_gate_up: np.ndarray  # [2*SI, H] bf16 bits
    sh_down: np.ndarray     # [H, SI] bf16 bits
    sh_gate: np.ndarray     # [1, H] bf16 bits
    banks: list             # six uint8 arrays [E, row_bytes] in bank order
    biased: bool = False

    def fields(self, expert: int):
        return [b[expert] for b in self.banks]


def make_layer(seed: int, hidden: int = 2048, inter: int = 512, experts: int = 256, top_k: int = 8,
               shared_inter: int = 512, zipf_alpha: float | None = None, global_scale=1.0) -> HostLayer:
    """`global_scale`: the f16 row global of every expert row, one value or a (gate_up, down) pair.  The
    benchmark configs use 1.0; (2^-6, 2^-10) gives layer outputs of magnitude O(0.1 .. 1), as real
    checkpoints have and as a multi-layer stack needs to keep its residual stream bounded."""
    rng = np.random.default_rng(seed)
    gate = rng.normal(0.0, 0.02, (experts, hidden)).astype(np.float32)
    if zipf_alpha is not None:
        gate[:, 0] = zipf_bias(rng, experts, zipf_alpha)
    gs = global_scale if isinstance(global_scale, (tuple, list)) else (global_scale, global_scale)
    f16s = [np.array([g], np.float16).view(np.uint16)[0] for g in gs]

    def bank(rows, cols, f16):
        packed = rng.integers(0, 256, (experts, rows * cols // 2), dtype=np.uint8)
        u = rng.uniform(-6.0, 0.0, (experts, rows * cols // 16))
        scale = nearest_e4m3(np.exp2(u))
        glob = np.full((experts, rows), f16, np.uint16).view(np.uint8).reshape(experts, rows * 2)
        return packed, scale, glob

    gu = bank(2 * inter, hidden, f16s[0])
    dn = bank(hidden, inter, f16s[1])
    n = lambda *s: f32_to_bf16_bits(rng.normal(0.0, 0.02, s).astype(np.float32))
    return HostLayer(hidden, inter, experts, top_k, shared_inter, f32_to_bf16_bits(gate),
                     n(2 * shared_inter, hidden), n(hidden, shared_inter), n(1, hidden), [*gu, *dn],
                     biased=zipf_alpha is not None)


def make_x(seed: int, tokens: int, hidden: int, biased: bool = False) -> np.ndarray:
    """Activations as bf16 bit patterns [T, hidden]."""
    rng = np.random.default_rng(seed ^ 0x5EED)
    x = rng.normal(0.0, 1.0, (tokens, hidden)).astype(np.float32)
    if biased:
        x[:, 0] = 1.0
    return f32_to_bf16_bits(x)


# ---- device-side generation for the benchmark --------------------------------------------------

def fill_banks_on_device(moe, layer: int, seed: int, experts: int | None = None, slot0: int = 0, chunk: int = 64,
                         expert0: int = 0, global_bits=(0x3C00, 0x3C00)):
    """Draws `experts` experts of `layer` (ids expert0, expert0 + 1, ..) straight into the adapter's banks
    (slot = slot0 + i) and marks them resident.  Same distributions as make_layer.  `global_bits`: f16 bit
    patterns of the gate_up and down row globals (1.0 by default; a multi-layer stack uses smaller ones so that
    the residual stream stays O(1))."""
    import torch
    experts = experts if experts is not None else moe.experts
    g = torch.Generator(device=f"cuda:{moe.device}").manual_seed(seed)
    banks = moe.bank_tensors()
    for b, t in enumerate(banks):
        rows = t[slot0:slot0 + experts]
        kind = b % 3
        for s in range(0, experts, chunk):
            part = rows[s:s + chunk]
            if kind == 0:
                part.copy_(torch.randint(0, 256, part.shape, generator=g, device=part.device, dtype=torch.uint8))
            elif kind == 1:
                u = torch.rand(part.shape, generator=g, device=part.device) * -6.0
                part.copy_(torch.exp2(u).to(torch.float8_e4m3fn).view(torch.uint8))
            else:
                part.view(torch.int16).fill_(global_bits[b // 3])
    torch.cuda.synchronize()
    for e in range(experts):
        moe.adopt(layer, expert0 + e, slot0 + e)


def set_global_bits_on_device(moe, slot0: int, slots: int, global_bits=(0x3C00, 0x3C00)):
    """Overwrites the f16 row globals of `slots` slots starting at slot0 (gate_up, down bit patterns)."""
    import torch
    banks = moe.bank_tensors()
    for b in (2, 5):
        banks[b][slot0:slot0 + slots].view(torch.int16).fill_(global_bits[b // 3])
    torch.cuda.synchronize()


def device_dense_weights(seed: int, device, hidden: int = 2048, experts: int = 256, shared_inter: int = 512,
                         zipf_alpha: float | None = None):
    """Router and shared-expert weights as bf16 CUDA tensors: (gate_w, sh_gate_up, sh_down, sh_gate)."""
    import torch
    g = torch.Generator(device=device).manual_seed(seed ^ 0xD15E)
    n = lambda *s: (torch.randn(s, generator=g, device=device) * 0.02)
    gate = n(experts, hidden)
    if zipf_alpha is not None:
        rank = torch.randperm(experts, generator=g, device=device).float() + 1
        gate[:, 0] = -zipf_alpha * torch.log(rank)
    bf = torch.bfloat16
    return gate.to(bf), n(2 * shared_inter, hidden).to(bf), n(hidden, shared_inter).to(bf), n(1, hidden).to(bf)


def device_x(seed: int, tokens: int, hidden: int, device, biased: bool = False):
    import torch
    g = torch.Generator(device=device).manual_seed(seed ^ 0x5EED)
    x = torch.randn((tokens, hidden), generator=g, device=device)
    if biased:
        x[:, 0] = 1.0
    return x.to(torch.bfloat16)
