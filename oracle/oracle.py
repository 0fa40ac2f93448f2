"""ctypes front end of the CPU checker (TEST INFRASTRUCTURE ONLY).

Everything here runs on host memory with numpy arrays; it exists so the tests
can compare the CUDA path against the reference's host algorithm.
"""
from __future__ import annotations

import ctypes as C
import os
import sys
from dataclasses import dataclass

import numpy as np

from . import build as _build

_lib = None

OK, BAD, SLOT_OUT_OF_RANGE = 0, 1, 2


class OracleError(Exception):
    """Mirrors MoEError (src/domain/expert_kernel.rs:21-39)."""

    def __init__(self, kind: str, msg: str, slot: int | None = None, capacity: int | None = None):
        super().__init__(msg)
        self.kind, self.slot, self.capacity = kind, slot, capacity


class _Banks(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("gu_packed", "gu_scale", "gu_global", "dn_packed",
                                          "dn_scale", "dn_global")] + \
               [(n, C.c_size_t) for n in ("gu_packed_len", "gu_scale_len", "gu_global_len",
                                          "dn_packed_len", "dn_scale_len", "dn_global_len",
                                          "slots", "gu_rows", "gu_cols", "dn_rows", "dn_cols")]


class _Layer(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in ("hidden", "inter", "experts", "top_k", "shared_inter")] + \
               [(n, C.c_void_p) for n in ("gate_w", "sh_gate_up", "sh_down", "sh_gate")] + \
               [("banks", _Banks)]


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(_build.build())
        f32, u16, u8 = C.c_float, C.c_uint16, C.c_uint8
        _lib.ftmo_bf16_to_f32.restype = f32
        _lib.ftmo_bf16_to_f32.argtypes = [u16]
        _lib.ftmo_f16_to_f32.restype = f32
        _lib.ftmo_f16_to_f32.argtypes = [u16]
        _lib.ftmo_e4m3fn_to_f32.restype = f32
        _lib.ftmo_e4m3fn_to_f32.argtypes = [u8]
        _lib.ftmo_fp4_nibble.restype = f32
        _lib.ftmo_fp4_nibble.argtypes = [u8, C.c_int]
        _lib.ftmo_f32_to_bf16.restype = u16
        _lib.ftmo_f32_to_bf16.argtypes = [f32]
        _lib.ftmo_expf.restype = f32
        _lib.ftmo_expf.argtypes = [f32]
        _lib.ftmo_silu.restype = f32
        _lib.ftmo_silu.argtypes = [f32]
        _lib.ftmo_sigmoid.restype = f32
        _lib.ftmo_sigmoid.argtypes = [f32]
        _lib.ftmo_add_rmsnorm.restype = None
        _lib.ftmo_rms_norm.restype = None
        _lib.ftmo_nvfp4_dense_gemv.restype = None
        _lib.ftmo_cache_new.restype = C.c_void_p
        _lib.ftmo_cache_new.argtypes = [C.c_size_t] * 3
        _lib.ftmo_cache_free.argtypes = [C.c_void_p]
        _lib.ftmo_cache_slot_of.restype = C.c_int32
        _lib.ftmo_cache_slot_of.argtypes = [C.c_void_p, C.c_size_t, C.c_uint32]
        _lib.ftmo_cache_id_of_slot.restype = C.c_int32
        _lib.ftmo_cache_id_of_slot.argtypes = [C.c_void_p, C.c_size_t]
        _lib.ftmo_cache_ensure.restype = C.c_size_t
        _lib.ftmo_cache_ensure.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t,
                                           C.c_void_p, C.c_void_p, C.c_void_p]
    return _lib


def _p(a: np.ndarray) -> C.c_void_p:
    return C.c_void_p(a.ctypes.data)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def max_threads() -> int:
    return int(lib().ftmo_max_threads())


# ---- scalar decoders -------------------------------------------------------
def bf16_to_f32(bits: int) -> float:
    return float(lib().ftmo_bf16_to_f32(bits))


def f16_to_f32(bits: int) -> float:
    return float(lib().ftmo_f16_to_f32(bits))


def e4m3fn_to_f32(bits: int) -> float:
    return float(lib().ftmo_e4m3fn_to_f32(bits))


def fp4_nibble(byte: int, high: bool) -> float:
    return float(lib().ftmo_fp4_nibble(byte, 1 if high else 0))


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even narrowing, vectorised (same rule as ftmo_f32_to_bf16)."""
    u = _c(a, np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def expf(x: float) -> float:
    return float(lib().ftmo_expf(x))


def silu(x: float) -> float:
    return float(lib().ftmo_silu(x))


def sigmoid(x: float) -> float:
    return float(lib().ftmo_sigmoid(x))


def nvfp4_block(packed: np.ndarray, rows: int, cols: int, scale: np.ndarray) -> np.ndarray:
    packed, scale = _c(packed, np.uint8), _c(scale, np.uint8)
    out = np.empty((rows, cols), np.float32)
    lib().ftmo_nvfp4_block(_p(packed), C.c_size_t(rows), C.c_size_t(cols), _p(scale), _p(out))
    return out


# ---- banks ------------------------------------------------------------------
@dataclass
class HostBanks:
    """Slot-major byte banks (src/domain/expert_kernel.rs:429-441)."""
    gu_packed: np.ndarray
    gu_scale: np.ndarray
    gu_global: np.ndarray
    dn_packed: np.ndarray
    dn_scale: np.ndarray
    dn_global: np.ndarray
    slots: int
    gu_rows: int
    gu_cols: int
    dn_rows: int
    dn_cols: int

    def __post_init__(self):
        for n in ("gu_packed", "gu_scale", "gu_global", "dn_packed", "dn_scale", "dn_global"):
            setattr(self, n, np.ascontiguousarray(getattr(self, n)).view(np.uint8).reshape(-1))

    def c(self) -> _Banks:
        b = _Banks()
        for n in ("gu_packed", "gu_scale", "gu_global", "dn_packed", "dn_scale", "dn_global"):
            a = getattr(self, n)
            setattr(b, n, a.ctypes.data)
            setattr(b, n + "_len", a.size)
        b.slots, b.gu_rows, b.gu_cols = self.slots, self.gu_rows, self.gu_cols
        b.dn_rows, b.dn_cols = self.dn_rows, self.dn_cols
        return b

    def fields(self, slot: int):
        """The six byte fields of one slot, in bank order."""
        out = []
        for n in ("gu_packed", "gu_scale", "gu_global", "dn_packed", "dn_scale", "dn_global"):
            a = getattr(self, n)
            per = a.size // self.slots
            out.append(a[slot * per:(slot + 1) * per])
        return out


def gemv_rows(x, packed, scale, glob, rows: int, cols: int) -> np.ndarray:
    x, packed, scale = _c(x, np.float32), _c(packed, np.uint8), _c(scale, np.uint8)
    glob = _c(glob, np.uint8)
    y = np.empty(rows, np.float32)
    lib().ftmo_gemv_rows(_p(x), _p(packed), _p(scale), _p(glob), C.c_size_t(glob.size),
                         C.c_size_t(rows), C.c_size_t(cols), _p(y))
    return y


def tower_nvfp4_gemv(x, packed, scale, glob, rows: int, cols: int) -> np.ndarray:
    x, packed, scale = _c(x, np.float32), _c(packed, np.uint8), _c(scale, np.uint8)
    glob = _c(glob, np.uint8)
    y = np.empty(rows, np.float32)
    lib().ftmo_tower_nvfp4_gemv(_p(x), _p(packed), _p(scale), _p(glob), C.c_size_t(glob.size),
                                C.c_size_t(rows), C.c_size_t(cols), _p(y))
    return y


def grouped_moe_reference(banks: HostBanks, hidden: int, inter: int, x, top_k: int, routes,
                          weights, out: np.ndarray | None = None, want_abs_sum: bool = False):
    """`grouped_moe_reference(_abs_sum)`; raises OracleError like the Rust Result."""
    x = _c(x, np.float32).reshape(-1)
    routes = _c(routes, np.int32).reshape(-1)
    weights = _c(weights, np.float32).reshape(-1)
    tokens = x.size // hidden if hidden else 0
    if out is None:
        out = np.zeros(tokens * hidden, np.float32)
    abs_sum = np.zeros(tokens * hidden, np.float32) if want_abs_sum else None
    cb = banks.c()
    bad = C.c_size_t(0)
    rc = lib().ftmo_grouped_moe_reference(
        C.byref(cb), C.c_size_t(hidden), C.c_size_t(inter), _p(x), C.c_size_t(x.size),
        C.c_size_t(top_k), _p(routes), C.c_size_t(routes.size), _p(weights),
        C.c_size_t(weights.size), _p(out), C.c_size_t(out.size),
        _p(abs_sum) if abs_sum is not None else None,
        C.c_size_t(abs_sum.size if abs_sum is not None else 0), C.byref(bad))
    if rc == SLOT_OUT_OF_RANGE:
        raise OracleError("SlotOutOfRange", f"moe: slot {bad.value} out of range (capacity {banks.slots})",
                          slot=bad.value, capacity=banks.slots)
    if rc != OK:
        raise OracleError("Bad", "moe: bad request or bank shapes")
    out2 = out.reshape(tokens, hidden) if tokens else out
    if want_abs_sum:
        return out2, abs_sum.reshape(tokens, hidden)
    return out2


def grouped_moe_reference_mt(banks: HostBanks, hidden: int, inter: int, x, top_k: int, routes,
                             weights, threads: int | None = None) -> np.ndarray:
    x = _c(x, np.float32).reshape(-1, hidden)
    routes = _c(routes, np.int32).reshape(-1)
    weights = _c(weights, np.float32).reshape(-1)
    out = np.zeros_like(x)
    cb = banks.c()
    rc = lib().ftmo_grouped_moe_reference_mt(
        C.byref(cb), C.c_size_t(hidden), C.c_size_t(inter), _p(x), C.c_size_t(x.shape[0]),
        C.c_size_t(top_k), _p(routes), _p(weights), _p(out), C.c_int(threads or max_threads()))
    if rc != OK:
        raise OracleError("Bad" if rc == BAD else "SlotOutOfRange", "moe: bad request")
    return out


def route_lists(routes, tokens: int, top_k: int):
    routes = _c(routes, np.int32).reshape(-1)
    tok = np.empty(routes.size, np.int32)
    slot = np.empty(routes.size, np.int32)
    rc = lib().ftmo_route_lists(_p(routes), C.c_size_t(routes.size), C.c_size_t(tokens),
                                C.c_size_t(top_k), _p(tok), _p(slot))
    if rc != OK:
        raise OracleError("Bad", f"routes {routes.size} for {tokens} tokens x top_k {top_k}")
    return tok, slot


def build_grouped_csr(route_slot, slots: int):
    route_slot = _c(route_slot, np.int32).reshape(-1)
    seg = np.zeros(slots + 1, np.int32)
    idx = np.zeros(route_slot.size, np.int32)
    why = C.c_int(0)
    rc = lib().ftmo_build_grouped_csr(_p(route_slot), C.c_size_t(route_slot.size),
                                      C.c_size_t(slots), _p(seg), _p(idx), C.byref(why))
    if rc != OK:
        raise OracleError("Bad", "prefill grouped CSR: a route is not resident" if why.value == 1
                          else f"prefill grouped CSR: a route names a slot past the {slots}-slot bank")
    return seg, idx


# ---- router / shared expert / whole block -----------------------------------
def bf16_gemm(x, w_bits, t: int, rows: int, cols: int) -> np.ndarray:
    x, w_bits = _c(x, np.float32), _c(w_bits, np.uint16)
    y = np.empty((t, rows), np.float32)
    lib().ftmo_bf16_gemm(_p(x), _p(w_bits), C.c_size_t(t), C.c_size_t(rows), C.c_size_t(cols), _p(y))
    return y


def softmax_rows(logits: np.ndarray) -> np.ndarray:
    p = _c(logits, np.float32).copy()
    n, e = p.shape
    lib().ftmo_softmax_rows(_p(p), C.c_size_t(n), C.c_size_t(e))
    return p


def topk_renorm(p: np.ndarray, k: int):
    p = _c(p, np.float32)
    n, e = p.shape
    ids = np.empty((n, k), np.int32)
    w = np.empty((n, k), np.float32)
    lib().ftmo_topk_renorm(_p(p), C.c_size_t(n), C.c_size_t(e), C.c_size_t(k), _p(ids), _p(w))
    return ids, w


@dataclass
class Layer:
    """One MoE layer on the host: router, shared expert (bf16 bit patterns) and banks."""
    hidden: int
    inter: int
    experts: int
    top_k: int
    shared_inter: int
    gate_w: np.ndarray       # [experts, hidden] uint16 (bf16 bits)
    sh_gate_up: np.ndarray   # [2*shared_inter, hidden] uint16
    sh_down: np.ndarray      # [hidden, shared_inter] uint16
    sh_gate: np.ndarray      # [1, hidden] uint16
    banks: HostBanks

    def c(self) -> _Layer:
        for n in ("gate_w", "sh_gate_up", "sh_down", "sh_gate"):
            setattr(self, n, _c(getattr(self, n), np.uint16))
        L = _Layer()
        L.hidden, L.inter, L.experts = self.hidden, self.inter, self.experts
        L.top_k, L.shared_inter = self.top_k, self.shared_inter
        L.gate_w, L.sh_gate_up = self.gate_w.ctypes.data, self.sh_gate_up.ctypes.data
        L.sh_down, L.sh_gate = self.sh_down.ctypes.data, self.sh_gate.ctypes.data
        L.banks = self.banks.c()
        return L


def router(layer: Layer, x, want_probs: bool = False):
    x = _c(x, np.float32).reshape(-1, layer.hidden)
    t = x.shape[0]
    ids = np.empty((t, layer.top_k), np.int32)
    w = np.empty((t, layer.top_k), np.float32)
    probs = np.empty((t, layer.experts), np.float32) if want_probs else None
    cl = layer.c()
    lib().ftmo_router(C.byref(cl), _p(x), C.c_size_t(t), _p(ids), _p(w),
                      _p(probs) if probs is not None else None)
    return (ids, w, probs) if want_probs else (ids, w)


def shared_expert(layer: Layer, x) -> np.ndarray:
    x = _c(x, np.float32).reshape(-1, layer.hidden)
    out = np.empty_like(x)
    cl = layer.c()
    lib().ftmo_shared_expert(C.byref(cl), _p(x), C.c_size_t(x.shape[0]), _p(out))
    return out


def moe_block(layer: Layer, x, threads: int = 1, form: str = "gemv"):
    """The whole block (router, shared expert, routed experts, combine).

    form="gemv" follows the scalar tower; form="dequant_once" is the reference's
    inline prefill fallback (same sums, weights widened once per expert).
    Returns (out [T,H] f32, ids [T,k] i32, weights [T,k] f32)."""
    x = _c(x, np.float32).reshape(-1, layer.hidden)
    t = x.shape[0]
    out = np.empty_like(x)
    ids = np.empty((t, layer.top_k), np.int32)
    w = np.empty((t, layer.top_k), np.float32)
    cl = layer.c()
    if form == "dequant_once":
        rc = lib().ftmo_moe_block_dequant_once_mt(C.byref(cl), _p(x), C.c_size_t(t), _p(out),
                                                  C.c_int(threads))
        ids2, w2 = router(layer, x)
        ids[:], w[:] = ids2, w2
    elif threads == 1:
        rc = lib().ftmo_moe_block(C.byref(cl), _p(x), C.c_size_t(t), _p(out), _p(ids), _p(w))
    else:
        rc = lib().ftmo_moe_block_mt(C.byref(cl), _p(x), C.c_size_t(t), _p(out), _p(ids), _p(w),
                                     C.c_int(threads))
    if rc != OK:
        raise OracleError("Bad", "moe_block: bad layer shapes")
    return out, ids, w


# ---- stage dump ------------------------------------------------------------------
def trace_vec(stage: str, layer: int, v) -> None:
    """`trace_vec` of forward.rs:833-855: with FT_TRACE=1, one line per stage on stderr with the l2 norm and the
    largest magnitude of the stage's values.  The CUDA path prints the same lines."""
    if os.environ.get("FT_TRACE") != "1":
        return
    a = np.asarray(v, dtype=np.float64).reshape(-1)
    l2 = float(np.sqrt(np.sum(a * a)))
    amax = float(np.abs(a).max()) if a.size else 0.0
    print(f"TRACE {layer} {stage} l2={l2:.6f} amax={amax:.6f}", file=sys.stderr)


def moe_block_prenorm(layer: Layer, layer_index: int, attn_bits, residual_bits, norm_w_bits, eps: float, threads: int = 1):
    """forward.rs:942-954 around the block: sum2 = attn + residual, h2 = rms_norm(sum2), moe = block(h2); the three
    stages are dumped under FT_TRACE=1.  Returns (sum2 bits, h2 bits, out f32, ids, weights)."""
    s, h2 = add_rmsnorm(attn_bits, residual_bits, norm_w_bits, eps)
    out, ids, w = moe_block(layer, bf16_bits_to_f32(h2), threads=threads)
    trace_vec("sum2", layer_index, bf16_bits_to_f32(s))
    trace_vec("h2", layer_index, bf16_bits_to_f32(h2))
    trace_vec("moe", layer_index, out)
    return s, h2, out, ids, w


# ---- the steps either side of the block ---------------------------------------
def add_rmsnorm(x_bits, r_bits, w_bits, eps: float):
    """Fused residual add + RMSNorm on bf16 bit patterns: returns (sum_out, out) as bf16 bit patterns."""
    x, r, w = _c(x_bits, np.uint16), _c(r_bits, np.uint16), _c(w_bits, np.uint16).reshape(-1)
    rows, hidden = x.shape
    s = np.empty_like(x)
    y = np.empty_like(x)
    lib().ftmo_add_rmsnorm(_p(x), _p(r), _p(w), C.c_float(eps), C.c_size_t(rows), C.c_size_t(hidden), _p(s), _p(y))
    return s, y


def rms_norm(x, w, eps: float) -> np.ndarray:
    """The host tower's f32 rms_norm (forward.rs:48-61)."""
    x, w = _c(x, np.float32), _c(w, np.float32).reshape(-1)
    out = np.empty_like(x)
    lib().ftmo_rms_norm(_p(x), _p(w), C.c_float(eps), C.c_size_t(x.shape[0]), C.c_size_t(x.shape[1]), _p(out))
    return out


def nvfp4_dense_gemv(a, packed_kmajor, scale_kmajor, glob, threads: int | None = None) -> np.ndarray:
    """nvfp4_dense_gemv_reference on the K-major bank: packed [K/8, N] int32, scale [K/16, N] u8, global [N] f16."""
    a = _c(a, np.float32)
    packed = _c(packed_kmajor, np.uint32)
    scale = _c(scale_kmajor, np.uint8)
    g = _c(glob, np.uint16).reshape(-1)
    m, k = a.shape
    n = packed.shape[1]
    assert packed.shape == (k // 8, n) and scale.shape == (k // 16, n) and g.size == n
    c = np.empty((m, n), np.float32)
    lib().ftmo_nvfp4_dense_gemv(_p(a), _p(packed), _p(scale), _p(g), C.c_size_t(m), C.c_size_t(n), C.c_size_t(k), _p(c),
                                C.c_int(threads or max_threads()))
    return c


# ---- expert-slot LRU --------------------------------------------------------
class ExpertCache:
    """src/domain/expert_cache.rs:8-134"""

    def __init__(self, num_layers: int, num_experts: int, cache_size: int):
        self._h = lib().ftmo_cache_new(num_layers, num_experts, cache_size)
        if not self._h:
            raise OracleError("Bad", "cache needs layers*experts > 0 and cache_size > 0")
        self.num_layers, self.num_experts, self.cache_size = num_layers, num_experts, cache_size

    def __del__(self):
        if getattr(self, "_h", None):
            lib().ftmo_cache_free(self._h)
            self._h = None

    def slot_of(self, layer: int, expert: int) -> int:
        return int(lib().ftmo_cache_slot_of(self._h, layer, expert))

    def id_of_slot(self, slot: int) -> int:
        return int(lib().ftmo_cache_id_of_slot(self._h, slot))

    def ensure_experts(self, layer: int, routed):
        routed = _c(routed, np.uint32).reshape(-1)
        n = routed.size
        misses = np.zeros(max(n, 1), np.uint32)
        slots = np.zeros(max(n, 1), np.uint32)
        rewrites = np.zeros(max(n, 1), np.int32)
        m = lib().ftmo_cache_ensure(self._h, C.c_size_t(layer), _p(routed), C.c_size_t(n),
                                    _p(misses), _p(slots), _p(rewrites))
        return misses[:m].tolist(), slots[:m].tolist(), rewrites[:n].tolist()
