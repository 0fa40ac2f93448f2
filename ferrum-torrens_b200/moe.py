"""Host-side mirror of the reference's MoE ports over the C ABI of libftmoe.so.

The names, argument meanings and error behaviour follow the reference's traits so that code
written against them reads the same:

* `ExpertSlotStore` + `ExpertGemm`  -> `B200MoE`     (src/domain/expert_kernel.rs:140-161, :246-294;
                                                      adapter src/infrastructure/cuda_moe.rs:145-195)
* `MoEExecutor`                     -> `CachedExperts` (src/domain/expert_kernel.rs:372-424;
                                                      src/application/run_experts.rs:103-189)
* `ExpertCache`, `route_lists`, `run_experts`, `MoEGroup`, `MoEDeviceRequest`, `MoEError`

Device buffers are torch CUDA tensors (torch is only the allocator and stream provider); every
computation goes through the library, which has no CPU path.
"""
from __future__ import annotations

import ctypes as C
import os
import sys
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

from . import _lib as L

# bank order: gate_up then down, packed / scale / global within each (expert_kernel.rs:62-80)
BANKS = ("GateUpPacked", "GateUpScale", "GateUpGlobal", "DownPacked", "DownScale", "DownGlobal")


class MoEError(Exception):
    """MoEError (src/domain/expert_kernel.rs:21-39).  `kind` is the variant name."""

    KINDS = {L.ERR_BAD: "Bad", L.ERR_SLOT_OUT_OF_RANGE: "SlotOutOfRange", L.ERR_MISSING: "Missing",
             L.ERR_OUT_OF_MEMORY: "OutOfMemory", L.ERR_READ: "Read", L.ERR_NOT_SUPPORTED: "NotSupported",
             L.ERR_CUDA: "Bad"}

    def __init__(self, code: int, msg: str):
        super().__init__(msg)
        self.code = code
        self.kind = self.KINDS.get(code, "Bad")

    @property
    def retryable(self) -> bool:
        """Out of device memory is answered with a retryable 503 (expert_kernel.rs:17-19, :30-34)."""
        return self.kind == "OutOfMemory"


def bad(msg: str) -> MoEError:
    return MoEError(L.ERR_BAD, "moe: " + msg)


@dataclass(frozen=True)
class ExpertShapes:
    """ExpertShapes (expert_kernel.rs:179-219): gate_up [2*inter, hidden], down [hidden, inter]."""
    hidden: int
    inter: int

    def __post_init__(self):
        if self.hidden <= 0 or self.inter <= 0 or self.hidden % 16 or self.inter % 16:
            raise bad(f"expert shapes hidden {self.hidden} inter {self.inter} must be nonzero multiples of 16")

    def gate_up_rows(self) -> int:
        return 2 * self.inter

    def slab_shape(self, part: str):
        return (2 * self.inter, self.hidden) if part == "GateUp" else (self.hidden, self.inter)

    def bank_row_bytes(self, bank: str) -> int:
        rows, cols = self.slab_shape("GateUp" if bank.startswith("GateUp") else "Down")
        if bank.endswith("Packed"):
            return rows * cols // 2
        if bank.endswith("Scale"):
            return rows * cols // 16
        return rows * 2


def route_lists(routes: Sequence[int], tokens: int, top_k: int):
    """route_lists (expert_kernel.rs:223-243): flatten dense [tokens, top_k] slot ids."""
    routes = np.asarray(routes, np.int32).reshape(-1)
    if tokens == 0 or top_k == 0 or routes.size != tokens * top_k:
        raise bad(f"routes {routes.size} for {tokens} tokens x top_k {top_k}")
    return np.repeat(np.arange(tokens, dtype=np.int32), top_k), routes.copy()


@dataclass
class MoEGroup:
    """MoEGroup (expert_kernel.rs:167-174): host hand-off, routes are slot ids (-1 = skip)."""
    hidden: int
    inter: int
    x: np.ndarray
    top_k: int
    routes: np.ndarray
    weights: np.ndarray


@dataclass
class MoEDeviceRequest:
    """MoEDeviceRequest (expert_kernel.rs:332-340): everything on the device; `experts` are the
    router's dense ids [tokens, top_k]."""
    layer: int
    hidden: int
    inter: int
    top_k: int
    x: "torch.Tensor"
    experts: "torch.Tensor"
    weights: "torch.Tensor"


def _torch():
    import torch
    return torch


def _dtype_code(t) -> int:
    torch = _torch()
    table = {torch.bfloat16: L.BF16, torch.float32: L.F32, torch.int32: L.I32, torch.int64: L.I64}
    if t.dtype not in table:
        raise bad(f"tensor cannot be {t.dtype}")
    return table[t.dtype]


def _dev(t, what: str):
    if not t.is_cuda:
        raise bad(f"{what} must be a device tensor")
    if not t.is_contiguous():
        raise bad(f"{what} must be contiguous")
    return C.c_void_p(t.data_ptr())


def _stream_ptr(stream) -> C.c_void_p:
    if stream is None:
        return C.c_void_p(_torch().cuda.current_stream().cuda_stream)
    if isinstance(stream, int):
        return C.c_void_p(stream)
    return C.c_void_p(stream.cuda_stream)


def trace_on() -> bool:
    """FT_TRACE=1 switches the stage dump on (read at every call, so a test can set it)."""
    return os.environ.get("FT_TRACE") == "1"


def trace(stage: str, layer: int, t) -> None:
    """One line of the stage dump, in the reference's format (forward.rs:833-855, `trace_vec`): the l2 norm and the
    largest magnitude of a stage's tensor, on stderr.  The CPU path prints the same lines (oracle.trace_vec), so
    two runs can be compared stage by stage and the first divergence located.  Synchronises the device."""
    if not trace_on():
        return
    torch = _torch()
    v = t.detach().to(torch.float64)
    l2 = float(v.pow(2).sum().sqrt())
    amax = float(v.abs().max()) if v.numel() else 0.0
    print(f"TRACE {layer} {stage} l2={l2:.6f} amax={amax:.6f}", file=sys.stderr)


class _RawDeviceArray:
    """A borrowed device range exposed through __cuda_array_interface__ (no ownership)."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self._owner = owner
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class B200MoE:
    """The device adapter: `ExpertSlotStore` + `ExpertGemm` over the C ABI (CudaMoE).

    `source`, when given, is an ExpertSlabSource: an object with `slab(layer, expert, part)`
    returning `(packed, scale, global)` uint8 arrays (expert_kernel.rs:121-131); `load` reads
    through it like the reference adapter does (cuda_moe.rs:552-576).
    """

    def __init__(self, device: int, shapes: ExpertShapes, slots: int, *, source=None, experts: int = 256,
                 layers: int = 1, top_k: int = 8, shared_inter: int = 512, max_tokens: int = 2048, ep_rank: int = 0,
                 ep_size: int = 1, stream=None):
        self._h = C.c_void_p()
        self._lib = L.lib()
        self.shapes, self.source = shapes, source
        self.experts, self.layers, self.top_k = experts, layers, top_k
        self.shared_inter, self.max_tokens = shared_inter, max_tokens
        self.device = device
        cfg = L.Config(device, shapes.hidden, shapes.inter, top_k, experts, layers, slots, shared_inter, max_tokens,
                       ep_rank, ep_size)
        sp = _stream_ptr(stream) if stream is not None else C.c_void_p(0)
        h = C.c_void_p()
        rc = self._lib.ftm_create(C.byref(cfg), sp, C.byref(h))
        if rc != L.OK:
            raise MoEError(rc, (self._lib.ftm_last_error(None) or b"").decode())
        self._h = h

    # -- plumbing ---------------------------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None):
            self._lib.ftm_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != L.OK:
            raise MoEError(rc, (self._lib.ftm_last_error(self._h) or b"").decode())

    # -- ExpertSlotStore --------------------------------------------------------------------
    def load(self, layer: int, expert: int, slot: int, fields=None):
        """load(layer, expert, slot): stage one expert's six byte fields into `slot`.

        `fields` (six uint8 arrays in bank order, numpy or CUDA tensors) overrides the source."""
        if fields is None:
            if self.source is None:
                raise MoEError(L.ERR_MISSING, f"moe: no expert bank entry L{layer:05d}")
            gu = self.source.slab(layer, expert, "GateUp")
            dn = self.source.slab(layer, expert, "Down")
            fields = [*gu, *dn]
        if len(fields) != L.NUM_BANKS:
            raise bad(f"{len(fields)} expert fields, expected {L.NUM_BANKS}")
        ptrs = (C.c_void_p * L.NUM_BANKS)()
        lens = (C.c_size_t * L.NUM_BANKS)()
        on_device = hasattr(fields[0], "is_cuda") and fields[0].is_cuda
        keep = []
        for b, f in enumerate(fields):
            if on_device:
                keep.append(f)
                ptrs[b], lens[b] = f.data_ptr(), f.numel() * f.element_size()
            else:
                a = np.ascontiguousarray(f).view(np.uint8).reshape(-1)
                keep.append(a)
                ptrs[b], lens[b] = a.ctypes.data, a.size
        fn = self._lib.ftm_load_expert_dev if on_device else self._lib.ftm_load_expert
        self._check(fn(self._h, layer, expert, slot, ptrs, lens))

    def slots(self) -> int:
        return int(self._lib.ftm_slots(self._h))

    def release_banks(self):
        self._check(self._lib.ftm_release_banks(self._h))

    def rehydrate_banks(self):
        self._check(self._lib.ftm_rehydrate_banks(self._h))

    def banks_resident(self) -> bool:
        return bool(self._lib.ftm_banks_resident(self._h))

    def bank_ptrs(self) -> list[int]:
        out = (C.c_uint64 * L.NUM_BANKS)()
        self._check(self._lib.ftm_bank_ptrs(self._h, out))
        return [int(v) for v in out]

    def bank_row_bytes(self, bank: int) -> int:
        return int(self._lib.ftm_bank_row_bytes(self._h, bank))

    def bank_tensors(self):
        """The six banks as uint8 CUDA tensors [slots, row_bytes] aliasing the adapter's memory."""
        torch = _torch()
        out = []
        for b, ptr in enumerate(self.bank_ptrs()):
            rb = self.bank_row_bytes(b)
            raw = _RawDeviceArray(ptr, rb * self.slots(), self)
            out.append(torch.as_tensor(raw, device=f"cuda:{self.device}").view(self.slots(), rb))
        return out

    def adopt(self, layer: int, expert: int, slot: int):
        """Marks (layer, expert) resident in `slot` whose bytes were written through bank_tensors()."""
        ptrs = (C.c_void_p * L.NUM_BANKS)()
        lens = (C.c_size_t * L.NUM_BANKS)()
        for b, base in enumerate(self.bank_ptrs()):
            rb = self.bank_row_bytes(b)
            ptrs[b], lens[b] = base + slot * rb, rb
        self._check(self._lib.ftm_load_expert_dev(self._h, layer, expert, slot, ptrs, lens))

    def slot_of(self, layer: int, expert: int) -> int:
        return int(self._lib.ftm_slot_of(self._h, layer, expert))

    # -- ExpertGemm -------------------------------------------------------------------------
    def grouped_moe(self, req: MoEGroup, out: np.ndarray):
        """grouped_moe(&MoEGroup, &mut [f32]): host hand-off, synchronous."""
        if req.hidden != self.shapes.hidden or req.inter != self.shapes.inter:
            raise bad(f"the adapter is built for hidden {self.shapes.hidden} inter {self.shapes.inter}, "
                      f"not {req.hidden}x{req.inter}")
        x = np.ascontiguousarray(req.x, np.float32).reshape(-1)
        routes = np.ascontiguousarray(req.routes, np.int32).reshape(-1)
        weights = np.ascontiguousarray(req.weights, np.float32).reshape(-1)
        if out.dtype != np.float32 or not out.flags.c_contiguous:
            raise bad("out must be contiguous f32")
        p = lambda a: C.c_void_p(a.ctypes.data)
        self._check(self._lib.ftm_grouped_moe_host(self._h, p(x), x.size, req.top_k, p(routes), routes.size,
                                                   p(weights), weights.size, p(out), out.size))

    def grouped_moe_dev(self, hidden: int, inter: int, top_k: int, x, routes, weights, out, stream=None):
        """grouped_moe_dev(&MoEDeviceGroup, out): x / weights / out on the device, routes on the host."""
        if hidden != self.shapes.hidden or inter != self.shapes.inter:
            raise bad(f"the adapter is built for hidden {self.shapes.hidden} inter {self.shapes.inter}")
        if x.numel() == 0 or x.numel() % hidden:
            raise bad(f"grouped_moe: {x.numel()} activations for hidden {hidden}")
        tokens = x.numel() // hidden
        routes = np.ascontiguousarray(routes, np.int32).reshape(-1)
        if weights.numel() < tokens * top_k:
            raise bad(f"grouped_moe: {routes.size} routes and {weights.numel()} weights for {tokens} tokens x top_k {top_k}")
        if out.numel() != tokens * hidden:
            raise bad(f"out holds {out.numel()}, the step produces {tokens * hidden}")
        if weights.dtype != _torch().float32:
            raise bad("route weights must be f32")
        self._check(self._lib.ftm_grouped_moe_dev(self._h, _dev(x, "the activations"), _dtype_code(x), tokens, top_k,
                                                  C.c_void_p(routes.ctypes.data), routes.size,
                                                  _dev(weights, "the weights"), _dev(out, "the output"),
                                                  _dtype_code(out), _stream_ptr(stream)))

    def grouped_moe_staged(self, req: MoEDeviceRequest, out, *, path: int = L.PATH_AUTO, stream=None):
        """grouped_moe_staged(&MoEDeviceRequest, out): the serving call, asynchronous."""
        tokens = _check_device_step(req)
        if req.hidden != self.shapes.hidden or req.inter != self.shapes.inter:
            raise bad(f"the adapter is built for hidden {self.shapes.hidden} inter {self.shapes.inter}")
        if out.numel() != tokens * req.hidden:
            raise bad(f"out holds {out.numel()}, the step produces {tokens * req.hidden}")
        if req.weights.dtype != _torch().float32:
            raise bad("route weights must be f32")
        if req.top_k != self.top_k:
            raise bad(f"the adapter was built for top_k {self.top_k}, got {req.top_k}")
        self._check(self._lib.ftm_moe_layer_staged(
            self._h, req.layer, _dev(req.x, "the activations"), _dtype_code(req.x), _dev(req.experts, "the expert ids"),
            _dtype_code(req.experts), _dev(req.weights, "the weights"), tokens, _dev(out, "the output"),
            _dtype_code(out), path, _stream_ptr(stream)))

    def begin_staged(self, req: MoEDeviceRequest, stream=None):
        """begin_staged: `None` means "no overlapped path, call grouped_moe_staged" (expert_kernel.rs:275-281)."""
        tokens = _check_device_step(req)
        rc = self._lib.ftm_moe_begin(self._h, req.layer, _dev(req.x, "x"), _dtype_code(req.x), _dev(req.experts, "ids"),
                                     _dtype_code(req.experts), _dev(req.weights, "w"), tokens, _stream_ptr(stream))
        if rc == L.ERR_NOT_SUPPORTED:
            return None
        self._check(rc)
        return None

    def staged_route_cap(self) -> int:
        return int(self._lib.ftm_route_cap(self._h))

    def reset_staging(self):
        self._check(self._lib.ftm_reset_staging(self._h))

    def steps(self) -> int:
        return int(self._lib.ftm_steps(self._h))

    def sync_status(self, stream=None):
        """Waits for the stream; raises if an asynchronous step saw a bad expert id or gave up a wait."""
        self._check(self._lib.ftm_sync_status(self._h, _stream_ptr(stream)))

    def kernel_launches(self) -> int:
        return int(self._lib.ftm_kernel_launches(self._h))

    def set_sm_budget(self, sms: int):
        """SMs the persistent expert kernels may occupy (0 = all): leaves room for exchange kernels."""
        self._check(self._lib.ftm_set_sm_budget(self._h, int(sms)))

    def profile(self, on: bool):
        """Per-kernel CUDA-event timing (FT_PROFILE, src/infrastructure/profile.rs:1-14)."""
        self._check(self._lib.ftm_profile_enable(self._h, 1 if on else 0))

    def profile_read(self) -> dict:
        """{kernel kind: (total_ms, launches)} since profiling was enabled."""
        out, k = {}, 0
        while True:
            name = self._lib.ftm_profile_kind_name(k)
            if not name:
                return out
            ms, n = C.c_double(0), C.c_uint64(0)
            self._check(self._lib.ftm_profile_read(self._h, k, C.byref(ms), C.byref(n)))
            if n.value:
                out[name.decode()] = (ms.value, int(n.value))
            k += 1

    # -- router, permutation, shared expert, combine, whole block ----------------------------
    def router(self, x, gate_w, stream=None):
        """Gate projection + fused_topk_softmax: returns (ids [T,k] i32, weights [T,k] f32)."""
        torch = _torch()
        tokens = x.numel() // self.shapes.hidden
        ids = torch.empty((tokens, self.top_k), dtype=torch.int32, device=x.device)
        w = torch.empty((tokens, self.top_k), dtype=torch.float32, device=x.device)
        if x.dtype != torch.bfloat16 or gate_w.dtype != torch.bfloat16:
            raise bad("router activations and gate weight must be bf16")
        if gate_w.numel() != self.experts * self.shapes.hidden:
            raise bad(f"gate weight holds {gate_w.numel()}, expected {self.experts}x{self.shapes.hidden}")
        self._check(self._lib.ftm_router(self._h, _dev(x, "x"), _dev(gate_w, "gate"), tokens, _dev(ids, "ids"),
                                         _dev(w, "w"), _stream_ptr(stream)))
        return ids, w

    def fused_topk_softmax(self, logits, stream=None):
        """Tensor::fused_topk_softmax(k) on f32 logits [T, experts] (cudarc.rs:1147-1171)."""
        torch = _torch()
        if logits.dtype != torch.float32 or logits.shape[-1] != self.experts:
            raise bad(f"logits must be f32 [T, {self.experts}]")
        tokens = logits.numel() // self.experts
        ids = torch.empty((tokens, self.top_k), dtype=torch.int32, device=logits.device)
        w = torch.empty((tokens, self.top_k), dtype=torch.float32, device=logits.device)
        self._check(self._lib.ftm_router_from_logits(self._h, _dev(logits, "logits"), tokens, _dev(ids, "ids"),
                                                     _dev(w, "w"), _stream_ptr(stream)))
        return ids, w

    def csr_build(self, route_slot, bins: int, stream=None):
        """csr_build: (seg [bins+1], route_idx [R], bad flag) (cuda_moe.rs:1198-1253)."""
        torch = _torch()
        if route_slot.dtype != torch.int32:
            raise bad("route slots must be i32")
        r = route_slot.numel()
        seg = torch.zeros(bins + 1, dtype=torch.int32, device=route_slot.device)
        idx = torch.full((r,), -1, dtype=torch.int32, device=route_slot.device)
        self._check(self._lib.ftm_csr_build(self._h, _dev(route_slot, "route_slot"), r, bins, _dev(seg, "seg"),
                                            _dev(idx, "idx"), _stream_ptr(stream)))
        flag = C.c_int32(0)
        self._check(self._lib.ftm_csr_bad(self._h, _stream_ptr(stream), C.byref(flag)))
        return seg, idx, int(flag.value)

    def shared_expert(self, x, gate_up, down, shared_gate, stream=None):
        """Returns (shared [T,H] f32 ungated, se_gate [T] f32)."""
        torch = _torch()
        tokens = x.numel() // self.shapes.hidden
        shared = torch.empty((tokens, self.shapes.hidden), dtype=torch.float32, device=x.device)
        gate = torch.empty((tokens,), dtype=torch.float32, device=x.device)
        for t, n in ((x, "x"), (gate_up, "gate_up"), (down, "down"), (shared_gate, "shared_gate")):
            if t.dtype != torch.bfloat16:
                raise bad(f"shared expert {n} must be bf16")
        self._check(self._lib.ftm_shared_expert(self._h, _dev(x, "x"), tokens, _dev(gate_up, "gate_up"),
                                                _dev(down, "down"), _dev(shared_gate, "shared_gate"),
                                                _dev(shared, "shared"), _dev(gate, "gate"), _stream_ptr(stream)))
        return shared, gate

    def combine(self, routed, shared, se_gate, out, stream=None):
        tokens = routed.numel() // self.shapes.hidden
        self._check(self._lib.ftm_combine(self._h, _dev(routed, "routed"), _dtype_code(routed), _dev(shared, "shared"),
                                          _dev(se_gate, "se_gate"), tokens, _dev(out, "out"), _dtype_code(out),
                                          _stream_ptr(stream)))

    def ep_pack(self, x, ids, weights, ep_size: int, stream=None):
        """Sort this rank's routes by owning rank / expert and fill the all-to-all send buffers.
        Returns (send_x [R,H] bf16, send_expert [R] i32, send_weight [R] f32, route_idx [R] i32, counts [n] i32)."""
        torch = _torch()
        tokens = x.numel() // self.shapes.hidden
        r = tokens * self.top_k
        dev = x.device
        send_x = torch.empty((r, self.shapes.hidden), dtype=torch.bfloat16, device=dev)
        send_e = torch.empty((r,), dtype=torch.int32, device=dev)
        send_w = torch.empty((r,), dtype=torch.float32, device=dev)
        route_idx = torch.empty((r,), dtype=torch.int32, device=dev)
        counts = torch.empty((ep_size,), dtype=torch.int32, device=dev)
        if x.dtype != torch.bfloat16 or ids.dtype != torch.int32 or weights.dtype != torch.float32:
            raise bad("ep_pack takes bf16 activations, i32 ids and f32 weights")
        self._check(self._lib.ftm_ep_pack(self._h, _dev(x, "x"), _dev(ids, "ids"), _dev(weights, "weights"), tokens,
                                          ep_size, _dev(send_x, "send_x"), _dev(send_e, "send_e"), _dev(send_w, "send_w"),
                                          _dev(route_idx, "route_idx"), _dev(counts, "counts"), _stream_ptr(stream)))
        return send_x, send_e, send_w, route_idx, counts

    def ep_plan(self, ids, ep_size: int, stream=None):
        """Sort this rank's routes by (owner, expert): returns (route_idx [R] i32, counts [ep_size] i32)."""
        torch = _torch()
        tokens = ids.numel() // self.top_k
        route_idx = torch.empty((ids.numel(),), dtype=torch.int32, device=ids.device)
        counts = torch.empty((ep_size,), dtype=torch.int32, device=ids.device)
        self._check(self._lib.ftm_ep_plan(self._h, _dev(ids, "ids"), tokens, ep_size, _dev(route_idx, "route_idx"),
                                          _dev(counts, "counts"), _stream_ptr(stream)))
        return route_idx, counts

    def ep_dispatch(self, x, ids, weights, route_idx, ep_size: int, ep_rank: int, counts_all, peer_x: int, peer_meta: int,
                    capacity_rows: int, stream=None):
        """Store every route's row, expert id and weight into its owner's receive buffers over peer memory.
        peer_x / peer_meta: device addresses of the arrays of ep_size buffer pointers."""
        tokens = x.numel() // self.shapes.hidden
        self._check(self._lib.ftm_ep_dispatch(self._h, _dev(x, "x"), _dev(ids, "ids"), _dev(weights, "weights"),
                                              _dev(route_idx, "route_idx"), tokens, ep_size, ep_rank,
                                              _dev(counts_all, "counts_all"), C.c_void_p(peer_x), C.c_void_p(peer_meta),
                                              capacity_rows, _stream_ptr(stream)))

    def ep_return(self, y, ep_size: int, ep_rank: int, counts_all, peer_back: int, capacity_rows: int, stream=None):
        """Owner side: store the rows of y (receive order, bf16) into their sources' back buffers."""
        rows = y.numel() // self.shapes.hidden
        self._check(self._lib.ftm_ep_return(self._h, _dev(y, "y"), rows, ep_size, ep_rank, _dev(counts_all, "counts_all"),
                                            C.c_void_p(peer_back), capacity_rows, _stream_ptr(stream)))

    def ep_experts_sorted(self, layer: int, x, expert_ids, weights, stream=None) -> bool:
        """Owner side: the grouped GEMMs on the received rows, results left sorted by expert inside the adapter for
        ep_return_sorted.  False when the step is too small for that path (use grouped_moe_staged + ep_return)."""
        rows = x.numel() // self.shapes.hidden
        rc = self._lib.ftm_ep_experts_sorted(self._h, layer, _dev(x, "x"), _dev(expert_ids, "ids"), _dev(weights, "weights"),
                                             rows, _stream_ptr(stream))
        if rc == L.ERR_NOT_SUPPORTED:
            return False
        self._check(rc)
        return True

    def ep_experts_return(self, layer: int, x, expert_ids, weights, ep_size: int, ep_rank: int, counts_all, peer_back: int,
                          capacity_rows: int, stream=None) -> bool:
        """Owner side: the grouped GEMMs on the received rows, every finished row stored by the down GEMM itself into
        its source's back buffer.  False when the step is too small for that path (use grouped_moe_staged + ep_return)."""
        rows = x.numel() // self.shapes.hidden
        rc = self._lib.ftm_ep_experts_return(self._h, layer, _dev(x, "x"), _dev(expert_ids, "ids"), _dev(weights, "weights"),
                                             rows, ep_size, ep_rank, _dev(counts_all, "counts_all"), C.c_void_p(peer_back),
                                             capacity_rows, _stream_ptr(stream))
        if rc == L.ERR_NOT_SUPPORTED:
            return False
        self._check(rc)
        return True

    def ep_plan_seg(self, ids, stream=None):
        """ep_plan that also returns the prefix of the send order over the layer's experts: (route_idx [T*k],
        seg [experts + 1]), both int32 on the device."""
        torch = _torch()
        tokens = ids.numel() // self.top_k
        route_idx = torch.empty((tokens * self.top_k,), dtype=torch.int32, device=ids.device)
        seg = torch.empty((self.experts + 1,), dtype=torch.int32, device=ids.device)
        self._check(self._lib.ftm_ep_plan_seg(self._h, _dev(ids, "ids"), tokens, _dev(route_idx, "route_idx"), _dev(seg, "seg"),
                                              _stream_ptr(stream)))
        return route_idx, seg

    def ep_dispatch_sorted(self, x, ids, weights, route_idx, ep_size: int, ep_rank: int, seg_all, peer_xg: int, peer_weight: int,
                           peer_row_scale: int, capacity_rows: int, stream=None):
        """Store every route's row (f16, scaled by a power of two), weight and row scale at its place in the owner's
        matrix sorted by expert; seg_all [ep_size, experts + 1] are the all-gathered prefixes of ep_plan_seg."""
        tokens = x.numel() // self.shapes.hidden
        self._check(self._lib.ftm_ep_dispatch_sorted(
            self._h, _dev(x, "x"), _dev(ids, "ids"), _dev(weights, "weights"), _dev(route_idx, "route_idx"), tokens, ep_size,
            ep_rank, _dev(seg_all, "seg_all"), C.c_void_p(peer_xg), C.c_void_p(peer_weight), C.c_void_p(peer_row_scale),
            capacity_rows, _stream_ptr(stream)))

    def ep_experts_presorted(self, layer: int, xg, weights, row_scale, rows: int, ep_size: int, ep_rank: int, seg_all,
                             peer_back: int, back_capacity_rows: int, stream=None):
        """Owner side of ep_dispatch_sorted: both GEMMs on the first `rows` rows of xg [capacity, hidden] f16, every
        finished row stored by the down GEMM into its source's back buffer."""
        self._check(self._lib.ftm_ep_experts_presorted(
            self._h, layer, _dev(xg, "xg"), _dev(weights, "weights"), _dev(row_scale, "row_scale"), rows, xg.shape[0], ep_size,
            ep_rank, _dev(seg_all, "seg_all"), C.c_void_p(peer_back), back_capacity_rows, _stream_ptr(stream)))

    def ep_return_sorted(self, rows: int, ep_size: int, ep_rank: int, counts_all, peer_back: int, capacity_rows: int,
                         stream=None):
        """Owner side: store the rows ep_experts_sorted left in the adapter into their sources' back buffers."""
        self._check(self._lib.ftm_ep_return_sorted(self._h, rows, ep_size, ep_rank, _dev(counts_all, "counts_all"),
                                                   C.c_void_p(peer_back), capacity_rows, _stream_ptr(stream)))

    def ep_combine(self, y, route_idx, shared, se_gate, out, stream=None):
        """out[t] = se_gate[t] * shared[t] + sum_j y[position of route t*k + j] (weights applied by the owner)."""
        tokens = out.numel() // self.shapes.hidden
        null = C.c_void_p(0)
        self._check(self._lib.ftm_ep_combine(self._h, _dev(y, "y"), _dtype_code(y), _dev(route_idx, "route_idx"),
                                             _dev(shared, "shared") if shared is not None else null,
                                             _dev(se_gate, "se_gate") if se_gate is not None else null, tokens,
                                             _dev(out, "out"), _dtype_code(out), _stream_ptr(stream)))

    def moe_block(self, layer: int, x, gate_w, sh_gate_up, sh_down, sh_gate, out, *, ids_out=None, weights_out=None,
                  path: int = L.PATH_AUTO, stream=None):
        """The whole block: router, routed experts, shared expert, combine (moe_parts)."""
        tokens = x.numel() // self.shapes.hidden
        if out.numel() != tokens * self.shapes.hidden:
            raise bad(f"out holds {out.numel()}, the block produces {tokens * self.shapes.hidden}")
        null = C.c_void_p(0)
        self._check(self._lib.ftm_moe_block(
            self._h, layer, _dev(x, "x"), tokens, _dev(gate_w, "gate"), _dev(sh_gate_up, "sh_gate_up"),
            _dev(sh_down, "sh_down"), _dev(sh_gate, "sh_gate"), _dev(out, "out"), _dtype_code(out),
            _dev(ids_out, "ids") if ids_out is not None else null,
            _dev(weights_out, "weights") if weights_out is not None else null, path, _stream_ptr(stream)))
        trace("moe", layer, out)


    # -- the steps either side of the block -----------------------------------------------------
    def add_rmsnorm(self, x, residual, norm_w, eps: float, stream=None):
        """Fused residual add + RMSNorm (norm.py `add_rmsnorm`): returns (sum_out, out), both [T, hidden] bf16."""
        torch = _torch()
        for t, n in ((x, "x"), (residual, "residual"), (norm_w, "norm_w")):
            if t.dtype != torch.bfloat16:
                raise bad(f"add_rmsnorm {n} must be bf16")
        tokens = x.numel() // self.shapes.hidden
        if residual.numel() != x.numel() or norm_w.numel() != self.shapes.hidden:
            raise bad(f"add_rmsnorm: x {x.numel()}, residual {residual.numel()}, norm_w {norm_w.numel()}")
        s, y = torch.empty_like(x), torch.empty_like(x)
        self._check(self._lib.ftm_add_rmsnorm(self._h, _dev(x, "x"), _dev(residual, "residual"), _dev(norm_w, "norm_w"),
                                              C.c_float(eps), tokens, _dev(s, "sum_out"), _dev(y, "out"),
                                              _stream_ptr(stream)))
        return s, y

    def moe_block_prenorm(self, layer: int, attn_out, residual, norm_w, eps: float, gate_w, sh_gate_up, sh_down, sh_gate,
                          sum_out, out, *, h2_out=None, ids_out=None, weights_out=None, path: int = L.PATH_AUTO,
                          stream=None):
        """sum_out = attn_out + residual, h2 = rms_norm(sum_out), out = moe_block(h2) (forward.rs:942-953)."""
        tokens = attn_out.numel() // self.shapes.hidden
        if out.numel() != tokens * self.shapes.hidden or sum_out.numel() != attn_out.numel():
            raise bad(f"out holds {out.numel()}, the block produces {tokens * self.shapes.hidden}")
        null = C.c_void_p(0)
        opt = lambda t, n: _dev(t, n) if t is not None else null
        if trace_on() and h2_out is None:
            h2_out = _torch().empty_like(attn_out)       # the dump wants the normalised rows
        self._check(self._lib.ftm_moe_block_prenorm(
            self._h, layer, _dev(attn_out, "attn_out"), _dev(residual, "residual"), _dev(norm_w, "norm_w"), C.c_float(eps),
            tokens, _dev(gate_w, "gate"), _dev(sh_gate_up, "sh_gate_up"), _dev(sh_down, "sh_down"), _dev(sh_gate, "sh_gate"),
            _dev(sum_out, "sum_out"), opt(h2_out, "h2"), _dev(out, "out"), _dtype_code(out), opt(ids_out, "ids"),
            opt(weights_out, "weights"), path, _stream_ptr(stream)))
        if trace_on():
            trace("sum2", layer, sum_out)
            trace("h2", layer, h2_out)
            trace("moe", layer, out)

    def dense_gemv(self, a, packed_kmajor, scale_kmajor, glob, c=None, stream=None):
        """DenseGemv::gemv (cuda_linear.rs:48-175): c [M, N] f32 = a [M, K] @ dequant(W)^T for the K-major bank
        packed [K/8, N] int32, scale [K/16, N] uint8, global [N] f16 (as int16 / uint8 bytes)."""
        torch = _torch()
        if a.dim() != 2 or packed_kmajor.dim() != 2:
            raise bad("the dense gemv kernel was built for a = [M, K] and packed = [K // 8, N], not the shapes handed in")
        m, k = a.shape
        kw, n = packed_kmajor.shape
        if kw * 8 != k or packed_kmajor.dtype != torch.int32:
            raise bad("the dense gemv kernel was built for packed = [K // 8, N], not the shapes handed in")
        if tuple(scale_kmajor.shape) != (k // 16, n) or scale_kmajor.element_size() != 1:
            raise bad("the dense gemv kernel was built for scale = [K // 16, N], not the shapes handed in")
        if glob.numel() * glob.element_size() != n * 2:
            raise bad("the dense gemv kernel was built for global = [N] f16 (N * 2 bytes), not the shapes handed in")
        if c is None:
            c = torch.empty((m, n), dtype=torch.float32, device=a.device)
        elif tuple(c.shape) != (m, n) or c.dtype != torch.float32:
            raise bad("the dense gemv kernel was built for c = [M, N], not the shapes handed in")
        self._check(self._lib.ftm_dense_gemv(self._h, _dev(a, "a"), _dtype_code(a), _dev(packed_kmajor, "packed"),
                                             _dev(scale_kmajor, "scale"), _dev(glob, "global"), m, n, k, _dev(c, "c"),
                                             _stream_ptr(stream)))
        return c


def _check_device_step(step: MoEDeviceRequest) -> int:
    """check_device_step (src/application/run_experts.rs:251-268): element counts only."""
    hidden, top_k = step.hidden, step.top_k
    x_len, ne, nw = step.x.numel(), step.experts.numel(), step.weights.numel()
    if hidden == 0 or top_k == 0 or x_len == 0 or x_len % hidden:
        raise bad(f"device expert step: hidden {hidden} top_k {top_k} x {x_len}")
    tokens = x_len // hidden
    if ne != tokens * top_k or nw != tokens * top_k:
        raise bad(f"device expert step: {ne} experts and {nw} weights for {tokens} tokens x top_k {top_k}")
    return tokens


class ExpertCache:
    """ExpertCache (src/domain/expert_cache.rs:8-134) kept inside the adapter."""

    def __init__(self, moe: B200MoE):
        self._moe = moe
        self.num_layers, self.num_experts = moe.layers, moe.experts

    def cache_size(self) -> int:
        return self._moe.slots()

    def ensure_experts(self, layer: int, routed):
        """Returns (misses, write_slots, rewrites)."""
        routed = np.ascontiguousarray(routed, np.uint32).reshape(-1)
        n = routed.size
        misses = np.zeros(max(n, 1), np.uint32)
        slots = np.zeros(max(n, 1), np.uint32)
        rewrites = np.zeros(max(n, 1), np.int32)
        nm = C.c_size_t(0)
        p = lambda a: C.c_void_p(a.ctypes.data)
        m = self._moe
        m._check(m._lib.ftm_ensure_experts(m._h, layer, p(routed), n, p(misses), p(slots), p(rewrites), C.byref(nm)))
        return misses[:nm.value].tolist(), slots[:nm.value].tolist(), rewrites[:n].tolist()


def _stage_and_route(cache: ExpertCache, store: B200MoE, layer: int, experts) -> np.ndarray:
    """stage_and_route (run_experts.rs:318-338): plan, load the misses, hand back slot routes."""
    if cache.cache_size() < store.slots():
        raise bad(f"slot cache holds {cache.cache_size()} slots but the adapter stages {store.slots()}")
    misses, write_slots, rewrites = cache.ensure_experts(layer, experts)
    for e, s in zip(misses, write_slots):
        store.load(layer, e, s)
    return np.asarray(rewrites, np.int32)


def run_experts(cache: ExpertCache, store: B200MoE, gemm: B200MoE, layer: int, hidden: int, inter: int, top_k: int, x,
                experts, weights, out: np.ndarray):
    """run_experts (run_experts.rs:209-246): the host-plan step; `out` receives tokens*hidden f32."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    experts = np.ascontiguousarray(experts, np.uint32).reshape(-1)
    weights = np.ascontiguousarray(weights, np.float32).reshape(-1)
    if hidden == 0 or top_k == 0 or x.size % hidden:
        raise bad(f"expert step: hidden {hidden} top_k {top_k} x {x.size}")
    tokens = x.size // hidden
    if experts.size != tokens * top_k or weights.size != tokens * top_k:
        raise bad(f"expert step: {experts.size} experts and {weights.size} weights for {tokens} tokens x top_k {top_k}")
    routes = _stage_and_route(cache, store, layer, experts)
    gemm.grouped_moe(MoEGroup(hidden, inter, x, top_k, routes, weights), out)


class CachedExperts:
    """MoEExecutor over a B200MoE (src/application/run_experts.rs:103-189).

    staged=True hands the router's ids to the device path; staged=False runs the host plan."""

    def __init__(self, moe: B200MoE, staged: bool = True):
        self.moe, self.staged = moe, staged
        self.cache = ExpertCache(moe)
        self._steps = 0

    def steps(self) -> int:
        return self._steps

    def release_cache(self):
        self.moe.release_banks()

    def rehydrate_cache(self):
        self.moe.rehydrate_banks()

    def cache_resident(self) -> bool:
        return self.moe.banks_resident()

    def reset_staging(self):
        self.moe.reset_staging()

    def begin_device(self, req: MoEDeviceRequest):
        if not self.staged:
            return None
        return self.moe.begin_staged(req)

    def execute_device(self, req: MoEDeviceRequest, out, stream=None):
        # counted before the work, so a refused step still shows the port was reached
        self._steps += 1
        tokens = _check_device_step(req)
        if out.numel() < tokens * req.hidden:
            raise bad(f"device expert step: {out.numel()} outputs for {tokens} tokens x hidden {req.hidden}")
        if self.staged:
            return self.moe.grouped_moe_staged(req, out, stream=stream)
        experts = req.experts.to("cpu").reshape(-1).numpy().astype(np.uint32)
        routes = _stage_and_route(self.cache, self.moe, req.layer, experts)
        return self.moe.grouped_moe_dev(req.hidden, req.inter, req.top_k, req.x, routes, req.weights, out,
                                        stream=stream)
