"""FTW checkpoint index and expert-bank source over the C ABI of libftmoe.so.

Mirrors the reference's `FtwIndex` / `FtwReader` (src/infrastructure/ftw.rs) and `FtwBanks`
(src/infrastructure/banks.rs:84-199).  `FtwBanks` is an `ExpertSlabSource`: `slab(layer, expert, part)`
returns one expert's `(packed, scale, global)` byte arrays, so it can be handed to `B200MoE(source=...)`;
`load_layer` reads every expert of a layer straight into an adapter's resident banks.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import _lib as L
from .moe import MoEError

INDEX_NAME = "freetoken_weight.json"
PARTS = {"GateUp": 0, "Down": 1}


def layer_bank_entry(name: str):
    """`gate_up_packed#L00007` -> ("gate_up_packed", 7); None for any other name (ftw.rs:81-92)."""
    at = name.rfind("#L")
    if at <= 0:
        return None
    layer = name[at + 2:]
    if len(layer) != 5 or not layer.isdigit():
        return None
    return name[:at], int(layer)


class FtwIndex:
    """A parsed index.  `FtwIndex.parse(text)` validates like the reference; `FtwIndex.open(dir)` also opens
    the shard files so that ranges can be read."""

    def __init__(self, handle):
        self._lib = L.lib()
        self._h = handle

    @classmethod
    def _make(cls, fn, arg: bytes):
        lib = L.lib()
        h = C.c_void_p()
        rc = getattr(lib, fn)(arg, C.byref(h))
        if rc != L.OK:
            raise MoEError(rc, (lib.ftm_ftw_last_error(None) or b"").decode())
        return cls(h)

    @classmethod
    def parse(cls, doc: str) -> "FtwIndex":
        return cls._make("ftm_ftw_parse", doc.encode())

    @classmethod
    def open(cls, path: str) -> "FtwIndex":
        return cls._make("ftm_ftw_open", os.fspath(path).encode())

    def close(self):
        if getattr(self, "_h", None):
            self._lib.ftm_ftw_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != L.OK:
            raise MoEError(rc, (self._lib.ftm_ftw_last_error(self._h) or b"").decode())

    @property
    def total_bytes(self) -> int:
        return int(self._lib.ftm_ftw_total_bytes(self._h))

    def __len__(self) -> int:
        return int(self._lib.ftm_ftw_tensor_count(self._h))

    def shard_count(self) -> int:
        return int(self._lib.ftm_ftw_shard_count(self._h))

    def entry(self, name: str):
        """{global_off, nbytes, shape, experts_bank} or None."""
        off, nb, nd, eb = C.c_uint64(0), C.c_uint64(0), C.c_int32(0), C.c_int32(0)
        shape = (C.c_uint64 * 8)()
        rc = self._lib.ftm_ftw_entry(self._h, name.encode(), C.byref(off), C.byref(nb), shape, C.byref(nd), C.byref(eb))
        if rc == L.ERR_MISSING:
            return None
        self._check(rc)
        return {"global_off": off.value, "nbytes": nb.value, "shape": [int(shape[i]) for i in range(nd.value)],
                "experts_bank": bool(eb.value)}

    def pieces(self, global_off: int, nbytes: int):
        """[(shard index, file_off, dest_off, length)] of a byte range (FtwIndex::pieces)."""
        cap = max(1, self.shard_count())
        si = (C.c_int32 * cap)()
        fo, do, ln = (C.c_uint64 * cap)(), (C.c_uint64 * cap)(), (C.c_uint64 * cap)()
        n = C.c_int32(0)
        self._check(self._lib.ftm_ftw_pieces(self._h, global_off, nbytes, cap, si, fo, do, ln, C.byref(n)))
        return [(int(si[i]), int(fo[i]), int(do[i]), int(ln[i])) for i in range(n.value)]

    def read_range(self, global_off: int, nbytes: int) -> np.ndarray:
        out = np.empty(nbytes, np.uint8)
        self._check(self._lib.ftm_ftw_read_range(self._h, global_off, nbytes, C.c_void_p(out.ctypes.data), out.size))
        return out


class FtwBanks:
    """Checkpoint-backed slab source (banks.rs:84-199).  `prefix` "" for the target's layers, "draft_" for the
    MTP draft's single layer."""

    def __init__(self, index: FtwIndex, prefix: str = ""):
        self.index, self.prefix = index, prefix

    def slab(self, layer: int, expert: int, part: str):
        ix = self.index
        packed_entry = ix.entry(f"{self.prefix}{'gate_up' if part == 'GateUp' else 'down'}_packed#L{layer:05d}")
        if packed_entry is None or len(packed_entry["shape"]) != 3:
            cap = (1, 1, 1)
        else:
            _, rows, pc = packed_entry["shape"]
            cap = (rows * pc, rows * pc * 2 // 16, rows * 2)
        bufs = [np.empty(max(1, c), np.uint8) for c in cap]
        caps = (C.c_size_t * 3)(*[b.size for b in bufs])
        lens = (C.c_size_t * 3)()
        rows, cols = C.c_int32(0), C.c_int32(0)
        ix._check(ix._lib.ftm_ftw_expert_slab(ix._h, self.prefix.encode(), layer, expert, PARTS[part],
                                              *[C.c_void_p(b.ctypes.data) for b in bufs], caps, lens, C.byref(rows),
                                              C.byref(cols)))
        return tuple(b[:lens[i]] for i, b in enumerate(bufs))

    def load_layer(self, moe, layer: int, first_expert: int = 0, n_experts: int | None = None, slot0: int | None = None):
        """Every expert of `layer` into slots slot0, slot0 + 1, .. of the adapter (default: layer * experts + expert)."""
        n = moe.experts - first_expert if n_experts is None else n_experts
        s0 = layer * moe.experts + first_expert if slot0 is None else slot0
        ix = self.index
        ix._check(ix._lib.ftm_load_layer_from_ftw(moe._h, ix._h, self.prefix.encode(), layer, first_expert, n, s0))
