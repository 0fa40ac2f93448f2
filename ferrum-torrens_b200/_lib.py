"""Loads libftmoe.so and declares the C ABI of include/ftmoe.h for ctypes.

There is no fallback: if the library is missing or cannot be loaded the import fails, and every
compute entry point needs a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libftmoe.so")

OK, ERR_BAD, ERR_SLOT_OUT_OF_RANGE, ERR_MISSING, ERR_OUT_OF_MEMORY, ERR_READ, ERR_NOT_SUPPORTED, ERR_CUDA = range(8)
BF16, F32, I32, I64 = range(4)
PATH_AUTO, PATH_GEMV, PATH_GROUPED, PATH_SCALAR = range(4)
NUM_BANKS = 6


class Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("ordinal", "hidden", "inter", "top_k", "experts", "layers", "slots",
                                         "shared_inter", "max_tokens", "ep_rank", "ep_size")]


_vp, _i32, _sz, _int = C.c_void_p, C.c_int32, C.c_size_t, C.c_int
_PROTOS = {
    "ftm_abi_version": (_int, []),
    "ftm_create": (_int, [C.POINTER(Config), _vp, C.POINTER(_vp)]),
    "ftm_destroy": (None, [_vp]),
    "ftm_last_error": (C.c_char_p, [_vp]),
    "ftm_load_expert": (_int, [_vp, _i32, _i32, _i32, C.POINTER(_vp), C.POINTER(_sz)]),
    "ftm_load_expert_dev": (_int, [_vp, _i32, _i32, _i32, C.POINTER(_vp), C.POINTER(_sz)]),
    "ftm_slots": (_int, [_vp]),
    "ftm_release_banks": (_int, [_vp]),
    "ftm_rehydrate_banks": (_int, [_vp]),
    "ftm_banks_resident": (_int, [_vp]),
    "ftm_bank_ptrs": (_int, [_vp, C.POINTER(C.c_uint64)]),
    "ftm_bank_row_bytes": (_sz, [_vp, _int]),
    "ftm_slot_of": (_i32, [_vp, _i32, _i32]),
    "ftm_ensure_experts": (_int, [_vp, _i32, _vp, _sz, _vp, _vp, _vp, C.POINTER(_sz)]),
    "ftm_router": (_int, [_vp, _vp, _vp, _i32, _vp, _vp, _vp]),
    "ftm_router_from_logits": (_int, [_vp, _vp, _i32, _vp, _vp, _vp]),
    "ftm_csr_build": (_int, [_vp, _vp, _i32, _i32, _vp, _vp, _vp]),
    "ftm_csr_bad": (_int, [_vp, _vp, C.POINTER(_i32)]),
    "ftm_csr_build_noalloc": (_int, [_vp, _i32, _i32, _vp, _vp, _vp, _vp]),
    "ftm_grouped_moe_host": (_int, [_vp, _vp, _sz, _i32, _vp, _sz, _vp, _sz, _vp, _sz]),
    "ftm_grouped_moe_dev": (_int, [_vp, _vp, _int, _i32, _i32, _vp, _sz, _vp, _vp, _int, _vp]),
    "ftm_moe_layer_staged": (_int, [_vp, _i32, _vp, _int, _vp, _int, _vp, _i32, _vp, _int, _int, _vp]),
    "ftm_moe_begin": (_int, [_vp, _i32, _vp, _int, _vp, _int, _vp, _i32, _vp]),
    "ftm_moe_finish": (_int, [_vp, _vp, _int, _vp]),
    "ftm_route_cap": (_sz, [_vp]),
    "ftm_reset_staging": (_int, [_vp]),
    "ftm_steps": (C.c_uint64, [_vp]),
    "ftm_sync_status": (_int, [_vp, _vp]),
    "ftm_shared_expert": (_int, [_vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "ftm_combine": (_int, [_vp, _vp, _int, _vp, _vp, _i32, _vp, _int, _vp]),
    "ftm_moe_block": (_int, [_vp, _i32, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _int, _vp, _vp, _int, _vp]),
    "ftm_add_rmsnorm": (_int, [_vp, _vp, _vp, _vp, C.c_float, _i32, _vp, _vp, _vp]),
    "ftm_moe_block_prenorm": (_int, [_vp, _i32, _vp, _vp, _vp, C.c_float, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _int,
                                     _vp, _vp, _int, _vp]),
    "ftm_dense_gemv": (_int, [_vp, _vp, _int, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp]),
    "ftm_ftw_open": (_int, [C.c_char_p, C.POINTER(_vp)]),
    "ftm_ftw_parse": (_int, [C.c_char_p, C.POINTER(_vp)]),
    "ftm_ftw_close": (None, [_vp]),
    "ftm_ftw_last_error": (C.c_char_p, [_vp]),
    "ftm_ftw_tensor_count": (C.c_int64, [_vp]),
    "ftm_ftw_shard_count": (C.c_int64, [_vp]),
    "ftm_ftw_total_bytes": (C.c_uint64, [_vp]),
    "ftm_ftw_entry": (_int, [_vp, C.c_char_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64),
                             C.POINTER(_i32), C.POINTER(_i32)]),
    "ftm_ftw_pieces": (_int, [_vp, C.c_uint64, C.c_uint64, _i32, _vp, _vp, _vp, _vp, C.POINTER(_i32)]),
    "ftm_ftw_read_range": (_int, [_vp, C.c_uint64, C.c_uint64, _vp, _sz]),
    "ftm_ftw_expert_slab": (_int, [_vp, C.c_char_p, _i32, C.c_uint32, _i32, _vp, _vp, _vp, C.POINTER(_sz), C.POINTER(_sz),
                                   C.POINTER(_i32), C.POINTER(_i32)]),
    "ftm_load_layer_from_ftw": (_int, [_vp, _vp, C.c_char_p, _i32, _i32, _i32, _i32]),
    "ftm_set_sm_budget": (C.c_int, [_vp, C.c_int32]),
    "ftm_kernel_launches": (C.c_uint64, [_vp]),
    "ftm_ep_pack": (_int, [_vp, _vp, _vp, _vp, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "ftm_ep_plan": (_int, [_vp, _vp, _i32, _i32, _vp, _vp, _vp]),
    "ftm_ep_dispatch": (_int, [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp, C.c_int64, _vp]),
    "ftm_ep_return": (_int, [_vp, _vp, _i32, _i32, _i32, _vp, _vp, C.c_int64, _vp]),
    "ftm_ep_experts_sorted": (_int, [_vp, _i32, _vp, _vp, _vp, _i32, _vp]),
    "ftm_ep_experts_return": (_int, [_vp, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp, C.c_int64, _vp]),
    "ftm_ep_plan_seg": (_int, [_vp, _vp, _i32, _vp, _vp, _vp]),
    "ftm_ep_dispatch_sorted": (_int, [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, C.c_int64, _vp]),
    "ftm_ep_experts_presorted": (_int, [_vp, _i32, _vp, _vp, _vp, _i32, C.c_int64, _i32, _i32, _vp, _vp, C.c_int64, _vp]),
    "ftm_ep_return_sorted": (_int, [_vp, _i32, _i32, _i32, _vp, _vp, C.c_int64, _vp]),
    "ftm_ep_combine": (_int, [_vp, _vp, _int, _vp, _vp, _vp, _i32, _vp, _int, _vp]),
    "ftm_profile_enable": (_int, [_vp, _int]),
    "ftm_profile_read": (_int, [_vp, _int, C.POINTER(C.c_double), C.POINTER(C.c_uint64)]),
    "ftm_profile_kind_name": (C.c_char_p, [_int]),
}

_lib = None


def exported_symbols() -> list[str]:
    return sorted(_PROTOS)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python ferrum-torrens_b200/build.py` "
                              "(there is no CPU or framework fallback)")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in _PROTOS.items():
            fn = getattr(l, name)  # AttributeError if the library does not export it
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib
