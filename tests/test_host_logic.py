"""CPU-side checks: the library loads and exports the whole C ABI, refuses to run without a GPU,
and the host logic (shapes, route lists, slot machine, synthetic generators) behaves like the
reference's."""
import importlib
import os
import re
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pkg = importlib.import_module("ferrum-torrens_b200")
L = pkg._lib


@pytest.fixture(scope="module")
def built():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as ge
    ge.build()
    return L.lib()


def test_library_exports_every_declared_symbol(built):
    header = open(os.path.join(ROOT, "include", "ftmoe.h")).read()
    declared = sorted(set(re.findall(r"FTM_API[^;]*?\b(ftm_\w+)\s*\(", header)))
    assert len(declared) >= 30
    assert declared == L.exported_symbols()
    for name in declared:
        assert hasattr(built, name), name
    assert built.ftm_abi_version() == 1


def test_create_fails_loudly_without_a_device(built):
    import ctypes as C
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(pkg.MoEError) as e:
        pkg.B200MoE(0, pkg.ExpertShapes(2048, 512), 256)
    assert "no CUDA device" in str(e.value) and "no CPU path" in str(e.value)


def test_config_is_validated_before_any_device_work(built):
    for kw, msg in ((dict(slots=0), "at least one slot"), (dict(top_k=0), "top_k"), (dict(max_tokens=0), "max_tokens")):
        args = dict(slots=4, top_k=8, max_tokens=16)
        args.update(kw)
        with pytest.raises(pkg.MoEError, match=msg):
            pkg.B200MoE(0, pkg.ExpertShapes(64, 32), args["slots"], top_k=args["top_k"], max_tokens=args["max_tokens"])


def test_shapes_need_multiples_of_sixteen():
    """src/domain/expert_kernel.rs:654-664, :682-696"""
    pkg.ExpertShapes(1024, 512)
    for h, i in ((1000, 512), (1024, 0)):
        with pytest.raises(pkg.MoEError):
            pkg.ExpertShapes(h, i)
    s = pkg.ExpertShapes(2048, 512)
    assert s.slab_shape("GateUp") == (1024, 2048) and s.slab_shape("Down") == (2048, 512)
    want = [1024 * 2048 // 2, 1024 * 2048 // 16, 1024 * 2, 2048 * 512 // 2, 2048 * 512 // 16, 2048 * 2]
    assert [s.bank_row_bytes(b) for b in pkg.BANKS] == want
    assert sum(want) == 1775616


def test_routes_flatten_token_major():
    tok, slot = pkg.route_lists([3, -1, 1, 1, 0, 2], 3, 2)
    assert tok.tolist() == [0, 0, 1, 1, 2, 2] and slot.tolist() == [3, -1, 1, 1, 0, 2]
    for args in (([0, 1], 2, 2), ([], 0, 1), ([0], 1, 0)):
        with pytest.raises(pkg.MoEError):
            pkg.route_lists(*args)


def test_error_kinds_map_onto_the_reference_variants():
    kinds = {c: pkg.MoEError(c, "x").kind for c in range(1, 8)}
    assert kinds == {1: "Bad", 2: "SlotOutOfRange", 3: "Missing", 4: "OutOfMemory", 5: "Read", 6: "NotSupported",
                     7: "Bad"}
    assert pkg.MoEError(4, "moe: out of device memory: x").retryable


def test_slot_machine_matches_the_reference_cases(tmp_path):
    exe = tmp_path / "test_expert_cache"
    src = os.path.join(ROOT, "tests", "cpp", "test_expert_cache.cpp")
    subprocess.run(["/usr/bin/g++", "-std=c++17", "-O1", src, "-o", str(exe)], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout


def test_synthetic_layer_distributions():
    s = pkg.synth
    lay = s.make_layer(3, hidden=64, inter=32, experts=8, top_k=2, shared_inter=32)
    assert [b.shape for b in lay.banks] == [(8, 64 * 64 // 2), (8, 64 * 64 // 16), (8, 128), (8, 64 * 32 // 2),
                                            (8, 64 * 32 // 16), (8, 128)]
    sc = lay.banks[1]
    assert sc.min() >= 0x08 and sc.max() <= 0x38          # 2^-6 .. 2^0, positive, finite
    assert (lay.banks[2].view(np.uint16) == 0x3C00).all()  # f16 1.0 row globals
    again = s.make_layer(3, hidden=64, inter=32, experts=8, top_k=2, shared_inter=32)
    assert all(np.array_equal(a, b) for a, b in zip(lay.banks, again.banks))
    codes = s.nearest_e4m3(np.array([1.0, 0.5, 0.015625, 1.06, 1.07]))
    assert codes.tolist() == [0x38, 0x30, 0x08, 0x38, 0x39]
    x = s.make_x(1, 4, 64)
    assert x.dtype == np.uint16 and x.shape == (4, 64)
