"""The permutation build that allocates nothing, against the regular entry point.

Some hosts cannot call cudaMalloc once they are running: an inference engine that hands out all of
its device memory at start-up and then locks the allocator, or code running where allocation is not
allowed.  `ftm_csr_build_noalloc` serves them: no adapter handle, scratch in a fixed array inside the
library.  This file is collected last on purpose, so a failure here cannot hide another test.
"""
import ctypes as C
import importlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
pkg = importlib.import_module("ferrum-torrens_b200")
L = pkg._lib


def _run_noalloc(route_slot, bins):
    lib = L.lib()
    dev = route_slot.device
    seg = torch.full((bins + 1,), -7, dtype=torch.int32, device=dev)
    idx = torch.full((route_slot.numel(),), -7, dtype=torch.int32, device=dev)
    bad = torch.full((1,), -7, dtype=torch.int32, device=dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.ftm_csr_build_noalloc(C.c_void_p(route_slot.data_ptr()), route_slot.numel(), bins,
                                   C.c_void_p(seg.data_ptr()), C.c_void_p(idx.data_ptr()), C.c_void_p(bad.data_ptr()),
                                   stream)
    torch.cuda.synchronize()
    return rc, seg, idx, int(bad.item())


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    dev = torch.device("cuda:0")
    moe = pkg.B200MoE(0, pkg.ExpertShapes(64, 32), 4, experts=4, layers=1, top_k=2, shared_inter=16, max_tokens=40000)
    rng = np.random.default_rng(0)
    # two calls in a row with different sizes and contents: the second must not see the first's leftovers
    for n, bins in ((70001, 256), (5000, 37)):
        routes = torch.from_numpy(rng.integers(0, bins, n).astype(np.int32)).to(dev)
        want_seg, want_idx, want_bad = moe.csr_build(routes, bins)
        rc, seg, idx, bad = _run_noalloc(routes, bins)
        assert rc == L.OK
        assert torch.equal(seg, want_seg) and torch.equal(idx, want_idx)
        assert bad == want_bad == 0
    # a slot outside the bins raises the flag, and the next call starts clean again
    routes = torch.tensor([0, 5, 1], dtype=torch.int32, device=dev)
    rc, _, _, bad = _run_noalloc(routes, 3)
    assert rc == L.OK and bad == 1
    routes = torch.tensor([2, 0, 2, 0, 0, 1], dtype=torch.int32, device=dev)
    rc, seg, idx, bad = _run_noalloc(routes, 3)
    assert rc == L.OK and bad == 0
    assert seg.cpu().tolist() == [0, 3, 4, 6] and idx.cpu().tolist() == [1, 3, 4, 5, 0, 2]
    moe.close()


def test_noalloc_rejects_sizes_beyond_its_fixed_scratch():
    dev = torch.device("cuda:0")
    routes = torch.zeros(8, dtype=torch.int32, device=dev)
    lib = L.lib()
    null = C.c_void_p(0)
    p = C.c_void_p(routes.data_ptr())
    assert lib.ftm_csr_build_noalloc(p, 262145, 8, p, p, null, null) == L.ERR_BAD
    assert lib.ftm_csr_build_noalloc(p, 8, 1025, p, p, null, null) == L.ERR_BAD
    assert lib.ftm_csr_build_noalloc(p, 0, 8, p, p, null, null) == L.ERR_BAD
    assert lib.ftm_csr_build_noalloc(null, 8, 8, p, p, null, null) == L.ERR_BAD
