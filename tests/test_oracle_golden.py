"""The CPU checker against outputs of the reference's own Python torch oracle.

tests/golden/ref_torch_oracle.npz was produced by tests/golden/make_golden.py
from python/ferrum_kernel/selftest.py (`nvfp4_dequant`, `grouped_moe_reference`,
`random_case`) of the reference.  The torch oracle does a dense matmul, so its
f32 sums associate differently from the scalar loop; agreement is checked against
the size of the summed terms (abs_sum), the yardstick the reference itself uses
(tests/cuda_moe_matches_reference.rs:43-53).
"""
import importlib.util
import os

import numpy as np
import pytest

from oracle import oracle as o

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
mg = importlib.util.module_from_spec(spec)
spec.loader.exec_module(mg)
G = np.load(os.path.join(HERE, "golden", "ref_torch_oracle.npz"))

SMALL = [("default", s, 64, 32, 4, 2) for s in range(4)] + \
        [("many-routes", s, 256, 128, 4, 4) for s in range(2)]


def banks_from(gu, dn, slots, hidden, inter):
    return o.HostBanks(gu[0], gu[1], np.ascontiguousarray(gu[2]).view(np.uint8), dn[0], dn[1],
                       np.ascontiguousarray(dn[2]).view(np.uint8), slots, 2 * inter, hidden, hidden, inter)


@pytest.mark.parametrize("label,seed,hidden,inter,slots,top_k", SMALL)
def test_small_cases_match_reference_torch_oracle(label, seed, hidden, inter, slots, top_k):
    k = f"{label}/{seed}/"
    gu = [G[k + n] for n in ("gu_packed", "gu_scale", "gu_global")]
    dn = [G[k + n] for n in ("dn_packed", "dn_scale", "dn_global")]
    banks = banks_from(gu, dn, slots, hidden, inter)
    out, abs_sum = o.grouped_moe_reference(banks, hidden, inter, G[k + "x"], top_k, G[k + "slot"],
                                           G[k + "weight"], want_abs_sum=True)
    want = G[k + "want"]
    assert np.abs(out - want).max() <= 2e-5 * max(abs_sum.max(), 1e-6)
    # route_lists gives the token list the reference case carries
    tok, slot = o.route_lists(G[k + "slot"], out.shape[0], top_k)
    assert np.array_equal(tok, G[k + "token"]) and np.array_equal(slot, G[k + "slot"])


@pytest.mark.parametrize("seed", range(4))
def test_dense_widening_matches_reference_dequant(seed):
    k = f"default/{seed}/"
    slots, rows, cols = 4, 64, 64
    packed, scale = G[k + "gu_packed"], G[k + "gu_scale"]
    glob = G[k + "gu_global"].view(np.float16).astype(np.float32).reshape(slots, rows)
    for s in range(slots):
        w = o.nvfp4_block(packed[s], rows, cols, scale[s]) * glob[s][:, None]
        assert np.array_equal(w.astype(np.float32), G[k + "gu_dense"][s])


@pytest.mark.parametrize("case", mg.LARGE_CASES, ids=[c[0] for c in mg.LARGE_CASES])
def test_large_cases_match_reference_torch_oracle(case):
    label, tokens, hidden, inter, slots, top_k, seed = case
    x, gu, dn, slot, weight = mg.golden_inputs(tokens, hidden, inter, slots, top_k, seed)
    assert mg.checksum(x, *gu, *dn, slot, weight) == int(G[f"{label}/crc"][0]), "input stream changed"
    banks = banks_from(gu, dn, slots, hidden, inter)
    out, abs_sum = o.grouped_moe_reference(banks, hidden, inter, x, top_k, slot, weight, want_abs_sum=True)
    want = G[f"{label}/want"]
    assert np.abs(out - want).max() <= 2e-5 * abs_sum.max()
    # the threaded form is the same arithmetic
    mt = o.grouped_moe_reference_mt(banks, hidden, inter, x, top_k, slot, weight, threads=4)
    assert np.array_equal(mt, out)
