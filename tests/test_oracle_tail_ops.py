"""The CPU checker's restatements of the two steps either side of the MoE block, pinned to outputs of the
reference's own Python oracles (tests/golden/ref_tail_ops.npz, produced by tests/golden/make_golden_tail.py
from python/ferrum_kernel/norm.py `add_rmsnorm_reference` and python/ferrum_kernel/linear.py
`nvfp4_dense_gemv_reference`)."""
import importlib.util
import os

import numpy as np
import pytest

from oracle import oracle as o

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("make_golden_tail", os.path.join(HERE, "golden", "make_golden_tail.py"))
mg = importlib.util.module_from_spec(spec)
spec.loader.exec_module(mg)
G = np.load(os.path.join(HERE, "golden", "ref_tail_ops.npz"))


def bf(bits):
    return o.bf16_bits_to_f32(bits)


@pytest.mark.parametrize("case", mg.NORM_CASES, ids=[c[0] for c in mg.NORM_CASES])
def test_add_rmsnorm_matches_the_reference_oracle(case):
    label, rows, hidden, eps, seed = case
    x, r, w = mg.norm_inputs(rows, hidden, seed)
    assert mg.checksum(x, r, w) == int(G[f"{label}/crc"][0]), "input stream changed"
    s, y = o.add_rmsnorm(x, r, w, eps)
    # the residual sum is one rounding of an exact f32 add: bit-exact
    assert np.array_equal(s, G[f"{label}/sum"])
    # the torch oracle reduces the row in another order than the host tower: the reciprocal can differ in its
    # last bits, which moves a normalised value by at most one bf16 unit in the last place, rarely
    want = G[f"{label}/out"]
    diff = np.abs(y.astype(np.int32) - want.astype(np.int32))
    assert diff.max() <= 1
    assert (diff != 0).mean() <= 0.01
    # and against the host tower's own f32 rms_norm of the same sum: within bf16 rounding
    tower = o.rms_norm(bf(s), bf(w), eps)
    assert np.abs(bf(y) - tower).max() <= np.abs(tower).max() * 2.0 ** -8


def test_rms_norm_known_answer():
    """x = [3, 4] per row: mean of squares 12.5, so out = x / sqrt(12.5 + eps) * w."""
    x = np.array([[3.0, 4.0], [0.0, 0.0]], np.float32)
    w = np.array([1.0, 2.0], np.float32)
    out = o.rms_norm(x, w, 0.0 + 1e-6)
    inv = np.float32(1.0) / np.sqrt(np.float32(12.5) + np.float32(1e-6), dtype=np.float32)
    assert np.allclose(out[0], [3.0 * inv, 8.0 * inv], rtol=1e-6)
    assert np.array_equal(out[1], np.zeros(2, np.float32))


@pytest.mark.parametrize("case", mg.GEMV_CASES, ids=[c[0] for c in mg.GEMV_CASES])
def test_dense_gemv_matches_the_reference_oracle(case):
    label, m, n, k, seed = case
    a, packed, scale, glob = mg.gemv_inputs(m, n, k, seed)
    assert mg.checksum(a, packed, scale, glob) == int(G[f"{label}/crc"][0]), "input stream changed"
    pk, sk = mg.kmajor(packed, scale)
    assert pk.shape == (k // 8, n) and sk.shape == (k // 16, n)
    c = o.nvfp4_dense_gemv(bf(a), pk, sk, glob.view(np.uint16))
    want = G[f"{label}/c"]
    # same products, the torch matmul sums them in another order: compare against the size of the summed terms
    dense = np.stack([o.nvfp4_block(packed[i:i + 1].reshape(-1), 1, k, scale[i]) for i in range(n)]).reshape(n, k)
    dense = dense * glob.astype(np.float32)[:, None]
    abs_sum = np.abs(bf(a)) @ np.abs(dense).T
    assert np.abs(c - want).max() <= 2e-5 * abs_sum.max()
    # and the K-major words hold nibble j = code k = 8w + j of the row (cuda_linear.rs:103-111)
    row, w = 5, 3
    codes = [(int(pk[w, row]) >> (4 * j)) & 0xF for j in range(8)]
    want_codes = []
    for j in range(8):
        byte = int(packed[row, (8 * w + j) // 2])
        want_codes.append((byte >> 4) if j % 2 else (byte & 0xF))
    assert codes == want_codes


def test_stage_dump_prints_the_reference_format(capfd, monkeypatch):
    """FT_TRACE=1: `TRACE <layer> <stage> l2=<..> amax=<..>` on stderr (forward.rs:833-855), nothing without it."""
    v = np.array([3.0, -4.0], np.float32)
    o.trace_vec("moe", 7, v)
    assert capfd.readouterr().err == ""
    monkeypatch.setenv("FT_TRACE", "1")
    o.trace_vec("moe", 7, v)
    assert capfd.readouterr().err == "TRACE 7 moe l2=5.000000 amax=4.000000\n"
