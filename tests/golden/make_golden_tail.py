"""Regenerates tests/golden/ref_tail_ops.npz from the reference's own Python oracles of the two steps either
side of the MoE block:

* `ferrum_kernel.norm.add_rmsnorm_reference`   (python/ferrum_kernel/norm.py:97-107)
* `ferrum_kernel.linear.nvfp4_dense_gemv_reference`   (python/ferrum_kernel/linear.py:152-168)

    python tests/golden/make_golden_tail.py /path/to/reference

Inputs are rebuilt by `norm_inputs()` / `gemv_inputs()` from a frozen numpy RandomState stream (identical in
the generator and in the tests); the file stores the reference outputs and a checksum of the inputs.  The
tests never import the reference; they read the .npz.
"""
from __future__ import annotations

import os
import sys
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

# (label, rows, hidden, eps, seed)
NORM_CASES = [("norm-small", 3, 64, 1e-6, 21), ("norm-qwen", 5, 2048, 1e-6, 22)]
# (label, M, N, K, seed)
GEMV_CASES = [("gemv-small", 2, 64, 128, 31), ("gemv-wide", 3, 256, 2048, 32)]


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def norm_inputs(rows, hidden, seed):
    """x, r, w as bf16 bit patterns."""
    rs = np.random.RandomState(seed)
    x = to_bf16_bits(rs.randn(rows, hidden).astype(np.float32))
    r = to_bf16_bits((rs.randn(rows, hidden) * 3.0).astype(np.float32))
    w = to_bf16_bits((1.0 + rs.randn(hidden) * 0.1).astype(np.float32))
    return x, r, w


def gemv_inputs(m, n, k, seed):
    """a [M, K] bf16 bits; the weight ROW-major as the Python oracle takes it: packed [N, K/2] u8 (low nibble =
    even k), scale [N, K/16] e4m3 codes (positive, 2^-6 .. 2), global [N] f16."""
    rs = np.random.RandomState(seed)
    a = to_bf16_bits((rs.rand(m, k) * 2.0 - 1.0).astype(np.float32))
    packed = rs.randint(0, 256, (n, k // 2)).astype(np.uint8)
    scale = rs.randint(0x08, 0x41, (n, k // 16)).astype(np.uint8)
    glob = (rs.rand(n) * 1.5 + 0.5).astype(np.float16)
    return a, packed, scale, glob


def kmajor(packed: np.ndarray, scale: np.ndarray):
    """Row-major [N, K/2] u8 / [N, K/16] -> the K-major resident bank: packed [K/8, N] int32 (nibble j of a word =
    code k = 8w + j), scale [K/16, N]."""
    n = packed.shape[0]
    words = np.ascontiguousarray(packed).view("<u4").reshape(n, -1)     # little endian: byte b = codes 2b, 2b+1
    return np.ascontiguousarray(words.T), np.ascontiguousarray(scale.T)


def checksum(*arrays) -> int:
    c = 0
    for a in arrays:
        c = zlib.crc32(np.ascontiguousarray(a).view(np.uint8).tobytes(), c)
    return c


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "python"))
    import torch
    from ferrum_kernel import linear, norm

    bf = lambda bits: torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16)
    out = {}
    for label, rows, hidden, eps, seed in NORM_CASES:
        x, r, w = norm_inputs(rows, hidden, seed)
        s, y = norm.add_rmsnorm_reference(bf(x), bf(r), bf(w), eps)
        out[f"{label}/sum"] = s.view(torch.int16).numpy().view(np.uint16)
        out[f"{label}/out"] = y.view(torch.int16).numpy().view(np.uint16)
        out[f"{label}/crc"] = np.array([checksum(x, r, w)], np.uint32)
    for label, m, n, k, seed in GEMV_CASES:
        a, packed, scale, glob = gemv_inputs(m, n, k, seed)
        c = linear.nvfp4_dense_gemv_reference(bf(a), torch.from_numpy(packed),
                                              torch.from_numpy(scale).view(torch.float8_e4m3fn), torch.from_numpy(glob))
        out[f"{label}/c"] = c.numpy().astype(np.float32)
        out[f"{label}/crc"] = np.array([checksum(a, packed, scale, glob)], np.uint32)
    np.savez_compressed(os.path.join(HERE, "ref_tail_ops.npz"), **out)
    print("wrote", os.path.join(HERE, "ref_tail_ops.npz"), len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden_tail.py <path to a checkout of butzist/ferrum-torrens>")
    main(sys.argv[1])
