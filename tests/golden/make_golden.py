"""Regenerates tests/golden/ref_torch_oracle.npz from the reference's own Python oracle.

Run in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports `ferrum_kernel.selftest` (python/ferrum_kernel/selftest.py:48-115 in
the reference: `nvfp4_dequant`, `grouped_moe_reference`, `random_case`) and
stores

* for the reference's own seeded `random_case` shapes small enough to commit:
  the inputs and the reference output;
* for larger shapes (up to the real hidden 2048 / inter 512): only the reference
  output, with inputs that `golden_inputs()` below rebuilds from a frozen
  `numpy.random.RandomState` stream, plus a checksum of those inputs.

The tests never import the reference; they read the .npz.
"""
from __future__ import annotations

import os
import sys
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

# (label, tokens, hidden, inter, slots, top_k, seed)
LARGE_CASES = [
    ("wide-k", 2, 512, 256, 3, 2, 11),
    ("qwen-shape", 4, 2048, 512, 4, 2, 12),
    ("qwen-top8", 2, 2048, 512, 9, 8, 13),
]


def e4m3_codes_to_f32(codes: np.ndarray) -> np.ndarray:
    c = codes.astype(np.int32)
    sign = np.where(c & 0x80, -1.0, 1.0)
    exp = (c >> 3) & 0xF
    man = c & 7
    mag = np.where(exp == 0, man * 2.0 ** -9, (1 + man / 8.0) * np.exp2(exp - 7.0))
    return (sign * mag).astype(np.float32)


def golden_inputs(tokens, hidden, inter, slots, top_k, seed):
    """Inputs of a LARGE_CASES entry; identical in the generator and in the tests."""
    rs = np.random.RandomState(seed)

    def bank(rows, cols):
        packed = rs.randint(0, 256, (slots, rows, cols // 2)).astype(np.uint8)
        # positive, finite e4m3 codes between 2^-6 and 2 (0x08 .. 0x40)
        scale = rs.randint(0x08, 0x41, (slots, rows, cols // 16)).astype(np.uint8)
        glob = (rs.rand(slots, rows) * 1.5 + 0.5).astype(np.float16)
        return packed, scale, glob

    gu = bank(2 * inter, hidden)
    dn = bank(hidden, inter)
    x = (rs.rand(tokens, hidden) * 2.0 - 1.0).astype(np.float32)
    # keep x on the bf16 grid so the device path (bf16 activations) sees the same numbers
    x = ((x.view(np.uint32) + 0x8000) & 0xFFFF0000).view(np.float32)
    slot = rs.randint(-1, slots, tokens * top_k).astype(np.int32)
    weight = (rs.rand(tokens * top_k) * 0.5).astype(np.float32)
    return x, gu, dn, slot, weight


def checksum(*arrays) -> int:
    c = 0
    for a in arrays:
        c = zlib.crc32(np.ascontiguousarray(a).view(np.uint8).tobytes(), c)
    return c


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "python"))
    import torch
    from ferrum_kernel import selftest as st

    out = {}
    # 1) the reference's own random_case at its default and many-routes shapes
    small = [("default", {}), ("many-routes", dict(tokens=8, hidden=256, inter=128, slots=4, top_k=4))]
    for label, shape in small:
        for seed in range(4 if label == "default" else 2):
            x, gu, dn, slot, token, weight = st.random_case("cpu", seed=seed, **shape)
            want = st.grouped_moe_reference(x, *gu, *dn, slot, token, weight)
            k = f"{label}/{seed}/"
            out[k + "x"] = x.numpy()
            for name, t in zip(("gu_packed", "gu_scale", "gu_global"), gu):
                out[k + name] = t.view(torch.uint8).numpy() if t.dtype != torch.uint8 else t.numpy()
            for name, t in zip(("dn_packed", "dn_scale", "dn_global"), dn):
                out[k + name] = t.view(torch.uint8).numpy() if t.dtype != torch.uint8 else t.numpy()
            out[k + "slot"] = slot.numpy()
            out[k + "token"] = token.numpy()
            out[k + "weight"] = weight.numpy()
            out[k + "want"] = want.numpy()
            # the dense widening too (selftest.py:48-61)
            if label == "default":
                out[k + "gu_dense"] = st.nvfp4_dequant(*gu).numpy().astype(np.float32)
    # 2) larger shapes, inputs rebuilt from the frozen stream
    for label, tokens, hidden, inter, slots, top_k, seed in LARGE_CASES:
        x, gu, dn, slot, weight = golden_inputs(tokens, hidden, inter, slots, top_k, seed)
        tt = lambda a: torch.from_numpy(a)
        gu_t = (tt(gu[0]), tt(gu[1]).view(torch.float8_e4m3fn), tt(gu[2]))
        dn_t = (tt(dn[0]), tt(dn[1]).view(torch.float8_e4m3fn), tt(dn[2]))
        token = torch.arange(tokens, dtype=torch.int32).repeat_interleave(top_k)
        want = st.grouped_moe_reference(tt(x), *gu_t, *dn_t, tt(slot), token, tt(weight))
        out[f"{label}/want"] = want.numpy()
        out[f"{label}/crc"] = np.array([checksum(x, *gu, *dn, slot, weight)], np.uint32)
    np.savez_compressed(os.path.join(HERE, "ref_torch_oracle.npz"), **out)
    print("wrote", os.path.join(HERE, "ref_torch_oracle.npz"), len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to a checkout of butzist/ferrum-torrens>")
    main(sys.argv[1])
