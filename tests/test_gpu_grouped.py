"""The tcgen05 grouped GEMM (FTM_PATH_GROUPED; FTM_PATH_AUTO above 2048 routes) against the CPU checker.

Same bars as the decode path: the permutation is exact by construction (the CSR tests cover it), outputs
are compared with the f32 restatement of the reference's host path (src/domain/expert_kernel.rs:547-618).
The cases cover: one token, fewer tokens than one accumulator tile, experts cut into several passes of 128
rows (tokens all routed to a few experts), experts that are not resident, f32 and bf16 activations and
outputs, and ids given as i64.
"""
import importlib

import numpy as np
import pytest
import torch

from oracle import oracle as o

pkg = importlib.import_module("ferrum-torrens_b200")
L = pkg._lib

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda:0")


def bf16_dev(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(dev()).view(torch.bfloat16)


def rel_l2(got, want):
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


@pytest.fixture(scope="module")
def layer():
    lay = pkg.synth.make_layer(77)
    shapes = pkg.ExpertShapes(lay.hidden, lay.inter)
    moe = pkg.B200MoE(0, shapes, lay.experts, experts=lay.experts, layers=1, top_k=lay.top_k,
                      shared_inter=lay.shared_inter, max_tokens=1024)
    for e in range(lay.experts):
        moe.load(0, e, e, lay.fields(e))
    banks = o.HostBanks(*lay.banks, slots=lay.experts, gu_rows=2 * lay.inter, gu_cols=lay.hidden,
                        dn_rows=lay.hidden, dn_cols=lay.inter)
    yield lay, moe, banks
    moe.close()


def _ids(rng, tokens, experts, top_k, pool=None):
    pool = np.arange(experts) if pool is None else np.asarray(pool)
    return np.stack([rng.choice(pool, top_k, replace=False) for _ in range(tokens)]).astype(np.int32)


def _run(moe, lay, xb, ids, w, odt, path, ids_dtype=torch.int32, x_f32=False):
    tokens = ids.shape[0]
    x = bf16_dev(xb)
    if x_f32:
        x = x.float()
    out = torch.empty((tokens, lay.hidden), dtype=odt, device=dev())
    req = pkg.MoEDeviceRequest(0, lay.hidden, lay.inter, lay.top_k, x, torch.from_numpy(ids).to(dev()).to(ids_dtype),
                               torch.from_numpy(w).to(dev()))
    moe.grouped_moe_staged(req, out, path=path)
    moe.sync_status()
    return out.float().cpu().numpy()


@pytest.mark.parametrize("tokens", [1, 5, 64, 129, 300])
def test_grouped_path_matches_cpu_path(layer, tokens):
    lay, moe, banks = layer
    rng = np.random.default_rng(tokens)
    xb = pkg.synth.make_x(tokens, tokens, lay.hidden)
    ids = _ids(rng, tokens, lay.experts, lay.top_k)
    w = rng.uniform(0.05, 0.5, ids.shape).astype(np.float32)
    got = _run(moe, lay, xb, ids, w, torch.float32, L.PATH_GROUPED)
    want = o.grouped_moe_reference_mt(banks, lay.hidden, lay.inter, pkg.synth.bf16_bits_to_f32(xb), lay.top_k,
                                      ids.reshape(-1), w.reshape(-1))
    assert rel_l2(got, want) < 1e-3            # f16 rounding of the intermediate activations: ~3e-4
    assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()


def test_hot_experts_take_several_passes_and_tiles(layer):
    """700 tokens over 12 experts: ~467 routes per expert, i.e. four passes of <= 128 rows with a ragged last
    pass."""
    lay, moe, banks = layer
    rng = np.random.default_rng(3)
    tokens = 700
    xb = pkg.synth.make_x(5, tokens, lay.hidden)
    ids = _ids(rng, tokens, lay.experts, lay.top_k, pool=[3, 9, 17, 64, 65, 100, 128, 200, 201, 254, 255, 0])
    w = rng.uniform(0.05, 0.5, ids.shape).astype(np.float32)
    want = o.grouped_moe_reference_mt(banks, lay.hidden, lay.inter, pkg.synth.bf16_bits_to_f32(xb), lay.top_k,
                                      ids.reshape(-1), w.reshape(-1))
    got = _run(moe, lay, xb, ids, w, torch.float32, L.PATH_AUTO)       # 5600 routes: AUTO takes the grouped GEMM
    assert rel_l2(got, want) < 1e-3
    got16 = _run(moe, lay, xb, ids, w, torch.bfloat16, L.PATH_AUTO, ids_dtype=torch.int64, x_f32=True)
    assert rel_l2(got16, want) < 1e-2
    assert np.abs(got16 - want).max() <= 2e-2 * np.abs(want).max()


def test_grouped_path_agrees_with_decode_path_and_is_deterministic(layer):
    lay, moe, banks = layer
    rng = np.random.default_rng(11)
    tokens = 200
    xb = pkg.synth.make_x(12, tokens, lay.hidden)
    ids = _ids(rng, tokens, lay.experts, lay.top_k)
    w = rng.uniform(0.05, 0.5, ids.shape).astype(np.float32)
    a = _run(moe, lay, xb, ids, w, torch.float32, L.PATH_GROUPED)
    b = _run(moe, lay, xb, ids, w, torch.float32, L.PATH_GROUPED)
    c = _run(moe, lay, xb, ids, w, torch.float32, L.PATH_GEMV)
    assert np.array_equal(a, b), "fixed summation order: two runs are bit-equal"
    assert rel_l2(a, c) < 1e-3


def test_experts_that_are_not_resident_contribute_nothing():
    lay = pkg.synth.make_layer(78, experts=32)
    shapes = pkg.ExpertShapes(lay.hidden, lay.inter)
    moe = pkg.B200MoE(0, shapes, 32, experts=32, layers=1, top_k=lay.top_k, shared_inter=0, max_tokens=512)
    resident = [e for e in range(32) if e % 3 != 1]
    for e in resident:
        moe.load(0, e, e, lay.fields(e))
    banks = o.HostBanks(*lay.banks, slots=32, gu_rows=2 * lay.inter, gu_cols=lay.hidden, dn_rows=lay.hidden,
                        dn_cols=lay.inter)
    rng = np.random.default_rng(5)
    tokens = 300
    xb = pkg.synth.make_x(9, tokens, lay.hidden)
    ids = _ids(rng, tokens, 32, lay.top_k)
    w = rng.uniform(0.05, 0.5, ids.shape).astype(np.float32)
    got = _run(moe, lay, xb, ids, w, torch.float32, L.PATH_GROUPED)
    w_res = np.where(np.isin(ids, resident), w, 0.0).astype(np.float32)
    want = o.grouped_moe_reference_mt(banks, lay.hidden, lay.inter, pkg.synth.bf16_bits_to_f32(xb), lay.top_k,
                                      ids.reshape(-1), w_res.reshape(-1))
    assert rel_l2(got, want) < 1e-3
    moe.close()


@pytest.mark.parametrize("tokens", [256, 300, 700])
def test_shared_expert_on_tensor_memory_path(layer, tokens):
    """256 tokens and more: the shared expert runs as two tcgen05 GEMMs (ic2 crosses as a bf16 hi + lo pair).
    Ragged last tile at 300 and 700 tokens."""
    lay, moe, banks = layer
    ol = o.Layer(lay.hidden, lay.inter, lay.experts, lay.top_k, lay.shared_inter, lay.gate_w, lay.sh_gate_up,
                 lay.sh_down, lay.sh_gate, banks)
    xb = pkg.synth.make_x(1000 + tokens, tokens, lay.hidden)
    xf = pkg.synth.bf16_bits_to_f32(xb)
    shared, gate = moe.shared_expert(bf16_dev(xb), bf16_dev(lay.sh_gate_up), bf16_dev(lay.sh_down), bf16_dev(lay.sh_gate))
    moe.sync_status()
    want = o.shared_expert(ol, xf)
    got = shared.cpu().numpy()
    assert rel_l2(got, want) <= 2e-4
    assert np.abs(got - want).max() <= 2e-4 * np.abs(want).max()
    g = o.bf16_gemm(xf, lay.sh_gate, tokens, 1, lay.hidden).reshape(-1)
    want_gate = 1.0 / (1.0 + np.exp(-g.astype(np.float64)))
    assert np.abs(gate.cpu().numpy() - want_gate).max() <= 1e-5


def test_whole_block_512_tokens_against_cpu_path(layer):
    """Router, grouped GEMM, tcgen05 shared expert and combine in one call, against the CPU checker's block."""
    lay, moe, banks = layer
    ol = o.Layer(lay.hidden, lay.inter, lay.experts, lay.top_k, lay.shared_inter, lay.gate_w, lay.sh_gate_up,
                 lay.sh_down, lay.sh_gate, banks)
    tokens = 512
    xb = pkg.synth.make_x(4243, tokens, lay.hidden)
    out = torch.empty((tokens, lay.hidden), dtype=torch.bfloat16, device=dev())
    ids = torch.empty((tokens, lay.top_k), dtype=torch.int32, device=dev())
    w = torch.empty((tokens, lay.top_k), dtype=torch.float32, device=dev())
    moe.moe_block(0, bf16_dev(xb), bf16_dev(lay.gate_w), bf16_dev(lay.sh_gate_up), bf16_dev(lay.sh_down),
                  bf16_dev(lay.sh_gate), out, ids_out=ids, weights_out=w)
    moe.sync_status()
    want, want_ids, want_w = o.moe_block(ol, pkg.synth.bf16_bits_to_f32(xb), threads=o.max_threads())
    assert np.array_equal(ids.cpu().numpy(), want_ids), "routed expert ids must be bit-exact"
    assert np.abs(w.cpu().numpy() - want_w).max() <= 1e-6
    got = out.float().cpu().numpy()
    assert rel_l2(got, want) <= 1e-2
    assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()


def test_grouped_path_second_layer_and_slot_offsets():
    """Two layers in one adapter, the second one's experts stored in reverse slot order: the grouped GEMM must find
    every expert's rows through the residency table (bank row = slot, not expert id)."""
    E2 = 32
    lays = [pkg.synth.make_layer(300 + l, experts=E2) for l in range(2)]
    shapes = pkg.ExpertShapes(lays[0].hidden, lays[0].inter)
    moe = pkg.B200MoE(0, shapes, 2 * E2, experts=E2, layers=2, top_k=lays[0].top_k, shared_inter=0, max_tokens=512)
    for e in range(E2):
        moe.load(0, e, e, lays[0].fields(e))
        moe.load(1, e, 2 * E2 - 1 - e, lays[1].fields(e))
    lay = lays[1]
    banks = o.HostBanks(*lay.banks, slots=E2, gu_rows=2 * lay.inter, gu_cols=lay.hidden, dn_rows=lay.hidden,
                        dn_cols=lay.inter)
    rng = np.random.default_rng(8)
    tokens = 400
    xb = pkg.synth.make_x(13, tokens, lay.hidden)
    ids = _ids(rng, tokens, E2, lay.top_k)
    w = rng.uniform(0.05, 0.5, ids.shape).astype(np.float32)
    out = torch.empty((tokens, lay.hidden), dtype=torch.float32, device=dev())
    req = pkg.MoEDeviceRequest(1, lay.hidden, lay.inter, lay.top_k, bf16_dev(xb), torch.from_numpy(ids).to(dev()),
                               torch.from_numpy(w).to(dev()))
    moe.grouped_moe_staged(req, out)          # 3200 routes: AUTO takes the grouped GEMM
    moe.sync_status()
    want = o.grouped_moe_reference_mt(banks, lay.hidden, lay.inter, pkg.synth.bf16_bits_to_f32(xb), lay.top_k,
                                      ids.reshape(-1), w.reshape(-1))
    assert rel_l2(out.cpu().numpy(), want) < 1e-3
    moe.close()
