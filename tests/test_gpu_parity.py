"""GPU parity: the CUDA path, called through the C ABI, against the CPU checker.

Bars (from the build's target):
* routed expert ids and the permutation: bit-exact (ties to the lowest expert index);
* router weights: within 1e-6 of the CPU path (tests/cudarc_forward.rs:253-254 of the reference);
* layer outputs: relative L2 <= 1e-2 and max |diff| <= 2e-2.
  The benchmark's synthetic experts (unit globals, block scales up to 1) produce outputs of magnitude
  ~1e4, where a bf16 ulp alone is 64; for those fixtures the max-abs bound is taken relative to
  max |reference| (`check_close`), the same normalisation the reference's kernel gate uses
  (python/ferrum_kernel/selftest.py:936).  The ABSOLUTE bound is asserted on layers whose row globals
  (2^-6 gate_up, 2^-10 down) give outputs of magnitude O(0.1 .. 1), as real checkpoints have
  (`check_close_abs`): decode, grouped GEMM, whole block and a four-layer stack.
"""
import importlib
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
pkg = importlib.import_module("ferrum-torrens_b200")
from oracle import oracle as o  # noqa: E402

REL_L2 = 1e-2
MAX_ABS_REL = 2e-2
HERE = os.path.dirname(os.path.abspath(__file__))


def dev():
    return torch.device("cuda:0")


def bf16_dev(bits: np.ndarray):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(dev()).view(torch.bfloat16)


def check_close(got: np.ndarray, want: np.ndarray, rel_l2=REL_L2, max_abs_rel=MAX_ABS_REL):
    denom = np.linalg.norm(want)
    rel = np.linalg.norm(got - want) / max(denom, 1e-30)
    mx = np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)
    assert rel <= rel_l2, f"relative L2 {rel:.3e}"
    assert mx <= max_abs_rel, f"max abs (relative to max |ref|) {mx:.3e}"
    return rel, mx


MAX_ABS = 2e-2


def check_close_abs(got: np.ndarray, want: np.ndarray, rel_l2=REL_L2, max_abs=MAX_ABS):
    """The stated bar as written: relative L2 and ABSOLUTE max |diff|."""
    rel = np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)
    mx = np.abs(got - want).max()
    assert rel <= rel_l2, f"relative L2 {rel:.3e}"
    assert mx <= max_abs, f"max abs {mx:.3e}"
    return rel, mx


def oracle_layer(lay):
    banks = o.HostBanks(*lay.banks, slots=lay.experts, gu_rows=2 * lay.inter, gu_cols=lay.hidden,
                        dn_rows=lay.hidden, dn_cols=lay.inter)
    return o.Layer(lay.hidden, lay.inter, lay.experts, lay.top_k, lay.shared_inter, lay.gate_w, lay.sh_gate_up,
                   lay.sh_down, lay.sh_gate, banks)


def make_moe(lay, max_tokens=256, layers=1, slots=None):
    moe = pkg.B200MoE(0, pkg.ExpertShapes(lay.hidden, lay.inter), slots or lay.experts * layers, experts=lay.experts,
                      layers=layers, top_k=lay.top_k, shared_inter=lay.shared_inter, max_tokens=max_tokens)
    return moe


def load_all(moe, lay, layer=0, slot0=0):
    for e in range(lay.experts):
        moe.load(layer, e, slot0 + e, lay.fields(e))


# ------------------------------------------------------------------ small layer shared by many tests
@pytest.fixture(scope="module")
def small():
    lay = pkg.synth.make_layer(11, hidden=256, inter=128, experts=32, top_k=4, shared_inter=64)
    moe = make_moe(lay, max_tokens=4096)
    load_all(moe, lay)
    yield lay, moe, oracle_layer(lay)
    moe.close()


@pytest.fixture(scope="module")
def full():
    """The benchmark layer: hidden 2048, inter 512, 256 experts, top-8, shared 512."""
    lay = pkg.synth.make_layer(2024)
    moe = make_moe(lay, max_tokens=2048)
    load_all(moe, lay)
    yield lay, moe, oracle_layer(lay)
    moe.close()


# ------------------------------------------------------------------ router
@pytest.mark.parametrize("tokens", [1, 3, 8, 33, 300])
def test_router_ids_bit_exact_small(small, tokens):
    lay, moe, ol = small
    xb = pkg.synth.make_x(tokens, tokens, lay.hidden)
    ids, w = moe.router(bf16_dev(xb), bf16_dev(lay.gate_w))
    want_ids, want_w = o.router(ol, pkg.synth.bf16_bits_to_f32(xb))
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    assert np.abs(w.cpu().numpy() - want_w).max() <= 1e-6
    assert np.array_equal(w.cpu().numpy(), want_w), "same operations in the same order: weights are bit-equal too"


@pytest.mark.parametrize("tokens", [1, 16, 64, 512, 1100])
def test_router_ids_bit_exact_full(full, tokens):
    lay, moe, ol = full
    xb = pkg.synth.make_x(100 + tokens, tokens, lay.hidden)
    ids, w = moe.router(bf16_dev(xb), bf16_dev(lay.gate_w))
    want_ids, want_w = o.router(ol, pkg.synth.bf16_bits_to_f32(xb))
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    assert np.abs(w.cpu().numpy() - want_w).max() <= 1e-6


def test_router_ids_bit_exact_at_4200_tokens():
    """Batches of 4096 tokens and more take a kernel of their own (32 chains per thread); 4200 tokens leave a
    ragged last tile of eight.  Ids and weights equal the CPU path's bit for bit."""
    lay = pkg.synth.make_layer(31, hidden=2048, inter=512, experts=256, top_k=8, shared_inter=512)
    moe = pkg.B200MoE(0, pkg.ExpertShapes(2048, 512), 1, experts=256, layers=1, top_k=8, shared_inter=0, max_tokens=4200)
    ol = oracle_layer(lay)
    xb = pkg.synth.make_x(4242, 4200, lay.hidden)
    ids, w = moe.router(bf16_dev(xb), bf16_dev(lay.gate_w))
    want_ids, want_w = o.router(ol, pkg.synth.bf16_bits_to_f32(xb))
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    assert np.array_equal(w.cpu().numpy(), want_w)
    moe.close()


def test_router_ties_take_the_lowest_index(small):
    lay, moe, _ = small
    e = lay.experts
    logits = np.zeros((3, e), np.float32)
    logits[1, [5, 9, 20]] = 2.0          # three-way tie on top, the rest tie at zero
    logits[2] = np.linspace(1, 0, e)     # strictly descending: ids 0..k-1
    ids, w = moe.fused_topk_softmax(torch.from_numpy(logits).to(dev()))
    ids = ids.cpu().numpy()
    assert ids[0].tolist() == [0, 1, 2, 3]
    assert ids[1].tolist() == [5, 9, 20, 0]
    assert ids[2].tolist() == [0, 1, 2, 3]
    want_ids, want_w = o.topk_renorm(o.softmax_rows(logits), lay.top_k)
    assert np.array_equal(ids, want_ids)
    assert np.array_equal(w.cpu().numpy(), want_w)
    assert np.allclose(w.cpu().numpy().sum(1), 1.0, atol=1e-6)


def test_router_from_logits_matches_reference_topk_case(small):
    """forward.rs:1229-1236 in probability form: p = [.5, .2, .3] -> ids [0, 2]."""
    lay, moe, _ = small
    logits = np.full((1, lay.experts), -30.0, np.float32)
    logits[0, :3] = np.log(np.array([0.5, 0.2, 0.3], np.float32))
    ids, w = moe.fused_topk_softmax(torch.from_numpy(logits).to(dev()))
    assert ids.cpu().numpy()[0, :2].tolist() == [0, 2]


# ------------------------------------------------------------------ permutation
CSR_CASES = [([2, 0, 2, 0, 0, 1], 3), ([0] * 37, 8), ([7], 8), ([3, 3, 3, 1, 1, 2, 2, 2, 2], 8), ([5, 5, 5, 5], 8)]


@pytest.mark.parametrize("routes,bins", CSR_CASES)
def test_csr_reference_cases(small, routes, bins):
    """cuda_moe.rs:2718-2720 and the fixed cases of :2764-2769."""
    _, moe, _ = small
    seg, idx, badf = moe.csr_build(torch.tensor(routes, dtype=torch.int32, device=dev()), bins)
    want_seg, want_idx = o.build_grouped_csr(routes, bins)
    assert seg.cpu().numpy().tolist() == want_seg.tolist()
    assert idx.cpu().numpy().tolist() == want_idx.tolist()
    assert badf == 0
    if routes == [2, 0, 2, 0, 0, 1]:
        assert want_seg.tolist() == [0, 3, 4, 6] and want_idx.tolist() == [1, 3, 4, 5, 0, 2]


@pytest.mark.parametrize("n,bins", [(1, 8), (2, 8), (7, 8), (33, 8), (128, 8), (1025, 8), (2048, 256), (2049, 256),
                                    (16384, 256), (13001, 32), (12000, 300), (4097, 1)])
def test_csr_random_matches_host(small, n, bins):
    """xorshift-seeded cases as in cuda_moe.rs:2752-2772, plus the sizes of both builds: one CTA (at most 2048
    routes) and several CTAs, with 1, 32, 256 and 300 bins."""
    _, moe, _ = small
    seed = 0x2545F4914F6CDD1D
    vals = []
    for _ in range(n):
        seed ^= (seed << 13) & 0xFFFFFFFFFFFFFFFF
        seed ^= seed >> 7
        seed ^= (seed << 17) & 0xFFFFFFFFFFFFFFFF
        vals.append(seed % bins)
    seg, idx, badf = moe.csr_build(torch.tensor(vals, dtype=torch.int32, device=dev()), bins)
    want_seg, want_idx = o.build_grouped_csr(vals, bins)
    assert np.array_equal(seg.cpu().numpy(), want_seg)
    assert np.array_equal(idx.cpu().numpy(), want_idx)
    assert badf == 0
    # size-independent properties: a complete permutation, sorted by bin, ascending inside a bin
    got = idx.cpu().numpy()
    assert np.array_equal(np.sort(got), np.arange(n))
    b = np.asarray(vals)[got]
    assert (np.diff(b) >= 0).all()
    assert all((np.diff(got[seg_a:seg_b]) > 0).all() for seg_a, seg_b in zip(want_seg[:-1], want_seg[1:]))


def test_csr_flags_slots_outside_the_bank(small):
    _, moe, _ = small
    for routes in ([-1, 0], [3], [0, 1, 2] * 1000 + [3], [2] * 5000 + [-7] + [1] * 4000):
        seg, idx, badf = moe.csr_build(torch.tensor(routes, dtype=torch.int32, device=dev()), 3)
        assert badf == 1
        good = [i for i, b in enumerate(routes) if 0 <= b < 3]
        assert int(seg[3]) == len(good), "the routes inside the bank are still bucketed"


# ------------------------------------------------------------------ routed half, known answers
H16 = 16
F16 = {0.5: 0x3800, 1.0: 0x3C00, -1.0: 0xBC00, 4.0: 0x4400}


def slab(rows, cols, packed, scale, glob):
    g = np.tile(np.array([F16[glob] & 0xFF, F16[glob] >> 8], np.uint8), rows)
    return [np.full(rows * cols // 2, packed, np.uint8), np.full(rows * cols // 16, scale, np.uint8), g]


def tiny_moe(gus, dns, h=H16, i=H16, top_k=1):
    moe = pkg.B200MoE(0, pkg.ExpertShapes(h, i), len(gus), experts=len(gus), layers=1, top_k=top_k, shared_inter=16,
                      max_tokens=8)
    for s, (g, d) in enumerate(zip(gus, dns)):
        moe.load(0, s, s, [*g, *d])
    return moe


def silu(v):
    v = np.float32(v)
    return float(v / (np.float32(1.0) + np.exp(-v, dtype=np.float32)))


def run_host(moe, h, i, x, top_k, routes, weights):
    out = np.full(len(x) // h * h, 7.0, np.float32)
    moe.grouped_moe(pkg.MoEGroup(h, i, np.asarray(x, np.float32), top_k, np.asarray(routes, np.int32),
                                 np.asarray(weights, np.float32)), out)
    return out


def test_hand_computed_case_matches():
    """expert_kernel.rs:744-790"""
    moe = tiny_moe([slab(32, 16, 0x10, 0x38, 1.0)], [slab(16, 16, 0x10, 0x38, 1.0)])
    out = run_host(moe, 16, 16, np.ones(16), 1, [0], [0.5])
    want = 0.5 * (8.0 * 0.5 * silu(4.0) * 4.0)
    assert np.allclose(out, want, rtol=1e-4)
    moe.close()


def test_non_resident_route_contributes_nothing():
    """expert_kernel.rs:851-888"""
    moe = tiny_moe([slab(32, 16, 0x10, 0x38, 1.0)], [slab(16, 16, 0x10, 0x38, 1.0)])
    out = run_host(moe, 16, 16, np.ones(16), 1, [-1], [1.0])
    assert np.array_equal(out, np.zeros(16, np.float32))
    moe.close()


def test_slot_selects_its_own_expert_and_cancelling_routes():
    """expert_kernel.rs:890-979 and :792-849"""
    moe = tiny_moe([slab(32, 16, 0x01, 0x38, 1.0), slab(32, 16, 0x10, 0x38, 1.0)],
                   [slab(16, 16, 0x01, 0x38, 1.0), slab(16, 16, 0x10, 0x38, 1.0)])
    x = np.array([1.0 if k % 2 == 0 else 2.0 for k in range(16)], np.float32)
    assert np.allclose(run_host(moe, 16, 16, x, 1, [0], [1.0]), 8.0 * 0.5 * silu(4.0) * 4.0, rtol=1e-4)
    assert np.allclose(run_host(moe, 16, 16, x, 1, [1], [1.0]), 8.0 * 0.5 * silu(8.0) * 8.0, rtol=1e-4)
    moe.close()
    moe = tiny_moe([slab(32, 16, 0x10, 0x38, 1.0)] * 2, [slab(16, 16, 0x10, 0x38, 1.0), slab(16, 16, 0x10, 0x38, -1.0)],
                   top_k=2)
    out = run_host(moe, 16, 16, np.ones(16), 2, [0, 1], [1.0, 1.0])
    assert np.abs(out).max() <= 1e-4 * 2 * 4.0 * silu(4.0) * 4.0
    moe.close()


def test_global_and_block_scales():
    """expert_kernel.rs:981-1023 and :1025-1075"""
    moe = tiny_moe([slab(32, 16, 0x10, 0x38, 4.0)], [slab(16, 16, 0x10, 0x38, 0.5)])
    out = run_host(moe, 16, 16, np.ones(16), 1, [0], [1.0])
    ic2 = silu(16.0) * 16.0
    assert np.allclose(out, 8.0 * 0.5 * ic2 * 0.5, rtol=1e-4)
    moe.close()
    s1 = slab(32, 32, 0x10, 0x40, 1.0)
    s1[1] = np.array([0x40 if b % 2 == 1 else 0x38 for b in range(32 * 32 // 16)], np.uint8)
    moe = tiny_moe([slab(32, 32, 0x10, 0x38, 1.0), s1], [slab(32, 16, 0x10, 0x38, 1.0)] * 2, h=32, i=16)
    out = run_host(moe, 32, 16, np.ones(32), 1, [1], [1.0])
    ic2 = silu(12.0) * 12.0
    assert np.allclose(out, 8.0 * 0.5 * ic2, rtol=1e-4)
    moe.close()


def test_shape_and_slot_mismatches_are_errors():
    """expert_kernel.rs:1141-1181; the adapter validates before any launch (cuda_moe.rs:959-1003)."""
    moe = tiny_moe([slab(32, 16, 0x10, 0x38, 1.0)], [slab(16, 16, 0x10, 0x38, 1.0)])
    with pytest.raises(pkg.MoEError) as e:
        run_host(moe, 32, 16, np.ones(16), 1, [0], [1.0])
    assert e.value.kind == "Bad"
    with pytest.raises(pkg.MoEError) as e:
        run_host(moe, 16, 16, np.ones(16), 1, [5], [1.0])
    assert e.value.kind == "SlotOutOfRange" and "slot 5 out of range (capacity 1)" in str(e.value)
    with pytest.raises(pkg.MoEError) as e:
        run_host(moe, 16, 16, np.ones(16), 1, [0, 0], [1.0, 1.0])
    assert e.value.kind == "Bad"
    with pytest.raises(pkg.MoEError) as e:
        moe.load(0, 0, 3, [*slab(32, 16, 0, 0, 1.0), *slab(16, 16, 0, 0, 1.0)])
    assert e.value.kind == "SlotOutOfRange"
    with pytest.raises(pkg.MoEError) as e:
        moe.load(0, 0, 0, [*slab(32, 16, 0, 0, 1.0), *slab(16, 32, 0, 0, 1.0)])
    assert e.value.kind == "Bad"
    moe.close()


# ------------------------------------------------------------------ routed half vs the reference's torch oracle
def _golden():
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    return mg, np.load(os.path.join(HERE, "golden", "ref_torch_oracle.npz"))


@pytest.mark.parametrize("case", [0, 1, 2])
def test_routed_half_matches_reference_fixtures(case):
    mg, G = _golden()
    label, tokens, hidden, inter, slots, top_k, seed = mg.LARGE_CASES[case]
    x, gu, dn, slot, weight = mg.golden_inputs(tokens, hidden, inter, slots, top_k, seed)
    moe = pkg.B200MoE(0, pkg.ExpertShapes(hidden, inter), slots, experts=slots, layers=1, top_k=top_k,
                      shared_inter=16, max_tokens=16)
    for s in range(slots):
        moe.load(0, s, s, [gu[0][s], gu[1][s], gu[2][s].view(np.uint8), dn[0][s], dn[1][s], dn[2][s].view(np.uint8)])
    out = run_host(moe, hidden, inter, x.reshape(-1), top_k, slot, weight).reshape(tokens, hidden)
    want = G[f"{label}/want"]
    banks = o.HostBanks(gu[0], gu[1], gu[2].view(np.uint8), dn[0], dn[1], dn[2].view(np.uint8), slots, 2 * inter,
                        hidden, hidden, inter)
    mine, abs_sum = o.grouped_moe_reference(banks, hidden, inter, x, top_k, slot, weight, want_abs_sum=True)
    # the reference's own yardstick: error against the size of the summed terms.  The per-route f32
    # kernels differ from the host sums only by association (2e-5); the tensor-core decode kernels round
    # ic2 to bf16 like the reference's device path, whose gate is 4 * 2^-9 of the term magnitude
    # (tests/cuda_moe_matches_reference.rs:43-53)
    tol = 4.0 / 512.0 if (hidden, inter) == (2048, 512) else 2e-5
    assert np.abs(out - want).max() <= tol * abs_sum.max()
    assert np.abs(out - mine).max() <= tol * abs_sum.max()
    moe.close()


# ------------------------------------------------------------------ device hand-offs on a small layer
@pytest.mark.parametrize("tokens", [1, 5, 64, 257])
@pytest.mark.parametrize("xdt,odt", [("bf16", "bf16"), ("f32", "f32")])
def test_staged_call_matches_cpu_path(small, tokens, xdt, odt):
    lay, moe, ol = small
    rng = np.random.default_rng(tokens)
    xb = pkg.synth.make_x(tokens + 7, tokens, lay.hidden)
    xf = pkg.synth.bf16_bits_to_f32(xb)
    ids = np.stack([rng.permutation(lay.experts)[:lay.top_k] for _ in range(tokens)]).astype(np.int32)
    w = rng.uniform(0.05, 0.5, (tokens, lay.top_k)).astype(np.float32)
    x_d = bf16_dev(xb) if xdt == "bf16" else torch.from_numpy(xf).to(dev())
    out = torch.empty((tokens, lay.hidden), dtype=torch.bfloat16 if odt == "bf16" else torch.float32, device=dev())
    before = moe.steps()
    req = pkg.MoEDeviceRequest(0, lay.hidden, lay.inter, lay.top_k, x_d, torch.from_numpy(ids).to(dev()),
                               torch.from_numpy(w).to(dev()))
    moe.grouped_moe_staged(req, out)
    torch.cuda.synchronize()
    assert moe.steps() == before + 1
    want = o.grouped_moe_reference_mt(ol.banks, lay.hidden, lay.inter, xf, lay.top_k, ids.reshape(-1), w.reshape(-1))
    check_close(out.float().cpu().numpy(), want)
    # i64 ids are accepted too (cuda_moe.rs:67-86)
    req64 = pkg.MoEDeviceRequest(0, lay.hidden, lay.inter, lay.top_k, x_d, torch.from_numpy(ids.astype(np.int64)).to(dev()),
                                 torch.from_numpy(w).to(dev()))
    out2 = torch.empty_like(out)
    moe.grouped_moe_staged(req64, out2)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)


def test_device_group_with_host_routes_and_missing_slots(small):
    lay, moe, ol = small
    tokens = 6
    rng = np.random.default_rng(5)
    xb = pkg.synth.make_x(55, tokens, lay.hidden)
    xf = pkg.synth.bf16_bits_to_f32(xb)
    routes = rng.integers(-1, lay.experts, tokens * lay.top_k).astype(np.int32)
    routes[:3] = -1
    w = rng.uniform(0.05, 0.5, tokens * lay.top_k).astype(np.float32)
    out = torch.empty((tokens, lay.hidden), dtype=torch.float32, device=dev())
    moe.grouped_moe_dev(lay.hidden, lay.inter, lay.top_k, bf16_dev(xb), routes, torch.from_numpy(w).to(dev()), out)
    torch.cuda.synchronize()
    want = o.grouped_moe_reference(ol.banks, lay.hidden, lay.inter, xf, lay.top_k, routes, w)
    check_close(out.cpu().numpy(), want)
    with pytest.raises(pkg.MoEError) as e:
        bad_routes = routes.copy()
        bad_routes[0] = lay.experts + 3
        moe.grouped_moe_dev(lay.hidden, lay.inter, lay.top_k, bf16_dev(xb), bad_routes, torch.from_numpy(w).to(dev()), out)
    assert e.value.kind == "SlotOutOfRange"


def test_shared_expert_and_combine(small):
    lay, moe, ol = small
    tokens = 19
    xb = pkg.synth.make_x(9, tokens, lay.hidden)
    xf = pkg.synth.bf16_bits_to_f32(xb)
    shared, gate = moe.shared_expert(bf16_dev(xb), bf16_dev(lay.sh_gate_up), bf16_dev(lay.sh_down), bf16_dev(lay.sh_gate))
    torch.cuda.synchronize()
    want = o.shared_expert(ol, xf)
    check_close(shared.cpu().numpy(), want, rel_l2=2e-4, max_abs_rel=2e-4)
    g = o.bf16_gemm(xf, lay.sh_gate, tokens, 1, lay.hidden).reshape(-1)
    want_gate = np.array([o.sigmoid(float(v)) for v in g], np.float32)
    assert np.abs(gate.cpu().numpy() - want_gate).max() <= 1e-5
    routed = torch.randn((tokens, lay.hidden), device=dev())
    out = torch.empty((tokens, lay.hidden), dtype=torch.float32, device=dev())
    moe.combine(routed, shared, gate, out)
    torch.cuda.synchronize()
    assert torch.allclose(out, shared * gate[:, None] + routed, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("tokens", [1, 7, 64, 300])
def test_whole_block_small(small, tokens):
    lay, moe, ol = small
    xb = pkg.synth.make_x(1000 + tokens, tokens, lay.hidden)
    out = torch.empty((tokens, lay.hidden), dtype=torch.bfloat16, device=dev())
    ids = torch.empty((tokens, lay.top_k), dtype=torch.int32, device=dev())
    w = torch.empty((tokens, lay.top_k), dtype=torch.float32, device=dev())
    moe.moe_block(0, bf16_dev(xb), bf16_dev(lay.gate_w), bf16_dev(lay.sh_gate_up), bf16_dev(lay.sh_down),
                  bf16_dev(lay.sh_gate), out, ids_out=ids, weights_out=w)
    torch.cuda.synchronize()
    want, want_ids, want_w = o.moe_block(ol, pkg.synth.bf16_bits_to_f32(xb), threads=o.max_threads())
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    assert np.abs(w.cpu().numpy() - want_w).max() <= 1e-6
    check_close(out.float().cpu().numpy(), want)


# ------------------------------------------------------------------ the benchmark layer (configs 1 and 2)
@pytest.mark.parametrize("tokens", [16, 1, 8, 64])
def test_whole_block_full_size(full, tokens):
    """Config 1 (T=16) and the decode sizes of config 2 at hidden 2048 / 256 experts / top-8."""
    lay, moe, ol = full
    xb = pkg.synth.make_x(4242 + tokens, tokens, lay.hidden)
    out = torch.empty((tokens, lay.hidden), dtype=torch.bfloat16, device=dev())
    ids = torch.empty((tokens, lay.top_k), dtype=torch.int32, device=dev())
    w = torch.empty((tokens, lay.top_k), dtype=torch.float32, device=dev())
    moe.moe_block(0, bf16_dev(xb), bf16_dev(lay.gate_w), bf16_dev(lay.sh_gate_up), bf16_dev(lay.sh_down),
                  bf16_dev(lay.sh_gate), out, ids_out=ids, weights_out=w)
    moe.sync_status()
    want, want_ids, want_w = o.moe_block(ol, pkg.synth.bf16_bits_to_f32(xb), threads=o.max_threads())
    assert np.array_equal(ids.cpu().numpy(), want_ids), "routed expert ids must be bit-exact"
    assert np.abs(w.cpu().numpy() - want_w).max() <= 1e-6
    check_close(out.float().cpu().numpy(), want)
    # permutation of these routes: bit-exact against the host CSR
    seg, idx, badf = moe.csr_build(ids.reshape(-1), lay.experts)
    want_seg, want_idx = o.build_grouped_csr(want_ids.reshape(-1), lay.experts)
    assert np.array_equal(seg.cpu().numpy(), want_seg) and np.array_equal(idx.cpu().numpy(), want_idx) and badf == 0


def test_linearity_in_route_weights_full_size(full):
    """A size-independent property of the routed half: doubling the route weights doubles the sum."""
    lay, moe, _ = full
    tokens = 32
    xb = pkg.synth.make_x(77, tokens, lay.hidden)
    rng = np.random.default_rng(3)
    ids = np.stack([rng.permutation(lay.experts)[:lay.top_k] for _ in range(tokens)]).astype(np.int32)
    w = rng.uniform(0.05, 0.5, (tokens, lay.top_k)).astype(np.float32)
    outs = []
    for scale in (1.0, 2.0):
        out = torch.empty((tokens, lay.hidden), dtype=torch.float32, device=dev())
        req = pkg.MoEDeviceRequest(0, lay.hidden, lay.inter, lay.top_k, bf16_dev(xb), torch.from_numpy(ids).to(dev()),
                                   torch.from_numpy(w * np.float32(scale)).to(dev()))
        moe.grouped_moe_staged(req, out)
        torch.cuda.synchronize()
        outs.append(out.cpu().numpy())
    assert np.array_equal(outs[1], 2.0 * outs[0])


# ------------------------------------------------------------------ slot store behaviour
def test_slot_store_release_rehydrate_and_residency():
    lay = pkg.synth.make_layer(5, hidden=64, inter=32, experts=4, top_k=2, shared_inter=16)
    moe = make_moe(lay, max_tokens=8, layers=2, slots=8)
    assert moe.slots() == 8 and moe.banks_resident()
    ptrs = moe.bank_ptrs()
    assert len(ptrs) == 6 and all(p % 256 == 0 for p in ptrs)
    load_all(moe, lay, layer=1, slot0=4)
    assert moe.bank_ptrs() == ptrs, "bank addresses are stable for the adapter's life"
    assert moe.slot_of(1, 2) == 6 and moe.slot_of(0, 2) == -1
    # a layer whose experts are not resident contributes nothing (slot -1)
    xb = pkg.synth.make_x(1, 3, 64)
    ids = torch.tensor([[0, 1], [2, 3], [1, 2]], dtype=torch.int32, device=dev())
    w = torch.full((3, 2), 0.5, device=dev())
    out = torch.empty((3, 64), dtype=torch.float32, device=dev())
    moe.grouped_moe_staged(pkg.MoEDeviceRequest(0, 64, 32, 2, bf16_dev(xb), ids, w), out)
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0
    moe.grouped_moe_staged(pkg.MoEDeviceRequest(1, 64, 32, 2, bf16_dev(xb), ids, w), out)
    torch.cuda.synchronize()
    assert float(out.abs().max()) > 0.0
    # loading another expert into an occupied slot displaces the occupant
    moe.load(0, 0, 4, lay.fields(0))
    assert moe.slot_of(0, 0) == 4 and moe.slot_of(1, 0) == -1
    moe.reset_staging()
    assert moe.slot_of(0, 0) == -1
    moe.release_banks()
    assert not moe.banks_resident()
    with pytest.raises(pkg.MoEError):
        moe.grouped_moe_staged(pkg.MoEDeviceRequest(1, 64, 32, 2, bf16_dev(xb), ids, w), out)
    moe.rehydrate_banks()
    assert moe.banks_resident() and moe.slot_of(1, 2) == -1
    assert moe.begin_staged(pkg.MoEDeviceRequest(1, 64, 32, 2, bf16_dev(xb), ids, w)) is None
    assert moe.staged_route_cap() == 8 * 2
    moe.close()


def test_host_plan_executor_matches_staged_executor():
    """run_experts / CachedExperts (src/application/run_experts.rs): host plan with a slot cache that
    holds every expert gives the same sum as the device-staged path."""
    lay = pkg.synth.make_layer(6, hidden=64, inter=32, experts=8, top_k=2, shared_inter=16)

    class Source:
        def slab(self, layer, expert, part):
            f = lay.fields(expert)
            return f[:3] if part == "GateUp" else f[3:]

    moe = pkg.B200MoE(0, pkg.ExpertShapes(64, 32), 8, source=Source(), experts=8, layers=1, top_k=2, shared_inter=16,
                      max_tokens=8)
    tokens = 5
    xb = pkg.synth.make_x(2, tokens, 64)
    xf = pkg.synth.bf16_bits_to_f32(xb)
    rng = np.random.default_rng(1)
    experts = np.stack([rng.permutation(8)[:2] for _ in range(tokens)]).astype(np.uint32)
    w = rng.uniform(0.1, 0.6, (tokens, 2)).astype(np.float32)
    out = np.zeros(tokens * 64, np.float32)
    cache = pkg.ExpertCache(moe)
    pkg.run_experts(cache, moe, moe, 0, 64, 32, 2, xf, experts, w, out)
    ol = oracle_layer(lay)
    want = o.grouped_moe_reference(ol.banks, 64, 32, xf, 2, experts.astype(np.int32).reshape(-1), w.reshape(-1))
    check_close(out.reshape(tokens, 64), want)
    ex = pkg.CachedExperts(moe, staged=True)
    out_d = torch.empty((tokens, 64), dtype=torch.float32, device=dev())
    req = pkg.MoEDeviceRequest(0, 64, 32, 2, bf16_dev(xb), torch.from_numpy(experts.astype(np.int32)).to(dev()),
                               torch.from_numpy(w).to(dev()))
    ex.execute_device(req, out_d)
    torch.cuda.synchronize()
    assert ex.steps() == 1
    assert np.array_equal(out_d.cpu().numpy().reshape(-1), out)
    ex2 = pkg.CachedExperts(moe, staged=False)
    out_h = torch.empty((tokens, 64), dtype=torch.float32, device=dev())
    ex2.execute_device(req, out_h)
    torch.cuda.synchronize()
    assert np.array_equal(out_h.cpu().numpy().reshape(-1), out)
    moe.close()


# ------------------------------------------------------------------ grouped decode path (plan + TMA + mma.sync)
@pytest.mark.parametrize("tokens,hot", [(1, 0), (8, 0), (64, 0), (40, 3), (200, 5)])
def test_decode_path_with_skew_and_missing_slots(full, tokens, hot):
    """Routes concentrated on a few experts (groups of more than 8 routes per slot are cut into
    several), some experts not resident (-1 contributes nothing): the grouped decode path, the
    per-route scalar path and the CPU path agree."""
    lay, moe, ol = full
    rng = np.random.default_rng(100 + tokens)
    xb = pkg.synth.make_x(900 + tokens, tokens, lay.hidden)
    xf = pkg.synth.bf16_bits_to_f32(xb)
    ids = np.stack([rng.permutation(lay.experts)[:lay.top_k] for _ in range(tokens)]).astype(np.int32)
    if hot:
        # every token also routes to the same `hot` experts
        ids[:, :hot] = np.arange(hot, dtype=np.int32)[None, :] + 7
        for t in range(tokens):  # keep ids distinct per token
            rest = [e for e in rng.permutation(lay.experts) if e not in ids[t, :hot]][:lay.top_k - hot]
            ids[t, hot:] = rest
    w = rng.uniform(0.05, 0.5, (tokens, lay.top_k)).astype(np.float32)
    routes = ids.reshape(-1).copy()
    if tokens > 1:
        routes[rng.integers(0, routes.size, max(1, routes.size // 16))] = -1
    outs = {}
    for name, path in (("mma", pkg._lib.PATH_GEMV), ("scalar", pkg._lib.PATH_SCALAR)):
        out = torch.empty((tokens, lay.hidden), dtype=torch.float32, device=dev())
        # routes carry slot ids here (slot = expert for this layer), -1 = not resident
        moe.grouped_moe_dev(lay.hidden, lay.inter, lay.top_k, bf16_dev(xb), routes, torch.from_numpy(w).to(dev()), out) \
            if path == pkg._lib.PATH_GEMV else None
        if path == pkg._lib.PATH_SCALAR:
            ids_dev = torch.from_numpy(np.where(routes < 0, lay.experts + 5, routes).astype(np.int32).reshape(tokens, -1)).to(dev())
            req = pkg.MoEDeviceRequest(0, lay.hidden, lay.inter, lay.top_k, bf16_dev(xb), ids_dev, torch.from_numpy(w).to(dev()))
            moe.grouped_moe_staged(req, out, path=path)
        torch.cuda.synchronize()
        outs[name] = out.cpu().numpy()
    try:
        moe.sync_status()
    except pkg.MoEError as e:  # the out-of-layer ids used above to express "not resident" raise the id flag
        assert "expert id" in str(e)
    want = o.grouped_moe_reference_mt(ol.banks, lay.hidden, lay.inter, xf, lay.top_k, routes, w.reshape(-1))
    check_close(outs["scalar"], want, rel_l2=1e-5, max_abs_rel=1e-5)
    check_close(outs["mma"], want)   # ic2 is rounded to bf16 on this path
    rel = np.linalg.norm(outs["mma"] - want) / np.linalg.norm(want)
    assert rel < 5e-3, rel


def test_decode_path_reports_no_async_errors(full):
    lay, moe, _ = full
    tokens = 4
    xb = pkg.synth.make_x(1, tokens, lay.hidden)
    ids = torch.arange(tokens * lay.top_k, dtype=torch.int32, device=dev()).reshape(tokens, lay.top_k)
    w = torch.full((tokens, lay.top_k), 0.125, device=dev())
    out = torch.empty((tokens, lay.hidden), dtype=torch.bfloat16, device=dev())
    moe.grouped_moe_staged(pkg.MoEDeviceRequest(0, lay.hidden, lay.inter, lay.top_k, bf16_dev(xb), ids, w), out)
    moe.sync_status()
    bad_ids = ids.clone()
    bad_ids[0, 0] = lay.experts
    moe.grouped_moe_staged(pkg.MoEDeviceRequest(0, lay.hidden, lay.inter, lay.top_k, bf16_dev(xb), bad_ids, w), out)
    with pytest.raises(pkg.MoEError, match="expert id"):
        moe.sync_status()
    moe.sync_status()


# ------------------------------------------------------------------ large batches (prefill sizes)
def _zipf_ids(rng, tokens, experts, top_k, alpha):
    """Skewed routing: expert popularity ~ rank^-alpha, top_k distinct experts per token."""
    p = (np.arange(1, experts + 1) ** -alpha)
    p /= p.sum()
    p = p[rng.permutation(experts)]
    return np.stack([rng.choice(experts, top_k, replace=False, p=p) for _ in range(tokens)]).astype(np.int32)


@pytest.mark.parametrize("tokens", [300, 512])
def test_large_batch_path_matches_cpu_path(full, tokens):
    """More than 2048 routes take the tcgen05 grouped GEMM: CSR buckets cut into passes of at most 128 sorted
    rows per expert (Zipf 1.1 skew: some experts get no token, hot ones several passes)."""
    lay, moe, ol = full
    rng = np.random.default_rng(tokens)
    xb = pkg.synth.make_x(31 + tokens, tokens, lay.hidden)
    xf = pkg.synth.bf16_bits_to_f32(xb)
    ids = _zipf_ids(rng, tokens, lay.experts, lay.top_k, 1.1)
    w = rng.uniform(0.05, 0.5, (tokens, lay.top_k)).astype(np.float32)
    out = torch.empty((tokens, lay.hidden), dtype=torch.float32, device=dev())
    req = pkg.MoEDeviceRequest(0, lay.hidden, lay.inter, lay.top_k, bf16_dev(xb), torch.from_numpy(ids).to(dev()),
                               torch.from_numpy(w).to(dev()))
    moe.grouped_moe_staged(req, out)
    moe.sync_status()
    want = o.grouped_moe_reference_mt(ol.banks, lay.hidden, lay.inter, xf, lay.top_k, ids.reshape(-1), w.reshape(-1))
    rel, _ = check_close(out.cpu().numpy(), want)
    assert rel < 1e-3
    counts = np.bincount(ids.reshape(-1), minlength=lay.experts)
    assert counts.max() > 16, "the case must cut at least one expert into several groups"


def test_prefill_2048_tokens_paths_agree_and_block_properties(full):
    """T = 2048 (config 3 size): the grouped tensor-core path against the per-route scalar path on the same
    routes, and the whole block's routed ids against the CPU router."""
    lay, moe, ol = full
    tokens = 2048
    rng = np.random.default_rng(7)
    xb = pkg.synth.make_x(2048, tokens, lay.hidden)
    ids = _zipf_ids(rng, tokens, lay.experts, lay.top_k, 1.1)
    w = rng.uniform(0.05, 0.5, (tokens, lay.top_k)).astype(np.float32)
    req = pkg.MoEDeviceRequest(0, lay.hidden, lay.inter, lay.top_k, bf16_dev(xb), torch.from_numpy(ids).to(dev()),
                               torch.from_numpy(w).to(dev()))
    outs = []
    for path in (pkg._lib.PATH_AUTO, pkg._lib.PATH_SCALAR):
        out = torch.empty((tokens, lay.hidden), dtype=torch.float32, device=dev())
        moe.grouped_moe_staged(req, out, path=path)
        moe.sync_status()
        outs.append(out.cpu().numpy())
    rel, _ = check_close(outs[0], outs[1])
    assert rel < 1e-3
    # whole block: ids bit-exact against the CPU router at the full size
    out = torch.empty((tokens, lay.hidden), dtype=torch.bfloat16, device=dev())
    got_ids = torch.empty((tokens, lay.top_k), dtype=torch.int32, device=dev())
    got_w = torch.empty((tokens, lay.top_k), dtype=torch.float32, device=dev())
    moe.moe_block(0, bf16_dev(xb), bf16_dev(lay.gate_w), bf16_dev(lay.sh_gate_up), bf16_dev(lay.sh_down),
                  bf16_dev(lay.sh_gate), out, ids_out=got_ids, weights_out=got_w)
    moe.sync_status()
    want_ids, want_w = o.router(ol, pkg.synth.bf16_bits_to_f32(xb))
    assert np.array_equal(got_ids.cpu().numpy(), want_ids)
    assert np.abs(got_w.cpu().numpy() - want_w).max() <= 1e-6
    assert torch.isfinite(out.float()).all()


# ------------------------------------------------------------------ config 3 through the real router
@pytest.mark.parametrize("tokens", [512, 2048])
def test_config3_whole_block_zipf_through_the_router_matches_cpu_path(tokens):
    """Prefill sizes with a Zipf(1.1) popularity bias carried through the real router (hidden column 0 of the
    gate weight, x[:, 0] = 1): ids bit-exact, outputs against the CPU path directly (not against another CUDA
    path).  Some experts get no token, hot ones are cut into several passes of the grouped GEMM."""
    lay = pkg.synth.make_layer(3033, zipf_alpha=1.1)
    moe = make_moe(lay, max_tokens=tokens)
    load_all(moe, lay)
    ol = oracle_layer(lay)
    xb = pkg.synth.make_x(600 + tokens, tokens, lay.hidden, biased=True)
    out = torch.empty((tokens, lay.hidden), dtype=torch.bfloat16, device=dev())
    ids = torch.empty((tokens, lay.top_k), dtype=torch.int32, device=dev())
    w = torch.empty((tokens, lay.top_k), dtype=torch.float32, device=dev())
    moe.moe_block(0, bf16_dev(xb), bf16_dev(lay.gate_w), bf16_dev(lay.sh_gate_up), bf16_dev(lay.sh_down),
                  bf16_dev(lay.sh_gate), out, ids_out=ids, weights_out=w)
    moe.sync_status()
    want, want_ids, want_w = o.moe_block(ol, pkg.synth.bf16_bits_to_f32(xb), threads=o.max_threads())
    assert np.array_equal(ids.cpu().numpy(), want_ids), "routed expert ids must be bit-exact"
    assert np.abs(w.cpu().numpy() - want_w).max() <= 1e-6
    rel, _ = check_close(out.float().cpu().numpy(), want)
    assert rel < 5e-3, rel
    counts = np.bincount(want_ids.reshape(-1), minlength=lay.experts)
    if tokens == 2048:
        assert counts.min() == 0 and counts.max() > 200, "config 3: some experts idle, hot ones above 200 tokens"
    # the permutation of these routes, bit-exact
    seg, idx, badf = moe.csr_build(ids.reshape(-1), lay.experts)
    want_seg, want_idx = o.build_grouped_csr(want_ids.reshape(-1), lay.experts)
    assert np.array_equal(seg.cpu().numpy(), want_seg) and np.array_equal(idx.cpu().numpy(), want_idx) and badf == 0
    moe.close()


# ------------------------------------------------------------------ the absolute max-abs bar
SMALL_GLOBALS = (2.0 ** -6, 2.0 ** -10)


@pytest.fixture(scope="module")
def unit_scale():
    """The benchmark layer with row globals 2^-6 / 2^-10: outputs of magnitude O(0.1 .. 1)."""
    lay = pkg.synth.make_layer(4141, global_scale=SMALL_GLOBALS)
    moe = make_moe(lay, max_tokens=512)
    load_all(moe, lay)
    yield lay, moe, oracle_layer(lay)
    moe.close()


@pytest.mark.parametrize("tokens,odt", [(1, "bf16"), (8, "bf16"), (64, "bf16"), (64, "f32"), (300, "bf16")])
def test_whole_block_meets_the_absolute_bar(unit_scale, tokens, odt):
    """rel-L2 <= 1e-2 AND max |diff| <= 2e-2 in absolute terms: decode kernels (1, 8, 64 tokens) and the
    tcgen05 grouped GEMM (300 tokens = 2400 routes)."""
    lay, moe, ol = unit_scale
    xb = pkg.synth.make_x(5150 + tokens, tokens, lay.hidden)
    out = torch.empty((tokens, lay.hidden), dtype=torch.bfloat16 if odt == "bf16" else torch.float32, device=dev())
    ids = torch.empty((tokens, lay.top_k), dtype=torch.int32, device=dev())
    moe.moe_block(0, bf16_dev(xb), bf16_dev(lay.gate_w), bf16_dev(lay.sh_gate_up), bf16_dev(lay.sh_down),
                  bf16_dev(lay.sh_gate), out, ids_out=ids)
    moe.sync_status()
    want, want_ids, _ = o.moe_block(ol, pkg.synth.bf16_bits_to_f32(xb), threads=o.max_threads())
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    assert 0.05 < np.abs(want).max() < 4.0, "the case must have outputs where the absolute bar means something"
    check_close_abs(out.float().cpu().numpy(), want)


@pytest.mark.parametrize("path", ["gemv", "grouped"])
def test_routed_half_meets_the_absolute_bar_on_both_expert_paths(unit_scale, path):
    """The serving call with given ids on the decode kernels and on the grouped GEMM (forced), 320 tokens."""
    lay, moe, ol = unit_scale
    tokens = 320
    rng = np.random.default_rng(12)
    xb = pkg.synth.make_x(6160, tokens, lay.hidden)
    ids = _zipf_ids(rng, tokens, lay.experts, lay.top_k, 1.1)
    w = rng.uniform(0.05, 0.5, (tokens, lay.top_k)).astype(np.float32)
    out = torch.empty((tokens, lay.hidden), dtype=torch.bfloat16, device=dev())
    req = pkg.MoEDeviceRequest(0, lay.hidden, lay.inter, lay.top_k, bf16_dev(xb), torch.from_numpy(ids).to(dev()),
                               torch.from_numpy(w).to(dev()))
    moe.grouped_moe_staged(req, out, path=pkg._lib.PATH_GEMV if path == "gemv" else pkg._lib.PATH_GROUPED)
    moe.sync_status()
    want = o.grouped_moe_reference_mt(ol.banks, lay.hidden, lay.inter, pkg.synth.bf16_bits_to_f32(xb), lay.top_k,
                                      ids.reshape(-1), w.reshape(-1))
    check_close_abs(out.float().cpu().numpy(), want)


# ------------------------------------------------------------------ config 4 in small: a stack of blocks
def test_four_layer_stack_matches_the_chained_cpu_path():
    """x <- x + block_l(x) over four independently seeded layers (bf16 residual stream, as the stack benchmark
    runs it).  Every layer is checked against the CPU path fed the SAME input bits (ids bit-exact, outputs to
    the absolute bar), and the free-running CPU chain is compared at the end."""
    L, tokens = 4, 48
    lays = [pkg.synth.make_layer(7000 + l, global_scale=SMALL_GLOBALS) for l in range(L)]
    moe = make_moe(lays[0], max_tokens=tokens, layers=L)
    for l, lay in enumerate(lays):
        load_all(moe, lay, layer=l, slot0=l * lay.experts)
    H = lays[0].hidden
    xb = pkg.synth.make_x(7100, tokens, H)
    cur = bf16_dev(xb).clone()
    chain = pkg.synth.bf16_bits_to_f32(xb)          # the CPU chain, free-running
    chain_ok = True
    for l, lay in enumerate(lays):
        ol = oracle_layer(lay)
        out = torch.empty((tokens, H), dtype=torch.bfloat16, device=dev())
        ids = torch.empty((tokens, lay.top_k), dtype=torch.int32, device=dev())
        moe.moe_block(l, cur, bf16_dev(lay.gate_w), bf16_dev(lay.sh_gate_up), bf16_dev(lay.sh_down),
                      bf16_dev(lay.sh_gate), out, ids_out=ids)
        moe.sync_status()
        x_in = cur.float().cpu().numpy()
        want, want_ids, _ = o.moe_block(ol, x_in, threads=o.max_threads())
        assert np.array_equal(ids.cpu().numpy(), want_ids), f"layer {l}: ids"
        check_close_abs(out.float().cpu().numpy(), want)
        cur = cur + out                              # bf16 residual add
        c_out, c_ids, _ = o.moe_block(ol, chain, threads=o.max_threads())
        chain_ok = chain_ok and np.array_equal(c_ids, want_ids)
        chain = pkg.synth.bf16_bits_to_f32(pkg.synth.f32_to_bf16_bits(
            chain + pkg.synth.bf16_bits_to_f32(pkg.synth.f32_to_bf16_bits(c_out))))
    got = cur.float().cpu().numpy()
    assert np.isfinite(got).all()
    if chain_ok:   # a routing tie broken differently by a one-ulp input difference would fork the two chains
        check_close_abs(got, chain, rel_l2=1e-2, max_abs=5e-2)
    moe.close()


# ------------------------------------------------------------------ steps of one or two tokens
@pytest.mark.parametrize("case", ["one-token", "two-tokens-shared-experts", "sixteen-routes-one-slot", "missing-slots"])
def test_small_steps_build_their_plan_inside_the_expert_kernels(full, case):
    """At most 16 routes: no plan kernel, every CTA ranks the routes itself and four warps split K.  Routes that
    share an expert (two tokens per group), a slot with more than eight routes (two groups of one slot) and
    routes without a resident expert, against the CPU path and against the per-route scalar kernels."""
    lay, moe, ol = full
    rng = np.random.default_rng(17)
    tokens = 1 if case == "one-token" else 2
    xb = pkg.synth.make_x(8800 + tokens, tokens, lay.hidden)
    xf = pkg.synth.bf16_bits_to_f32(xb)
    if case == "one-token":
        routes = rng.permutation(lay.experts)[:lay.top_k].astype(np.int32)
    elif case == "two-tokens-shared-experts":
        first = rng.permutation(lay.experts)[:lay.top_k].astype(np.int32)
        second = first.copy()
        second[:3] = (first[:3] + 100) % lay.experts         # five experts shared by both tokens
        routes = np.concatenate([first, second[::-1]])
    elif case == "sixteen-routes-one-slot":
        routes = np.full(16, 5, np.int32)                      # slot ids are not required to differ per token here
    else:
        routes = rng.permutation(lay.experts)[:16].astype(np.int32)
        routes[[0, 7, 9]] = -1
    w = rng.uniform(0.05, 0.5, routes.size).astype(np.float32)
    out = torch.empty((tokens, lay.hidden), dtype=torch.float32, device=dev())
    moe.grouped_moe_dev(lay.hidden, lay.inter, lay.top_k, bf16_dev(xb), routes, torch.from_numpy(w).to(dev()), out)
    moe.sync_status()
    want = o.grouped_moe_reference(ol.banks, lay.hidden, lay.inter, xf, lay.top_k, routes, w)
    rel, _ = check_close(out.cpu().numpy(), want)
    assert rel < 5e-3, rel
