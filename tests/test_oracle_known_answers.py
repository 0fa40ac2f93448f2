"""The CPU checker against the reference's own known-answer tests.

Every case below restates, as data, a unit test of the reference (file:line in
the docstring); the expected values are the reference's hand-computed ones.
"""
import math

import numpy as np
import pytest

from oracle import oracle as o

H = 16
I = 16
E4M3_ONE = 0x38
E4M3_TWO = 0x40
F16 = {0.5: 0x3800, 1.0: 0x3C00, -1.0: 0xBC00, 4.0: 0x4400}


def slab(rows, cols, packed, scale, glob):
    """One slab whose every packed byte / scale byte is constant (expert_kernel.rs:702-708)."""
    g = np.tile(np.array([F16[glob] & 0xFF, F16[glob] >> 8], np.uint8), rows)
    return (np.full(rows * cols // 2, packed, np.uint8), np.full(rows * cols // 16, scale, np.uint8), g)


def banks_of(gus, dns, h=H, i=I):
    cat = lambda slabs, f: np.concatenate([s[f] for s in slabs])
    return o.HostBanks(cat(gus, 0), cat(gus, 1), cat(gus, 2), cat(dns, 0), cat(dns, 1), cat(dns, 2),
                       slots=len(gus), gu_rows=2 * i, gu_cols=h, dn_rows=h, dn_cols=i)


def silu(v):
    v = np.float32(v)
    return float(v / (np.float32(1.0) + np.exp(-v, dtype=np.float32)))


def close(a, b):
    assert abs(a - b) <= 1e-4 * max(abs(b), 1.0), (a, b)


# ---- src/domain/numerics.rs:75-136 -----------------------------------------
def test_bf16_roundtrip():
    for bits, want in [(0x3F80, 1.0), (0xC000, -2.0), (0x0000, 0.0), (0x8000, -0.0),
                       (0x7F80, math.inf), (0x3F00, 0.5)]:
        assert o.bf16_to_f32(bits) == want
    third = np.float32(1.0 / 3.0)
    b = int(third.view(np.uint32)) >> 16
    assert abs(o.bf16_to_f32(b) - 1.0 / 3.0) < 0.01


def test_f16_values():
    assert o.f16_to_f32(0x3C00) == 1.0
    assert o.f16_to_f32(0xC000) == -2.0
    assert o.f16_to_f32(0x0000) == 0.0
    assert o.f16_to_f32(0x8000) == 0.0 and math.copysign(1, o.f16_to_f32(0x8000)) == -1
    assert o.f16_to_f32(0x7C00) == math.inf
    assert o.f16_to_f32(0xFC00) == -math.inf
    assert o.f16_to_f32(0x0001) == 2.0 ** -24
    assert o.f16_to_f32(0x3800) == 0.5


def test_f16_matches_numpy_on_every_normal_code():
    codes = np.arange(0x10000, dtype=np.uint16)
    want = codes.view(np.float16).astype(np.float32)
    for c in range(0, 0x10000, 7):
        exp, man = (c >> 10) & 0x1F, c & 0x3FF
        got = o.f16_to_f32(c)
        if exp == 0x1F and man:
            assert math.isnan(got)
        elif exp == 0 and man and (c & 0x8000):
            # the reference drops the sign of negative subnormals (numerics.rs:19-22)
            assert got == -float(want[c])
        else:
            assert got == float(want[c]), hex(c)


def test_e4m3fn_values():
    assert o.e4m3fn_to_f32(0x00) == 0.0
    assert math.copysign(1, o.e4m3fn_to_f32(0x80)) == -1 and o.e4m3fn_to_f32(0x80) == 0.0
    assert o.e4m3fn_to_f32(0x38) == 1.0
    assert o.e4m3fn_to_f32(0x3C) == 1.5
    assert o.e4m3fn_to_f32(0xB8) == -1.0
    assert o.e4m3fn_to_f32(0x77) == 240.0
    assert o.e4m3fn_to_f32(0x7E) == 448.0
    assert math.isnan(o.e4m3fn_to_f32(0x7F))
    assert math.isnan(o.e4m3fn_to_f32(0xFF))
    assert o.e4m3fn_to_f32(0x01) == 2.0 ** -9
    assert o.e4m3fn_to_f32(0x03) == 3.0 * 2.0 ** -9


def test_e4m3fn_matches_torch_on_every_code():
    torch = pytest.importorskip("torch")
    codes = torch.arange(256, dtype=torch.uint8)
    want = codes.view(torch.float8_e4m3fn).to(torch.float32)
    for c in range(256):
        got = o.e4m3fn_to_f32(c)
        if math.isnan(float(want[c])):
            assert math.isnan(got)
        else:
            assert got == float(want[c])


def test_fp4_lut_covers_all_codes():
    lut = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
    for code, want in enumerate(lut):
        assert o.fp4_nibble(code & 0x0F, False) == want
        assert o.fp4_nibble((code << 4) & 0xFF, True) == want
    # low nibble is the even k (expert_kernel.rs:1253-1257)
    assert o.fp4_nibble(0x10, False) == 0.0 and o.fp4_nibble(0x10, True) == 0.5
    assert o.fp4_nibble(0x01, False) == 0.5 and o.fp4_nibble(0x01, True) == 0.0


# ---- src/domain/dequant.rs:285-299: fp4 * e4m3 is exact in bf16 ---------------
def test_block_product_is_exact_in_bf16():
    packed = np.arange(256, dtype=np.uint8).repeat(8)  # 256 rows x 16 k
    for s in (0x01, 0x08, 0x38, 0x3C, 0x47, 0x7E):
        w = o.nvfp4_block(packed, 256, 16, np.full(256, s, np.uint8))
        assert np.array_equal(o.bf16_bits_to_f32(o.f32_to_bf16_bits(w)), w)


# ---- src/domain/expert_kernel.rs:744-790 ------------------------------------
def test_hand_computed_case_matches():
    want = 0.5 * (8.0 * 0.5 * silu(4.0) * 4.0)
    banks = banks_of([slab(2 * I, H, 0x10, E4M3_ONE, 1.0)], [slab(H, I, 0x10, E4M3_ONE, 1.0)])
    out = o.grouped_moe_reference(banks, H, I, np.ones(H, np.float32), 1, [0], [0.5])
    for v in out.reshape(-1):
        close(v, want)


# ---- :792-849 ---------------------------------------------------------------
def test_abs_sum_reports_the_terms_a_cancelling_sum_hides():
    term = 4.0 * silu(4.0) * 4.0
    banks = banks_of([slab(2 * I, H, 0x10, E4M3_ONE, 1.0)] * 2,
                     [slab(H, I, 0x10, E4M3_ONE, 1.0), slab(H, I, 0x10, E4M3_ONE, -1.0)])
    out, abs_sum = o.grouped_moe_reference(banks, H, I, np.ones(H, np.float32), 2, [0, 1],
                                           [1.0, 1.0], want_abs_sum=True)
    for a, b in zip(out.reshape(-1), abs_sum.reshape(-1)):
        close(a, 0.0)
        close(b, 2.0 * term)


# ---- :851-888 ---------------------------------------------------------------
def test_non_resident_route_contributes_nothing():
    banks = banks_of([slab(2 * I, H, 0x10, E4M3_ONE, 1.0)], [slab(H, I, 0x10, E4M3_ONE, 1.0)])
    out = np.full(H, 7.0, np.float32)
    o.grouped_moe_reference(banks, H, I, np.ones(H, np.float32), 1, [-1], [1.0], out=out)
    assert np.array_equal(out, np.zeros(H, np.float32))


# ---- :890-979 ---------------------------------------------------------------
def test_slot_selects_its_own_expert():
    gus = [slab(2 * I, H, 0x01, E4M3_ONE, 1.0), slab(2 * I, H, 0x10, E4M3_ONE, 1.0)]
    dns = [slab(H, I, 0x01, E4M3_ONE, 1.0), slab(H, I, 0x10, E4M3_ONE, 1.0)]
    x = np.array([1.0 if k % 2 == 0 else 2.0 for k in range(H)], np.float32)
    run = lambda b, s: o.grouped_moe_reference(b, H, I, x, 1, [s], [1.0]).reshape(-1)
    banks = banks_of(gus, dns)
    want0 = 8.0 * 0.5 * silu(4.0) * 4.0
    want1 = 8.0 * 0.5 * silu(8.0) * 8.0
    for v in run(banks, 0):
        close(v, want0)
    for v in run(banks, 1):
        close(v, want1)
    zero_gu = (np.zeros(2 * I * H // 2, np.uint8), np.zeros(2 * I * H // 16, np.uint8), np.zeros(4 * I, np.uint8))
    zero_dn = (np.zeros(H * I // 2, np.uint8), np.zeros(H * I // 16, np.uint8), np.zeros(2 * H, np.uint8))
    banks = banks_of([gus[0], zero_gu], [dns[0], zero_dn])
    assert np.array_equal(run(banks, 1), np.zeros(H, np.float32))
    assert (run(banks, 0) > 0).all()


# ---- :981-1023 --------------------------------------------------------------
def test_global_scale_applies_once_after_the_k_reduction():
    banks = banks_of([slab(2 * I, H, 0x10, E4M3_ONE, 4.0)], [slab(H, I, 0x10, E4M3_ONE, 0.5)])
    out = o.grouped_moe_reference(banks, H, I, np.ones(H, np.float32), 1, [0], [1.0])
    ic2 = silu(16.0) * 16.0
    for v in out.reshape(-1):
        close(v, 8.0 * 0.5 * ic2 * 0.5)


# ---- :1025-1075 -------------------------------------------------------------
def test_block_scale_is_per_sixteen_k():
    s0 = slab(2 * I, 32, 0x10, E4M3_ONE, 1.0)
    s1 = list(slab(2 * I, 32, 0x10, E4M3_TWO, 1.0))
    s1[1] = np.array([E4M3_TWO if b % 2 == 1 else E4M3_ONE for b in range(2 * I * 32 // 16)], np.uint8)
    banks = banks_of([s0, tuple(s1)], [slab(32, I, 0x10, E4M3_ONE, 1.0)] * 2, h=32, i=I)
    out = o.grouped_moe_reference(banks, 32, I, np.ones(32, np.float32), 1, [1], [1.0])
    ic2 = silu(12.0) * 12.0
    for v in out.reshape(-1):
        close(v, 8.0 * 0.5 * ic2)


# ---- :1077-1139 -------------------------------------------------------------
def test_routes_sum_weighted_over_top_k():
    banks = banks_of([slab(2 * I, H, 0x10, E4M3_ONE, 1.0), slab(2 * I, H, 0x11, E4M3_ONE, 1.0)],
                     [slab(H, I, 0x10, E4M3_ONE, 1.0), slab(H, I, 0x11, E4M3_ONE, 1.0)])
    x = np.ones(H, np.float32)
    one = lambda s, w: o.grouped_moe_reference(banks, H, I, x, 1, [s], [w]).reshape(-1)
    both = o.grouped_moe_reference(banks, H, I, x, 2, [0, 1], [0.25, 0.75]).reshape(-1)
    a, b = one(0, 0.25), one(1, 0.75)
    for i in range(H):
        close(both[i], a[i] + b[i])


# ---- :1141-1181 -------------------------------------------------------------
def test_shape_and_slot_mismatches_are_errors():
    banks = banks_of([slab(2 * I, H, 0x10, E4M3_ONE, 1.0)], [slab(H, I, 0x10, E4M3_ONE, 1.0)])
    x = np.ones(H, np.float32)
    with pytest.raises(o.OracleError) as e:
        o.grouped_moe_reference(banks, H + 16, I, x, 1, [0], [1.0])
    assert e.value.kind == "Bad"
    with pytest.raises(o.OracleError) as e:
        o.grouped_moe_reference(banks, H, I, x, 1, [5], [1.0])
    assert (e.value.kind, e.value.slot, e.value.capacity) == ("SlotOutOfRange", 5, 1)


# ---- :1183-1245 -------------------------------------------------------------
def test_reference_matches_the_scalar_gemv_order():
    rows = 2 * I
    packed = np.array([(i * 37 + 11) & 0xFF for i in range(rows * H // 2)], np.uint8)
    scale = np.array([(i * 7 + 3) & 0xFF for i in range(rows * H // 16)], np.uint8)
    glob = np.tile(np.array([0x00, 0x3C], np.uint8), rows)
    dn = slab(H, I, 0x21, E4M3_ONE, 1.0)
    banks = o.HostBanks(packed, scale, glob, dn[0], dn[1], dn[2], 1, rows, H, H, I)
    x = np.array([((k * 13 % 9) * 0.25) - 1.0 for k in range(H)], np.float32)
    out = o.grouped_moe_reference(banks, H, I, x, 1, [0], [1.0]).reshape(-1)
    ic1 = o.tower_nvfp4_gemv(x, packed, scale, glob, rows, H)
    ic2 = np.array([silu(ic1[k]) * ic1[I + k] for k in range(I)], np.float32)
    ic3 = o.tower_nvfp4_gemv(ic2, dn[0], dn[1], dn[2], H, I)
    for i in range(H):
        close(out[i], ic3[i])


# ---- :641-652 ---------------------------------------------------------------
def test_routes_flatten_token_major():
    tok, slot = o.route_lists([3, -1, 1, 1, 0, 2], 3, 2)
    assert tok.tolist() == [0, 0, 1, 1, 2, 2]
    assert slot.tolist() == [3, -1, 1, 1, 0, 2]
    for args in (([0, 1], 2, 2), ([], 0, 1), ([0], 1, 0)):
        with pytest.raises(o.OracleError):
            o.route_lists(*args)


# ---- src/infrastructure/cuda_moe.rs:2711-2733 --------------------------------
def test_grouped_csr_buckets_and_refuses_bad_slots():
    seg, idx = o.build_grouped_csr([2, 0, 2, 0, 0, 1], 3)
    assert seg.tolist() == [0, 3, 4, 6]
    assert idx.tolist() == [1, 3, 4, 5, 0, 2]
    with pytest.raises(o.OracleError, match="not resident"):
        o.build_grouped_csr([-1, 0], 3)
    with pytest.raises(o.OracleError, match="past the"):
        o.build_grouped_csr([3], 3)


# ---- src/models/qwen3_6/forward.rs:1219-1236 ---------------------------------
def test_shared_expert_gate_is_sigmoid():
    assert abs(o.sigmoid(2.0) - 0.8807971) < 1e-6
    assert abs(o.sigmoid(0.0) - 0.5) < 1e-6
    assert abs(o.sigmoid(-2.0) - 0.11920292) < 1e-6


def test_topk_renormalizes():
    ids, w = o.topk_renorm(np.array([[0.5, 0.2, 0.3]], np.float32), 2)
    assert ids.tolist() == [[0, 2]]
    assert abs(w[0, 0] - 0.5 / 0.8) < 1e-6 and abs(w[0, 1] - 0.3 / 0.8) < 1e-6


def test_topk_ties_take_the_lowest_index():
    """elementwise.py:372-373 / tests/cudarc_forward.rs:89-97"""
    p = np.array([[0.1, 0.3, 0.3, 0.1, 0.2, 0.0]], np.float32)
    ids, w = o.topk_renorm(p, 4)
    assert ids.tolist() == [[1, 2, 4, 0]]
    assert np.allclose(w.sum(1), 1.0, atol=1e-6)


# ---- bank bytes: src/infrastructure/cuda_moe.rs:2910-2921 --------------------
def test_bank_bytes_per_expert():
    h, i = 2048, 512
    rows = [(2 * i) * h // 2, (2 * i) * h // 16, (2 * i) * 2, h * i // 2, h * i // 16, h * 2]
    assert rows == [1048576, 131072, 2048, 524288, 65536, 4096]
    assert sum(rows) == 1775616


# ---- src/domain/expert_cache.rs:141-283 --------------------------------------
def test_cache_fills_free_slots_first_lowest_slot():
    c = o.ExpertCache(2, 4, 8)
    misses, slots, rew = c.ensure_experts(0, [2, 0])
    assert (misses, slots, rew) == ([0, 2], [0, 1], [1, 0])
    assert c.slot_of(0, 0) == 0 and c.slot_of(0, 2) == 1
    assert c.id_of_slot(0) == 0 and c.id_of_slot(1) == 2


def test_cache_hits_are_resident_and_noop():
    c = o.ExpertCache(1, 4, 8)
    c.ensure_experts(0, [1, 3])
    misses, _, rew = c.ensure_experts(0, [3, 1, 3])
    assert misses == []
    assert rew == [c.slot_of(0, 3), c.slot_of(0, 1), c.slot_of(0, 3)]
    assert all(s >= 0 for s in rew)


def test_cache_full_within_one_layer_never_misses():
    c = o.ExpertCache(1, 6, 6)
    assert c.ensure_experts(0, [0, 1, 2, 3, 4, 5])[1] == [0, 1, 2, 3, 4, 5]
    misses, _, rew = c.ensure_experts(0, [5, 2, 0])
    assert misses == [] and rew == [5, 2, 0]


def test_cache_lru_victim_is_the_coldest_slot():
    c = o.ExpertCache(1, 8, 6)
    c.ensure_experts(0, [0, 1, 2, 3, 4, 5])
    c.ensure_experts(0, [5, 0])
    misses, slots, _ = c.ensure_experts(0, [6])
    assert misses == [6] and slots == [1]
    assert c.slot_of(0, 1) == -1 and c.slot_of(0, 5) == 5


def test_cache_same_step_hits_not_evicted():
    c = o.ExpertCache(1, 8, 6)
    assert c.ensure_experts(0, [0, 1, 2, 3, 4, 5])[1] == [0, 1, 2, 3, 4, 5]
    c.ensure_experts(0, [0, 1])
    assert c.ensure_experts(0, [6, 7])[1] == [2, 3]
    assert c.slot_of(0, 0) == 0 and c.slot_of(0, 1) == 1 and c.slot_of(0, 2) == -1


def test_cache_layer_id_space_is_flat_and_cross_layer():
    c = o.ExpertCache(2, 4, 8)
    c.ensure_experts(0, [0])
    c.ensure_experts(1, [0, 0])
    assert c.slot_of(0, 0) != -1 and c.slot_of(1, 0) != -1 and c.slot_of(0, 0) != c.slot_of(1, 0)
    assert len(c.ensure_experts(1, [1, 2, 3])[2]) == 3
    c = o.ExpertCache(3, 4, 4)
    c.ensure_experts(0, [1, 3])
    c.ensure_experts(1, [0, 2])
    assert c.ensure_experts(0, [1, 3])[0] == []
    assert c.ensure_experts(2, [0])[0] == [0] and c.slot_of(2, 0) >= 0


def test_cache_duplicates_and_small_cache():
    c = o.ExpertCache(1, 4, 8)
    misses, _, rew = c.ensure_experts(0, [2, 2, 2])
    assert misses == [2] and rew == [c.slot_of(0, 2)] * 3
    c = o.ExpertCache(1, 6, 3)
    misses, slots, rew = c.ensure_experts(0, [5, 4, 3, 2])
    assert misses == [2, 3, 4, 5] and slots == [0, 1, 2, 0]
    assert rew == [c.slot_of(0, 5), c.slot_of(0, 4), c.slot_of(0, 3), c.slot_of(0, 2)]
    assert c.slot_of(0, 5) >= 0 and c.slot_of(0, 4) >= 0 and c.slot_of(0, 3) >= 0


# ---- the reproducible exponential ---------------------------------------------
def test_expf_is_faithful():
    xs = np.concatenate([np.linspace(-103, 88, 20001, dtype=np.float32),
                         -np.abs(np.random.default_rng(0).normal(0, 3, 20000)).astype(np.float32)])
    got = np.array([o.expf(float(v)) for v in xs], np.float32)
    want64 = np.exp(xs.astype(np.float64))
    ulp = np.spacing(np.maximum(np.abs(want64.astype(np.float32)), np.float32(1e-45)))
    err = np.abs(got.astype(np.float64) - want64) / ulp
    assert err.max() < 1.0, err.max()
    assert o.expf(0.0) == 1.0 and o.expf(-200.0) == 0.0 and o.expf(100.0) == math.inf
    # monotone on a dense grid around the values the router sees
    g = np.array([o.expf(float(v)) for v in np.linspace(-12, 0, 50001, dtype=np.float32)])
    assert (np.diff(g) >= 0).all()
