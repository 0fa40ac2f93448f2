"""GPU parity of the two steps either side of the MoE block, through the C ABI against the CPU checker:
the fused residual add + RMSNorm (and the block called through it), and the dense K-major NVFP4 GEMV of the
decode tail (lm_head)."""
import importlib
import importlib.util
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
pkg = importlib.import_module("ferrum-torrens_b200")
from oracle import oracle as o  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("make_golden_tail", os.path.join(HERE, "golden", "make_golden_tail.py"))
mg = importlib.util.module_from_spec(spec)
spec.loader.exec_module(mg)
G = np.load(os.path.join(HERE, "golden", "ref_tail_ops.npz"))


def dev():
    return torch.device("cuda:0")


def bf16_dev(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(dev()).view(torch.bfloat16)


def bits_of(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def tiny_handle(hidden, max_tokens=64):
    return pkg.B200MoE(0, pkg.ExpertShapes(hidden, 16), 1, experts=1, layers=1, top_k=1, shared_inter=16,
                       max_tokens=max_tokens)


# ------------------------------------------------------------------ fused residual add + RMSNorm
@pytest.mark.parametrize("case", mg.NORM_CASES, ids=[c[0] for c in mg.NORM_CASES])
def test_add_rmsnorm_matches_reference_fixture_and_cpu_path(case):
    label, rows, hidden, eps, seed = case
    x, r, w = mg.norm_inputs(rows, hidden, seed)
    moe = tiny_handle(hidden)
    s, y = moe.add_rmsnorm(bf16_dev(x), bf16_dev(r), bf16_dev(w), eps)
    torch.cuda.synchronize()
    want_s, want_y = o.add_rmsnorm(x, r, w, eps)
    assert np.array_equal(bits_of(s), want_s), "the residual sum is bit-exact"
    assert np.array_equal(bits_of(s), G[f"{label}/sum"])
    # the row reduction is a warp tree here, left to right in the CPU path, torch's order in the fixture: the
    # reciprocal may differ in its last bits, a normalised value then by one bf16 unit in the last place
    for want in (want_y, G[f"{label}/out"]):
        diff = np.abs(bits_of(y).astype(np.int32) - want.astype(np.int32))
        assert diff.max() <= 1 and (diff != 0).mean() <= 0.01
    moe.close()


@pytest.mark.parametrize("tokens", [1, 7, 64, 300])
def test_add_rmsnorm_ragged_row_counts(tokens):
    hidden = 2048
    x, r, w = mg.norm_inputs(tokens, hidden, 100 + tokens)
    moe = tiny_handle(hidden, max_tokens=512)
    s, y = moe.add_rmsnorm(bf16_dev(x), bf16_dev(r), bf16_dev(w), 1e-6)
    torch.cuda.synchronize()
    want_s, want_y = o.add_rmsnorm(x, r, w, 1e-6)
    assert np.array_equal(bits_of(s), want_s)
    diff = np.abs(bits_of(y).astype(np.int32) - want_y.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() <= 0.01
    moe.close()


@pytest.mark.parametrize("tokens", [1, 8, 64, 320])
def test_block_behind_the_post_attention_norm(tokens):
    """sum2 = attn_out + residual, h2 = rms_norm(sum2), out = moe_block(h2) in one call
    (forward.rs:942-953): the residual bit-exact, the normalised rows within one bf16 unit of the CPU path, and
    the block against the CPU path fed the same normalised rows (ids bit-exact, outputs to the absolute bar)."""
    lay = pkg.synth.make_layer(9090, global_scale=(2.0 ** -6, 2.0 ** -10))
    H = lay.hidden
    moe = pkg.B200MoE(0, pkg.ExpertShapes(H, lay.inter), lay.experts, experts=lay.experts, layers=1, top_k=lay.top_k,
                      shared_inter=lay.shared_inter, max_tokens=tokens)
    for e in range(lay.experts):
        moe.load(0, e, e, lay.fields(e))
    attn, resid, w = mg.norm_inputs(tokens, H, 500 + tokens)
    banks = o.HostBanks(*lay.banks, slots=lay.experts, gu_rows=2 * lay.inter, gu_cols=H, dn_rows=H, dn_cols=lay.inter)
    ol = o.Layer(H, lay.inter, lay.experts, lay.top_k, lay.shared_inter, lay.gate_w, lay.sh_gate_up, lay.sh_down,
                 lay.sh_gate, banks)
    sum_out = torch.empty((tokens, H), dtype=torch.bfloat16, device=dev())
    h2 = torch.empty((tokens, H), dtype=torch.bfloat16, device=dev())
    out = torch.empty((tokens, H), dtype=torch.bfloat16, device=dev())
    ids = torch.empty((tokens, lay.top_k), dtype=torch.int32, device=dev())
    moe.moe_block_prenorm(0, bf16_dev(attn), bf16_dev(resid), bf16_dev(w), 1e-6, bf16_dev(lay.gate_w),
                          bf16_dev(lay.sh_gate_up), bf16_dev(lay.sh_down), bf16_dev(lay.sh_gate), sum_out, out,
                          h2_out=h2, ids_out=ids)
    moe.sync_status()
    want_s, want_h2 = o.add_rmsnorm(attn, resid, w, 1e-6)
    assert np.array_equal(bits_of(sum_out), want_s)
    diff = np.abs(bits_of(h2).astype(np.int32) - want_h2.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() <= 0.01
    want, want_ids, _ = o.moe_block(ol, o.bf16_bits_to_f32(bits_of(h2)), threads=o.max_threads())
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    got = out.float().cpu().numpy()
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel <= 1e-2 and np.abs(got - want).max() <= 2e-2, (rel, np.abs(got - want).max())
    # without the optional h2 buffer the same block comes out (the rows then live in the adapter's scratch)
    out2 = torch.empty_like(out)
    moe.moe_block_prenorm(0, bf16_dev(attn), bf16_dev(resid), bf16_dev(w), 1e-6, bf16_dev(lay.gate_w),
                          bf16_dev(lay.sh_gate_up), bf16_dev(lay.sh_down), bf16_dev(lay.sh_gate), sum_out, out2)
    moe.sync_status()
    assert torch.equal(out, out2)
    moe.close()


def _trace_lines(err: str):
    out = []
    for ln in err.splitlines():
        if ln.startswith("TRACE "):
            _, layer, stage, l2, amax = ln.split()
            out.append((int(layer), stage, float(l2.split("=")[1]), float(amax.split("=")[1])))
    return out


def test_stage_dump_of_the_cuda_path_lines_up_with_the_cpu_path(capfd, monkeypatch):
    """FT_TRACE=1 (forward.rs:833-855): both paths print `TRACE <layer> <stage> l2= amax=` for sum2, h2 and moe of a
    layer; the two dumps name the same stages in the same order and agree stage by stage, so a divergence can be
    pinned to the first stage whose lines differ."""
    tokens = 24
    lay = pkg.synth.make_layer(9191, global_scale=(2.0 ** -6, 2.0 ** -10))
    H = lay.hidden
    moe = pkg.B200MoE(0, pkg.ExpertShapes(H, lay.inter), lay.experts, experts=lay.experts, layers=4, top_k=lay.top_k,
                      shared_inter=lay.shared_inter, max_tokens=tokens)
    for e in range(lay.experts):
        moe.load(3, e, e, lay.fields(e))
    attn, resid, w = mg.norm_inputs(tokens, H, 777)
    banks = o.HostBanks(*lay.banks, slots=lay.experts, gu_rows=2 * lay.inter, gu_cols=H, dn_rows=H, dn_cols=lay.inter)
    ol = o.Layer(H, lay.inter, lay.experts, lay.top_k, lay.shared_inter, lay.gate_w, lay.sh_gate_up, lay.sh_down,
                 lay.sh_gate, banks)
    sum_out = torch.empty((tokens, H), dtype=torch.bfloat16, device=dev())
    out = torch.empty((tokens, H), dtype=torch.float32, device=dev())
    args = (3, bf16_dev(attn), bf16_dev(resid), bf16_dev(w), 1e-6, bf16_dev(lay.gate_w), bf16_dev(lay.sh_gate_up),
            bf16_dev(lay.sh_down), bf16_dev(lay.sh_gate), sum_out, out)
    moe.moe_block_prenorm(*args)
    moe.sync_status()
    assert _trace_lines(capfd.readouterr().err) == [], "nothing is printed unless FT_TRACE=1"
    monkeypatch.setenv("FT_TRACE", "1")
    moe.moe_block_prenorm(*args)
    moe.sync_status()
    got = _trace_lines(capfd.readouterr().err)
    o.moe_block_prenorm(ol, 3, attn, resid, w, 1e-6, threads=o.max_threads())
    want = _trace_lines(capfd.readouterr().err)
    assert [(l, s) for l, s, _, _ in got] == [(3, "sum2"), (3, "h2"), (3, "moe")]
    assert [(l, s) for l, s, _, _ in got] == [(l, s) for l, s, _, _ in want]
    for (_, stage, l2, amax), (_, _, wl2, wamax) in zip(got, want):
        tol = 0.0 if stage == "sum2" else 5e-3
        assert abs(l2 - wl2) <= tol * wl2 + 1e-6 and abs(amax - wamax) <= 2 * tol * wamax + 1e-6, (stage, l2, wl2, amax, wamax)
    moe.close()


# ------------------------------------------------------------------ dense K-major NVFP4 GEMV (lm_head)
def _gemv_case(m, n, k, seed):
    a, packed, scale, glob = mg.gemv_inputs(m, n, k, seed)
    pk, sk = mg.kmajor(packed, scale)
    return a, pk, sk, glob


def _run_gemv(moe, a, pk, sk, glob):
    c = moe.dense_gemv(bf16_dev(a), torch.from_numpy(pk.view(np.int32)).to(dev()), torch.from_numpy(sk).to(dev()),
                       torch.from_numpy(glob.view(np.int16)).to(dev()))
    torch.cuda.synchronize()
    return c.cpu().numpy()


@pytest.mark.parametrize("case", mg.GEMV_CASES, ids=[c[0] for c in mg.GEMV_CASES])
def test_dense_gemv_matches_reference_fixture(case):
    label, m, n, k, seed = case
    a, pk, sk, glob = _gemv_case(m, n, k, seed)
    moe = tiny_handle(64)
    got = _run_gemv(moe, a, pk, sk, glob)
    want = G[f"{label}/c"]
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel <= 1e-5, rel
    moe.close()


@pytest.mark.parametrize("m,n,k", [(1, 4, 32), (1, 36, 64), (8, 1000, 512), (9, 128, 2048), (16, 260, 96), (17, 64, 2048),
                                   (40, 32, 256), (1, 448, 256), (3, 1056, 512), (12, 2000, 2048), (20, 464, 768)])
def test_dense_gemv_ragged_shapes_against_cpu_path(m, n, k):
    """Rows that are not a multiple of the 32-row tile, K with and without the two-way split, one to several
    token tiles and more than sixteen tokens (several passes over the weight).  The last four shapes (N a
    multiple of 16 and at least 448, K a multiple of 256) take the TMA-fed kernel: one tile exactly, a last
    tile of 160 and of 208 rows, a last tile of 16 rows."""
    a, pk, sk, glob = _gemv_case(m, n, k, 1000 + m + n + k)
    moe = tiny_handle(64)
    got = _run_gemv(moe, a, pk, sk, glob)
    want = o.nvfp4_dense_gemv(o.bf16_bits_to_f32(a), pk, sk, glob.view(np.uint16))
    rel = np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)
    assert rel <= 1e-5, rel
    assert np.abs(got - want).max() <= 1e-4 * np.abs(want).max()
    moe.close()


@pytest.mark.parametrize("m", [1, 8])
def test_dense_gemv_lm_head_size(m):
    """248 320 x 2048, the vocabulary projection: a strided sample of the rows against the CPU path, and
    linearity in the activations over all of them (a size-independent property)."""
    n, k = 248320, 2048
    g = torch.Generator(device=dev()).manual_seed(77)
    pk = torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 8, n), generator=g, device=dev(), dtype=torch.int64).to(torch.int32)
    u = torch.rand((k // 16, n), generator=g, device=dev()) * -6.0
    sk = torch.exp2(u).to(torch.float8_e4m3fn).view(torch.uint8)
    glob = torch.full((n,), 2.0 ** -4, dtype=torch.float16, device=dev())
    a_bits = pkg.synth.make_x(4321, m, k)
    moe = tiny_handle(64)
    a = bf16_dev(a_bits)
    c = moe.dense_gemv(a, pk, sk, glob.view(torch.int16))
    c2 = moe.dense_gemv(a * 2, pk, sk, glob.view(torch.int16))
    torch.cuda.synchronize()
    assert torch.equal(c2, c * 2), "doubling the activations doubles every logit exactly"
    rows = np.arange(0, n, 997)
    rows4 = np.unique(np.concatenate([rows // 4 * 4 + i for i in range(4)]))       # whole quads of rows
    want = o.nvfp4_dense_gemv(o.bf16_bits_to_f32(a_bits), pk[:, rows4].cpu().numpy().view(np.uint32),
                              sk[:, rows4].cpu().numpy(), glob[rows4].view(torch.int16).cpu().numpy().view(np.uint16))
    got = c[:, rows4].cpu().numpy()
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel <= 1e-5, rel
    moe.close()


def test_dense_gemv_rejects_shapes_it_was_not_built_for():
    moe = tiny_handle(64)
    a, pk, sk, glob = _gemv_case(1, 8, 64, 5)
    with pytest.raises(pkg.MoEError, match="not the shapes handed in"):
        moe.dense_gemv(bf16_dev(a), torch.from_numpy(pk.view(np.int32)).to(dev())[:, :6].contiguous(),
                       torch.from_numpy(sk).to(dev())[:, :6].contiguous(), torch.from_numpy(glob.view(np.int16)).to(dev())[:6])
    with pytest.raises(pkg.MoEError, match="not the shapes handed in"):
        moe.dense_gemv(bf16_dev(a), torch.from_numpy(pk.view(np.int32)).to(dev()), torch.from_numpy(sk).to(dev())[:2],
                       torch.from_numpy(glob.view(np.int16)).to(dev()))
    moe.close()
