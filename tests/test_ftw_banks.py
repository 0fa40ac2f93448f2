"""FTW checkpoint index and expert-bank reader (host code of the library; no GPU needed except the last test).

The cases restate the reference's own unit tests: src/infrastructure/banks.rs:283-420 (one layer of banks at
contiguous offsets, an echoing reader that shows which window was asked for; expert past the bank, missing
layer, a scale entry that does not match the packed shape, a failing read) and the index checks of
src/infrastructure/ftw.rs:95-252 (format tag, version, alignment, shard contiguity, tensor ranges) with
`pieces` over a tensor that spans two shards."""
import importlib
import json
import os

import numpy as np
import pytest

pkg = importlib.import_module("ferrum-torrens_b200")
ftw = pkg.ftw

EXPERTS, ROWS, COLS = 2, 32, 64     # gate_up [ROWS, COLS], down [COLS, ROWS]: the reference test's shape
ALIGN = 4096


def bank_tensors(layer, experts=EXPERTS, rows=ROWS, cols=COLS, off=ALIGN, prefix=""):
    """One layer of banks, three fields per part, every entry 4096-aligned (banks.rs:294-311)."""
    out = []
    for part, r, c in (("gate_up", rows, cols), ("down", cols, rows)):
        for field, unit in (("packed", c // 2), ("scale", c // 16), ("global", 2)):
            nbytes = experts * r * unit
            out.append({"name": f"{prefix}{part}_{field}#L{layer:05d}", "kind": "experts_bank", "dtype": "uint8",
                        "shape": [experts, r, unit], "global_off": off, "nbytes": nbytes})
            off += (nbytes + ALIGN - 1) // ALIGN * ALIGN
    return out, off


def index_doc(tensors, total, shards=None, **over):
    doc = {"format": "freetoken_weight", "version": 1, "align": ALIGN, "shard_limit": 1 << 30, "total_bytes": total,
           "tensors": tensors, "shards": shards if shards is not None else [{"file": "s0.ftw", "global_off": 0, "nbytes": total}],
           "quant_format": "nvfp4", "expert_bank_num_layers": 1}
    doc.update(over)
    return doc


def write_checkpoint(tmp_path, layer=7, shard_cut=None):
    """An index plus shard files whose byte at region offset o is (o * 7 + o // 251) % 256: every window read
    back can be checked against its own offset (the reference's echoing reader, with real files)."""
    tensors, total = bank_tensors(layer)
    region = ((np.arange(total, dtype=np.int64) * 7 + np.arange(total, dtype=np.int64) // 251) % 256).astype(np.uint8)
    cut = shard_cut or total
    shards = [{"file": "part-0.ftw", "global_off": 0, "nbytes": cut}]
    if cut < total:
        shards.append({"file": "part-1.ftw", "global_off": cut, "nbytes": total - cut})
    for sh in shards:
        region[sh["global_off"]:sh["global_off"] + sh["nbytes"]].tofile(os.path.join(tmp_path, sh["file"]))
    with open(os.path.join(tmp_path, ftw.INDEX_NAME), "w") as fh:
        json.dump(index_doc(tensors, total, shards), fh)
    return tensors, region


# ------------------------------------------------------------------ index
def test_parse_accepts_a_valid_index_and_finds_entries():
    tensors, total = bank_tensors(7)
    ix = ftw.FtwIndex.parse(json.dumps(index_doc(tensors, total)))
    assert len(ix) == 6 and ix.total_bytes == total and ix.shard_count() == 1
    e = ix.entry("gate_up_packed#L00007")
    assert e == {"global_off": ALIGN, "nbytes": EXPERTS * ROWS * COLS // 2, "shape": [EXPERTS, ROWS, COLS // 2], "experts_bank": True}
    assert ix.entry("down_packed#L00007")["shape"] == [EXPERTS, COLS, ROWS // 2]
    assert ix.entry("gate_up_packed#L00008") is None
    # an index parsed from text has no shard files behind it
    with pytest.raises(pkg.MoEError) as err:
        ix.read_range(ALIGN, 16)
    assert err.value.kind == "Read"


@pytest.mark.parametrize("mutate,kind,needle", [
    (lambda d: d.update(format="safetensors"), "Bad", "not an FTW checkpoint"),
    (lambda d: d.pop("format"), "Bad", "missing 'format'"),
    (lambda d: d.update(version=2), "Bad", "unsupported FTW version 2"),
    (lambda d: d.update(align=512), "Bad", "unexpected alignment 512"),
    (lambda d: d.pop("total_bytes"), "Bad", "missing 'total_bytes'"),
    (lambda d: d.pop("tensors"), "Bad", "missing 'tensors'"),
    (lambda d: d["tensors"][0].update(global_off=100), "Bad", "unaligned offset 100"),
    (lambda d: d["tensors"][0].update(nbytes=0), "Bad", "is empty"),
    (lambda d: d["tensors"][0].update(shape=[1, 1, 1]), "Bad", "shape*elsize"),
    (lambda d: d["tensors"][0].update(dtype="complex64"), "Bad", "unknown dtype"),
    (lambda d: d["tensors"][0].update(shape=[2, 32, 1.5]), "Bad", "non-integer shape"),
    (lambda d: d["tensors"][-1].update(global_off=1 << 40), "Bad", "exceeds total_bytes"),
    (lambda d: d["shards"].append({"file": "x", "global_off": 5, "nbytes": 9}), "Bad", "shards not contiguous"),
    (lambda d: d["shards"][0].update(nbytes=d["total_bytes"] - ALIGN), "Bad", "shards cover"),
    (lambda d: d["shards"][0].update(nbytes=0), "Bad", "empty shard"),
])
def test_parse_rejects_what_the_reference_rejects(mutate, kind, needle):
    tensors, total = bank_tensors(0)
    doc = index_doc(tensors, total)
    mutate(doc)
    with pytest.raises(pkg.MoEError) as err:
        ftw.FtwIndex.parse(json.dumps(doc))
    assert err.value.kind == kind and needle in str(err.value), str(err.value)


def test_parse_reports_json_syntax_errors():
    with pytest.raises(pkg.MoEError, match="JSON parse failure"):
        ftw.FtwIndex.parse('{"format": "freetoken_weight", ')
    with pytest.raises(pkg.MoEError, match="JSON parse failure"):
        ftw.FtwIndex.parse('{"format": "freetoken_weight"} trailing')


def test_layer_bank_entry_names():
    assert ftw.layer_bank_entry("gate_up_packed#L00007") == ("gate_up_packed", 7)
    assert ftw.layer_bank_entry("draft_down_scale#L00000") == ("draft_down_scale", 0)
    for bad in ("gate_up_packed", "#L00007", "x#L7", "x#L0000a", "x#L000007"):
        assert ftw.layer_bank_entry(bad) is None


def test_pieces_cut_a_range_at_the_shard_boundary():
    tensors, total = bank_tensors(0)
    cut = tensors[0]["global_off"] + ALIGN      # an aligned region offset
    shards = [{"file": "a", "global_off": 0, "nbytes": cut}, {"file": "b", "global_off": cut, "nbytes": total - cut}]
    ix = ftw.FtwIndex.parse(json.dumps(index_doc(tensors, total, shards)))
    # a range inside one shard: one piece; a range across the cut: two pieces, the second starting at file offset 0
    assert ix.pieces(100, 50) == [(0, 100, 0, 50)]
    assert ix.pieces(cut - 10, 30) == [(0, cut - 10, 0, 10), (1, 0, 10, 20)]
    assert ix.pieces(cut, 5) == [(1, 0, 0, 5)]
    with pytest.raises(pkg.MoEError, match="exceeds shards"):
        ix.pieces(total - 4, 8)


# ------------------------------------------------------------------ reader and slabs over real shard files
def test_slab_reads_one_experts_three_fields(tmp_path):
    """banks.rs:343-357 and :359-368: the second expert's packed window starts one expert into the entry."""
    tensors, region = write_checkpoint(tmp_path)
    ix = ftw.FtwIndex.open(tmp_path)
    src = ftw.FtwBanks(ix)
    packed, scale, glob = src.slab(7, 1, "GateUp")
    assert (packed.size, scale.size, glob.size) == (ROWS * COLS // 2, ROWS * COLS // 16, ROWS * 2)
    e = ix.entry("gate_up_packed#L00007")
    second = e["global_off"] + ROWS * COLS // 2
    assert np.array_equal(packed, region[second:second + packed.size])
    s = ix.entry("gate_up_scale#L00007")
    assert np.array_equal(scale, region[s["global_off"] + scale.size:s["global_off"] + 2 * scale.size])
    dp, ds, dg = src.slab(7, 0, "Down")
    d = ix.entry("down_packed#L00007")
    assert d["shape"] == [EXPERTS, COLS, ROWS // 2] and dp.size == COLS * ROWS // 2
    assert np.array_equal(dp, region[d["global_off"]:d["global_off"] + dp.size])


def test_reads_follow_a_tensor_across_shards(tmp_path):
    tensors, total = bank_tensors(7)
    tensors, region = write_checkpoint(tmp_path, shard_cut=tensors[3]["global_off"])   # second shard from the down bank on
    ix = ftw.FtwIndex.open(tmp_path)
    assert ix.shard_count() == 2
    lo = tensors[3]["global_off"] - 100
    assert np.array_equal(ix.read_range(lo, 300), region[lo:lo + 300])
    src = ftw.FtwBanks(ix)
    for part in ("GateUp", "Down"):
        for expert in range(EXPERTS):
            name = ("gate_up" if part == "GateUp" else "down") + "_packed#L00007"
            e = ix.entry(name)
            per = e["nbytes"] // EXPERTS
            got = src.slab(7, expert, part)[0]
            assert np.array_equal(got, region[e["global_off"] + expert * per:e["global_off"] + (expert + 1) * per])


def test_slab_errors_name_what_is_wrong(tmp_path):
    """banks.rs:370-420"""
    write_checkpoint(tmp_path)
    src = ftw.FtwBanks(ftw.FtwIndex.open(tmp_path))
    with pytest.raises(pkg.MoEError) as err:
        src.slab(7, EXPERTS, "GateUp")                      # expert past the bank
    assert err.value.kind == "Bad" and "past 2" in str(err.value)
    with pytest.raises(pkg.MoEError) as err:
        src.slab(9, 0, "GateUp")                            # a layer without entries
    assert err.value.kind == "Missing" and "gate_up_packed#L00009" in str(err.value)
    # a scale entry one scale row short per expert: the three fields no longer agree with the packed shape
    tensors, total = bank_tensors(0)
    tensors[1]["nbytes"] -= EXPERTS * (COLS // 16)
    tensors[1]["shape"] = [EXPERTS, ROWS - 1, COLS // 16]
    bad = ftw.FtwBanks(ftw.FtwIndex.parse(json.dumps(index_doc(tensors, total))))
    with pytest.raises(pkg.MoEError) as err:
        bad.slab(0, 0, "GateUp")
    assert err.value.kind in ("Bad", "Read")


def test_open_refuses_a_truncated_shard(tmp_path):
    tensors, region = write_checkpoint(tmp_path)
    path = os.path.join(tmp_path, "part-0.ftw")
    with open(path, "r+b") as fh:
        fh.truncate(region.size - 10)
    with pytest.raises(pkg.MoEError, match="index claims"):
        ftw.FtwIndex.open(tmp_path)
    os.remove(path)
    with pytest.raises(pkg.MoEError) as err:
        ftw.FtwIndex.open(tmp_path)
    assert err.value.kind == "Read"


def test_draft_prefix_names_the_draft_banks(tmp_path):
    tensors, total = bank_tensors(0, prefix="draft_")
    region = (np.arange(total) % 253).astype(np.uint8)
    region.tofile(os.path.join(tmp_path, "s0.ftw"))
    with open(os.path.join(tmp_path, ftw.INDEX_NAME), "w") as fh:
        json.dump(index_doc(tensors, total), fh)
    ix = ftw.FtwIndex.open(tmp_path)
    packed, _, _ = ftw.FtwBanks(ix, "draft_").slab(0, 0, "GateUp")
    off = ix.entry("draft_gate_up_packed#L00000")["global_off"]
    assert np.array_equal(packed, region[off:off + packed.size])
    with pytest.raises(pkg.MoEError) as err:
        ftw.FtwBanks(ix).slab(0, 0, "GateUp")               # the target's names are not in this checkpoint
    assert err.value.kind == "Missing"


# ------------------------------------------------------------------ into an adapter's resident banks
@pytest.mark.gpu
def test_load_layer_from_a_checkpoint_into_resident_banks(tmp_path):
    """A synthetic checkpoint of two layers x eight experts (hidden 64, inter 32), two shards; every expert of
    both layers goes from the shard files into the adapter's banks and the routed half then matches the CPU path."""
    torch = pytest.importorskip("torch")
    from oracle import oracle as o
    H, I, E, K = 64, 32, 8, 2
    lays = [pkg.synth.make_layer(300 + l, hidden=H, inter=I, experts=E, top_k=K, shared_inter=16) for l in range(2)]
    tensors, off = [], ALIGN
    blobs = []
    for l, lay in enumerate(lays):
        for b, (part, field) in enumerate([(p, f) for p in ("gate_up", "down") for f in ("packed", "scale", "global")]):
            data = np.ascontiguousarray(lay.banks[b]).reshape(-1)
            rows = 2 * I if part == "gate_up" else H
            tensors.append({"name": f"{part}_{field}#L{l:05d}", "kind": "experts_bank", "dtype": "uint8",
                            "shape": [E, rows, data.size // (E * rows)], "global_off": off, "nbytes": int(data.size)})
            blobs.append((off, data))
            off += (data.size + ALIGN - 1) // ALIGN * ALIGN
    region = np.zeros(off, np.uint8)
    for o_, d in blobs:
        region[o_:o_ + d.size] = d
    cut = tensors[7]["global_off"]
    shards = [{"file": "a.ftw", "global_off": 0, "nbytes": cut}, {"file": "b.ftw", "global_off": cut, "nbytes": off - cut}]
    region[:cut].tofile(os.path.join(tmp_path, "a.ftw"))
    region[cut:].tofile(os.path.join(tmp_path, "b.ftw"))
    with open(os.path.join(tmp_path, ftw.INDEX_NAME), "w") as fh:
        json.dump(index_doc(tensors, off, shards, expert_bank_num_layers=2), fh)
    src = ftw.FtwBanks(ftw.FtwIndex.open(tmp_path))
    moe = pkg.B200MoE(0, pkg.ExpertShapes(H, I), 2 * E, experts=E, layers=2, top_k=K, shared_inter=16, max_tokens=8)
    for l in range(2):
        src.load_layer(moe, l)
    banks = moe.bank_tensors()
    for l, lay in enumerate(lays):
        for b in range(6):
            got = banks[b][l * E:(l + 1) * E].cpu().numpy()
            assert np.array_equal(got, np.ascontiguousarray(lay.banks[b]).reshape(E, -1)), (l, b)
        assert moe.slot_of(l, 3) == l * E + 3
    # and the loaded experts compute
    dev = torch.device("cuda:0")
    tokens = 5
    xb = pkg.synth.make_x(3, tokens, H)
    rng = np.random.default_rng(1)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(tokens)]).astype(np.int32)
    w = rng.uniform(0.1, 0.6, (tokens, K)).astype(np.float32)
    out = torch.empty((tokens, H), dtype=torch.float32, device=dev)
    x_d = torch.from_numpy(xb.view(np.int16)).to(dev).view(torch.bfloat16)
    moe.grouped_moe_staged(pkg.MoEDeviceRequest(1, H, I, K, x_d, torch.from_numpy(ids).to(dev), torch.from_numpy(w).to(dev)), out)
    moe.sync_status()
    hb = o.HostBanks(*lays[1].banks, slots=E, gu_rows=2 * I, gu_cols=H, dn_rows=H, dn_cols=I)
    want = o.grouped_moe_reference(hb, H, I, pkg.synth.bf16_bits_to_f32(xb), K, ids.reshape(-1), w.reshape(-1))
    assert np.linalg.norm(out.cpu().numpy() - want) <= 1e-2 * np.linalg.norm(want)
    # a layer the checkpoint does not hold, a bank that does not fit the adapter's rows
    with pytest.raises(pkg.MoEError) as err:
        src.load_layer(moe, 1, first_expert=6, n_experts=4, slot0=0)
    assert err.value.kind == "Bad"
    moe.close()
