"""The peer-memory exchange kernels (ftm_ep_plan / ftm_ep_dispatch / ftm_ep_return / ftm_ep_combine) for
4 and 8 ranks, emulated on ONE GPU: every "rank" is a pair of adapter handles in this process and the peer
pointer arrays point at the other ranks' buffers on the same device.  The kernels of different ranks do not
wait for one another (the ordering between the phases is the host's), so they run one after the other here.
The result of every rank must equal the block computed by one adapter that holds all experts."""
import importlib

import numpy as np
import pytest
import torch

pkg = importlib.import_module("ferrum-torrens_b200")

pytestmark = pytest.mark.gpu

H, I, E, K, SI = 256, 64, 16, 4, 64


def _bf16(bits, dev):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(dev).view(torch.bfloat16)


@pytest.mark.parametrize("world,tokens", [(4, [37, 5, 64, 1]), (8, [9, 33, 2, 17, 40, 1, 8, 21])])
def test_peer_exchange_kernels_many_ranks_on_one_gpu(world, tokens):
    dev = torch.device("cuda:0")
    lay = pkg.synth.make_layer(91, hidden=H, inter=I, experts=E, top_k=K, shared_inter=SI)
    shapes = pkg.ExpertShapes(H, I)
    per = E // world
    maxtok = max(tokens)
    cap = sum(tokens) * K
    dense = [_bf16(a, dev) for a in (lay.gate_w, lay.sh_gate_up, lay.sh_down, lay.sh_gate)]

    solo = pkg.B200MoE(0, shapes, E, experts=E, layers=1, top_k=K, shared_inter=SI, max_tokens=maxtok)
    for e in range(E):
        solo.load(0, e, e, lay.fields(e))
    fronts, owners = [], []
    for r in range(world):
        fronts.append(pkg.B200MoE(0, shapes, 1, experts=E, layers=1, top_k=K, shared_inter=SI, max_tokens=maxtok))
        ow = pkg.B200MoE(0, shapes, per, experts=E, layers=1, top_k=1, shared_inter=0, max_tokens=cap)
        for e in range(r * per, (r + 1) * per):
            ow.load(0, e, e - r * per, lay.fields(e))
        owners.append(ow)

    xs = [_bf16(pkg.synth.make_x(700 + r, tokens[r], H), dev) for r in range(world)]
    recv_x = [torch.zeros((cap, H), dtype=torch.bfloat16, device=dev) for _ in range(world)]
    recv_m = [torch.zeros((cap, 2), dtype=torch.int32, device=dev) for _ in range(world)]
    back = [torch.zeros((tokens[r] * K, H), dtype=torch.bfloat16, device=dev) for r in range(world)]
    ptrs = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    peer_x, peer_m, peer_back = ptrs(recv_x), ptrs(recv_m), ptrs(back)

    routed = []
    for r in range(world):
        ids, w = fronts[r].router(xs[r], dense[0])
        route_idx, counts = fronts[r].ep_plan(ids, world)
        routed.append((ids, w, route_idx, counts))
    counts_all = torch.cat([c for _, _, _, c in routed]).contiguous()             # the all-gather
    ca = counts_all.reshape(world, world).cpu().numpy()
    assert ca.sum(axis=1).tolist() == [t * K for t in tokens]
    for r in range(world):
        ids, w, route_idx, _ = routed[r]
        fronts[r].ep_dispatch(xs[r], ids, w, route_idx, world, r, counts_all, peer_x.data_ptr(), peer_m.data_ptr(), cap)
    torch.cuda.synchronize()                                                       # the barrier
    for r in range(world):
        n = int(ca[:, r].sum())
        meta = recv_m[r][:n]
        assert bool(((meta[:, 0] // per) == r).all()), "a rank only receives routes of experts it owns"
        if n:
            y = torch.empty((n, H), dtype=torch.bfloat16, device=dev)
            req = pkg.MoEDeviceRequest(0, H, I, 1, recv_x[r][:n], meta[:, 0].contiguous().reshape(n, 1),
                                       meta[:, 1].contiguous().view(torch.float32).reshape(n, 1))
            owners[r].grouped_moe_staged(req, y)
            owners[r].ep_return(y, world, r, counts_all, peer_back.data_ptr(), min(tokens) * K)
    torch.cuda.synchronize()                                                       # the barrier
    # the smallest back buffer was given as the capacity of all: rows beyond it are dropped and reported, so
    # redo the return with each source's real capacity only when the sizes differ
    if len(set(tokens)) > 1:
        statuses = []
        for r in range(world):
            try:
                owners[r].sync_status()
                statuses.append(True)
            except pkg.MoEError:
                statuses.append(False)
        assert not all(statuses), "rows past the given capacity must be reported, not stored"
        cap_back = max(tokens) * K
        back = [torch.zeros((cap_back, H), dtype=torch.bfloat16, device=dev) for _ in range(world)]
        peer_back = ptrs(back)
        for r in range(world):
            n = int(ca[:, r].sum())
            if n:
                meta = recv_m[r][:n]
                y = torch.empty((n, H), dtype=torch.bfloat16, device=dev)
                req = pkg.MoEDeviceRequest(0, H, I, 1, recv_x[r][:n], meta[:, 0].contiguous().reshape(n, 1),
                                           meta[:, 1].contiguous().view(torch.float32).reshape(n, 1))
                owners[r].grouped_moe_staged(req, y)
                owners[r].ep_return(y, world, r, counts_all, peer_back.data_ptr(), cap_back)
        torch.cuda.synchronize()
    for r in range(world):
        owners[r].sync_status()
        fronts[r].sync_status()
        ids, w, route_idx, _ = routed[r]
        shared, se_gate = fronts[r].shared_expert(xs[r], dense[1], dense[2], dense[3])
        out = torch.empty((tokens[r], H), dtype=torch.float32, device=dev)
        fronts[r].ep_combine(back[r][:tokens[r] * K], route_idx, shared, se_gate, out)
        want = torch.empty((tokens[r], H), dtype=torch.float32, device=dev)
        want_ids = torch.empty((tokens[r], K), dtype=torch.int32, device=dev)
        solo.moe_block(0, xs[r], *dense, want, ids_out=want_ids)
        solo.sync_status()
        assert torch.equal(ids, want_ids)
        rel = float((out - want).norm() / want.norm())
        assert rel < 5e-3, (r, rel)     # one bf16 rounding per returned row
    for m in fronts + owners + [solo]:
        m.close()


def test_dispatch_reports_an_expert_id_outside_the_layer_instead_of_following_it():
    """An id outside [0, experts) reaches ftm_ep_plan / ftm_ep_dispatch: the permutation build flags it and
    leaves that route's position unwritten, and the dispatch kernel must raise the error status without
    indexing anything with it (every index is checked before the load that depends on it)."""
    dev = torch.device("cuda:0")
    world, tokens = 4, 6
    lay = pkg.synth.make_layer(92, hidden=H, inter=I, experts=E, top_k=K, shared_inter=SI)
    front = pkg.B200MoE(0, pkg.ExpertShapes(H, I), 1, experts=E, layers=1, top_k=K, shared_inter=SI, max_tokens=tokens)
    x = _bf16(pkg.synth.make_x(5, tokens, H), dev)
    ids, w = front.router(x, _bf16(lay.gate_w, dev))
    front.sync_status()
    cap = tokens * K
    recv_x = [torch.zeros((cap, H), dtype=torch.bfloat16, device=dev) for _ in range(world)]
    recv_m = [torch.zeros((cap, 2), dtype=torch.int32, device=dev) for _ in range(world)]
    ptrs = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    peer_x, peer_m = ptrs(recv_x), ptrs(recv_m)
    for bad in (-1, E + 3):
        bad_ids = ids.clone()
        bad_ids[2, 1] = bad
        route_idx, counts = front.ep_plan(bad_ids, world)
        counts_all = torch.zeros((world * world,), dtype=torch.int32, device=dev)
        counts_all[:world] = counts                 # this "rank" is rank 0, the others send nothing
        front.ep_dispatch(x, bad_ids, w, route_idx, world, 0, counts_all, peer_x.data_ptr(), peer_m.data_ptr(), cap)
        with pytest.raises(pkg.MoEError):
            front.sync_status()
        try:                                         # both flags (bad id, dropped row) may be pending: drain them
            front.sync_status()
        except pkg.MoEError:
            pass
        front.sync_status()
    # a clean step after the bad ones still works
    route_idx, counts = front.ep_plan(ids, world)
    counts_all = torch.zeros((world * world,), dtype=torch.int32, device=dev)
    counts_all[:world] = counts
    front.ep_dispatch(x, ids, w, route_idx, world, 0, counts_all, peer_x.data_ptr(), peer_m.data_ptr(), cap)
    front.sync_status()
    assert int(sum(int(m[:, 0].ge(0).sum()) for m in recv_m)) > 0
    front.close()


def test_sorted_return_on_the_grouped_gemm_path_emulated():
    """Steps large enough for the grouped GEMM (more than 2048 received rows per owner, production expert shape):
    the owner leaves its rows sorted by expert and the return kernel stores them from there
    (ftm_ep_experts_sorted + ftm_ep_return_sorted).  Two ranks on one GPU; every rank's result must equal the
    block computed by one adapter that holds all experts, and the ordinary return path on the same step."""
    dev = torch.device("cuda:0")
    Hh, Ii, Ee, Kk, Ss = 2048, 512, 16, 4, 512
    world, tokens = 2, [700, 650]
    lay = pkg.synth.make_layer(93, hidden=Hh, inter=Ii, experts=Ee, top_k=Kk, shared_inter=Ss)
    shapes = pkg.ExpertShapes(Hh, Ii)
    per = Ee // world
    cap = sum(tokens) * Kk
    dense = [_bf16(a, dev) for a in (lay.gate_w, lay.sh_gate_up, lay.sh_down, lay.sh_gate)]
    solo = pkg.B200MoE(0, shapes, Ee, experts=Ee, layers=1, top_k=Kk, shared_inter=Ss, max_tokens=max(tokens))
    for e in range(Ee):
        solo.load(0, e, e, lay.fields(e))
    fronts, owners = [], []
    for r in range(world):
        fronts.append(pkg.B200MoE(0, shapes, 1, experts=Ee, layers=1, top_k=Kk, shared_inter=Ss, max_tokens=max(tokens)))
        ow = pkg.B200MoE(0, shapes, per, experts=Ee, layers=1, top_k=1, shared_inter=0, max_tokens=cap)
        for e in range(r * per, (r + 1) * per):
            ow.load(0, e, e - r * per, lay.fields(e))
        owners.append(ow)
    xs = [_bf16(pkg.synth.make_x(800 + r, tokens[r], Hh), dev) for r in range(world)]
    recv_x = [torch.zeros((cap, Hh), dtype=torch.bfloat16, device=dev) for _ in range(world)]
    recv_m = [torch.zeros((cap, 2), dtype=torch.int32, device=dev) for _ in range(world)]
    ptrs = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    peer_x, peer_m = ptrs(recv_x), ptrs(recv_m)
    routed = []
    for r in range(world):
        ids, w = fronts[r].router(xs[r], dense[0])
        route_idx, counts = fronts[r].ep_plan(ids, world)
        routed.append((ids, w, route_idx, counts))
    counts_all = torch.cat([c for _, _, _, c in routed]).contiguous()
    ca = counts_all.reshape(world, world).cpu().numpy()
    for r in range(world):
        ids, w, route_idx, _ = routed[r]
        fronts[r].ep_dispatch(xs[r], ids, w, route_idx, world, r, counts_all, peer_x.data_ptr(), peer_m.data_ptr(), cap)
    torch.cuda.synchronize()
    results = {}
    for mode in ("sorted", "fused", "plain"):
        back = [torch.zeros((tokens[r] * Kk, Hh), dtype=torch.bfloat16, device=dev) for r in range(world)]
        peer_back = ptrs(back)
        for r in range(world):
            n = int(ca[:, r].sum())
            assert n > 2048, "the case must reach the grouped GEMM"
            meta = recv_m[r][:n]
            rids, rw = meta[:, 0].contiguous(), meta[:, 1].contiguous().view(torch.float32)
            if mode == "sorted":
                assert owners[r].ep_experts_sorted(0, recv_x[r][:n], rids, rw)
                owners[r].ep_return_sorted(n, world, r, counts_all, peer_back.data_ptr(), max(tokens) * Kk)
            elif mode == "fused":
                assert owners[r].ep_experts_return(0, recv_x[r][:n], rids, rw, world, r, counts_all, peer_back.data_ptr(),
                                                   max(tokens) * Kk)
            else:
                y = torch.empty((n, Hh), dtype=torch.bfloat16, device=dev)
                owners[r].grouped_moe_staged(pkg.MoEDeviceRequest(0, Hh, Ii, 1, recv_x[r][:n], rids.reshape(n, 1),
                                                                  rw.reshape(n, 1)), y)
                owners[r].ep_return(y, world, r, counts_all, peer_back.data_ptr(), max(tokens) * Kk)
        torch.cuda.synchronize()
        for r in range(world):
            owners[r].sync_status()
        results[mode] = back
    for r in range(world):
        assert torch.equal(results["sorted"][r], results["plain"][r]), "the same rows, whichever pass stored them"
        assert torch.equal(results["fused"][r], results["plain"][r]), "the same rows when the GEMM stores them itself"
        ids, w, route_idx, _ = routed[r]
        shared, se_gate = fronts[r].shared_expert(xs[r], dense[1], dense[2], dense[3])
        out = torch.empty((tokens[r], Hh), dtype=torch.float32, device=dev)
        fronts[r].ep_combine(results["sorted"][r], route_idx, shared, se_gate, out)
        want = torch.empty((tokens[r], Hh), dtype=torch.float32, device=dev)
        want_ids = torch.empty((tokens[r], Kk), dtype=torch.int32, device=dev)
        solo.moe_block(0, xs[r], *dense, want, ids_out=want_ids)
        solo.sync_status()
        assert torch.equal(ids, want_ids)
        rel = float((out - want).norm() / want.norm())
        assert rel < 5e-3, (r, rel)
    # the same step with the rows dispatched straight into the owners' sorted activation matrices: no permutation
    # build and no gather on the owner; the rows reach the GEMMs in the same order, so the results are bit-equal
    plans = [fronts[r].ep_plan_seg(routed[r][0]) for r in range(world)]
    seg_all = torch.stack([sg for _, sg in plans]).contiguous()
    for r in range(world):
        assert torch.equal(plans[r][0], routed[r][2]), "the same send order as ep_plan"
    xg = [torch.zeros((cap, Hh), dtype=torch.float16, device=dev) for _ in range(world)]
    wbuf = [torch.zeros((cap,), dtype=torch.float32, device=dev) for _ in range(world)]
    rsbuf = [torch.zeros((cap,), dtype=torch.float32, device=dev) for _ in range(world)]
    peer_xg, peer_w, peer_rs = ptrs(xg), ptrs(wbuf), ptrs(rsbuf)
    for r in range(world):
        ids, w, route_idx, _ = routed[r]
        fronts[r].ep_dispatch_sorted(xs[r], ids, w, route_idx, world, r, seg_all, peer_xg.data_ptr(), peer_w.data_ptr(),
                                     peer_rs.data_ptr(), cap)
    torch.cuda.synchronize()
    back = [torch.zeros((tokens[r] * Kk, Hh), dtype=torch.bfloat16, device=dev) for r in range(world)]
    peer_back = ptrs(back)
    for r in range(world):
        n = int(ca[:, r].sum())
        owners[r].ep_experts_presorted(0, xg[r], wbuf[r], rsbuf[r], n, world, r, seg_all, peer_back.data_ptr(), max(tokens) * Kk)
    torch.cuda.synchronize()
    for r in range(world):
        fronts[r].sync_status()
        owners[r].sync_status()
        assert torch.equal(back[r], results["plain"][r]), "the same rows when they arrive sorted"
    # a step of at most 2048 rows is not taken by this path
    n_small = 100
    assert owners[0].ep_experts_sorted(0, recv_x[0][:n_small], recv_m[0][:n_small, 0].contiguous(),
                                       recv_m[0][:n_small, 1].contiguous().view(torch.float32)) is False
    for m in fronts + owners + [solo]:
        m.close()


def test_sorted_dispatch_with_an_expert_that_is_not_resident_and_with_a_short_buffer():
    """ftm_ep_dispatch_sorted / ftm_ep_experts_presorted, two ranks on one GPU: the rows of an expert the owner does
    not hold come back as zeros and every other row equals the ordinary path's; a receive matrix that is too short
    raises the status flag instead of a store outside it."""
    dev = torch.device("cuda:0")
    Hh, Ii, Ee, Kk = 2048, 512, 16, 4
    world, tokens = 2, [680, 690]
    lay = pkg.synth.make_layer(97, hidden=Hh, inter=Ii, experts=Ee, top_k=Kk, shared_inter=0)
    shapes = pkg.ExpertShapes(Hh, Ii)
    per = Ee // world
    cap = sum(tokens) * Kk
    missing = 3
    gate = _bf16(lay.gate_w, dev)
    fronts, owners = [], []
    for r in range(world):
        fronts.append(pkg.B200MoE(0, shapes, 1, experts=Ee, layers=1, top_k=Kk, shared_inter=0, max_tokens=max(tokens)))
        ow = pkg.B200MoE(0, shapes, per, experts=Ee, layers=1, top_k=1, shared_inter=0, max_tokens=cap)
        for e in range(r * per, (r + 1) * per):
            if e != missing:
                ow.load(0, e, e - r * per, lay.fields(e))
        owners.append(ow)
    xs = [_bf16(pkg.synth.make_x(900 + r, tokens[r], Hh), dev) for r in range(world)]
    ptrs = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    routed, plans = [], []
    for r in range(world):
        ids, w = fronts[r].router(xs[r], gate)
        route_idx, seg = fronts[r].ep_plan_seg(ids)
        routed.append((ids, w, route_idx))
        plans.append(seg)
    seg_all = torch.stack(plans).contiguous()
    sa = seg_all.cpu().numpy()
    recv = [int(sum(sa[s][(p + 1) * per] - sa[s][p * per] for s in range(world))) for p in range(world)]
    assert min(recv) > 2048
    xg = [torch.zeros((cap, Hh), dtype=torch.float16, device=dev) for _ in range(world)]
    wbuf = [torch.zeros((cap,), dtype=torch.float32, device=dev) for _ in range(world)]
    rsbuf = [torch.zeros((cap,), dtype=torch.float32, device=dev) for _ in range(world)]
    # the address tables stay alive for as long as a kernel may read them
    peer_xg, peer_w, peer_rs = ptrs(xg), ptrs(wbuf), ptrs(rsbuf)
    for r in range(world):
        ids, w, route_idx = routed[r]
        fronts[r].ep_dispatch_sorted(xs[r], ids, w, route_idx, world, r, seg_all, peer_xg.data_ptr(), peer_w.data_ptr(),
                                     peer_rs.data_ptr(), cap)
    torch.cuda.synchronize()
    back = [torch.full((tokens[r] * Kk, Hh), 7.0, dtype=torch.bfloat16, device=dev) for r in range(world)]
    peer_back = ptrs(back)
    for r in range(world):
        owners[r].ep_experts_presorted(0, xg[r], wbuf[r], rsbuf[r], recv[r], world, r, seg_all, peer_back.data_ptr(),
                                       max(tokens) * Kk)
    torch.cuda.synchronize()
    for r in range(world):
        fronts[r].sync_status()
        owners[r].sync_status()
        ids, w, route_idx = routed[r]
        # reference: every route through the ordinary staged call on its owner (missing expert -> zeros)
        e_of_pos = ids.reshape(-1)[route_idx.long()]
        for p in range(world):
            sel = ((e_of_pos // per) == p).nonzero().reshape(-1)
            if sel.numel() == 0:
                continue
            rows = xs[r][(route_idx[sel] // Kk).long()].contiguous()
            y = torch.empty((sel.numel(), Hh), dtype=torch.bfloat16, device=dev)
            owners[p].grouped_moe_staged(pkg.MoEDeviceRequest(0, Hh, Ii, 1, rows, e_of_pos[sel].reshape(-1, 1).contiguous(),
                                                              w.reshape(-1)[route_idx[sel].long()].reshape(-1, 1).contiguous()), y)
            torch.cuda.synchronize()
            got = back[r][sel]
            gone = (e_of_pos[sel] == missing)
            assert torch.equal(got[gone], torch.zeros_like(got[gone])), "rows of the expert that is not resident are zeros"
            assert gone.any() or p != missing // per
            rel = float((got[~gone].float() - y[~gone].float()).norm() / y[~gone].float().norm())
            assert rel < 5e-3, (r, p, rel)
    # a receive matrix shorter than the rows it is sent: nothing is stored outside it, the status says so
    short = 100
    with pytest.raises(pkg.MoEError):
        fronts[0].ep_dispatch_sorted(xs[0], routed[0][0], routed[0][1], routed[0][2], world, 0, seg_all, peer_xg.data_ptr(),
                                     peer_w.data_ptr(), peer_rs.data_ptr(), short)
        fronts[0].sync_status()
    for m in fronts + owners:
        m.close()
