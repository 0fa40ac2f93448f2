"""Expert-parallel exchange logic on CPU: two gloo ranks, a numpy double over the CPU checker standing
in for the CUDA library on both sides of the all-to-all.  The n-rank result must equal the 1-rank
result on the same seeded inputs (ids bit-exact, outputs equal up to f32 summation order)."""
import importlib
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pkg = importlib.import_module("ferrum-torrens_b200")
ep = importlib.import_module("ferrum-torrens_b200.ep")
from oracle import oracle as o  # noqa: E402

H, I, E, K, SI = 64, 32, 8, 2, 32


def _oracle_layer(lay):
    banks = o.HostBanks(*lay.banks, slots=E, gu_rows=2 * I, gu_cols=H, dn_rows=H, dn_cols=I)
    return o.Layer(H, I, E, K, SI, lay.gate_w, lay.sh_gate_up, lay.sh_down, lay.sh_gate, banks)


class OracleBackend:
    """Same five methods as ep.LibBackend, on CPU tensors."""

    def __init__(self, rank, world, lay):
        self.rank, self.world, self.ol = rank, world, _oracle_layer(lay)
        self.per = E // world

    def route(self, x, gate_w):
        ids, w = o.router(self.ol, x.numpy())
        return torch.from_numpy(ids), torch.from_numpy(w)

    def shared(self, x, a, b, c):
        xf = x.numpy()
        g = o.bf16_gemm(xf, self.ol.sh_gate, xf.shape[0], 1, H).reshape(-1)
        gate = np.array([o.sigmoid(float(v)) for v in g], np.float32)
        return torch.from_numpy(o.shared_expert(self.ol, xf)), torch.from_numpy(gate)

    def pack(self, x, ids, w):
        flat = ids.numpy().reshape(-1)
        seg, route_idx = o.build_grouped_csr(flat, E)
        send_x = x[torch.from_numpy(route_idx // K).long()]
        counts = np.array([seg[(p + 1) * self.per] - seg[p * self.per] for p in range(self.world)], np.int32)
        return (send_x.contiguous(), torch.from_numpy(flat[route_idx].copy()),
                torch.from_numpy(w.numpy().reshape(-1)[route_idx].copy()), torch.from_numpy(route_idx), torch.from_numpy(counts))

    def experts_forward(self, layer, recv_x, recv_e, recv_w):
        e = recv_e.numpy()
        assert ((e // self.per) == self.rank).all(), "a rank only receives routes of experts it owns"
        if recv_x.shape[0] == 0:
            return torch.zeros((0, H))
        y = o.grouped_moe_reference(self.ol.banks, H, I, recv_x.numpy(), 1, e, recv_w.numpy())
        return torch.from_numpy(np.ascontiguousarray(y))

    def combine(self, y, route_idx, shared, se_gate, out):
        pos = np.empty(route_idx.numel(), np.int64)
        pos[route_idx.numpy()] = np.arange(route_idx.numel())
        yn = y.numpy()
        res = shared.numpy() * se_gate.numpy()[:, None]
        for t in range(out.shape[0]):
            for j in range(K):
                res[t] = res[t] + yn[pos[t * K + j]]
        out.copy_(torch.from_numpy(res))


def _worker(rank, world, port, tokens_per_rank, q):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=90))
    try:
        lay = pkg.synth.make_layer(21, hidden=H, inter=I, experts=E, top_k=K, shared_inter=SI)
        x = torch.from_numpy(pkg.synth.bf16_bits_to_f32(pkg.synth.make_x(100 + rank, tokens_per_rank[rank], H)))
        layer = ep.ExpertParallelMoE(OracleBackend(rank, world, lay), world)
        out = torch.empty((x.shape[0], H))
        ids, w = layer.forward(0, x, None, True, None, None, out)
        want, want_ids, want_w = o.moe_block(_oracle_layer(lay), x.numpy())
        assert np.array_equal(ids.numpy(), want_ids)
        err = np.abs(out.numpy() - want).max() / np.abs(want).max()
        sc, rc = layer.last_counts
        # the overlapped schedule (expert ranges exchanged and computed one after the other) gives the same block
        for chunks in (2, 4):
            out2 = torch.empty_like(out)
            ids2, _ = layer.forward_overlapped(0, x, None, True, None, None, out2, chunks=chunks)
            assert np.array_equal(ids2.numpy(), want_ids)
            assert np.abs(out2.numpy() - out.numpy()).max() <= 1e-6 * np.abs(want).max(), chunks
        q.put((rank, float(err), sc, rc, None))
    except BaseException as exc:   # the parent fails fast instead of waiting for the queue
        q.put((rank, float("inf"), [], [], repr(exc)[:500]))
        raise
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("tokens_per_rank", [(5, 9), (1, 0 + 3)])
def test_two_ranks_match_single_rank(tokens_per_rank):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, tokens_per_rank, q)) for r in range(2)]
    res = []
    try:
        for p in procs:
            p.start()
        for _ in procs:
            r = q.get(timeout=120)
            res.append(r)
            if r[4] is not None:
                break
        if all(r[4] is None for r in res):
            for p in procs:
                p.join(60)
    finally:
        for p in procs:   # no worker outlives the test
            if p.is_alive():
                p.kill()
                p.join(10)
    for r in res:
        assert r[4] is None, f"rank {r[0]} raised: {r[4]}"
    for p in procs:
        assert p.exitcode == 0
    res = sorted(r[:4] for r in res)
    for rank, err, sc, rc in res:
        assert err < 1e-5, (rank, err)
        assert sum(sc) == tokens_per_rank[rank] * K
    # what rank 0 sends to rank 1 is what rank 1 receives from rank 0, and vice versa
    assert res[0][2][1] == res[1][3][0] and res[1][2][0] == res[0][3][1]


def test_owner_partition():
    assert [ep.owner_of(e, 256, 8) for e in (0, 31, 32, 255)] == [0, 0, 1, 7]
