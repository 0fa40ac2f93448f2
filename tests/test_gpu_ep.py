"""Expert parallelism on real GPUs (needs at least two): the n-rank result equals the single-GPU result
on the same seeded inputs.  Needs two GPUs; skipped on a one-GPU box."""
import importlib
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
pkg = importlib.import_module("ferrum-torrens_b200")

H, I, E, K, SI = 2048, 512, 32, 8, 512


def _bf16(bits, dev):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(dev).view(torch.bfloat16)


def _worker(rank, world, port, tokens, q):
    import datetime
    import torch.distributed as dist
    ep = importlib.import_module("ferrum-torrens_b200.ep")
    # plain peer stores only: no NVLink multicast object is bound to the symmetric buffers, so a rank that
    # dies leaves nothing behind on its peers' GPUs
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    torch.cuda.set_device(rank)
    dev = torch.device(f"cuda:{rank}")
    # a short collective timeout: if the other rank raised before a collective, this one errors out of it
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        lay = pkg.synth.make_layer(77, hidden=H, inter=I, experts=E, top_k=K, shared_inter=SI)
        xb = pkg.synth.make_x(500 + rank, tokens, H)
        be = ep.LibBackend(rank, rank, world, pkg.ExpertShapes(H, I), experts=E, layers=1, top_k=K, shared_inter=SI,
                           max_tokens=tokens)
        for e in range(E):
            if be.owned(e):
                be.load_expert(0, e, lay.fields(e))
        layer = ep.ExpertParallelMoE(be, world)
        out = torch.empty((tokens, H), dtype=torch.float32, device=dev)
        w = [_bf16(a, dev) for a in (lay.gate_w, lay.sh_gate_up, lay.sh_down, lay.sh_gate)]
        ids, wts = layer.forward(0, _bf16(xb, dev), *w, out)
        be.front.sync_status()
        be.owner.sync_status()
        # the same tokens through one adapter that holds every expert
        solo = pkg.B200MoE(rank, pkg.ExpertShapes(H, I), E, experts=E, layers=1, top_k=K, shared_inter=SI,
                           max_tokens=tokens)
        for e in range(E):
            solo.load(0, e, e, lay.fields(e))
        want = torch.empty((tokens, H), dtype=torch.float32, device=dev)
        want_ids = torch.empty((tokens, K), dtype=torch.int32, device=dev)
        solo.moe_block(0, _bf16(xb, dev), *w, want, ids_out=want_ids)
        solo.sync_status()
        same_ids = bool(torch.equal(ids, want_ids))
        rel = float((out - want).norm() / want.norm())
        # the overlapped schedule (exchanges under compute) gives the same block
        out2 = torch.empty_like(out)
        layer.forward_overlapped(0, _bf16(xb, dev), *w, out2, chunks=2)
        be.front.sync_status()
        be.owner.sync_status()
        rel = max(rel, float((out2 - want).norm() / want.norm()))
        # both exchanges by the library's own kernels over peer memory (two steps: the buffers are reused)
        be.enable_peer_exchange()
        # (then the step cut into two and three micro-batches, each with its own region of the buffers)
        for micro, fused in ((1, False), (1, True), (2, False), (3, True)):
            out3 = torch.zeros_like(out)
            ids3, _ = layer.forward_p2p(0, _bf16(xb, dev), *w, out3, micro=micro, fused_return=fused)
            be.front.sync_status()
            be.owner.sync_status()
            same_ids = same_ids and bool(torch.equal(ids3, want_ids))
            rel = max(rel, float((out3 - want).norm() / want.norm()))
        # rows dispatched straight into the owner's sorted matrix (small steps fall back to the exchange above)
        out4 = torch.zeros_like(out)
        ids4, _ = layer.forward_p2p_sorted(0, _bf16(xb, dev), *w, out4)
        be.front.sync_status()
        be.owner.sync_status()
        same_ids = same_ids and bool(torch.equal(ids4, want_ids))
        rel = max(rel, float((out4 - want).norm() / want.norm()))
        q.put((rank, same_ids, rel, None))
        solo.close()
        be.close()
    except BaseException as exc:   # the parent fails fast instead of waiting for the queue
        q.put((rank, False, float("inf"), repr(exc)[:500]))
        raise
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("tokens", [16, 700])
def test_two_gpu_expert_parallel_matches_single_gpu(tokens):
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, tokens, q)) for r in range(2)]
    res = []
    try:
        for p in procs:
            p.start()
        for _ in procs:
            r = q.get(timeout=300)
            res.append(r)
            if r[3] is not None:   # a rank raised: do not wait for the other, it is killed below
                break
        if all(r[3] is None for r in res):
            for p in procs:
                p.join(60)
    finally:
        # no worker outlives the test: a rank left inside a collective would keep spinning on its GPU
        for p in procs:
            if p.is_alive():
                p.kill()
                p.join(10)
    for r in res:
        assert r[3] is None, f"rank {r[0]} raised: {r[3]}"
    assert len(res) == len(procs)
    for p in procs:
        assert p.exitcode == 0
    for rank, same_ids, rel, _ in res:
        assert same_ids
        # the owner returns bf16 rows (half the NVLink bytes); one rounding per route
        assert rel < 5e-3, (rank, rel)
