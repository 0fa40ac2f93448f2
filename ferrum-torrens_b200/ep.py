"""Expert-parallel MoE layer: 256 experts split evenly over the ranks of one node.

The reference is a single-GPU engine (README.md:132 of butzist/ferrum-torrens: "One GPU, one
process"), so this partition has no counterpart there; parity is defined as "the n-rank result equals
the 1-rank result on the same seeded inputs".

Per layer and rank (tokens are data-parallel, experts are owned in contiguous blocks):

    router (replicated gate weight)              ids [T, k], weights [T, k]
    pack     sort the routes by owner / expert   send_x, send_expert, send_weight, counts
    exchange counts, then all-to-all(v) of the three send buffers          (NCCL over NVLink)
    experts  the owner runs its resident experts on the received routes     y [R_recv, H] (weighted)
    exchange all-to-all(v) of y back
    combine  out[t] = se_gate[t] * shared[t] + sum_j y[position of route (t, j)]

`ExpertParallelMoE` drives the exchange; what runs on each side of it is a *backend*: `LibBackend`
(the CUDA library, two adapter handles per rank: a front handle for router / shared expert / pack /
combine, and an owner handle created with top_k = 1 that holds the rank's experts) or any object with
the same five methods (the CPU tests use a numpy double over the CPU checker).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import moe as _moe


@dataclass
class EPTimes:
    """CUDA events of one forward (None on CPU)."""
    events: list


def owner_of(expert: int, experts: int, world: int) -> int:
    return expert // (experts // world)


def exchange_counts(counts: torch.Tensor, group=None) -> torch.Tensor:
    """counts[p] = routes this rank sends to rank p  ->  recv[p] = routes rank p sends here."""
    recv = torch.empty_like(counts)
    dist.all_to_all_single(recv, counts, group=group)
    return recv


def all_to_all_rows(send: torch.Tensor, send_counts: list[int], recv_counts: list[int], group=None) -> torch.Tensor:
    """all-to-all(v) of the leading dimension."""
    out = send.new_empty((sum(recv_counts),) + tuple(send.shape[1:]))
    dist.all_to_all_single(out, send, output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    return out


class _Done:
    def wait(self):
        return True


def all_to_all_views(outs, ins, group=None):
    """Asynchronous all-to-all of one tensor view per peer (no staging copy with NCCL).  Backends
    without the list form (gloo, on the CPU tests) go through one contiguous exchange."""
    if dist.get_backend(group) == "nccl":
        return dist.all_to_all(outs, ins, group=group, async_op=True)
    width = 1
    for d in ins[0].shape[1:]:
        width *= d
    flat_in = torch.cat([t.reshape(t.shape[0], width) for t in ins])
    n_out = sum(t.shape[0] for t in outs)
    flat_out = flat_in.new_empty((n_out, width))
    dist.all_to_all_single(flat_out, flat_in, output_split_sizes=[t.shape[0] for t in outs],
                           input_split_sizes=[t.shape[0] for t in ins], group=group)
    at = 0
    for t in outs:
        t.copy_(flat_out[at:at + t.shape[0]].reshape(t.shape))
        at += t.shape[0]
    return _Done()


class LibBackend:
    """The CUDA library on both sides of the exchange."""

    def __init__(self, device: int, rank: int, world: int, shapes: _moe.ExpertShapes, *, experts: int = 256,
                 layers: int = 1, top_k: int = 8, shared_inter: int = 512, max_tokens: int = 8192,
                 recv_capacity: int | None = None, comm_sms: int = 0):
        if experts % world:
            raise _moe.bad(f"{experts} experts do not split over {world} ranks")
        self.rank, self.world, self.experts, self.layers, self.top_k = rank, world, experts, layers, top_k
        self.per = experts // world
        self.shapes = shapes
        # front: router, shared expert, pack, combine (its banks are never used: one slot)
        self.front = _moe.B200MoE(device, shapes, 1, experts=experts, layers=layers, top_k=top_k,
                                  shared_inter=shared_inter, max_tokens=max_tokens)
        self._fronts = [self.front]
        # owner: this rank's experts, one received route = one token with top_k = 1
        self.recv_capacity = recv_capacity or 4 * max_tokens * top_k
        self.owner = _moe.B200MoE(device, shapes, layers * self.per, experts=experts, layers=layers, top_k=1,
                                  shared_inter=0, max_tokens=self.recv_capacity)
        # the expert kernels hold one CTA per SM for their whole duration: leave `comm_sms` SMs to the
        # exchange kernels that should run at the same time (forward_overlapped)
        if comm_sms:
            sms = torch.cuda.get_device_properties(device).multi_processor_count
            self.owner.set_sm_budget(max(1, sms - comm_sms))

    def enable_peer_exchange(self, group=None):
        """Allocate the receive / back buffers in symmetric memory and exchange their addresses, so that
        dispatch and return can store straight into a peer's memory over NVLink (forward_p2p).  Collective:
        every rank of the group calls it."""
        import torch.distributed._symmetric_memory as symm
        g = group if group is not None else dist.group.WORLD
        dev = torch.device("cuda", self.front.device)
        H = self.shapes.hidden
        self.send_capacity = (self.front.max_tokens + 8) * self.top_k
        self.p2p_recv_x = symm.empty((self.recv_capacity, H), dtype=torch.bfloat16, device=dev)
        self.p2p_recv_meta = symm.empty((self.recv_capacity, 2), dtype=torch.int32, device=dev)
        self.p2p_back = symm.empty((self.send_capacity, H), dtype=torch.bfloat16, device=dev)
        self._symm = [symm.rendezvous(t, g.group_name) for t in (self.p2p_recv_x, self.p2p_recv_meta, self.p2p_back)]
        self.peer_x, self.peer_meta, self.peer_back = (h.buffer_ptrs_dev for h in self._symm)
        # the sorted exchange (forward_p2p_sorted): the owner's activation matrix as scaled f16, route weights, row scales
        self.p2p_xg = self.p2p_w = self.p2p_rs = None
        if H == 2048:
            self.p2p_xg = symm.empty((self.recv_capacity, H), dtype=torch.float16, device=dev)
            self.p2p_w = symm.empty((self.recv_capacity,), dtype=torch.float32, device=dev)
            self.p2p_rs = symm.empty((self.recv_capacity,), dtype=torch.float32, device=dev)
            self._symm_sorted = [symm.rendezvous(t, g.group_name) for t in (self.p2p_xg, self.p2p_w, self.p2p_rs)]
            self.peer_xg, self.peer_w, self.peer_rs = (h.buffer_ptrs_dev for h in self._symm_sorted)
        self._tick = torch.zeros((1,), dtype=torch.int32, device=dev)
        self._regions = {}

    def micro_fronts(self, micro: int):
        """One front adapter per micro-batch of forward_p2p: a plan lives in its adapter until its dispatch and
        combine have read it, so batches in flight at the same time need an adapter each."""
        while len(self._fronts) < micro:
            self._fronts.append(_moe.B200MoE(self.front.device, self.shapes, 1, experts=self.experts, layers=self.layers,
                                             top_k=self.top_k, shared_inter=0, max_tokens=self.front.max_tokens))
        return self._fronts[:micro]

    def peer_regions(self, micro: int):
        """Per micro-batch: device tables of every rank's receive-row, receive-meta and back-buffer addresses,
        offset to that batch's region of the buffers."""
        if micro not in self._regions:
            dev = torch.device("cuda", self.front.device)
            H = self.shapes.hidden
            rcap, scap = self.recv_capacity // micro, -(-self.front.max_tokens // micro) * self.top_k
            tabs = []
            for m in range(micro):
                row = []
                for hnd, stride, cap in ((self._symm[0], H * 2, rcap), (self._symm[1], 8, rcap), (self._symm[2], H * 2, scap)):
                    t = torch.tensor([int(p) + m * cap * stride for p in hnd.buffer_ptrs], dtype=torch.int64, device=dev)
                    row.append(t)
                tabs.append(row)
            self._region_tabs = getattr(self, "_region_tabs", []) + [tabs]     # keeps the tables alive
            self._regions[micro] = [tuple(t.data_ptr() for t in row) for row in tabs]
        return self._regions[micro]

    def owned(self, expert: int) -> bool:
        return expert // self.per == self.rank

    def local_slot(self, layer: int, expert: int) -> int:
        return layer * self.per + (expert - self.rank * self.per)

    def load_expert(self, layer: int, expert: int, fields):
        """Stage one OWNED expert (global id) of `layer`."""
        self.owner.load(layer, expert, self.local_slot(layer, expert), fields)

    def route(self, x, gate_w):
        return self.front.router(x, gate_w)

    def shared(self, x, sh_gate_up, sh_down, sh_gate):
        return self.front.shared_expert(x, sh_gate_up, sh_down, sh_gate)

    def pack(self, x, ids, weights):
        return self.front.ep_pack(x, ids, weights, self.world)

    def experts_forward(self, layer: int, recv_x, recv_expert, recv_weight):
        n = recv_x.shape[0]
        if n > self.recv_capacity:
            raise _moe.bad(f"{n} routes received, the owner handle was sized for {self.recv_capacity}")
        y = torch.empty((n, self.shapes.hidden), dtype=torch.bfloat16, device=recv_x.device)
        if n:
            req = _moe.MoEDeviceRequest(layer, self.shapes.hidden, self.shapes.inter, 1, recv_x,
                                        recv_expert.reshape(n, 1), recv_weight.reshape(n, 1))
            self.owner.grouped_moe_staged(req, y)
        return y

    def combine(self, y, route_idx, shared, se_gate, out):
        self.front.ep_combine(y, route_idx, shared, se_gate, out)

    def close(self):
        for f in self._fronts:
            f.close()
        self.owner.close()


class ExpertParallelMoE:
    """Drives one expert-parallel MoE block over `backend` and the default process group."""

    def __init__(self, backend, world: int, group=None):
        self.b, self.world, self.group = backend, world, group
        self.last_counts = None

    def forward(self, layer: int, x, gate_w, sh_gate_up, sh_down, sh_gate, out, record=None):
        """`record(name)` is called at the phase boundaries (the benchmark records CUDA events there)."""
        mark = record or (lambda name: None)
        b = self.b
        ids, w = b.route(x, gate_w)
        shared, se_gate = b.shared(x, sh_gate_up, sh_down, sh_gate) if sh_gate_up is not None else (None, None)
        send_x, send_e, send_w, route_idx, counts = b.pack(x, ids, w)
        mark("packed")
        recv_counts = exchange_counts(counts, self.group)
        sc, rc = counts.tolist(), recv_counts.tolist()          # the one host read-back: NCCL needs the split sizes
        self.last_counts = (sc, rc)
        recv_x = all_to_all_rows(send_x, sc, rc, self.group)
        recv_e = all_to_all_rows(send_e, sc, rc, self.group)
        recv_w = all_to_all_rows(send_w, sc, rc, self.group)
        mark("dispatched")
        y = b.experts_forward(layer, recv_x, recv_e, recv_w)
        mark("computed")
        back = all_to_all_rows(y, rc, sc, self.group)
        mark("returned")
        b.combine(back, route_idx, shared, se_gate, out)
        mark("combined")
        return ids, w

    def forward_p2p(self, layer: int, x, gate_w, sh_gate_up, sh_down, sh_gate, out, record=None, micro: int = 1,
                    fused_return: bool = True):
        """The same block with both exchanges done by this library's own kernels over peer memory: the
        dispatch kernel reads a token's activation row once and stores it straight into the owner's
        receive buffer (no send buffer, no collective); the return kernel stores every output row at the
        position its source expects: with `fused_return` (large steps) the owner's down GEMM stores them there
        itself, 16 bytes per thread, while it runs; otherwise a return kernel reads the rows where the grouped
        GEMM left them (sorted by expert).  The backend must have called enable_peer_exchange().

        The step's tokens are cut into `micro` batches with a region of the receive and back buffers each,
        so that the stores of batch m + 1 cross NVLink (exchange stream) while the owner's GEMMs of batch m
        run (compute stream):

            compute:   route, plans, all-gather of the counts | experts 0 | experts 1 | ... | barrier | combine
            exchange:                                dispatch 0, barrier | dispatch 1, barrier | ...
            side:      shared expert

        One host read-back of the counts per step (the launches are sized by them).  Every rank must pass
        the same `micro`."""
        mark = record or (lambda name: None)
        b = self.b
        world = self.world
        T = x.shape[0]
        micro = max(1, min(int(micro), T))
        fronts = b.micro_fronts(micro)
        bounds = [T * m // micro for m in range(micro + 1)]
        ids, w = b.route(x, gate_w)
        plans = [fronts[m].ep_plan(ids[bounds[m]:bounds[m + 1]], world) for m in range(micro)]
        counts = torch.cat([c for _, c in plans]) if micro > 1 else plans[0][1]
        gathered = torch.empty((world * micro * world,), dtype=torch.int32, device=counts.device)
        dist.all_gather_into_tensor(gathered, counts, group=self.group)
        # [source, batch, owner] -> one [source, owner] table per batch
        counts_all = gathered.reshape(world, micro, world).permute(1, 0, 2).contiguous()
        cur = torch.cuda.current_stream() if x.is_cuda else None
        # the shared expert (tensor cores) runs on a side stream under the dispatch (NVLink stores)
        shared = se_gate = None
        side = None
        if sh_gate_up is not None and x.is_cuda:
            side = self._side_stream(x.device, "_side")
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                shared, se_gate = b.shared(x, sh_gate_up, sh_down, sh_gate)
        elif sh_gate_up is not None:
            shared, se_gate = b.shared(x, sh_gate_up, sh_down, sh_gate)
        ca = counts_all.tolist()                                    # the one host read-back
        sc = [ca[m][b.rank] for m in range(micro)]
        rc = [[ca[m][s][b.rank] for s in range(world)] for m in range(micro)]
        self.last_counts = ([sum(v[p] for v in sc) for p in range(world)], [sum(v[s] for v in rc) for s in range(world)])
        # a batch holds at most ceil(max_tokens / micro) tokens: its back region is sized for that (the back
        # buffer has eight tokens of slack for the rounding)
        if micro > 8:
            raise _moe.bad(f"{micro} micro-batches: at most 8")
        recv_cap, send_cap = b.recv_capacity // micro, -(-b.front.max_tokens // micro) * b.top_k
        for m in range(micro):
            if sum(rc[m]) > recv_cap:
                raise _moe.bad(f"{sum(rc[m])} routes received, the receive region was sized for {recv_cap}")
            if sum(sc[m]) > send_cap:
                raise _moe.bad(f"{sum(sc[m])} routes sent, the back region was sized for {send_cap}")
        peers = b.peer_regions(micro)
        mark("packed")
        # exchange stream: every batch's rows go out as soon as the plan is known
        arrived = []
        xchg = self._side_stream(x.device, "_xchg") if (micro > 1 and x.is_cuda) else None
        if xchg is not None:
            xchg.wait_stream(cur)
        for m in range(micro):
            lo, hi = bounds[m], bounds[m + 1]
            px, pm, _ = peers[m]
            if xchg is None:
                fronts[m].ep_dispatch(x[lo:hi], ids[lo:hi], w[lo:hi], plans[m][0], world, b.rank, counts_all[m], px, pm, recv_cap)
                self._barrier(b)
                arrived.append(None)
            else:
                with torch.cuda.stream(xchg):
                    fronts[m].ep_dispatch(x[lo:hi], ids[lo:hi], w[lo:hi], plans[m][0], world, b.rank, counts_all[m], px, pm,
                                          recv_cap)
                    self._barrier(b)
                    ev = torch.cuda.Event()
                    ev.record(xchg)
                    arrived.append(ev)
        computed = False
        for m in range(micro):
            if arrived[m] is not None:
                cur.wait_event(arrived[m])
            if m == 0:
                mark("dispatched")
            n = sum(rc[m])
            if not n:
                continue
            rx = b.p2p_recv_x[m * recv_cap:m * recv_cap + n]
            meta = b.p2p_recv_meta[m * recv_cap:m * recv_cap + n]
            rids, rw = meta[:, 0].contiguous(), meta[:, 1].contiguous().view(torch.float32)
            # large steps: the rows leave from where the grouped GEMM put them (or from its epilogue)
            if fused_return and b.owner.ep_experts_return(layer, rx, rids, rw, world, b.rank, counts_all[m], peers[m][2],
                                                          send_cap):
                continue
            if b.owner.ep_experts_sorted(layer, rx, rids, rw):
                if micro == 1:
                    mark("computed")
                b.owner.ep_return_sorted(n, world, b.rank, counts_all[m], peers[m][2], send_cap)
            else:
                y = b.experts_forward(layer, rx, rids, rw)
                if micro == 1:
                    mark("computed")
                b.owner.ep_return(y, world, b.rank, counts_all[m], peers[m][2], send_cap)
            computed = micro == 1
        if not computed:
            mark("computed")
        self._barrier(b)
        mark("returned")
        if side is not None:
            cur.wait_stream(side)
            shared.record_stream(cur)       # allocated on the side stream, read on this one
            se_gate.record_stream(cur)
        for m in range(micro):
            lo, hi = bounds[m], bounds[m + 1]
            fronts[m].ep_combine(b.p2p_back[m * send_cap:m * send_cap + sum(sc[m])], plans[m][0],
                                 shared[lo:hi] if shared is not None else None,
                                 se_gate[lo:hi] if se_gate is not None else None, out[lo:hi])
        mark("combined")
        return ids, w

    def forward_p2p_sorted(self, layer: int, x, gate_w, sh_gate_up, sh_down, sh_gate, out, record=None):
        """forward_p2p without a permutation build or a gather pass on the owner: the ranks all-gather the prefixes
        of their send orders over the experts, from which every rank knows where each of its routes lands in the
        owner's activation matrix SORTED BY EXPERT; the dispatch kernel stores the rows there as the scaled f16 the
        grouped GEMM reads, and the owner runs its two GEMMs on them at once (the down GEMM returns the rows, as in
        forward_p2p).  Steps in which some owner receives too few rows for the grouped GEMM (at most 2048) take
        forward_p2p; the decision is made from the all-gathered prefixes, so every rank makes the same one."""
        mark = record or (lambda name: None)
        b = self.b
        world = self.world
        if getattr(b, "p2p_xg", None) is None:
            return self.forward_p2p(layer, x, gate_w, sh_gate_up, sh_down, sh_gate, out, record=record)
        ids, w = b.route(x, gate_w)
        route_idx, seg = b.front.ep_plan_seg(ids)
        E = b.experts
        seg_all = torch.empty((world * (E + 1),), dtype=torch.int32, device=seg.device)
        dist.all_gather_into_tensor(seg_all, seg, group=self.group)
        cur = torch.cuda.current_stream()
        shared = se_gate = None
        side = None
        if sh_gate_up is not None:
            side = self._side_stream(x.device, "_side")
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                shared, se_gate = b.shared(x, sh_gate_up, sh_down, sh_gate)
        bounds = seg_all.reshape(world, E + 1)[:, ::b.per].tolist()     # the one host read-back: [source][owner boundary]
        sent = [[bounds[s][p + 1] - bounds[s][p] for p in range(world)] for s in range(world)]
        recv = [sum(sent[s][p] for s in range(world)) for p in range(world)]
        sc, rc = sent[b.rank], [sent[s][b.rank] for s in range(world)]
        self.last_counts = (sc, rc)
        n = recv[b.rank]
        if min(recv) <= 2048:
            # the small-step exchange; its own plan and counts (this one's are not in its format)
            if side is not None:
                cur.wait_stream(side)
            return self.forward_p2p(layer, x, gate_w, sh_gate_up, sh_down, sh_gate, out, record=record)
        if n > b.recv_capacity:
            raise _moe.bad(f"{n} routes received, the receive buffer was sized for {b.recv_capacity}")
        mark("packed")
        b.front.ep_dispatch_sorted(x, ids, w, route_idx, world, b.rank, seg_all, b.peer_xg, b.peer_w, b.peer_rs, b.recv_capacity)
        self._barrier(b)
        mark("dispatched")
        b.owner.ep_experts_presorted(layer, b.p2p_xg, b.p2p_w, b.p2p_rs, n, world, b.rank, seg_all, b.peer_back, b.send_capacity)
        mark("computed")
        self._barrier(b)
        mark("returned")
        if side is not None:
            cur.wait_stream(side)
            shared.record_stream(cur)
            se_gate.record_stream(cur)
        b.combine(b.p2p_back[:sum(sc)], route_idx, shared, se_gate, out)
        mark("combined")
        return ids, w

    def _side_stream(self, device, name):
        if getattr(self, name, None) is None:
            setattr(self, name, torch.cuda.Stream(device=device))
        return getattr(self, name)

    def _barrier(self, b):
        # every rank's stores before this point are complete before any rank goes on
        dist.all_reduce(b._tick, group=self.group)

    def forward_overlapped(self, layer: int, x, gate_w, sh_gate_up, sh_down, sh_gate, out, chunks: int = 2, record=None):
        """The same block with the exchanges under the compute.  The send buffers are sorted by (owner,
        expert), so every owner's experts are cut into `chunks` contiguous ranges and each range is
        exchanged and computed on its own; an expert's routes stay in one range, so no weight is
        dequantised twice:

            route, pack, counts per (owner, range)         one host read-back, as in `forward`
            dispatch of every range (async, in order)      the shared expert runs under the first one
            range c: wait dispatch | experts | return (async)    experts of c run under dispatch of c + 1
                                                                  and the return of c - 1
            wait the returns | combine

        The returned rows land in send order, so the combine is the one of `forward`.  Every rank must
        pass the same `chunks`; it must divide the experts per rank."""
        mark = record or (lambda name: None)
        b = self.b
        world = self.world
        per = b.per
        if chunks < 1 or per % chunks:
            raise _moe.bad(f"{per} experts per rank cannot be cut into {chunks} ranges")
        sub = per // chunks
        ids, w = b.route(x, gate_w)
        send_x, send_e, send_w, route_idx, _ = b.pack(x, ids, w)
        # routes per (owner, range): the send buffers are sorted by expert id
        counts = torch.bincount((send_e // sub).long(), minlength=world * chunks).to(torch.int32)
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=self.group)           # [source][range]
        sc = counts.reshape(world, chunks).tolist()                             # the one host read-back
        rc = recv_counts.reshape(world, chunks).tolist()
        self.last_counts = ([sum(r) for r in sc], [sum(r) for r in rc])
        mark("packed")
        # one meta row per route (expert id, weight bits): one exchange instead of two
        send_m = torch.stack((send_e, send_w.view(torch.int32)), dim=1)
        soff = [0]
        for p in range(world):
            for c in range(chunks):
                soff.append(soff[-1] + sc[p][c])
        pending = []
        for c in range(chunks):
            n = sum(rc[s][c] for s in range(world))
            recv_x = send_x.new_empty((n,) + tuple(send_x.shape[1:]))
            recv_m = send_m.new_empty((n, 2))
            roff = [0]
            for s in range(world):
                roff.append(roff[-1] + rc[s][c])
            ins_x = [send_x[soff[p * chunks + c]:soff[p * chunks + c + 1]] for p in range(world)]
            ins_m = [send_m[soff[p * chunks + c]:soff[p * chunks + c + 1]] for p in range(world)]
            outs_x = [recv_x[roff[s]:roff[s + 1]] for s in range(world)]
            outs_m = [recv_m[roff[s]:roff[s + 1]] for s in range(world)]
            works = [all_to_all_views(outs_x, ins_x, self.group), all_to_all_views(outs_m, ins_m, self.group)]
            pending.append((works, recv_x, recv_m, roff))
        shared, se_gate = b.shared(x, sh_gate_up, sh_down, sh_gate) if sh_gate_up is not None else (None, None)
        mark("shared")
        back = None
        returns = []
        for c, (works, recv_x, recv_m, roff) in enumerate(pending):
            for wk in works:
                wk.wait()
            mark(f"dispatched{c}")
            y = b.experts_forward(layer, recv_x, recv_m[:, 0].contiguous(), recv_m[:, 1].contiguous().view(torch.float32))
            mark(f"computed{c}")
            if back is None:
                back = y.new_empty((soff[-1],) + tuple(y.shape[1:]))
            ins = [y[roff[s]:roff[s + 1]] for s in range(world)]
            outs = [back[soff[p * chunks + c]:soff[p * chunks + c + 1]] for p in range(world)]
            returns.append((all_to_all_views(outs, ins, self.group), y))
        for wk, _ in returns:
            wk.wait()
        mark("returned")
        b.combine(back, route_idx, shared, se_gate, out)
        mark("combined")
        return ids, w
