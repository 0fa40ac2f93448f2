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


class LibBackend:
    """The CUDA library on both sides of the exchange."""

    def __init__(self, device: int, rank: int, world: int, shapes: _moe.ExpertShapes, *, experts: int = 256,
                 layers: int = 1, top_k: int = 8, shared_inter: int = 512, max_tokens: int = 8192,
                 recv_capacity: int | None = None):
        if experts % world:
            raise _moe.bad(f"{experts} experts do not split over {world} ranks")
        self.rank, self.world, self.experts, self.layers, self.top_k = rank, world, experts, layers, top_k
        self.per = experts // world
        self.shapes = shapes
        # front: router, shared expert, pack, combine (its banks are never used: one slot)
        self.front = _moe.B200MoE(device, shapes, 1, experts=experts, layers=layers, top_k=top_k,
                                  shared_inter=shared_inter, max_tokens=max_tokens)
        # owner: this rank's experts, one received route = one token with top_k = 1
        self.recv_capacity = recv_capacity or 4 * max_tokens * top_k
        self.owner = _moe.B200MoE(device, shapes, layers * self.per, experts=experts, layers=layers, top_k=1,
                                  shared_inter=0, max_tokens=self.recv_capacity)

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
        self.front.close()
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
