"""Communication backends behind one protocol.

The reference's ``CommWorker`` trait (src/operator/comm.rs:20-34) has operators load their gradients or
parameters into a flat device buffer, calls ``communicate()``, and stores the result back. Here the network
already keeps parameters and gradients in flat vectors, so a backend works on those vectors in place.
Every data-parallel flavour of the reference maps to one backend:

==========================  ================================================================================
backend                     reference component
==========================  ================================================================================
``NullComm``                NullCommWorker (comm.rs:75-88)
``AllreduceComm``           device ring all-reduce (arch_new.rs:554-573) / MPI all-reduce
                            (worker/allreduce_dist.rs:211-241): library collective + separate optimizer step;
                            this is the NCCL *baseline* path on GPUs and the gloo path on CPU ranks
``FusedAllreduceSgdComm``   same semantics, one hand-written kernel over peer memory (parallel/p2p.py)
``PairGossipComm``          synchronous pair gossip with a shared-seed permutation (comm.rs:125-296,
                            worker/gossip_dist.rs:64-438)
``PullGossipComm``          pull from uniformly random peers, ``num_rounds``, ``repeat``
                            (worker/gossip_pull_dist_rdma.rs:517-589)
``PushGossipComm``          push to a uniformly random target, count-normalised mean
                            (worker/gossip_dist.rs:883-976)
``GroupAllreduceGossipComm``group all-reduce + pull gossip between groups (gossip_pull_allreduce_dist_rdma*.rs)
``ElasticComm``             elastic averaging against a centre held by rank 0, beta = 0.8/N
                            (worker/elasticserver_dist.rs:249-255,711-715)
==========================  ================================================================================

The backends in this file use ``torch.distributed`` collectives (gloo on CPU ranks, NCCL on GPUs); they define
the semantics and serve as baseline and test oracle. The peer-memory kernels that do the same exchanges inside
one CUDA kernel live in ``parallel/p2p.py`` and subclass these.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..utils.rng import XorShift128Plus


@dataclass
class GossipConfig:
    num_rounds: int = 1
    buf_size: int = 0


@dataclass
class ParameterServerConfig:
    com_interval: int = 1
    buf_size: int = 0


class CommWorker:
    """Base protocol. `flat` arguments are 1-D fp32 tensors that live on the worker's device."""

    name = "base"

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.step_size = 0.0
        self.iter = 0
        self.bytes_moved = 0          # payload bytes this rank contributed to exchanges (for bus-bandwidth reports)

    def num_workers(self):
        return self.world

    def next(self):
        """Advance the round counter (the reference's CommWorker::next)."""
        self.iter += 1

    def hack_set_step_size(self, s):
        self.step_size = s

    # ---- gradient / parameter exchanges
    def allreduce_average(self, flat: torch.Tensor) -> None:
        """flat <- mean over ranks (sync_grads_v2 with an all-reduce backend)."""
        raise NotImplementedError

    def sync_params(self, flat: torch.Tensor, repeat: bool = False) -> None:
        """Backend-specific parameter mix (sync_params_v2). `repeat` reuses the previous round's partners."""
        raise NotImplementedError

    def first_one_way_sync(self, flat: torch.Tensor) -> None:
        """communicate_first: parameter-server backends upload rank 0's parameters as the centre."""

    def exact_sync(self, flat: torch.Tensor) -> None:
        """communicate_exact: true mean over all ranks (used at checkpoints)."""
        if self.world > 1:
            dist.all_reduce(flat, group=self.group)
            flat.div_(self.world)

    # ---- small host-side collectives
    def allreduce_stats(self, values: Sequence[float]) -> List[float]:
        if self.world <= 1:
            return list(values)
        t = torch.tensor(list(values), dtype=torch.float64)
        if dist.get_backend(self.group) == "nccl":
            t = t.cuda()
        dist.all_reduce(t, group=self.group)
        return t.cpu().tolist()

    def broadcast_seed(self, seed):
        if self.world <= 1:
            return tuple(seed)
        t = torch.tensor(list(seed), dtype=torch.int64)
        if dist.get_backend(self.group) == "nccl":
            t = t.cuda()
        dist.broadcast(t, 0, group=self.group)
        return tuple(int(v) for v in t.cpu().tolist())

    def barrier(self):
        if self.world > 1:
            dist.barrier(group=self.group)

    # checkpoint barrier of the reference: signal, then poll wait (always immediate here)
    def signal_barrier(self):
        self.barrier()

    def wait_barrier(self) -> bool:
        return True


class NullComm(CommWorker):
    name = "null"

    def __init__(self):
        self.group = None
        self.rank, self.world = 0, 1
        self.step_size, self.iter, self.bytes_moved = 0.0, 0, 0

    def allreduce_average(self, flat):
        pass

    def sync_params(self, flat, repeat=False):
        pass

    def exact_sync(self, flat):
        pass


def plan_buckets(net, bucket_elems: int, min_bucket_elems: int, align: int = 64):
    """Ranges of the flat vectors in the order backward completes them: [(trigger operator index, offset, length)].
    Operators are visited last to first; their segments are merged into contiguous ranges, flushed once at least
    `min_bucket_elems` are pending, and cut into pieces of at most `bucket_elems`."""
    ops = net.ops
    pending, pending_elems, out = [], 0, []

    def merge(ranges):
        res = []
        for lo, hi in sorted(ranges):
            if res and res[-1][1] == lo:
                res[-1] = (res[-1][0], hi)
            else:
                res.append((lo, hi))
        return res

    for idx in range(len(ops) - 2, 0, -1):
        for s in ops[idx].segs:
            n = (s.numel + align - 1) // align * align
            pending.append((s.offset, s.offset + n))
            pending_elems += n
        if pending and (pending_elems >= min_bucket_elems or idx == 1):
            for lo, hi in merge(pending):
                o = lo
                while o < hi:
                    n = min(bucket_elems, hi - o)
                    out.append((idx, o, n))
                    o += n
            pending, pending_elems = [], 0
    return out


class LocalOverlapComm(NullComm):
    """One worker, no exchange -- but the optimizer step of a gradient bucket starts as soon as backward has
    finished the bucket, on a second stream and with blocks small enough to sit beside the GEMM CTAs, instead of
    one sweep over all parameters after backward. The update is bound by HBM traffic and the convolutions by
    shared-memory fill, so the two overlap well."""
    name = "null"
    graph_safe = True
    overlap_single = True

    def __init__(self, bucket_bytes: int = 32 << 20, min_bucket_bytes: int = 4 << 20, blocks: int = 296):
        super().__init__()
        self.bucket_elems = bucket_bytes // 4 // 64 * 64
        self.min_bucket_elems = min_bucket_bytes // 4
        self.blocks = blocks
        self.kernel_launches_per_step = 0

    def attach(self, engine):
        self.engine = engine
        net = engine.net
        self.side = torch.cuda.Stream(net.device, priority=-1)
        self._ready, self._done = torch.cuda.Event(), torch.cuda.Event()
        self._by_trigger = {}
        for idx, off, n in plan_buckets(net, self.bucket_elems, self.min_bucket_elems):
            self._by_trigger.setdefault(idx, []).append((off, n))

    def prepare(self, stepper, lr):
        self._stepper, self._lr = stepper, float(lr)
        self._forked = False

    def on_op_backward(self, op_index):
        recs = self._by_trigger.get(op_index)
        if not recs:
            return
        self._forked = True
        self._ready.record(torch.cuda.current_stream())
        self.side.wait_event(self._ready)
        with torch.cuda.stream(self.side):
            for off, n in recs:
                self._stepper.step(self._lr, lo=off, hi=off + n, grid=(self.blocks, 128))

    def fused_grads_step(self, stepper, lr):
        if self._forked:
            self._done.record(self.side)
            torch.cuda.current_stream().wait_event(self._done)


class AllreduceComm(CommWorker):
    """Library all-reduce of the whole flat vector followed by a 1/N scale."""
    name = "allreduce"

    def allreduce_average(self, flat):
        if self.world <= 1:
            return
        dist.all_reduce(flat, group=self.group)
        flat.div_(self.world)
        self.bytes_moved += flat.numel() * 4

    def sync_params(self, flat, repeat=False):
        self.allreduce_average(flat)


def _exchange(flat: torch.Tensor, send_to: int, recv_from: int, rank: int, group) -> Optional[torch.Tensor]:
    """Send `flat` to one peer and receive a vector from another (either may be this rank)."""
    recv = torch.empty_like(flat) if recv_from != rank else None
    if dist.get_backend(group) == "nccl":
        # one collective over the whole group: point-to-point calls between pairs that have not talked before
        # set up a connection per pair, in an order that differs between ranks of a long cycle
        world = dist.get_world_size(group)
        n = flat.numel()
        in_split = [n if (r == send_to and send_to != rank) else 0 for r in range(world)]
        out_split = [n if (r == recv_from and recv_from != rank) else 0 for r in range(world)]
        src = flat if send_to != rank else flat[:0]
        dst = recv if recv is not None else flat[:0]
        dist.all_to_all_single(dst, src.contiguous(), out_split, in_split, group=group)
        return recv
    if send_to == rank and recv_from == rank:
        return None
    # point-to-point operations name their peer by global rank; `send_to` / `recv_from` are ranks within `group`
    to_global = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)
    ops = []
    if send_to != rank:
        ops.append(dist.P2POp(dist.isend, flat, to_global(send_to), group))
    if recv_from != rank:
        ops.append(dist.P2POp(dist.irecv, recv, to_global(recv_from), group))
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    return recv


class PairGossipComm(CommWorker):
    """Every round all ranks draw the same permutation from a shared-seed stream; rank r sends to perm[r],
    receives from the inverse, and keeps the average of its own and the received vector."""
    name = "gossip_pair"

    def __init__(self, group=None, seed=(17, 29), cfg: GossipConfig = GossipConfig()):
        super().__init__(group)
        self.rng = XorShift128Plus(*seed)
        self.cfg = cfg
        self._last = None

    def draw(self, repeat=False):
        if repeat and self._last is not None:
            return self._last
        perm = self.rng.permutation(self.world)
        inv = [0] * self.world
        for i, p in enumerate(perm):
            inv[p] = i
        self._last = (perm, inv)
        return self._last

    def sync_params(self, flat, repeat=False):
        if self.world <= 1:
            return
        for _ in range(max(1, self.cfg.num_rounds)):
            perm, inv = self.draw(repeat)
            got = _exchange(flat, perm[self.rank], inv[self.rank], self.rank, self.group)
            if got is not None:
                flat.add_(got).mul_(0.5)
                self.bytes_moved += flat.numel() * 4

    allreduce_average = CommWorker.exact_sync


class PullGossipComm(CommWorker):
    """Each rank pulls the vector of a uniformly random rank (possibly itself) per round and averages the
    `num_rounds` + 1 vectors. The peer table is all-gathered so that senders know who pulls from them."""
    name = "gossip_pull"

    def __init__(self, group=None, seed=(31, 37), cfg: GossipConfig = GossipConfig()):
        super().__init__(group)
        # per-rank stream: choices are independent across ranks, as in the reference
        self.rng = XorShift128Plus(seed[0] + 1000003 * self.rank, seed[1])
        self.cfg = cfg
        self._last_table = None
        # point-to-point operations name their peer by global rank; the peer table holds ranks within `group`
        self._global = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)

    def draw_table(self, repeat=False):
        if repeat and self._last_table is not None:
            return self._last_table
        mine = [self.rng.below(self.world) for _ in range(max(1, self.cfg.num_rounds))]
        table = [None] * self.world
        dist.all_gather_object(table, mine, group=self.group)
        self._last_table = table
        return table

    def sync_params(self, flat, repeat=False):
        if self.world <= 1:
            return
        table = self.draw_table(repeat)
        snapshot = flat.clone()   # peers read the published copy, not the vector being mixed
        total = flat.clone()
        for rnd in range(len(table[0])):
            src = table[self.rank][rnd]
            ops, recv = [], None
            for r in range(self.world):
                if table[r][rnd] == self.rank and r != self.rank:
                    ops.append(dist.P2POp(dist.isend, snapshot, self._global(r), self.group))
            if src != self.rank:
                recv = torch.empty_like(flat)
                ops.append(dist.P2POp(dist.irecv, recv, self._global(src), self.group))
            if ops:
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
            total.add_(recv if recv is not None else snapshot)
            self.bytes_moved += flat.numel() * 4
        flat.copy_(total.div_(len(table[0]) + 1))

    allreduce_average = CommWorker.exact_sync


class PushGossipComm(CommWorker):
    """Each rank pushes its vector to a uniformly random target; a rank that received k vectors keeps
    (w_self * own + sum received) / (w_self + k) with w_self = 2 if it targeted itself, else 1."""
    name = "gossip_push"

    def __init__(self, group=None, seed=(41, 43)):
        super().__init__(group)
        self.rng = XorShift128Plus(seed[0] + 7919 * self.rank, seed[1])
        self._global = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)

    def sync_params(self, flat, repeat=False):
        if self.world <= 1:
            return
        target = self.rng.below(self.world)
        targets = [None] * self.world
        dist.all_gather_object(targets, target, group=self.group)
        senders = [r for r in range(self.world) if targets[r] == self.rank and r != self.rank]
        bufs = [torch.empty_like(flat) for _ in senders]
        ops = [dist.P2POp(dist.irecv, b, self._global(r), self.group) for b, r in zip(bufs, senders)]
        snapshot = flat.clone()
        if target != self.rank:
            ops.append(dist.P2POp(dist.isend, snapshot, self._global(target), self.group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        w_self = 2.0 if target == self.rank else 1.0
        if bufs:
            acc = flat.mul(w_self)
            for b in bufs:
                acc.add_(b)
            flat.copy_(acc.div_(w_self + len(bufs)))
        self.bytes_moved += flat.numel() * 4

    allreduce_average = CommWorker.exact_sync


class GroupAllreduceGossipComm(CommWorker):
    """Hierarchical: the mean inside groups of `group_size` consecutive ranks, then gossip between groups.

    version 2 (default; gossip_pull_allreduce_dist_rdma_v2.rs:327-384): every rank pulls the group mean of a random
    rank and keeps 0.5 * (pulled + own group mean).
    version 1 (gossip_pull_allreduce_dist_rdma.rs:327-402): only the group leaders (first rank of each group) gossip:
    a leader pulls the group mean of a random leader, keeps 0.5 * (pulled + own) unless it drew itself, and
    broadcasts the result to its group."""
    name = "group_allreduce_gossip"

    def __init__(self, group=None, group_size=2, seed=(53, 59), version=2):
        super().__init__(group)
        if version not in (1, 2):
            raise ValueError("version must be 1 or 2")
        self.group_size = max(1, min(group_size, self.world))
        self.version = version
        self.subgroup = None
        self.pull = None
        if self.world > 1:
            for g0 in range(0, self.world, self.group_size):
                ranks = list(range(g0, min(self.world, g0 + self.group_size)))
                sg = dist.new_group(ranks)
                if self.rank in ranks:
                    self.subgroup, self.sub_n = sg, len(ranks)
            if version == 2:
                self.pull = PullGossipComm(group, seed)
            else:
                leaders = list(range(0, self.world, self.group_size))
                leader_group = dist.new_group(leaders)       # collective: every rank creates it, leaders use it
                self.leader = self.rank // self.group_size * self.group_size
                if self.rank == self.leader and len(leaders) > 1:
                    self.pull = PullGossipComm(leader_group, seed)

    def sync_params(self, flat, repeat=False):
        if self.world <= 1:
            return
        dist.all_reduce(flat, group=self.subgroup)
        flat.div_(self.sub_n)
        if self.pull is not None:
            self.pull.sync_params(flat, repeat)
        if self.version == 1 and self.sub_n > 1:
            dist.broadcast(flat, self.leader, group=self.subgroup)

    allreduce_average = CommWorker.exact_sync


class ElasticComm(CommWorker):
    """Elastic averaging SGD: the centre variable lives on rank 0. On each exchange a client reads the centre,
    both move toward each other:  centre += beta (x - centre_read),  x = (1-beta) x + beta centre_read."""
    name = "elastic"

    def __init__(self, group=None, beta: Optional[float] = None):
        super().__init__(group)
        self.beta = beta if beta is not None else 0.8 / max(1, self.world)
        self.center = None

    def first_one_way_sync(self, flat):
        """Rank 0's parameters become the centre; every rank starts from it."""
        if self.world > 1:
            dist.broadcast(flat, 0, group=self.group)
        if self.rank == 0:
            self.center = flat.clone()

    def sync_params(self, flat, repeat=False):
        if self.world <= 1:
            return
        # every client mixes with the same centre snapshot; the centre receives the sum of the pulls
        center = self.center.clone() if self.rank == 0 else torch.empty_like(flat)
        dist.broadcast(center, 0, group=self.group)
        pull = (flat - center).mul_(self.beta)
        flat.sub_(pull)
        dist.reduce(pull, 0, group=self.group)
        if self.rank == 0:
            self.center.add_(pull)
        self.bytes_moved += flat.numel() * 8

    def exact_sync(self, flat):
        """Broadcast the centre to every rank."""
        if self.world <= 1:
            return
        if self.rank == 0:
            flat.copy_(self.center)
        dist.broadcast(flat, 0, group=self.group)

    allreduce_average = CommWorker.exact_sync


class DownpourServerComm(CommWorker):
    """Placeholder, as in the reference (worker/paramserver_dist.rs:1 is an empty struct)."""
    name = "downpour"


def make_comm(name: str, **kw) -> CommWorker:
    table = {c.name: c for c in (NullComm, AllreduceComm, PairGossipComm, PullGossipComm, PushGossipComm,
                                 GroupAllreduceGossipComm, ElasticComm)}
    if name == "fused_allreduce_sgd" or name.endswith("_p2p"):
        from . import p2p
        return p2p.make(name, **kw)
    if name not in table:
        raise ValueError(f"unknown comm backend {name!r}")
    return table[name](**kw) if name != "null" else NullComm()
