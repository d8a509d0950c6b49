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
                            (worker/gossip_dist.rs:883-976); ``asynchronous=True``: a receiving thread
                            accumulates whatever arrives, nobody waits (worker/gossip_dist.rs:474-593)
``GroupAllreduceGossipComm``group all-reduce + pull gossip between groups (gossip_pull_allreduce_dist_rdma*.rs)
``ElasticComm``             elastic averaging against a centre held by rank 0, beta = 0.8/N
                            (worker/elasticserver_dist.rs:249-255,711-715); ``asynchronous=True``: a serving
                            thread on rank 0 handles one client at a time, in the order they ask
==========================  ================================================================================

The backends in this file use ``torch.distributed`` collectives (gloo on CPU ranks, NCCL on GPUs); they define
the semantics and serve as baseline and test oracle. The peer-memory kernels that do the same exchanges inside
one CUDA kernel live in ``parallel/p2p.py`` and subclass these.
"""
from __future__ import annotations

import os
import threading
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

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

    def close(self) -> None:
        """Stop background threads and drain messages in flight. Collective: every rank calls it once, after its
        last exchange. Nothing to do for the lock-step backends."""


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

    def __init__(self, bucket_bytes: int = 32 << 20, min_bucket_bytes: int = 4 << 20, blocks: Optional[int] = None):
        super().__init__()
        if blocks is None:
            blocks = int(os.environ.get("RB_OVERLAP_BLOCKS", "296"))
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


class _NoLock:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_LOCK = _NoLock()


class _Inbox(threading.Thread):
    """Background receiver of the asynchronous library backends: the reference's passive thread
    (worker/gossip_dist.rs:474-593, worker/elasticserver_dist.rs:249-255).

    It blocks in a receive from ANY rank on a process group of its own (so its traffic never meets the main
    thread's collectives), hands every message of `n` floats to `on_message(sender, payload)`, and ends after it
    has seen one closing message from each of the `world - 1` peers. Messages of one sender arrive in the order
    sent, so by then everything that sender pushed earlier has been handled. The last element of a message is
    its kind: >= 0 data, < 0 closing."""

    def __init__(self, group, world: int, n: int, dtype, on_message: Callable[[int, torch.Tensor], None]):
        super().__init__(daemon=True, name="rb-comm-inbox")
        self.group, self.world, self.n, self.on_message = group, world, n, on_message
        self.buf = torch.empty(n + 1, dtype=dtype)
        self.error: Optional[BaseException] = None

    def run(self):
        closed = 0
        try:
            while closed < self.world - 1:
                sender = dist.recv(self.buf, group=self.group)
                if float(self.buf[self.n]) < 0:
                    closed += 1
                else:
                    self.on_message(dist.get_group_rank(self.group, sender), self.buf[:self.n])
        except BaseException as e:      # surfaced by the owner's next call
            self.error = e


def _async_group(group):
    """A gloo group over the same ranks for one-sided style traffic. Receiving from any source exists in gloo only;
    on GPUs the asynchronous exchanges are the kernel backends of ``parallel/p2p.py``."""
    if dist.get_backend(group) != "gloo":
        raise ValueError("the asynchronous library backends need gloo (CPU ranks); on GPUs use the kernel "
                         "backends gossip_push_p2p / elastic_p2p, which are asynchronous by default")
    ranks = dist.get_process_group_ranks(group) if group is not None else list(range(dist.get_world_size()))
    timeout = None
    try:    # same time limit as the group it shadows, so that a peer that died ends a receive with an error there too
        pg = group if group is not None else dist.distributed_c10d._get_default_group()
        timeout = pg._get_backend(torch.device("cpu")).options._timeout
    except (AttributeError, RuntimeError):
        pass
    return dist.new_group(ranks, backend="gloo", timeout=timeout)


class PushGossipComm(CommWorker):
    """Each rank pushes its vector to a uniformly random target; a rank that received k vectors keeps
    (w_self * own + sum received) / (w_self + k) with w_self = 2 if it targeted itself, else 1.

    Lock-step by default: the ranks agree on the round's targets and every push of a round is folded in that
    round. ``asynchronous=True`` is the reference's form (worker/gossip_dist.rs:474-593, 883-976): a background
    thread adds whatever arrives, from whichever rank, into an accumulator and counts it; an exchange pushes to
    its target and folds in what has arrived since the last one (possibly nothing). No rank waits for another.
    It needs gloo and a `close()` by every rank at the end."""
    name = "gossip_push"

    def __init__(self, group=None, seed=(41, 43), asynchronous: bool = False):
        super().__init__(group)
        self.rng = XorShift128Plus(seed[0] + 7919 * self.rank, seed[1])
        self._global = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)
        self.asynchronous = bool(asynchronous) and self.world > 1
        self.synchronous = not self.asynchronous
        self.folded = 0               # vectors folded in so far (asynchronous form)
        self._inbox = None
        if self.asynchronous:
            self._pg = _async_group(group)
            self._lock = threading.Lock()
            self._acc, self._count, self._msg = None, 0, None

    # ---- asynchronous form
    def _on_push(self, sender: int, payload: torch.Tensor) -> None:
        with self._lock:
            self._acc.add_(payload)
            self._count += 1

    def _start(self, flat: torch.Tensor) -> None:
        n = flat.numel()
        self._acc = torch.zeros(n, dtype=flat.dtype)
        self._msg = torch.empty(n + 1, dtype=flat.dtype)
        self._inbox = _Inbox(self._pg, self.world, n, flat.dtype, self._on_push)
        self._inbox.start()

    def _sync_async(self, flat: torch.Tensor) -> None:
        if self._inbox is None:
            self._start(flat)
        if self._inbox.error is not None:
            raise RuntimeError("push gossip: the receiving thread stopped") from self._inbox.error
        n = flat.numel()
        target = self.rng.below(self.world)
        if target != self.rank:
            self._msg[:n].copy_(flat.reshape(-1))
            self._msg[n] = 1.0
            dist.send(self._msg, dist.get_global_rank(self._pg, target), group=self._pg)
        w_self = 2.0 if target == self.rank else 1.0
        with self._lock:
            k = self._count
            if k:
                flat.mul_(w_self).add_(self._acc.view_as(flat)).div_(w_self + k)
                self._acc.zero_()
                self._count = 0
        self.folded += k
        self.bytes_moved += n * 4

    def close(self) -> None:
        if not self.asynchronous or self._inbox is None:
            return
        self._msg[self._msg.numel() - 1] = -1.0
        for r in range(self.world):
            if r != self.rank:
                dist.send(self._msg, dist.get_global_rank(self._pg, r), group=self._pg)
        self._inbox.join()
        error, self._inbox = self._inbox.error, None
        if error is not None:
            raise RuntimeError("push gossip: a peer never sent its closing message") from error

    def first_one_way_sync(self, flat: torch.Tensor) -> None:
        """Asynchronous form: start listening before any rank can push (every rank calls this before training)."""
        if self.asynchronous and self._inbox is None:
            self._start(flat)
            dist.barrier(group=self.group)

    def pending(self) -> int:
        """Vectors that have arrived and are not folded in yet (asynchronous form)."""
        if not self.asynchronous or self._acc is None:
            return 0
        with self._lock:
            return self._count

    # ---- lock-step form
    def sync_params(self, flat, repeat=False):
        if self.world <= 1:
            return
        if self.asynchronous:
            return self._sync_async(flat)
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
    both move toward each other:  centre += beta (x - centre_read),  x = (1-beta) x + beta centre_read.

    Lock-step by default (every client mixes with the same centre snapshot of the round). ``asynchronous=True``
    is the reference's server (worker/elasticserver_dist.rs:249-255, 667-715): a thread on rank 0 takes one
    client's vector at a time, from whichever client asks, answers with the centre as it is then and moves the
    centre toward that client; no client waits for another. `request_log` on rank 0 lists the clients in the
    order served, which makes a run replayable. It needs gloo and a `close()` by every rank at the end."""
    name = "elastic"

    def __init__(self, group=None, beta: Optional[float] = None, asynchronous: bool = False):
        super().__init__(group)
        self.beta = beta if beta is not None else 0.8 / max(1, self.world)
        self.center = None
        self.asynchronous = bool(asynchronous) and self.world > 1
        self.synchronous = not self.asynchronous
        self.request_log: List[int] = []
        self._inbox = None
        if self.asynchronous:
            self._pg = _async_group(group)
            self._lock = threading.Lock()
            self._msg = None

    def first_one_way_sync(self, flat):
        """Rank 0's parameters become the centre; every rank starts from it."""
        if self.world > 1:
            dist.broadcast(flat, 0, group=self.group)
        if self.asynchronous and self.rank != 0 and self._msg is None:
            self._msg = torch.zeros(flat.numel() + 1, dtype=flat.dtype)
        if self.rank == 0:
            self.center = flat.clone()
            if self.asynchronous and self._inbox is None:
                self._inbox = _Inbox(self._pg, self.world, flat.numel(), flat.dtype, self._serve)
                self._inbox.start()

    # ---- asynchronous form
    def _mix_center(self, client: int, x: torch.Tensor) -> torch.Tensor:
        """Serve one client under the lock: returns the centre as read, then moves it toward `x`."""
        with self._lock:
            read = self.center.reshape(-1).clone()
            self.center.reshape(-1).add_(x.reshape(-1) - read, alpha=self.beta)
            self.request_log.append(client)
        return read

    def _serve(self, client: int, payload: torch.Tensor) -> None:
        read = self._mix_center(client, payload)
        dist.send(read, dist.get_global_rank(self._pg, client), group=self._pg, tag=1)

    def _sync_async(self, flat: torch.Tensor) -> None:
        n = flat.numel()
        if self.rank == 0:
            if self._inbox is not None and self._inbox.error is not None:
                raise RuntimeError("elastic averaging: the serving thread stopped") from self._inbox.error
            read = self._mix_center(0, flat)
        else:
            self._msg[:n].copy_(flat.reshape(-1))
            self._msg[n] = 1.0
            root = dist.get_global_rank(self._pg, 0)
            dist.send(self._msg, root, group=self._pg)
            read = torch.empty(n, dtype=flat.dtype)
            dist.recv(read, root, group=self._pg, tag=1)
        flat.mul_(1.0 - self.beta).add_(read.view_as(flat), alpha=self.beta)
        self.bytes_moved += n * 8

    def close(self) -> None:
        if not self.asynchronous:
            return
        if self.rank != 0:
            if self._msg is None:
                return                      # first_one_way_sync never ran: no server is listening
            self._msg[self._msg.numel() - 1] = -1.0
            dist.send(self._msg, dist.get_global_rank(self._pg, 0), group=self._pg)
        elif self._inbox is not None:
            self._inbox.join()
            error, self._inbox = self._inbox.error, None
            if error is not None:
                raise RuntimeError("elastic averaging: a client never sent its closing message") from error

    # ---- lock-step form
    def sync_params(self, flat, repeat=False):
        if self.world <= 1:
            return
        if self.asynchronous:
            return self._sync_async(flat)
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
            with (self._lock if self.asynchronous else _NO_LOCK):
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
    if name in ("gossip_push_async", "elastic_async"):
        # the asynchronous forms of the two library backends that have one (gloo ranks only)
        return table[name[:-len("_async")]](asynchronous=True, **kw)
    if name not in table:
        raise ValueError(f"unknown comm backend {name!r}")
    return table[name](**kw) if name != "null" else NullComm()
