"""Communication backends whose data path is our own CUDA kernels over peer-visible (symmetric) memory.

``torch.distributed`` (NCCL) is used for plumbing only: rendezvous, exchange of memory handles through
``torch.distributed._symmetric_memory``, the broadcast of the shared seed and tiny host-side statistics. The
gradient exchange, the optimizer step that follows it, and the gossip / elastic parameter mixes are kernels from
``csrc/comm_p2p.cu`` that load from and store to the other GPUs' memory directly.

``FusedAllreduceSgdComm`` overlaps the exchange with the backward pass: the flat gradient vector is cut into
buckets (25 MB by default) in the order backward produces them; as soon as the operators of a bucket have run, the
bucket's kernels are launched on one of two side streams while backward continues. The exchange is push based
(posted remote stores saturate NVLink from a grid small enough to sit beside the GEMM CTAs; remote loads do not):
a push kernel copies shard p of the local gradients into peer p's staging buffer, a one-warp kernel waits for the
peers' flags, and the reducing kernel sums the staged copies, applies 1/N + SGD to its shard and stores the new
bf16 weights into every peer. Master weights and momentum are sharded over the ranks by that kernel (rank r owns
shard r of every bucket); ``gather_master`` re-assembles full fp32 vectors when a checkpoint needs them.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import native_ops as K
from .._native import check
from ..utils.rng import XorShift128Plus
from . import p2p_kernels as PK
from .comm import AllreduceComm, CommWorker, GossipConfig

ALIGN = 64


GUARD_PATTERN = 0xA5


def guard_bytes() -> int:
    """Size of the guard band on each side of a peer-visible buffer: 256 bytes with RB_ARENA_GUARD=1, else none."""
    return 256 if os.environ.get("RB_ARENA_GUARD", "0") == "1" else 0


def arm_guards(raw: torch.Tensor, guard_elems: int) -> torch.Tensor:
    """Fill the first and last `guard_elems` elements of `raw` with the guard pattern; returns the payload view."""
    if guard_elems == 0:
        return raw
    b = raw.view(torch.uint8)
    gb = guard_elems * raw.element_size()
    b[:gb] = GUARD_PATTERN
    b[-gb:] = GUARD_PATTERN
    return raw[guard_elems: raw.numel() - guard_elems]


def guards_intact(raw: torch.Tensor, guard_elems: int) -> bool:
    if guard_elems == 0:
        return True
    b = raw.view(torch.uint8)
    gb = guard_elems * raw.element_size()
    return bool((b[:gb] == GUARD_PATTERN).all()) and bool((b[-gb:] == GUARD_PATTERN).all())


class SymmetricArena:
    """Peer-visible device tensors (one allocation per name) and their per-rank addresses.

    With RB_ARENA_GUARD=1 every buffer gets a 256-byte band of a fixed pattern before and after its payload; peers
    address the payload, so a kernel of any rank that writes outside a buffer it was given lands in a band and
    `damaged()` names the buffer (a debugging aid in place of a memory checker; off by default)."""

    def __init__(self, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self._symm = symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.tensors, self.handles = {}, {}
        self._raw, self._guard = {}, {}

    def alloc(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        dev = torch.device("cuda", torch.cuda.current_device())
        g = guard_bytes() // torch.empty(0, dtype=dtype).element_size()
        raw = self._symm.empty(int(numel) + 2 * g, dtype=dtype, device=dev)
        raw.zero_()
        t = arm_guards(raw, g)
        h = self._symm.rendezvous(raw, self.group.group_name)
        self.tensors[name], self.handles[name] = t, h
        self._raw[name], self._guard[name] = raw, g
        return t

    def _payload_offset(self, name: str) -> int:
        return self._guard[name] * self._raw[name].element_size()

    def ptrs(self, name: str) -> List[int]:
        off = self._payload_offset(name)
        return [int(p) + off for p in self.handles[name].buffer_ptrs]

    def multicast_ptr(self, name: str) -> int:
        try:
            mc = int(self.handles[name].multicast_ptr or 0)
        except (AttributeError, RuntimeError):
            return 0      # this torch build / this fabric has no multicast object for the allocation
        return mc + self._payload_offset(name) if mc else 0

    def damaged(self) -> List[str]:
        """Names of this rank's buffers whose guard bands no longer hold the pattern (always empty without guards)."""
        return [n for n, raw in self._raw.items() if not guards_intact(raw, self._guard[n])]

    def barrier(self, name: str):
        self.handles[name].barrier()


def _fill_ptrs(arr, ptrs):
    for i in range(PK.MAX_RANKS):
        arr[i] = ptrs[i] if i < len(ptrs) else None


class _P2PBase:
    """State shared by the kernel-driven backends: arena, flag pad, per-slot epoch counters."""

    def _init_p2p(self, group, num_slots=256):
        self.arena = SymmetricArena(group)
        self.num_slots = num_slots
        dev = torch.device("cuda", torch.cuda.current_device())
        self.flags = self.arena.alloc("flags", num_slots * 2 * PK.MAX_RANKS, torch.int32)
        self.epochs = torch.zeros(num_slots, dtype=torch.int32, device=dev)
        self.counters = torch.zeros(num_slots, dtype=torch.int32, device=dev)
        self.status = K.status_word()
        torch.cuda.synchronize()
        dist.barrier(self.arena.group)

    def _flag_ptrs(self):
        return self.arena.ptrs("flags")

    # limit of every wait on a peer inside the kernels of this backend, in ns (0 = the kernels' 3 s default)
    wait_ns = 0

    def _barrier_kernel(self, slot, stream):
        a = PK.BarrierArgs()
        _fill_ptrs(a.flags, self._flag_ptrs())
        a.epoch_ptr = self.epochs[slot:].data_ptr()
        a.status = self.status.data_ptr()
        a.rank, a.world, a.slot = self.rank, self.world, slot
        a.wait_ns = int(self.wait_ns)
        check(PK.fn("rb_barrier_p2p")(C.byref(a), stream.cuda_stream), "rb_barrier_p2p")


class FusedAllreduceSgdComm(AllreduceComm, _P2PBase):
    name = "fused_allreduce_sgd"
    graph_safe = True

    def __init__(self, group=None, bucket_bytes: int = 25 << 20, min_bucket_bytes: int = 4 << 20, blocks: int = 148,
                 one_shot_bytes: int = 256 << 10, replicate_master: bool = False, use_multimem: Optional[bool] = None):
        AllreduceComm.__init__(self, group)
        self._init_p2p(group)
        self.bucket_elems = bucket_bytes // 4 // ALIGN * ALIGN
        self.min_bucket_elems = min_bucket_bytes // 4
        self.one_shot_elems = one_shot_bytes // 4
        self.blocks = blocks
        self.replicate_master = replicate_master
        if use_multimem is None:
            use_multimem = os.environ.get("RB_MULTIMEM", "0") == "1"
        self.use_multimem = use_multimem
        # overlap=False launches every bucket after backward instead of from inside it; split_wait puts the wait
        # for the peers into a one-warp kernel so that the reducing kernel's blocks never spin on an SM
        self.overlap = os.environ.get("RB_COMM_OVERLAP", "1") == "1"
        self.split_wait = os.environ.get("RB_COMM_SPLIT_WAIT", "1") == "1"
        self.blocks = int(os.environ.get("RB_COMM_BLOCKS", self.blocks))
        self.wait_ok = torch.zeros(self.num_slots, dtype=torch.int32,
                                   device=torch.device("cuda", torch.cuda.current_device()))
        self.engine = None
        self.launches = []        # [(trigger op index, off, n, slot)]
        self._by_trigger = {}
        self._hyper = None
        self.kernel_launches_per_step = 0

    # the network asks us where its flat vectors should live
    def flat_allocator(self, name, n, dtype):
        if name in ("grads", "params16") or (name == "params" and self.replicate_master):
            return self.arena.alloc(name, n, dtype)
        return torch.zeros(n, dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()))

    def attach(self, engine):
        self.engine = engine
        net = engine.net
        self.net = net
        if self.world > 1 and "RB_GEMM_PDL" not in os.environ:
            # The compute kernels are launched without programmatic stream serialization while buckets are exchanged
            # beside the backward pass: with it their blocks sit resident on the SMs before they may run, and the
            # exchange kernels find fewer free thread slots (2.05 instead of 1.99 ms per AlexNet step on 2 GPUs; on
            # one GPU the same switch saves 3 %).
            K.gemm_set_option("pdl", 0)
        self.comm_stream = torch.cuda.Stream(net.device, priority=-1)
        # One stream: the buckets run one after another beside the backward pass. Alternating them between two
        # streams (RB_COMM_STREAMS=2: the push of bucket k+1 beside the reduction of bucket k) measured SLOWER on
        # AlexNet, 2.05 vs 1.94 ms per step on 2 GPUs and 2.09 vs 1.99 ms on 4: the backward pass's GEMMs then share
        # the SMs with two exchange kernels instead of one, and they are what the step waits for.
        self.comm_streams = [self.comm_stream]
        if int(os.environ.get("RB_COMM_STREAMS", "1")) > 1:
            self.comm_streams.append(torch.cuda.Stream(net.device, priority=-1))
        self._done2 = torch.cuda.Event()
        self._ready = torch.cuda.Event()
        self._done = torch.cuda.Event()
        self._plan(net)
        self.mc_grads = self.arena.multicast_ptr("grads") if self.use_multimem else 0
        self.mc_w16 = self.arena.multicast_ptr("params16") if self.use_multimem else 0
        self.setup_stage()

    def _shard_len(self, n):
        per = (n + self.world - 1) // self.world
        return (per + 7) // 8 * 8

    def setup_stage(self, avg_elems: Optional[int] = None):
        """Staging memory of the push-based exchange: per bucket, one slot per source rank of the length a rank
        reduces (its shard, or the whole bucket for one-shot buckets); one more region for `allreduce_average`."""
        self._stage_off = {}
        off = 0
        for _, _o, n, slot in self.launches:
            per = n if n <= self.one_shot_elems else self._shard_len(n)
            self._stage_off[slot] = off
            off += self.world * per
        avg = self.bucket_elems if avg_elems is None else avg_elems
        self._stage_off[self.num_slots - 1] = off
        off += self.world * self._shard_len(avg) + 64
        self._avg_cap = avg
        if self.world > 1 and not self.mc_grads:
            self.arena.alloc("stage", off, torch.float32)

    # ---- bucket plan: ranges of the flat vectors in the order backward completes them
    def _plan(self, net):
        ops = net.ops
        pending, pending_elems = [], 0
        slot = 0
        self.launches = []
        for idx in range(len(ops) - 2, 0, -1):
            op = ops[idx]
            for s in op.segs:
                n = (s.numel + ALIGN - 1) // ALIGN * ALIGN
                pending.append((s.offset, s.offset + n))
                pending_elems += n
            last = idx == 1
            if pending and (pending_elems >= self.min_bucket_elems or last):
                for lo, hi in self._merge(pending):
                    o = lo
                    while o < hi:
                        n = min(self.bucket_elems, hi - o)
                        self.launches.append((idx, o, n, slot))
                        slot += 1
                        o += n
                pending, pending_elems = [], 0
        if slot > self.num_slots:
            raise RuntimeError("too many gradient buckets for the flag pad")
        self._by_trigger = {}
        for rec in self.launches:
            self._by_trigger.setdefault(rec[0], []).append(rec)

    @staticmethod
    def _merge(ranges):
        out = []
        for lo, hi in sorted(ranges):
            if out and out[-1][1] == lo:
                out[-1] = (out[-1][0], hi)
            else:
                out.append((lo, hi))
        return out

    def shard_bounds(self, n):
        per = (n + self.world - 1) // self.world
        per = (per + 7) // 8 * 8
        return [(min(n, r * per), min(n, r * per + per)) for r in range(self.world)]

    # ---- per-step protocol driven by the engine
    def prepare(self, stepper, lr):
        self.kernel_launches_per_step = 0
        self._hyper = (float(lr), stepper.mu, stepper.l2, 1.0 / self.world, stepper.mode)

    def on_op_backward(self, op_index):
        recs = self._by_trigger.get(op_index)
        if not recs or not self.overlap:
            return
        cur = torch.cuda.current_stream()
        self._ready.record(cur)
        for s in self.comm_streams:
            s.wait_event(self._ready)
        for _, off, n, slot in recs:
            self._launch(off, n, slot, op=0)

    def fused_grads_step(self, stepper, lr):
        """Everything was launched from the backward hooks; join the communication streams."""
        if not self.overlap:
            self._ready.record(torch.cuda.current_stream())
            for s in self.comm_streams:
                s.wait_event(self._ready)
            for _, off, n, slot in self.launches:
                self._launch(off, n, slot, op=0)
        cur = torch.cuda.current_stream()
        for s, ev in zip(self.comm_streams, (self._done, self._done2)):
            ev.record(s)
            cur.wait_event(ev)

    def _launch(self, off, n, slot, op, buf="grads", scale=None):
        net = self.net
        a = PK.ArSgdArgs()
        _fill_ptrs(a.grads, self.arena.ptrs(buf))
        _fill_ptrs(a.w16, self.arena.ptrs("params16") if op == 0 else [])
        _fill_ptrs(a.w32, self.arena.ptrs("params") if (op == 0 and self.replicate_master) else [])
        _fill_ptrs(a.flags, self._flag_ptrs())
        a.w, a.v = net.params.data_ptr(), net.mom.data_ptr()
        a.mc_grads = (self.mc_grads or None) if buf == "grads" else None
        a.mc_w16 = self.mc_w16 or None
        push = self.world > 1 and not a.mc_grads
        if push:
            if buf != "grads":
                raise ValueError("the push exchange stages the gradient buffer only")
            _fill_ptrs(a.stage, self.arena.ptrs("stage"))
            a.stage_off = self._stage_off[slot]
            if slot == self.num_slots - 1 and n > self._avg_cap:
                raise ValueError("bucket larger than the staging region")
        a.zero_grads = 1 if (op == 0 and push) else 0
        a.epoch_ptr = self.epochs[slot:].data_ptr()
        a.block_counter = self.counters[slot:].data_ptr()
        a.status = self.status.data_ptr()
        a.off, a.n, a.decay_len = off, n, net.decay_len
        a.rank, a.world, a.slot = self.rank, self.world, slot
        a.one_shot = 1 if (op == 0 and n <= self.one_shot_elems) else 0
        a.op = op
        a.avg_scale = scale if scale is not None else 1.0 / self.world
        a.wait_ns = int(self.wait_ns)
        if op == 0:
            lr, mu, l2, gs, mode = self._hyper
            a.h.lr, a.h.mu, a.h.l2, a.h.grad_scale, a.h.mode, a.h.phase = lr, mu, l2, gs, mode, 3
        work = n if a.one_shot else (n + self.world - 1) // self.world
        blocks = max(1, min(self.blocks, (work // 8 + 127) // 128))
        streams = getattr(self, "comm_streams", None) or [self.comm_stream]
        stream = streams[slot % len(streams)] if op == 0 else self.comm_stream
        with torch.cuda.stream(stream):
            if push:
                pwork = (n if a.one_shot else self._shard_len(n)) * (self.world - 1)
                pblocks = max(1, min(self.blocks, (pwork // 16 + 127) // 128))
                check(PK.fn("rb_allreduce_push_p2p")(C.byref(a), pblocks, stream.cuda_stream),
                      "rb_allreduce_push_p2p")
                self.kernel_launches_per_step += 1
            if self.split_wait and self.world > 1:
                a.wait_ok = self.wait_ok[slot:].data_ptr()
                check(PK.fn("rb_allreduce_wait_p2p")(C.byref(a), stream.cuda_stream),
                      "rb_allreduce_wait_p2p")
                self.kernel_launches_per_step += 1
            check(PK.fn("rb_allreduce_sgd_p2p")(C.byref(a), blocks, stream.cuda_stream),
                  "rb_allreduce_sgd_p2p")
            if op == 0 and not push:
                # every peer has finished reading this bucket when the kernel ends; the push kernels zero
                # what they read themselves
                net.grads[off:off + n].zero_()
        self.bytes_moved += n * 4
        self.kernel_launches_per_step += 1

    # ---- whole-vector operations
    def allreduce_average(self, flat):
        """In-place average of the symmetric gradient buffer with the P2P kernel; other tensors use NCCL."""
        if self.world <= 1:
            return
        if flat.data_ptr() == self.net.grads.data_ptr():
            cur = torch.cuda.current_stream()
            self._ready.record(cur)
            self.comm_stream.wait_event(self._ready)
            off = 0
            slot = self.num_slots - 1
            total = flat.numel() // 8 * 8
            while off < total:
                n = min(self.bucket_elems, total - off)
                self._launch(off, n, slot, op=1)
                off += n
            self._done.record(self.comm_stream)
            cur.wait_event(self._done)
        else:
            super().allreduce_average(flat)

    def gather_master(self):
        """Make the fp32 master weights and momentum complete on every rank (owners broadcast their shards)."""
        if self.world <= 1 or self.replicate_master:
            return
        net = self.net
        torch.cuda.synchronize()
        for _, off, n, _slot in self.launches:
            if n <= self.one_shot_elems:
                continue
            for r, (s0, s1) in enumerate(self.shard_bounds(n)):
                if s1 > s0:
                    dist.broadcast(net.params[off + s0: off + s1], r, group=self.group)
                    dist.broadcast(net.mom[off + s0: off + s1], r, group=self.group)
        torch.cuda.synchronize()

    def exact_sync(self, flat):
        # replicas hold identical bf16 weights by construction; assembling the master is what a checkpoint needs
        self.gather_master()


class GossipP2PComm(CommWorker, _P2PBase):
    """Pair gossip (shared-seed permutation, synchronous) or pull gossip (random peer) through one kernel that
    reads the peer's published parameter snapshot over NVLink and mixes it in: x <- x - alpha (x - x_peer)."""
    name = "gossip_p2p"
    graph_safe = False

    def __init__(self, group=None, mode: str = "pair", alpha: float = 0.5, seed=(17, 29), blocks: int = 96,
                 cfg: GossipConfig = GossipConfig(), synchronous: Optional[bool] = None):
        CommWorker.__init__(self, group)
        self._init_p2p(group, num_slots=8)
        self.mode, self.alpha, self.blocks, self.cfg = mode, alpha, blocks, cfg
        # synchronous: wait until the peer has published the snapshot of the same exchange (always for pair gossip; pull gossip
        # is asynchronous by default and takes whichever snapshot the peer published last)
        self.synchronous = (mode == "pair") if synchronous is None else bool(synchronous)
        self.rng = XorShift128Plus(seed[0] + (0 if mode == "pair" else 1000003 * self.rank), seed[1])
        self.pub = None
        self._last_peer = None
        self.net = None

    def attach(self, engine):
        self.net = engine.net
        self.pub = self.arena.alloc("pub", 2 * self.net.flat_len, torch.float32)

    def _peers(self, repeat):
        """Peers of this exchange: one for pair gossip; `num_rounds` independent draws for pull gossip."""
        if repeat and self._last_peer is not None:
            return self._last_peer
        if self.mode == "pair":
            # the shared-seed permutation of the reference: rank r sends to perm[r], so r receives from the
            # rank whose target it is -- here r pulls from that rank
            perm = self.rng.permutation(self.world)
            peers = [perm.index(self.rank)]
        else:
            peers = [self.rng.below(self.world) for _ in range(max(1, self.cfg.num_rounds))]
        self._last_peer = peers
        return peers

    def sync_params(self, flat, repeat=False):
        """Pair gossip: x <- (1 - alpha) x + alpha x_peer. Pull gossip: x <- mean of x and the snapshots of
        `num_rounds` randomly drawn ranks (src/worker/gossip_pull_dist_rdma.rs:517-589), as a running mean:
        pull k mixes with weight 1 / (k + 1)."""
        if self.world <= 1:
            return
        net = self.net
        is_params = flat.data_ptr() == net.params.data_ptr()
        peers = self._peers(repeat)
        st = torch.cuda.current_stream()
        a = PK.MixArgs()
        _fill_ptrs(a.flags, self._flag_ptrs())
        a.w = flat.data_ptr()
        a.w16 = net.params16.data_ptr() if is_params else None
        a.pub_local = self.pub.data_ptr()
        slot = 0 if is_params else 1
        a.epoch_ptr = self.epochs[slot:].data_ptr()
        a.block_counter = self.counters[slot:].data_ptr()
        a.status = self.status.data_ptr()
        a.n = flat.numel() // 4 * 4
        a.rank, a.world, a.slot = self.rank, self.world, slot
        a.wait_peer = 1 if self.synchronous else 0
        a.wait_ns = int(self.wait_ns)
        a.mix_self = 0 if self.mode == "pair" else 1
        a.w_self = 1.0
        a.peer = peers[0]
        check(PK.fn("rb_publish_p2p")(C.byref(a), self.blocks, st.cuda_stream), "rb_publish_p2p")
        for k, peer in enumerate(peers):
            a.peer = peer
            a.pub_peer = self.arena.ptrs("pub")[peer]
            a.alpha = self.alpha if self.mode == "pair" else 1.0 / (k + 2)
            a.not_last = 0 if k == len(peers) - 1 else 1
            check(PK.fn("rb_gossip_mix_p2p")(C.byref(a), self.blocks, st.cuda_stream), "rb_gossip_mix_p2p")
            self.bytes_moved += a.n * 4

    def allreduce_average(self, flat):
        CommWorker.exact_sync(self, flat)


class GroupGossipP2PComm(GossipP2PComm):
    """Hierarchical exchange on the gossip kernels: first the mean over this rank's group of `group_size` consecutive
    ranks, then gossip between groups.

    version 2 (default; src/worker/gossip_pull_allreduce_dist_rdma_v2.rs:327-384): every rank pulls the group mean of
    one uniformly random rank and keeps 0.5 * (pulled + own group mean).
    version 1 (src/worker/gossip_pull_allreduce_dist_rdma.rs:327-402): only the group leaders (first rank of each
    group) gossip -- a leader pulls the group mean of a uniformly random leader and keeps 0.5 * (pulled + own) unless it
    drew itself -- and every other rank then takes its leader's result.

    All phases use the publish + mix kernels of the flat gossip: in phase one a rank pulls the snapshots of its group
    peers as a running mean (pull k with weight 1 / (k + 2)); in the gossip phase it publishes the group mean and pulls
    one more snapshot with weight 1/2; version 1 adds a phase in which the followers pull their leader's snapshot
    with weight 1. Every rank runs every phase, so the epochs of the flag protocol stay in step; a rank with nothing
    to do in a phase issues a mix that lands on itself and changes nothing.
    """
    name = "group_allreduce_gossip_p2p"

    def __init__(self, group=None, group_size: int = 2, seed=(53, 59), blocks: int = 96, version: int = 2):
        super().__init__(group, mode="pull", seed=seed, blocks=blocks, synchronous=True)
        if version not in (1, 2):
            raise ValueError("version must be 1 or 2")
        self.version = version
        self._init_groups(group_size, seed)

    def _init_groups(self, group_size, seed):
        self.group_size = max(1, min(group_size, self.world))
        g0 = self.rank // self.group_size * self.group_size
        self.leader = g0
        self.num_groups = (self.world + self.group_size - 1) // self.group_size
        self.group_peers = [r for r in range(g0, min(self.world, g0 + self.group_size)) if r != self.rank]
        # version 1: a leader's draws come from its own stream, indexed by its position among the leaders (the
        # stream the library backend gives the leaders' pull gossip)
        self.leader_rng = XorShift128Plus(seed[0] + 1000003 * (self.rank // self.group_size), seed[1])

    def _phase(self, a, peers, weights, mix_self, st):
        a.mix_self = mix_self
        a.peer = peers[0]
        check(PK.fn("rb_publish_p2p")(C.byref(a), self.blocks, st.cuda_stream), "rb_publish_p2p")
        for k, (peer, alpha) in enumerate(zip(peers, weights)):
            a.peer = peer
            a.pub_peer = self.arena.ptrs("pub")[peer]
            a.alpha = alpha
            a.not_last = 0 if k == len(peers) - 1 else 1
            check(PK.fn("rb_gossip_mix_p2p")(C.byref(a), self.blocks, st.cuda_stream), "rb_gossip_mix_p2p")
            self.bytes_moved += a.n * 4

    def sync_params(self, flat, repeat=False):
        if self.world <= 1:
            return
        net = self.net
        is_params = flat.data_ptr() == net.params.data_ptr()
        if not (repeat and self._last_peer is not None):
            if self.version == 2:
                self._last_peer = [self.rng.below(self.world)]
            elif self.rank == self.leader and self.num_groups > 1:
                self._last_peer = [self.leader_rng.below(self.num_groups) * self.group_size]
            else:
                self._last_peer = [self.rank]
        st = torch.cuda.current_stream()
        a = PK.MixArgs()
        _fill_ptrs(a.flags, self._flag_ptrs())
        a.w = flat.data_ptr()
        a.w16 = net.params16.data_ptr() if is_params else None
        a.pub_local = self.pub.data_ptr()
        slot = 0 if is_params else 1
        a.epoch_ptr = self.epochs[slot:].data_ptr()
        a.block_counter = self.counters[slot:].data_ptr()
        a.status = self.status.data_ptr()
        a.n = flat.numel() // 4 * 4
        a.rank, a.world, a.slot = self.rank, self.world, slot
        a.wait_peer = 1
        a.wait_ns = int(self.wait_ns)
        a.w_self = 1.0
        peers = self.group_peers or [self.rank]
        self._phase(a, peers, [1.0 / (k + 2) for k in range(len(peers))], 0, st)
        if self.version == 2:
            self._phase(a, self._last_peer, [0.5], 1, st)
            return
        # version 1: leaders gossip (a self-draw keeps the own group mean: mix_self = 0), then followers copy
        self._phase(a, self._last_peer, [0.5], 0, st)
        self._phase(a, [self.leader], [1.0], 0, st)


class ElasticP2PComm(CommWorker, _P2PBase):
    """Elastic averaging with the centre in rank 0's memory (beta = 0.8 / N, src/worker/elasticserver_dist.rs:249).

    Asynchronous (the default, as in the reference): a client takes the centre's lock word with a compare-and-swap,
    mixes with the centre as it is at that moment -- x <- x - beta (x - c), c <- c + beta (x - c), read and written
    through peer memory in one kernel -- and releases the lock. Clients are served one at a time and may be any number
    of iterations apart; nobody waits for another rank to reach a round. A client that does not get the lock within
    `lock_wait_ns` gives that exchange up (`skipped_exchanges()` counts them).

    `synchronous=True` is the lock-step form: every client mixes with the same centre snapshot, the pulls are summed
    into rank 0's accumulator and folded into the centre between two cross-GPU barriers."""
    name = "elastic_p2p"
    graph_safe = False

    def __init__(self, group=None, beta: Optional[float] = None, blocks: int = 96, synchronous: bool = False,
                 lock_wait_ns: int = 200_000_000):
        CommWorker.__init__(self, group)
        self._init_p2p(group, num_slots=8)
        self.beta = beta if beta is not None else 0.8 / max(1, self.world)
        self.blocks = blocks
        self.synchronous = bool(synchronous)
        self.lock_wait_ns = int(lock_wait_ns)
        self.net = None

    def attach(self, engine):
        self.net = engine.net
        n = self.net.flat_len
        self.center = self.arena.alloc("center", n, torch.float32)
        self.delta = self.arena.alloc("delta", n, torch.float32)
        self.lock = self.arena.alloc("lock", 8, torch.int64)
        self.ticket = torch.zeros(4, dtype=torch.int32, device=self.center.device)
        self.skipped = torch.zeros(1, dtype=torch.int32, device=self.center.device)

    def first_one_way_sync(self, flat):
        if self.world > 1:
            dist.broadcast(flat, 0, group=self.group)
        self.center.copy_(flat)
        torch.cuda.synchronize()
        dist.barrier(self.group)

    def skipped_exchanges(self) -> int:
        """Exchanges this rank gave up because the centre stayed locked for longer than `lock_wait_ns`."""
        return int(self.skipped.item())

    def sync_params(self, flat, repeat=False):
        if self.world <= 1:
            return
        net = self.net
        st = torch.cuda.current_stream()
        a = PK.MixArgs()
        _fill_ptrs(a.flags, self._flag_ptrs())
        a.w = flat.data_ptr()
        a.w16 = net.params16.data_ptr() if flat.data_ptr() == net.params.data_ptr() else None
        a.pub_peer = self.arena.ptrs("center")[0]
        a.status = self.status.data_ptr()
        a.n = flat.numel() // 4 * 4
        a.rank, a.world = self.rank, self.world
        a.alpha = self.beta
        if not self.synchronous:
            a.gate = self.arena.ptrs("lock")[0]
            a.ticket = self.ticket.data_ptr()
            a.skipped = self.skipped.data_ptr()
            a.block_counter = self.counters[4:].data_ptr()
            a.wait_ns = self.lock_wait_ns
            check(PK.fn("rb_elastic_begin_p2p")(C.byref(a), st.cuda_stream), "rb_elastic_begin_p2p")
            check(PK.fn("rb_elastic_mix_p2p")(C.byref(a), self.blocks, st.cuda_stream), "rb_elastic_mix_p2p")
            self.bytes_moved += a.n * 8
            return
        a.acc_target = self.arena.ptrs("delta")[0]
        a.wait_ns = int(self.wait_ns)
        check(PK.fn("rb_elastic_pull_p2p")(C.byref(a), self.blocks, st.cuda_stream), "rb_elastic_pull_p2p")
        self._barrier_kernel(2, st)
        if self.rank == 0:
            check(PK.fn("rb_elastic_apply")(self.center.data_ptr(), self.delta.data_ptr(), a.n, st.cuda_stream),
                  "rb_elastic_apply")
        self._barrier_kernel(3, st)
        self.bytes_moved += a.n * 8

    def exact_sync(self, flat):
        if self.world <= 1:
            return
        if self.rank == 0:
            flat.copy_(self.center)
        dist.broadcast(flat, 0, group=self.group)

    allreduce_average = CommWorker.exact_sync


class PushGossipP2PComm(CommWorker, _P2PBase):
    """Push gossip: every rank adds its vector into a random target's accumulator with peer-to-peer reductions and
    keeps (w_self * own + received) / (w_self + count), w_self = 2 when it drew itself.

    Asynchronous (the default, as in the reference, src/worker/gossip_dist.rs:474-593,883-976): no barrier. A pusher
    registers at the target's gate word, adds into whichever of the target's two accumulators is open, and counts
    itself in; at its own exchange a rank closes its open accumulator, waits only for pushes already in flight into it
    and folds in whatever arrived -- nothing, if nobody pushed (`recv_count == 0`). A push that arrives after the
    close lands in the other accumulator and is folded one exchange later. Ranks may be any number of iterations apart.

    `synchronous=True` is the lock-step form: push, cross-GPU barrier, fold, barrier."""
    name = "gossip_push_p2p"
    graph_safe = False

    def __init__(self, group=None, seed=(41, 43), blocks: int = 96, synchronous: bool = False):
        CommWorker.__init__(self, group)
        self._init_p2p(group, num_slots=8)
        self.rng = XorShift128Plus(seed[0] + 7919 * self.rank, seed[1])
        self.blocks = blocks
        self.synchronous = bool(synchronous)
        self.net = None

    def attach(self, engine):
        self.net = engine.net
        n = self.net.flat_len
        self.acc = self.arena.alloc("acc", 2 * n, torch.float32)     # two accumulators (the synchronous form uses one)
        self.count = self.arena.alloc("count", ALIGN, torch.float32)
        self.gate = self.arena.alloc("gate", 8, torch.int64)
        self.ticket = torch.zeros(4, dtype=torch.int32, device=self.acc.device)

    def sync_params(self, flat, repeat=False):
        if self.world <= 1:
            return
        net = self.net
        target = self.rng.below(self.world)
        st = torch.cuda.current_stream()
        a = PK.MixArgs()
        _fill_ptrs(a.flags, self._flag_ptrs())
        a.w = flat.data_ptr()
        a.w16 = net.params16.data_ptr() if flat.data_ptr() == net.params.data_ptr() else None
        a.acc_target = self.arena.ptrs("acc")[target]
        a.count_target = self.arena.ptrs("count")[target]
        a.block_counter = self.counters[4:].data_ptr()
        a.status = self.status.data_ptr()
        a.n = flat.numel() // 4 * 4
        a.rank, a.world, a.peer = self.rank, self.world, target
        a.w_self = 2.0 if target == self.rank else 1.0
        a.wait_ns = int(self.wait_ns)
        if not self.synchronous:
            a.gate = self.arena.ptrs("gate")[target]
            a.ticket = self.ticket.data_ptr()
            check(PK.fn("rb_push_begin_p2p")(C.byref(a), st.cuda_stream), "rb_push_begin_p2p")
            check(PK.fn("rb_push_add_async_p2p")(C.byref(a), self.blocks, st.cuda_stream), "rb_push_add_async_p2p")
            a.gate = self.gate.data_ptr()
            a.ticket = self.ticket[1:].data_ptr()
            a.acc_target = self.acc.data_ptr()
            a.count_target = self.count.data_ptr()
            a.block_counter = self.counters[5:].data_ptr()
            check(PK.fn("rb_fold_begin_p2p")(C.byref(a), st.cuda_stream), "rb_fold_begin_p2p")
            check(PK.fn("rb_fold_p2p")(C.byref(a), self.blocks, st.cuda_stream), "rb_fold_p2p")
            self.bytes_moved += a.n * 4
            return
        check(PK.fn("rb_push_add_p2p")(C.byref(a), self.blocks, st.cuda_stream), "rb_push_add_p2p")
        self._barrier_kernel(2, st)
        a.acc_target = self.acc.data_ptr()
        a.count_target = self.count.data_ptr()
        check(PK.fn("rb_push_finalize")(C.byref(a), self.blocks, st.cuda_stream), "rb_push_finalize")
        self._barrier_kernel(3, st)
        self.bytes_moved += a.n * 4

    allreduce_average = CommWorker.exact_sync


def make(name: str, **kw) -> CommWorker:
    if name == "fused_allreduce_sgd":
        return FusedAllreduceSgdComm(**kw)
    if name == "gossip_p2p":
        return GossipP2PComm(**kw)
    if name == "gossip_pull_p2p":
        return GossipP2PComm(mode="pull", **kw)
    if name == "gossip_push_p2p":
        return PushGossipP2PComm(**kw)
    if name == "elastic_p2p":
        return ElasticP2PComm(**kw)
    if name == GroupGossipP2PComm.name:
        return GroupGossipP2PComm(**kw)
    raise ValueError(name)
