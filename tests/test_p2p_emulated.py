"""Host-side orchestration of the kernel-driven gossip backends, with the kernels replaced by CPU stand-ins.

The stand-ins implement what the publish / mix kernels are specified to do (snapshot the vector; mix with a peer's
snapshot of the same epoch), so these tests pin the sequence of launches, peers and weights that the Python side
issues -- the part that needs no GPU. The kernels themselves are checked against library collectives on GPUs.
"""
import types

import pytest
import torch

from rembrandt_b200.parallel import p2p
from rembrandt_b200.parallel import p2p_kernels as PK
from rembrandt_b200.utils.rng import XorShift128Plus


class FakeWorld:
    """All ranks in one process; launches are queued per rank and run phase by phase (publish, then the mixes)."""

    def __init__(self, world, n):
        self.world, self.n = world, n
        self.w = [torch.zeros(n) for _ in range(world)]
        self.queue = [[] for _ in range(world)]
        self.current = 0

    def fn(self, name):
        def launch(args_ref, blocks, stream):
            a = args_ref._obj
            self.queue[self.current].append((name, a.peer, a.alpha, a.not_last, a.mix_self, a.wait_peer))
            return 0
        return launch

    def run(self):
        phases = []
        for r in range(self.world):
            mine, cur = [], None
            for op in self.queue[r]:
                if op[0] == "rb_publish_p2p":
                    cur = []
                    mine.append(cur)
                else:
                    cur.append(op)
            phases.append(mine)
        assert len({len(p) for p in phases}) == 1, "every rank must run the same number of publish phases"
        for ph in range(len(phases[0])):
            snap = [w.clone() for w in self.w]
            for r in range(self.world):
                ops = phases[r][ph]
                assert ops, "a phase without a mix would never advance the epoch"
                assert [o[3] for o in ops] == [1] * (len(ops) - 1) + [0], "only the last mix of a phase ends the epoch"
                for _, peer, alpha, _, mix_self, wait_peer in ops:
                    assert wait_peer == 1
                    if peer != r or mix_self:
                        self.w[r].copy_((1 - alpha) * self.w[r] + alpha * snap[peer])     # in place: callers hold it
        self.queue = [[] for _ in range(self.world)]


def _make(rank, world, group_size, seed, fake):
    c = object.__new__(p2p.GroupGossipP2PComm)
    c.rank, c.world, c.group, c.bytes_moved = rank, world, None, 0
    c.mode, c.alpha, c.blocks, c.synchronous = "pull", 0.5, 8, True
    c.rng = XorShift128Plus(seed[0] + 1000003 * rank, seed[1])
    c._last_peer = None
    c.version = 2
    c._init_groups(group_size, seed)
    c.net = types.SimpleNamespace(params=fake.w[rank], params16=torch.zeros(1))
    c.pub = torch.zeros(1)
    c.epochs = torch.zeros(4, dtype=torch.int32)
    c.counters = torch.zeros(4, dtype=torch.int32)
    c.status = torch.zeros(1, dtype=torch.int32)
    c.arena = types.SimpleNamespace(ptrs=lambda name: [0] * world)
    return c


@pytest.mark.parametrize("world,group_size", [(2, 1), (2, 2), (4, 2), (5, 3), (8, 4)])
def test_group_gossip_launch_sequence_gives_group_mean_then_half_pull(monkeypatch, world, group_size):
    n = 16
    fake = FakeWorld(world, n)
    monkeypatch.setattr(PK, "fn", fake.fn)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda: types.SimpleNamespace(cuda_stream=0))
    comms = [_make(r, world, group_size, (53, 59), fake) for r in range(world)]
    for rnd in range(3):
        torch.manual_seed(rnd)
        start = [torch.randn(n) for _ in range(world)]
        for r in range(world):
            fake.w[r] = start[r].clone()
            comms[r].net.params = fake.w[r]
        for r in range(world):
            fake.current = r
            comms[r].sync_params(fake.w[r])
        fake.run()
        gmean = []
        for r in range(world):
            g0 = r // group_size * group_size
            members = range(g0, min(world, g0 + group_size))
            gmean.append(sum(start[m] for m in members) / len(members))
        for r in range(world):
            peer = comms[r]._last_peer[0]
            assert torch.allclose(fake.w[r], 0.5 * (gmean[r] + gmean[peer]), atol=1e-6), (rnd, r)
    # the draws are the per-rank streams of the library backend, so both backends pick the same peers
    ref = XorShift128Plus(53 + 1000003 * 1, 59)
    assert [ref.below(world) for _ in range(3)][-1] == comms[1]._last_peer[0]


@pytest.mark.parametrize("world,group_size", [(2, 1), (4, 2), (6, 2), (8, 4), (5, 3)])
def test_leader_gossip_launch_sequence_gives_every_group_its_leaders_result(monkeypatch, world, group_size):
    """First version of the hierarchical scheme: group mean, gossip among the group leaders only, followers take their
    leader's result (src/worker/gossip_pull_allreduce_dist_rdma.rs:327-402)."""
    n = 16
    fake = FakeWorld(world, n)
    monkeypatch.setattr(PK, "fn", fake.fn)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda: types.SimpleNamespace(cuda_stream=0))
    comms = [_make(r, world, group_size, (53, 59), fake) for r in range(world)]
    for c in comms:
        c.version = 1
    groups = (world + group_size - 1) // group_size
    shadows = {g: XorShift128Plus(53 + 1000003 * g, 59) for g in range(groups)}
    mixed = 0
    for rnd in range(4):
        torch.manual_seed(70 + rnd)
        start = [torch.randn(n) for _ in range(world)]
        for r in range(world):
            fake.w[r] = start[r].clone()
            comms[r].net.params = fake.w[r]
        for r in range(world):
            fake.current = r
            comms[r].sync_params(fake.w[r])
        fake.run()

        def gmean(g):
            members = range(g * group_size, min(world, (g + 1) * group_size))
            return sum(start[m] for m in members) / len(members)

        for g in range(groups):
            drawn = shadows[g].below(groups) if groups > 1 else g
            want = gmean(g) if drawn == g else 0.5 * (gmean(g) + gmean(drawn))
            mixed += drawn != g
            for r in range(g * group_size, min(world, (g + 1) * group_size)):
                assert torch.allclose(fake.w[r], want, atol=1e-6), (rnd, r, drawn)
    assert groups == 1 or mixed > 0


def test_guard_bands_detect_writes_outside_the_payload(monkeypatch):
    monkeypatch.setenv("RB_ARENA_GUARD", "1")
    assert p2p.guard_bytes() == 256
    for dtype in (torch.float32, torch.int32, torch.bfloat16, torch.uint8):
        g = p2p.guard_bytes() // torch.empty(0, dtype=dtype).element_size()
        raw = torch.zeros(100 + 2 * g, dtype=dtype)
        payload = p2p.arm_guards(raw, g)
        assert payload.numel() == 100 and payload.data_ptr() == raw.data_ptr() + 256
        payload.fill_(3)
        assert p2p.guards_intact(raw, g)
        raw[g - 1] = 1                      # one element before the payload
        assert not p2p.guards_intact(raw, g)
        p2p.arm_guards(raw, g)
        raw[g + 100] = 1                    # one element after it
        assert not p2p.guards_intact(raw, g)
    monkeypatch.setenv("RB_ARENA_GUARD", "0")
    assert p2p.guard_bytes() == 0
    raw = torch.zeros(8)
    assert p2p.arm_guards(raw, 0) is raw and p2p.guards_intact(raw, 0)


def test_trace_spans_are_inert_without_cuda(monkeypatch):
    from rembrandt_b200.utils import trace
    with trace.span("x"):
        pass
    monkeypatch.setattr(trace, "ENABLED", True)
    with trace.span("forward"):             # no CUDA here: still nothing to push
        pass
    assert trace.span("a") is trace.span("b")


def _make_flat(rank, world, mode, seed, fake, rounds=1, alpha=0.5):
    from rembrandt_b200.parallel.comm import GossipConfig
    c = object.__new__(p2p.GossipP2PComm)
    c.rank, c.world, c.group, c.bytes_moved = rank, world, None, 0
    c.mode, c.alpha, c.blocks, c.cfg = mode, alpha, 8, GossipConfig(num_rounds=rounds)
    c.synchronous = True
    c.rng = XorShift128Plus(seed[0] + (0 if mode == "pair" else 1000003 * rank), seed[1])
    c._last_peer = None
    c.net = types.SimpleNamespace(params=fake.w[rank], params16=torch.zeros(1))
    c.pub = torch.zeros(1)
    c.epochs = torch.zeros(4, dtype=torch.int32)
    c.counters = torch.zeros(4, dtype=torch.int32)
    c.status = torch.zeros(1, dtype=torch.int32)
    c.arena = types.SimpleNamespace(ptrs=lambda name: [0] * world)
    return c


@pytest.mark.parametrize("world", [2, 5, 8])
def test_pair_gossip_launches_follow_the_shared_permutation(monkeypatch, world):
    n = 12
    fake = FakeWorld(world, n)
    monkeypatch.setattr(PK, "fn", fake.fn)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda: types.SimpleNamespace(cuda_stream=0))
    comms = [_make_flat(r, world, "pair", (17, 29), fake, alpha=0.25) for r in range(world)]
    shadow = XorShift128Plus(17, 29)
    for rnd in range(4):
        torch.manual_seed(10 + rnd)
        start = [torch.randn(n) for _ in range(world)]
        for r in range(world):
            fake.w[r] = start[r].clone()
            comms[r].net.params = fake.w[r]
            fake.current = r
            comms[r].sync_params(fake.w[r])
        fake.run()
        perm = shadow.permutation(world)
        for r in range(world):
            src = perm.index(r)                      # the rank whose target r is
            want = start[r] if src == r else 0.75 * start[r] + 0.25 * start[src]
            assert torch.allclose(fake.w[r], want, atol=1e-6), (rnd, r)


@pytest.mark.parametrize("rounds", [1, 3])
def test_pull_gossip_launches_average_own_vector_and_drawn_snapshots(monkeypatch, rounds):
    world, n = 6, 12
    fake = FakeWorld(world, n)
    monkeypatch.setattr(PK, "fn", fake.fn)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda: types.SimpleNamespace(cuda_stream=0))
    comms = [_make_flat(r, world, "pull", (31, 37), fake, rounds=rounds) for r in range(world)]
    for rnd in range(3):
        torch.manual_seed(20 + rnd)
        start = [torch.randn(n) for _ in range(world)]
        for r in range(world):
            fake.w[r] = start[r].clone()
            comms[r].net.params = fake.w[r]
            fake.current = r
            comms[r].sync_params(fake.w[r])
        fake.run()
        for r in range(world):
            peers = comms[r]._last_peer
            assert len(peers) == rounds
            want = (start[r] + sum(start[p] for p in peers)) / (rounds + 1)
            assert torch.allclose(fake.w[r], want, atol=1e-6), (rnd, r, peers)
    again = comms[0]._last_peer
    fake.current = 0
    comms[0].sync_params(fake.w[0], repeat=True)      # `repeat` reuses the drawn peers (parameters, then gradients)
    assert comms[0]._last_peer == again


# ---- push gossip and elastic averaging: launches separated by barrier kernels, buffers named by raw addresses ------
class PtrWorld:
    """All ranks in one process. Launches are queued per rank and run stage by stage, a stage ending at each barrier
    launch; addresses in the argument blocks are resolved back to the CPU tensors registered here."""

    def __init__(self, world, n):
        self.world, self.n = world, n
        self.tensors, self.shared = [], {}
        self.queue = [[] for _ in range(world)]
        self.current = 0

    def reg(self, t):
        self.tensors.append(t)
        return t

    def view(self, ptr):
        for t in self.tensors:
            lo = t.data_ptr()
            if lo <= ptr < lo + t.numel() * 4:
                return t.reshape(-1)[(ptr - lo) // 4:]
        raise KeyError(hex(ptr))

    def arena(self, rank):
        def alloc(name, numel, dtype):
            t = self.reg(torch.zeros(int(numel), dtype=dtype))
            self.shared.setdefault(name, {})[rank] = t
            return t
        return types.SimpleNamespace(alloc=alloc, ptrs=lambda name: [self.shared[name][r].data_ptr()
                                                                     for r in range(self.world)])

    def fn(self, name):
        def launch(*args):
            a = args[0]
            if hasattr(a, "_obj"):
                a = type(a._obj).from_buffer_copy(a._obj)
            self.queue[self.current].append((name, a, args[1:]))
            return 0
        return launch

    def run(self):
        stages = []
        for q in self.queue:
            mine, cur = [], []
            for item in q:
                if item[0] == "rb_barrier_p2p":
                    mine.append(cur)
                    cur = []
                else:
                    cur.append(item)
            assert not cur, "every exchange must end with a barrier"
            stages.append(mine)
        assert len({len(s) for s in stages}) == 1
        for k in range(len(stages[0])):
            for r in range(self.world):
                for name, a, rest in stages[r][k]:
                    getattr(self, "_" + name)(a, rest)
        self.queue = [[] for _ in range(self.world)]

    def _rb_push_add_p2p(self, a, rest):
        if a.peer != a.rank:
            self.view(a.acc_target)[: a.n] += self.view(a.w)[: a.n]
            self.view(a.count_target)[0] += 1.0

    def _rb_push_finalize(self, a, rest):
        cnt = float(self.view(a.count_target)[0])
        if cnt > 0:
            w, acc = self.view(a.w)[: a.n], self.view(a.acc_target)[: a.n]
            w.copy_((a.w_self * w + acc) / (a.w_self + cnt))
            acc.zero_()
        self.view(a.count_target)[0] = 0.0

    def _rb_elastic_pull_p2p(self, a, rest):
        w, c = self.view(a.w)[: a.n], self.view(a.pub_peer)[: a.n]
        d = a.alpha * (w - c)
        w.sub_(d)
        self.view(a.acc_target)[: a.n] += d

    def _rb_elastic_apply(self, center_ptr, rest):
        delta_ptr, n = rest[0], rest[1]
        c, d = self.view(center_ptr)[:n], self.view(delta_ptr)[:n]
        c.add_(d)
        d.zero_()


def _bare(cls, pw, rank, world):
    c = object.__new__(cls)
    c.rank, c.world, c.group, c.bytes_moved, c.blocks = rank, world, None, 0, 8
    c.arena = pw.arena(rank)
    c.flags = c.arena.alloc("flags", 64, torch.int32)
    c.epochs = torch.zeros(8, dtype=torch.int32)
    c.counters = torch.zeros(8, dtype=torch.int32)
    c.status = torch.zeros(1, dtype=torch.int32)
    w = pw.reg(torch.zeros(pw.n))
    c.net = types.SimpleNamespace(params=w, params16=torch.zeros(1), flat_len=pw.n)
    return c, w


def test_push_gossip_launches_give_the_count_normalised_mean(monkeypatch):
    world, n = 5, 16
    pw = PtrWorld(world, n)
    monkeypatch.setattr(PK, "fn", pw.fn)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda: types.SimpleNamespace(cuda_stream=0))
    comms, ws = [], []
    for r in range(world):
        c, w = _bare(p2p.PushGossipP2PComm, pw, r, world)
        c.rng = XorShift128Plus(41 + 7919 * r, 43)
        c.synchronous = True
        c.attach(types.SimpleNamespace(net=c.net))
        comms.append(c)
        ws.append(w)
    shadows = [XorShift128Plus(41 + 7919 * r, 43) for r in range(world)]
    for rnd in range(4):
        torch.manual_seed(30 + rnd)
        start = [torch.randn(n) for _ in range(world)]
        targets = [s.below(world) for s in shadows]
        for r in range(world):
            ws[r].copy_(start[r])
            pw.current = r
            comms[r].sync_params(ws[r])
        pw.run()
        for r in range(world):
            received = [start[s] for s in range(world) if targets[s] == r and s != r]
            w_self = 2.0 if targets[r] == r else 1.0
            want = (w_self * start[r] + sum(received)) / (w_self + len(received)) if received else start[r]
            assert torch.allclose(ws[r], want, atol=1e-6), (rnd, r, targets)
            assert float(comms[r].acc.abs().sum()) == 0.0 and float(comms[r].count[0]) == 0.0


# ---- the asynchronous forms: no barrier launches; every launch runs the moment it is issued ------------------------
class AsyncWorld(PtrWorld):
    """Kernels run immediately, in the order the ranks issue them: a sequential schedule of an asynchronous exchange.
    The stand-ins restate the gate / ticket / lock protocol of the kernels on CPU tensors."""

    def view64(self, ptr):
        for t in self.tensors:
            lo = t.data_ptr()
            if t.dtype == torch.int64 and lo <= ptr < lo + t.numel() * 8:
                return t.reshape(-1)[(ptr - lo) // 8:]
        raise KeyError(hex(ptr))

    def view32(self, ptr):
        for t in self.tensors:
            lo = t.data_ptr()
            if t.dtype == torch.int32 and lo <= ptr < lo + t.numel() * 4:
                return t.reshape(-1)[(ptr - lo) // 4:]
        raise KeyError(hex(ptr))

    def fn(self, name):
        def launch(*args):
            a = args[0]
            if hasattr(a, "_obj"):
                a = type(a._obj).from_buffer_copy(a._obj)
            self.log.append((self.current, name))
            getattr(self, "_" + name)(a, args[1:])
            return 0
        return launch

    def _rb_push_begin_p2p(self, a, rest):
        buf = -1
        if a.peer != a.rank:
            gate = self.view64(a.gate)
            buf = (int(gate[0]) >> 32) & 1
            gate[0] += 1 << (16 * buf)
        self.view32(a.ticket)[0] = buf

    def _rb_push_add_async_p2p(self, a, rest):
        buf = int(self.view32(a.ticket)[0])
        if buf < 0:
            return
        self.view(a.acc_target)[buf * a.n: (buf + 1) * a.n] += self.view(a.w)[: a.n]
        self.view(a.count_target)[buf] += 1.0
        self.view64(a.gate)[0] -= 1 << (16 * buf)

    def _rb_fold_begin_p2p(self, a, rest):
        gate = self.view64(a.gate)
        closed = (int(gate[0]) >> 32) & 1
        gate[0] += 1 << 32
        assert (int(gate[0]) >> (16 * closed)) & 0xFFFF == 0, "a sequential schedule leaves no push in flight"
        self.view32(a.ticket)[0] = closed

    def _rb_fold_p2p(self, a, rest):
        buf = int(self.view32(a.ticket)[0])
        cnt = float(self.view(a.count_target)[buf])
        if cnt > 0:
            w, acc = self.view(a.w)[: a.n], self.view(a.acc_target)[buf * a.n: (buf + 1) * a.n]
            w.copy_((a.w_self * w + acc) / (a.w_self + cnt))
            acc.zero_()
        self.view(a.count_target)[buf] = 0.0

    def _rb_elastic_begin_p2p(self, a, rest):
        lock = self.view64(a.gate)
        got = 0
        if int(lock[0]) == 0:
            lock[0] = a.rank + 1
            got = 1
        else:
            self.view32(a.skipped)[0] += 1
        self.view32(a.ticket)[0] = got

    def _rb_elastic_mix_p2p(self, a, rest):
        if int(self.view32(a.ticket)[0]) != 1:
            return
        w, c = self.view(a.w)[: a.n], self.view(a.pub_peer)[: a.n]
        d = a.alpha * (w - c)
        w.sub_(d)
        c.add_(d)
        self.view64(a.gate)[0] = 0


def _bare_async(cls, pw, rank, world):
    c, w = _bare(cls, pw, rank, world)
    real_alloc = c.arena.alloc

    def alloc(name, numel, dtype):
        return pw.reg(real_alloc(name, numel, dtype)) if dtype != torch.float32 else real_alloc(name, numel, dtype)
    c.arena.alloc = alloc
    return c, w


def test_asynchronous_push_gossip_follows_the_sequential_oracle_with_ranks_steps_apart(monkeypatch):
    """Rank 0 exchanges three times as often as the others; nobody waits. Oracle: the accumulate / count / fold rules
    written out per rank (src/worker/gossip_dist.rs:474-593,883-976): a push lands in the target's open accumulator, a
    fold closes it and keeps (w_self x + received) / (w_self + count), or x itself when nothing arrived."""
    world, n = 4, 16
    pw = AsyncWorld(world, n)
    pw.log = []
    monkeypatch.setattr(PK, "fn", pw.fn)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda: types.SimpleNamespace(cuda_stream=0))
    monkeypatch.setattr(torch, "zeros", _registering_zeros(pw, torch.zeros))
    comms, ws = [], []
    for r in range(world):
        c, w = _bare_async(p2p.PushGossipP2PComm, pw, r, world)
        c.rng = XorShift128Plus(41 + 7919 * r, 43)
        c.synchronous = False
        c.attach(types.SimpleNamespace(net=c.net))
        comms.append(c)
        ws.append(w)
    shadows = [XorShift128Plus(41 + 7919 * r, 43) for r in range(world)]
    torch.manual_seed(50)
    x = [torch.randn(n) for _ in range(world)]
    for r in range(world):
        ws[r].copy_(x[r])
    acc = [[torch.zeros(n), torch.zeros(n)] for _ in range(world)]
    cnt = [[0, 0] for _ in range(world)]
    epoch = [0] * world
    schedule = [0, 1, 0, 0, 2, 0, 3, 0, 0, 1, 0, 2, 0, 0, 3, 1, 2, 0]
    empty_folds = 0
    for r in schedule:
        pw.current = r
        comms[r].sync_params(ws[r])
        t = shadows[r].below(world)
        if t != r:
            acc[t][epoch[t] & 1] += x[r]
            cnt[t][epoch[t] & 1] += 1
        closed = epoch[r] & 1
        epoch[r] += 1
        w_self = 2.0 if t == r else 1.0
        if cnt[r][closed]:
            x[r] = (w_self * x[r] + acc[r][closed]) / (w_self + cnt[r][closed])
            acc[r][closed] = torch.zeros(n)
            cnt[r][closed] = 0
        else:
            empty_folds += 1
        assert torch.allclose(ws[r], x[r], atol=1e-6), (r, t)
    assert empty_folds > 0, "the schedule should contain exchanges in which nothing had arrived"
    assert all(name != "rb_barrier_p2p" for _, name in pw.log), "the asynchronous form launches no barrier"


def _registering_zeros(pw, real):
    """torch.zeros that also registers what it makes with the fake world (the backends' local ticket / counter words)."""
    def zeros(*a, **k):
        k.pop("device", None)
        t = real(*a, **k)
        if t.dtype in (torch.int32, torch.int64):
            pw.reg(t)
        return t
    return zeros


def test_asynchronous_elastic_averaging_serves_clients_one_at_a_time(monkeypatch):
    """Clients mix with the centre as it is when they get the lock (src/worker/elasticserver_dist.rs:667-715), in any
    order and any number of times; a client that finds the centre locked gives the exchange up and counts it."""
    world, n, beta = 3, 16, 0.25
    pw = AsyncWorld(world, n)
    pw.log = []
    monkeypatch.setattr(PK, "fn", pw.fn)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda: types.SimpleNamespace(cuda_stream=0))
    monkeypatch.setattr(torch, "zeros", _registering_zeros(pw, torch.zeros))
    comms, ws = [], []
    for r in range(world):
        c, w = _bare_async(p2p.ElasticP2PComm, pw, r, world)
        c.beta, c.synchronous, c.lock_wait_ns = beta, False, 1000
        c.attach(types.SimpleNamespace(net=c.net))
        comms.append(c)
        ws.append(w)
    torch.manual_seed(60)
    centre = torch.randn(n)
    comms[0].center.copy_(centre)
    x = [torch.randn(n) for _ in range(world)]
    for r in range(world):
        ws[r].copy_(x[r])
    for r in [1, 1, 2, 0, 1, 2, 2, 0]:
        pw.current = r
        comms[r].sync_params(ws[r])
        d = beta * (x[r] - centre)
        x[r] = x[r] - d
        centre = centre + d
        assert torch.allclose(ws[r], x[r], atol=1e-6) and torch.allclose(comms[0].center, centre, atol=1e-6)
    assert int(comms[0].lock[0]) == 0 and all(c.skipped_exchanges() == 0 for c in comms)
    # somebody else holds the lock: the exchange is skipped, counted, and changes nothing
    comms[0].lock[0] = 7
    pw.current = 2
    comms[2].sync_params(ws[2])
    assert torch.allclose(ws[2], x[2], atol=0) and torch.allclose(comms[0].center, centre, atol=1e-6)
    assert comms[2].skipped_exchanges() == 1 and int(comms[0].lock[0]) == 7
    assert all(name != "rb_barrier_p2p" for _, name in pw.log)


def test_elastic_averaging_launches_move_clients_and_centre_toward_each_other(monkeypatch):
    world, n, beta = 4, 16, 0.2
    pw = PtrWorld(world, n)
    monkeypatch.setattr(PK, "fn", pw.fn)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda: types.SimpleNamespace(cuda_stream=0))
    comms, ws = [], []
    for r in range(world):
        c, w = _bare(p2p.ElasticP2PComm, pw, r, world)
        c.beta, c.synchronous, c.lock_wait_ns = beta, True, 0
        c.attach(types.SimpleNamespace(net=c.net))
        comms.append(c)
        ws.append(w)
    torch.manual_seed(40)
    centre = torch.randn(n)
    comms[0].center.copy_(centre)
    for rnd in range(3):
        start = [torch.randn(n) for _ in range(world)]
        for r in range(world):
            ws[r].copy_(start[r])
            pw.current = r
            comms[r].sync_params(ws[r])
        pw.run()
        for r in range(world):      # every client mixes with the same centre snapshot
            assert torch.allclose(ws[r], start[r] - beta * (start[r] - centre), atol=1e-6), (rnd, r)
        centre = centre + sum(beta * (start[r] - centre) for r in range(world))
        assert torch.allclose(comms[0].center, centre, atol=1e-5)
        assert float(comms[0].delta.abs().sum()) == 0.0


def test_two_device_branch_engines_with_pair_gossip(monkeypatch):
    """Step locally, then mix parameters with the partner of the shared permutation: two engines on their device
    branch with the kernel backend against two CPU engines mixed by hand."""
    import kernel_emulation
    from test_engine_emulated import _Ctx, _Event, _Stream
    from rembrandt_b200.engine import StepEngine
    from rembrandt_b200.models import zoo
    from rembrandt_b200.models.net import Net
    from rembrandt_b200.optim.sgd import Momentum, SgdOptConfig, StepSizeSchedule, SyncOrder
    world, batch = 2, 4
    kernel_emulation.install(monkeypatch)
    monkeypatch.setattr(torch.cuda, "Stream", lambda *a, **k: _Stream())
    monkeypatch.setattr(torch.cuda, "Event", _Event)
    monkeypatch.setattr(torch.cuda, "stream", lambda s: _Ctx())
    monkeypatch.setattr(torch.cuda, "current_stream", lambda *a: _Stream())
    monkeypatch.setattr(torch.Tensor, "pin_memory", lambda self, *a, **k: self)
    opt = SgdOptConfig(minibatch_size=batch, step_size=StepSizeSchedule.constant(0.01), momentum=Momentum.UPDATE, mu=0.9,
                       sync_order=SyncOrder.STEP_THEN_SYNC_PARAMS, display_iters=0)
    monkeypatch.setattr(Net, "device_path_on_cpu", True)
    dev_nets = [Net(zoo.mnist_fc2(), batch, device="cpu", seed=(5, 6)) for _ in range(world)]
    monkeypatch.setattr(Net, "device_path_on_cpu", False)
    cpu_nets = [Net(zoo.mnist_fc2(), batch, device="cpu", seed=(5, 6)) for _ in range(world)]
    fake = FakeWorld(world, dev_nets[0].flat_len)
    monkeypatch.setattr(PK, "fn", fake.fn)
    comms = []
    for r in range(world):
        fake.w[r] = dev_nets[r].params
        c = _make_flat(r, world, "pair", (17, 29), fake)
        c.net = dev_nets[r]
        c.iter, c.step_size = 0, 0.0
        c.attach = lambda engine: None
        comms.append(c)
        with torch.no_grad():
            dev_nets[r].params.copy_(dev_nets[r].params16.float())
            cpu_nets[r].params.copy_(dev_nets[r].params16.float())
    dev_engs = [StepEngine(dev_nets[r], opt, comms[r], use_graph=False) for r in range(world)]
    cpu_engs = [StepEngine(cpu_nets[r], SgdOptConfig(minibatch_size=batch, step_size=StepSizeSchedule.constant(0.01),
                                                     momentum=Momentum.UPDATE, mu=0.9, display_iters=0))
                for r in range(world)]
    shadow = XorShift128Plus(17, 29)
    g = torch.Generator().manual_seed(9)
    mixed = 0
    for step in range(6):
        for r in range(world):
            x = torch.randint(0, 256, (batch, 1, 28, 28), dtype=torch.uint8, generator=g)
            y = torch.randint(0, 10, (batch,), dtype=torch.int32, generator=g)
            fake.current = r
            dev_engs[r].feed(x, y)
            dev_engs[r].step()
            cpu_engs[r].feed(x, y)
            cpu_engs[r].step()
        fake.run()
        for n in dev_nets:
            n.refresh_shadow()      # what the engine does after the exchange; here the exchange ran late
        perm = shadow.permutation(world)
        with torch.no_grad():
            before = [n.params.detach().clone() for n in cpu_nets]
            for r in range(world):
                src = perm.index(r)
                if src != r:
                    cpu_nets[r].params.copy_(0.5 * before[r] + 0.5 * before[src])
                    mixed += 1
    assert mixed > 0, "the permutations never paired the two ranks"
    for r in range(world):
        want = cpu_nets[r].params.detach()
        rel = float((dev_nets[r].params - want).norm() / want.norm())
        assert rel < 3e-2, (r, rel)
