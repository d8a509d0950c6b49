"""Per-rank bodies of the CPU communication tests (top-level functions so that spawn can pickle them)."""
import time

import torch
import torch.distributed as dist

from rembrandt_b200.parallel import comm as C
from rembrandt_b200.utils.rng import XorShift128Plus


def _vec(rank, n=257, rnd=0):
    g = torch.Generator().manual_seed(100 * rnd + rank)
    return torch.randn(n, generator=g)


def _all(world, n=257, rnd=0):
    return [_vec(r, n, rnd) for r in range(world)]


def allreduce(rank, world):
    c = C.AllreduceComm()
    x = _vec(rank)
    c.allreduce_average(x)
    assert torch.allclose(x, sum(_all(world)) / world, atol=1e-6)
    assert c.allreduce_stats([1.0, float(rank)]) == [float(world), float(sum(range(world)))]
    assert c.broadcast_seed((rank + 5, rank + 9)) == (5, 9)


def pair_gossip(rank, world):
    c = C.PairGossipComm(seed=(17, 29))
    shadow = XorShift128Plus(17, 29)
    for rnd in range(5):
        x = _vec(rank, rnd=rnd)
        c.sync_params(x)
        perm = shadow.permutation(world)
        src = perm.index(rank)                     # the rank that sends to me
        every = _all(world, rnd=rnd)
        expect = every[rank] if src == rank and perm[rank] == rank else 0.5 * (every[rank] + every[src])
        if src == rank:
            expect = every[rank]
        assert torch.allclose(x, expect, atol=1e-6), f"round {rnd}"
    # repeat=True reuses the partners of the previous round (params and grads mixed with the same peer)
    x, y = _vec(rank, rnd=50), _vec(rank, rnd=51)
    c.sync_params(x)
    c.sync_params(y, repeat=True)
    perm = shadow.permutation(world)
    src = perm.index(rank)
    if src != rank:
        assert torch.allclose(y, 0.5 * (_vec(rank, rnd=51) + _vec(src, rnd=51)), atol=1e-6)


def pull_gossip(rank, world, rounds):
    c = C.PullGossipComm(seed=(31, 37), cfg=C.GossipConfig(num_rounds=rounds))
    shadows = [XorShift128Plus(31 + 1000003 * r, 37) for r in range(world)]
    for rnd in range(4):
        x = _vec(rank, rnd=rnd)
        c.sync_params(x)
        every = _all(world, rnd=rnd)
        peers = [[s.below(world) for _ in range(rounds)] for s in shadows][rank]
        expect = (every[rank] + sum(every[p] for p in peers)) / (rounds + 1)
        assert torch.allclose(x, expect, atol=1e-6), f"round {rnd}"


def push_gossip(rank, world):
    c = C.PushGossipComm(seed=(41, 43))
    shadows = [XorShift128Plus(41 + 7919 * r, 43) for r in range(world)]
    for rnd in range(5):
        x = _vec(rank, rnd=rnd)
        c.sync_params(x)
        every = _all(world, rnd=rnd)
        targets = [s.below(world) for s in shadows]
        received = [every[r] for r in range(world) if targets[r] == rank and r != rank]
        w_self = 2.0 if targets[rank] == rank else 1.0
        expect = every[rank] if not received else (w_self * every[rank] + sum(received)) / (w_self + len(received))
        assert torch.allclose(x, expect, atol=1e-6), f"round {rnd}"


def elastic(rank, world):
    beta = 0.8 / world
    c = C.ElasticComm()
    assert abs(c.beta - beta) < 1e-12
    x = _vec(rank)
    c.first_one_way_sync(x)
    center = _vec(0)
    assert torch.allclose(x, center)               # everybody starts from rank 0's parameters
    xs = [center.clone() for _ in range(world)]
    for rnd in range(3):
        noise = [_vec(r, rnd=10 + rnd) * 0.1 for r in range(world)]
        x += noise[rank]
        xs = [a + n for a, n in zip(xs, noise)]
        c.sync_params(x)
        pulls = [beta * (a - center) for a in xs]
        xs = [a - p for a, p in zip(xs, pulls)]
        center = center + sum(pulls)
        assert torch.allclose(x, xs[rank], atol=1e-6)
        if rank == 0:
            assert torch.allclose(c.center, center, atol=1e-6)
    y = torch.zeros_like(x)
    c.exact_sync(y)
    assert torch.allclose(y, center, atol=1e-6)    # exact sync broadcasts the centre


def _wait_for(cond, seconds=20.0):
    t_end = time.time() + seconds
    while not cond():
        assert time.time() < t_end, "condition not reached in time"
        time.sleep(0.002)


def push_gossip_async_one_at_a_time(rank, world):
    """Asynchronous push gossip with one rank exchanging at a time, so that what each exchange folds in is known:
    every rank replays all ranks' draws, pushes and folds and compares its own vector after each of its exchanges."""
    c = C.PushGossipComm(seed=(41, 43), asynchronous=True)
    x = _vec(rank)
    c.first_one_way_sync(x)
    shadows = [XorShift128Plus(41 + 7919 * r, 43) for r in range(world)]
    xs = _all(world)
    inbox = [[] for _ in range(world)]
    folded = [0] * world
    for rnd in range(4 * world):
        a = rnd % world
        target = shadows[a].below(world)
        if target != a:
            inbox[target].append(xs[a].clone())
        if rank == a:
            _wait_for(lambda: c.pending() == len(inbox[a]))     # the earlier pushes to this rank have all arrived
            c.sync_params(x)
        w_self = 2.0 if target == a else 1.0
        if inbox[a]:
            xs[a] = (w_self * xs[a] + sum(inbox[a])) / (w_self + len(inbox[a]))
            folded[a] += len(inbox[a])
            inbox[a] = []
        if rank == a:
            assert torch.allclose(x, xs[a], atol=1e-6), f"exchange {rnd}"
            assert c.folded == folded[a]
        dist.barrier()
    c.close()
    assert c.pending() == len(inbox[rank])                      # close() returns once every push has arrived


def push_gossip_async_nobody_waits(rank, world):
    """Free-running asynchronous push gossip with a rank that sleeps 50 ms before each of its exchanges: the other
    ranks finish their exchanges in a fraction of the sleeper's time, vectors stay convex combinations of the
    initial ones, and after close() every pushed vector is accounted for (folded or still pending)."""
    rounds, nap = 24, 0.05
    c = C.PushGossipComm(seed=(5, 11), asynchronous=True)
    x = torch.full((1031,), float(rank))
    c.first_one_way_sync(x)
    t0 = time.time()
    for _ in range(rounds):
        if rank == 1:
            time.sleep(nap)
        c.sync_params(x)
        assert float(x.min()) >= -1e-5 and float(x.max()) <= world - 1 + 1e-5
    mine = time.time() - t0
    c.close()
    shadows = [XorShift128Plus(5 + 7919 * r, 11) for r in range(world)]
    pushed_here = sum(1 for r in range(world) if r != rank for _ in range(rounds) if shadows[r].below(world) == rank)
    assert c.folded + c.pending() == pushed_here
    if rank != 1:
        assert mine < 0.5 * rounds * nap, f"rank {rank} took {mine:.2f} s: it waited for the sleeping rank"


def elastic_async_replay(rank, world):
    """Asynchronous elastic averaging, free-running: rank 0's log of the order in which clients were served,
    replayed sequentially, reproduces the centre and every client's vector."""
    rounds = 6
    c = C.ElasticComm(asynchronous=True)
    beta = c.beta
    x = _vec(rank)
    c.first_one_way_sync(x)
    for k in range(rounds):
        x += 0.1 * _vec(rank, rnd=20 + k)
        if rank == 2:
            time.sleep(0.01)
        c.sync_params(x)
    c.close()
    finals = [torch.zeros_like(x) for _ in range(world)]
    dist.all_gather(finals, x)
    if rank == 0:
        log = c.request_log
        assert sorted(log) == sorted(list(range(world)) * rounds)
        center = _vec(0)
        xs = [center.clone() for _ in range(world)]
        served = [0] * world
        for client in log:
            xs[client] = xs[client] + 0.1 * _vec(client, rnd=20 + served[client])
            served[client] += 1
            read = center.clone()
            center = center + beta * (xs[client] - read)
            xs[client] = (1 - beta) * xs[client] + beta * read
        assert torch.allclose(c.center, center, atol=1e-5)
        for r in range(world):
            assert torch.allclose(finals[r], xs[r], atol=1e-5), f"client {r}"
    y = torch.zeros_like(x)
    c.exact_sync(y)                                             # still a plain broadcast of the centre
    ref = [torch.zeros_like(y) for _ in range(world)]
    dist.all_gather(ref, y)
    assert all(torch.equal(ref[0], t) for t in ref)


def elastic_async_slow_client(rank, world):
    """A client that sleeps between its exchanges does not slow the others down."""
    rounds, nap = 20, 0.05
    c = C.ElasticComm(asynchronous=True)
    x = _vec(rank)
    c.first_one_way_sync(x)
    t0 = time.time()
    for _ in range(rounds):
        if rank == 1:
            time.sleep(nap)
        c.sync_params(x)
    mine = time.time() - t0
    c.close()
    if rank != 1:
        assert mine < 0.5 * rounds * nap, f"rank {rank} took {mine:.2f} s"


def hierarchical(rank, world):
    c = C.GroupAllreduceGossipComm(group_size=2, seed=(53, 59))
    x = _vec(rank)
    c.sync_params(x)
    every = _all(world)
    g0 = rank // 2 * 2
    members = [r for r in range(g0, min(world, g0 + 2))]
    group_mean = sum(every[r] for r in members) / len(members)
    shadows = [XorShift128Plus(53 + 1000003 * r, 59) for r in range(world)]
    peer = [s.below(world) for s in shadows][rank]
    pg0 = peer // 2 * 2
    pmem = [r for r in range(pg0, min(world, pg0 + 2))]
    peer_mean = sum(every[r] for r in pmem) / len(pmem)
    assert torch.allclose(x, 0.5 * (group_mean + peer_mean), atol=1e-6)


def hierarchical_leaders(rank, world):
    """Version 1: only the first rank of each group of two gossips; its group follows it."""
    c = C.GroupAllreduceGossipComm(group_size=2, seed=(53, 59), version=1)
    every = _all(world)
    means = [sum(every[r] for r in range(g0, min(world, g0 + 2))) / len(range(g0, min(world, g0 + 2)))
             for g0 in range(0, world, 2)]
    shadows = [XorShift128Plus(53 + 1000003 * g, 59) for g in range(len(means))]   # one stream per leader
    x = _vec(rank)
    for rnd in range(3):
        draws = [s.below(len(means)) for s in shadows]
        c.sync_params(x)
        means = [0.5 * (means[g] + means[draws[g]]) for g in range(len(means))]
        assert torch.allclose(x, means[rank // 2], atol=1e-6), (rnd, rank)


def exact_sync(rank, world):
    for cls in (C.PairGossipComm, C.PullGossipComm, C.PushGossipComm):
        x = _vec(rank)
        cls().exact_sync(x)
        assert torch.allclose(x, sum(_all(world)) / world, atol=1e-6)


# ---- failure injection on the host: a rank that raises, never joins, or arrives late
def rank_raises_before_collective(rank, world):
    if rank == 1:
        raise RuntimeError("injected failure on rank 1")
    x = _vec(rank)
    C.AllreduceComm().allreduce_average(x)         # the survivors' collective must end with an error, not hang


def async_rank_leaves_without_closing(rank, world):
    """Asynchronous push gossip: rank 1 raises after a few exchanges and never sends its closing message. The
    others keep exchanging (nobody waits for it), and their close() ends with an error, not a hang."""
    c = C.PushGossipComm(seed=(7, 9), asynchronous=True)
    x = _vec(rank)
    c.first_one_way_sync(x)
    for k in range(6):
        if rank == 1 and k == 3:
            raise RuntimeError("injected failure on rank 1")
        c.sync_params(x)
    c.close()      # survivors: the receive from the dead rank ends with a reset connection or the group's time limit


def rank_never_joins(rank, world):
    if rank == world - 1:
        time.sleep(6)                              # misses the collective; the process-group timeout is shorter
        return
    C.AllreduceComm().allreduce_average(_vec(rank))


def straggler_is_tolerated(rank, world):
    c = C.AllreduceComm()
    for rnd in range(3):
        if rank == 0:
            time.sleep(0.3)                        # delayed, not dead: results are unchanged
        x = _vec(rank, rnd=rnd)
        c.allreduce_average(x)
        assert torch.allclose(x, sum(_all(world, rnd=rnd)) / world, atol=1e-6)


def dp_training_matches_single_process(rank, world):
    """Data-parallel SGD over `world` ranks == one process on the concatenated batch (mean gradient)."""
    from rembrandt_b200.engine import StepEngine
    from rembrandt_b200.models import zoo
    from rembrandt_b200.models.net import Net
    from rembrandt_b200.optim.sgd import Momentum, SgdOptConfig, StepSizeSchedule

    def opt(mb):
        return SgdOptConfig(minibatch_size=mb, step_size=StepSizeSchedule.constant(0.05), momentum=Momentum.UPDATE,
                            mu=0.9, l2_reg_coef=1e-3)
    per = 8
    comm = C.AllreduceComm()
    seed = comm.broadcast_seed((rank + 3, 7))
    net = Net(zoo.lenet(), per, device="cpu", seed=seed, minibatch_size=per)
    eng = StepEngine(net, opt(per), comm)
    g = torch.Generator().manual_seed(5)
    steps = [(torch.randint(0, 256, (per * world, 1, 28, 28), dtype=torch.uint8, generator=g),
              torch.randint(0, 10, (per * world,), dtype=torch.int32, generator=g)) for _ in range(3)]
    for x, y in steps:
        eng.feed(x[rank * per:(rank + 1) * per], y[rank * per:(rank + 1) * per])
        eng.step()
    if rank == 0:
        big = Net(zoo.lenet(), per * world, device="cpu", seed=seed, minibatch_size=per * world)
        beng = StepEngine(big, opt(per * world))
        for x, y in steps:
            beng.feed(x, y)
            beng.step()
        assert torch.allclose(net.params.detach(), big.params.detach(), atol=2e-6)
    ref = net.params.detach().clone()
    dist.broadcast(ref, 0)
    assert torch.equal(ref, net.params.detach()), "replicas diverged"


def rules_times_orders(rank, world):
    """Every momentum rule under every synchronisation order (6 x 4 pairs), two ranks each."""
    from rembrandt_b200.optim.sgd import Momentum, SyncOrder
    failures = []
    for mode in Momentum:
        for order in SyncOrder:
            try:
                _rule_and_order(rank, world, int(mode), order.value)
            except AssertionError as e:
                failures.append(str(e))
    # exchanges every second iteration, and two batches per iteration (gradient accumulation), under every order
    for order in SyncOrder:
        for interval, accum in ((2, 1), (1, 2), (3, 2)):
            try:
                _rule_and_order(rank, world, int(Momentum.UPDATE_NESTEROV), order.value, interval, accum)
            except AssertionError as e:
                failures.append(str(e))
    assert not failures, "\n".join(failures)


def _rule_and_order(rank, world, mode_value, order_value, interval=1, accum=1):
    """Two data-parallel ranks under one (momentum rule, synchronisation order) pair against a NumPy restatement of
    that pair which simulates both ranks in one process (gradients from single-process networks, the update rules and
    the averaging written out with NumPy)."""
    import numpy as np

    from rembrandt_b200.engine import StepEngine
    from rembrandt_b200.models import zoo
    from rembrandt_b200.models.net import Net
    from rembrandt_b200.optim.sgd import Momentum, SgdOptConfig, StepSizeSchedule, SyncOrder

    mode, order = Momentum(mode_value), SyncOrder(order_value)
    lr, mu, l2, per, steps = 0.05, 0.9, 1e-3, 8, 4 * accum
    mu_eff = 0.0 if mode == Momentum.ZERO else mu
    mb = per * accum

    def batch(r, s):
        g = torch.Generator().manual_seed(1000 * s + r)
        return (torch.randint(0, 256, (per, 1, 28, 28), dtype=torch.uint8, generator=g),
                torch.randint(0, 10, (per,), dtype=torch.int32, generator=g))

    opt = SgdOptConfig(minibatch_size=mb, step_size=StepSizeSchedule.constant(lr), momentum=mode, mu=mu,
                       l2_reg_coef=l2, sync_order=order, comm_interval=interval)
    net = Net(zoo.mnist_fc2(), per, device="cpu", seed=(3, 7), minibatch_size=mb)
    eng = StepEngine(net, opt, C.AllreduceComm())
    for s in range(steps):
        eng.feed(*batch(rank, s))
        eng.step()

    # ---- the restatement: both ranks, NumPy state
    sims = [Net(zoo.mnist_fc2(), per, device="cpu", seed=(3, 7), minibatch_size=mb) for _ in range(world)]
    d = sims[0].decay_len
    w = [n.params.detach().numpy().astype(np.float64).copy() for n in sims]
    v = [np.zeros_like(w[0]) for _ in sims]
    g = [np.zeros_like(w[0]) for _ in sims]
    lam = np.zeros_like(w[0])
    lam[:d] = l2
    m = int(mode)

    def accumulate(r):
        gp = g[r] + lam * w[r]
        if m in (0, 1):
            v[r] = mu_eff * v[r] - lr * gp
        elif m == 2:
            w[r] = w[r] - mu_eff * v[r]
            v[r] = mu_eff * v[r] - lr * (g[r] + lam * (w[r] + mu_eff * v[r]))   # regulariser sees the stored parameters
        elif m in (3, 4):
            v[r] = mu_eff * v[r] + gp

    def apply(r):
        gp = g[r] + lam * w[r]
        if m in (0, 1):
            w[r] = w[r] + v[r]
        elif m == 2:
            w[r] = w[r] + v[r] + mu_eff * v[r]
        elif m == 3:
            w[r] = w[r] - lr * v[r]
        elif m == 4:
            w[r] = w[r] - lr * gp - lr * mu_eff * v[r]
        elif m == 5:
            w[r] = w[r] - lr * gp
        g[r] = mu_eff * gp if m == 5 else np.zeros_like(gp)

    def mean(xs):
        avg = sum(xs) / len(xs)
        return [avg.copy() for _ in xs]

    for s in range(steps):
        for r, n in enumerate(sims):
            with torch.no_grad():
                n.params.copy_(torch.from_numpy(w[r]).float())
                n.grads.zero_()
            n.load_batch(*batch(r, s))
            n.forward(True)
            n.backward()
            n.read_stats()
            g[r] = g[r] + n.grads.detach().numpy().astype(np.float64)
        if (s + 1) % accum:
            continue                                   # inside a gradient-accumulation group
        it = (s + 1) // accum                          # the iteration is counted before the interval is tested
        if it % interval:
            mean_now = lambda xs: xs                   # no exchange in this iteration
        else:
            mean_now = mean
        if order == SyncOrder.SYNC_GRADS_THEN_STEP:
            g = mean_now(g)
            for r in range(world):
                accumulate(r)
                apply(r)
        elif order == SyncOrder.STEP_THEN_SYNC_PARAMS:
            for r in range(world):
                accumulate(r)
                apply(r)
            w = mean_now(w)
        elif order == SyncOrder.SYNC_PARAMS_THEN_STEP:
            for r in range(world):
                accumulate(r)
            w = mean_now(w)
            for r in range(world):
                apply(r)
        else:
            w = mean_now(w)
            g = mean_now(g)
            for r in range(world):
                accumulate(r)
                apply(r)
    got = net.params.detach().numpy().astype(np.float64)
    err = np.abs(got - w[rank]).max()
    assert err < 5e-5, (f"{mode.name} x {order.name} (interval {interval}, {accum} batches per iteration): rank {rank} "
                        f"differs from the restatement by {err:.3g}")


def barrier_free_loop_with_async_exchanges(rank, world, directory, backend):
    """The barrier-free optimizer loop over an asynchronous library exchange: ranks run different numbers of
    iterations per second (rank 1 naps), nobody waits, every rank checkpoints into its own directory, and the
    replicas end closer to each other than independent runs would."""
    import os

    from rembrandt_b200.data import BatchIter, RandomSampleDataIter, SyntheticDataSource, partition_shard
    from rembrandt_b200.engine import StepEngine
    from rembrandt_b200.models import zoo
    from rembrandt_b200.models.net import Net
    from rembrandt_b200.optim.async_sgd import AsyncSgdOpt
    from rembrandt_b200.optim.sgd import Momentum, SgdOptConfig, StepSizeSchedule, SyncOrder

    src = SyntheticDataSource(256, (28, 28, 1), 10, seed=1, separable=True)
    comm = C.make_comm(backend)
    assert comm.asynchronous and not comm.synchronous
    order = SyncOrder.STEP_THEN_SYNC_PARAMS if "gossip" in backend else SyncOrder.SYNC_PARAMS_THEN_STEP
    opt = SgdOptConfig(minibatch_size=16, step_size=StepSizeSchedule.constant(0.05), momentum=Momentum.UPDATE, mu=0.9,
                       l2_reg_coef=1e-4, sync_order=order, display_iters=4, checkpoint_iters=6, save_iters=6,
                       valid_iters=0, checkpoint_dir=directory)
    net = Net(zoo.mnist_fc1(), 16, device="cpu", seed=(3, 4), minibatch_size=16)
    sgd = AsyncSgdOpt(opt, StepEngine(net, opt, comm), quiet=True)
    train = BatchIter(RandomSampleDataIter(partition_shard(src, rank, world), seed=(9 + rank, 9)), 16, src.dims)

    def forever():
        while True:
            for b in train:
                if rank == 1:
                    time.sleep(0.02)
                yield b
    t0 = time.time()
    sgd.train(forever(), None, max_iters=12)
    mine = time.time() - t0
    sgd.trace.close()
    comm.close()
    assert os.path.exists(os.path.join(directory, f"rank{rank}", "params.t_12.blob"))
    times = [torch.zeros(1, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(times, torch.tensor([mine], dtype=torch.float64))
    if rank == 0:
        assert float(times[1]) >= 12 * 0.02
    finals = [torch.empty_like(net.params.detach()) for _ in range(world)]
    dist.all_gather(finals, net.params.detach().clone())
    assert all(torch.isfinite(f).all() for f in finals)


def gossip_training_loop(rank, world, directory):
    """The whole training loop on several ranks with pair gossip: checkpoint windows (exact averaging, rank-0
    parameter blob, per-rank state), validation statistics summed over ranks, both checkpoint behaviours, resume."""
    import os

    from rembrandt_b200.data import BatchIter, CyclicSampleDataIter, RandomSampleDataIter, SyntheticDataSource, partition_shard
    from rembrandt_b200.engine import StepEngine
    from rembrandt_b200.models import zoo
    from rembrandt_b200.models.net import Net
    from rembrandt_b200.optim.sgd import CheckpointBehavior, Momentum, SgdOptConfig, StepSizeSchedule, SyncOrder
    from rembrandt_b200.trainer import SgdOpt

    src = SyntheticDataSource(384, (28, 28, 1), 10, seed=1, separable=True)
    valid_src = SyntheticDataSource(96, (28, 28, 1), 10, seed=2, separable=True)

    def run(behavior, sub, iters, resume=False):
        d = os.path.join(directory, sub)
        comm = C.PairGossipComm(seed=(17, 29))
        seed = comm.broadcast_seed((rank + 40, 5))
        opt = SgdOptConfig(minibatch_size=16, step_size=StepSizeSchedule.constant(0.05), momentum=Momentum.UPDATE,
                           mu=0.9, l2_reg_coef=1e-4, sync_order=SyncOrder.STEP_THEN_SYNC_PARAMS, checkpoint=behavior,
                           display_iters=4, checkpoint_iters=4, save_iters=4, valid_iters=2, checkpoint_dir=d)
        net = Net(zoo.mnist_fc1(), 16, device="cpu", seed=seed, minibatch_size=16)
        sgd = SgdOpt(opt, StepEngine(net, opt, comm), quiet=True)
        train = BatchIter(RandomSampleDataIter(partition_shard(src, rank, world), seed=(9 + rank, 9)), 16, src.dims)
        valid = BatchIter(CyclicSampleDataIter(partition_shard(valid_src, rank, world)), 16, valid_src.dims)

        def forever():
            while True:
                for b in train:
                    yield b
        sgd.train(forever(), valid, max_iters=iters)
        sgd.trace.close()
        return sgd, net, d

    def gathered(t):
        out = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(out, t)
        return out

    # KEEP: after the checkpoint window at the last iteration every rank holds the exact average, which is the blob
    sgd, net, d = run(CheckpointBehavior.KEEP, "keep", 8)
    everyone = gathered(net.params.detach())
    assert all(torch.equal(everyone[0], e) for e in everyone[1:]), "KEEP: replicas must equal the averaged model"
    dist.barrier()
    assert net.encode_params() == open(os.path.join(d, "params.t_8.blob"), "rb").read()
    assert open(os.path.join(d, "checkpoint")).read() == "8\n"
    assert all(os.path.exists(os.path.join(d, f"state.latest.blob.{r}")) for r in range(world))
    # validation statistics are summed over ranks: every rank reports the same numbers, over all shards
    vh = torch.tensor([list(v) for v in sgd.valid_history], dtype=torch.float64)
    assert vh.shape == (2, 3) and all(torch.equal(vh, o) for o in gathered(vh))
    # the progress line statistics agree too
    hist = torch.tensor([list(h) for h in sgd.history], dtype=torch.float64)
    assert all(torch.equal(hist, o) for o in gathered(hist))

    # DISCARD: the averaged model is written and validated, but every rank continues from its own parameters
    sgd2, net2, d2 = run(CheckpointBehavior.DISCARD, "discard", 8)
    mine = gathered(net2.params.detach())
    assert not torch.equal(mine[0], mine[1]), "DISCARD: replicas keep their own parameters"
    mean = sum(mine) / world
    blob_net = Net(zoo.mnist_fc1(), 16, device="cpu", seed=(1, 1), minibatch_size=16)
    blob_net.decode_params(open(os.path.join(d2, "params.t_8.blob"), "rb").read())
    assert torch.allclose(blob_net.params.detach(), mean, atol=1e-6), "the blob is the exact mean of the replicas"

    # resume: a second run in the same directory starts at iteration 8 from this rank's own state
    sgd3, net3, _ = run(CheckpointBehavior.DISCARD, "discard", 12, resume=True)
    assert sgd3.engine.iter == 12
    steps = [r for r in open(os.path.join(d2, f"trace_sgd.{rank}.log.1")).read().splitlines() if ",step," in r]
    assert [int(r.split(",")[0]) for r in steps] == [9, 10, 11, 12]
