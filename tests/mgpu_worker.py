"""Multi-GPU test worker, launched by tests/test_multigpu.py through torch.distributed.run (one rank per GPU).

Each case checks a kernel-driven communication backend against the same exchange done with library
collectives (NCCL) or a closed-form expectation, and exits non-zero on a mismatch.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rembrandt_b200.api import default_opt, model_config
from rembrandt_b200.engine import StepEngine
from rembrandt_b200.models.net import Net
from rembrandt_b200.ops import native_ops as K
from rembrandt_b200.parallel import comm as comm_mod
from rembrandt_b200.parallel import p2p


def batches(rank, steps, batch, hw, ch, classes):
    g = torch.Generator().manual_seed(100 + rank)
    return [(torch.randint(0, 256, (batch, ch, hw, hw), dtype=torch.uint8, generator=g).pin_memory(),
             torch.randint(0, classes, (batch,), dtype=torch.int32, generator=g).pin_memory()) for _ in range(steps)]


def case_fused_allreduce_sgd(rank, world, use_graph):
    """Fused P2P all-reduce + SGD (overlapped with backward) == NCCL all-reduce + separate optimizer step."""
    batch, steps = 8, 5
    cfg = lambda: model_config("cifar", augment=False)
    fused = p2p.FusedAllreduceSgdComm(min_bucket_bytes=64 << 10, bucket_bytes=128 << 10, one_shot_bytes=16 << 10)
    net_a = Net(cfg(), batch, device="cuda", seed=(11, 12), flat_allocator=fused.flat_allocator)
    eng_a = StepEngine(net_a, default_opt(batch, fused.name), fused, use_graph=use_graph)
    base = comm_mod.AllreduceComm()
    net_b = Net(cfg(), batch, device="cuda", seed=(11, 12))
    eng_b = StepEngine(net_b, default_opt(batch, base.name), base, use_graph=False)
    assert torch.equal(net_a.params, net_b.params)
    assert len(fused.launches) >= 3, fused.launches
    data = batches(rank, steps, batch, 32, 3, 10)
    for x, y in data:
        for eng in (eng_a, eng_b):
            eng.feed(x, y)
            eng.step()
    la, lb = eng_a.flush(), eng_b.flush()
    torch.cuda.synchronize()
    assert K.read_status() == 0, "a bounded wait ran out"
    assert abs(la[0] - lb[0]) < 2e-2 * max(1.0, abs(lb[0])), (la, lb)
    a16, b16 = net_a.params16.float(), net_b.params16.float()
    rel = float((a16 - b16).norm() / b16.norm())
    assert rel < 2e-3, f"bf16 weights differ: rel {rel}"
    # sharded master: after gathering, the fp32 master equals the baseline's
    fused.gather_master()
    rel = float((net_a.params - net_b.params).norm() / net_b.params.norm())
    assert rel < 1e-3, f"fp32 master differs after gather: rel {rel}"  # split-K atomics reorder fp32 sums
    assert float(net_a.grads.abs().max()) == 0.0
    # every rank holds the same weights
    mine = net_a.params16.float().clone()
    ref = mine.clone()
    dist.broadcast(ref, 0)
    assert torch.equal(mine, ref), "replicas diverged"


def case_p2p_allreduce(rank, world):
    """The plain in-place average (op 1) of the gradient buffer against NCCL, two-shot and multi-bucket."""
    fused = p2p.FusedAllreduceSgdComm(bucket_bytes=1 << 20)
    net = Net(model_config("lenet"), 4, device="cuda", seed=(1, 2), flat_allocator=fused.flat_allocator)
    StepEngine(net, default_opt(4, fused.name), fused, use_graph=False)
    torch.manual_seed(rank)
    net.grads.copy_(torch.randn_like(net.grads))
    ref = net.grads.clone()
    dist.all_reduce(ref)
    ref /= world
    fused.allreduce_average(net.grads)
    torch.cuda.synchronize()
    assert K.read_status() == 0
    n = net.grads.numel() // 8 * 8
    assert torch.allclose(net.grads[:n], ref[:n], rtol=1e-5, atol=1e-6)


def _param_engine(comm):
    net = Net(model_config("lenet"), 4, device="cuda", seed=(1, 2))
    eng = StepEngine(net, default_opt(4, comm.name), comm, use_graph=False)
    return net, eng


def case_gossip_pair(rank, world):
    comm = p2p.GossipP2PComm(mode="pair", alpha=0.5, seed=(17, 29))
    oracle = comm_mod.PairGossipComm(seed=(17, 29))
    net, _ = _param_engine(comm)
    for rnd in range(4):
        torch.manual_seed(1000 * rnd + rank)
        net.params.copy_(torch.randn_like(net.params))
        expect = net.params.clone()
        oracle.sync_params(expect)
        comm.sync_params(net.params)
        torch.cuda.synchronize()
        assert K.read_status() == 0
        n = net.params.numel() // 4 * 4
        assert torch.allclose(net.params[:n], expect[:n], rtol=1e-6, atol=1e-6), f"round {rnd}"
        assert torch.equal(net.params16[:n], net.params[:n].bfloat16())


def case_pull_rounds(rank, world):
    """Pull gossip with three pulls per exchange: the result is the mean of the own vector and the published
    snapshots of the drawn ranks (a self-draw contributes the own snapshot)."""
    comm = p2p.GossipP2PComm(mode="pull", seed=(31, 37), cfg=comm_mod.GossipConfig(num_rounds=3), synchronous=True)
    net, _ = _param_engine(comm)
    for rnd in range(3):
        torch.manual_seed(2000 * rnd + rank)
        net.params.copy_(torch.randn_like(net.params))
        everyone = [torch.empty_like(net.params) for _ in range(world)]
        dist.all_gather(everyone, net.params)
        comm.sync_params(net.params)
        torch.cuda.synchronize()
        assert K.read_status() == 0
        peers = comm._last_peer
        assert len(peers) == 3
        expect = (everyone[rank] + sum(everyone[p] for p in peers)) / 4.0
        n = net.params.numel() // 4 * 4
        assert torch.allclose(net.params[:n], expect[:n], rtol=1e-5, atol=1e-5), f"round {rnd}"
        assert torch.equal(net.params16[:n], net.params[:n].bfloat16())
        dist.barrier()


def case_group_gossip(rank, world, group_size):
    """Group mean + one pull on the gossip kernels: every rank ends with 0.5 * (own group mean + group mean of the
    rank it drew), the scheme of the library backend (GroupAllreduceGossipComm)."""
    comm = p2p.GroupGossipP2PComm(group_size=group_size, seed=(53, 59))
    net, _ = _param_engine(comm)
    for rnd in range(4):
        torch.manual_seed(3000 * rnd + rank)
        net.params.copy_(torch.randn_like(net.params))
        everyone = [torch.empty_like(net.params) for _ in range(world)]
        dist.all_gather(everyone, net.params)
        comm.sync_params(net.params)
        torch.cuda.synchronize()
        assert K.read_status() == 0

        def group_mean(r):
            g0 = r // group_size * group_size
            members = range(g0, min(world, g0 + group_size))
            return sum(everyone[m] for m in members) / len(members)

        expect = 0.5 * (group_mean(rank) + group_mean(comm._last_peer[0]))
        n = net.params.numel() // 4 * 4
        assert torch.allclose(net.params[:n], expect[:n], rtol=1e-5, atol=1e-5), f"round {rnd}"
        assert torch.equal(net.params16[:n], net.params[:n].bfloat16())
        dist.barrier()


def case_group_gossip_v1(rank, world, group_size):
    """Leader gossip on the kernels: every rank of a group ends with its leader's result, which is the group mean or,
    when the leader drew another group, the mean of the two group means."""
    comm = p2p.GroupGossipP2PComm(group_size=group_size, seed=(53, 59), version=1)
    net, _ = _param_engine(comm)
    for rnd in range(4):
        torch.manual_seed(4000 * rnd + rank)
        net.params.copy_(torch.randn_like(net.params))
        net.refresh_shadow()       # a leader that draws itself mixes nothing and leaves the compute copy as it is
        everyone = [torch.empty_like(net.params) for _ in range(world)]
        dist.all_gather(everyone, net.params)
        comm.sync_params(net.params)
        torch.cuda.synchronize()
        assert K.read_status() == 0
        draws = [torch.zeros(1, dtype=torch.int64, device="cuda") for _ in range(world)]
        dist.all_gather(draws, torch.tensor([comm._last_peer[0]], device="cuda"))
        drawn = draws[comm.leader]                  # what this rank's leader drew

        def group_mean(r):
            g0 = r // group_size * group_size
            members = range(g0, min(world, g0 + group_size))
            return sum(everyone[m] for m in members) / len(members)

        d = int(drawn)
        expect = group_mean(rank) if d == comm.leader else 0.5 * (group_mean(rank) + group_mean(d))
        n = net.params.numel() // 4 * 4
        assert torch.allclose(net.params[:n], expect[:n], rtol=1e-5, atol=1e-5), f"round {rnd}"
        assert torch.equal(net.params16[:n], net.params[:n].bfloat16())
        dist.barrier()


def case_elastic(rank, world):
    comm = p2p.ElasticP2PComm(beta=0.25, synchronous=True)
    oracle = comm_mod.ElasticComm(beta=0.25)
    net, _ = _param_engine(comm)
    torch.manual_seed(7)
    start = torch.randn_like(net.params)
    net.params.copy_(start)
    expect = start.clone()
    comm.first_one_way_sync(net.params)
    oracle.first_one_way_sync(expect)
    for rnd in range(3):
        torch.manual_seed(50 * rnd + rank)
        noise = torch.randn_like(net.params) * 0.1
        net.params.add_(noise)
        expect.add_(noise)
        comm.sync_params(net.params)
        oracle.sync_params(expect)
        torch.cuda.synchronize()
        assert K.read_status() == 0
        n = net.params.numel() // 4 * 4
        assert torch.allclose(net.params[:n], expect[:n], rtol=1e-5, atol=1e-5), f"round {rnd}"
    if rank == 0:
        n = net.params.numel() // 4 * 4
        assert torch.allclose(comm.center[:n], oracle.center[:n], rtol=1e-5, atol=1e-5)


def case_push(rank, world):
    comm = p2p.PushGossipP2PComm(seed=(41, 43), synchronous=True)
    oracle = comm_mod.PushGossipComm(seed=(41, 43))
    net, _ = _param_engine(comm)
    for rnd in range(4):
        torch.manual_seed(300 * rnd + rank)
        net.params.copy_(torch.randn_like(net.params))
        expect = net.params.clone()
        oracle.sync_params(expect)
        comm.sync_params(net.params)
        torch.cuda.synchronize()
        assert K.read_status() == 0
        n = net.params.numel() // 4 * 4
        assert torch.allclose(net.params[:n], expect[:n], rtol=1e-5, atol=1e-5), f"round {rnd}"


def _turns(world, rounds):
    """A schedule in which rank 0 exchanges three times as often as the others: a list of ranks, one per turn."""
    turns = []
    for _ in range(rounds):
        for r in range(world):
            turns += [0, r] if r else [0]
    return turns


def case_push_async(rank, world):
    """Asynchronous push gossip with the ranks any number of exchanges apart: ranks take turns (the others are idle on
    the host), nobody waits for anybody inside an exchange, and the result equals the sequential restatement of the
    accumulate / count / fold rules. A turn must also be fast: an exchange that waited for a peer would sit in a wait
    until its limit."""
    import time
    from rembrandt_b200.utils.rng import XorShift128Plus
    comm = p2p.PushGossipP2PComm(seed=(41, 43))
    assert not comm.synchronous
    comm.wait_ns = 20_000_000_000      # a wait on a peer, if there were one, would take 20 s
    net, _ = _param_engine(comm)
    torch.manual_seed(900 + rank)
    net.params.copy_(torch.randn_like(net.params))
    net.refresh_shadow()           # an exchange in which nothing arrived leaves the compute copy as it is
    everyone = [torch.empty_like(net.params) for _ in range(world)]
    dist.all_gather(everyone, net.params)
    n = net.params.numel() // 4 * 4
    x = [e[:n].clone() for e in everyone]
    acc = [[torch.zeros_like(x[0]), torch.zeros_like(x[0])] for _ in range(world)]
    cnt = [[0, 0] for _ in range(world)]
    epoch = [0] * world
    shadows = [XorShift128Plus(41 + 7919 * r, 43) for r in range(world)]
    empty = 0
    for turn, r in enumerate(_turns(world, 4)):
        if rank == r:
            t0 = time.time()
            comm.sync_params(net.params)
            torch.cuda.synchronize()
            assert time.time() - t0 < 5.0, "an asynchronous exchange must not wait for a peer"
        t = shadows[r].below(world)
        if t != r:
            acc[t][epoch[t] & 1] += x[r]
            cnt[t][epoch[t] & 1] += 1
        closed = epoch[r] & 1
        epoch[r] += 1
        w_self = 2.0 if t == r else 1.0
        if cnt[r][closed]:
            x[r] = (w_self * x[r] + acc[r][closed]) / (w_self + cnt[r][closed])
            acc[r][closed].zero_()
            cnt[r][closed] = 0
        else:
            empty += 1
        dist.barrier()          # host-side turn taking only: the exchange itself contains no barrier
        assert K.read_status() == 0
        assert torch.allclose(net.params[:n], x[rank], rtol=1e-5, atol=1e-5), f"turn {turn} (rank {r})"
    assert torch.equal(net.params16[:n], net.params[:n].bfloat16())


def case_elastic_async(rank, world):
    """Asynchronous elastic averaging: clients take the centre's lock one at a time, in any order and any number of
    times, and each mixes with the centre as it is then; the lock is free afterwards and nothing was skipped."""
    comm = p2p.ElasticP2PComm(beta=0.25)
    assert not comm.synchronous
    net, _ = _param_engine(comm)
    torch.manual_seed(7)
    net.params.copy_(torch.randn_like(net.params))
    comm.first_one_way_sync(net.params)
    n = net.params.numel() // 4 * 4
    centre = net.params[:n].clone()
    torch.manual_seed(70 + rank)
    net.params.add_(torch.randn_like(net.params) * 0.1)
    everyone = [torch.empty_like(net.params) for _ in range(world)]
    dist.all_gather(everyone, net.params)
    x = [e[:n].clone() for e in everyone]
    for turn, r in enumerate(_turns(world, 3)):
        if rank == r:
            comm.sync_params(net.params)
            torch.cuda.synchronize()
        d = 0.25 * (x[r] - centre)
        x[r] = x[r] - d
        centre = centre + d
        dist.barrier()
        assert K.read_status() == 0
        assert torch.allclose(net.params[:n], x[rank], rtol=1e-5, atol=1e-5), f"turn {turn} (rank {r})"
    if rank == 0:
        assert torch.allclose(comm.center[:n], centre, rtol=1e-5, atol=1e-5)
        assert int(comm.lock[0]) == 0
    assert comm.skipped_exchanges() == 0
    # all clients at once: the lock serialises them; every exchange either ran alone or was given up and counted
    before = net.params[:n].clone()
    comm.sync_params(net.params)
    torch.cuda.synchronize()
    dist.barrier()
    assert K.read_status() == 0
    moved = not torch.equal(before, net.params[:n])
    assert moved or comm.skipped_exchanges() == 1
    if rank == 0:
        assert int(comm.lock[0]) == 0


def main():
    case = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    try:
        if case == "fused_eager":
            case_fused_allreduce_sgd(rank, world, False)
        elif case == "fused_graph":
            case_fused_allreduce_sgd(rank, world, True)
        elif case == "p2p_allreduce":
            case_p2p_allreduce(rank, world)
        elif case == "gossip_pair":
            case_gossip_pair(rank, world)
        elif case == "pull_rounds":
            case_pull_rounds(rank, world)
        elif case.startswith("group_gossip_v1"):
            case_group_gossip_v1(rank, world, int(case.rsplit("_", 1)[1]))
        elif case.startswith("group_gossip"):
            case_group_gossip(rank, world, int(case.rsplit("_", 1)[1]))
        elif case == "elastic":
            case_elastic(rank, world)
        elif case == "push":
            case_push(rank, world)
        elif case == "push_async":
            case_push_async(rank, world)
        elif case == "elastic_async":
            case_elastic_async(rank, world)
        else:
            raise SystemExit(f"unknown case {case}")
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            print(f"case {case}: ok on {world} ranks")
    except BaseException:
        # leave at once: the other ranks may be inside a collective that this rank will never join, and the launcher
        # ends them as soon as one worker has failed
        import traceback
        traceback.print_exc()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(1)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
