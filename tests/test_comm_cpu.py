"""Every communication algorithm on CPU ranks (gloo, child processes), checked against closed-form
expectations, plus host-side failure injection: a rank that raises, a rank that never joins, a straggler."""
import pytest

import comm_cases as cases
from cpu_ranks import run_ranks


@pytest.mark.parametrize("world", [2, 3])
def test_allreduce_average_and_host_collectives(world):
    run_ranks(world, cases.allreduce)


@pytest.mark.parametrize("world", [2, 4])
def test_pair_gossip_follows_the_shared_seed_permutation(world):
    run_ranks(world, cases.pair_gossip)


@pytest.mark.parametrize("rounds", [1, 2])
def test_pull_gossip_averages_with_random_peers(rounds):
    run_ranks(3, cases.pull_gossip, rounds)


def test_push_gossip_count_normalised_mean():
    run_ranks(4, cases.push_gossip)


def test_elastic_averaging_against_rank0_centre():
    run_ranks(3, cases.elastic)


def test_async_push_gossip_folds_exactly_what_arrived():
    run_ranks(3, cases.push_gossip_async_one_at_a_time)


def test_async_push_gossip_does_not_wait_for_a_slow_rank():
    run_ranks(4, cases.push_gossip_async_nobody_waits)


def test_async_elastic_matches_a_replay_of_the_serving_order():
    run_ranks(3, cases.elastic_async_replay)


def test_async_elastic_does_not_wait_for_a_slow_client():
    run_ranks(3, cases.elastic_async_slow_client)


@pytest.mark.parametrize("backend", ["gossip_push_async", "elastic_async"])
def test_barrier_free_loop_over_asynchronous_library_exchanges(tmp_path, backend):
    run_ranks(3, cases.barrier_free_loop_with_async_exchanges, str(tmp_path), backend, timeout_s=180)


def test_group_allreduce_then_gossip():
    run_ranks(4, cases.hierarchical)


@pytest.mark.parametrize("world", [4, 5])
def test_group_leaders_gossip_and_broadcast(world):
    run_ranks(world, cases.hierarchical_leaders)


def test_exact_sync_is_a_true_mean_for_gossip_backends():
    run_ranks(3, cases.exact_sync)


def test_a_rank_that_raises_ends_the_others_with_an_error_not_a_hang():
    codes, msgs = run_ranks(3, cases.rank_raises_before_collective, timeout_s=8, expect_failure=True)
    assert all(c is not None for c in codes), "a rank hung"
    assert codes[1] != 0 and any("injected failure" in m for _, m in msgs)
    assert all(c != 0 for c in codes), "survivors must see the failure (connection reset or timeout)"


def test_async_exchange_survivors_see_a_rank_that_left_without_closing():
    codes, msgs = run_ranks(3, cases.async_rank_leaves_without_closing, timeout_s=8, expect_failure=True)
    assert all(c is not None for c in codes), "a rank hung"
    assert codes[1] != 0 and any("injected failure" in m for _, m in msgs)
    assert all(c != 0 for c in codes), "survivors must see the failure when they close"


def test_a_rank_that_never_joins_times_the_collective_out():
    codes, msgs = run_ranks(3, cases.rank_never_joins, timeout_s=3, expect_failure=True)
    assert all(c is not None for c in codes), "a rank hung"
    assert codes[0] != 0 and codes[1] != 0


def test_a_straggler_only_delays():
    run_ranks(3, cases.straggler_is_tolerated)


def test_data_parallel_training_equals_single_process_on_the_global_batch():
    run_ranks(2, cases.dp_training_matches_single_process, timeout_s=120)


def test_every_momentum_rule_under_every_sync_order_matches_a_numpy_restatement():
    run_ranks(2, cases.rules_times_orders, timeout_s=240)


def test_gossip_training_loop_checkpoints_validates_and_resumes_on_three_ranks(tmp_path):
    run_ranks(3, cases.gossip_training_loop, str(tmp_path), timeout_s=240)


def test_plan_buckets_covers_every_parameter_once_in_backward_order():
    """Bucket plan of the overlapped exchanges: ranges follow the order backward completes them, cover every
    parameter segment exactly once and respect the size bounds."""
    from rembrandt_b200.models import zoo
    from rembrandt_b200.models.net import Net
    from rembrandt_b200.parallel.comm import plan_buckets
    net = Net(zoo.cifar_krizh26(), 4, device="cpu")
    plan = plan_buckets(net, bucket_elems=16 * 1024, min_bucket_elems=4 * 1024)
    covered = []
    last_trigger = len(net.ops)
    for idx, off, n in plan:
        assert 0 < n <= 16 * 1024
        assert idx <= last_trigger, "triggers must not move towards the loss"
        last_trigger = idx
        covered.append((off, off + n))
    covered.sort()
    for (a0, a1), (b0, b1) in zip(covered, covered[1:]):
        assert a1 <= b0, "ranges overlap"
    for s in net.segs:
        assert any(lo <= s.offset and s.offset + s.numel <= hi for lo, hi in _merged(covered)), s.name
    # every range becomes available only after the operator that owns its last-written segment has run backward
    for idx, off, n in plan:
        owners = [i for i, op in enumerate(net.ops) for s in op.segs if s.offset < off + n and off < s.offset + s.numel]
        assert min(owners) >= idx


def _merged(ranges):
    out = []
    for lo, hi in ranges:
        if out and out[-1][1] == lo:
            out[-1] = (out[-1][0], hi)
        else:
            out.append((lo, hi))
    return out


def test_exchange_staging_regions_do_not_overlap():
    """Staging layout of the push-based exchange: every bucket gets `world` slots of the length a rank reduces, and
    no two regions overlap (checked on the planning code alone, with a stand-in for the symmetric-memory arena)."""
    import types
    from rembrandt_b200.parallel import p2p

    class _Arena:
        def __init__(self):
            self.allocs = {}

        def alloc(self, name, n, dtype):
            self.allocs[name] = n
            return None

    comm = types.SimpleNamespace(world=8, one_shot_elems=64 * 1024, bucket_elems=6 * 1024 * 1024, num_slots=256,
                                 mc_grads=0, arena=_Arena())
    comm._shard_len = types.MethodType(p2p.FusedAllreduceSgdComm._shard_len, comm)
    sizes = [1000 * 64, 6 * 1024 * 1024, 4096, 123 * 64, 6 * 1024 * 1024, 64]
    comm.launches, off = [], 0
    for slot, n in enumerate(sizes):
        comm.launches.append((0, off, n, slot))
        off += n
    p2p.FusedAllreduceSgdComm.setup_stage(comm)
    regions = []
    for _, _o, n, slot in comm.launches:
        per = n if n <= comm.one_shot_elems else comm._shard_len(n)
        assert per % 8 == 0 or n <= comm.one_shot_elems
        regions.append((comm._stage_off[slot], comm._stage_off[slot] + comm.world * per))
    regions.append((comm._stage_off[comm.num_slots - 1],
                    comm._stage_off[comm.num_slots - 1] + comm.world * comm._shard_len(comm.bucket_elems)))
    regions.sort()
    for (a0, a1), (b0, b1) in zip(regions, regions[1:]):
        assert a1 <= b0
    assert comm.arena.allocs["stage"] >= regions[-1][1]
