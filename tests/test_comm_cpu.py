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


def test_group_allreduce_then_gossip():
    run_ranks(4, cases.hierarchical)


def test_exact_sync_is_a_true_mean_for_gossip_backends():
    run_ranks(3, cases.exact_sync)


def test_a_rank_that_raises_ends_the_others_with_an_error_not_a_hang():
    codes, msgs = run_ranks(3, cases.rank_raises_before_collective, timeout_s=8, expect_failure=True)
    assert all(c is not None for c in codes), "a rank hung"
    assert codes[1] != 0 and any("injected failure" in m for _, m in msgs)
    assert all(c != 0 for c in codes), "survivors must see the failure (connection reset or timeout)"


def test_a_rank_that_never_joins_times_the_collective_out():
    codes, msgs = run_ranks(3, cases.rank_never_joins, timeout_s=3, expect_failure=True)
    assert all(c is not None for c in codes), "a rank hung"
    assert codes[0] != 0 and codes[1] != 0


def test_a_straggler_only_delays():
    run_ranks(3, cases.straggler_is_tolerated)


def test_data_parallel_training_equals_single_process_on_the_global_batch():
    run_ranks(2, cases.dp_training_matches_single_process, timeout_s=120)
