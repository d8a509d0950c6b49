"""Hierarchical (group mean + pull) gossip on the peer-to-peer kernels against the library backend, 2+ GPUs."""
import pytest
import torch

from test_multigpu import _run

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("group_size", [1, 2])
def test_group_gossip_two_ranks(group_size):
    _run(f"group_gossip_{group_size}")


def test_group_gossip_four_ranks_in_pairs():
    if torch.cuda.device_count() < 4:
        pytest.skip("needs at least 4 GPUs")
    _run("group_gossip_2", nproc=4)


@pytest.mark.parametrize("group_size", [1, 2])
def test_leader_gossip_two_ranks(group_size):
    _run(f"group_gossip_v1_{group_size}")


def test_leader_gossip_four_ranks_in_pairs():
    if torch.cuda.device_count() < 4:
        pytest.skip("needs at least 4 GPUs")
    _run("group_gossip_v1_2", nproc=4)
