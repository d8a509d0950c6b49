"""Kernel-driven communication backends on 2+ GPUs (skipped with fewer), one process per GPU.

Each case runs tests/mgpu_worker.py under torch.distributed.run with a time limit; the worker compares
the peer-to-peer kernels with the same exchange done through NCCL collectives.
"""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(case, nproc=None, timeout=240):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    nproc = nproc or 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(HERE, "mgpu_worker.py"), case]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, (r.stdout[-3000:] + "\n" + r.stderr[-6000:])
    assert f"case {case}: ok" in r.stdout


@pytest.mark.parametrize("case", ["p2p_allreduce", "fused_eager", "fused_graph", "gossip_pair", "pull_rounds", "elastic", "push"])
def test_p2p_backend(case):
    _run(case)


@pytest.mark.parametrize("case", ["p2p_allreduce", "fused_graph"])
def test_p2p_backend_all_gpus(case):
    """The gradient-exchange cases on every GPU of the box (8 ranks: one staged slot / one peer flag per rank in
    use). The gossip / elastic cases compare against library collectives and run on two ranks."""
    n = torch.cuda.device_count()
    if n <= 4:
        pytest.skip("covered by test_p2p_backend")
    _run(case, nproc=n)
