"""Kernel-driven communication backends on 2+ GPUs (skipped with fewer), one process per GPU.

Each case runs tests/mgpu_worker.py under torch.distributed.run with a time limit; the worker compares
the peer-to-peer kernels with the same exchange done through NCCL collectives.
"""
import os
import signal
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


def _run(case, nproc=None, timeout=120):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    nproc = nproc or 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(HERE, "mgpu_worker.py"), case]
    # its own session, so that a run that overstays is ended with all of its workers (a launcher killed alone would
    # leave them on the GPUs)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, start_new_session=True)
    try:
        out, err = proc.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)
        out, err = proc.communicate()
        raise AssertionError(f"case {case} overstayed {timeout} s\n" + out[-3000:] + "\n" + err[-6000:])
    assert proc.returncode == 0, (out[-3000:] + "\n" + err[-14000:])
    assert f"case {case}: ok" in out


@pytest.mark.parametrize("case", ["p2p_allreduce", "fused_eager", "fused_graph", "gossip_pair", "pull_rounds", "elastic", "push",
                                  "push_async", "elastic_async"])
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
