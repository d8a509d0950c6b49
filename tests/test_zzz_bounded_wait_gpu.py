"""A bounded device wait that really runs out, in the form that leaves the GPU healthy: the barrier kernel is told
there are two ranks, both ranks' flag pads are ordinary local buffers, and nothing ever raises the second rank's flag.
With a 2 ms limit the kernel gives up, records the time-out in the status word and returns; the context stays usable.
That real status word is then fed through the training loop's check, which must write this rank's state beside the
regular checkpoints and stop the loop."""
import ctypes as C
import os
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

from rembrandt_b200._native import check
from rembrandt_b200.ops import native_ops as K
from rembrandt_b200.parallel import p2p_kernels as PK

PEER_TIMEOUT = 2


def _barrier(flags, epochs, status, world, wait_ns):
    a = PK.BarrierArgs()
    for i in range(PK.MAX_RANKS):
        a.flags[i] = flags[i].data_ptr() if i < world else None
    a.epoch_ptr = epochs.data_ptr()
    a.status = status.data_ptr()
    a.rank, a.world, a.slot = 0, world, 0
    a.wait_ns = wait_ns
    check(PK.fn("rb_barrier_p2p")(C.byref(a), torch.cuda.current_stream().cuda_stream), "rb_barrier_p2p")


@pytest.fixture
def clean_status():
    status = K.status_word()
    status.zero_()
    yield status
    status.zero_()          # the word is shared by every test of the process


def test_a_wait_on_a_peer_that_never_arrives_gives_up_and_reports(clean_status):
    status = clean_status
    flags = [torch.zeros(2 * PK.MAX_RANKS * 4, dtype=torch.int32, device="cuda") for _ in range(2)]
    epochs = torch.zeros(4, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    t0 = time.time()
    _barrier(flags, epochs, status, world=2, wait_ns=2_000_000)
    torch.cuda.synchronize()
    assert time.time() - t0 < 1.0, "the 2 ms limit was not honoured"
    assert K.read_status() & PEER_TIMEOUT
    # the kernel announced itself in both pads before it waited
    assert int(flags[0][0]) == 1 and int(flags[1][0]) == 1
    # the context is healthy: the next launch (a barrier among one rank) completes without a new error
    status.zero_()
    _barrier(flags, epochs, status, world=1, wait_ns=2_000_000)
    torch.cuda.synchronize()
    assert K.read_status() == 0
    x = torch.arange(8, device="cuda").sum()
    assert int(x) == 28


def test_the_training_loop_stops_on_that_status_and_keeps_its_state(clean_status, tmp_path):
    from rembrandt_b200.api import build_replica, default_opt
    from rembrandt_b200.trainer import DeviceWaitTimeout, SgdOpt
    status = clean_status
    d = str(tmp_path / "run")
    opt = default_opt(8)
    opt.checkpoint_dir = d
    eng = build_replica("lenet", 8, device="cuda", use_graph=False, opt=opt)
    sgd = SgdOpt(opt, eng, quiet=True)
    sgd._check_device_status(1)              # healthy so far: nothing happens
    flags = [torch.zeros(2 * PK.MAX_RANKS * 4, dtype=torch.int32, device="cuda") for _ in range(2)]
    epochs = torch.zeros(4, dtype=torch.int32, device="cuda")
    _barrier(flags, epochs, status, world=2, wait_ns=2_000_000)
    torch.cuda.synchronize()
    with pytest.raises(DeviceWaitTimeout):
        sgd._check_device_status(2)
    assert os.path.exists(os.path.join(d, "state.abort.blob.0"))
