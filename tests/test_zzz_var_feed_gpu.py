"""Variable-size batches through the step engine's pinned double buffer (GPU only): the per-sample size table must
travel with the pixels, so the engine path gives the same loss as loading the batch straight into the network."""
import pytest
import torch

from test_var_input import _var_cfg

from rembrandt_b200.api import default_opt
from rembrandt_b200.engine import StepEngine
from rembrandt_b200.models.net import Net
from rembrandt_b200.models.operators import VarDataOp
from rembrandt_b200.parallel.comm import NullComm

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("as_list", [True, False])
def test_engine_feeds_variable_size_batches(as_list):
    # scale range of one value and no flip: the input kernel is deterministic in training mode too
    direct = Net(_var_cfg(32, 32, 32, flip=False), 4, device="cuda", seed=(5, 6))
    net = Net(_var_cfg(32, 32, 32, flip=False), 4, device="cuda", seed=(5, 6))
    eng = StepEngine(net, default_opt(4, "null"), NullComm(), use_graph=False)
    labels = torch.tensor([0, 3, 5, 7], dtype=torch.int32)
    losses = []
    for seed in (9, 10):
        # square samples of different sizes: all rescale to exactly 32 x 32, which leaves the crop no freedom
        g = torch.Generator().manual_seed(seed)
        imgs = [torch.randint(0, 256, (3, 32 + 8 * i, 32 + 8 * i), dtype=torch.uint8, generator=g) for i in range(4)]
        feed = imgs if as_list else tuple(t.pin_memory() for t in VarDataOp.pack(imgs, net.input_op.in_stride))
        # the direct network holds the weights the engine has before this step
        eng.synchronize()
        with torch.no_grad():
            direct.params.copy_(net.params)
            direct.params16.copy_(net.params16)
        torch.cuda.synchronize()
        eng.feed(feed, labels.pin_memory())
        eng.step()
        direct.load_batch(imgs, labels.cuda())
        direct.read_stats()
        direct.forward(False)
        losses.append(direct.read_stats()[0])
    got = eng.flush()
    assert got is not None and eng.h2d_bytes_per_step() == 4 * net.input_op.in_stride + 4 * 4 + 4 * 2 * 4
    # the second engine step saw the second batch with its own size table: its loss equals the direct evaluation
    # made with the weights the engine had before that step
    assert abs(got[0] - losses[1]) < 0.05 * max(1.0, abs(losses[1])), (got, losses)
