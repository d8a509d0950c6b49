"""The distillation optimizer and the barrier-free optimizer on the device (their logic is tested on CPU; this checks
the device plumbing: teacher inference on the compute stream, soft targets in a fixed buffer under CUDA graphs)."""
import os

import pytest
import torch

from rembrandt_b200.api import default_opt
from rembrandt_b200.engine import StepEngine
from rembrandt_b200.models import zoo
from rembrandt_b200.models.net import Net
from rembrandt_b200.ops import native_ops as K
from rembrandt_b200.optim.async_sgd import AsyncSgdOpt
from rembrandt_b200.optim.mimic import MimicSgdOpt
from rembrandt_b200.parallel.comm import NullComm
from rembrandt_b200.trainer import SgdOpt

pytestmark = pytest.mark.gpu


def _kl(teacher, student, x, y):
    outs = []
    for n in (teacher, student):
        n.loss_op.enable_probs()
        n.load_batch(x.cuda(), y.cuda().int())
        n.forward(False)
        n.read_stats()
        outs.append(n.loss_op.probs.clone().clamp_min(1e-12))
    q, p = outs
    return float((q * (q.log() - p.log())).sum(1).mean())


@pytest.mark.parametrize("use_graph", [False, True])
def test_student_approaches_teacher(use_graph):
    teacher = Net(zoo.mnist_fc1(), 16, device="cuda", seed=(11, 12), training=False)
    student = Net(zoo.mnist_fc1(), 16, device="cuda", seed=(21, 22))
    torch.manual_seed(0)
    x = torch.randint(0, 256, (16, 1, 28, 28), dtype=torch.uint8)
    y = torch.randint(0, 10, (16,), dtype=torch.int32)
    before = _kl(teacher, student, x, y)
    cfg = default_opt(16, "null")
    cfg.max_iters, cfg.display_iters, cfg.checkpoint_iters = 60, 0, 0
    eng = StepEngine(student, cfg, NullComm(), use_graph=use_graph)
    eng.set_lr(0.1)
    MimicSgdOpt(cfg, eng, teacher, quiet=True).train([(x.pin_memory(), y.pin_memory())] * 60, max_iters=60)
    torch.cuda.synchronize()
    assert K.read_status() == 0
    after = _kl(teacher, student, x, y)
    assert after < 0.7 * before, (before, after)


@pytest.mark.parametrize("use_graph", [False, True])
def test_low_rank_student_approaches_teacher_activations(use_graph):
    """Distillation of activations: the teacher's pre-softmax outputs are the L2 targets of a low-rank student; the
    targets live in a fixed device buffer that the captured step reads."""
    from rembrandt_b200.models.config import Data3dCfg, MimicAffineCfg, PointwiseLossCfg, SequentialOperatorConfig
    teacher = Net(zoo.mnist_fc2(hidden=64), 16, device="cuda", seed=(11, 12), training=False)
    scfg = (SequentialOperatorConfig().data3d(Data3dCfg((28, 28, 1), normalize=True))
            .mimic_affine(MimicAffineCfg(bottleneck_rank=32, hidden_channels=64, out_channels=10), "m")
            .pointwise_loss(PointwiseLossCfg(10, "l2")))
    student = Net(scfg, 16, device="cuda", seed=(21, 22))
    torch.manual_seed(0)
    x = torch.randint(0, 256, (16, 1, 28, 28), dtype=torch.uint8)
    y = torch.randint(0, 10, (16,), dtype=torch.int32)

    def gap():
        outs = []
        for n in (teacher, student):
            n.load_batch(x.cuda(), y.cuda())
            n.forward(False)
            torch.cuda.synchronize()
            outs.append(n.loss_op._logits()[0].reshape(16, -1)[:, :10].float().clone())
        return float(((outs[0] - outs[1]) ** 2).sum(1).mean())

    cfg = default_opt(16, "null")
    cfg.max_iters, cfg.display_iters, cfg.checkpoint_iters = 80, 0, 0
    eng = StepEngine(student, cfg, NullComm(), use_graph=use_graph)
    eng.set_lr(0.05)
    opt = MimicSgdOpt(cfg, eng, teacher, target="activations", quiet=True)
    student.loss_op.load_targets(torch.zeros(16, 10, device="cuda"))
    before = gap()
    opt.train([(x.pin_memory(), y.pin_memory())] * 80, max_iters=80)
    torch.cuda.synchronize()
    assert K.read_status() == 0
    after = gap()
    assert after < 0.6 * before, (before, after)


def test_barrier_free_loop_matches_the_synchronous_one(tmp_path):
    def batches(n):
        g = torch.Generator().manual_seed(1)
        for _ in range(n):
            yield (torch.rand(16, 1, 28, 28, generator=g).mul(255).to(torch.uint8).pin_memory(),
                   torch.randint(0, 10, (16,), generator=g, dtype=torch.int32).pin_memory())

    nets = []
    for cls, sub in ((AsyncSgdOpt, "a"), (SgdOpt, "s")):
        cfg = default_opt(16, "null")
        cfg.display_iters, cfg.checkpoint_iters, cfg.save_iters = 0, 4, 4
        cfg.checkpoint_dir = str(tmp_path / sub)
        net = Net(zoo.mnist_fc1(), 16, device="cuda", seed=(3, 4), minibatch_size=16)
        eng = StepEngine(net, cfg, NullComm(), use_graph=False)
        cls(cfg, eng, quiet=True).train(batches(8), None, max_iters=8)
        torch.cuda.synchronize()
        nets.append(net)
    assert os.path.exists(os.path.join(tmp_path, "a", "rank0", "params.t_8.blob"))
    assert torch.allclose(nets[0].params, nets[1].params, atol=1e-6)
