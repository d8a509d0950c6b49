"""The training loop on CPU: the MNIST-shaped softmax-regression configuration, sync orders, gradient
accumulation, CSV traces, checkpoint + resume, validation, straggler injection."""
import csv
import os

import pytest
import torch

from rembrandt_b200.data import BatchIter, CyclicSampleDataIter, RandomSampleDataIter, RangeDataShard, SyntheticDataSource
from rembrandt_b200.engine import StepEngine
from rembrandt_b200.models import zoo
from rembrandt_b200.models.net import Net
from rembrandt_b200.optim.sgd import (InitBehavior, Momentum, SgdOptConfig, StepSizeReference, StepSizeSchedule, SyncOrder)
from rembrandt_b200.trainer import ExperimentConfig, SgdOpt


def mnist_shape_batches(seed, batch=64, steps=100):
    g = torch.Generator().manual_seed(seed)
    for _ in range(steps):
        yield (torch.rand(batch, 1, 28, 28, generator=g).mul(255).to(torch.uint8),
               torch.randint(0, 10, (batch,), generator=g, dtype=torch.int32))


def make(cfg_fn=zoo.mnist_fc1, batch=64, **opt_kw):
    opt_kw.setdefault("minibatch_size", batch)
    opt_kw.setdefault("step_size", StepSizeSchedule.constant(0.01))
    opt_kw.setdefault("momentum", Momentum.UPDATE)
    opt_kw.setdefault("display_iters", 0)
    opt = SgdOptConfig(**opt_kw)
    net = Net(cfg_fn(), batch, device="cpu", seed=(0, 0), minibatch_size=opt.minibatch_size)
    return opt, StepEngine(net, opt), net


def test_mnist_shape_softmax_regression_100_steps_seed0():
    """Input [64,784] uniform, labels uniform 0..9, affine 784->10 + softmax CE, SGD lr 0.01 momentum 0.9, 100 steps:
    labels carry no signal, so the loss must stay near ln(10) while the plumbing runs end to end."""
    opt, eng, net = make()
    sgd = SgdOpt(opt, eng, quiet=True)
    losses = []
    for x, y in mnist_shape_batches(0):
        eng.feed(x, y)
        losses.append(eng.step()[0])
    assert eng.iter == 100 and net.t == 100
    assert all(1.9 < l < 2.9 for l in losses), (min(losses), max(losses))
    assert float(net.mom.abs().sum()) > 0 and float(net.grads.abs().sum()) == 0


def test_learns_separable_data_and_validates():
    src = SyntheticDataSource(512, (28, 28, 1), 10, seed=1, separable=True)
    opt, eng, net = make(batch=32, step_size=StepSizeSchedule.constant(0.05), valid_iters=4, display_iters=10)
    sgd = SgdOpt(opt, eng, quiet=True)
    train = BatchIter(RandomSampleDataIter(RangeDataShard(src), seed=(3, 4)), 32, src.dims)
    hist = sgd.train(train, None, max_iters=60)
    assert hist[-1][1] < 0.5 * hist[0][1] and hist[-1][2] > 0.9
    loss, acc = sgd.validate(BatchIter(CyclicSampleDataIter(RangeDataShard(src)), 32, src.dims), 4)
    assert acc > 0.9 and loss < 0.7


@pytest.mark.parametrize("order", list(SyncOrder))
def test_sync_orders_agree_on_a_single_worker(order):
    """With one worker nothing is exchanged, so every order must give the same parameters."""
    ref_opt, ref_eng, ref_net = make(sync_order=SyncOrder.SYNC_GRADS_THEN_STEP)
    opt, eng, net = make(sync_order=order)
    for x, y in mnist_shape_batches(5, steps=5):
        for e in (ref_eng, eng):
            e.feed(x, y)
            e.step()
    assert torch.allclose(net.params.detach(), ref_net.params.detach(), atol=1e-7)


def test_gradient_accumulation_equals_one_large_batch():
    opt_a, eng_a, net_a = make(batch=64, minibatch_size=64)
    opt_b, eng_b, net_b = make(batch=16, minibatch_size=64)
    assert eng_b.accum == 4
    x, y = next(mnist_shape_batches(9))
    eng_a.feed(x, y)
    eng_a.step()
    for i in range(4):
        eng_b.feed(x[16 * i:16 * i + 16], y[16 * i:16 * i + 16])
        eng_b.step()
    assert eng_b.iter == 1 and net_b.t == 4
    assert torch.allclose(net_a.params.detach(), net_b.params.detach(), atol=1e-6)


@pytest.mark.parametrize("rule", [Momentum.UPDATE, Momentum.UPDATE_NESTEROV])
def test_trace_csv_checkpoint_and_resume(tmp_path, rule):
    d = str(tmp_path / "run")
    common = dict(checkpoint_iters=4, save_iters=4, checkpoint_dir=d, momentum=rule)
    opt, eng, net = make(batch=16, **common)
    sgd = SgdOpt(opt, eng, quiet=True)
    sgd.train(mnist_shape_batches(1, 16, 8), None, max_iters=8)
    sgd.trace.close()
    rows = list(csv.reader(open(os.path.join(d, "trace_sgd.0.log"))))
    assert rows[0] == ["t", "event", "loss", "error", "elapsed"]
    assert [r[1] for r in rows[1:]].count("step") == 8
    assert open(os.path.join(d, "checkpoint")).read() == "8\n"
    assert os.path.exists(os.path.join(d, "params.t_4.blob")) and os.path.exists(os.path.join(d, "state.latest.blob.0"))
    # an uninterrupted 12-iteration run ...
    opt_u, eng_u, net_u = make(batch=16, momentum=rule)
    SgdOpt(opt_u, eng_u, quiet=True).train(mnist_shape_batches(1, 16, 12), None, max_iters=12)
    # ... equals resuming from the checkpoint at 8 and running 4 more on the same data stream
    opt_r, eng_r, net_r = make(batch=16, **common)
    sgd_r = SgdOpt(opt_r, eng_r, quiet=True)
    stream = mnist_shape_batches(1, 16, 12)
    for _ in range(8):
        next(stream)
    sgd_r.train(stream, None, max_iters=12)
    assert eng_r.iter == 12
    assert torch.allclose(net_r.params.detach(), net_u.params.detach(), atol=1e-6)
    # a second run in the same directory does not overwrite the first trace
    assert os.path.exists(os.path.join(d, "trace_sgd.0.log.1"))


def test_resume_from_a_given_iteration(tmp_path):
    d = str(tmp_path / "run")
    opt, eng, net = make(batch=16, checkpoint_iters=2, save_iters=2, checkpoint_dir=d)
    SgdOpt(opt, eng, quiet=True).train(mnist_shape_batches(2, 16, 4), None, max_iters=4)
    opt2, eng2, net2 = make(batch=16, checkpoint_dir=d, init=InitBehavior.RESUME_FROM, resume_t=2)
    sgd2 = SgdOpt(opt2, eng2, quiet=True)
    assert sgd2._init_or_resume() == 2
    assert net2.encode_params() == open(os.path.join(d, "params.t_2.blob"), "rb").read()


def test_step_size_reference_checkpoint_freezes_the_rate_between_checkpoints():
    sched = StepSizeSchedule.anneal1(0.1, 3, 0.01)
    opt, eng, net = make(batch=16, step_size=sched, step_ref=StepSizeReference.CHECKPOINT, checkpoint_iters=4)
    sgd = SgdOpt(opt, eng, quiet=True)
    seen = []
    orig = eng._update

    def spy():
        seen.append(eng.lr)
        orig()
    eng._update = spy
    sgd.train(mnist_shape_batches(3, 16, 8), None, max_iters=8)
    assert seen[:4] == [0.1] * 4 and seen[5:] == [0.01] * 3       # changes only after the checkpoint at t = 4


def test_straggler_injection_only_delays():
    opt, eng, net = make(batch=16)
    opt2, eng2, net2 = make(batch=16)
    SgdOpt(opt, eng, ExperimentConfig([0], 5), quiet=True).train(mnist_shape_batches(4, 16, 5), None, max_iters=5)
    SgdOpt(opt2, eng2, quiet=True).train(mnist_shape_batches(4, 16, 5), None, max_iters=5)
    assert torch.equal(net.params.detach(), net2.params.detach())


def test_nesterov_prelookahead_and_report_hook():
    class Rep:
        def __init__(self):
            self.t = []

        def update_training(self, t, loss, acc):
            self.t.append(t)

        def update_validation(self, *a):
            pass
    opt, eng, net = make(batch=16, momentum=Momentum.UPDATE_NESTEROV, display_iters=2)
    rep = Rep()
    SgdOpt(opt, eng, report=rep, quiet=True).train(mnist_shape_batches(6, 16, 6), None, max_iters=6)
    assert rep.t == [2, 4, 6]


def test_mimic_training_pulls_student_towards_teacher():
    """Distillation: the student's output distribution approaches the teacher's on the training batch."""
    import torch.nn.functional as F
    from rembrandt_b200.api import default_opt
    from rembrandt_b200.engine import StepEngine
    from rembrandt_b200.models import zoo
    from rembrandt_b200.models.net import Net
    from rembrandt_b200.optim.mimic import MimicSgdOpt
    from rembrandt_b200.parallel.comm import NullComm
    teacher = Net(zoo.mnist_fc1(), 16, device="cpu", seed=(11, 12), training=False)
    student = Net(zoo.mnist_fc1(), 16, device="cpu", seed=(21, 22))
    torch.manual_seed(0)
    x = torch.randint(0, 256, (16, 1, 28, 28), dtype=torch.uint8)
    y = torch.randint(0, 10, (16,))

    def kl():
        outs = []
        for n in (teacher, student):
            n.load_batch(x, y)
            with torch.no_grad():
                n.forward(False)
            n.read_stats()
            outs.append(F.log_softmax(n._cpu_logits.flatten(1), 1))
        return float((outs[0].exp() * (outs[0] - outs[1])).sum(1).mean())

    before = kl()
    cfg = default_opt(16, "null")
    cfg.max_iters = 60
    cfg.display_iters = 0
    cfg.checkpoint_iters = 0
    eng = StepEngine(student, cfg, NullComm(), use_graph=False)
    eng.set_lr(0.1)
    opt = MimicSgdOpt(cfg, eng, teacher, quiet=True)
    opt.train([(x, y)] * 60, max_iters=60)
    after = kl()
    assert after < 0.5 * before, (before, after)


def test_mimic_training_on_activations_fits_a_low_rank_student_to_the_teacher():
    """The other hand-over of the reference's mimic optimizer: the activations that enter the teacher's loss become
    the L2 targets of a student (here a low-rank one) that ends in an L2 head."""
    from rembrandt_b200.api import default_opt
    from rembrandt_b200.engine import StepEngine
    from rembrandt_b200.models import zoo
    from rembrandt_b200.models.config import (Data3dCfg, MimicAffineCfg, PointwiseLossCfg,
                                              SequentialOperatorConfig)
    from rembrandt_b200.models.net import Net
    from rembrandt_b200.optim.mimic import MimicSgdOpt
    from rembrandt_b200.parallel.comm import NullComm
    teacher = Net(zoo.mnist_fc2(hidden=64), 16, device="cpu", seed=(11, 12), training=False)
    scfg = (SequentialOperatorConfig().data3d(Data3dCfg((28, 28, 1), normalize=True))
            .mimic_affine(MimicAffineCfg(bottleneck_rank=8, hidden_channels=32, out_channels=10), "m")
            .pointwise_loss(PointwiseLossCfg(10, "l2")))
    student = Net(scfg, 16, device="cpu", seed=(21, 22))
    torch.manual_seed(0)
    x = torch.randint(0, 256, (16, 1, 28, 28), dtype=torch.uint8)
    y = torch.randint(0, 10, (16,))

    def gap():
        outs = []
        for n in (teacher, student):
            n.load_batch(x, y)
            with torch.no_grad():
                n.forward(False)
            n.read_stats()
            outs.append(n._cpu_logits.flatten(1).clone())
        return float(((outs[0] - outs[1]) ** 2).sum(1).mean())

    cfg = default_opt(16, "null")
    cfg.max_iters, cfg.display_iters, cfg.checkpoint_iters = 80, 0, 0
    eng = StepEngine(student, cfg, NullComm(), use_graph=False)
    eng.set_lr(0.05)
    opt = MimicSgdOpt(cfg, eng, teacher, target="activations", quiet=True)
    student.loss_op.load_targets(torch.zeros(16, 10))     # so that the first measurement has targets to ignore
    before = gap()
    opt.train([(x, y)] * 80, max_iters=80)
    after = gap()
    assert after < 0.5 * before, (before, after)
    with pytest.raises(ValueError):
        MimicSgdOpt(cfg, StepEngine(Net(zoo.mnist_fc1(), 16, device="cpu"), cfg, NullComm(), use_graph=False), teacher,
                    target="activations", quiet=True)


def test_async_sgd_opt_checkpoints_locally_without_barriers(tmp_path):
    """The barrier-free loop trains like the synchronous one on a single worker, never calls a barrier, and
    writes its checkpoints under a per-rank directory."""
    from rembrandt_b200.optim.async_sgd import AsyncSgdOpt
    d = str(tmp_path / "run")
    opt, eng, net = make(batch=16, checkpoint_iters=4, save_iters=4, checkpoint_dir=d)
    calls = []
    eng.comm.barrier = lambda: calls.append("barrier")
    sgd = AsyncSgdOpt(opt, eng, quiet=True)
    sgd.train(mnist_shape_batches(1, 16, 8), None, max_iters=8)
    assert eng.iter == 8 and not calls
    assert os.path.exists(os.path.join(d, "rank0", "params.t_8.blob"))
    assert os.path.exists(os.path.join(d, "rank0", "state.latest.blob.0"))
    opt_s, eng_s, net_s = make(batch=16)
    SgdOpt(opt_s, eng_s, quiet=True).train(mnist_shape_batches(1, 16, 8), None, max_iters=8)
    assert torch.allclose(net.params.detach(), net_s.params.detach(), atol=1e-6)


def test_a_device_wait_that_ran_out_stops_the_loop_and_keeps_local_state(tmp_path):
    """The status word is faked on the host (nothing on a GPU is made to time out): from iteration 6 on it reports a
    peer timeout; the loop must stop at the next display point, leave the regular checkpoints alone and write this
    rank's state under its own name."""
    from rembrandt_b200.trainer import DeviceWaitTimeout
    opt, eng, net = make(display_iters=4, checkpoint_iters=4, save_iters=4, checkpoint_dir=str(tmp_path))
    sgd = SgdOpt(opt, eng, quiet=True)
    sgd._device_status = lambda: 0x2 if eng.iter >= 6 else 0
    with pytest.raises(DeviceWaitTimeout, match="status 0x2 at iteration 8"):
        sgd.train(mnist_shape_batches(3, steps=40), max_iters=40)
    assert eng.iter == 8
    names = sorted(os.listdir(tmp_path))
    assert "state.abort.blob.0" in names and "params.t_4.blob" in names and "params.t_8.blob" not in names
    rows = list(csv.reader(open(os.path.join(tmp_path, "trace_sgd.0.log"))))
    assert rows[-1][:2] == ["8", "abort"]
    # the aborted state is a complete state blob: a fresh network can load it
    other = Net(zoo.mnist_fc1(), 64, device="cpu", seed=(5, 5), minibatch_size=64)
    other.decode_state(open(os.path.join(tmp_path, "state.abort.blob.0"), "rb").read())
    assert torch.equal(other.params, net.params)


def test_exchange_rate_uses_the_bus_bandwidth_convention():
    import types
    opt, eng, net = make()
    sgd = SgdOpt(opt, eng, quiet=True)
    assert sgd._exchange_rate(10, 5.0) is None                     # one worker: nothing is exchanged
    sgd.world = 8
    sgd.comm = types.SimpleNamespace(name="fused_allreduce_sgd")
    per_iter = net.flat_len * 4.0
    assert sgd._exchange_rate(10, 5.0) == pytest.approx(10 * per_iter * 1.75 / 5e-3 / 1e9)
    sgd.comm = types.SimpleNamespace(name="gossip_p2p")
    assert sgd._exchange_rate(10, 5.0) == pytest.approx(10 * per_iter / 5e-3 / 1e9)


def test_lenet_reaches_full_accuracy_on_separable_synthetic_digits():
    """Convergence smoke test: the convolutional LeNet template on seeded, class-separable synthetic images."""
    src = SyntheticDataSource(1024, (28, 28, 1), 10, seed=1, separable=True)
    opt = SgdOptConfig(minibatch_size=32, step_size=StepSizeSchedule.constant(0.02), momentum=Momentum.UPDATE_NESTEROV,
                       mu=0.9, l2_reg_coef=5e-4, display_iters=20)
    net = Net(zoo.lenet(pad=2), 32, device="cpu", seed=(0, 0), minibatch_size=32)
    sgd = SgdOpt(opt, StepEngine(net, opt), quiet=True)
    batches = BatchIter(RandomSampleDataIter(RangeDataShard(src), seed=(3, 4)), 32, src.dims)

    def forever():
        while True:
            for b in batches:
                yield b
    hist = sgd.train(forever(), None, max_iters=120)
    assert hist[-1][2] == 1.0 and hist[-1][1] < 1e-2 * hist[0][1]
    loss, acc = sgd.validate(BatchIter(CyclicSampleDataIter(RangeDataShard(src)), 32, src.dims), 8)
    assert acc == 1.0 and loss < 1e-2
