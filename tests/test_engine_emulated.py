"""The CUDA branch of `StepEngine` (double-buffered staging, lagged statistics, gradient accumulation, the update in
the configured order) on CPU tensors: streams and events are replaced by inert stand-ins, the kernel fronts by the
plain-torch ones of tests/kernel_emulation.py. The result is compared with the CPU branch of the same engine."""
import pytest
import torch

import kernel_emulation
from rembrandt_b200.engine import StepEngine
from rembrandt_b200.models import zoo
from rembrandt_b200.models.net import Net
from rembrandt_b200.optim.sgd import Momentum, SgdOptConfig, StepSizeSchedule
from rembrandt_b200.trainer import SgdOpt


class _Stream:
    cuda_stream = 0

    def wait_event(self, ev):
        pass

    def synchronize(self):
        pass


class _Event:
    def __init__(self, *a, **k):
        pass

    def record(self, stream=None):
        pass

    def synchronize(self):
        pass

    def elapsed_time(self, other):
        return 1.0


class _Ctx:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def _device_engine(monkeypatch, cfg_fn, batch, opt):
    kernel_emulation.install(monkeypatch)
    monkeypatch.setattr(torch.cuda, "Stream", lambda *a, **k: _Stream())
    monkeypatch.setattr(torch.cuda, "Event", _Event)
    monkeypatch.setattr(torch.cuda, "stream", lambda s: _Ctx())
    monkeypatch.setattr(torch.cuda, "current_stream", lambda *a: _Stream())
    monkeypatch.setattr(torch.Tensor, "pin_memory", lambda self, *a, **k: self)
    monkeypatch.setattr(Net, "device_path_on_cpu", True)
    net = Net(cfg_fn(), batch, device="cpu", seed=(2, 3), minibatch_size=opt.minibatch_size)
    monkeypatch.setattr(Net, "device_path_on_cpu", False)
    return StepEngine(net, opt, use_graph=False), net


def _batches(n, batch):
    g = torch.Generator().manual_seed(11)
    return [(torch.randint(0, 256, (batch, 1, 28, 28), dtype=torch.uint8, generator=g),
             torch.randint(0, 10, (batch,), dtype=torch.int32, generator=g)) for _ in range(n)]


@pytest.mark.parametrize("accum", [1, 2])
@pytest.mark.parametrize("mode", [Momentum.UPDATE, Momentum.UPDATE_NESTEROV])
def test_device_branch_of_the_engine_matches_the_cpu_branch(monkeypatch, accum, mode):
    batch = 8
    opt = SgdOptConfig(minibatch_size=batch * accum, step_size=StepSizeSchedule.constant(0.01), momentum=mode, mu=0.9,
                       l2_reg_coef=1e-3, display_iters=0)
    cpu_net = Net(zoo.lenet(pad=2), batch, device="cpu", seed=(2, 3), minibatch_size=batch * accum)
    cpu_eng = StepEngine(cpu_net, opt)
    dev_eng, dev_net = _device_engine(monkeypatch, lambda: zoo.lenet(pad=2), batch, opt)
    assert dev_eng.is_cuda and dev_eng.accum == accum
    with torch.no_grad():                      # both start from the bf16-rounded weights
        cpu_net.params.copy_(dev_net.params16.float())
        dev_net.params.copy_(dev_net.params16.float())
    data = _batches(6, batch)
    dev_stats, cpu_stats = [], []
    for x, y in data:
        dev_eng.feed(x, y)
        s = dev_eng.step()
        if s is not None:
            dev_stats.append(s)
        cpu_eng.feed(x, y)
        cpu_stats.append(cpu_eng.step())
    dev_stats.append(dev_eng.flush())
    assert dev_eng.iter == cpu_eng.iter == 6 // accum and dev_net.t == 6
    # statistics arrive one step late on the device branch, and are the same numbers
    assert len(dev_stats) == len(cpu_stats) == 6
    for (dl, dc), (cl, cc) in zip(dev_stats, cpu_stats):
        assert abs(dl - cl) < 3e-2 * max(1.0, abs(cl)), (dl, cl)
    rel = float((dev_net.params - cpu_net.params.detach()).norm() / cpu_net.params.detach().norm())
    assert rel < 6e-2, rel     # six steps of bf16 compute against fp32; a wiring mistake is of order one
    assert torch.equal(dev_net.params16, dev_net.params.bfloat16())
    assert dev_eng.h2d_bytes_per_step() == batch * 28 * 28 + batch * 4 and dev_eng.d2h_bytes_per_step() == 8


def test_training_loop_on_the_device_branch(monkeypatch):
    """`SgdOpt.train` over the device branch: display points, device-timed throughput, checkpoint window."""
    opt = SgdOptConfig(minibatch_size=8, step_size=StepSizeSchedule.constant(0.05), momentum=Momentum.UPDATE, mu=0.9,
                       display_iters=2, checkpoint_iters=4)
    eng, net = _device_engine(monkeypatch, zoo.mnist_fc1, 8, opt)
    sgd = SgdOpt(opt, eng, quiet=True)
    hist = sgd.train(iter(_batches(8, 8)), None, max_iters=8)
    assert eng.iter == 8 and [h[0] for h in hist] == [2, 4, 6, 8]
    assert all(0.0 < h[1] < 10.0 for h in hist)


def test_distillation_on_the_device_branch(monkeypatch):
    """Teacher inference on the compute stream, its probabilities as soft targets of the student's fused head."""
    from rembrandt_b200.optim.mimic import MimicSgdOpt
    opt = SgdOptConfig(minibatch_size=16, step_size=StepSizeSchedule.constant(0.1), momentum=Momentum.UPDATE, mu=0.9,
                       display_iters=0)
    eng, student = _device_engine(monkeypatch, zoo.mnist_fc1, 16, opt)
    monkeypatch.setattr(Net, "device_path_on_cpu", True)
    teacher = Net(zoo.mnist_fc1(), 16, device="cpu", seed=(11, 12), training=False)
    monkeypatch.setattr(Net, "device_path_on_cpu", False)
    torch.manual_seed(0)
    x = torch.randint(0, 256, (16, 1, 28, 28), dtype=torch.uint8)
    y = torch.randint(0, 10, (16,), dtype=torch.int32)

    def kl():
        outs = []
        for n in (teacher, student):
            n.loss_op.enable_probs()
            n.load_batch(x, y)
            n.forward(False)
            n.read_stats()
            outs.append(n.loss_op.probs.clone().clamp_min(1e-12))
        q, p = outs
        return float((q * (q.log() - p.log())).sum(1).mean())

    before = kl()
    MimicSgdOpt(opt, eng, teacher, quiet=True).train([(x, y)] * 60, max_iters=60)
    after = kl()
    assert after < 0.5 * before, (before, after)


@pytest.mark.parametrize("as_list", [True, False])
def test_variable_size_batches_through_the_engine(monkeypatch, as_list):
    """The per-sample size table travels through the staging slots with the pixels: the loss of an engine step equals
    a direct evaluation of the same batch with the weights the engine had before the step."""
    from test_var_input import _var_cfg
    from rembrandt_b200.models.operators import VarDataOp
    opt = SgdOptConfig(minibatch_size=4, step_size=StepSizeSchedule.constant(0.01), momentum=Momentum.UPDATE, mu=0.9,
                       display_iters=0)
    eng, net = _device_engine(monkeypatch, lambda: _var_cfg(32, 32, 32, flip=False), 4, opt)
    monkeypatch.setattr(Net, "device_path_on_cpu", True)
    direct = Net(_var_cfg(32, 32, 32, flip=False), 4, device="cpu", seed=(2, 3), minibatch_size=4)
    monkeypatch.setattr(Net, "device_path_on_cpu", False)
    labels = torch.tensor([0, 3, 5, 7], dtype=torch.int32)
    seen = []
    for seed in (9, 10):
        g = torch.Generator().manual_seed(seed)
        order = [0, 1, 2, 3] if seed == 9 else [3, 1, 0, 2]            # the second batch has another size table
        imgs = [torch.randint(0, 256, (3, 32 + 8 * i, 32 + 8 * i), dtype=torch.uint8, generator=g) for i in order]
        with torch.no_grad():
            direct.params.copy_(net.params)
            direct.params16.copy_(net.params16)
        eng.feed(imgs if as_list else VarDataOp.pack(imgs, net.input_op.in_stride), labels)
        stats = eng.step()
        if stats is not None:
            seen.append(stats[0])
        direct.load_batch(imgs, labels)
        direct.read_stats()
        direct.forward(True)
        want = direct.read_stats()[0]
        if seed == 10:
            seen.append(eng.flush()[0])
            assert abs(seen[-1] - want) < 1e-5 * max(1.0, abs(want)), (seen, want)
    assert eng.h2d_bytes_per_step() == 4 * net.input_op.in_stride + 4 * 4 + 4 * 2 * 4


def test_phase_timing_helper_runs_the_three_phases(monkeypatch):
    from rembrandt_b200.utils.timing import time_phases
    opt = SgdOptConfig(minibatch_size=8, step_size=StepSizeSchedule.constant(0.01), momentum=Momentum.UPDATE, mu=0.9,
                       display_iters=0)
    eng, net = _device_engine(monkeypatch, zoo.mnist_fc1, 8, opt)
    x, y = _batches(1, 8)[0]
    net.load_batch(x, y)
    before = net.params.clone()
    out = time_phases(eng, iters=2, warmup=1)
    # the inert events report 1 ms between any two marks
    assert out == {"forward_ms": 1.0, "backward_ms": 1.0, "exchange_update_tail_ms": 1.0, "step_ms": 3.0}
    assert not torch.equal(net.params, before) and int(net.step_counter) == 3


def test_overlapped_local_update_equals_one_sweep_after_backward(monkeypatch):
    """The per-bucket optimizer launches from the backward hooks cover every parameter exactly once."""
    from rembrandt_b200.parallel.comm import LocalOverlapComm
    opt = SgdOptConfig(minibatch_size=8, step_size=StepSizeSchedule.constant(0.02), momentum=Momentum.UPDATE_NESTEROV,
                       mu=0.9, l2_reg_coef=1e-3, display_iters=0)
    plain, net_a = _device_engine(monkeypatch, lambda: zoo.lenet(pad=2), 8, opt)
    monkeypatch.setattr(Net, "device_path_on_cpu", True)
    net_b = Net(zoo.lenet(pad=2), 8, device="cpu", seed=(2, 3), minibatch_size=8)
    monkeypatch.setattr(Net, "device_path_on_cpu", False)
    comm = LocalOverlapComm(bucket_bytes=64 << 10, min_bucket_bytes=4 << 10)
    overlapped = StepEngine(net_b, opt, comm, use_graph=False)
    assert overlapped._overlapped() and len(comm._by_trigger) >= 2
    for eng in (plain, overlapped):
        eng.stepper.nesterov_lookahead(+1.0)
    for x, y in _batches(4, 8):
        for eng in (plain, overlapped):
            eng.feed(x, y)
            eng.step()
    assert torch.allclose(net_a.params, net_b.params, atol=1e-6)
    assert torch.equal(net_a.params16, net_b.params16) and float(net_b.grads.abs().sum()) == 0.0
