"""The CUDA execution path of the network container against its own CPU reference path (GPU only)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from rembrandt_b200.models import zoo
from rembrandt_b200.models.config import (Act, AffineCfg, Conv2dCfg, Data3dCfg, DropoutCfg, LrnCfg, ParamsInit,
                                          Pool2dCfg, PoolKind, SequentialOperatorConfig, SoftmaxKLLossCfg)
from rembrandt_b200.models.net import Net
from rembrandt_b200.ops import native_ops as K
from rembrandt_b200.optim.sgd import Momentum
from rembrandt_b200.optim.stepper import SgdStepper


def small_cfg(first_stride=1, hw=20):
    k = ParamsInit.kaiming()
    cfg = SequentialOperatorConfig().data3d(Data3dCfg((hw, hw, 3), normalize=True))
    if first_stride > 1:
        cfg.conv2d(Conv2dCfg(7, first_stride, 0, 24, Act.RECT, k), "conv1")
    else:
        cfg.conv2d(Conv2dCfg(3, 1, 1, 24, Act.RECT, k), "conv1")
    cfg.lrn(LrnCfg(5, 1e-2, 0.75, 2.0), "rnorm1")
    cfg.pool2d(Pool2dCfg(3, 2, 0, PoolKind.MAX), "pool1")
    cfg.conv2d(Conv2dCfg(3, 1, 1, 40, Act.IDENTITY, k), "conv2")
    cfg.pool2d(Pool2dCfg(2, 2, 0, PoolKind.AVERAGE, act=Act.RECT), "pool2")
    cfg.conv2d(Conv2dCfg(1, 1, 0, 64, Act.RECT, k), "conv3")
    cfg.affine(AffineCfg(48, Act.RECT, ParamsInit.xavier()), "fc1")
    cfg.dropout(DropoutCfg(0.0), "drop")
    cfg.affine(AffineCfg(10, Act.IDENTITY, ParamsInit.xavier()), "fc2")
    return cfg.softmax_kl_loss(SoftmaxKLLossCfg(10))


def run_pair(cfg_fn, batch, hw):
    g = Net(cfg_fn(), batch, device="cuda", seed=(3, 4))
    c = Net(cfg_fn(), batch, device="cpu", seed=(3, 4))
    assert torch.equal(g.params.cpu(), c.params.detach()), "same seed must give the same parameters"
    # the reference path must see the bf16-rounded weights the kernels use
    with torch.no_grad():
        c.params.copy_(g.params16.float().cpu())
    torch.manual_seed(0)
    x = torch.randint(0, 256, (batch, 3, hw, hw), dtype=torch.uint8)
    y = torch.randint(0, 10, (batch,))
    g.load_batch(x.cuda(), y.cuda().int())
    c.load_batch(x, y)
    g.forward(True)
    g.backward()
    c.forward(True)
    c.backward()
    torch.cuda.synchronize()
    assert K.read_status() == 0
    return g, c


@pytest.mark.parametrize("stride,hw", [(1, 20), (2, 31)])
def test_forward_backward_matches_reference_path(stride, hw):
    g, c = run_pair(lambda: small_cfg(stride, hw), 6, hw)
    gl, gc = g.read_stats()
    cl, cc = c.read_stats()
    assert abs(gl - cl) < 3e-2 * max(1.0, abs(cl)), (gl, cl)
    gg, cg = g.grads.cpu(), c.grads
    for seg in g.segs:
        a = gg[seg.offset: seg.offset + seg.numel]
        b = cg[seg.offset: seg.offset + seg.numel]
        # activations and deltas are bf16 on the device and fp32 in the reference path, so errors build up
        # layer by layer: bound the relative Frobenius error tightly and the worst element loosely
        scale = float(b.abs().max().clamp_min(1e-6))
        err = float((a - b).abs().max())
        rel = float((a - b).norm() / b.norm().clamp_min(1e-12))
        assert rel < 8e-2, f"{seg.name}: relative error {rel:.4g}"
        assert err < 0.15 * scale, f"{seg.name}: max err {err:.4g} vs scale {scale:.4g}"


def test_training_reduces_loss_and_matches_cpu_trajectory():
    cfg_fn = lambda: small_cfg(1, 20)
    g = Net(cfg_fn(), 16, device="cuda", seed=(5, 6))
    st = SgdStepper(g, Momentum.UPDATE, 0.9, 5e-4)
    torch.manual_seed(1)
    x = torch.randint(0, 256, (16, 3, 20, 20), dtype=torch.uint8).cuda()
    y = torch.randint(0, 10, (16,)).int().cuda()
    losses = []
    # a step size well inside the stable range: at 0.05 the trajectory spikes and where it ends depends on
    # rounding-level differences between kernel versions
    for t in range(60):
        g.load_batch(x, y)
        g.forward(True, t)
        g.backward()
        st.step(0.02)
        losses.append(g.read_stats()[0])
    assert min(losses[-5:]) < 0.75 * losses[0], losses
    assert float(g.grads.abs().max()) == 0.0, "the fused step must leave the gradients zeroed"
    assert K.read_status() == 0


def test_checkpoint_blob_round_trip_on_device():
    g = Net(zoo.lenet(), 8, device="cuda", seed=(7, 8))
    blob = g.encode_params()
    p0 = g.params.clone()
    g.params.zero_()
    g.decode_params(blob)
    assert torch.equal(g.params, p0)
    assert torch.equal(g.params16, p0.bfloat16())


def test_alexnet_and_nin_build_and_step():
    for fn, hw, b in ((zoo.alexnet, 227, 8), (zoo.nin, 224, 4)):
        net = Net(fn(scale=1.0 / 255.0), b, device="cuda")
        x = torch.randint(0, 256, (b, 3, hw, hw), dtype=torch.uint8).cuda()
        y = torch.randint(0, 1000, (b,)).int().cuda()
        net.load_batch(x, y)
        net.forward(True)
        net.backward()
        loss, _ = net.read_stats()
        assert 5.0 < loss < 9.0, loss   # ~ln(1000) at random initialisation
        assert torch.isfinite(net.grads).all()
        assert K.read_status() == 0
    assert Net(zoo.alexnet(), 2, device="cpu").params_len == 62378344


def _without_dropout(cfg):
    for op in cfg.hidden_ops:
        if isinstance(op.cfg, DropoutCfg):
            op.cfg.drop_ratio = 0.0     # the host path draws its masks from another generator
    return cfg


@pytest.mark.parametrize("model,hw", [("alexnet", 227), ("nin", 224)])
def test_flagship_gradients_match_the_reference_path_at_full_shapes(model, hw):
    """Every tile and tail configuration the benchmark shapes use (11x11 stride 4 over the space-to-depth input,
    5x5 pad 2, 3x3 pad 1, the 1x1 layers and the global pooling head of NIN, 9216x4096 weights) against the fp32
    host path, whole network, batch 4, per parameter segment."""
    fn = getattr(zoo, model)
    g = Net(_without_dropout(fn(scale=1.0 / 73.9)), 4, device="cuda", seed=(11, 12))
    c = Net(_without_dropout(fn(scale=1.0 / 73.9)), 4, device="cpu", seed=(11, 12))
    with torch.no_grad():
        c.params.copy_(g.params16.float().cpu())
    torch.manual_seed(3)
    x = torch.randint(0, 256, (4, 3, hw, hw), dtype=torch.uint8)
    y = torch.randint(0, 1000, (4,))
    g.load_batch(x.cuda(), y.cuda().int())
    c.load_batch(x, y)
    for net in (g, c):
        net.forward(True)
        net.backward()
    torch.cuda.synchronize()
    assert K.read_status() == 0
    gl, cl = g.read_stats()[0], c.read_stats()[0]
    assert abs(gl - cl) < 2e-2 * abs(cl), (gl, cl)
    gg, cg = g.grads.cpu(), c.grads
    rows = []
    for seg in g.segs:
        a = gg[seg.offset: seg.offset + seg.numel].double()
        b = cg[seg.offset: seg.offset + seg.numel].double()
        rel = float((a - b).norm() / b.norm().clamp_min(1e-30))
        cos = float((a * b).sum() / (a.norm() * b.norm()).clamp_min(1e-60))
        rows.append((seg.name, rel, cos))
    table = "\n".join(f"{n:12s} rel {r:.4f} cos {c:.5f}" for n, r, c in rows)
    print(f"{model}: gradient of every parameter segment, device against host path\n{table}")
    # Activations and deltas are bf16 on the device and fp32 on the host path, and eight layers of ReLU masks and
    # max-pool routing sit between the loss and the first layer: a unit that is barely on in one path and off in the
    # other moves a whole gradient entry. So the error grows towards the input; what a wrong tile, tail or stride
    # would do is different in kind (a segment that points somewhere else), and that is what the bounds catch.
    for name, rel, cos in rows:
        assert cos > 0.95 and rel < 0.32, f"{model} {name}: relative error {rel:.4g}, cosine {cos:.5f}\n{table}"
    head = rows[-2:]   # the classifier's weights and bias see no mask or pooling above them
    assert all(rel < 0.03 for _, rel, _ in head), table


@pytest.mark.parametrize("use_graph", [False, True])
def test_overlapped_local_update_equals_single_sweep(use_graph):
    """The per-bucket optimizer step launched from inside backward gives the same parameters (up to the
    summation order of split-K gradient reductions, which differs from run to run)."""
    from rembrandt_b200.api import default_opt, model_config
    from rembrandt_b200.engine import StepEngine
    from rembrandt_b200.parallel.comm import LocalOverlapComm, NullComm
    torch.manual_seed(3)
    xs = [torch.randint(0, 256, (32, 3, 32, 32), dtype=torch.uint8).pin_memory() for _ in range(4)]
    ys = [torch.randint(0, 10, (32,), dtype=torch.int32).pin_memory() for _ in range(4)]
    finals = []
    for comm in (NullComm(), LocalOverlapComm(bucket_bytes=64 << 10, min_bucket_bytes=16 << 10)):
        net = Net(model_config("cifar"), 32, device="cuda", seed=(9, 9))
        eng = StepEngine(net, default_opt(32, "null"), comm, use_graph=use_graph)
        for i in range(4):
            eng.feed(xs[i], ys[i])
            eng.step()
        eng.flush()
        eng.synchronize()
        finals.append((net.params.clone(), net.mom.clone(), net.params16.clone()))
        assert float(net.grads.abs().max()) == 0.0
    for a, b in zip(*finals):
        assert torch.allclose(a.float(), b.float(), rtol=1e-3, atol=2e-4)
    assert K.read_status() == 0


def test_residual_network_matches_reference_path_and_averages_statistics():
    """Batch-normalised residual blocks (identity + strided projection) on the device against the CPU path:
    loss, gradients, and the running statistics after two steps (factor 1 at step 0, then 0.1)."""
    from rembrandt_b200.models.config import (BNormConv2dCfg, ProjStackResConv2dCfg, StackResConv2dCfg)
    k = ParamsInit.kaiming()

    def cfg_fn():
        return (SequentialOperatorConfig().data3d(Data3dCfg((16, 16, 3), normalize=True))
                .bnorm_conv2d(BNormConv2dCfg(3, 1, 1, 32, Act.RECT, k), "stem")
                .stack_res_conv2d(StackResConv2dCfg(k), "res1")
                .proj_stack_res_conv2d(ProjStackResConv2dCfg(64, None, k), "res2")
                .pool2d(Pool2dCfg(8, 1, 0, PoolKind.AVERAGE), "gap")
                .affine(AffineCfg(10, Act.IDENTITY, ParamsInit.xavier()), "fc")
                .softmax_kl_loss(SoftmaxKLLossCfg(10)))

    g = Net(cfg_fn(), 8, device="cuda", seed=(3, 4))
    c = Net(cfg_fn(), 8, device="cpu", seed=(3, 4))
    with torch.no_grad():
        c.params.copy_(g.params16.float().cpu())
    torch.manual_seed(0)
    for step in range(2):
        x = torch.randint(0, 256, (8, 3, 16, 16), dtype=torch.uint8)
        y = torch.randint(0, 10, (8,))
        g.load_batch(x.cuda(), y.cuda().int())
        c.load_batch(x, y)
        g.reset_grads()
        c.reset_grads()
        g.forward(True, step)
        g.backward()
        c.forward(True, step)
        c.backward()
        torch.cuda.synchronize()
        assert K.read_status() == 0
        gl, cl = g.read_stats()[0], c.read_stats()[0]
        assert abs(gl - cl) < 5e-2 * max(1.0, abs(cl)), (step, gl, cl)
    gg, cg = g.grads.cpu(), c.grads
    for seg in g.segs:
        a, b = gg[seg.offset: seg.offset + seg.numel], cg[seg.offset: seg.offset + seg.numel]
        if not seg.trainable:
            continue
        # bf16 activations and deltas through five normalised convolutions: the error of the deepest layer's
        # gradient reaches ~13 % in Frobenius norm; a wrong kernel gives order-one errors
        rel = float((a - b).norm() / b.norm().clamp_min(1e-12))
        assert rel < 0.2, f"{seg.name}: relative error {rel:.4g}"
    # running mean / variance of the stem after step 0 (factor 1) and step 1 (factor 0.1)
    stem_g, stem_c = g.hidden_ops[0].u, c.hidden_ops[0].u
    for seg_g, seg_c in ((stem_g.seg_rm, stem_c.seg_rm), (stem_g.seg_rv, stem_c.seg_rv)):
        a, b = g.seg_view(seg_g).float().cpu(), c.seg_view(seg_c).detach()
        assert torch.allclose(a, b, rtol=5e-2, atol=5e-3), float((a - b).abs().max())


def test_strided_normalised_stem_runs_on_the_space_to_depth_input():
    """A 7 x 7 stride-2 pad-3 batch-normalised first layer (the ResNet stem) against the host path: the device runs
    it as a 4 x 4 stride-1 convolution on the space-to-depth'd image, with the padding absorbed by the input kernel."""
    from rembrandt_b200.models.config import BNormConv2dCfg, StackResConv2dCfg
    k = ParamsInit.kaiming()

    def cfg_fn():
        return (SequentialOperatorConfig().data3d(Data3dCfg((38, 38, 3), normalize=True))
                .bnorm_conv2d(BNormConv2dCfg(7, 2, 3, 32, Act.RECT, k), "stem")
                .pool2d(Pool2dCfg(3, 2, 1, PoolKind.MAX), "pool1")
                .stack_res_conv2d(StackResConv2dCfg(k), "res1")
                .pool2d(Pool2dCfg(10, 1, 0, PoolKind.AVERAGE), "gap")
                .affine(AffineCfg(10, Act.IDENTITY, ParamsInit.xavier()), "fc")
                .softmax_kl_loss(SoftmaxKLLossCfg(10)))

    g = Net(cfg_fn(), 8, device="cuda", seed=(5, 6))
    c = Net(cfg_fn(), 8, device="cpu", seed=(5, 6))
    assert g.hidden_ops[0].u.s2d is not None and g.input_op.mode == "s2d"
    assert torch.equal(g.params.cpu(), c.params.detach())
    with torch.no_grad():
        c.params.copy_(g.params16.float().cpu())
    torch.manual_seed(2)
    x = torch.randint(0, 256, (8, 3, 38, 38), dtype=torch.uint8)
    y = torch.randint(0, 10, (8,))
    g.load_batch(x.cuda(), y.cuda().int())
    c.load_batch(x, y)
    for net in (g, c):
        net.forward(True)
        net.backward()
    torch.cuda.synchronize()
    assert K.read_status() == 0
    gl, cl = g.read_stats()[0], c.read_stats()[0]
    assert abs(gl - cl) < 5e-2 * max(1.0, abs(cl)), (gl, cl)
    gg, cg = g.grads.cpu(), c.grads
    for seg in g.segs:
        if not seg.trainable:
            continue
        a, b = gg[seg.offset: seg.offset + seg.numel], cg[seg.offset: seg.offset + seg.numel]
        rel = float((a - b).norm() / b.norm().clamp_min(1e-12))
        assert rel < 0.15, f"{seg.name}: relative error {rel:.4g}"
    # a checkpoint written from the rearranged filter reads back as the 7 x 7 filter of the host path
    blob_g = g.encode_params()
    fresh = Net(cfg_fn(), 8, device="cpu", seed=(5, 6))           # the same seed: the same (unrounded) parameters
    c2 = Net(cfg_fn(), 8, device="cpu", seed=(9, 9))
    c2.decode_params(blob_g)
    for seg in c2.segs:
        if not seg.trainable:
            continue                     # the running statistics moved with the training pass above
        a = c2.params.detach()[seg.offset: seg.offset + seg.numel]
        b = fresh.params.detach()[seg.offset: seg.offset + seg.numel]
        assert torch.allclose(a, b, atol=1e-6), seg.name
    assert len(blob_g) == len(fresh.encode_params())

