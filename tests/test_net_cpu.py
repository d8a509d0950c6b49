"""The reference (CPU) execution path against an independently written torch model, the internal parameter
layouts against the reference's blob layout, and checkpoint / resume (CPU)."""
import os

import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from rembrandt_b200.models import zoo
from rembrandt_b200.models.config import (Act, AffineCfg, BNormConv2dCfg, Conv2dCfg, Data3dCfg, MimicAffineCfg,
                                          ParamsInit, Pool2dCfg,
                                          PoolKind, ProjStackResConv2dCfg, SequentialOperatorConfig, SoftmaxKLLossCfg,
                                          StackResConv2dCfg)
from rembrandt_b200.models.net import Net
from rembrandt_b200.ops import layout
from rembrandt_b200.utils import blob, checkpoint as ckpt


class TorchLeNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.c1, self.c2 = nn.Conv2d(1, 20, 5), nn.Conv2d(20, 50, 5)
        self.f1, self.f2 = nn.Linear(800, 500), nn.Linear(500, 10)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.c1(x)), 2)
        x = F.max_pool2d(F.relu(self.c2(x)), 2)
        return self.f2(F.relu(self.f1(x.flatten(1))))


def load_blob_into_torch(model, blob_bytes):
    """The blob stores, per layer, weights as (fan_in, out) first-dimension-fastest = torch's own memory order."""
    recs, _ = blob.decode_records(blob_bytes)
    mods = [model.c1, model.c2, model.f1, model.f2]
    for m, (w, wd, _), (b, bd, _) in zip(mods, recs[0::2], recs[1::2]):
        assert wd == (m.weight[0].numel(), m.weight.shape[0]) and bd == (1, m.bias.numel())
        with torch.no_grad():
            m.weight.copy_(torch.from_numpy(w).reshape(m.weight.shape))
            m.bias.copy_(torch.from_numpy(b))


def test_lenet_matches_an_independent_torch_model_through_the_blob():
    net = Net(zoo.lenet(), 5, device="cpu", seed=(1, 2))
    with torch.no_grad():
        for op in net.hidden_ops:      # non-zero biases make the check stricter
            if op.has_params:
                op.view(op.seg_b).normal_(0, 0.1)
    model = TorchLeNet()
    load_blob_into_torch(model, net.encode_params())
    x = torch.randint(0, 256, (5, 1, 28, 28), dtype=torch.uint8)
    y = torch.randint(0, 10, (5,))
    net.load_batch(x, y)
    net.forward(True)
    net.backward()
    loss, _ = net.read_stats()
    ref = F.cross_entropy(model(x.float() / 255.0), y, reduction="sum") / 5
    ref.backward()
    assert abs(loss - float(ref)) < 1e-5
    # gradients, compared in the reference layout
    conv1 = net.hidden_ops[0]
    g = layout.conv_weight_from_internal(conv1.view(conv1.seg_w, "grads"), 1, 5, 5)
    assert torch.allclose(g, model.c1.weight.grad, atol=1e-6)
    fc1 = net.hidden_ops[4]
    gf = fc1._w_ref(fc1.view(fc1.seg_w, "grads"))
    assert torch.allclose(gf, model.f1.weight.grad, atol=1e-6)


def test_strided_first_layer_reference_path_equals_plain_conv():
    cfg = (SequentialOperatorConfig().data3d(Data3dCfg((23, 23, 3), normalize=True))
           .conv2d(Conv2dCfg(7, 2, 0, 8, Act.RECT, ParamsInit.kaiming()), "conv1")
           .pool2d(Pool2dCfg(9, 1, 0, PoolKind.AVERAGE), "gap")
           .affine(AffineCfg(4, Act.IDENTITY, ParamsInit.xavier()), "fc")
           .softmax_kl_loss(SoftmaxKLLossCfg(4)))
    net = Net(cfg, 3, device="cpu", seed=(4, 4))
    conv = net.hidden_ops[0]
    assert conv.s2d                                                    # stored in space-to-depth layout ...
    recs, _ = blob.decode_records(net.encode_params())
    assert recs[0][1] == (7 * 7 * 3, 8)                                # ... but written as a 7x7x3 filter bank
    w = torch.from_numpy(recs[0][0]).reshape(8, 3, 7, 7)
    x = torch.randint(0, 256, (3, 3, 23, 23), dtype=torch.uint8)
    out = conv.ref_forward(x.float() / 255.0, False, 0)
    assert torch.allclose(out, torch.relu(F.conv2d(x.float() / 255.0, w, None, stride=2)), atol=1e-5)


def test_params_blob_round_trip_is_byte_exact_for_every_template():
    for fn in (zoo.lenet, lambda: zoo.cifar_krizh26(augment=False), zoo.resnet20_cifar, zoo.mnist_fc2):
        a = Net(fn(), 2, device="cpu", seed=(5, 6))
        b = Net(fn(), 2, device="cpu", seed=(7, 8))
        raw = a.encode_params()
        assert raw != b.encode_params()
        b.decode_params(raw)
        assert b.encode_params() == raw
        assert torch.equal(a.params.detach(), b.params.detach())


def test_state_blob_carries_momentum():
    a = Net(zoo.lenet(), 2, device="cpu", seed=(5, 6))
    with torch.no_grad():
        a.mom.normal_()
        # padded entries of the momentum never become non-zero in training
        for op in a.hidden_ops:
            for s in op.segs:
                pass
    b = Net(zoo.lenet(), 2, device="cpu", seed=(9, 9))
    b.decode_state(a.encode_state())
    assert torch.equal(a.params.detach(), b.params.detach())
    for op_a, op_b in zip(a.hidden_ops, b.hidden_ops):
        if op_a.has_params:
            assert op_a.encode_params()[0][0].equal(op_b.encode_params()[0][0])


def test_residual_blocks_run_and_have_resnet_parameter_layout():
    k = ParamsInit.kaiming()
    cfg = (SequentialOperatorConfig().data3d(Data3dCfg((16, 16, 3), normalize=True))
           .bnorm_conv2d(BNormConv2dCfg(3, 1, 1, 8, Act.RECT, k), "stem")
           .stack_res_conv2d(StackResConv2dCfg(k), "res1")
           .proj_stack_res_conv2d(ProjStackResConv2dCfg(16, None, k), "res2")
           .pool2d(Pool2dCfg(8, 1, 0, PoolKind.AVERAGE), "gap")
           .affine(AffineCfg(5, Act.IDENTITY, ParamsInit.xavier()), "fc")
           .softmax_kl_loss(SoftmaxKLLossCfg(5)))
    net = Net(cfg, 4, device="cpu", seed=(2, 3))
    # W + 4*Cout per normalised conv: stem 1, identity block 2, projection block 3
    expect = (3 * 9 * 8 + 32) + 2 * (8 * 9 * 8 + 32) + (8 * 9 * 16 + 64) + (16 * 9 * 16 + 64) + (8 * 16 + 64) + 16 * 5 + 5
    assert net.params_len == expect
    assert net.ops[3].out_hwc == (8, 8, 16)                            # projection halves the spatial size
    x = torch.randint(0, 256, (4, 3, 16, 16), dtype=torch.uint8)
    y = torch.randint(0, 5, (4,))
    net.load_batch(x, y)
    net.forward(True)
    net.backward()
    assert torch.isfinite(net.grads).all() and float(net.grads.abs().sum()) > 0
    stem = net.hidden_ops[0].u
    assert float(net.seg_view(stem.seg_rm).abs().sum()) > 0            # running statistics were updated
    assert float(net.seg_view(stem.seg_rm, "grads").abs().sum()) == 0  # and never receive gradients
    assert not stem.seg_g.decay and stem.seg_w.decay                    # L2 skips the normalisation parameters


def test_checkpoint_directory_layout_and_resume(tmp_path):
    d = str(tmp_path / "ck")
    net = Net(zoo.lenet(), 2, device="cpu", seed=(1, 1))
    assert ckpt.can_rollback(d) is None
    ckpt.checkpoint_state(net, d, rank=0)
    p100 = ckpt.checkpoint_params(net, 100, d)
    with torch.no_grad():
        net.params.add_(1.0)
    ckpt.checkpoint_params(net, 200, d)
    assert sorted(os.listdir(d)) == ["checkpoint", "checkpoint.0", "params.latest.blob", "params.t_100.blob",
                                     "params.t_200.blob", "state.latest.blob.0"]
    assert open(os.path.join(d, "checkpoint")).read() == "200\n"
    assert open(os.path.join(d, "checkpoint.0")).read() == "100\n"
    assert os.readlink(os.path.join(d, "params.latest.blob")) == "params.t_200.blob"
    assert ckpt.can_rollback(d, 0) == 200 and ckpt.can_rollback(d, 1) is None
    other = Net(zoo.lenet(), 2, device="cpu", seed=(3, 3))
    assert ckpt.rollback_params(other, d, 100) == 100
    assert other.encode_params() == open(p100, "rb").read()
    assert ckpt.rollback_params(other, d) == 200
    with pytest.raises(ValueError):
        ckpt.rollback_params(other, d, 300)
    # a truncated state blob is reported, not silently accepted
    path = os.path.join(d, "state.latest.blob.0")
    raw = open(path, "rb").read()
    open(path, "wb").write(raw[: len(raw) // 2])
    with pytest.raises(blob.BlobError):
        ckpt.rollback_state(other, d, 0)


def test_gen1_binary_checkpoint_index_is_readable(tmp_path):
    import struct
    (tmp_path / "checkpoint").write_bytes(struct.pack("<Q", 4242))
    assert ckpt.latest_iteration(str(tmp_path)) == 4242


def test_reshape_conv_out_channels():
    net = Net(zoo.lenet(), 2, device="cpu", seed=(1, 1))
    raw = net.encode_params()
    small = ckpt.reshape_conv_out_channels(raw, {0: 12})
    recs, _ = blob.decode_records(small)
    full, _ = blob.decode_records(raw)
    assert recs[0][1] == (25, 12) and recs[1][1] == (1, 12)
    assert np.array_equal(recs[0][0], full[0][0][: 25 * 12])
    assert recs[2][1] == full[2][1]


def test_masked_and_multi_head_softmax_reference_path():
    """Admissibility masks renormalise over the allowed categories; look-ahead heads sum their losses."""
    import torch.nn.functional as F
    from rembrandt_b200.models import config as C
    from rembrandt_b200.models.net import Net
    cfg = C.SequentialOperatorConfig().data3d(C.Data3dCfg((4, 4, 2)))
    cfg.affine(C.AffineCfg(12)).multi_softmax_kl_loss(C.MultiSoftmaxKLLossCfg(6, 2))
    net = Net(cfg, 3, device="cpu")
    x = torch.randint(0, 256, (3, 2, 4, 4), dtype=torch.uint8)
    labels = torch.tensor([[1, 2], [0, -1], [5, 3]])
    mask = torch.ones(3, 2, 6, dtype=torch.bool)
    mask[0, 0, 4] = False
    mask[2, 1, 0] = False
    net.loss_op.load_mask(mask)
    net.load_batch(x, labels)
    net.forward(True)
    net.backward()
    loss, correct = net.read_stats()
    logits = net._cpu_logits.reshape(3, 2, 6).masked_fill(~mask, float("-inf"))
    want = 0.0
    for b in range(3):
        for l in range(2):
            if labels[b, l] >= 0:
                want += float(F.cross_entropy(logits[b, l][None], labels[b, l][None])) / 3
    assert abs(loss - want) < 1e-4 * max(1.0, abs(want))
    assert correct == int((logits[:, 0].argmax(1) == labels[:, 0]).sum())
    assert torch.isfinite(net.grads).all()


@pytest.mark.parametrize("kind", ["logistic", "l2"])
def test_pointwise_heads_reference_path(kind):
    from rembrandt_b200.models import config as C
    from rembrandt_b200.models.net import Net
    cfg = C.SequentialOperatorConfig().data3d(C.Data3dCfg((4, 4, 2)))
    cfg.affine(C.AffineCfg(3)).pointwise_loss(C.PointwiseLossCfg(3, kind))
    net = Net(cfg, 5, device="cpu")
    x = torch.randint(0, 256, (5, 2, 4, 4), dtype=torch.uint8)
    t = (torch.rand(5, 3) > 0.5).float() if kind == "logistic" else torch.randn(5, 3)
    net.load_batch(x, t)
    net.forward(True)
    net.backward()
    loss, _ = net.read_stats()
    z = net._cpu_logits.flatten(1)
    if kind == "logistic":
        want = torch.nn.functional.binary_cross_entropy_with_logits(z, t, reduction="sum") / 5
    else:
        want = 0.5 * ((z - t) ** 2).sum() / 5
    assert abs(loss - float(want)) < 1e-4 * max(1.0, abs(float(want)))
    assert float(net.grads.abs().sum()) > 0


@pytest.mark.parametrize("kind", ["softmax_ind", "antilogistic_kl", "antilogistic_ind"])
def test_categorical_objective_heads_reference_path(kind):
    """Softmax indicator and the two antilogistic heads against the formulas written out by hand."""
    from rembrandt_b200.models import config as C
    from rembrandt_b200.models.net import Net
    cfg = C.SequentialOperatorConfig().data3d(C.Data3dCfg((4, 4, 2), normalize=True))
    cfg.affine(C.AffineCfg(6)).categorical_obj_loss(C.CategoricalObjLossCfg(6, kind))
    net = Net(cfg, 5, device="cpu")
    if kind != "softmax_ind":
        with torch.no_grad():
            net.params.add_(0.3)      # mostly positive scores, as the antilogistic heads expect
    x = torch.randint(0, 256, (5, 2, 4, 4), dtype=torch.uint8)
    y = torch.tensor([0, 3, 5, 1, 2])
    net.load_batch(x, y)
    net.forward(True)
    net.backward()
    loss, _ = net.read_stats()
    z = net._cpu_logits.flatten(1)
    if kind == "softmax_ind":
        v = torch.softmax(z, 1)
    else:
        v = z.clamp_min(0) / z.clamp_min(0).sum(1, keepdim=True).clamp_min(1e-6)
    mass = v[torch.arange(5), y]
    want = (-torch.log(mass.clamp_min(1e-6)) if kind == "antilogistic_kl" else 1 - mass).sum() / 5
    assert abs(loss - float(want)) < 1e-5 * max(1.0, abs(float(want)))
    assert float(net.grads.abs().sum()) > 0
    if kind == "softmax_ind":
        # a weight per category in place of the label: the marginalised form
        net.loss_op.set_target_weights([0.5, 0.0, 0.25, 0.0, 0.0, 0.25])
        net.load_batch(x, y)
        net.forward(True)
        loss2, _ = net.read_stats()
        tw = torch.tensor([0.5, 0.0, 0.25, 0.0, 0.0, 0.25])
        assert abs(loss2 - float((1 - (v * tw).sum(1)).sum() / 5)) < 1e-5


def test_softmax_head_sampling_respects_mask_and_temperature():
    from rembrandt_b200.models import config as C
    from rembrandt_b200.models.net import Net
    cfg = C.SequentialOperatorConfig().data3d(C.Data3dCfg((4, 4, 1)))
    cfg.affine(C.AffineCfg(6)).softmax_kl_loss(C.SoftmaxKLLossCfg(6))
    net = Net(cfg, 64, device="cpu")
    x = torch.randint(0, 256, (64, 1, 4, 4), dtype=torch.uint8)
    mask = torch.ones(64, 6, dtype=torch.bool)
    mask[:, 2] = False
    net.loss_op.load_mask(mask)
    net.load_batch(x, torch.zeros(64, dtype=torch.long))
    with torch.no_grad():
        net.forward(False)
    g = torch.Generator().manual_seed(0)
    draws = torch.stack([net.loss_op.sample_categories(1.0, g) for _ in range(20)])
    assert not (draws == 2).any(), "a masked category must never be drawn"
    assert draws.unique().numel() > 1
    # a very low temperature draws the arg-max among the admissible categories
    cold = net.loss_op.sample_categories(1e-4, g)
    best = net._cpu_logits.flatten(1).masked_fill(~mask, float("-inf")).argmax(1)
    assert torch.equal(cold, best)


@pytest.mark.parametrize("act,fn", [(Act.LOGISTIC, torch.sigmoid), (Act.TANH, torch.tanh),
                                    (Act.BOUNDED_RECT, lambda v: v.clamp(0.0, 6.0))])
def test_smooth_and_clipped_activations_reference_path(act, fn):
    cfg = (SequentialOperatorConfig().data3d(Data3dCfg((8, 8, 3), normalize=True))
           .conv2d(Conv2dCfg(3, 1, 1, 6, act, ParamsInit.kaiming()), "conv1")
           .affine(AffineCfg(5, act, ParamsInit.xavier()), "fc1")
           .affine(AffineCfg(4, Act.IDENTITY, ParamsInit.xavier()), "fc2")
           .softmax_kl_loss(SoftmaxKLLossCfg(4)))
    net = Net(cfg, 2, device="cpu", seed=(1, 2))
    conv, fc1, _ = net.hidden_ops
    recs, _ = blob.decode_records(net.encode_params())
    w = torch.from_numpy(recs[0][0]).reshape(6, 3, 3, 3)
    b = torch.from_numpy(recs[1][0]).reshape(6)
    x = torch.rand(2, 3, 8, 8) * 4 - 2
    out = conv.ref_forward(x, False, 0)
    assert torch.allclose(out, fn(F.conv2d(x, w, b, padding=1)), atol=1e-5)
    w1 = torch.from_numpy(recs[2][0]).reshape(5, -1)
    b1 = torch.from_numpy(recs[3][0]).reshape(5)
    assert torch.allclose(fc1.ref_forward(out, False, 0).flatten(1), fn(out.flatten(1) @ w1.t() + b1), atol=1e-5)
    assert Act.parse("sigmoid") is Act.LOGISTIC and Act.parse("bounded_rect") is Act.BOUNDED_RECT


def test_mimic_affine_expands_into_a_low_rank_chain():
    cfg = (SequentialOperatorConfig().data3d(Data3dCfg((6, 6, 2), normalize=True))
           .mimic_affine(MimicAffineCfg(bottleneck_rank=5, hidden_channels=12, out_channels=4), "m")
           .softmax_kl_loss(SoftmaxKLLossCfg(4)))
    net = Net(cfg, 3, device="cpu", seed=(7, 8))
    assert [op.name for op in net.hidden_ops] == ["m.down", "m.up", "m.out"]
    recs, _ = blob.decode_records(net.encode_params())
    # downsample and upsample carry no bias: three weight records and one bias record, as in the reference's layer
    assert [r[1] for r in recs] == [(72, 5), (5, 12), (12, 4), (1, 4)]
    wd, wu, wo = (torch.from_numpy(recs[i][0]).reshape(recs[i][1][1], recs[i][1][0]) for i in range(3))
    b = torch.from_numpy(recs[3][0]).reshape(-1)
    x = torch.rand(3, 2, 6, 6)
    y = x
    for op in net.hidden_ops:
        y = op.ref_forward(y, False, 0)
    want = torch.relu(x.flatten(1) @ wd.t() @ wu.t()) @ wo.t() + b
    assert torch.allclose(y.flatten(1), want, atol=1e-5)
    other = Net(cfg, 3, device="cpu", seed=(9, 9))
    other.decode_params(net.encode_params())
    assert torch.equal(other.params, net.params)


def test_loss_head_dense_row_of_a_spatial_producer():
    """The device path hands the loss kernel one dense row per sample in the reference's order (channel slowest);
    the copies in and out of that row are plain strided copies, checked here on CPU tensors."""
    import types
    from rembrandt_b200.models.operators import SoftmaxKLLossOp
    from rembrandt_b200.ops.native_ops import pad_channels
    n, h, w, c, cp = 3, 5, 4, 2, 32
    op = object.__new__(SoftmaxKLLossOp)
    op.net = types.SimpleNamespace(batch=n, is_cuda=True, training_capable=True, device="cpu")
    nchw = torch.randn(n, c, h, w).bfloat16()
    out = torch.zeros(n, h, w, cp, dtype=torch.bfloat16)
    out[..., :c] = nchw.permute(0, 2, 3, 1)
    op.prev = types.SimpleNamespace(out=out, dout=torch.zeros_like(out), out_hwc=(h, w, c), out_cp=cp)
    op._setup_flat()
    assert op.spatial and op.ld == pad_channels(h * w * c)
    op._alloc_flat()
    logits, dbuf = op._logits()
    assert torch.equal(logits[:, : h * w * c], nchw.flatten(1)) and torch.all(logits[:, h * w * c:] == 0)
    dbuf.copy_(torch.randn_like(dbuf.float()).bfloat16())
    op._scatter_delta()
    assert torch.equal(op.prev.dout[..., :c].permute(0, 3, 1, 2).flatten(1), dbuf[:, : h * w * c])
    assert torch.all(op.prev.dout[..., c:] == 0)
    # a 1 x 1 producer is used in place
    op.prev = types.SimpleNamespace(out=out[:, :1, :1], dout=None, out_hwc=(1, 1, 10), out_cp=cp)
    op._setup_flat()
    assert not op.spatial and op.ld == cp and op._logits()[0] is op.prev.out


def test_residual_convolution_and_scaled_logistic_reference_path():
    from rembrandt_b200.models.config import ResConv2dCfg
    cfg = (SequentialOperatorConfig().data3d(Data3dCfg((8, 8, 3), normalize=True))
           .conv2d(Conv2dCfg(3, 1, 1, 6, Act.RECT, ParamsInit.kaiming()), "stem")
           .res_conv2d(ResConv2dCfg(3, Act.RECT), "res1")
           .res_conv2d(ResConv2dCfg(5, Act.SCALED_LOGISTIC, act_param=2.0), "res2")
           .pool2d(Pool2dCfg(8, 1, 0, PoolKind.AVERAGE), "gap")
           .affine(AffineCfg(4, Act.IDENTITY, ParamsInit.xavier()), "fc")
           .softmax_kl_loss(SoftmaxKLLossCfg(4)))
    net = Net(cfg, 2, device="cpu", seed=(1, 2))
    stem, res1, res2 = net.hidden_ops[:3]
    assert res1.out_hwc == (8, 8, 6) and res2.cfg.conv_pad == 2
    recs, _ = blob.decode_records(net.encode_params())
    assert [r[1] for r in recs[:6]] == [(27, 6), (1, 6), (54, 6), (1, 6), (150, 6), (1, 6)]
    x = torch.rand(2, 3, 8, 8)
    a = stem.ref_forward(x, False, 0)
    w1 = torch.from_numpy(recs[2][0]).reshape(6, 6, 3, 3)
    b = res1.ref_forward(a, False, 0)
    assert torch.allclose(b, torch.relu(F.conv2d(a, w1, None, padding=1) + a), atol=1e-5)
    w2 = torch.from_numpy(recs[4][0]).reshape(6, 6, 5, 5)
    c = res2.ref_forward(b, False, 0)
    assert torch.allclose(c, torch.sigmoid(2.0 * (F.conv2d(b, w2, None, padding=2) + b)), atol=1e-5)
    net.load_batch((x * 255).to(torch.uint8), torch.tensor([1, 3]))
    net.forward(True)
    net.backward()
    assert float(net.grads.abs().sum()) > 0
    with pytest.raises(ValueError):
        Net(SequentialOperatorConfig().data3d(Data3dCfg((8, 8, 3))).res_conv2d(ResConv2dCfg(4), "bad")
            .softmax_kl_loss(SoftmaxKLLossCfg(4)), 2, device="cpu")


def test_lighting_noise_on_the_reference_path():
    from rembrandt_b200.models.config import Preproc
    vecs = [0.5, 0.1, 0.0, 0.2, 0.7, 0.0, 0.1, 0.3, 1.0]
    cfg = (SequentialOperatorConfig()
           .data3d(Data3dCfg((6, 6, 3), normalize=True,
                             preprocs=[Preproc("pca_noise", std=0.1, eigenvalues=[0.2, 0.02, 0.004], eigenvectors=vecs)]))
           .affine(AffineCfg(4, Act.IDENTITY, ParamsInit.xavier()), "fc").softmax_kl_loss(SoftmaxKLLossCfg(4)))
    net = Net(cfg, 3, device="cpu", seed=(1, 2))
    x = torch.randint(0, 256, (3, 3, 6, 6), dtype=torch.uint8)
    clean = net.input_op.ref_forward(x, False, 0)
    noisy = net.input_op.ref_forward(x, True, 0)
    shift = noisy - clean
    # one shift per sample and channel, the same for every pixel; it lies in the span of the scaled eigenvectors
    assert torch.allclose(shift, shift[:, :, :1, :1].expand_as(shift), atol=1e-6) and float(shift.abs().max()) > 0
    basis = torch.tensor(vecs).reshape(3, 3) * torch.tensor([0.2, 0.02, 0.004])
    alpha = torch.linalg.solve(basis, shift[:, :, 0, 0].t())
    assert float(alpha.abs().max()) < 1.0                 # alphas of a N(0, 0.1) draw


@pytest.mark.parametrize("per_batch", [True, False])
def test_crop_and_flip_draws_per_batch_or_per_sample_on_the_reference_path(per_batch):
    from rembrandt_b200.models.config import Preproc
    pre = [Preproc("crop", crop_width=5, crop_height=5), Preproc("flip_x")]
    cfg = (SequentialOperatorConfig().data3d(Data3dCfg((12, 12, 1), preprocs=pre, per_batch_draws=per_batch))
           .affine(AffineCfg(4, Act.IDENTITY, ParamsInit.xavier()), "fc").softmax_kl_loss(SoftmaxKLLossCfg(4)))
    net = Net(cfg, 16, device="cpu", seed=(1, 2))
    # every pixel encodes its own position, so the crop window and the flip of each sample can be read back
    img = (torch.arange(12).reshape(1, 12) + 12 * torch.arange(12).reshape(12, 1)).to(torch.uint8)
    x = img.reshape(1, 1, 12, 12).repeat(16, 1, 1, 1)
    out = net.input_op.ref_forward(x, True, 0)
    assert out.shape == (16, 1, 5, 5)
    corners = {(int(o[0, 0, 0]), int(o[0, 0, 4])) for o in out}
    assert (len(corners) == 1) == per_batch, corners
    for o in out:
        row = o[0, 0].long() % 12
        assert torch.equal(row, torch.arange(int(row[0]), int(row[0]) + 5)) or \
            torch.equal(row, torch.arange(int(row[0]), int(row[0]) - 5, -1))
