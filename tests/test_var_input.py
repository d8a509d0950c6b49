"""Variable-size input operator: bicubic (Catmull-Rom) rescale + crop + flip, CPU restatement and CUDA kernel."""
import pytest
import torch

from rembrandt_b200.models import config as C
from rembrandt_b200.models.net import Net
from rembrandt_b200.models.operators import VarDataOp


def _cubic_keys(img, rh, rw, a=-0.5):
    """Independent cubic-convolution resize (Keys kernel with parameter a; a = -0.5 is Catmull-Rom)."""
    c, h, w = img.shape

    def taps(n, src):
        f = (torch.arange(n).float() + 0.5) * (torch.tensor(float(src)) / torch.tensor(float(n))) - 0.5
        fl = torch.floor(f)
        t = f - fl

        def k(x):
            x = x.abs()
            return torch.where(x <= 1, (a + 2) * x ** 3 - (a + 3) * x ** 2 + 1,
                               torch.where(x < 2, a * x ** 3 - 5 * a * x ** 2 + 8 * a * x - 4 * a, torch.zeros_like(x)))
        wts = torch.stack([k(t + 1), k(t), k(1 - t), k(2 - t)], 1)
        idx = (fl.long()[:, None] - 1 + torch.arange(4)[None]).clamp(0, src - 1)
        return wts, idx

    wx, xi = taps(rw, w)
    wy, yi = taps(rh, h)
    out = torch.zeros(c, rh, rw)
    for j in range(4):
        for k_ in range(4):
            out += wy[:, j][None, :, None] * wx[:, k_][None, None, :] * img[:, yi[:, j]][:, :, xi[:, k_]]
    return out.clamp(0, 255)


def test_ref_sample_identity_flip_and_resize():
    torch.manual_seed(0)
    img = torch.randint(0, 256, (3, 40, 60), dtype=torch.uint8)
    assert torch.equal(VarDataOp.ref_sample(img, 0, 5, 3, False, 32, 32), img[:, 3:35, 5:37].float())
    assert torch.equal(VarDataOp.ref_sample(img, 0, 5, 3, True, 32, 32), img[:, 3:35, 5:37].float().flip(-1))
    # shorter side (height 40) -> 80: full rescaled image is 80 x 120
    assert VarDataOp.scaled_dims(60, 40, 80) == (120, 80)
    full = VarDataOp.ref_sample(img, 80, 0, 0, False, 120, 80)
    assert torch.allclose(full, _cubic_keys(img.float(), 80, 120), atol=1e-3)
    win = VarDataOp.ref_sample(img, 80, 17, 9, False, 64, 48)
    assert torch.allclose(win, full[:, 9:57, 17:81], atol=1e-4)
    # a window that leaves the rescaled image reads zeros there
    out = VarDataOp.ref_sample(img, 20, -3, -2, False, 36, 24)
    assert torch.all(out[:, :2] == 0) and torch.all(out[:, :, :3] == 0) and torch.all(out[:, 22:] == 0)


def _var_cfg(crop, lo, hi, flip=True, stride=1, mean=(0.4, 0.5, 0.6)):
    pre = [C.Preproc("scale_bicubic", lower=lo, upper=hi), C.Preproc("crop", crop_width=crop, crop_height=crop)]
    if flip:
        pre.append(C.Preproc("flip_x"))
    cfg = C.SequentialOperatorConfig()
    cfg.var_data3d(C.Data3dCfg((96, 96, 3), normalize=True, preprocs=pre, max_dims=(96, 96, 3), channel_mean=mean))
    cfg.conv2d(C.Conv2dCfg(5 if stride > 1 else 3, stride, 0 if stride > 1 else 1, 16))
    cfg.pool2d(C.Pool2dCfg(2, 2))
    cfg.affine(C.AffineCfg(10))
    cfg.softmax_kl_loss(C.SoftmaxKLLossCfg(10))
    return cfg


def _batch(n, seed=3):
    g = torch.Generator().manual_seed(seed)
    dims = [(50, 70), (96, 64), (33, 33), (80, 96), (64, 41), (96, 96), (40, 90), (72, 56)]
    return [torch.randint(0, 256, (3, h, w), dtype=torch.uint8, generator=g) for (w, h) in dims[:n]]


def test_var_data_net_cpu_steps():
    net = Net(_var_cfg(32, 36, 48), 4, device="cpu")
    imgs = _batch(4)
    labels = torch.tensor([1, 2, 3, 4])
    net.load_batch(imgs, labels)
    net.forward(train=True)
    net.backward()
    assert torch.isfinite(net.grads).all() and float(net.grads.abs().sum()) > 0
    # inference: scale_lower, centred crop, no flip -> deterministic and equal to the per-sample restatement
    op = net.input_op
    out = op.ref_forward(imgs, False, 0)
    for i, im in enumerate(imgs):
        _, h, w = im.shape
        rw, rh = VarDataOp.scaled_dims(w, h, 36)
        v = VarDataOp.ref_sample(im, 36, (rw - 32) // 2, (rh - 32) // 2, False, 32, 32) / 255.0
        v = v - torch.tensor([0.4, 0.5, 0.6]).reshape(3, 1, 1)
        assert torch.allclose(out[i], v, atol=1e-6)
    padded, shapes = VarDataOp.pack(imgs, 3 * 96 * 96)
    assert torch.allclose(op.ref_forward((padded, shapes), False, 0), out)


@pytest.mark.gpu
@pytest.mark.parametrize("train", [False, True])
def test_var_input_kernel_matches_restatement(train):
    net = Net(_var_cfg(32, 36, 48), 8, device="cuda")
    op = net.input_op
    imgs = _batch(8)
    net.load_batch(imgs, torch.zeros(8, dtype=torch.int32))
    op.forward(train, 0)
    torch.cuda.synchronize()
    out = op.out.float().cpu()          # [B, 32, 32, Cp]
    draws = op.draws.cpu()
    assert torch.all(out[..., 3:] == 0)
    mean = torch.tensor([0.4, 0.5, 0.6]).reshape(3, 1, 1)
    seen_flip = set()
    for i, im in enumerate(imgs):
        sdim, ox, oy, flip = (int(v) for v in draws[i])
        _, h, w = im.shape
        rw, rh = VarDataOp.scaled_dims(w, h, sdim)
        if train:
            assert 36 <= sdim <= 48 and 0 <= ox <= max(0, rw - 32) and 0 <= oy <= max(0, rh - 32)
        else:
            assert (sdim, ox, oy, flip) == (36, (rw - 32) // 2, (rh - 32) // 2, 0)
        seen_flip.add(flip)
        ref = VarDataOp.ref_sample(im, sdim, ox, oy, bool(flip), 32, 32) / 255.0 - mean
        got = out[i, :, :, :3].permute(2, 0, 1)
        assert torch.allclose(got, ref, atol=6e-3, rtol=8e-3), float((got - ref).abs().max())
    if train:
        assert seen_flip == {0, 1}


@pytest.mark.gpu
def test_var_input_space_to_depth_feeds_strided_conv():
    """A strided first convolution reads the space-to-depth form; logits must match the CPU reference path."""
    cfg = _var_cfg(35, 40, 40, flip=False, stride=2)
    gpu = Net(cfg, 4, device="cuda", seed=(5, 6))
    cpu = Net(_var_cfg(35, 40, 40, flip=False, stride=2), 4, device="cpu", seed=(5, 6))
    assert gpu.input_op.mode == "s2d"
    imgs = _batch(4, seed=9)
    labels = torch.tensor([0, 3, 5, 7], dtype=torch.int32)
    gpu.load_batch(imgs, labels)
    cpu.load_batch(imgs, labels.long())
    gpu.forward(False)
    cpu.forward(False)
    lg, lc = gpu.read_stats()[0], cpu.read_stats()[0]
    assert abs(lg - lc) < 0.03 * max(1.0, abs(lc)), (lg, lc)


def test_variable_size_resnet_template_builds_and_steps_on_cpu():
    from rembrandt_b200.models import zoo
    cfg = zoo.resnet18_var(num_classes=7, in_hw=32, scale=(36, 48), max_hw=64, channel_mean=(0.4, 0.5, 0.6))
    net = Net(cfg, 2, device="cpu", seed=(1, 2))
    assert isinstance(net.input_op, VarDataOp) and net.input_op.scale_range == (36, 48)
    assert net.input_op.flip and net.input_op.pca is not None
    fixed = Net(zoo.resnet18(num_classes=7, in_hw=32, raw_hw=40), 2, device="cpu", seed=(1, 2))
    assert net.params_len == fixed.params_len                 # the same network behind a different input operator
    g = torch.Generator().manual_seed(0)
    imgs = [torch.randint(0, 256, (3, 40, 64), dtype=torch.uint8, generator=g),
            torch.randint(0, 256, (3, 57, 38), dtype=torch.uint8, generator=g)]
    net.load_batch(imgs, torch.tensor([1, 5]))
    net.forward(True)
    net.backward()
    loss, _ = net.read_stats()
    assert 0.5 < loss < 6.0 and torch.isfinite(net.grads).all() and float(net.grads.abs().sum()) > 0
