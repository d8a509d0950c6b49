"""Logistic / tanh / clipped-ReLU activation kernels, the sparsity counter, the low-rank affine block and the
CUDA-core convolution backend against fp32 torch (GPU only).

Sorted after the other GPU files on purpose: these kernels are elementwise helpers of the older layer generations,
not part of any benchmarked network.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

from rembrandt_b200.models import config as C
from rembrandt_b200.models.config import (Act, AffineCfg, Conv2dCfg, Data3dCfg, MimicAffineCfg, ParamsInit, Pool2dCfg,
                                          PoolKind,
                                          SequentialOperatorConfig, SoftmaxKLLossCfg)
from rembrandt_b200.models.net import Net
from rembrandt_b200.ops import native_ops as K

KINDS = [(K.ACT_LOGISTIC, torch.sigmoid), (K.ACT_TANH, torch.tanh),
         (K.ACT_BOUNDED_RECT, lambda x: x.clamp(0.0, 1.5)), (K.ACT_RECT, torch.relu),
         (K.ACT_SCALED_LOGISTIC, lambda x: torch.sigmoid(1.5 * x))]


@pytest.mark.parametrize("kind,fn", KINDS)
@pytest.mark.parametrize("rows,ld,n_valid", [(37, 32, 20), (1000, 64, 64), (5, 96, 90)])
def test_activation_forward_and_backward(kind, fn, rows, ld, n_valid):
    torch.manual_seed(kind * 100 + rows)
    x = (torch.randn(rows, ld) * 2.0).bfloat16()
    x[:, n_valid:] = 0
    y = x.cuda().clone()
    K.act_fwd(y, rows, ld, n_valid, kind, 1.5)
    xr = x.float().requires_grad_(True)
    ref = fn(xr)
    got = y.float().cpu()
    assert torch.all(got[:, n_valid:] == 0), "padded columns must stay zero"
    assert torch.allclose(got[:, :n_valid], ref[:, :n_valid].detach(), atol=1e-2, rtol=1e-2)

    d = torch.randn(rows, ld).bfloat16()
    dd = d.cuda().clone()
    K.act_bwd(dd, y, rows, ld, n_valid, kind, 1.5)
    # the slope is evaluated at the bf16-rounded output, as the kernel sees it
    yo = got
    slope = {K.ACT_LOGISTIC: yo * (1 - yo), K.ACT_TANH: 1 - yo * yo,
             K.ACT_BOUNDED_RECT: ((yo > 0) & (yo < 1.5)).float(), K.ACT_RECT: (yo > 0).float(),
             K.ACT_SCALED_LOGISTIC: 1.5 * yo * (1 - yo)}[kind]
    want = d.float() * slope
    gd = dd.float().cpu()
    assert torch.all(gd[:, n_valid:] == 0)
    assert torch.allclose(gd[:, :n_valid], want[:, :n_valid], atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_count_above(dtype):
    torch.manual_seed(5)
    x = torch.randn(100_003)
    x[::3] = 0
    xd = x.to(dtype).cuda()
    out = torch.zeros(1, dtype=torch.int64, device="cuda")
    K.count_above(xd, 0.0, out)
    K.count_above(xd, 1.0, out)
    xf = xd.float().cpu()
    assert int(out.item()) == int((xf.abs() > 0).sum()) + int((xf.abs() > 1.0).sum())


def _cfg():
    k = ParamsInit.kaiming()
    return (SequentialOperatorConfig().data3d(Data3dCfg((12, 12, 3), normalize=True))
            .conv2d(Conv2dCfg(3, 1, 1, 20, Act.TANH, k), "conv1")
            .pool2d(Pool2dCfg(2, 2, 0, PoolKind.MAX), "pool1")
            .conv2d(Conv2dCfg(3, 1, 1, 24, Act.BOUNDED_RECT, k), "conv2")
            .affine(AffineCfg(30, Act.LOGISTIC, ParamsInit.xavier()), "fc1")
            .affine(AffineCfg(10, Act.IDENTITY, ParamsInit.xavier()), "fc2")
            .softmax_kl_loss(SoftmaxKLLossCfg(10)))


def _mimic_cfg():
    k = ParamsInit.kaiming()
    return (SequentialOperatorConfig().data3d(Data3dCfg((12, 12, 3), normalize=True))
            .conv2d(Conv2dCfg(3, 1, 1, 32, Act.RECT, k), "conv1")
            .pool2d(Pool2dCfg(2, 2, 0, PoolKind.MAX), "pool1")
            .mimic_affine(MimicAffineCfg(bottleneck_rank=64, hidden_channels=96, out_channels=10), "m")
            .softmax_kl_loss(SoftmaxKLLossCfg(10)))


def _direct_cfg():
    k = ParamsInit.kaiming()
    d = C.ConvBackend.DIRECT
    return (SequentialOperatorConfig().data3d(Data3dCfg((13, 13, 3), normalize=True))
            .conv2d(Conv2dCfg(5, 2, 1, 24, Act.RECT, k, backend=d), "conv1")
            .conv2d(Conv2dCfg(3, 1, 1, 40, Act.RECT, k, backend=d), "conv2")
            .conv2d(Conv2dCfg(3, 2, 1, 32, Act.RECT, k, backend=d), "conv3")
            .affine(AffineCfg(10, Act.IDENTITY, ParamsInit.xavier()), "fc")
            .softmax_kl_loss(SoftmaxKLLossCfg(10)))


def _res_cfg():
    k = ParamsInit.kaiming()
    return (SequentialOperatorConfig().data3d(Data3dCfg((12, 12, 3), normalize=True))
            .conv2d(Conv2dCfg(3, 1, 1, 32, Act.RECT, k), "stem")
            .res_conv2d(C.ResConv2dCfg(3, Act.RECT), "res1")
            .res_conv2d(C.ResConv2dCfg(3, Act.SCALED_LOGISTIC, act_param=2.0), "res2")
            .pool2d(Pool2dCfg(12, 1, 0, PoolKind.AVERAGE), "gap")
            .affine(AffineCfg(10, Act.IDENTITY, ParamsInit.xavier()), "fc")
            .softmax_kl_loss(SoftmaxKLLossCfg(10)))


@pytest.mark.parametrize("_cfg", [_cfg, _mimic_cfg, _direct_cfg, _res_cfg],
                         ids=["smooth_activations", "low_rank_affine", "direct_conv_backend", "residual_convolution"])
def test_network_matches_reference_path(_cfg):
    batch = 8
    g = Net(_cfg(), batch, device="cuda", seed=(3, 4))
    c = Net(_cfg(), batch, device="cpu", seed=(3, 4))
    with torch.no_grad():
        c.params.copy_(g.params16.float().cpu())
    torch.manual_seed(0)
    hw = g.input_op.src_hwc[0]
    x = torch.randint(0, 256, (batch, 3, hw, hw), dtype=torch.uint8)
    y = torch.randint(0, 10, (batch,))
    g.load_batch(x.cuda(), y.cuda().int())
    c.load_batch(x, y)
    for n in (g, c):
        n.forward(True)
        n.backward()
    torch.cuda.synchronize()
    assert K.read_status() == 0
    gl, _ = g.read_stats()
    cl, _ = c.read_stats()
    assert abs(gl - cl) < 3e-2 * max(1.0, abs(cl)), (gl, cl)
    gg, cg = g.grads.cpu(), c.grads
    for seg in g.segs:
        a, b = gg[seg.offset: seg.offset + seg.numel], cg[seg.offset: seg.offset + seg.numel]
        rel = float((a - b).norm() / b.norm().clamp_min(1e-12))
        assert rel < 0.1, f"{seg.name}: relative error {rel:.4g}"
    assert C.ACT_BOUND > 0
