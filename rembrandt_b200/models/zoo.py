"""Model templates.

The reference builds its networks in code: ``src/templates/{vgg,resnet,resnet_new}.rs`` and the ``build_*``
functions inside ``tools/train-mnist.rs``, ``tools/train-cifar10.rs`` and ``tools/train-imagenet.rs``. The
same architectures are provided here as functions returning a ``SequentialOperatorConfig``. The synthetic
benchmark shapes (LeNet on 28x28x1, the CIFAR convnet, AlexNet on 227x227x3, NIN on 224x224x3) are the ones
the framework's headline benchmark is quoted on.
"""
from __future__ import annotations

from .config import (Act, AffineCfg, BNormConv2dCfg, BNormMovingAverage, Conv2dCfg, Data3dCfg, DropoutCfg, LrnCfg,
                     ParamsInit, Pool2dCfg, PoolKind, Preproc, ProjStackResConv2dCfg, SequentialOperatorConfig,
                     SoftmaxKLLossCfg, StackResConv2dCfg)

# eigen-decomposition of ImageNet RGB covariance used for PCA lighting noise (AlexNet paper values)
PCA_EIGVALS = (0.2175, 0.0188, 0.0045)
PCA_EIGVECS = (-0.5675, 0.7192, 0.4009, -0.5808, -0.0045, -0.8140, -0.5836, -0.6948, 0.4203)


def mnist_fc1(num_classes=10):
    """784 -> 10 softmax regression (tests/mnist-1layer-fc.rs)."""
    return (SequentialOperatorConfig()
            .data3d(Data3dCfg((28, 28, 1), normalize=True))
            .affine(AffineCfg(num_classes, Act.IDENTITY, ParamsInit.normal(0.01)), "fc1")
            .softmax_kl_loss(SoftmaxKLLossCfg(num_classes)))


def mnist_fc2(hidden=800, num_classes=10):
    """784 -> 800 ReLU -> 10 (tests/mnist-2layer-fc.rs)."""
    return (SequentialOperatorConfig()
            .data3d(Data3dCfg((28, 28, 1), normalize=True))
            .affine(AffineCfg(hidden, Act.RECT, ParamsInit.xavier()), "fc1")
            .affine(AffineCfg(num_classes, Act.IDENTITY, ParamsInit.xavier()), "fc2")
            .softmax_kl_loss(SoftmaxKLLossCfg(num_classes)))


def lenet(pad=0, num_classes=10):
    """conv5x5 20 -> maxpool2 -> conv5x5 50 -> maxpool2 -> fc 500 ReLU -> fc 10.

    pad=0 gives the 800-input fc of the benchmark configuration; pad=2 is the variant of
    tools/train-mnist.rs:74-147 (2450-input fc).
    """
    k = ParamsInit.kaiming()
    return (SequentialOperatorConfig()
            .data3d(Data3dCfg((28, 28, 1), normalize=True))
            .conv2d(Conv2dCfg(5, 1, pad, 20, Act.RECT, k), "conv1")
            .pool2d(Pool2dCfg(2, 2, 0, PoolKind.MAX), "pool1")
            .conv2d(Conv2dCfg(5, 1, pad, 50, Act.RECT, k), "conv2")
            .pool2d(Pool2dCfg(2, 2, 0, PoolKind.MAX), "pool2")
            .affine(AffineCfg(500, Act.RECT, ParamsInit.xavier()), "fc1")
            .affine(AffineCfg(num_classes, Act.IDENTITY, ParamsInit.xavier()), "fc2")
            .softmax_kl_loss(SoftmaxKLLossCfg(num_classes)))


def cifar_krizh26(augment=True, mean=None, num_classes=10):
    """conv5x5 32 -> maxpool3/2 -> conv5x5 32 -> avgpool3/2 -> conv5x5 64 -> avgpool3/2 -> fc 10
    (tools/train-cifar10.rs:58-150). With `augment`: mean subtraction, pad-4 random crop, flip."""
    pre = []
    if mean is not None:
        pre.append(Preproc("subtract_mean", mean=mean, normalize=True))
    if augment:
        pre += [Preproc("flip_x"), Preproc("crop", crop_width=32, crop_height=32, pad=4)]
    n = ParamsInit.normal
    return (SequentialOperatorConfig()
            .data3d(Data3dCfg((32, 32, 3), normalize=True, preprocs=pre))
            .conv2d(Conv2dCfg(5, 1, 2, 32, Act.RECT, n(0.0001)), "conv1")
            .pool2d(Pool2dCfg(3, 2, 0, PoolKind.MAX), "pool1")
            .conv2d(Conv2dCfg(5, 1, 2, 32, Act.RECT, n(0.01)), "conv2")
            .pool2d(Pool2dCfg(3, 2, 0, PoolKind.AVERAGE), "pool2")
            .conv2d(Conv2dCfg(5, 1, 2, 64, Act.RECT, n(0.01)), "conv3")
            .pool2d(Pool2dCfg(3, 2, 0, PoolKind.AVERAGE), "pool3")
            .affine(AffineCfg(num_classes, Act.IDENTITY, n(0.01)), "fc")
            .softmax_kl_loss(SoftmaxKLLossCfg(num_classes)))


def alexnet(in_hw=227, num_classes=1000, raw_hw=None, mean=None, scale=None, lrn2=False):
    """Ungrouped AlexNet: conv11/4 96 -> LRN -> maxpool3/2 -> conv5 256 -> LRN -> maxpool -> conv3 384 -> conv3 384
    -> conv3 256 -> maxpool -> fc 4096 -> fc 4096 -> fc 1000, dropout 0.5 (62.4 M parameters at 227x227).
    `raw_hw` > `in_hw` adds a random crop + flip from raw_hw x raw_hw sources; `lrn2` adds the second
    normalisation layer of examples/imagenet_alexnet.model after conv2."""
    n = ParamsInit.normal
    pre = []
    src = in_hw
    if mean is not None:
        pre.append(Preproc("subtract_mean", mean=mean))
    if raw_hw and raw_hw > in_hw:
        src = raw_hw
        pre += [Preproc("flip_x"), Preproc("crop", crop_width=in_hw, crop_height=in_hw)]
    cfg = (SequentialOperatorConfig()
           .data3d(Data3dCfg((src, src, 3), preprocs=pre, scale=scale))
           .conv2d(Conv2dCfg(11, 4, 0, 96, Act.RECT, n(0.01)), "conv1")
           .lrn(LrnCfg(5, 1e-4, 0.75, 2.0), "rnorm1")
           .pool2d(Pool2dCfg(3, 2, 0, PoolKind.MAX), "pool1")
           .conv2d(Conv2dCfg(5, 1, 2, 256, Act.RECT, n(0.01)), "conv2"))
    if lrn2:
        cfg.lrn(LrnCfg(5, 1e-4, 0.75, 2.0), "rnorm2")
    return (cfg
            .pool2d(Pool2dCfg(3, 2, 0, PoolKind.MAX), "pool2")
            .conv2d(Conv2dCfg(3, 1, 1, 384, Act.RECT, n(0.03)), "conv3")
            .conv2d(Conv2dCfg(3, 1, 1, 384, Act.RECT, n(0.03)), "conv4")
            .conv2d(Conv2dCfg(3, 1, 1, 256, Act.RECT, n(0.03)), "conv5")
            .pool2d(Pool2dCfg(3, 2, 0, PoolKind.MAX), "pool3")
            .affine(AffineCfg(4096, Act.RECT, n(0.01)), "fc6")
            .dropout(DropoutCfg(0.5), "drop6")
            .affine(AffineCfg(4096, Act.RECT, n(0.01)), "fc7")
            .dropout(DropoutCfg(0.5), "drop7")
            .affine(AffineCfg(num_classes, Act.IDENTITY, n(0.01)), "fc8")
            .softmax_kl_loss(SoftmaxKLLossCfg(num_classes)))


def nin(in_hw=224, num_classes=1000, scale=None):
    """Network-in-Network: four mlpconv blocks with ceil-mode max pooling 54->27->13->6, dropout 0.5 before
    the last block, global average pooling (examples/imagenet_nin.model)."""
    n = ParamsInit.normal
    cfg = SequentialOperatorConfig().data3d(Data3dCfg((in_hw, in_hw, 3), scale=scale))

    def block(i, k, s, p, ch, stds, outs=None):
        outs = outs or (ch, ch, ch)
        cfg.conv2d(Conv2dCfg(k, s, p, outs[0], Act.RECT, n(stds[0])), f"conv{i}")
        cfg.conv2d(Conv2dCfg(1, 1, 0, outs[1], Act.RECT, n(stds[1])), f"cccp{2 * i - 1}")
        cfg.conv2d(Conv2dCfg(1, 1, 0, outs[2], Act.RECT, n(stds[2])), f"cccp{2 * i}")

    block(1, 11, 4, 0, 96, (0.01, 0.05, 0.05))
    cfg.pool2d(Pool2dCfg(3, 2, 0, PoolKind.MAX, ceil_mode=True), "pool1")
    block(2, 5, 1, 2, 256, (0.05, 0.05, 0.05))
    cfg.pool2d(Pool2dCfg(3, 2, 0, PoolKind.MAX, ceil_mode=True), "pool2")
    block(3, 3, 1, 1, 384, (0.01, 0.05, 0.05))
    cfg.pool2d(Pool2dCfg(3, 2, 0, PoolKind.MAX, ceil_mode=True), "pool3")
    cfg.dropout(DropoutCfg(0.5), "drop")
    block(4, 3, 1, 1, 1024, (0.05, 0.05, 0.01), outs=(1024, 1024, num_classes))
    hw = _nin_final_hw(in_hw)
    cfg.pool2d(Pool2dCfg(hw, 1, 0, PoolKind.AVERAGE), "pool4")
    cfg.softmax_kl_loss(SoftmaxKLLossCfg(num_classes))
    return cfg


def _nin_final_hw(in_hw):
    hw = (in_hw - 11) // 4 + 1
    for _ in range(3):
        hw = -(-(hw - 3) // 2) + 1
    return hw


def _vgg_a_trunk(in_hw, raw_hw, mean):
    k = ParamsInit.kaiming()
    pre = []
    if mean is not None:
        pre.append(Preproc("subtract_mean", mean=mean))
    src = in_hw
    if raw_hw and raw_hw > in_hw:
        src = raw_hw
        pre += [Preproc("flip_x"), Preproc("crop", crop_width=in_hw, crop_height=in_hw)]
    cfg = SequentialOperatorConfig().data3d(Data3dCfg((src, src, 3), normalize=True, preprocs=pre))
    i = 0
    for ch, reps in ((64, 1), (128, 1), (256, 2), (512, 2), (512, 2)):
        for _ in range(reps):
            i += 1
            cfg.conv2d(Conv2dCfg(3, 1, 1, ch, Act.RECT, k), f"conv{i}")
        cfg.pool2d(Pool2dCfg(2, 2, 0, PoolKind.MAX), f"pool{i}")
    return cfg


def vgg_a_avgpool(num_classes=1000, in_hw=256, mean=None):
    """The VGG-A convolutions followed by a global average pool and one classifier layer instead of the three fully
    connected ones (tools/train-imagenet.rs:270-468; 256 x 256 input, 8 x 8 average pool)."""
    cfg = _vgg_a_trunk(in_hw, None, mean)
    cfg.pool2d(Pool2dCfg(in_hw // 32, 1, 0, PoolKind.AVERAGE), "global_pool")
    cfg.affine(AffineCfg(num_classes, Act.IDENTITY, ParamsInit.xavier()), "fc")
    return cfg.softmax_kl_loss(SoftmaxKLLossCfg(num_classes))


def vgg_a(num_classes=1000, in_hw=224, raw_hw=256, mean=None):
    """VGG-A: 8 conv3x3 + 3 fc, dropout 0.5, Kaiming conv init, U(+-0.01) fc (src/templates/vgg.rs:50-260)."""
    u = ParamsInit.uniform(0.01)
    cfg = _vgg_a_trunk(in_hw, raw_hw, mean)
    cfg.affine(AffineCfg(4096, Act.RECT, u), "fc6").dropout(DropoutCfg(0.5), "drop6")
    cfg.affine(AffineCfg(4096, Act.RECT, u), "fc7").dropout(DropoutCfg(0.5), "drop7")
    cfg.affine(AffineCfg(num_classes, Act.IDENTITY, u), "fc8")
    return cfg.softmax_kl_loss(SoftmaxKLLossCfg(num_classes))


def _imagenet_resnet(blocks, num_classes, in_hw, raw_hw, mean, pca, ema, variable=None):
    """`variable` = (shorter-side lower, upper, largest width / height accepted) switches to the variable-size input
    operator: every image is rescaled so that its shorter side has a length drawn in [lower, upper], then cropped."""
    k = ParamsInit.kaiming()
    mov = BNormMovingAverage("exponential", ema)
    pre = []
    noise = [Preproc("pca_noise", std=0.1, eigenvalues=PCA_EIGVALS, eigenvectors=PCA_EIGVECS)] if pca else []
    if variable is not None:
        lower, upper, max_hw = variable
        pre = [Preproc("scale_bicubic", lower=lower, upper=upper),
               Preproc("crop", crop_width=in_hw, crop_height=in_hw), Preproc("flip_x")] + noise
        cfg = SequentialOperatorConfig().var_data3d(
            Data3dCfg((max_hw, max_hw, 3), normalize=True, preprocs=pre, max_dims=(max_hw, max_hw, 3),
                      channel_mean=list(mean) if mean is not None else None))
    else:
        if mean is not None:
            pre.append(Preproc("subtract_mean", mean=mean))
        src = in_hw
        if raw_hw and raw_hw > in_hw:
            src = raw_hw
            pre += [Preproc("flip_x"), Preproc("crop", crop_width=in_hw, crop_height=in_hw)]
        pre += noise
        cfg = SequentialOperatorConfig().data3d(Data3dCfg((src, src, 3), normalize=True, preprocs=pre))
    cfg.bnorm_conv2d(BNormConv2dCfg(7, 2, 3, 64, Act.RECT, k, mov), "conv1")
    cfg.pool2d(Pool2dCfg(3, 2, 1, PoolKind.MAX), "pool1")
    ch = 64
    for stage, reps in enumerate(blocks):
        out = 64 << stage
        for r in range(reps):
            name = f"res{stage + 2}_{r + 1}"
            if out != ch:
                cfg.proj_stack_res_conv2d(ProjStackResConv2dCfg(out, None, k, mov), name)
                ch = out
            else:
                cfg.stack_res_conv2d(StackResConv2dCfg(k, mov), name)
    hw = in_hw
    hw = (hw + 6 - 7) // 2 + 1
    hw = (hw + 2 - 3) // 2 + 1
    for _ in range(len(blocks) - 1):
        hw = (hw + 1) // 2
    cfg.pool2d(Pool2dCfg(hw, 1, 0, PoolKind.AVERAGE), "global_pool")
    cfg.affine(AffineCfg(num_classes, Act.IDENTITY, ParamsInit.xavier()), "fc")
    return cfg.softmax_kl_loss(SoftmaxKLLossCfg(num_classes))


def resnet18(num_classes=1000, in_hw=224, raw_hw=256, mean=None, pca=True, ema=0.1):
    """ResNet-18 (src/templates/resnet.rs:54-206, src/templates/resnet_new.rs:58-212)."""
    return _imagenet_resnet((2, 2, 2, 2), num_classes, in_hw, raw_hw, mean, pca, ema)


def resnet34(num_classes=1000, in_hw=224, raw_hw=256, mean=None, pca=True, ema=0.1):
    """ResNet-34 (src/templates/resnet.rs:208-365)."""
    return _imagenet_resnet((3, 4, 6, 3), num_classes, in_hw, raw_hw, mean, pca, ema)


def resnet18_var(num_classes=1000, in_hw=224, scale=(256, 480), max_hw=640, channel_mean=None, pca=True, ema=0.1):
    """ResNet-18 on images of any size: shorter side rescaled (bicubic) to a length drawn in `scale`, crop `in_hw`,
    flip, lighting noise; moving-average factor 0.1, epsilon 1e-5, Xavier classifier
    (src/templates/resnet_new.rs:58-212). `channel_mean` is an optional per-channel mean in [0, 1] units."""
    return _imagenet_resnet((2, 2, 2, 2), num_classes, in_hw, None, channel_mean, pca, ema,
                            variable=(scale[0], scale[1], max_hw))


def resnet34_var(num_classes=1000, in_hw=224, scale=(256, 480), max_hw=640, channel_mean=None, pca=True, ema=0.1):
    """ResNet-34 with the variable-size input chain (src/templates/resnet_new.rs:214-376)."""
    return _imagenet_resnet((3, 4, 6, 3), num_classes, in_hw, None, channel_mean, pca, ema,
                            variable=(scale[0], scale[1], max_hw))


def resnet20(num_classes=1000, in_hw=224, raw_hw=256, mean=None, pca=True, ema=0.1):
    """The 20-layer ImageNet variant of the reference's tool: 2 / 2 / 2 / 3 basic blocks
    (tools/train-imagenet.rs:731-876)."""
    return _imagenet_resnet((2, 2, 2, 3), num_classes, in_hw, raw_hw, mean, pca, ema)


def resnet10(num_classes=1000, in_hw=224, raw_hw=256, mean=None):
    """ResNet-10 (tools/train-imagenet.rs)."""
    return _imagenet_resnet((1, 1, 1, 1), num_classes, in_hw, raw_hw, mean, False, 0.1)


def resnet20_cifar(num_classes=10, mean=None, augment=True):
    """CIFAR ResNet-20: BN-conv stem 16, 3 x {16, 32, 64} basic blocks, global average pool, Xavier fc
    (tools/train-cifar10.rs:381-533); crop 28 in the reference, pad-4 crop 32 here when `augment`."""
    k = ParamsInit.kaiming()
    mov = BNormMovingAverage("exponential", 0.1)
    pre = []
    if mean is not None:
        pre.append(Preproc("subtract_mean", mean=mean, normalize=True))
    if augment:
        pre += [Preproc("flip_x"), Preproc("crop", crop_width=32, crop_height=32, pad=4)]
    cfg = SequentialOperatorConfig().data3d(Data3dCfg((32, 32, 3), normalize=True, preprocs=pre))
    cfg.bnorm_conv2d(BNormConv2dCfg(3, 1, 1, 16, Act.RECT, k, mov), "conv1")
    ch = 16
    for stage, out in enumerate((16, 32, 64)):
        for r in range(3):
            name = f"res{stage + 1}_{r + 1}"
            if out != ch:
                cfg.proj_stack_res_conv2d(ProjStackResConv2dCfg(out, None, k, mov), name)
                ch = out
            else:
                cfg.stack_res_conv2d(StackResConv2dCfg(k, mov), name)
    cfg.pool2d(Pool2dCfg(8, 1, 0, PoolKind.AVERAGE), "global_pool")
    cfg.affine(AffineCfg(num_classes, Act.IDENTITY, ParamsInit.xavier()), "fc")
    return cfg.softmax_kl_loss(SoftmaxKLLossCfg(num_classes))


def go_policy_net(planes=32, channels=128, layers=6, num_classes=361):
    """Convolutional move-prediction network on 19x19 bit-plane inputs (tools/train-gogod.rs:56-227)."""
    k = ParamsInit.kaiming()
    cfg = SequentialOperatorConfig().data3d(Data3dCfg((19, 19, planes), normalize=True))   # planes hold 0 / 255
    cfg.conv2d(Conv2dCfg(5, 1, 2, channels, Act.RECT, k), "conv1")
    for i in range(2, layers):
        cfg.conv2d(Conv2dCfg(3, 1, 1, channels, Act.RECT, k), f"conv{i}")
    cfg.conv2d(Conv2dCfg(3, 1, 1, 1, Act.IDENTITY, k), f"conv{layers}")
    return cfg.softmax_kl_loss(SoftmaxKLLossCfg(num_classes))


def go_policy_resnet(planes=32, channels=128, blocks=5, num_classes=361):
    """The residual move-prediction network the reference's Go tool trains (tools/train-gogod.rs:59-158): a
    batch-normalised 3x3 stem, `blocks` two-convolution residual blocks (moving-average factor 0.01, epsilon 1e-4)
    and a 3x3 convolution to one plane, whose 19 x 19 outputs are the 361 move logits."""
    k = ParamsInit.kaiming()
    cfg = SequentialOperatorConfig().data3d(Data3dCfg((19, 19, planes), normalize=True))
    mov = BNormMovingAverage("exponential", 0.01)
    cfg.bnorm_conv2d(BNormConv2dCfg(3, 1, 1, channels, Act.RECT, k, mov, 1e-4), "stem")
    for i in range(blocks):
        cfg.stack_res_conv2d(StackResConv2dCfg(k, mov, 1e-4), f"res{i + 1}")
    cfg.conv2d(Conv2dCfg(3, 1, 1, 1, Act.IDENTITY, k), "move")
    return cfg.softmax_kl_loss(SoftmaxKLLossCfg(num_classes))


TEMPLATES = {
    "mnist_fc1": mnist_fc1, "mnist_fc2": mnist_fc2, "lenet": lenet, "cifar_krizh26": cifar_krizh26,
    "alexnet": alexnet, "nin": nin, "vgg_a": vgg_a, "vgg_a_avgpool": vgg_a_avgpool, "resnet10": resnet10,
    "resnet18": resnet18, "resnet20": resnet20,
    "resnet34": resnet34, "resnet18_var": resnet18_var, "resnet34_var": resnet34_var,
    "resnet20_cifar": resnet20_cifar, "go_policy_net": go_policy_net, "go_policy_resnet": go_policy_resnet,
}
