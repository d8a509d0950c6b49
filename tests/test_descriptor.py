"""The shipped .model / .data descriptors parse as they are, and the networks they describe have the
reference's parameter counts (CPU)."""
import os

import pytest

from rembrandt_b200.models import descriptor, zoo
from rembrandt_b200.models import config as C
from rembrandt_b200.models.net import Net

# the descriptor files shipped with this repository
EX = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")

LENET_MODEL = """
[[layer]]
name = "data"
type = "data"
raw_width = 28
raw_height = 28
crop_width = 28
crop_height = 28
channels = 1
[[layer]]
name = "conv1"
type = "conv2d"
conv_size = 5
conv_stride = 1
conv_pad = 2
out_channels = 16
act_func = "rect"
init_weights = { kind = "normal", mean = 0.0, std = 0.01 }
[[layer]]
name = "pool1"
pool_size = 2
pool_stride = 2
pool_pad = 0
[[layer]]
names = ["fc1a", "fc1b"]
out_channels = 50
act_func = "relu"
[[layer]]
names = ["drop1a", "drop1b"]
type = "dropout"
drop_ratio = 0.1
[[layer]]
name = "fc2"
inputs = ["drop1a", "drop1b"]
type = "fully_conn"
out_channels = 10
act_func = "identity"
[[layer]]
name = "loss"
type = "softmax_loss"
num_categories = 10
[opt]
minibatch_size = 64
init_step_size = 0.01
momentum = 0.9
l2_reg_coef = 0.0005
annealing_policy = { kind = "step", step_iters = 200000, decay = 0.1 }
"""


def test_inline_descriptor_with_irregularities():
    d = descriptor.parse_model(LENET_MODEL)
    kinds = [type(o.cfg).__name__ for o in d.config.hidden_ops]
    assert kinds == ["Conv2dCfg", "Pool2dCfg", "AffineCfg", "DropoutCfg", "AffineCfg"]
    pool = d.config.hidden_ops[1].cfg
    assert pool.kind == C.PoolKind.MAX and pool.ceil_mode            # type and kind inferred
    fc1 = d.config.hidden_ops[2].cfg
    assert fc1.out_channels == 100 and fc1.act == C.Act.RECT         # towers merged, "relu" accepted
    assert d.opt.minibatch_size == 64 and d.opt.mu == 0.9 and d.opt.l2_reg_coef == 5e-4
    assert d.opt.step_size.at_iter(0) == 0.01 and abs(d.opt.step_size.at_iter(200000) - 0.001) < 1e-12
    net = Net(d.config, 2, device="cpu")
    assert net.params_len == (16 * 25 + 16) + (14 * 14 * 16 * 100 + 100) + (100 * 10 + 10)


@pytest.mark.parametrize("name,params", [("mnist_lenet", 431080), ("imagenet_nin", 7595176),
                                         ("imagenet_alexnet", 62378344)])
def test_shipped_models_parse(name, params):
    d = descriptor.load_model(f"{EX}/{name}.model", use_crop=False)
    net = Net(d.config, 1, device="cpu")
    assert net.params_len == params
    if name == "imagenet_alexnet":
        convs = [o.cfg.out_channels for o in d.config.hidden_ops if isinstance(o.cfg, C.Conv2dCfg)]
        assert convs == [96, 256, 384, 384, 256]
        assert sum(isinstance(o.cfg, C.LrnCfg) for o in d.config.hidden_ops) == 2
        assert [op.out_hwc[0] for op in net.ops if type(op).__name__ == "Pool2dOp"] == [27, 13, 6]
        assert d.opt.minibatch_size == 128 and d.opt.max_iters == 450000
        # with the crop the input operator stages 256 x 256 images and cuts 227 x 227 windows
        dc = descriptor.load_model(f"{EX}/{name}.model").config.input_op.cfg
        assert dc.in_dims[:2] == (256, 256) and [p.kind for p in dc.preprocs] == ["flip_x", "crop"]
    if name == "imagenet_nin":
        sizes = [op.out_hwc[0] for op in net.ops if type(op).__name__ == "Pool2dOp"]
        assert sizes == [27, 13, 6, 1]                                # ceil-mode pooling, global average


TWO_TOWER_MODEL = """
[[layer]]
name = "data"
raw_width = 35
raw_height = 35
channels = 3
[[layer]]
names = ["conv1a", "conv1b"]
conv_size = 11
conv_stride = 4
out_channels = 48
act_func = "rect"
[[layer]]
names = ["pool1a", "pool1b"]
inputs = ["conv1a", "conv1b"]
pool_size = 3
pool_stride = 2
act_func = "rect"
[[layer]]
names = ["norm1a", "norm1b"]
cross_size = 5
[[layer]]
name = "fc"
inputs = ["norm1a", "norm1b"]
out_channels = 10
[[layer]]
name = "loss"
num_categories = 10
"""


def test_two_tower_notation_becomes_the_ungrouped_network():
    """Layers written as towers (`names = [a, b]`, as Krizhevsky's two-GPU AlexNet is usually written down) merge into
    one layer with the summed channel count; types are inferred from the keys; an activation on a pool layer counts."""
    d = descriptor.parse_model(TWO_TOWER_MODEL)
    ops = d.config.hidden_ops
    assert [type(o.cfg).__name__ for o in ops] == ["Conv2dCfg", "Pool2dCfg", "LrnCfg", "AffineCfg"]
    assert ops[0].cfg.out_channels == 96 and ops[1].cfg.act == C.Act.RECT and ops[0].name == "conv1"
    net = Net(d.config, 1, device="cpu")
    assert net.params_len == (3 * 121 * 96 + 96) + (3 * 3 * 96 * 10 + 10)


def test_shipped_data_files_parse():
    m = descriptor.load_data(f"{EX}/mnist.data")
    assert m["train"].source == "mnist" and m["train"].normalize and m["valid"].labels_path.endswith("t10k-labels-idx1-ubyte")
    i = descriptor.load_data(f"{EX}/imagenet.data")
    assert i["train"].source == "lmdb_caffe" and i["train"].mean_path.endswith(".ndarray")


def test_template_parameter_counts():
    assert Net(zoo.lenet(), 1, device="cpu").params_len == 431080
    assert Net(zoo.cifar_krizh26(augment=False), 1, device="cpu").params_len == 85098
    assert Net(zoo.nin(), 1, device="cpu").params_len == 7595176
    assert Net(zoo.alexnet(), 1, device="cpu").params_len == 62378344


def test_bad_descriptors_are_rejected():
    with pytest.raises(descriptor.DescriptorError):
        descriptor.parse_model("[opt]\nmomentum = 0.9\n")
    with pytest.raises(descriptor.DescriptorError):
        descriptor.parse_model('[[layer]]\nname = "x"\nfoo = 1\n')
    with pytest.raises(descriptor.DescriptorError):
        descriptor.parse_data("[dataset.train]\ndata_path = 'x'\n")


def test_example_descriptors_shipped_with_this_framework_build_and_step():
    """examples/*.model and *.data of this repository parse, build and take a training step on CPU."""
    import torch
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    md = descriptor.load_model(os.path.join(here, "examples", "mnist_lenet.model"))
    net = Net(md.config, 4, device="cpu")
    assert net.params_len == 431080          # 20 / 50 / 500 / 10 LeNet without padding
    splits = descriptor.load_data(os.path.join(here, "examples", "synthetic_mnist.data"))
    assert splits["train"].source == "synthetic" and "valid" in splits
    x = torch.randint(0, 256, (4, 1, 28, 28), dtype=torch.uint8)
    net.load_batch(x, torch.tensor([1, 2, 3, 4]))
    net.forward(True)
    net.backward()
    assert float(net.grads.abs().sum()) > 0


def test_cifar_example_descriptor_with_an_optimizer_section():
    import torch
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    md = descriptor.load_model(os.path.join(here, "examples", "cifar10_krizh26.model"))
    net = Net(md.config, 2, device="cpu")
    assert [o.out_hwc for o in net.ops[1:8]] == [(32, 32, 32), (16, 16, 32), (16, 16, 32), (8, 8, 32), (8, 8, 64),
                                                 (4, 4, 64), (1, 1, 10)]
    assert net.params_len == (75 * 32 + 32) + (800 * 32 + 32) + (800 * 64 + 64) + (1024 * 10 + 10)
    assert md.opt.minibatch_size == 128 and md.opt.mu == 0.9
    assert [md.opt.step_size.at_iter(t) for t in (0, 40000, 60000)] == pytest.approx([0.01, 0.001, 0.0001])
    assert "valid" in descriptor.load_data(os.path.join(here, "examples", "synthetic_cifar10.data"))
    net.load_batch(torch.randint(0, 256, (2, 3, 32, 32), dtype=torch.uint8), torch.tensor([1, 2]))
    net.forward(True)
    net.backward()
    assert float(net.grads.abs().sum()) > 0


def test_sigmoid_and_tanh_layers_of_a_descriptor_build_and_step():
    text = LENET_MODEL.replace('act_func = "rect"', 'act_func = "sigmoid"', 1).replace('act_func = "relu"', 'act_func = "tanh"', 1)
    assert text != LENET_MODEL
    d = descriptor.parse_model(text)
    acts = [getattr(o.cfg, "act", None) for o in d.config.hidden_ops]
    assert C.Act.LOGISTIC in acts
    net = Net(d.config, 2, device="cpu")
    import torch
    net.load_batch(torch.randint(0, 256, (2, 1, 28, 28), dtype=torch.uint8), torch.tensor([1, 2]))
    net.forward(True)
    net.backward()
    assert float(net.grads.abs().sum()) > 0
    with pytest.raises(ValueError):
        Net(C.SequentialOperatorConfig().data3d(C.Data3dCfg((8, 8, 1)))
            .pool2d(C.Pool2dCfg(2, 2, 0, C.PoolKind.MAX, act=C.Act.TANH), "p").softmax_kl_loss(C.SoftmaxKLLossCfg(16)),
            2, device="cpu")
