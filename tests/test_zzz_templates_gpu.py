"""Every remaining network template builds and runs one forward + backward on the device (finite loss near the
log of the class count, finite gradients, no kernel reported a problem). AlexNet, NIN, LeNet, the CIFAR network and
ResNet-18 are covered by the other GPU files and by the benchmark."""
import math

import pytest
import torch

from rembrandt_b200.models import zoo
from rembrandt_b200.models.net import Net
from rembrandt_b200.ops import native_ops as K

pytestmark = pytest.mark.gpu

CASES = [
    ("mnist_fc1", lambda: zoo.mnist_fc1(), (1, 28, 28), 10, 8),
    ("mnist_fc2", lambda: zoo.mnist_fc2(), (1, 28, 28), 10, 8),
    ("cifar_krizh26", lambda: zoo.cifar_krizh26(), (3, 32, 32), 10, 8),
    ("resnet20_cifar", lambda: zoo.resnet20_cifar(), (3, 32, 32), 10, 4),
    ("vgg_a", lambda: zoo.vgg_a(), (3, 256, 256), 1000, 2),
    ("vgg_a_avgpool", lambda: zoo.vgg_a_avgpool(), (3, 256, 256), 1000, 2),
    ("resnet20", lambda: zoo.resnet20(), (3, 256, 256), 1000, 2),
    ("resnet10", lambda: zoo.resnet10(), (3, 256, 256), 1000, 2),
    ("resnet34", lambda: zoo.resnet34(), (3, 256, 256), 1000, 2),
]


@pytest.mark.parametrize("name,make,chw,classes,batch", CASES, ids=[c[0] for c in CASES])
def test_template_runs_on_the_device(name, make, chw, classes, batch):
    net = Net(make(), batch, device="cuda", seed=(11, 13))
    w, h, c = net.input_op.cfg.in_dims
    assert (c, h, w) == chw, "the template's raw input size changed; update the case"
    torch.manual_seed(0)
    x = torch.randint(0, 256, (batch, c, h, w), dtype=torch.uint8).cuda()
    y = torch.randint(0, classes, (batch,)).int().cuda()
    net.load_batch(x, y)
    net.forward(True)
    net.backward()
    loss, _ = net.read_stats()
    torch.cuda.synchronize()
    assert K.read_status() == 0
    assert math.isfinite(loss) and 0.3 * math.log(classes) < loss < 4.0 * math.log(classes), loss
    assert torch.isfinite(net.grads).all() and float(net.grads.abs().sum()) > 0
