"""Comparison baseline: the same models and optimizer on stock PyTorch (cuDNN / cuBLAS kernels, DDP over NCCL).

The reference itself (a 2016 Rust crate over cuDNN v4 and MPI) cannot be built offline, so the number to
beat is this: torch DDP + cuDNN/cuBLAS, bf16, channels-last activations, SGD momentum 0.9 with weight decay
5e-4, 25 MB gradient buckets, same synthetic input shape and batch per GPU -- driven eagerly, or with the whole
step captured in a CUDA graph, or compiled; the benchmark reports the fastest of the variants it was asked to
run. None of the framework's own kernels or engine is on this path.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class AlexNet(nn.Module):
    """Ungrouped AlexNet, 227x227 input, one LRN after conv1 (62,378,344 parameters)."""

    def __init__(self, num_classes=1000, lrn2=False):
        super().__init__()
        self.conv1 = nn.Conv2d(3, 96, 11, 4)
        self.conv2 = nn.Conv2d(96, 256, 5, 1, 2)
        self.conv3 = nn.Conv2d(256, 384, 3, 1, 1)
        self.conv4 = nn.Conv2d(384, 384, 3, 1, 1)
        self.conv5 = nn.Conv2d(384, 256, 3, 1, 1)
        self.fc6 = nn.Linear(9216, 4096)
        self.fc7 = nn.Linear(4096, 4096)
        self.fc8 = nn.Linear(4096, num_classes)
        self.lrn2 = lrn2

    def forward(self, x):
        x = F.relu(self.conv1(x))
        x = F.local_response_norm(x, 5, alpha=5e-4, beta=0.75, k=2.0)
        x = F.max_pool2d(x, 3, 2)
        x = F.relu(self.conv2(x))
        if self.lrn2:
            x = F.local_response_norm(x, 5, alpha=5e-4, beta=0.75, k=2.0)
        x = F.max_pool2d(x, 3, 2)
        x = F.relu(self.conv3(x))
        x = F.relu(self.conv4(x))
        x = F.relu(self.conv5(x))
        x = F.max_pool2d(x, 3, 2)
        x = x.flatten(1)
        x = F.dropout(F.relu(self.fc6(x)), 0.5, self.training)
        x = F.dropout(F.relu(self.fc7(x)), 0.5, self.training)
        return self.fc8(x)


class NiN(nn.Module):
    def __init__(self, num_classes=1000):
        super().__init__()

        def block(cin, k, s, p, outs):
            layers = []
            c = cin
            for i, o in enumerate(outs):
                layers += [nn.Conv2d(c, o, k if i == 0 else 1, s if i == 0 else 1, p if i == 0 else 0), nn.ReLU(True)]
                c = o
            return nn.Sequential(*layers)

        self.b1 = block(3, 11, 4, 0, (96, 96, 96))
        self.b2 = block(96, 5, 1, 2, (256, 256, 256))
        self.b3 = block(256, 3, 1, 1, (384, 384, 384))
        self.b4 = block(384, 3, 1, 1, (1024, 1024, num_classes))

    def forward(self, x):
        x = F.max_pool2d(self.b1(x), 3, 2, ceil_mode=True)
        x = F.max_pool2d(self.b2(x), 3, 2, ceil_mode=True)
        x = F.max_pool2d(self.b3(x), 3, 2, ceil_mode=True)
        x = self.b4(F.dropout(x, 0.5, self.training))
        return F.adaptive_avg_pool2d(x, 1).flatten(1)


class LeNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.c1, self.c2 = nn.Conv2d(1, 20, 5), nn.Conv2d(20, 50, 5)
        self.f1, self.f2 = nn.Linear(800, 500), nn.Linear(500, 10)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.c1(x)), 2)
        x = F.max_pool2d(F.relu(self.c2(x)), 2)
        return self.f2(F.relu(self.f1(x.flatten(1))))


class CifarNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.c1, self.c2, self.c3 = nn.Conv2d(3, 32, 5, 1, 2), nn.Conv2d(32, 32, 5, 1, 2), nn.Conv2d(32, 64, 5, 1, 2)
        self.f = nn.Linear(576, 10)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.c1(x)), 3, 2)
        x = F.avg_pool2d(F.relu(self.c2(x)), 3, 2)
        x = F.avg_pool2d(F.relu(self.c3(x)), 3, 2)
        return self.f(x.flatten(1))


def _resnet18():
    import torchvision
    return torchvision.models.resnet18(weights=None, num_classes=1000)


# name: (constructor, side of the staged image, channels, classes, side of the random crop fed to the network)
MODELS = {"alexnet": (AlexNet, 227, 3, 1000, 227), "nin": (NiN, 224, 3, 1000, 224), "lenet": (LeNet, 28, 1, 10, 28),
          "cifar": (CifarNet, 32, 3, 10, 32), "resnet18": (_resnet18, 256, 3, 1000, 224)}


class TorchBaseline:
    """One data-parallel replica; `step(images_u8, labels)` does input cast, forward, backward, all-reduce, SGD.

    `variant` picks how stock PyTorch is driven, so that the comparison is against its best form, not its slowest:

    * ``eager``    fp32 parameters, bf16 autocast, one kernel launch per operator from Python;
    * ``graph``    the same step (input cast, forward, backward, DDP all-reduce, fused SGD) captured once in a CUDA
                   graph and replayed: no launch or Python overhead, like this framework's own engine;
    * ``bf16_graph`` the module held in bf16 outright (no autocast casts, no fp32 master: less work than this
                   framework does), channels-last, captured in a CUDA graph;
    * ``compiled`` ``torch.compile(mode="max-autotune-no-cudagraphs")`` of the network, step captured in a CUDA graph.
    """

    VARIANTS = ("eager", "graph", "bf16_graph", "compiled")

    def __init__(self, model="alexnet", batch=128, world=1, rank=0, device="cuda", lr=0.01, momentum=0.9, wd=5e-4,
                 variant="eager"):
        cls, hw, c, k, crop = MODELS[model]
        self.hw, self.c, self.k, self.batch, self.crop = hw, c, k, batch, crop
        self.device = torch.device(device)
        self.variant = variant
        self.world = world
        torch.manual_seed(0)
        net = cls().to(self.device).to(memory_format=torch.channels_last)
        self.pure_bf16 = variant == "bf16_graph"
        if self.pure_bf16:
            net = net.to(torch.bfloat16)
        if variant == "compiled":
            net = torch.compile(net, mode="max-autotune-no-cudagraphs")
        self._stream = None
        if world > 1:
            if variant != "eager":
                # a captured DDP step must never touch the legacy default stream: the wrapper is built, warmed up and
                # captured on one side stream (its reducer keeps the stream that was current at construction)
                self._stream = torch.cuda.Stream(self.device)
                self._stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self._stream):
                    net = torch.nn.parallel.DistributedDataParallel(net, device_ids=[self.device.index],
                                                                    bucket_cap_mb=25, gradient_as_bucket_view=True)
                torch.cuda.current_stream().wait_stream(self._stream)
            else:
                net = torch.nn.parallel.DistributedDataParallel(net, device_ids=[self.device.index], bucket_cap_mb=25,
                                                                gradient_as_bucket_view=True)
        self.net = net
        self.opt = torch.optim.SGD(net.parameters(), lr=lr, momentum=momentum, weight_decay=wd, fused=True)
        self.loss = None
        self.graph = None
        self._static_x = self._static_y = None

    # ---- the step itself (what a graph captures)
    def _compute(self, x_u8, y):
        if self.crop < self.hw:
            if self.graph is not None or self.variant != "eager":
                o = (self.hw - self.crop) // 2      # a captured step cannot draw on the host: centre crop
                x_u8 = x_u8[:, :, o:o + self.crop, o:o + self.crop]
            else:   # one random crop offset per batch + flip coin
                oy, ox = (int(v) for v in torch.randint(0, self.hw - self.crop + 1, (2,)))
                x_u8 = x_u8[:, :, oy:oy + self.crop, ox:ox + self.crop]
                if int(torch.randint(0, 2, (1,))):
                    x_u8 = x_u8.flip(-1)
        x = (x_u8.float() - 127.5) * (1.0 / 73.9)
        x = x.contiguous(memory_format=torch.channels_last)
        if self.pure_bf16:
            out = self.net(x.to(torch.bfloat16))
            loss = F.cross_entropy(out.float(), y)
        else:
            with torch.autocast("cuda", dtype=torch.bfloat16):
                out = self.net(x)
                loss = F.cross_entropy(out.float(), y)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        return loss

    def _capture(self, images_u8, labels):
        """Warm up on a side stream (DDP needs 11 eager iterations before a capture), then capture one step."""
        self._static_x = torch.zeros((self.batch, self.c, self.hw, self.hw), dtype=torch.uint8, device=self.device)
        self._static_y = torch.zeros((self.batch,), dtype=torch.long, device=self.device)
        self._static_x.copy_(images_u8, non_blocking=True)
        self._static_y.copy_(labels.long(), non_blocking=True)
        s = self._stream if self._stream is not None else torch.cuda.Stream(self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(11 if self.world > 1 else 3):
                self._compute(self._static_x, self._static_y)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        self.opt.zero_grad(set_to_none=True)
        with torch.cuda.graph(g, stream=s):
            self._static_loss = self._compute(self._static_x, self._static_y)
        self.graph = g

    def step(self, images_u8, labels):
        if self.variant == "eager":
            x = images_u8.to(self.device, non_blocking=True)
            y = labels.to(self.device, non_blocking=True).long()
            self.loss = self._compute(x, y)
            return self.loss
        if self.graph is None:
            self._capture(images_u8, labels)
        self._static_x.copy_(images_u8, non_blocking=True)
        self._static_y.copy_(labels, non_blocking=True)
        self.graph.replay()
        self.loss = self._static_loss
        return self.loss
