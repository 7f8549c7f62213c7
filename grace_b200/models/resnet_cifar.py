"""ResNet-20 for 32x32 inputs (He et al. 2015, CIFAR variant): a 3x3 stem with
16 channels, three stages of three basic blocks at 16/32/64 channels with
stride-2 transitions, BatchNorm + ReLU, global average pool, 64->10 linear
(about 0.27 M parameters).  This is the plumbing model of the benchmark
configs; the reference's own example network is the DAWNBench ResNet-9
(``examples/dist/CIFAR10-dawndist/dawn.py:26-63``), available as ``resnet9``.
"""
import torch
from torch import nn
import torch.nn.functional as F


class BasicBlock(nn.Module):
    def __init__(self, cin, cout, stride):
        super().__init__()
        self.conv1 = nn.Conv2d(cin, cout, 3, stride, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(cout)
        self.conv2 = nn.Conv2d(cout, cout, 3, 1, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(cout)
        self.down = None
        if stride != 1 or cin != cout:
            self.down = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, bias=False), nn.BatchNorm2d(cout))

    def forward(self, x):
        y = F.relu(self.bn1(self.conv1(x)))
        y = self.bn2(self.conv2(y))
        return F.relu(y + (x if self.down is None else self.down(x)))


class ResNetCifar(nn.Module):
    def __init__(self, blocks_per_stage=3, num_classes=10, widths=(16, 32, 64)):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv2d(3, widths[0], 3, 1, 1, bias=False), nn.BatchNorm2d(widths[0]), nn.ReLU())
        layers, cin = [], widths[0]
        for i, w in enumerate(widths):
            for b in range(blocks_per_stage):
                layers.append(BasicBlock(cin, w, 2 if (b == 0 and i > 0) else 1))
                cin = w
        self.layers = nn.Sequential(*layers)
        self.fc = nn.Linear(cin, num_classes)

    def forward(self, x):
        x = self.layers(self.stem(x))
        return self.fc(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))


def resnet20(num_classes=10):
    return ResNetCifar(3, num_classes)


class _Res9Block(nn.Module):
    def __init__(self, cin, cout, pool=True):
        super().__init__()
        mods = [nn.Conv2d(cin, cout, 3, 1, 1, bias=False), nn.BatchNorm2d(cout), nn.ReLU()]
        if pool:
            mods.append(nn.MaxPool2d(2))
        self.body = nn.Sequential(*mods)

    def forward(self, x):
        return self.body(x)


class ResNet9(nn.Module):
    """DAWNBench-style ResNet-9: prep 64 -> 128 (+residual) -> 256 -> 512
    (+residual) -> max-pool -> linear scaled by 0.125."""

    def __init__(self, num_classes=10):
        super().__init__()
        self.prep = _Res9Block(3, 64, pool=False)
        self.l1 = _Res9Block(64, 128)
        self.r1 = nn.Sequential(_Res9Block(128, 128, False), _Res9Block(128, 128, False))
        self.l2 = _Res9Block(128, 256)
        self.l3 = _Res9Block(256, 512)
        self.r3 = nn.Sequential(_Res9Block(512, 512, False), _Res9Block(512, 512, False))
        self.fc = nn.Linear(512, num_classes, bias=False)

    def forward(self, x):
        x = self.l1(self.prep(x))
        x = x + self.r1(x)
        x = self.l3(self.l2(x))
        x = x + self.r3(x)
        x = F.adaptive_max_pool2d(x, 1).flatten(1)
        return self.fc(x) * 0.125


def resnet9(num_classes=10):
    return ResNet9(num_classes)
