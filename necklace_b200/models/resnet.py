"""ResNet-50 (bottleneck blocks [3, 4, 6, 3], 1000 classes) for the data-parallel
benchmark configuration.

Activations are channels-last bf16.  The 1x1 convolutions (about half of the model's
FLOPs) are plain GEMMs in that layout and run on the tcgen05 GEMM kernel
(``[N*H*W, C_in] @ W[C_out, C_in]^T``, no im2col, no copy); the 3x3 / 7x7 convolutions,
batch norm and pooling use PyTorch (cuDNN).  The reference itself only ships MNIST-sized
CNNs (examples/dp/mnist/pytorch/main.py); ResNet-50 comes from the benchmark configs.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import linear as nk_linear


class Conv1x1(nn.Module):
    """1x1 convolution as a GEMM over channels-last activations."""

    def __init__(self, cin, cout, stride=1):
        super().__init__()
        self.cin, self.cout, self.stride = cin, cout, stride
        self.weight = nn.Parameter(torch.empty(cout, cin))
        nn.init.kaiming_normal_(self.weight.view(cout, cin, 1, 1), mode="fan_out",
                                nonlinearity="relu")

    def forward(self, x):
        if self.stride > 1:
            x = x[:, :, ::self.stride, ::self.stride]
        if x.is_cuda and x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16:
            n, c, h, w = x.shape
            xl = x.permute(0, 2, 3, 1)
            if not xl.is_contiguous():
                xl = xl.contiguous()
            y = nk_linear(xl.reshape(-1, c), self.weight)
            return y.view(n, h, w, self.cout).permute(0, 3, 1, 2)
        return F.conv2d(x, self.weight.view(self.cout, self.cin, 1, 1).to(x.dtype))


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, cin, width, stride=1, downsample=None):
        super().__init__()
        self.conv1 = Conv1x1(cin, width)
        self.bn1 = nn.BatchNorm2d(width)
        self.conv2 = nn.Conv2d(width, width, 3, stride, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(width)
        self.conv3 = Conv1x1(width, width * 4)
        self.bn3 = nn.BatchNorm2d(width * 4)
        nn.init.zeros_(self.bn3.weight)
        self.downsample = downsample

    def forward(self, x):
        idt = x if self.downsample is None else self.downsample(x)
        out = F.relu(self.bn1(self.conv1(x)), inplace=True)
        out = F.relu(self.bn2(self.conv2(out)), inplace=True)
        out = self.bn3(self.conv3(out))
        return F.relu(out + idt, inplace=True)


class ResNet50(nn.Module):
    def __init__(self, classes: int = 1000, layers=(3, 4, 6, 3)):
        super().__init__()
        self.conv1 = nn.Conv2d(3, 64, 7, 2, 3, bias=False)
        self.bn1 = nn.BatchNorm2d(64)
        self.cin = 64
        self.layer1 = self._make(64, layers[0], 1)
        self.layer2 = self._make(128, layers[1], 2)
        self.layer3 = self._make(256, layers[2], 2)
        self.layer4 = self._make(512, layers[3], 2)
        self.fc = nn.Linear(2048, classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")

    def _make(self, width, blocks, stride):
        down = None
        if stride != 1 or self.cin != width * 4:
            down = nn.Sequential(Conv1x1(self.cin, width * 4, stride), nn.BatchNorm2d(width * 4))
        layers = [Bottleneck(self.cin, width, stride, down)]
        self.cin = width * 4
        layers += [Bottleneck(self.cin, width) for _ in range(1, blocks)]
        return nn.Sequential(*layers)

    def forward(self, x):
        x = F.relu(self.bn1(self.conv1(x)), inplace=True)
        x = F.max_pool2d(x, 3, 2, 1)
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        x = F.adaptive_avg_pool2d(x, 1).flatten(1)
        return self.fc(x)

    def parts(self):
        """``net_map`` units: stem + layer1, layer2, layer3, layer4 + head."""
        stem = nn.Sequential(self.conv1, self.bn1, nn.ReLU(inplace=True), nn.MaxPool2d(3, 2, 1),
                             self.layer1)
        head = nn.Sequential(self.layer4, nn.AdaptiveAvgPool2d(1), nn.Flatten(1), self.fc)
        return [stem, self.layer2, self.layer3, head]


class ResNetWithLoss(nn.Module):
    """``forward(images, labels) -> loss`` wrapper for the whole-step engine."""

    def __init__(self, net: nn.Module):
        super().__init__()
        self.net = net

    def forward(self, x, y):
        return F.cross_entropy(self.net(x).float(), y)
