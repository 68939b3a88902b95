"""ResNet-50 (bottleneck blocks [3, 4, 6, 3], 1000 classes) for the data-parallel
benchmark configuration, entirely on this library's kernels.

Activations are channels-last (``[N, H, W, C]``) bf16.  Every convolution is a GEMM on the
tcgen05 kernel: the 1x1 ones on the activation matrix as it is, the 3x3 / 7x7 / strided
ones on a gathered ``col`` matrix (``ops.conv``); batch norm, the residual add and ReLU
are one fused kernel after the statistics pass; max / average pooling, the classifier and
its cross-entropy are native kernels as well, so the step contains no cuDNN call.  The
reference itself only ships MNIST-sized CNNs (examples/dp/mnist/pytorch/main.py); ResNet-50
comes from the benchmark configurations.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops.conv import BatchNorm2d, Conv2d, global_avg_pool, max_pool_3x3_s2
from ..ops.loss import lm_head_loss


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, cin, width, stride=1, downsample=False, device=None):
        super().__init__()
        self.conv1 = Conv2d(cin, width, 1, device=device)
        self.bn1 = BatchNorm2d(width, relu=True, device=device)
        self.conv2 = Conv2d(width, width, 3, stride, 1, device=device)
        self.bn2 = BatchNorm2d(width, relu=True, device=device)
        self.conv3 = Conv2d(width, width * 4, 1, device=device)
        self.bn3 = BatchNorm2d(width * 4, relu=True, zero_init=True, device=device)  # + residual
        self.down_conv = self.down_bn = None
        if downsample:
            self.down_conv = Conv2d(cin, width * 4, 1, stride, 0, device=device)
            self.down_bn = BatchNorm2d(width * 4, device=device)

    def forward(self, x):
        idt = x if self.down_conv is None else self.down_bn(self.down_conv(x))
        out = self.bn1(self.conv1(x))
        out = self.bn2(self.conv2(out))
        return self.bn3(self.conv3(out), residual=idt)


class ResNet(nn.Module):
    def __init__(self, classes: int = 1000, layers=(3, 4, 6, 3), width: int = 64, device=None):
        super().__init__()
        self.classes = classes
        self.conv1 = Conv2d(3, width, 7, 2, 3, device=device)
        self.bn1 = BatchNorm2d(width, relu=True, device=device)
        self.cin = width
        self.layer1 = self._make(width, layers[0], 1, device)
        self.layer2 = self._make(width * 2, layers[1], 2, device)
        self.layer3 = self._make(width * 4, layers[2], 2, device)
        self.layer4 = self._make(width * 8, layers[3], 2, device)
        cp = (classes + 127) // 128 * 128
        feat = width * 8 * 4
        w = torch.zeros(cp, feat)
        nn.init.kaiming_uniform_(w[:classes], a=5 ** 0.5)
        self.fc_weight = nn.Parameter(w.bfloat16().to(device) if device is not None
                                      else w.bfloat16())
        self.fc_bias = nn.Parameter(torch.zeros(cp, dtype=torch.bfloat16, device=device))

    def _make(self, width, blocks, stride, device):
        mods = [Bottleneck(self.cin, width, stride, stride != 1 or self.cin != width * 4, device)]
        self.cin = width * 4
        mods += [Bottleneck(self.cin, width, device=device) for _ in range(1, blocks)]
        return nn.Sequential(*mods)

    def features(self, x):
        """``x``: images ``[N, 3, H, W]`` (any float dtype) or NHWC bf16."""
        if x.dim() == 4 and x.shape[1] == 3 and x.shape[-1] != 3:
            x = x.permute(0, 2, 3, 1)
        x = x.to(torch.bfloat16).contiguous()
        x = max_pool_3x3_s2(self.bn1(self.conv1(x)))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return global_avg_pool(x)

    def forward(self, x, labels=None):
        f = self.features(x)
        if labels is None:
            from ..ops.gemm import gemm
            return gemm(f, self.fc_weight, bias=self.fc_bias)[:, :self.classes]
        return lm_head_loss(f, self.fc_weight, labels, self.classes, self.fc_bias)


def ResNet50(classes: int = 1000, device=None):
    return ResNet(classes, (3, 4, 6, 3), 64, device)


class ResNetWithLoss(nn.Module):
    """``forward(images, labels) -> loss`` wrapper for the whole-step engine."""

    def __init__(self, net: nn.Module):
        super().__init__()
        self.net = net

    def forward(self, x, y):
        return self.net(x, y)
