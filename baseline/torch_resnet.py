"""Stock PyTorch baseline for the data-parallel ResNet-50 configuration (no code from this
framework): ``nn.Conv2d`` / ``nn.BatchNorm2d`` (cuDNN), channels-last, bf16 autocast,
``DistributedDataParallel`` (NCCL, bucketed all-reduce overlapped with backward, uncompressed
gradients) and ``torch.optim.SGD`` with momentum 0.9."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class Bottleneck(nn.Module):
    def __init__(self, cin, width, stride=1, down=False):
        super().__init__()
        self.c1, self.b1 = nn.Conv2d(cin, width, 1, bias=False), nn.BatchNorm2d(width)
        self.c2 = nn.Conv2d(width, width, 3, stride, 1, bias=False)
        self.b2 = nn.BatchNorm2d(width)
        self.c3, self.b3 = nn.Conv2d(width, width * 4, 1, bias=False), nn.BatchNorm2d(width * 4)
        nn.init.zeros_(self.b3.weight)
        self.down = nn.Sequential(nn.Conv2d(cin, width * 4, 1, stride, bias=False),
                                  nn.BatchNorm2d(width * 4)) if down else None

    def forward(self, x):
        idt = x if self.down is None else self.down(x)
        out = F.relu(self.b1(self.c1(x)))
        out = F.relu(self.b2(self.c2(out)))
        return F.relu(self.b3(self.c3(out)) + idt)


class ResNet50(nn.Module):
    def __init__(self, classes=1000, layers=(3, 4, 6, 3)):
        super().__init__()
        self.conv1, self.bn1 = nn.Conv2d(3, 64, 7, 2, 3, bias=False), nn.BatchNorm2d(64)
        self.cin = 64
        self.layers = nn.Sequential(*[self._make(64 * 2 ** i, n, 1 if i == 0 else 2)
                                      for i, n in enumerate(layers)])
        self.fc = nn.Linear(2048, classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")

    def _make(self, width, blocks, stride):
        mods = [Bottleneck(self.cin, width, stride, stride != 1 or self.cin != width * 4)]
        self.cin = width * 4
        mods += [Bottleneck(self.cin, width) for _ in range(1, blocks)]
        return nn.Sequential(*mods)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.bn1(self.conv1(x))), 3, 2, 1)
        x = self.layers(x)
        return self.fc(F.adaptive_avg_pool2d(x, 1).flatten(1))


class TorchDDPTrainer:
    def __init__(self, device, world, rank, layers=(3, 4, 6, 3)):
        torch.manual_seed(1234)
        net = ResNet50(layers=layers).to(device).to(memory_format=torch.channels_last)
        self.net = nn.parallel.DistributedDataParallel(net, device_ids=[device.index]) \
            if world > 1 else net
        self.opt = torch.optim.SGD(self.net.parameters(), lr=0.1, momentum=0.9)

    def step(self, x, y):
        """``x``: [N, H, W, 3] bf16 (channels-last storage), ``y``: [N] int64."""
        x = x.permute(0, 3, 1, 2)          # NCHW view of channels-last memory
        self.opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = F.cross_entropy(self.net(x).float(), y)
        loss.backward()
        self.opt.step()
        return loss.detach()
