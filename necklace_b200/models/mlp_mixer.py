"""MLP-Mixer cut into ``net_map`` units (input part, body parts, head part).

The reference's ZeRO examples train an MLP-Mixer on MNIST whose blocks are spread over
three or four sub-modules (examples/zero/mnist/pytorch/mlp_mixer.py:85-170,
train_mnist_zr_2_mlpmx.py).  This is the same architecture (patch embedding, ``depth``
mixer blocks of a token-mixing and a channel-mixing MLP with pre-norm and residuals, mean
pooling, linear classifier) written for this framework: the patch embedding is a
reshape + linear (no convolution needed for non-overlapping patches), and
``mixer_parts(n)`` returns the ``n`` units in execution order."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class MixerBlock(nn.Module):
    def __init__(self, dim, num_patch, token_dim, channel_dim):
        super().__init__()
        self.norm1, self.norm2 = nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.tok1, self.tok2 = nn.Linear(num_patch, token_dim), nn.Linear(token_dim, num_patch)
        self.ch1, self.ch2 = nn.Linear(dim, channel_dim), nn.Linear(channel_dim, dim)

    def forward(self, x):                                   # [B, P, C]
        y = self.norm1(x).transpose(1, 2)                   # mix over patches
        x = x + self.tok2(F.gelu(self.tok1(y))).transpose(1, 2)
        return x + self.ch2(F.gelu(self.ch1(self.norm2(x))))


class MixerInput(nn.Module):
    """Patch embedding + the first ``depth`` blocks."""

    def __init__(self, in_channels, dim, patch_size, image_size, depth, token_dim, channel_dim):
        super().__init__()
        assert image_size % patch_size == 0
        self.ps = patch_size
        self.num_patch = (image_size // patch_size) ** 2
        self.embed = nn.Linear(in_channels * patch_size * patch_size, dim)
        self.blocks = nn.ModuleList(MixerBlock(dim, self.num_patch, token_dim, channel_dim)
                                    for _ in range(depth))

    def forward(self, img):                                 # [B, C, H, W]
        B, C, H, W = img.shape
        p = self.ps
        x = img.view(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5).reshape(
            B, self.num_patch, C * p * p)
        x = self.embed(x)
        for b in self.blocks:
            x = b(x)
        return x


class MixerBody(nn.Module):
    def __init__(self, dim, num_patch, depth, token_dim, channel_dim):
        super().__init__()
        self.blocks = nn.ModuleList(MixerBlock(dim, num_patch, token_dim, channel_dim)
                                    for _ in range(depth))

    def forward(self, x):
        for b in self.blocks:
            x = b(x)
        return x


class MixerHead(MixerBody):
    def __init__(self, dim, num_patch, depth, token_dim, channel_dim, num_classes):
        super().__init__(dim, num_patch, depth, token_dim, channel_dim)
        self.norm = nn.LayerNorm(dim)
        self.fc = nn.Linear(dim, num_classes)

    def forward(self, x):
        x = super().forward(x)
        return self.fc(self.norm(x).mean(1))


def mixer_parts(n_parts=3, in_channels=1, image_size=28, patch_size=7, num_classes=10, dim=64,
                depth=6, token_dim=32, channel_dim=128, seed=0):
    """``n_parts`` units (>= 2) that share ``depth`` mixer blocks as evenly as possible."""
    assert n_parts >= 2
    torch.manual_seed(seed)
    per = [depth // n_parts + (1 if i < depth % n_parts else 0) for i in range(n_parts)]
    num_patch = (image_size // patch_size) ** 2
    parts = [MixerInput(in_channels, dim, patch_size, image_size, per[0], token_dim, channel_dim)]
    parts += [MixerBody(dim, num_patch, d, token_dim, channel_dim) for d in per[1:-1]]
    parts.append(MixerHead(dim, num_patch, per[-1], token_dim, channel_dim, num_classes))
    return parts


class MLPMixer(nn.Sequential):
    """The whole network (the parts in sequence): the single-process counterpart."""

    def __init__(self, **kw):
        super().__init__(*mixer_parts(**kw))
