"""Module wrapper that fetches the owner's weights before forward and returns the
gradients to the owner in backward (the reference leaves this class as a stub,
necklace/frmwrk/pytorch/zrnn/zrmdwrp.py:10-27)."""
from __future__ import annotations

import torch.nn as nn

from .zrfn import zr_pg_bcast, zr_pg_reduce


class ZrModuleWrapper(nn.Module):
    def __init__(self, net, owner_rank=0):
        super().__init__()
        self.net, self.owner_rank = net, owner_rank

    def fetch_weights(self):
        for p in self.net.parameters():
            zr_pg_bcast(p.data, self.owner_rank)

    def return_grads(self):
        for p in self.net.parameters():
            if p.grad is not None:
                zr_pg_reduce(p.grad, self.owner_rank)

    def forward(self, *args, **kwargs):
        self.fetch_weights()
        return self.net(*args, **kwargs)
