"""Stock PyTorch baseline for the headline benchmark (no code from this framework).

GPT-2 in plain ``torch.nn`` (cuBLAS linears, ``scaled_dot_product_attention``,
``F.layer_norm``, ``F.cross_entropy``), bf16 weights with fp32 master weights and
fused ``torch.optim.AdamW``; ZeRO over all ranks with
``dist.reduce_scatter_tensor`` / ``dist.all_gather_into_tensor`` on flat buffers
(NCCL).  It stands in for the reference's own build, which cannot be installed
offline, as the "same trainer mode on stock torch.distributed" baseline.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

CONFIGS = {
    "gpt2-medium": dict(n_layer=24, d_model=1024, n_head=16, d_ff=4096, vocab=50257, max_seq=1024),
    "gpt2-tiny": dict(n_layer=2, d_model=128, n_head=2, d_ff=512, vocab=1000, max_seq=128),
}


class Block(nn.Module):
    def __init__(self, c):
        super().__init__()
        d = c["d_model"]
        self.h = c["n_head"]
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.fc1, self.fc2 = nn.Linear(d, c["d_ff"]), nn.Linear(c["d_ff"], d)

    def forward(self, x):
        B, S, C = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, S, 3, self.h, C // self.h).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(B, S, C))
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x)), approximate="tanh"))


class GPT2(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.vocab = c["vocab"]
        vp = (c["vocab"] + 127) // 128 * 128
        self.wte = nn.Embedding(vp, c["d_model"])
        nn.init.normal_(self.wte.weight, std=0.02)
        self.wpe = nn.Embedding(c["max_seq"], c["d_model"])
        self.blocks = nn.ModuleList(Block(c) for _ in range(c["n_layer"]))
        self.ln_f = nn.LayerNorm(c["d_model"])

    def forward(self, idx, targets):
        B, S = idx.shape
        x = self.wte(idx) + self.wpe(torch.arange(S, device=idx.device))
        for b in self.blocks:
            x = b(x)
        logits = F.linear(self.ln_f(x), self.wte.weight)[..., :self.vocab]
        return F.cross_entropy(logits.float().view(-1, self.vocab), targets.view(-1))


class TorchZeroTrainer:
    def __init__(self, model_name, device, world, rank):
        c = CONFIGS[model_name]
        self.vocab, self.max_seq = c["vocab"], c["max_seq"]
        self.world, self.rank = world, rank
        torch.manual_seed(1234)
        self.model = GPT2(c).to(device=device, dtype=torch.bfloat16)
        params = [p for p in self.model.parameters()]
        n = sum(p.numel() for p in params)
        pad = (-n) % (world * 8)
        self.n = n + pad
        self.flat = torch.zeros(self.n, dtype=torch.bfloat16, device=device)
        self.gflat = torch.zeros(self.n, dtype=torch.bfloat16, device=device)
        off = 0
        for p in params:
            self.flat[off:off + p.numel()].copy_(p.data.view(-1))
            p.data = self.flat[off:off + p.numel()].view(p.shape)
            p.grad = self.gflat[off:off + p.numel()].view(p.shape)
            off += p.numel()
        self.params = params
        shard = self.n // world
        self.shard = shard
        self.master = nn.Parameter(self.flat[rank * shard:(rank + 1) * shard].float())
        self.master.grad = torch.zeros_like(self.master)
        self.gshard = torch.zeros(shard, dtype=torch.bfloat16, device=device)
        self.opt = torch.optim.AdamW([self.master], lr=3e-4, betas=(0.9, 0.95), eps=1e-8,
                                     weight_decay=0.1, fused=True)

    def step(self, x, y):
        self.gflat.zero_()
        loss = self.model(x, y)
        loss.backward()
        if self.world > 1:
            dist.reduce_scatter_tensor(self.gshard, self.gflat, op=dist.ReduceOp.AVG)
            self.master.grad.copy_(self.gshard)
        else:
            self.master.grad.copy_(self.gflat)
        self.opt.step()
        mine = self.flat[self.rank * self.shard:(self.rank + 1) * self.shard]
        mine.copy_(self.master.data)
        if self.world > 1:
            dist.all_gather_into_tensor(self.flat, mine.clone())
        return loss.detach()
