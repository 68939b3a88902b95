"""GPT-2 style decoder built on the native operators.

Every matmul is the tcgen05 GEMM (bias, GELU and the residual add run in GEMM
epilogues), attention reads Q/K/V in place from the fused projection, and the
LM head is fused with the cross-entropy loss (bf16 logits become their own
gradient in place).  The model can be cut into ``net_map`` units
(embedding / blocks / head) for the pipeline and ZeRO trainers.

The reference ships only MNIST-sized models (e.g. examples/zero/mnist/pytorch/
mlp_mixer.py:85-170); this family exists for the transformer benchmark configs.
"""
from __future__ import annotations

from dataclasses import dataclass

import os

import torch
import torch.nn as nn

from ..ops import Embedding, LayerNorm, attention_qkv, linear, lm_head_loss, mlp


@dataclass
class GPT2Config:
    n_layer: int = 24
    d_model: int = 1024
    n_head: int = 16
    d_ff: int = 4096
    vocab: int = 50257
    max_seq: int = 1024
    dtype: torch.dtype = torch.bfloat16

    @property
    def vocab_padded(self) -> int:
        return (self.vocab + 127) // 128 * 128

    @staticmethod
    def medium() -> "GPT2Config":
        return GPT2Config()

    @staticmethod
    def tiny() -> "GPT2Config":
        return GPT2Config(n_layer=2, d_model=128, n_head=2, d_ff=512, vocab=1000, max_seq=128)


# NKB_NORM_SPLIT=0 falls back to plain norms (autograd then adds the residual-path gradient
# with a separate kernel); kept as a switch for A/B timing.
_NORM_SPLIT = os.environ.get("NKB_NORM_SPLIT", "1") != "0"


class Block(nn.Module):
    def __init__(self, cfg: GPT2Config, device=None):
        super().__init__()
        C, dt = cfg.d_model, cfg.dtype
        self.n_head = cfg.n_head
        self.ln1 = LayerNorm(C, dtype=dt, device=device)
        self.ln2 = LayerNorm(C, dtype=dt, device=device)
        std = 0.02
        pstd = 0.02 / (2 * cfg.n_layer) ** 0.5
        mk = lambda o, i, s: nn.Parameter(torch.randn(o, i, device=device).mul_(s).to(dt))
        zb = lambda o: nn.Parameter(torch.zeros(o, dtype=dt, device=device))
        self.w_qkv, self.b_qkv = mk(3 * C, C, std), zb(3 * C)
        self.w_proj, self.b_proj = mk(C, C, pstd), zb(C)
        self.w_fc1, self.b_fc1 = mk(cfg.d_ff, C, std), zb(cfg.d_ff)
        self.w_fc2, self.b_fc2 = mk(C, cfg.d_ff, pstd), zb(C)

    def forward(self, x):
        if not _NORM_SPLIT:
            h = self.ln1(x)
        else:
            x, h = self.ln1.split(x)  # the residual-path gradient is added in the norm backward
        qkv = linear(h, self.w_qkv, self.b_qkv)
        a = attention_qkv(qkv, self.n_head, True)
        x = linear(a, self.w_proj, self.b_proj, residual=x)
        if not _NORM_SPLIT:
            h = self.ln2(x)
        else:
            x, h = self.ln2.split(x)
        return mlp(h, self.w_fc1, self.b_fc1, self.w_fc2, self.b_fc2, residual=x, act="gelu")


class GPT2Embed(nn.Module):
    def __init__(self, cfg: GPT2Config, device=None):
        super().__init__()
        self.emb = Embedding(cfg.vocab_padded, cfg.d_model, cfg.max_seq, dtype=cfg.dtype,
                             device=device)

    def forward(self, idx):
        return self.emb(idx)


class GPT2Head(nn.Module):
    """Final LayerNorm + LM head (+ loss).  ``wte`` is shared with the embedding when
    both live in the same process; a pipeline stage that holds only the head owns
    its own copy."""

    computes_loss = True      # forward(x, targets) -> loss (see zroppt's native engine)

    def __init__(self, cfg: GPT2Config, wte: nn.Parameter | None = None, device=None):
        super().__init__()
        self.vocab = cfg.vocab
        self.ln_f = LayerNorm(cfg.d_model, dtype=cfg.dtype, device=device)
        if wte is None:
            wte = nn.Parameter(torch.randn(cfg.vocab_padded, cfg.d_model, device=device)
                               .mul_(0.02).to(cfg.dtype))
        self.wte = wte

    def forward(self, x, targets):
        return lm_head_loss(self.ln_f(x), self.wte, targets, self.vocab)

    def logits(self, x):
        return linear(self.ln_f(x), self.wte)[..., :self.vocab]


class GPT2(nn.Module):
    def __init__(self, cfg: GPT2Config, device=None):
        super().__init__()
        self.cfg = cfg
        self.embed = GPT2Embed(cfg, device)
        self.blocks = nn.ModuleList(Block(cfg, device) for _ in range(cfg.n_layer))
        self.head = GPT2Head(cfg, self.embed.emb.wte, device)

    def forward(self, idx, targets=None):
        x = self.embed(idx)
        for blk in self.blocks:
            x = blk(x)
        if targets is None:
            return self.head.logits(x)
        return self.head(x, targets)

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def flops_per_token(self, seq: int) -> float:
        """Training FLOPs per token (fwd+bwd), attention counted causal."""
        c = self.cfg
        dense = 2 * c.n_layer * (4 * c.d_model ** 2 + 2 * c.d_model * c.d_ff) \
            + 2 * c.d_model * c.vocab_padded
        attn = 2 * 2 * c.n_layer * seq * c.d_model / 2
        return 3.0 * (dense + attn)

    def net_map_units(self):
        """Units in execution order for pipeline / ZeRO partitioning."""
        return [self.embed, *self.blocks, self.head]
