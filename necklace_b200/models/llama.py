"""Llama-style decoder (RMSNorm, rotary embedding, SwiGLU, no biases) on the native
operators, with optional tensor parallelism (heads and FFN split over the mp group,
Megatron column -> row pairs) so the same module serves the ``dp+pp+mp`` and
``dp+zr+mp`` benchmark configurations.  The reference has no transformer model."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from ..ops import Embedding, RMSNorm, attention_qkv, linear, lm_head_loss
from ..ops.rotary import linear_rope, swiglu


@dataclass
class LlamaConfig:
    n_layer: int = 32
    d_model: int = 4096
    n_head: int = 32
    d_ff: int = 11008
    vocab: int = 32000
    max_seq: int = 2048
    rope_base: float = 10000.0
    dtype: torch.dtype = torch.bfloat16
    mp: int = 1          # tensor-parallel ways
    mp_rank: int = 0

    @staticmethod
    def llama7b(**kw):
        return LlamaConfig(**kw)

    @staticmethod
    def llama13b(**kw):
        return LlamaConfig(n_layer=40, d_model=5120, n_head=40, d_ff=13824, max_seq=4096, **kw)

    @staticmethod
    def tiny(**kw):
        return LlamaConfig(n_layer=2, d_model=256, n_head=4, d_ff=512, vocab=1000, max_seq=256, **kw)


def _shard(full: torch.Tensor, dim: int, mp: int, rank: int) -> torch.Tensor:
    return full if mp == 1 else full.chunk(mp, dim=dim)[rank].contiguous()


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig, layer: int, device=None, seed: int = 0):
        super().__init__()
        C, F, dt, mp, r = cfg.d_model, cfg.d_ff, cfg.dtype, cfg.mp, cfg.mp_rank
        assert cfg.n_head % mp == 0 and F % mp == 0
        self.cfg, self.n_head_local = cfg, cfg.n_head // mp
        self.ln1 = RMSNorm(C, dtype=dt, device=device)
        self.ln2 = RMSNorm(C, dtype=dt, device=device)
        g = torch.Generator().manual_seed(seed * 1000 + layer)
        mk = lambda o, i, s: torch.randn(o, i, generator=g) * s
        pstd = 0.02 / (2 * cfg.n_layer) ** 0.5
        wq, wk, wv = mk(C, C, 0.02), mk(C, C, 0.02), mk(C, C, 0.02)
        # column parallel: heads split over ranks; packed [q_local; k_local; v_local]
        wqkv = torch.cat([_shard(w, 0, mp, r) for w in (wq, wk, wv)], 0)
        wo = _shard(mk(C, C, pstd), 1, mp, r)            # row parallel
        wg, wu = _shard(mk(F, C, 0.02), 0, mp, r), _shard(mk(F, C, 0.02), 0, mp, r)
        wd = _shard(mk(C, F, pstd), 1, mp, r)
        P = lambda t: nn.Parameter(t.to(dt).to(device) if device is not None else t.to(dt))
        self.w_qkv, self.w_o = P(wqkv), P(wo)
        self.w_gu, self.w_down = P(torch.cat([wg, wu], 0)), P(wd)
        for p in (self.w_qkv, self.w_o, self.w_gu, self.w_down):
            p.model_parallel = mp > 1

    def _reduce(self, x):
        if self.cfg.mp == 1:
            return x
        from ..frmwrk.pytorch.mpnn.mappings import reduce_from_model_parallel_region
        return reduce_from_model_parallel_region(x)

    def _copy(self, x):
        if self.cfg.mp == 1:
            return x
        from ..frmwrk.pytorch.mpnn.mappings import copy_to_model_parallel_region
        return copy_to_model_parallel_region(x)

    def forward(self, x):
        h = self._copy(self.ln1(x))
        qkv = linear_rope(h, self.w_qkv, self.n_head_local, self.cfg.rope_base)
        a = attention_qkv(qkv, self.n_head_local, True)
        if self.cfg.mp == 1:
            x = linear(a, self.w_o, None, residual=x)
        else:
            x = x + self._reduce(linear(a, self.w_o))
        h = self._copy(self.ln2(x))
        f = swiglu(linear(h, self.w_gu))
        if self.cfg.mp == 1:
            return linear(f, self.w_down, None, residual=x)
        return x + self._reduce(linear(f, self.w_down))


class LlamaEmbed(nn.Module):
    def __init__(self, cfg, device=None):
        super().__init__()
        self.emb = Embedding((cfg.vocab + 127) // 128 * 128, cfg.d_model, None, dtype=cfg.dtype,
                             device=device)

    def forward(self, idx):
        return self.emb(idx)


class LlamaHead(nn.Module):
    def __init__(self, cfg, device=None):
        super().__init__()
        self.vocab = cfg.vocab
        self.norm = RMSNorm(cfg.d_model, dtype=cfg.dtype, device=device)
        vp = (cfg.vocab + 127) // 128 * 128
        self.w_out = nn.Parameter((torch.randn(vp, cfg.d_model, generator=torch.Generator()
                                               .manual_seed(7)) * 0.02).to(cfg.dtype)
                                  .to(device if device is not None else "cpu"))

    def forward(self, x, targets):
        return lm_head_loss(self.norm(x), self.w_out, targets, self.vocab)


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig, device=None, layers: range | None = None,
                 with_embed: bool = True, with_head: bool = True, seed: int = 0):
        """``layers`` / ``with_embed`` / ``with_head`` select a pipeline stage's slice."""
        super().__init__()
        self.cfg = cfg
        layers = range(cfg.n_layer) if layers is None else layers
        self.embed = LlamaEmbed(cfg, device) if with_embed else None
        self.blocks = nn.ModuleList(LlamaBlock(cfg, i, device, seed) for i in layers)
        self.head = LlamaHead(cfg, device) if with_head else None

    def forward(self, x, targets=None):
        if self.embed is not None:
            x = self.embed(x)
        for b in self.blocks:
            x = b(x)
        if self.head is not None and targets is not None:
            return self.head(x, targets)
        return x

    def num_params(self):
        return sum(p.numel() for p in self.parameters())
