"""Llama-style decoder (RMSNorm, rotary embedding, SwiGLU, no biases) on the native
operators, with optional tensor parallelism (heads and FFN split over the mp group,
Megatron column -> row pairs) so the same module serves the ``dp+pp+mp`` and
``dp+zr+mp`` benchmark configurations.  The reference has no transformer model.

Two tensor-parallel layouts:

``tp_group`` set (a ``PeerGroup``, or a ``TorchGroup`` as its unfused stand-in)
    Sequence-parallel layout on the fused kernels.  The residual stream between blocks is
    row-sharded (``[tokens/p, C]`` per rank); every column-parallel projection is one
    all-gather -> GEMM kernel, every row-parallel projection one GEMM -> reduce-scatter
    kernel (with the residual add in its epilogue), RMSNorm runs on the shard, the token
    embedding and the output projection + cross-entropy are vocabulary-parallel.  No NCCL
    call on the path.
``mp > 1`` without ``tp_group``
    The reference's layout (replicated activations, all-reduce after each row-parallel
    linear through ``mpnn.mappings``); kept as the NCCL baseline.
"""
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
    tp_group: object = None   # fused sequence-parallel path on this group (sets mp, mp_rank)

    def __post_init__(self):
        if self.tp_group is not None:
            self.mp, self.mp_rank = self.tp_group.world, self.tp_group.rank

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
        # full matrices are drawn from a per-layer seed and then sliced, so that every
        # tensor-parallel layout assembles into the same model; on a GPU they are drawn there
        # (a 7B-parameter stage takes minutes to draw on the host)
        gdev = torch.device(device) if device is not None and torch.device(device).type == "cuda" \
            else torch.device("cpu")
        g = torch.Generator(device=gdev).manual_seed(seed * 1000 + layer)
        mk = lambda o, i, s: torch.randn(o, i, generator=g, device=gdev) * s
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
        for p, dim, stride in ((self.w_qkv, 0, 3), (self.w_o, 1, 1), (self.w_gu, 0, 2),
                               (self.w_down, 1, 1)):
            p.model_parallel, p.partition_dim, p.partition_stride = mp > 1, dim, stride

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

    def forward_sp(self, x, batch):
        """``x``: this rank's ``[T/p, C]`` rows of the residual stream (T = batch * seq)."""
        from ..ops.rotary import rope
        from ..parallel.tensor import ag_linear, linear_rs
        g, cfg = self.cfg.tp_group, self.cfg
        qkv = ag_linear(self.ln1(x), self.w_qkv, None, g)               # [T, 3C/p]
        qkv = rope(qkv.view(batch, -1, qkv.shape[-1]), self.n_head_local, cfg.rope_base)
        a = attention_qkv(qkv, self.n_head_local, True)                 # [B, S, C/p]
        x = linear_rs(a.view(-1, a.shape[-1]), self.w_o, None, x, g)    # [T/p, C] (+ residual)
        f = swiglu(ag_linear(self.ln2(x), self.w_gu, None, g))          # [T, F/p]
        return linear_rs(f, self.w_down, None, x, g)

    def forward(self, x, batch=None):
        if self.cfg.tp_group is not None:
            return self.forward_sp(x, batch)
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


def _padded_vocab(cfg) -> int:
    q = 128 * cfg.mp
    return (cfg.vocab + q - 1) // q * q


class LlamaEmbed(nn.Module):
    """Token embedding; with ``tp_group`` the vocabulary rows are split over the group and the
    output is this rank's ``[T/p, C]`` rows."""

    def __init__(self, cfg, device=None):
        super().__init__()
        self.cfg = cfg
        vp = _padded_vocab(cfg)
        full = torch.randn(vp, cfg.d_model, generator=torch.Generator().manual_seed(5)) * 0.02
        if cfg.tp_group is not None:
            full = _shard(full, 0, cfg.mp, cfg.mp_rank)
        self.wte = nn.Parameter(full.to(cfg.dtype).to(device if device is not None else "cpu"))
        if cfg.tp_group is not None:
            self.wte.model_parallel, self.wte.partition_dim = cfg.mp > 1, 0

    def forward(self, idx):
        if self.cfg.tp_group is not None:
            from ..parallel.tensor import vocab_parallel_embed
            return vocab_parallel_embed(idx, self.wte, self.cfg.tp_group)
        from ..ops.loss import EmbedFn
        return EmbedFn.apply(idx, self.wte, None)


class LlamaHead(nn.Module):
    """Final norm, output projection and mean cross-entropy; vocabulary-parallel with
    ``tp_group`` (reference counterpart: ``VocabParallelEmbedding`` + all-reduce,
    necklace/frmwrk/pytorch/mpnn/layers.py:75-131)."""

    def __init__(self, cfg, device=None):
        super().__init__()
        self.cfg = cfg
        self.vocab = cfg.vocab
        self.norm = RMSNorm(cfg.d_model, dtype=cfg.dtype, device=device)
        vp = _padded_vocab(cfg)
        full = torch.randn(vp, cfg.d_model, generator=torch.Generator().manual_seed(7)) * 0.02
        if cfg.tp_group is not None:
            full = _shard(full, 0, cfg.mp, cfg.mp_rank)
        self.w_out = nn.Parameter(full.to(cfg.dtype).to(device if device is not None else "cpu"))
        if cfg.tp_group is not None:
            self.w_out.model_parallel, self.w_out.partition_dim = cfg.mp > 1, 0

    def forward(self, x, targets):
        if self.cfg.tp_group is not None:
            from ..parallel.tensor import vocab_parallel_lm_head_loss
            return vocab_parallel_lm_head_loss(self.norm(x), self.w_out, targets, self.vocab,
                                               self.cfg.tp_group)
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

    def forward(self, x, targets=None, batch=None):
        """First stage: ``x`` = token ids ``[B, S]``; later stages: the previous stage's
        activations.  With ``tp_group`` activations are ``[B*S/p, C]`` row shards and
        ``batch`` (= B) must accompany them on stages without the embedding."""
        if self.embed is not None:
            batch = x.shape[0]
            x = self.embed(x)
        for b in self.blocks:
            x = b(x, batch) if self.cfg.tp_group is not None else b(x)
        if self.head is not None and targets is not None:
            return self.head(x, targets)
        return x

    def num_params(self):
        return sum(p.numel() for p in self.parameters())

    def make_grad_sync(self):
        """Callable for ``TrainEngine(grad_sync=...)``: with the fused tensor-parallel layout
        the norm weights' gradients must be summed over the group once per step (see
        ``parallel.tensor.ReplicatedGradSync``).  None when there is nothing to do."""
        g = self.cfg.tp_group
        if g is None or g.world == 1:
            return None
        from ..parallel.tensor import ReplicatedGradSync
        rep = [p for p in self.parameters() if not getattr(p, "model_parallel", False)]
        return ReplicatedGradSync(rep, g)
