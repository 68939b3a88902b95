"""Cross entropy over logits whose last (vocabulary) dimension is split over the
model-parallel group.  The reference lists ``vocab_parallel_cross_entropy`` among the exports
of its ``mpnn`` package but ships them commented out (necklace/frmwrk/pytorch/mpnn/
__init__.py:1); this is the operation its ``VocabParallelEmbedding`` / column-parallel output
layers need to train without gathering the logits.

Three small all-reduces over the group per call (row maximum, the target's logit, the sum of
exponentials); the backward needs none.  The fused kernel form of the same arithmetic, where
the logits never exist in full precision, is ``parallel.tensor.VocabParallelLMHeadLossFn``."""
from __future__ import annotations

import torch

from ....comm import fns
from . import initialize as mpu
from .utils import VocabUtility


class _VocabParallelCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target):
        group = mpu.get_model_parallel_group()
        ws, rank = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
        x = logits.float()
        mx = x.max(dim=-1).values
        if ws > 1:
            fns.all_reduce(mx, op="max", group=group)
        x = x - mx.unsqueeze(-1)
        per = x.size(-1)
        first, last = VocabUtility.vocab_range_from_per_partition_vocab_size(per, rank, ws)
        mine = (target >= first) & (target < last)
        local = (target - first).clamp(0, per - 1)
        picked = x.gather(-1, local.unsqueeze(-1)).squeeze(-1) * mine
        ex = x.exp()
        denom = ex.sum(dim=-1)
        if ws > 1:
            fns.all_reduce(picked, group=group)
            fns.all_reduce(denom, group=group)
        loss = denom.log() - picked
        ctx.save_for_backward(ex / denom.unsqueeze(-1), mine, local)
        ctx.in_dtype = logits.dtype
        return loss

    @staticmethod
    def backward(ctx, grad_out):
        softmax, mine, local = ctx.saved_tensors
        g = softmax.clone()
        g.scatter_add_(-1, local.unsqueeze(-1), -mine.unsqueeze(-1).to(g.dtype))
        return (g * grad_out.unsqueeze(-1)).to(ctx.in_dtype), None


def vocab_parallel_cross_entropy(vocab_parallel_logits, target):
    """Per-token loss ``[...]`` from ``[..., vocab / p]`` logits and global target ids."""
    return _VocabParallelCrossEntropy.apply(vocab_parallel_logits, target)
