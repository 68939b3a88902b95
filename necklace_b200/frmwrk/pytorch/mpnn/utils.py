"""Divisibility helpers and vocabulary range arithmetic
(reference: necklace/frmwrk/pytorch/mpnn/utils.py:4-70)."""
from __future__ import annotations

import torch


def ensure_divisibility(numerator, denominator):
    assert numerator % denominator == 0, f"{numerator} is not divisible by {denominator}"


def divide(numerator, denominator):
    ensure_divisibility(numerator, denominator)
    return numerator // denominator


def split_tensor_along_last_dim(tensor, num_partitions, contiguous_split_chunks=False):
    last = tensor.dim() - 1
    chunks = torch.split(tensor, divide(tensor.size(last), num_partitions), dim=last)
    return tuple(c.contiguous() for c in chunks) if contiguous_split_chunks else chunks


class VocabUtility:
    """[first, last) vocabulary index range owned by a rank."""

    @staticmethod
    def vocab_range_from_per_partition_vocab_size(per_partition_vocab_size, rank, world_size):
        first = rank * per_partition_vocab_size
        return first, first + per_partition_vocab_size

    @staticmethod
    def vocab_range_from_global_vocab_size(global_vocab_size, rank, world_size):
        return VocabUtility.vocab_range_from_per_partition_vocab_size(
            divide(global_vocab_size, world_size), rank, world_size)
