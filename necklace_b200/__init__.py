"""necklace_b200: a Blackwell-native hybrid-parallel training framework.

Scheduler + one worker process per GPU, a ZeroMQ control plane, the trainer
modes ``no / dp / pp / mp / zr`` and their mixes, Megatron-style tensor-parallel
layers, and hand-written sm_100a kernels for the hot paths.
"""
from __future__ import annotations

__version__ = "0.1.0"


def init_mp() -> None:
    """Force the ``spawn`` start method so worker processes never inherit a CUDA
    context by fork (same purpose as the reference's ``necklace.init_mp``,
    necklace/__init__.py:8-13)."""
    import multiprocessing as mp
    try:
        mp.set_start_method("spawn", force=True)
    except RuntimeError:
        pass


def init_nb(gpu_dev_i: int | str = 0) -> None:
    """Make GPU ``gpu_dev_i`` the current device before anything else touches it (the
    reference selects the numba device here, necklace/__init__.py:19-30; no numba kernels
    remain, so this selects the torch device)."""
    import torch
    if torch.cuda.is_available():
        torch.cuda.set_device(int(gpu_dev_i))


def init(gpu_dev_i: int | str = 0) -> None:
    """Process-wide initialisation: spawn start method and device selection
    (reference: necklace/__init__.py:34-38)."""
    init_mp()
    init_nb(gpu_dev_i)
