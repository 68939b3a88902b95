"""``MpiWrp``: what the launcher told this process, read from its environment; no MPI library
is needed.  The reference's ``mpirun`` example uses ``MpiWrp().world_size`` and ``.rank`` to
overwrite its ``-w`` / ``-k`` arguments (examples/dp/mnist/pytorch/
train_nklc_nccl_mnist_1_mpirun.py:241-246).

Launchers recognised (first that is set): Open MPI (``OMPI_COMM_WORLD_RANK`` / ``_SIZE`` /
``_LOCAL_RANK``), MPICH / Intel MPI (``PMI_RANK`` / ``PMI_SIZE``, ``MPI_LOCALRANKID``), Slurm
(``SLURM_PROCID`` / ``SLURM_NTASKS`` / ``SLURM_LOCALID``), torchrun (``RANK`` / ``WORLD_SIZE`` /
``LOCAL_RANK``).  Started by hand, a process is rank 0 of 1."""
from __future__ import annotations

import os

_ENV = (("OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_RANK"),
        ("PMI_RANK", "PMI_SIZE", "MPI_LOCALRANKID"),
        ("SLURM_PROCID", "SLURM_NTASKS", "SLURM_LOCALID"),
        ("RANK", "WORLD_SIZE", "LOCAL_RANK"))


def rank_size_from_env(env=None):
    """``(rank, world_size, local_rank or None, launcher variable or None)``."""
    env = os.environ if env is None else env
    for r, s, l in _ENV:
        if env.get(r) is not None and env.get(s) is not None:
            lr = env.get(l)
            return int(env[r]), int(env[s]), (int(lr) if lr is not None else None), r
    return 0, 1, None, None


class MpiWrp:
    def __init__(self, env=None):
        self.rank, self.world_size, self.local_rank, self.launcher = rank_size_from_env(env)

    # the few collective-shaped calls an MPI wrapper is asked for; they need the process
    # group that the trainer's communicator bring-up creates
    def barrier(self):
        import torch.distributed as dist
        if dist.is_initialized() and self.world_size > 1:
            dist.barrier()

    def do_all_reduce(self, send, recv=None, sz=None, *args, **kwargs):
        """Sum over all ranks of a CPU tensor / numpy array (into ``recv`` when given)."""
        import numpy as np
        import torch
        import torch.distributed as dist
        t = torch.from_numpy(send) if isinstance(send, np.ndarray) else send
        out = t if recv is None else (torch.from_numpy(recv) if isinstance(recv, np.ndarray) else recv)
        if out is not t:
            out.copy_(t)
        if dist.is_initialized() and self.world_size > 1:
            dist.all_reduce(out)
        return recv if recv is not None else send

    def stream_sync(self):
        pass
