"""``broadcast_data``: the members of a model-parallel group train on the same batch; rank 0
of the group holds it and hands it to the others (listed, commented out, among the exports of
the reference's ``mpnn`` package, necklace/frmwrk/pytorch/mpnn/__init__.py:3; its trainers do
the same with ``dtdist.dt_shape_do_nccl_broadcast`` + ``dt_input_do_nccl_broadcast``,
necklace/trainer/tnoppt.py:285-317)."""
from __future__ import annotations

import torch

from ....data import dtdist
from . import initialize as mpu


def broadcast_data(keys, data, datatype, ndims=None, device=None):
    """``data``: dict of tensors on the group's rank 0 (anything on the others).  Returns a
    dict with the same keys on every member.  ``ndims``: number of dimensions per key
    (default 2, the ``[batch, sequence]`` token case)."""
    group = mpu.get_model_parallel_group()
    if group is None or mpu.get_model_parallel_world_size() == 1:
        return {k: data[k].to(datatype) for k in keys}
    is_root = mpu.get_model_parallel_rank() == 0
    if device is None:
        device = data[keys[0]].device if is_root else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
            else torch.device("cpu"))
    nd = [ndims.get(k, 2) if isinstance(ndims, dict) else (ndims or 2) for k in keys]
    out = dtdist.broadcast_batch([data[k] for k in keys] if is_root else [None] * len(keys), nd,
                                 [datatype] * len(keys), device, 0, group)
    return dict(zip(keys, out))
