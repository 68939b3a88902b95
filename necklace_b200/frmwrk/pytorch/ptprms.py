"""Parameter / gradient / tensor traffic for the DP, PP and ZeRO trainers.

Function names and call shapes follow the reference module
(necklace/frmwrk/pytorch/ptprms.py:18-450); ``nc`` is a group (``GroupInfo``) or None
for "data-parallel group, else main group".  What changed underneath:

* parameter averaging and broadcast are bucketed (one collective per 256 MB bucket
  instead of one per parameter tensor);
* collectives are ordered on the current stream, with no device-wide
  synchronisation around them;
* ``grad_comp_cfg`` is honoured: gradients go through the 2-bit threshold codec with
  error feedback (residuals kept per bucket) and only the codes cross the wire (the
  reference reads the config but never uses it, ptprms.py:319-338);
* point-to-point tensors carry their own dtype (the reference hard-codes fp32
  activations and int64 targets).
"""
from __future__ import annotations

import numpy as np
import torch

from ...comm import fns, groups as G
from ...ops.quant import dequantize_flat, quantize_flat

broadcast_bucket_size = 10 * 1024 * 1024
nccl_reduce_bucket_size = 256 * 1024 * 1024

_RESIDUALS: dict = {}


def _group(nc):
    return nc if nc is not None else G.get_nccl_group_dp_or_main()


# -- numpy state for RPC ---------------------------------------------------------
def get_weights(model):
    return {k: v.detach().float().cpu().numpy() for k, v in model.state_dict().items()}


def set_weights(model, weights):
    sd = model.state_dict()
    for k, v in weights.items():
        sd[k].copy_(torch.as_tensor(np.asarray(v)).to(sd[k].dtype))


def collect_gradients_by_optimizer(optimizer):
    opts = optimizer if isinstance(optimizer, (list, tuple)) else [optimizer]
    return [p.grad for o in opts for g in o.param_groups for p in g["params"]
            if p.grad is not None]


def collect_gradients_by_parameters(model):
    return [p.grad for p in model.parameters() if p.grad is not None]


def grads_get(model):
    return {n: p.grad.detach().float().cpu().numpy() for n, p in model.named_parameters()
            if p.grad is not None}


# -- buckets -----------------------------------------------------------------------
def _take_tensors(tensors, size_limit):
    """Group tensors (same dtype per bucket) into buckets of at most ``size_limit`` bytes."""
    by_type: dict = {}
    for t in tensors:
        by_type.setdefault((t.dtype, t.device), []).append(t)
    for ts in by_type.values():
        bucket, size = [], 0
        for t in ts:
            nbytes = t.numel() * t.element_size()
            if bucket and size + nbytes > size_limit:
                yield bucket
                bucket, size = [], 0
            bucket.append(t)
            size += nbytes
        if bucket:
            yield bucket


def _flatten(bucket):
    return torch.cat([t.reshape(-1) for t in bucket])


def _unflatten_into(flat, bucket):
    off = 0
    for t in bucket:
        n = t.numel()
        t.copy_(flat[off:off + n].view_as(t))
        off += n


def compressed_allreduce(flat, key, thr, group):
    """Sum over the group of the 2-bit coded ``flat`` (+ residual kept under ``key``)."""
    res = _RESIDUALS.get(key)
    if res is None or res.numel() != flat.numel() or res.device != flat.device:
        res = torch.zeros(flat.numel(), dtype=torch.float32, device=flat.device)
        _RESIDUALS[key] = res
    src = flat if flat.dtype in (torch.float32, torch.bfloat16) else flat.float()
    codes = quantize_flat(src.contiguous(), res, thr)
    ws = G.get_world_size(group)
    if ws > 1:
        allc = torch.empty(ws, codes.numel(), dtype=codes.dtype, device=codes.device)
        fns.all_gather(allc, codes, group=group)
    else:
        allc = codes.view(1, -1)
    out = torch.zeros(flat.numel(), dtype=torch.float32, device=flat.device)
    for r in range(ws):
        dequantize_flat(allc[r].contiguous(), out, thr, accumulate=True)
    return out


def nccl_allreduce_by_buckets(nc, kn, all_grads, grad_comp_cfg=None, average=True):
    group = _group(nc)
    for bi, bucket in enumerate(_take_tensors(all_grads, nccl_reduce_bucket_size)):
        flat = _flatten(bucket) if len(bucket) > 1 or not bucket[0].is_contiguous() \
            else bucket[0].view(-1)
        if grad_comp_cfg and flat.numel() >= int(grad_comp_cfg.get("grad_size_threshold", 0)):
            red = compressed_allreduce(flat, ("ar", id(group), bi, flat.numel()),
                                       float(grad_comp_cfg.get("grad_comp_threshold", 0.5)), group)
            flat = red.to(bucket[0].dtype)
        else:
            fns.all_reduce(flat, group=group)
        if average and kn > 1:
            flat = flat / kn if flat.is_floating_point() else flat
        if flat.data_ptr() != bucket[0].data_ptr() or len(bucket) > 1:
            _unflatten_into(flat, bucket)
        else:
            bucket[0].copy_(flat.view_as(bucket[0]))


def nccl_reduce_by_buckets(nc, kn, root, all_grads):
    """Sum to ``root`` of the group (no averaging, like the reference: ptprms.py:387)."""
    group = _group(nc)
    for bucket in _take_tensors(all_grads, nccl_reduce_bucket_size):
        flat = _flatten(bucket)
        fns.reduce(flat, root, group=group)
        if G.get_rank(group) == root:
            _unflatten_into(flat, bucket)


# -- parameters --------------------------------------------------------------------
def init_params_recvs(model):
    return None  # receive buffers are not needed: collectives run in place


def params_do_nccl_allreduce(nc, kn, model, prm_revs=None):
    """Average the weights over the group (initial weight sync; ``typ='weig'`` mode)."""
    params = [p.data for p in model.parameters()]
    nccl_allreduce_by_buckets(nc, kn, params, average=True)


def params_do_nccl_broadcast(nc, kn, root, model, prm_revs=None):
    group = _group(nc)
    params = [p.data for p in model.parameters()]
    for bucket in _take_tensors(params, nccl_reduce_bucket_size):
        flat = _flatten(bucket)
        fns.broadcast(flat, root, group=group)
        if G.get_rank(group) != root:
            _unflatten_into(flat, bucket)


def params_fltn_do_nccl_broadcast(nc, kn, root, d_arr_send, sz=None):
    flat = d_arr_send if sz is None else d_arr_send[:sz]
    fns.broadcast(flat, root, group=_group(nc))


# -- gradients -----------------------------------------------------------------------
def grads_do_nccl_allreduce(nc, kn, model, prm_revs=None, grad_comp_cfg=None):
    nccl_allreduce_by_buckets(nc, kn, collect_gradients_by_parameters(model), grad_comp_cfg)


def opt_one_grads_do_nccl_allreduce(nc, kn, opt, prm_revs=None, grad_comp_cfg=None):
    nccl_allreduce_by_buckets(nc, kn, collect_gradients_by_optimizer(opt), grad_comp_cfg)


def opt_grads_do_nccl_allreduce(nc, kn, opt, prm_revs=None, grad_comp_cfg=None):
    for o in (opt if isinstance(opt, (list, tuple)) else [opt]):
        opt_one_grads_do_nccl_allreduce(nc, kn, o, prm_revs, grad_comp_cfg)


def opt_one_grads_do_nccl_reduce(nc, kn, root, opt, prm_revs=None, grad_comp_cfg=None):
    nccl_reduce_by_buckets(nc, kn, root, collect_gradients_by_optimizer(opt))


def opt_grads_do_nccl_reduce(nc, kn, root, opt, prm_revs=None, grad_comp_cfg=None):
    for o in (opt if isinstance(opt, (list, tuple)) else [opt]):
        opt_one_grads_do_nccl_reduce(nc, kn, root, o, prm_revs, grad_comp_cfg)


def opt_grads_fltn_do_nccl_reduce(nc, kn, root, d_arr_send, sz=None, grad_comp_cfg=None):
    flat = d_arr_send if sz is None else d_arr_send[:sz]
    fns.reduce(flat, root, group=_group(nc))


# -- point to point ------------------------------------------------------------------
def init_tensors_recv(shps, ctx=None, dtype=torch.float32, dtypes=None):
    dev = ctx if ctx is not None else "cpu"
    dts = dtypes or [dtype] * len(shps)
    return [torch.zeros(tuple(s), dtype=dt, device=dev) for s, dt in zip(shps, dts)]


def tensors_do_nccl_p2p_send(nc, rank_send, rank_recv, send_tensors, dtype=None):
    """Send every tensor to global rank ``rank_recv`` (all posted, then waited)."""
    works = [fns.send(t, rank_recv) for t in send_tensors]
    for w in works:
        w.wait()


def tensors_do_nccl_p2p_recv(nc, rank_send, rank_recv, recv_tensors, dtype=None):
    works = [fns.recv(t, rank_send) for t in recv_tensors]
    for w in works:
        w.wait()
    return recv_tensors


def nccl_nc_allreduce(nc, p_arr_send, p_arr_recv, sz=None):
    """``p_arr_recv`` = sum over the group of ``p_arr_send`` (tensors where the reference
    passes device addresses, necklace/frmwrk/pytorch/ptprms.py:85-92)."""
    if p_arr_recv.data_ptr() != p_arr_send.data_ptr():
        p_arr_recv.copy_(p_arr_send)
    fns.all_reduce(p_arr_recv, group=_group(nc))
    return p_arr_recv


nccl_pg_allreduce = nccl_nc_allreduce


def nccl_pg_broadcast(pg, p_arr_send, p_arr_recv, sz=None, root=0):
    if p_arr_recv.data_ptr() != p_arr_send.data_ptr():
        p_arr_recv.copy_(p_arr_send)
    fns.broadcast(p_arr_recv, root, _group(pg))
    return p_arr_recv


def nccl_pg_reduce(pg, p_arr_send, p_arr_recv, sz=None, root=0):
    if p_arr_recv.data_ptr() != p_arr_send.data_ptr():
        p_arr_recv.copy_(p_arr_send)
    fns.reduce(p_arr_recv, root, group=_group(pg))
    return p_arr_recv
