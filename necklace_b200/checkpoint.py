"""Checkpoint / resume.

The reference only has helpers (``torch.save(state, 'checkpoint.pth.tar')`` plus a best
copy, ``module.``-prefix stripping, whole-model assembly for ZeRO / pipeline parts;
necklace/frmwrk/pytorch/callback.py:16-19, ptutils.py:21-35, mdwrp.py:148-155) and no resume
logic.  Here a checkpoint is one ``torch.save`` file holding

    {"state_dict": un-sharded parameter tensors by their ordinary names (fp32 master values),
     "optim": {"kind", "step", "s1", "s2"  (flat fp32, un-sharded)},
     "meta": {"epoch", "step", "rng", "layout"}}

so it loads into a plain ``nn.Module`` with ``load_state_dict`` and re-shards onto any
number of ZeRO ranks.  Tensor-parallel parameters (``model_parallel`` attribute with a
``partition_dim``) are concatenated on save and re-split on load; pipeline / ZeRO parts are
assembled under the reference's ``whole_md.<i>...`` keys.
"""
from __future__ import annotations

import os
import shutil
from collections import OrderedDict

import torch
import torch.distributed as dist


# ----------------------------------------------------------------------- engine (dp / zero)
def _gather_flat(engine, t: torch.Tensor, group=None) -> torch.Tensor:
    """Full-length fp32 copy on the CPU of a per-rank optimizer-state tensor (the engine
    knows how its shards interleave: one slice per rank in every bucket)."""
    return engine.gather_state(t.detach(), group).float().cpu()


def engine_state(engine, epoch: int = 0, extra: dict | None = None) -> dict:
    """Consolidated state of a ``TrainEngine`` (collective when the engine is sharded)."""
    f = engine.flat
    pg = getattr(getattr(engine.group, "heap", None), "group", None) if engine.sharded else None
    master = _gather_flat(engine, engine.master, pg)
    sd = OrderedDict()
    for name, p, off in zip(f.names, f.params, f.offsets):
        sd[name] = master[off:off + p.numel()].view(p.shape).clone()
    optim = {"kind": engine.optim.kind, "step": engine.step_count}
    for key in ("s1", "s2"):
        t = getattr(engine, key)
        optim[key] = None if t is None else _gather_flat(engine, t, pg)
    meta = {"epoch": epoch, "step": engine.step_count, "rng": torch.get_rng_state(),
            "layout": {"names": f.names, "offsets": f.offsets, "numel": f.numel,
                       "world": engine.world, "mode": engine.mode}}
    if extra:
        meta.update(extra)
    return {"state_dict": sd, "optim": optim, "meta": meta}


def load_engine_state(engine, state: dict) -> dict:
    """Load a consolidated state into an engine of any world size (re-shards)."""
    f = engine.flat
    full = torch.zeros(f.numel, dtype=torch.float32)
    for name, p, off in zip(f.names, f.params, f.offsets):
        full[off:off + p.numel()] = state["state_dict"][name].reshape(-1).float()
    dev = engine.master.device
    engine.master.copy_(engine.shard_of(full).to(dev))
    f.flat.copy_(full.to(dev).to(f.flat.dtype))
    old = state["meta"]["layout"]
    for key in ("s1", "s2"):
        src, dst = state["optim"].get(key), getattr(engine, key)
        if src is None or dst is None:
            continue
        buf = torch.zeros(f.numel, dtype=torch.float32)
        if old["names"] == f.names and old["offsets"] == f.offsets:
            buf[:min(f.numel, src.numel())] = src[:min(f.numel, src.numel())]
        else:  # different padding / order: move slice by slice
            o_off = dict(zip(old["names"], old["offsets"]))
            for name, p, off in zip(f.names, f.params, f.offsets):
                buf[off:off + p.numel()] = src[o_off[name]:o_off[name] + p.numel()]
        dst.copy_(engine.shard_of(buf).to(dev))
    engine.set_step_count(int(state["optim"].get("step", 0)))
    if state["meta"].get("rng") is not None:
        torch.set_rng_state(state["meta"]["rng"])
    return state["meta"]


def save(state: dict, filename: str = "checkpoint.pth.tar", is_best: bool = False,
         best: str = "model_best.pth.tar", rank: int = 0) -> None:
    """Written by one rank, atomically (temp file + rename)."""
    if rank != 0:
        return
    tmp = filename + ".tmp"
    torch.save(state, tmp)
    os.replace(tmp, filename)
    if is_best:
        shutil.copyfile(filename, best)


def load(filename: str) -> dict:
    return torch.load(filename, map_location="cpu", weights_only=False)


# ------------------------------------------------------------------ tensor-parallel modules
# A sharded parameter carries three attributes: ``model_parallel`` (True), ``partition_dim``
# (the dimension that is split: 0 for column-parallel weights and their biases, 1 for
# row-parallel weights) and ``partition_stride`` (how many independently split blocks are
# packed along that dimension: 3 for a fused q/k/v projection, 2 for gate/up, default 1).
# With stride s the full tensor is the sequence of pieces
#     block 0 rank 0, block 0 rank 1, ..., block 1 rank 0, ...
# which is the layout the reference builds with ``stride`` in
# necklace/frmwrk/pytorch/mpnn/layers.py:40-72.
def tp_concat(shards: list[torch.Tensor], dim: int = 0, stride: int = 1) -> torch.Tensor:
    """Un-sharded tensor from the per-rank shards (rank order)."""
    if len(shards) == 1:
        return shards[0]
    if stride == 1:
        return torch.cat(list(shards), dim=dim)
    pieces = [s.chunk(stride, dim=dim) for s in shards]
    return torch.cat([pieces[r][j] for j in range(stride) for r in range(len(shards))], dim=dim)


def tp_split(full: torch.Tensor, ws: int, rank: int, dim: int = 0, stride: int = 1
             ) -> torch.Tensor:
    """Rank ``rank``'s shard of an un-sharded tensor (inverse of ``tp_concat``)."""
    if ws == 1:
        return full
    blocks = full.chunk(stride, dim=dim)
    return torch.cat([b.chunk(ws, dim=dim)[rank] for b in blocks], dim=dim).contiguous()


def _tp_attrs(p):
    return (getattr(p, "model_parallel", False), getattr(p, "partition_dim", 0),
            getattr(p, "partition_stride", 1))


def gather_tp_state_dict(module: torch.nn.Module, mp_group=None) -> OrderedDict:
    """Un-sharded state dict of a tensor-parallel module (collective over the mp group)."""
    from .comm import fns
    ws = mp_group.world_size if mp_group is not None else 1
    out = OrderedDict()
    for name, p in module.named_parameters():
        t = p.detach()
        sharded, dim, stride = _tp_attrs(p)
        if ws > 1 and sharded:
            buf = torch.empty((ws,) + tuple(t.shape), dtype=t.dtype, device=t.device)
            fns.all_gather(buf, t.contiguous(), group=mp_group)
            t = tp_concat(list(buf.unbind(0)), dim, stride)
        out[name] = t.float().cpu()
    for name, b in module.named_buffers():
        out[name] = b.detach().cpu()
    return out


def load_tp_state_dict(module: torch.nn.Module, full: dict, mp_group=None, ws: int | None = None,
                       rank: int | None = None) -> None:
    """Load an un-sharded state dict into a module sharded ``ws`` ways (``ws`` / ``rank``
    default to the mp group's)."""
    if ws is None:
        ws = mp_group.world_size if mp_group is not None else 1
    if rank is None:
        rank = mp_group.rank if mp_group is not None else 0
    with torch.no_grad():
        for name, p in module.named_parameters():
            t = full[name]
            sharded, dim, stride = _tp_attrs(p)
            if sharded:
                want = p.shape[dim] * ws
                if t.shape[dim] != want and stride == 1:
                    # padded vocabulary tables: the padding depends on the number of ranks
                    if t.shape[dim] > want:
                        t = t.narrow(dim, 0, want)
                    else:
                        pad = list(t.shape)
                        pad[dim] = want - t.shape[dim]
                        t = torch.cat([t, torch.zeros(pad, dtype=t.dtype)], dim=dim)
            if ws > 1 and sharded:
                t = tp_split(t, ws, rank, dim, stride)
            p.copy_(t.to(p.dtype).to(p.device))


# ---------------------------------------------------------------- pipeline / ZeRO parts
def whole_state_dict(parts) -> OrderedDict:
    """State dict of all parts under the reference's ``whole_md.<i>.`` keys."""
    from .frmwrk.pytorch.mdwrp import MdWrpWholeNet
    return MdWrpWholeNet(list(parts)).state_dict()


def strip_module_prefix(sd: dict) -> OrderedDict:
    return OrderedDict((k[7:] if k.startswith("module.") else k, v) for k, v in sd.items())
