"""Epoch checkpoints of a trainer operator and resuming from them.

The reference has no resume logic: the epoch and step counters live in the operator
(necklace/trainer/tnoppt.py:59-62) and the scheduler (necklace/trainer/tndsnc.py:430), and
``callback.save_checkpoint`` writes ``{'state_dict': ...}`` files (callback.py:16-19).  Here a
hook writes one such file per rank and epoch (a rank's own modules and optimizers: the whole
net in ``no`` / ``dp``, a pipeline stage, or the ZeRO units it owns), an operator loads the
newest epoch that *every* rank has completed, and the scheduler starts counting there.

    <dir>/rank<k>/ckpt_e<E>.pth.tar     state after E finished epochs (last ``keep`` kept)
"""
from __future__ import annotations

import glob
import os
import re

import torch

from ..utils.hookbase import NklcHookBase

_PAT = re.compile(r"ckpt_e(\d+)\.pth\.tar$")


def _rank_dir(ckpt_dir, rank):
    return os.path.join(ckpt_dir, f"rank{rank}")


def epochs_of_rank(ckpt_dir, rank):
    out = []
    for f in glob.glob(os.path.join(_rank_dir(ckpt_dir, rank), "ckpt_e*.pth.tar")):
        m = _PAT.search(f)
        if m:
            out.append(int(m.group(1)))
    return sorted(out)


def resume_epoch(ckpt_dir, world):
    """Newest number of finished epochs for which all ``world`` ranks have a checkpoint; 0 when
    there is none."""
    if not ckpt_dir or not os.path.isdir(ckpt_dir):
        return 0
    common = None
    for r in range(world):
        e = set(epochs_of_rank(ckpt_dir, r))
        common = e if common is None else common & e
    return max(common) if common else 0


def _modules_and_optimizers(trnr):
    """What a rank owns, keyed so that the same keys come back at load time."""
    nets = getattr(trnr, "nets", None)
    if nets:                                     # ZeRO flavours: list of units + dict of optimizers
        mods = {f"unit{i}": m for i, m in enumerate(nets)}
        opts = {f"unit{i}": o for i, o in (getattr(trnr, "opts", None) or {}).items()}
        return mods, opts
    mods = {"net": trnr.net} if getattr(trnr, "net", None) is not None else {}
    opt = getattr(trnr, "opt", None)
    opts = {}
    if opt is not None:
        for i, o in enumerate(opt if isinstance(opt, (list, tuple)) else [opt]):
            opts[f"opt{i}"] = o
    return mods, opts


def save_trainer(trnr, ckpt_dir, epochs_done, keep=2):
    mods, opts = _modules_and_optimizers(trnr)
    state = {"epoch": int(epochs_done),
             "state_dict": {k: m.state_dict() for k, m in mods.items()},
             "optimizer": {k: o.state_dict() for k, o in opts.items()},
             "rng": torch.get_rng_state()}
    if torch.cuda.is_available():
        state["cuda_rng"] = torch.cuda.get_rng_state()
    d = _rank_dir(ckpt_dir, trnr.ti)
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, f"ckpt_e{int(epochs_done)}.pth.tar")
    torch.save(state, path + ".tmp")
    os.replace(path + ".tmp", path)              # a reader never sees a half-written file
    for e in epochs_of_rank(ckpt_dir, trnr.ti)[:-keep]:
        try:
            os.remove(os.path.join(d, f"ckpt_e{e}.pth.tar"))
        except FileNotFoundError:
            pass
    return path


def load_trainer(trnr, ckpt_dir, epochs_done):
    """Restore this rank's modules, optimizers, RNG and epoch counter."""
    path = os.path.join(_rank_dir(ckpt_dir, trnr.ti), f"ckpt_e{int(epochs_done)}.pth.tar")
    state = torch.load(path, map_location="cpu", weights_only=False)
    mods, opts = _modules_and_optimizers(trnr)
    for k, m in mods.items():
        m.load_state_dict(state["state_dict"][k])
    for k, o in opts.items():
        if k in state["optimizer"]:
            o.load_state_dict(state["optimizer"][k])
    torch.set_rng_state(state["rng"])
    if torch.cuda.is_available() and "cuda_rng" in state:
        torch.cuda.set_rng_state(state["cuda_rng"])
    trnr.e = int(state["epoch"])
    return state


class HookCheckpoint(NklcHookBase):
    """``trnr.register_hook_after_epoch(HookCheckpoint(dir))``: write this rank's checkpoint
    after every ``every``-th epoch."""

    def __init__(self, ckpt_dir, every=1, keep=2):
        super().__init__()
        self.dir, self.every, self.keep = ckpt_dir, max(1, int(every)), keep
        self.saved = []

    def __call__(self, trnr=None, *args, **kwargs):
        done = trnr.e + 1                        # the hook runs before the counter moves on
        if done % self.every == 0:
            self.saved.append(save_trainer(trnr, self.dir, done, self.keep))


def attach(trnr, ckpt_dir, world, resume=False, every=1, keep=2):
    """Register the checkpoint hook on an operator and, with ``resume``, load the newest
    epoch every rank has.  Returns the number of epochs already done (0 = fresh start); give
    the same number to the scheduler as ``start_epoch``."""
    done = resume_epoch(ckpt_dir, world) if resume else 0
    if done:
        load_trainer(trnr, ckpt_dir, done)
    trnr.register_hook_after_epoch(HookCheckpoint(ckpt_dir, every, keep))
    return done
