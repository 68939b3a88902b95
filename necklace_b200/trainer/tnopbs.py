"""Trainer operator bases: the hook machinery and communicator bring-up.

``ModelWrapperHooks`` gives every operator six events (train, epoch, data_batch, batch,
do_a_batch_grads, do_a_train_step), each with "before" and "after" hook lists and
``register_hook_{before,after}_<event>`` methods; a public method runs the before hooks,
its ``_method`` and the after hooks, and an after hook that returns something other
than ``None`` replaces the result (reference: necklace/trainer/tnopbs.py:115-393).

``TrainerOPBase`` adds the communicator life cycle the scheduler drives
(``cre_nccl`` / ``cre_nccl_nuid`` / ``init_nccl_comm`` / ``*_pg``; reference
tnopbs.py:407-451).  The "unique id" that the reference relays over RPC becomes the
rendezvous address of the ``torch.distributed`` job (created by rank 0), and one
``init_nccl_comm`` call brings up every group of the layout, so the per-group messages
are accepted and answered but have nothing left to do.
"""
from __future__ import annotations

import logging
import socket
from collections import OrderedDict

from ..comm import backend as comm_backend
from ..comm import groups as G

logging.basicConfig(level=logging.INFO)
EVENTS = ("train", "epoch", "data_batch", "batch", "do_a_batch_grads", "do_a_train_step")


class TrainerOPAbs:
    def __init__(self, cfg=None):
        self.cfg = cfg or {}

    def check_msg(self, msg, *args, **kwargs):
        raise NotImplementedError

    def if_stop(self):
        return False

    def clear(self):
        pass


class ModelWrapperHooks(TrainerOPAbs):
    def __init__(self, cfg=None):
        super().__init__(cfg)
        self._hooks = {(when, ev): OrderedDict() for ev in EVENTS for when in ("before", "after")}
        self.hook_vars = {}

    # registration / dispatch ----------------------------------------------------
    def get_hook_func_name(self, func):
        return getattr(func, "__name__", func.__class__.__name__) + "-" + str(id(func))

    def register_hook(self, when, event, func, *args, **kwargs):
        self._hooks[(when, event)][self.get_hook_func_name(func)] = (func, args, kwargs)
        return func

    def hook_iter_run_before(self, funcs, *args, **kwargs):
        for func, a, k in funcs.values():
            func(self, *a, *args, **k, **kwargs)

    def hook_iter_run_after(self, funcs, *args, **kwargs):
        ret = None
        for func, a, k in funcs.values():
            r = func(self, *a, *args, **k, **kwargs)
            if r is not None:
                ret = r
        return ret

    def _run(self, event, fn, *args, **kwargs):
        self.hook_iter_run_before(self._hooks[("before", event)])
        r = fn(*args, **kwargs)
        rh = self.hook_iter_run_after(self._hooks[("after", event)], r) \
            if event not in ("train", "epoch") else \
            self.hook_iter_run_after(self._hooks[("after", event)])
        return rh if rh is not None else r

    # events -------------------------------------------------------------------------
    def before_train(self, rank=0, *args, **kwargs):
        self.hook_iter_run_before(self._hooks[("before", "train")])
        self._before_train(rank, *args, **kwargs)

    def after_train(self, rank=0, *args, **kwargs):
        self._after_train(rank, *args, **kwargs)
        self.hook_iter_run_after(self._hooks[("after", "train")])

    def before_epoch(self, rank=0, *args, **kwargs):
        self.hook_iter_run_before(self._hooks[("before", "epoch")])
        self._before_epoch(rank, *args, **kwargs)

    def after_epoch(self, rank=0, *args, **kwargs):
        self._after_epoch(rank, *args, **kwargs)
        self.hook_iter_run_after(self._hooks[("after", "epoch")])

    def get_a_data_batch(self, rank=0, *args, **kwargs):
        return self._run("data_batch", self._get_a_data_batch, rank, *args, **kwargs)

    def one_step(self, rank=0, *args, **kwargs):
        return self._run("batch", self._one_step, rank, *args, **kwargs)

    def do_a_batch_grads(self, *args, **kwargs):
        return self._run("do_a_batch_grads", self._do_a_batch_grads, *args, **kwargs)

    def do_a_train_step(self, stp=None):
        return self._run("do_a_train_step", self._do_a_train_step, stp=stp)

    def _before_train(self, rank=0, *args, **kwargs):
        pass

    def _after_train(self, rank=0, *args, **kwargs):
        pass

    def _before_epoch(self, rank=0, *args, **kwargs):
        pass

    def _after_epoch(self, rank=0, *args, **kwargs):
        pass

    def _get_a_data_batch(self, rank=0, *args, **kwargs):
        raise NotImplementedError

    def _one_step(self, rank=0, *args, **kwargs):
        raise NotImplementedError

    def _do_a_batch_grads(self, *args, **kwargs):
        raise NotImplementedError

    def _do_a_train_step(self, stp=None):
        raise NotImplementedError


def _make_register(when, event):
    def register(self, func, *args, **kwargs):
        return self.register_hook(when, event, func, *args, **kwargs)
    register.__name__ = f"register_hook_{when}_{event}"
    return register


for _ev in EVENTS:
    for _when in ("before", "after"):
        setattr(ModelWrapperHooks, f"register_hook_{_when}_{_ev}", _make_register(_when, _ev))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class TrainerOPBase(ModelWrapperHooks):
    DEFAULT_TMODE = "dp"

    def __init__(self, cfg=None):
        super().__init__(cfg)
        self.kn = self.cfg.get("kn", 1)       # number of workers
        self.ti = self.cfg.get("ti", 0)       # my global rank
        self.ctx = self.cfg.get("ctx")        # device
        self.comm_cfg = {}
        self.heap = None
        self.stopped = False

    # communicator life cycle -------------------------------------------------------
    def cre_nccl(self, msg=None, *args, **kwargs):
        """Record world size / rank / device (the reference creates its NcclWrp here)."""
        cfg = (msg or {}).get("cfg", {}) if isinstance(msg, dict) else {}
        self.comm_cfg.update(cfg)
        return "ok"

    def cre_nccl_nuid(self, msg=None, *args, **kwargs):
        """Rank 0 invents the rendezvous address every rank will join."""
        addr = self.cfg.get("master_addr", "127.0.0.1")
        return {"master_addr": addr, "master_port": self.cfg.get("master_port") or _free_port()}

    def init_nccl_comm(self, msg=None, *args, **kwargs):
        nuid = (msg or {}).get("nuid") or {}
        # no mode given and no group map built by the script: the operator's own flavour (all
        # workers are one data-parallel group / one pipeline / one ZeRO group, which is what
        # the reference's single-group examples mean)
        tmode = self.cfg.get("tmode") or (msg or {}).get("tmode") or \
            (G._S.tmode if G._S.inited else self.DEFAULT_TMODE)
        pg_cfg = dict(self.cfg.get("pg_cfg") or {})
        pg_cfg.setdefault("world_size", self.kn)
        pg_cfg.setdefault("my_rank", self.ti)
        dev = self.ctx
        self.heap = comm_backend.init_backend(
            tmode, pg_cfg, comm_type=self.cfg.get("comm_type", "nccl"), device=dev,
            master_addr=nuid.get("master_addr", "127.0.0.1"),
            master_port=int(nuid.get("master_port", 29400)),
            heap_bytes=int(self.cfg.get("heap_bytes") or self._default_heap_bytes()),
            timeout_s=float(self.cfg.get("comm_timeout_s", 120)))
        return "ok"

    def _default_heap_bytes(self) -> int:
        """Symmetric-heap size when the user gives none: room for the parameters and gradients
        of this worker's module(s) (the data-parallel / ZeRO buffers live there), the 2-bit
        code and count buffers, plus 256 MiB for the fused kernels' staging buffers."""
        if self.cfg.get("comm_type", "nccl") != "peer":
            return 0
        n = 0
        mods = []
        if getattr(self, "net", None) is not None:
            mods.append(self.net)
        for v in (self.cfg.get("net_map") or {}).values():
            if v.get("net") is not None:
                mods.append(v["net"])
        for m in mods:
            for mod in (m if isinstance(m, (list, tuple)) else [m]):
                if hasattr(mod, "parameters"):
                    n += sum(p.numel() * p.element_size() for p in mod.parameters())
        return int(n * 2.6) + (256 << 20)

    def del_nccl_comm(self, msg=None, *args, **kwargs):
        comm_backend.shutdown_backend()

    def cre_nccl_nuid_pg(self, msg=None, *args, **kwargs):
        return {}

    def init_nccl_comm_pg(self, msg=None, *args, **kwargs):
        return "ok"

    def del_nccl_comm_pg(self, msg=None, *args, **kwargs):
        pass

    def nccl_stream_sync(self, *args, **kwargs):
        import torch
        if torch.cuda.is_available() and self.ctx is not None and \
                torch.device(self.ctx).type == "cuda":
            torch.cuda.current_stream().synchronize()

    def if_stop(self):
        return self.stopped

    def clear(self):
        dl = getattr(self, "train_data", None)
        if dl is not None and hasattr(dl, "clear"):
            dl.clear()
        self.after_train(self.ti)
        self.del_nccl_comm()
        self.stopped = True
