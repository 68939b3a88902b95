"""``TrainerOPPytorch``: the per-worker operator for modes ``no``, ``dp``, ``mp`` and ``dp+mp``.

Message interface of the reference (necklace/trainer/tnoppt.py:325-391): ``check_msg``
accepts ``weights_sync``, ``dt_sampler_sync``, ``one_step``, ``nccl_all_reduce``
(``typ`` = ``grad`` | ``weig`` | anything else = optimizer step only) and
``next_epoch`` and answers with a ``ret`` string.  Added: ``run_epoch`` runs a whole
epoch inside the worker (no RPC between steps; gradient collective ordered on the
stream, device-timed throughput) and ``run_steps`` does the same for ``n`` steps.

cfg keys are the reference's (tnoppt.py:33-55): ``kn, ti, ctx, net, net_init, opt, loss,
mtrc, optimizer_params, batch_size, epochs, dataset_len, dataloader_type (ori|dp|mp|mpdp),
dataloader_data_shape_dims, dataloader_data_typs, dataloader_creator[_args|_kwargs],
use_dist_data_sampler, log_interval, grad_comp_cfg, my_kwargs``; plus ``tmode``,
``comm_type``, ``pg_cfg`` and ``autocast`` (bf16 autocast around forward/loss).
"""
from __future__ import annotations

import time

import torch

from ..comm import groups as G
from ..data import dtdist
from ..frmwrk.pytorch import ptprms
from ..utils.tmrit import DeviceTimer
from .tnopbs import TrainerOPBase


def _to_ctx(x, ctx):
    if x is None or ctx is None:
        return x
    if isinstance(x, torch.Tensor):
        return x.to(ctx, non_blocking=True)
    if isinstance(x, (list, tuple)):
        return type(x)(_to_ctx(v, ctx) for v in x)
    if isinstance(x, dict):
        return {k: _to_ctx(v, ctx) for k, v in x.items()}
    return x


class TrainerOPPytorch(TrainerOPBase):
    def __init__(self, cfg=None):
        super().__init__(cfg)
        c = self.cfg
        self.net = c.get("net")
        self.net_init = c.get("net_init")
        self.opt = c.get("opt")
        self.loss_fn = c.get("loss")
        self.mtrc = c.get("mtrc")
        self.optimizer_params = c.get("optimizer_params")
        self.batch_size = c.get("batch_size", 1)
        self.epochs = c.get("epochs", 1)
        self.dataset_len = c.get("dataset_len")
        self.dataloader_type = c.get("dataloader_type", "ori")
        self.dataloader_data_shape_dims = c.get("dataloader_data_shape_dims", [4, 1])
        self.dataloader_data_typs = c.get("dataloader_data_typs", [torch.float32, torch.int64])
        self.dataloader_creator = c.get("dataloader_creator")
        self.dataloader_creator_args = c.get("dataloader_creator_args", ())
        self.dataloader_creator_kwargs = c.get("dataloader_creator_kwargs", {})
        self.use_dist_data_sampler = c.get("use_dist_data_sampler", False)
        self.log_interval = c.get("log_interval", 10)
        self.grad_comp_cfg = c.get("grad_comp_cfg")
        self.my_kwargs = c.get("my_kwargs", {})
        self.autocast = c.get("autocast", False)
        self.e = 0   # epoch
        self.i = 0   # batch index inside the epoch
        self.bn = 0  # batches since the last log line
        self.train_data = None
        self.train_data_it = None
        self.last_loss = None
        self._t_log = time.time()
        self.timer = DeviceTimer(enabled=c.get("device_timing", False))
        if self.net is not None and self.ctx is not None:
            self.net.to(self.ctx)
        if self.net_init is not None:
            self.net_init(self.net)
        self.before_train_done = False

    # -------------------------------------------- small helpers hooks may call
    def to_ctx(self, x):
        """Tensor (or nested list / tuple of tensors) on this operator's device."""
        return _to_ctx(x, self.ctx)

    def try_to_ctx(self, x):
        """Like ``to_ctx``; anything that cannot be moved comes back unchanged."""
        try:
            return _to_ctx(x, self.ctx)
        except (TypeError, RuntimeError):
            return x

    @staticmethod
    def to_list(x):
        return list(x) if isinstance(x, (list, tuple)) else [x]

    def cuda_sync(self):
        """Wait for this operator's stream (the reference synchronises stream and device
        around every collective, necklace/trainer/tnoppt.py:551-554; here only callers that
        need host-visible results do)."""
        self.nccl_stream_sync()

    def check_if_last_batch(self):
        n = len(self.train_data) if hasattr(self.train_data, "__len__") else -1
        return n > 0 and self.i + 1 >= n

    def clear_train_data(self):
        dl = self.train_data
        if dl is not None and hasattr(dl, "clear"):
            dl.clear()
        self.train_data, self.train_data_it = None, None

    def train_loop(self, typ="grad"):
        """All epochs in this process without a scheduler (the reference's stand-alone loop,
        necklace/trainer/tnoppt.py ``train_loop``): for scripts that drive one operator by hand."""
        while self.e < self.epochs:
            self.run_steps(typ)
            self.next_epoch()

    # ------------------------------------------------------------------ data
    def init_train_data_it(self, *args, **kwargs):
        if self.train_data is None and self.dataloader_creator is not None:
            self.train_data = self.dataloader_creator(*self.dataloader_creator_args,
                                                      **self.dataloader_creator_kwargs)
        self.train_data_it = iter(self.train_data) if self.train_data is not None else None
        self.i = 0

    def cre_distdt_indices(self, msg=None, *args, **kwargs):
        """Rank 0 draws the epoch's global sample order (legacy central sampler)."""
        n = int(self.dataset_len or 0)
        idx = torch.randperm(n) if (msg or {}).get("shuffle", True) else torch.arange(n)
        return idx.tolist()

    def reset_distdt_indices(self, msg=None, *args, **kwargs):
        idx = (msg or {}).get("dt_indices")
        if self.train_data is None:
            self.init_train_data_it()
        if idx is not None and getattr(self.train_data, "_attr_ngn_dataloader", False) \
                and self.use_dist_data_sampler:
            from ..data.sampler import SliceSampler
            per = len(idx) // self.kn
            self.train_data.reset_batch_sampler(
                SliceSampler(indices=idx[self.ti * per:(self.ti + 1) * per]))
            self.train_data_it = iter(self.train_data)

    def dtld_check_if_mpdp(self):
        return "mp" in (self.dataloader_type or "")

    def dtld_sync_mp_input(self, data, target):
        """Broadcast the batch from local rank 0 of my tensor-parallel group."""
        grp = G.get_nccl_group_mp_or_main()
        if grp is None or grp.world_size == 1:
            return data, target
        is_root = grp.rank == 0
        flag = torch.zeros(1, dtype=torch.int64, device=self.ctx or "cpu")
        if is_root and data is not None:
            flag += 1
        dtdist.dt_shape_do_nccl_broadcast(flag, 0, grp)
        if int(flag.item()) == 0:
            return None, None
        tensors = [data, target] if is_root else [None, None]
        out = dtdist.broadcast_batch(tensors, self.dataloader_data_shape_dims,
                                     self.dataloader_data_typs, self.ctx or "cpu", 0, grp)
        return out[0], out[1]

    def _get_a_data_batch(self, rank=0, *args, **kwargs):
        if self.train_data_it is None:
            self.init_train_data_it()
        try:
            batch = next(self.train_data_it)
        except StopIteration:
            batch = None
        data, target = (None, None) if batch is None else (batch[0], batch[1])
        if self.dtld_check_if_mpdp():
            data, target = self.dtld_sync_mp_input(data, target)
        return data, target

    # ------------------------------------------------------------------ step
    def _one_step(self, rank=0, *args, **kwargs):
        if not self.before_train_done:
            self.before_train(self.ti)
            self.before_epoch(self.ti)
            self.before_train_done = True
        data, target = self.get_a_data_batch(rank)
        if data is None:
            return "epoch_end"
        self.do_a_batch_grads(data, target)
        self.metric_log()
        self.i += 1
        self.bn += 1
        return "one_step"

    def _forward(self, data):
        if isinstance(data, dict):
            return self.net(**data)
        if isinstance(data, (list, tuple)):
            return self.net(*data)
        return self.net(data)

    def _do_a_batch_grads(self, data, target, *args, **kwargs):
        data, target = _to_ctx(data, self.ctx), _to_ctx(target, self.ctx)
        for o in self._opts():
            o.zero_grad(set_to_none=False)
        dev_type = torch.device(self.ctx).type if self.ctx is not None else "cpu"
        with torch.autocast(dev_type, dtype=torch.bfloat16, enabled=bool(self.autocast)):
            output = self._forward(data)
            loss = self.loss_fn(output, target)
        if isinstance(loss, (list, tuple)):
            for k, l in enumerate(loss):
                l.backward(retain_graph=k < len(loss) - 1)
            self.last_loss = sum(l.detach() for l in loss)
        else:
            loss.backward()
            self.last_loss = loss.detach()
        if self.mtrc is not None:
            self.mtrc.update(target, output)
        return self.last_loss

    def _opts(self):
        if self.opt is None:
            return []
        return list(self.opt) if isinstance(self.opt, (list, tuple)) else [self.opt]

    def _do_a_train_step(self, stp=None):
        for o in self._opts():
            o.step()
        return "ok"

    # -------------------------------------------------------------- collectives
    def do_params_nccl_all_reduce(self, *args, **kwargs):
        grp = G.get_nccl_group_dp_or_main()
        if grp is not None and grp.world_size > 1 and self._dp_applies():
            ptprms.params_do_nccl_allreduce(grp, grp.world_size, self.net)

    def init_nccl_comm(self, msg=None, *args, **kwargs):
        r = super().init_nccl_comm(msg, *args, **kwargs)
        self._setup_heap_grads()
        return r

    def _setup_heap_grads(self):
        """With the peer-memory communicator the data-parallel gradients live in the
        symmetric heap and are reduced by the fused kernels, bucket by bucket under backward
        (``parallel.flat.HeapGradReducer``); ``grad_comp_cfg`` then means the fused 2-bit
        kernel.  Without it (NCCL / gloo communicator, CPU) the bucketed collective path of
        ``ptprms`` is used."""
        self.heap_grads = None
        grp = G.get_nccl_group_dp_or_main()
        peer = getattr(getattr(grp, "comm", None), "peer", None) if grp is not None else None
        if peer is None or peer.world == 1 or self.net is None or not self._dp_applies():
            return
        params = [p for p in self.net.parameters() if p.requires_grad]
        if not params or not params[0].is_cuda or len({p.dtype for p in params}) != 1 or \
                params[0].dtype not in (torch.float32, torch.bfloat16):
            return
        from ..parallel.flat import HeapGradReducer
        self.heap_grads = HeapGradReducer(
            self.net, peer, self.heap, self.grad_comp_cfg,
            bucket_mb=float(self.cfg.get("grad_bucket_mb", 25.0)),
            overlap=bool(self.cfg.get("grad_overlap", True)))

    def do_grads_nccl_all_reduce(self, *args, **kwargs):
        grp = G.get_nccl_group_dp_or_main()
        if grp is not None and grp.world_size > 1 and self._dp_applies():
            if getattr(self, "heap_grads", None) is not None:
                self.heap_grads.finish()
                return
            ptprms.opt_grads_do_nccl_allreduce(grp, grp.world_size, self.opt,
                                               grad_comp_cfg=self.grad_comp_cfg)

    def _dp_applies(self):
        """False when the only group is a tensor-parallel one (weights differ per rank)."""
        return G.get_nccl_group_dp() is not None or G.get_nccl_group_mp() is None

    # ------------------------------------------------------------------ messages
    def check_msg(self, msg, *args, **kwargs):
        cmd, typ = msg.get("cmd"), msg.get("typ", "grad")
        ret = {"ret": None}
        if cmd == "weights_sync":
            self.do_params_nccl_all_reduce()
            ret["ret"] = "weights_synced"
        elif cmd == "dt_sampler_sync":
            self.reset_distdt_indices(msg)
            ret["ret"] = "dt_sampler_synced"
        elif cmd == "one_step":
            ret["ret"] = self.one_step(self.ti)
        elif cmd == "nccl_all_reduce":
            self.all_reduce_and_step(typ)
            ret["ret"] = "nccl_all_reduced"
        elif cmd == "next_epoch":
            self.next_epoch()
            ret["ret"] = "next_epoch"
        elif cmd in ("run_epoch", "run_steps"):
            ret.update(self.run_steps(typ, msg.get("n") if cmd == "run_steps" else None))
        else:
            ret["ret"] = "err"
            ret["err"] = f"unknown cmd {cmd!r}"
        return ret

    def all_reduce_and_step(self, typ="grad"):
        if typ == "grad":
            self.do_grads_nccl_all_reduce()
            self.do_a_train_step()
        elif typ == "weig":
            self.do_a_train_step()
            self.do_params_nccl_all_reduce()
        else:  # 'oopt': optimizer only (pure tensor parallel)
            self.do_a_train_step()

    def next_epoch(self):
        self.after_epoch(self.ti)
        self.e += 1
        if self.mtrc is not None and hasattr(self.mtrc, "reset"):
            self.mtrc.reset()
        self.init_train_data_it()
        self.before_epoch(self.ti)

    def run_steps(self, typ="grad", n=None):
        """Steps back to back inside the worker until ``n`` steps ran or the epoch ends."""
        done, t0 = 0, time.time()
        self.timer.start("run_steps")
        status = "steps_done"
        while n is None or done < n:
            if self.one_step(self.ti) == "epoch_end":
                status = "epoch_end"
                break
            self.all_reduce_and_step(typ)
            done += 1
        self.timer.end("run_steps")
        self.nccl_stream_sync()
        dt = time.time() - t0
        return {"ret": status, "steps": done, "seconds": dt,
                "loss": float(self.last_loss) if self.last_loss is not None else None}

    # ------------------------------------------------------------------- logging
    def metric_log(self):
        n = len(self.train_data) if hasattr(self.train_data, "__len__") else -1
        if self.log_interval and ((self.i + 1) % self.log_interval == 0 or self.i + 1 == n):
            now = time.time()
            reps = G.get_nccl_group_dp().world_size if G.get_nccl_group_dp() else \
                (1 if G.get_nccl_group_mp() else max(self.kn, 1))
            speed = self.batch_size * reps * max(self.bn, 1) / max(now - self._t_log, 1e-9)
            if self.mtrc is not None and hasattr(self.mtrc, "get"):
                name, val = self.mtrc.get()
                tail = f"{name}={val:.6f}"
            else:
                tail = f"loss={float(self.last_loss):.6f}" if self.last_loss is not None else ""
            print(f"[{self.ti}]Epoch[{self.e}] Batch [{self.i + 1} / {n}] "
                  f"Speed: {speed:.2f} samples/sec  {tail}", flush=True)
            self._t_log, self.bn = now, 0

    def get_weights(self):
        return ptprms.get_weights(self.net)

    def set_weights(self, weights):
        ptprms.set_weights(self.net, weights)
