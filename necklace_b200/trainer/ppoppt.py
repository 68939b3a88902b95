"""``TrainerMPOPPytorch`` for pipeline modes (``pp``, ``dp+pp``, ``dp+pp+mp``).

One class serves what the reference splits into ``mpoppt`` (one pipeline group) and
``ppoppt`` (several groups + data parallelism) (necklace/trainer/mpoppt.py:29-581,
necklace/trainer/ppoppt.py:228-606).  The stage of this worker is
``net_map[net_map_order]['net']`` wrapped in ``ModelPartWrapper``; only the first stage
creates a data loader.

Stepwise commands (reference protocol): ``one_mp_step_start``, ``one_mp_step_forward``,
``one_mp_step_trans_outputs``, ``one_mp_step_calc_loss``, ``one_mp_step_trans_grads``,
``one_mp_step_backward``, ``nccl_all_reduce`` (data-parallel gradient all-reduce over the
dp group, then the optimizer step), ``next_epoch``.

Fast path: ``run_epoch`` / ``run_steps`` run a micro-batched 1F1B schedule inside the
worker (``micro_batches`` in cfg, default 1 = the reference's sequential pipeline), with
self-describing p2p transfers, so neither shapes nor phases go through the scheduler.
"""
from __future__ import annotations

import time

import torch

from ..comm import groups as G
from ..frmwrk.pytorch import ptprms
from ..frmwrk.pytorch.mputils import ModelPartWrapper
from ..parallel import pipeline as pl
from .tnoppt import TrainerOPPytorch, _to_ctx


class TrainerMPOPPytorch(TrainerOPPytorch):
    DEFAULT_TMODE = "pp"

    def __init__(self, cfg=None):
        cfg = dict(cfg or {})
        self.net_map = cfg.get("net_map")
        self.net_map_order = cfg.get("net_map_order", 0)
        self.net_map_maxlen = cfg.get("net_map_maxlen") or (len(self.net_map) if self.net_map else 1)
        if cfg.get("net") is None and self.net_map:
            cfg["net"] = self.net_map[self.net_map_order]["net"]
        super().__init__(cfg)
        if not isinstance(self.net, ModelPartWrapper):
            self.net = ModelPartWrapper(self.net, mp_order=self.net_map_order)
            if self.ctx is not None:
                self.net.to(self.ctx)
        self.is_first = self.net_map_order == 0
        self.is_last = self.net_map_order == self.net_map_maxlen - 1
        self.micro_batches = int(cfg.get("micro_batches", 1))
        self.targets = None
        self.recv_inputs = None
        self.recv_grads = None
        self.stage = None

    # group helpers ----------------------------------------------------------------
    def is_first_part(self):
        return self.is_first

    def is_last_part(self):
        return self.is_last

    def pp_ranks(self):
        g = G.get_nccl_group_pp()
        if g is not None:
            return g.pg_ranks
        if self.net_map and all("worker_rank" in v for v in self.net_map.values()):
            return [v["worker_rank"] for _, v in sorted(self.net_map.items())]
        return list(range(self.net_map_maxlen))

    def _has_loader(self):
        return self.is_first

    def init_train_data_it(self, *args, **kwargs):
        if self._has_loader():
            super().init_train_data_it()
        else:
            self.i = 0

    # collectives: only a real dp group averages gradients in pipeline modes -------------
    def _dp_applies(self):
        return G.get_nccl_group_dp() is not None

    def do_params_nccl_all_reduce(self, *args, **kwargs):
        grp = G.get_nccl_group_dp()
        if grp is not None and grp.world_size > 1:
            ptprms.params_do_nccl_allreduce(grp, grp.world_size, self.net)

    # ------------------------------------------------------------------ stepwise protocol
    def check_msg(self, msg, *args, **kwargs):
        cmd = msg.get("cmd")
        fn = getattr(self, "_cmd_" + cmd, None) if cmd and cmd.startswith("one_mp_step") else None
        if fn is not None:
            return fn(msg)
        return super().check_msg(msg, *args, **kwargs)

    def _cmd_one_mp_step_start(self, msg):
        if not self.before_train_done:
            self.before_train(self.ti)
            self.before_epoch(self.ti)
            self.before_train_done = True
        for o in self._opts():
            o.zero_grad(set_to_none=False)
        return {"ret": "one_mp_step_started"}

    def _cmd_one_mp_step_forward(self, msg):
        if self.is_first:
            data, target = self.get_a_data_batch(self.ti)
            if data is None:
                return {"ret": "mp_epoch_end", "net_map_order": self.net_map_order}
            inputs = [_to_ctx(data, self.ctx)]
            self.targets = [_to_ctx(target, self.ctx)]
        else:
            inputs = self.recv_inputs
        out = self.net(*inputs)
        outs = list(out) if isinstance(out, (tuple, list)) else [out]
        self.outputs = outs
        ret = {"ret": "one_mp_step_forwarded", "net_map_order": self.net_map_order,
               "output_shps": [list(o.shape) for o in outs],
               "output_dts": [str(o.dtype) for o in outs]}
        if self.is_first:
            ret["target_shps"] = [list(t.shape) for t in self.targets]
        return ret

    def _cmd_one_mp_step_trans_outputs(self, msg):
        if self.ti == msg["from_rank"]:
            pl.p2p_send([o.detach() for o in self.outputs], msg["to_rank"], self.ctx)
            pl.flush_sends()
        elif self.ti == msg["to_rank"]:
            self.recv_inputs = pl.p2p_recv(msg["from_rank"], self.ctx)
        return {"ret": "one_mp_step_outputs_transed"}

    def _cmd_one_mp_step_calc_loss(self, msg):
        frm, to = msg["from_rank"], msg["to_rank"]
        if frm != to:
            if self.ti == frm:
                self._send_far(self.targets, to)
            if self.ti == to:
                self.targets = self._recv_far(frm)
        ret = {"ret": "one_mp_step_loss_calced"}
        if self.ti == to:
            out = self.outputs[0] if len(self.outputs) == 1 else self.outputs
            loss = self.loss_fn(out, self.targets[0])
            loss.backward()
            self.last_loss = loss.detach()
            self.input_grads = self.net.get_input_grads()
            ret["grads_shps"] = [list(g.shape) for g in self.input_grads]
        return ret

    def _send_far(self, tensors, dst):
        """first -> last stage transfer (targets); neighbours share a channel, distant
        stages use the main group."""
        import torch.distributed as dist
        if pl._chan(self.ti, dst) is not None:
            pl.p2p_send(tensors, dst, self.ctx)
            pl.flush_sends()
        else:
            dev = pl._hdr_device(self.ctx)
            for t in tensors:
                meta = torch.tensor([t.dim(), *t.shape] + [0] * (7 - t.dim()), dtype=torch.int64)
                dist.send(meta.to(dev), dst)
                dist.send(t.contiguous().to(dev), dst)

    def _recv_far(self, src):
        import torch.distributed as dist
        if pl._chan(src, self.ti) is not None:
            return pl.p2p_recv(src, self.ctx)
        dev = pl._hdr_device(self.ctx)
        meta = torch.zeros(8, dtype=torch.int64, device=dev)
        dist.recv(meta, src)
        meta = meta.cpu()
        t = torch.empty([int(x) for x in meta[1:1 + int(meta[0])]], dtype=torch.int64, device=dev)
        dist.recv(t, src)
        return [t.to(self.ctx)]

    def _cmd_one_mp_step_trans_grads(self, msg):
        if self.ti == msg["from_rank"]:
            pl.p2p_send(self.input_grads, msg["to_rank"], self.ctx)
            pl.flush_sends()
        elif self.ti == msg["to_rank"]:
            self.recv_grads = pl.p2p_recv(msg["from_rank"], self.ctx)
        return {"ret": "one_mp_step_grads_transed"}

    def _cmd_one_mp_step_backward(self, msg):
        self.net.mp_backward(self.recv_grads)
        self.input_grads = self.net.get_input_grads()
        return {"ret": "one_mp_step_backwarded"}

    def all_reduce_and_step(self, typ="grad"):
        grp = G.get_nccl_group_dp()
        if grp is not None and grp.world_size > 1:
            ptprms.opt_grads_do_nccl_allreduce(grp, grp.world_size, self.opt,
                                               grad_comp_cfg=self.grad_comp_cfg)
        self.do_a_train_step()
        self.i += 1

    # ------------------------------------------------------------------ fast path: 1F1B
    def _split_mb(self, data, target):
        m = self.micro_batches
        if m == 1:
            return [(data, target)]
        return list(zip(torch.chunk(data, m), torch.chunk(target, m)))

    def run_steps(self, typ="grad", n=None):
        if not self.before_train_done:
            self.before_train(self.ti)
            self.before_epoch(self.ti)
            self.before_train_done = True
        if self.stage is None:
            self.stage = pl.PipelineStage(self.net.net, self.net_map_order, self.pp_ranks(),
                                          loss_fn=self.loss_fn, device=self.ctx or "cpu")
        done, t0, status = 0, time.time(), "steps_done"
        while n is None or done < n:
            for o in self._opts():
                o.zero_grad(set_to_none=False)
            if self.is_first:
                data, target = self.get_a_data_batch(self.ti)
                mbs = None if data is None else self._split_mb(data, target)
            else:
                mbs = [(None, None)] * self.micro_batches
            r = self.stage.run_step(mbs)
            if r is False:
                status = "epoch_end"
                break
            if self.is_last:
                self.last_loss = r
            self.all_reduce_and_step(typ)
            self.bn += 1
            if self.is_last:
                self.i -= 1
                self.metric_log()
                self.i += 1
            done += 1
        self.nccl_stream_sync()
        return {"ret": status, "steps": done, "seconds": time.time() - t0,
                "loss": float(self.last_loss) if self.last_loss is not None else None}
