"""``TrainerMPOPPytorch`` for ZeRO modes (``zr``, ``dp+zr``, ``zr+mp``, ``dp+zr+mp``).

Two execution styles share this class.

*Layer-owner style* (the reference's semantics, necklace/trainer/zroppt.py:438-680):
sub-module *i* of ``net_map`` is owned by zr-rank ``i % zr_world``; before its forward
the owner's weights are broadcast, after its backward the gradients are reduced (summed,
as in the reference) to the owner, only the owner keeps an optimizer for it, and the
backward recomputes each part's forward (``MdWrpWithSelfBkwd``).  The stepwise commands
``one_zr_step_{start, fwd_weig_brcast, calc_loss, bcwd_grad_reduce, bcwd_weig_brcast,
opt_one_step}`` drive it phase by phase; ``run_epoch`` runs the same phases in a local
loop.  ``offload=True`` parks inactive sub-modules in (pinned) host memory like the
reference; ``flat=True`` (the ``zroppf`` flavour) moves them through one flat device
buffer pair so a broadcast / reduce is one collective per sub-module.

*Sharded style* (``engine='native'``): parameters, gradients and optimizer state are
sharded uniformly over the zr group and one fused kernel per step does gradient
reduce-scatter + optimizer + parameter all-gather (``parallel.engine.TrainEngine``);
``net_map`` still defines the units and ``optimizer_creator`` the hyper-parameters.

``typ`` = ``oozr`` (zr only), ``dpzr`` / ``dpzrmp`` (weights averaged over the dp group
after the step), ``zrmp``.
"""
from __future__ import annotations

import time

import torch
import torch.nn as nn

from ..comm import fns, groups as G
from ..frmwrk.pytorch import ptprms
from ..frmwrk.pytorch.mdwrp import MdWrpWholeNet, MdWrpWithSelfBkwd
from ..frmwrk.pytorch.tsmem import PtCudaFltnMemManager, md_grads_numel_total_size, \
    md_params_numel_total_size
from ..utils.tmrit import TimerItLogger
from .tnoppt import TrainerOPPytorch, _to_ctx


class TrainerMPOPPytorch(TrainerOPPytorch):
    DEFAULT_TMODE = "zr"
    FLAT = False

    def __init__(self, cfg=None):
        cfg = dict(cfg or {})
        self.net_map = cfg.get("net_map") or {}
        self.net_map_maxlen = cfg.get("net_map_maxlen") or len(self.net_map)
        self.optimizer_creator = cfg.get("optimizer_creator")
        self.optimizer_creator_args = cfg.get("optimizer_creator_args", ())
        self.optimizer_creator_kwargs = cfg.get("optimizer_creator_kwargs", {})
        self.offload = bool(cfg.get("offload", False))
        self.flat = bool(cfg.get("flat", self.FLAT))
        self.do_acts_ckpt = bool(cfg.get("do_acts_ckpt", True))
        self.engine_kind = cfg.get("engine", "owner")
        cfg.setdefault("net", None)
        super().__init__(cfg)
        self.tmr = TimerItLogger(do_print=bool(cfg.get("timer_print", False)))
        n = self.net_map_maxlen
        self.nets = []
        for i in range(n):
            part = MdWrpWithSelfBkwd(self.net_map[i]["net"], mp_order=i, is_last_part=(i == n - 1),
                                     do_acts_ckpt=self.do_acts_ckpt)
            self.nets.append(part)
        self.home = torch.device("cpu") if self.offload else (self.ctx or torch.device("cpu"))
        for p in self.nets:
            p.to(self.home)
        self.opts = {}
        self.mm = None
        if self.flat and self.ctx is not None:
            mw = max(md_params_numel_total_size(p) for p in self.nets)
            mg = max(md_grads_numel_total_size(p) for p in self.nets)
            dt = next(self.nets[0].parameters()).dtype
            self.mm = PtCudaFltnMemManager(mw, mg, self.ctx, dtype=dt)
            for p in self.nets:
                self.mm.register(p)
        self.mp_grads = None
        self.outputs = None
        self.targets = None
        self.native = None

    # ------------------------------------------------------------------ helpers
    def zr_group(self):
        return G.get_nccl_group_zr_or_main()

    def owner_of(self, i):
        return i % max(self.zr_group().world_size, 1)

    def i_own(self, i):
        return self.owner_of(i) == self.zr_group().rank

    def _opt_for(self, i):
        if i not in self.opts:
            self.opts[i] = self.optimizer_creator(self.nets[i], *self.optimizer_creator_args,
                                                  **self.optimizer_creator_kwargs)
        return self.opts[i]

    def _activate(self, i):
        net = self.nets[i]
        if self.mm is not None:
            self.mm.md_to_gpu(net)
        elif self.offload and self.ctx is not None:
            net.to(self.ctx)
        return net

    def _park(self, i):
        net = self.nets[i]
        if self.mm is not None:
            self.mm.md_to_cpu(net)
        elif self.offload:
            net.to("cpu")

    def is_first_part(self, i=None):
        """Is unit ``i`` (default: the unit this rank owns) the first / last of the network?"""
        return (self.cfg.get("net_map_order", self.ti) if i is None else i) == 0

    def is_last_part(self, i=None):
        return (self.cfg.get("net_map_order", self.ti) if i is None else i) == len(self.nets) - 1

    def opts_zero_grad(self):
        for o in self.opts.values():
            o.zero_grad(set_to_none=False)

    def get_whole_net_cpu(self):
        """All parts in order as one CPU module (evaluation, whole-model checkpoints)."""
        parts = [p.to("cpu") if self.mm is None else p for p in self.nets]
        if self.mm is not None:
            for p in parts:
                self.mm.md_to_cpu(p)
        return MdWrpWholeNet(parts)

    # ---------------------------------------------------------------- collectives
    def do_params_nccl_broadcast(self, i):
        net, grp = self.nets[i], self.zr_group()
        if grp.world_size == 1:
            return
        if self.mm is not None:
            ptprms.params_fltn_do_nccl_broadcast(grp, grp.world_size, self.owner_of(i),
                                                 self.mm.weights_flat(net))
        else:
            ptprms.params_do_nccl_broadcast(grp, grp.world_size, self.owner_of(i), net)

    def do_grads_nccl_reduce_to_me(self, i):
        net, grp = self.nets[i], self.zr_group()
        if grp.world_size == 1:
            return
        if self.mm is not None:
            ptprms.opt_grads_fltn_do_nccl_reduce(grp, grp.world_size, self.owner_of(i),
                                                 self.mm.grads_flat(net))
        else:
            grads = [p.grad for p in net.parameters() if p.grad is not None]
            ptprms.nccl_reduce_by_buckets(grp, grp.world_size, self.owner_of(i), grads)

    # ------------------------------------------------------------ stepwise protocol
    def check_msg(self, msg, *args, **kwargs):
        cmd = msg.get("cmd") or ""
        if cmd.startswith("one_zr_step"):
            return getattr(self, "_cmd_" + cmd)(msg)
        return super().check_msg(msg, *args, **kwargs)

    def _cmd_one_zr_step_start(self, msg):
        if not self.before_train_done:
            self.before_train(self.ti)
            self.before_epoch(self.ti)
            self.before_train_done = True
        return {"ret": "one_zr_step_started"}

    def _cmd_one_zr_step_fwd_weig_brcast(self, msg):
        i = msg["one_zr_step_order_i"]
        self.tmr.start("fwd_weig_brcast")
        if i == 0:
            data, target = self.get_a_data_batch(self.ti)
            if data is None:
                return {"ret": "zr_epoch_end"}
            self.outputs = [_to_ctx(data, self.ctx)]
            self.targets = _to_ctx(target, self.ctx)
            self.saved_inputs = {}
        net = self._activate(i)
        self.do_params_nccl_broadcast(i)
        inputs = self.outputs
        self.saved_inputs[i] = inputs
        out = net(*inputs)
        self.outputs = list(out) if isinstance(out, (tuple, list)) else [out]
        if i < len(self.nets) - 1:
            self.outputs = [o.detach() for o in self.outputs]
            self._park(i)
        self.tmr.end("fwd_weig_brcast")
        return {"ret": "one_zr_step_fwd_weig_brcast_resp"}

    def _cmd_one_zr_step_calc_loss(self, msg):
        i = len(self.nets) - 1
        out = self.outputs[0] if len(self.outputs) == 1 else self.outputs
        loss = self.loss_fn(out, self.targets)
        loss.backward()
        self.last_loss = loss.detach()
        self.mp_grads = self.nets[i].get_input_grads()
        if self.mtrc is not None:
            self.mtrc.update(self.targets, out)
        return {"ret": "one_zr_step_loss_calced"}

    def _cmd_one_zr_step_bcwd_grad_reduce(self, msg):
        i = msg["one_zr_step_order_i"]
        self._activate(i)
        self.do_grads_nccl_reduce_to_me(i)
        if self.cfg.get("zr_grad_average") and self.i_own(i) and self.zr_group().world_size > 1:
            # the reference sums the contributions of the zr ranks; averaging is optional
            for p in self.nets[i].parameters():
                if p.grad is not None:
                    p.grad.div_(self.zr_group().world_size)
        if not self.i_own(i) and self.mm is None:
            for p in self.nets[i].parameters():
                p.grad = None
        self._park(i)
        return {"ret": "one_zr_step_bcwd_grad_reduce_resp"}

    def _cmd_one_zr_step_bcwd_weig_brcast(self, msg):
        """Back-propagate through part ``i`` (its forward is recomputed with a graph)."""
        i = msg["one_zr_step_order_i"]
        net = self._activate(i)
        net.inputs = net._graded(self.saved_inputs[i])
        net.mp_backward(self.mp_grads)
        self.mp_grads = net.get_input_grads()
        return {"ret": "one_zr_step_bcwd_weig_brcast_resp"}

    def _cmd_one_zr_step_opt_one_step(self, msg):
        typ = msg.get("typ", "oozr")
        for i in range(len(self.nets)):
            if self.i_own(i):
                self._activate(i)
                self._opt_for(i).step()
                self._park(i)
        for i, net in enumerate(self.nets):
            if self.mm is not None:
                self.mm.zero_grad(net)
            for p in net.parameters():
                if p.grad is not None:
                    p.grad.zero_()
        if typ in ("dpzr", "dpzrmp"):
            grp = G.get_nccl_group_dp()
            if grp is not None and grp.world_size > 1:
                for i in range(len(self.nets)):
                    if self.i_own(i):
                        ptprms.params_do_nccl_allreduce(grp, grp.world_size, self.nets[i])
        self.i += 1
        self.bn += 1
        return {"ret": "one_zr_step_opt_one_step_resp"}

    # --------------------------------------------------------------- fast path
    def run_steps(self, typ="oozr", n=None):
        if self.engine_kind == "native":
            return self._run_steps_native(typ, n)
        done, t0, status = 0, time.time(), "steps_done"
        nsub = len(self.nets)
        while n is None or done < n:
            self._cmd_one_zr_step_start({})
            ended = False
            for i in range(nsub):
                r = self._cmd_one_zr_step_fwd_weig_brcast({"one_zr_step_order_i": i})
                if r["ret"] == "zr_epoch_end":
                    ended = True
                    break
            if ended:
                status = "epoch_end"
                break
            self._cmd_one_zr_step_calc_loss({})
            for i in range(nsub - 1, -1, -1):
                self._cmd_one_zr_step_bcwd_grad_reduce({"one_zr_step_order_i": i})
                if i > 0:
                    self._cmd_one_zr_step_bcwd_weig_brcast({"one_zr_step_order_i": i - 1})
            self._cmd_one_zr_step_opt_one_step({"typ": typ})
            self.i -= 1
            self.metric_log()
            self.i += 1
            done += 1
        self.nccl_stream_sync()
        return {"ret": status, "steps": done, "seconds": time.time() - t0,
                "loss": float(self.last_loss) if self.last_loss is not None else None}

    def _native_engine(self):
        if self.native is None:
            from ..comm.backend import get_heap
            from ..parallel.engine import OptimConfig, TrainEngine
            loss_fn = self.loss_fn

            class _Whole(nn.Module):
                def __init__(s, parts):
                    super().__init__()
                    s.parts = nn.ModuleList(p.net for p in parts)

                def forward(s, data, target):
                    x = data
                    for m in s.parts[:-1]:
                        x = m(x)
                    last = s.parts[-1]
                    # a last unit that fuses its projection with the loss (no logits
                    # tensor) takes the target itself
                    if getattr(last, "computes_loss", False):
                        return last(x, target)
                    return loss_fn(last(x), target)

            whole = _Whole(self.nets).to(self.ctx)
            ok = self.cfg.get("optimizer_params") or {}
            oc = OptimConfig(kind=ok.get("kind", "adam"), lr=ok.get("lr", 1e-3),
                             beta1=ok.get("beta1", ok.get("momentum", 0.9)),
                             beta2=ok.get("beta2", 0.999), eps=ok.get("eps", 1e-8),
                             weight_decay=ok.get("weight_decay", 0.0))
            grp = self.zr_group()
            comm = getattr(grp, "comm", None)
            peer = getattr(comm, "peer", None)
            group = peer if peer is not None else comm
            ek = dict(self.cfg.get("engine_kwargs") or {})   # use_cuda_graph, bucket_mb, ...
            self.native = TrainEngine(whole, mode="zero", group=group, heap=get_heap(), optim=oc,
                                      **ek)
        return self.native

    def _run_steps_native(self, typ, n):
        eng = self._native_engine()
        done, t0, status = 0, time.time(), "steps_done"
        while n is None or done < n:
            data, target = self.get_a_data_batch(self.ti)
            if data is None:
                status = "epoch_end"
                break
            self.last_loss = eng.step(_to_ctx(data, self.ctx), _to_ctx(target, self.ctx))
            self.i += 1
            self.bn += 1
            done += 1
        self.nccl_stream_sync()
        return {"ret": status, "steps": done, "seconds": time.time() - t0,
                "loss": float(self.last_loss) if self.last_loss is not None else None}

    def sync_all_parts(self):
        """Bring every rank's copy of every sub-module up to date with its owner (between
        steps non-owners lag one update behind, which the next forward's broadcast would
        repair; evaluation hooks and checkpoints want the current weights now)."""
        if self.zr_group().world_size == 1 or self.engine_kind == "native":
            return
        for i in range(len(self.nets)):
            self._activate(i)
            self.do_params_nccl_broadcast(i)
            self._park(i)

    def next_epoch(self):
        self.sync_all_parts()
        self.after_epoch(self.ti)
        self.e += 1
        self.init_train_data_it()
        self.before_epoch(self.ti)
