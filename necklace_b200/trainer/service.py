"""Scheduler and worker services: one state machine for every trainer mode.

Process model and wire protocol are the reference's (one scheduler + N workers, the
cast-then-callback pattern: the scheduler calls ``fn_X_start`` on a worker, the endpoint
only queues the job and returns ``'ok'``, the worker's ``check_state`` timer runs
``trnr.check_msg(msg)`` and then calls ``fn_X_end`` back on the scheduler, which counts
acks; necklace/trainer/tndsnc.py:190-222, :364-372, :605-726).  Endpoint names, ``cmd``
strings and ``ret`` values are those of the six reference service files
(tndsnc / tndsms / tndsmp / tndspp / tndszr / tndszd).

What differs:

* one implementation: the per-mode protocol is a *phase program* (a generator that
  yields "send this command to these ranks and wait for that many acks"), instead of
  six copied files with numeric state codes;
* a fast mode (default): the scheduler sends ``run_epoch`` once per epoch and the
  workers run every step, collective and optimizer update of that epoch without any
  RPC in between; ``stepwise=True`` replays the reference's per-phase protocol;
* no fixed sleeps: communicator bring-up is acknowledged like any other phase;
* failure handling: every phase has a deadline, workers send heartbeats from a thread of
  their own (so a long epoch or communicator bring-up does not silence them, and a worker
  that died or hangs is noticed within ``heartbeat_timeout``, not ``phase_timeout``), RPC
  errors are checked; on a missing worker the scheduler broadcasts ``fn_abort`` and ends with
  an error status instead of waiting forever (the reference never checks RPC returns
  and waits for registrations indefinitely, tndsnc.py:464-499).
"""
from __future__ import annotations

import os
import threading
import time
import traceback

from ..rpc import ilog, svctmp, zrpc

# Log channels.  The reference numbers four channels per service flavour (worker / scheduler,
# RPC server "SVR" / state machine "SVC"; tndsmp.py:14-17, tndspp.py:14-21, tndszr.py:14-26) and
# user scripts switch them on with ``ilog.il_add(tndszd.ILOG_I_ZR_SVR_WKR)``.  One service
# serves all flavours here, so a message goes out if any flavour's channel of its kind is on;
# the flavour modules (tndsmp, tndspp, tndszr, tndszd) export the reference's names and numbers.
ILOG_I_SVC_WORKER, ILOG_I_SVC_SCHEDULER = 500001, 500002
ILOG_I_MP_WORKER, ILOG_I_MP_SCHEDULER = 600001, 600002
ILOG_I_ZR_WORKER, ILOG_I_ZR_SCHEDULER = 800001, 800002
ILOG_CHANNELS = {
    "svr_wkr": (600001, 600011, 800001),            # worker: RPC endpoints
    "svc_wkr": (500001, 600002, 600012, 800002),    # worker: state machine
    "svr_sch": (600003, 600021, 800003),            # scheduler: RPC endpoints
    "svc_sch": (500002, 600004, 600022, 800004),    # scheduler: state machine / phases
    "prt_wkr": (600015, 600016),                    # verbose (pipeline flavour)
    "prt_sch": (600025, 600026),
}


def _dbg(kind, *args):
    ilog.debug_any(ILOG_CHANNELS[kind], *args)

# command endpoint on the worker -> callback endpoint on the scheduler
PHASES = {
    "fn_init_nccl_comm": "fn_init_nccl_comm_end",
    "fn_init_nccl_comm_pg": "fn_init_nccl_comm_pg_end",
    "fn_reset_distdt_indices": "fn_reset_distdt_indices_end",
    "fn_weights_sync_start": "fn_weights_sync_end",
    "fn_one_step_start": "fn_one_step_end",
    "fn_nccl_all_reduce_start": "fn_nccl_all_reduce_end",
    "fn_next_epoch_start": "fn_next_epoch_end",
    "fn_run_epoch_start": "fn_run_epoch_end",
    "fn_one_mp_step_start": "fn_one_mp_step_ack",
    "fn_one_mp_step_forward": "fn_one_mp_step_forwarded",
    "fn_one_mp_step_trans_outputs": "fn_one_mp_step_outputs_transed",
    "fn_one_mp_step_calc_loss": "fn_one_mp_step_loss_calced",
    "fn_one_mp_step_trans_grads": "fn_one_mp_step_grads_transed",
    "fn_one_mp_step_backward": "fn_one_mp_step_backwarded",
    "fn_one_zr_step_start": "fn_one_zr_step_ack",
    "fn_one_zr_step_fwd_weig_brcast": "fn_one_zr_step_fwd_weig_brcast_resp",
    "fn_one_zr_step_calc_loss": "fn_one_zr_step_loss_calced",
    "fn_one_zr_step_bcwd_grad_reduce": "fn_one_zr_step_bcwd_grad_reduce_resp",
    "fn_one_zr_step_bcwd_weig_brcast": "fn_one_zr_step_bcwd_weig_brcast_resp",
    "fn_one_zr_step_opt_one_step": "fn_one_zr_step_opt_one_step_resp",
}

Q_STATE_REG, Q_STATE_CMD, Q_STATE_STOP, Q_STATE_ABORT, Q_STATE_RET = 40, 11, 20, 21, 42


class TrainAborted(RuntimeError):
    pass


# =============================================================================== worker
class SVRWorker(svctmp.TmplServer):
    """RPC endpoints of a worker.  ``self.trnr`` is the operator."""

    def __init__(self, cfg):
        super().__init__(cfg)
        self.scheduler_url = cfg.get("scheduler_url")
        trainer_cls, trainer_cfg = cfg.get("trainer_cls"), dict(cfg.get("trainer_cfg") or {})
        trainer_cfg.setdefault("ti", self.rank)
        self.trnr = trainer_cls(trainer_cfg) if trainer_cls is not None else None
        self.schd = None

    def scheduler_cli(self):
        if self.schd is None:
            self.schd = self.mk_rpc_cli(self.scheduler_url, rank=self.rank,
                                        zc_hb_timeout=self.cfg.get("rpc_timeout", 100))
        return self.schd

    # synchronous endpoints ---------------------------------------------------------
    def fn_init_train(self, msg):
        return self.msg_pck(self.mk_rpc_ret("fn_init_train", "ok"))

    def fn_cre_nccl(self, msg):
        m = self.msg_unpck(msg)
        self.trnr.cre_nccl(m.get("msg"))
        return self.msg_pck(self.mk_rpc_ret("fn_cre_nccl", "ok"))

    def fn_cre_nccl_nuid(self, msg):
        return self.msg_pck(self.mk_rpc_ret("fn_cre_nccl_nuid", "ok",
                                            nuid=self.trnr.cre_nccl_nuid()))

    def fn_cre_nccl_nuid_pg(self, msg):
        return self.msg_pck(self.mk_rpc_ret("fn_cre_nccl_nuid_pg", "ok",
                                            nuid=self.trnr.cre_nccl_nuid_pg()))

    def fn_cre_distdt_indices(self, msg):
        m = self.msg_unpck(msg)
        return self.msg_pck(self.mk_rpc_ret("fn_cre_distdt_indices", "ok",
                                            dt_indices=self.trnr.cre_distdt_indices(m.get("msg"))))

    def fn_stop_train(self, msg=None):
        self.q_put_state(Q_STATE_STOP)
        return self.msg_pck(self.mk_rpc_ret("fn_stop_train", "ok"))

    def fn_abort(self, msg=None):
        self.q_put_state(Q_STATE_ABORT, self.msg_unpck(msg) if msg else {})
        return self.msg_pck(self.mk_rpc_ret("fn_abort", "ok"))

    def _phase_endpoint(self, fn, msg):
        m = self.msg_unpck(msg)
        _dbg("svr_wkr", f"worker {self.rank}: <- {fn}")
        self.q_put_state(Q_STATE_CMD, fn, m.get("msg") or {})
        return self.msg_pck(self.mk_rpc_ret(fn, "ok"))


def _mk_worker_endpoint(fn):
    def endpoint(self, msg):
        return self._phase_endpoint(fn, msg)
    endpoint.__name__ = fn
    return endpoint


for _fn in PHASES:
    setattr(SVRWorker, _fn, _mk_worker_endpoint(_fn))


class SVCWorker(svctmp.TmplService):
    def __init__(self, cfg):
        super().__init__(cfg)
        self.svr = SVRWorker(cfg)
        self.rank = self.svr.rank
        self.hb_interval = float(cfg.get("heartbeat", 2.0))
        # the scheduler may come up much later than a worker (each process first builds its
        # copy of the model): keep knocking for half an hour by default
        self.reg_deadline = time.time() + float(cfg.get("register_timeout", 1800))
        self.exit_status = "running"
        self.q_put_state(Q_STATE_REG)
        self._hb_thread = None
        self._hb_stop = threading.Event()

    # --------------------------------------------------------------------- timers
    def tm_to_sleep(self):
        return 0.0  # check_state blocks on the queue instead

    def _heartbeat_loop(self):
        """Runs in its own daemon thread with its own client socket (ZeroMQ sockets must not
        be shared between threads): the service thread may sit inside ``run_epoch`` for the
        whole epoch, and the scheduler must still hear from this process."""
        cli = self.svr.mk_rpc_cli(self.svr.scheduler_url, rank=self.rank,
                                  zc_hb_timeout=max(self.hb_interval, 1.0))
        try:
            while not self._hb_stop.wait(self.hb_interval):
                if self.exit_status != "registered":
                    continue
                try:
                    cli.call("fn_heartbeat", self.rank, timeout=max(self.hb_interval, 1.0))
                except zrpc.RpcError:
                    pass
        finally:
            cli.close()

    def start_heartbeats(self):
        if self.hb_interval > 0 and self._hb_thread is None:
            self._hb_thread = threading.Thread(target=self._heartbeat_loop, daemon=True,
                                               name=f"heartbeat-{self.rank}")
            self._hb_thread.start()

    def stop(self):
        self._hb_stop.set()
        super().stop()

    def check_state(self, *args, **kwargs):
        state, a, k = self.q_get_state(timeout=0.05)
        if state is None:
            return
        try:
            if state == Q_STATE_REG:
                self.do_worker_reg()
            elif state == Q_STATE_CMD:
                self.do_cmd(*a)
            elif state == Q_STATE_STOP:
                _dbg("svc_wkr", f"worker {self.rank}: stop")
                self.svr.trnr.clear()
                self.exit_status = "stopped"
                self.stop()
            elif state == Q_STATE_ABORT:
                ilog.debug(1, f"worker {self.rank}: abort {a}")
                try:
                    self.svr.trnr.del_nccl_comm()
                except Exception:  # noqa: BLE001
                    pass
                self.exit_status = "aborted"
                self.stop()
        except Exception as e:  # noqa: BLE001
            ilog.debug(1, f"worker {self.rank} failed in state {state}: {e}\n"
                          f"{traceback.format_exc()}")
            self.report_failure(repr(e))
            self.exit_status = "failed"
            self.stop()

    # --------------------------------------------------------------------- actions
    def do_worker_reg(self):
        svr = self.svr
        try:
            rep = svr.do_rpc_call(svr.scheduler_cli(), "fn_worker_reg", url=svr.url)
            if rep.get("ret") == "ok":
                self.exit_status = "registered"
                self.start_heartbeats()
                return
        except zrpc.RpcError:
            pass
        if time.time() > self.reg_deadline:
            raise TrainAborted(f"worker {self.rank}: scheduler {svr.scheduler_url} unreachable")
        time.sleep(0.2)
        self.q_put_state(Q_STATE_REG)

    def do_cmd(self, fn, msg):
        svr = self.svr
        _dbg("svc_wkr", f"worker {self.rank}: do {fn}")
        _dbg("prt_wkr", f"worker {self.rank}: {fn} msg keys {sorted(msg) if isinstance(msg, dict) else msg}")
        if fn == "fn_init_nccl_comm":
            svr.trnr.init_nccl_comm(msg)
            ret = {"ret": "nccl_comm_inited"}
        elif fn == "fn_init_nccl_comm_pg":
            svr.trnr.init_nccl_comm_pg(msg)
            ret = {"ret": "nccl_comm_pg_inited"}
        elif fn == "fn_reset_distdt_indices":
            svr.trnr.reset_distdt_indices(msg)
            ret = {"ret": "distdt_indices_reset"}
        else:
            ret = svr.trnr.check_msg(msg)
        svr.do_rpc_call(svr.scheduler_cli(), PHASES[fn], **ret)

    def report_failure(self, why):
        try:
            self.svr.do_rpc_call(self.svr.scheduler_cli(), "fn_worker_failed", why=why)
        except Exception:  # noqa: BLE001
            pass


# ============================================================================ scheduler
class SVRScheduler(svctmp.TmplServer):
    def __init__(self, cfg):
        super().__init__(cfg)
        self.heartbeats = {}

    def fn_worker_reg(self, msg):
        m = self.msg_unpck(msg)
        self.q_put_state(Q_STATE_REG, m["rank"], m["msg"]["url"])
        return self.msg_pck(self.mk_rpc_ret("fn_worker_reg", "ok"))

    def fn_heartbeat(self, rank):
        self.heartbeats[rank] = time.time()
        return "ok"

    def fn_worker_failed(self, msg):
        m = self.msg_unpck(msg)
        self.q_put_state(Q_STATE_ABORT, m["rank"], m["msg"].get("why"))
        return self.msg_pck(self.mk_rpc_ret("fn_worker_failed", "ok"))

    def _ack(self, fn, msg):
        m = self.msg_unpck(msg)
        _dbg("svr_sch", f"scheduler: <- {fn} from worker {m.get('rank')}")
        self.q_put_state(Q_STATE_RET, fn, m["rank"], m["msg"])
        return self.msg_pck(self.mk_rpc_ret(fn, "ok"))


def _mk_sched_endpoint(fn):
    def endpoint(self, msg):
        return self._ack(fn, msg)
    endpoint.__name__ = fn
    return endpoint


for _fn in set(PHASES.values()):
    setattr(SVRScheduler, _fn, _mk_sched_endpoint(_fn))


class Phase:
    def __init__(self, fn, ranks, msg, n_acks=None, per_rank=None):
        self.fn, self.ranks, self.msg = fn, list(ranks), msg
        self.per_rank = per_rank or {}            # rank -> extra msg fields
        self.n_acks = len(self.ranks) if n_acks is None else n_acks
        self.acks = {}


class SVCScheduler(svctmp.TmplService):
    """cfg: ``url, workers (count), epochs, nccl_allreduce_typ, net_map, stepwise,
    nccl_groups_grp_map, phase_timeout (600 s), heartbeat_timeout (15 s; 0 = off),
    register_timeout (1800 s: the reference waits for registrations without limit), start_epoch (epochs a resumed job has already done, see
    trainer/resume.py)``."""

    def __init__(self, cfg):
        super().__init__(cfg)
        self.svr = SVRScheduler(cfg)
        self.workers_n = int(cfg.get("workers") or cfg.get("wdsz") or 1)
        self.epochs = int(cfg.get("epochs", 1))
        self.typ = cfg.get("nccl_allreduce_typ", "grad")
        # per-phase protocol of the reference instead of one command per epoch; NKB_STEPWISE=1
        # switches it on for scripts that cannot pass the cfg key
        self.stepwise = bool(cfg.get("stepwise", os.environ.get("NKB_STEPWISE", "0") == "1"))
        self.phase_timeout = float(cfg.get("phase_timeout", 600))
        # a worker that has sent a heartbeat once and then stays silent this long is taken
        # for dead (workers send one every 2 s by default); 0 switches the check off
        self.hb_timeout = float(cfg.get("heartbeat_timeout", 15))
        self.reg_deadline = time.time() + float(cfg.get("register_timeout", 1800))
        self.net_map = cfg.get("net_map")
        self.grp_map = cfg.get("nccl_groups_grp_map") or {}
        self.worker_urls, self.worker_clis = {}, {}
        self.program = None
        self.phase: Phase | None = None
        self.phase_started = 0.0
        self.epoch = int(cfg.get("start_epoch", 0))   # epochs already done (resumed job)
        self.exit_status = "running"
        self.history = []  # (fn, ret values) per completed phase, for tests / debugging

    def tm_to_sleep(self):
        return 0.0

    @property
    def all_ranks(self):
        return list(range(self.workers_n))

    # ---------------------------------------------------------------- sending
    def send(self, rank, fn, **kwargs):
        return self.svr.do_rpc_call(self.worker_clis[rank], fn, **kwargs)

    def start_phase(self, ph: Phase):
        self.phase, self.phase_started = ph, time.time()
        _dbg("svc_sch", f"scheduler: phase {ph.fn} -> workers {list(ph.ranks)}")
        _dbg("prt_sch", f"scheduler: phase {ph.fn} msg keys {sorted(ph.msg)}")
        for r in ph.ranks:
            rep = self.send(r, ph.fn, **{**ph.msg, **ph.per_rank.get(r, {})})
            if rep.get("ret") != "ok":
                raise TrainAborted(f"worker {r} rejected {ph.fn}: {rep}")

    def abort(self, why):
        ilog.debug(1, f"scheduler: abort: {why}")
        for r, cli in self.worker_clis.items():
            try:
                cli.call("fn_abort", self.svr.msg_pck(self.svr.mk_rpc_msg("fn_abort", why=why)),
                         timeout=2)
            except Exception:  # noqa: BLE001
                pass
        self.exit_status = "aborted: " + str(why)
        self.stop()

    # ---------------------------------------------------------------- state machine
    def check_state(self, *args, **kwargs):
        state, a, k = self.q_get_state(timeout=0.05)
        try:
            if state == Q_STATE_REG:
                self.on_worker_reg(*a)
            elif state == Q_STATE_RET:
                self.on_ack(*a)
            elif state == Q_STATE_ABORT:
                self.abort(f"worker {a[0]} failed: {a[1]}")
                return
            self.check_deadlines()
        except zrpc.RpcError as e:
            self.abort(f"rpc failure: {e}")
        except TrainAborted as e:
            self.abort(str(e))

    def check_deadlines(self):
        now = time.time()
        if self.program is None:
            if now > self.reg_deadline:
                raise TrainAborted(f"only {len(self.worker_urls)} of {self.workers_n} workers "
                                   f"registered in time")
            return
        if self.phase is not None and now - self.phase_started > self.phase_timeout:
            missing = [r for r in self.phase.ranks if r not in self.phase.acks]
            raise TrainAborted(f"phase {self.phase.fn} timed out waiting for ranks {missing}")
        if self.hb_timeout > 0:
            for r in self.all_ranks:
                last = self.svr.heartbeats.get(r)
                if last is not None and now - last > self.hb_timeout:
                    raise TrainAborted(f"worker {r} stopped sending heartbeats")

    def on_worker_reg(self, rank, url):
        self.worker_urls[rank] = url
        _dbg("svc_sch", f"scheduler: worker {rank} registered at {url}")
        if len(self.worker_urls) == self.workers_n and self.program is None:
            for r, u in self.worker_urls.items():
                self.worker_clis[r] = self.svr.mk_rpc_cli(
                    u, rank=r, zc_hb_timeout=self.cfg.get("rpc_timeout", 100))
            self.program = self.make_program()
            self.advance(None)

    def on_ack(self, fn, rank, msg):
        ph = self.phase
        if ph is None or PHASES.get(ph.fn) != fn:
            return  # late ack of an abandoned phase
        ph.acks[rank] = msg
        if len(ph.acks) >= ph.n_acks:
            self.history.append((ph.fn, {r: m.get("ret") for r, m in ph.acks.items()}))
            self.phase = None
            self.advance(ph.acks)

    def advance(self, acks):
        try:
            ph = self.program.send(acks)
        except StopIteration:
            self.finish()
            return
        self.start_phase(ph)

    def finish(self):
        for r in self.all_ranks:
            try:
                self.send(r, "fn_stop_train")
            except zrpc.RpcError:
                pass
        self.exit_status = "finished"
        self.stop()

    # ---------------------------------------------------------------- programs
    # The reference has one scheduler class per flavour and picks the protocol by class
    # (tndsnc: dp, tndsmp / tndspp: pipeline over net_map, tndszr / tndszd: ZeRO); the flavour
    # modules here subclass with FLAVOUR set, so a script that builds ``tndszr.MPSVCScheduler``
    # with the reference's default ``nccl_allreduce_typ='grad'`` still gets the ZeRO program.
    FLAVOUR = None

    def make_program(self):
        yield from self.prog_init()
        if self.FLAVOUR == "zr" and self.typ in ("grad", "weig", None):
            self.typ = "oozr"
        typ = self.typ
        if typ in ("oozr", "dpzr", "dpzrmp", "zrmp"):
            yield from self.prog_zr()
        elif self.net_map and typ not in ("oozr",) and self.cfg.get("pp_mode", True) and \
                any("worker_rank" in v for v in self.net_map.values()):
            yield from self.prog_pp()
        else:
            yield from self.prog_dp()

    def prog_init(self):
        for r in self.all_ranks:
            self.send(r, "fn_init_train")
            self.send(r, "fn_cre_nccl", cfg={"kn": self.workers_n, "rank": r})
        nuid = self.send(0, "fn_cre_nccl_nuid")["msg"]["nuid"]
        yield Phase("fn_init_nccl_comm", self.all_ranks, {"nuid": nuid})
        # per-group bring-up of the reference protocol (state 900011): the groups already
        # exist after fn_init_nccl_comm; the messages are kept for protocol parity
        if self.stepwise and self.grp_map:
            for key, groups in self.grp_map.items():
                for grp in groups:
                    g_nuid = self.send(grp[0], "fn_cre_nccl_nuid_pg")["msg"]["nuid"]
                    yield Phase("fn_init_nccl_comm_pg", grp, {}, per_rank={
                        r: {"cfg": {"wkr_rank": r, "nuid": g_nuid, "pg_rank": i,
                                    "world_size": len(grp), "pg_key": key}}
                        for i, r in enumerate(grp)})

    def prog_dp(self):
        typ = self.typ
        if typ in ("grad", "weig"):
            yield Phase("fn_weights_sync_start", self.all_ranks, {"cmd": "weights_sync", "typ": typ})
        while self.epoch < self.epochs:
            if self.cfg.get("use_dist_data_sampler"):
                idx = self.send(0, "fn_cre_distdt_indices")["msg"]["dt_indices"]
                yield Phase("fn_reset_distdt_indices", self.all_ranks, {"dt_indices": idx})
            if not self.stepwise:
                yield Phase("fn_run_epoch_start", self.all_ranks, {"cmd": "run_epoch", "typ": typ})
            else:
                while True:
                    acks = yield Phase("fn_one_step_start", self.all_ranks,
                                       {"cmd": "one_step", "typ": typ})
                    if all(m.get("ret") == "epoch_end" for m in acks.values()):
                        break
                    yield Phase("fn_nccl_all_reduce_start", self.all_ranks,
                                {"cmd": "nccl_all_reduce", "typ": typ})
            self.epoch += 1
            yield Phase("fn_next_epoch_start", self.all_ranks, {"cmd": "next_epoch"})

    # pipeline: stage i of every pp group is addressed together ---------------------
    def _pp_groups(self):
        groups = self.grp_map.get("pp_group")
        if groups:
            return groups
        ranks = [v["worker_rank"] for _, v in sorted(self.net_map.items())]
        return [ranks]

    def prog_pp(self):
        typ = self.typ
        pp_groups = self._pp_groups()
        n_stage = len(pp_groups[0])
        stage_ranks = [[g[i] for g in pp_groups] for i in range(n_stage)]
        yield Phase("fn_weights_sync_start", self.all_ranks, {"cmd": "weights_sync", "typ": typ})
        while self.epoch < self.epochs:
            if not self.stepwise:
                yield Phase("fn_run_epoch_start", self.all_ranks, {"cmd": "run_epoch", "typ": typ})
            else:
                while True:
                    yield Phase("fn_one_mp_step_start", self.all_ranks,
                                {"cmd": "one_mp_step_start", "typ": typ})
                    ended, shp = False, {}
                    for i in range(n_stage):
                        acks = yield Phase("fn_one_mp_step_forward", stage_ranks[i],
                                           {"cmd": "one_mp_step_forward", "typ": typ})
                        if any(m.get("ret") == "mp_epoch_end" for m in acks.values()):
                            ended = True
                            break
                        shp = next(iter(acks.values()))
                        if i < n_stage - 1:
                            pr = {}
                            for g in pp_groups:
                                m = {"cmd": "one_mp_step_trans_outputs", "from_rank": g[i],
                                     "to_rank": g[i + 1], "output_shps": shp.get("output_shps"),
                                     "output_dts": shp.get("output_dts")}
                                pr[g[i]] = m
                                pr[g[i + 1]] = m
                            yield Phase("fn_one_mp_step_trans_outputs",
                                        stage_ranks[i] + stage_ranks[i + 1], {"typ": typ},
                                        per_rank=pr)
                    if ended:
                        break
                    pr = {}
                    for g in pp_groups:
                        m = {"cmd": "one_mp_step_calc_loss", "from_rank": g[0], "to_rank": g[-1]}
                        pr[g[0]] = m
                        pr[g[-1]] = m
                    tgt = sorted(set(stage_ranks[0] + stage_ranks[-1]))
                    acks = yield Phase("fn_one_mp_step_calc_loss", tgt, {"typ": typ}, per_rank=pr)
                    for i in range(n_stage - 1, 0, -1):
                        pr = {}
                        for g in pp_groups:
                            m = {"cmd": "one_mp_step_trans_grads", "from_rank": g[i],
                                 "to_rank": g[i - 1]}
                            pr[g[i]] = m
                            pr[g[i - 1]] = m
                        yield Phase("fn_one_mp_step_trans_grads",
                                    stage_ranks[i] + stage_ranks[i - 1], {"typ": typ}, per_rank=pr)
                        yield Phase("fn_one_mp_step_backward", stage_ranks[i - 1],
                                    {"cmd": "one_mp_step_backward", "typ": typ})
                    yield Phase("fn_nccl_all_reduce_start", self.all_ranks,
                                {"cmd": "nccl_all_reduce", "typ": typ})
            self.epoch += 1
            yield Phase("fn_next_epoch_start", self.all_ranks, {"cmd": "next_epoch"})

    # ZeRO ------------------------------------------------------------------------------
    def prog_zr(self):
        typ = self.typ
        n_sub = len(self.net_map) if self.net_map else int(self.cfg.get("net_map_maxlen", 1))
        while self.epoch < self.epochs:
            if not self.stepwise:
                yield Phase("fn_run_epoch_start", self.all_ranks, {"cmd": "run_epoch", "typ": typ})
            else:
                while True:
                    yield Phase("fn_one_zr_step_start", self.all_ranks,
                                {"cmd": "one_zr_step_start", "typ": typ})
                    ended = False
                    for i in range(n_sub):
                        acks = yield Phase("fn_one_zr_step_fwd_weig_brcast", self.all_ranks,
                                           {"cmd": "one_zr_step_fwd_weig_brcast", "typ": typ,
                                            "one_zr_step_order_i": i})
                        if any(m.get("ret") == "zr_epoch_end" for m in acks.values()):
                            ended = True
                            break
                    if ended:
                        break
                    yield Phase("fn_one_zr_step_calc_loss", self.all_ranks,
                                {"cmd": "one_zr_step_calc_loss", "typ": typ,
                                 "one_zr_step_order_i": n_sub - 1})
                    for i in range(n_sub - 1, -1, -1):
                        yield Phase("fn_one_zr_step_bcwd_grad_reduce", self.all_ranks,
                                    {"cmd": "one_zr_step_bcwd_grad_reduce", "typ": typ,
                                     "one_zr_step_order_i": i})
                        if i > 0:
                            yield Phase("fn_one_zr_step_bcwd_weig_brcast", self.all_ranks,
                                        {"cmd": "one_zr_step_bcwd_weig_brcast", "typ": typ,
                                         "one_zr_step_order_i": i - 1})
                    yield Phase("fn_one_zr_step_opt_one_step", self.all_ranks,
                                {"cmd": "one_zr_step_opt_one_step", "typ": typ})
            self.epoch += 1
            yield Phase("fn_next_epoch_start", self.all_ranks, {"cmd": "next_epoch"})


# names used by the pipeline / ZeRO service modules of the reference
MPSVRWorker, MPSVCWorker = SVRWorker, SVCWorker
MPSVRScheduler, MPSVCScheduler = SVRScheduler, SVCScheduler
