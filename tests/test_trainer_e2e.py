"""Scheduler + worker processes over ipc:// on CPU (gloo), and host-side failure injection."""
import json
import os
import subprocess
import sys
import time

import pytest
import torch
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXAMPLE = os.path.join(ROOT, "examples", "dp", "train_mnist_dp.py")


def _spawn(args, log):
    return subprocess.Popen([sys.executable, EXAMPLE, *args], stdout=open(log, "w"),
                            stderr=subprocess.STDOUT, cwd=ROOT)


def _run_job(tmp_path, world, extra_sched=(), extra_worker=(), epochs=1, dataset_len=400,
             batch=50, timeout=150):
    svr = f"ipc://{tmp_path}/svr.ipc"
    procs = [_spawn(["-r", "scheduler", "-w", str(world), "-u", svr, "-e", str(epochs),
                     *extra_sched], tmp_path / "s.log")]
    for r in range(world):
        procs.append(_spawn(["-r", "worker", "-w", str(world), "-k", str(r), "-u",
                             f"ipc://{tmp_path}/w{r}.ipc", "-s", svr,
                             "-t", "dp" if world > 1 else "no", "--no-cuda", "-e", str(epochs),
                             "--dataset-len", str(dataset_len), "-b", str(batch),
                             "--out", str(tmp_path / f"o{r}.json"), *extra_worker],
                            tmp_path / f"w{r}.log"))
    t0 = time.time()
    codes = []
    for p in procs:
        try:
            codes.append(p.wait(timeout=max(1, timeout - (time.time() - t0))))
        except subprocess.TimeoutExpired:
            p.kill()
            codes.append(-9)
    outs = []
    for r in range(world):
        f = tmp_path / f"o{r}.json"
        outs.append(json.load(open(f)) if f.exists() else None)
    return codes, outs


def _single_process(world, epochs, dataset_len, batch, lr=0.01, seed=1):
    """The same training in one process on the global batch (mean of per-rank means)."""
    sys.path.insert(0, ROOT)
    from necklace_b200.data.dtset import SyntheticDataset
    from necklace_b200.models.lenet import LeNet
    torch.manual_seed(seed)
    net = LeNet()
    opt = torch.optim.SGD(net.parameters(), lr=lr)
    ds = SyntheticDataset(dataset_len, (1, 28, 28), classes=10, seed=seed)
    per = dataset_len // world
    ce = nn.CrossEntropyLoss()
    for _ in range(epochs):
        for i in range(per // batch):
            opt.zero_grad()
            loss = 0
            for r in range(world):
                idx = range(r * per + i * batch, r * per + (i + 1) * batch)
                x = torch.stack([ds[j][0] for j in idx])
                y = torch.tensor([ds[j][1] for j in idx])
                loss = loss + ce(net(x), y) / world
            loss.backward()
            opt.step()
    return float(sum(p.double().sum() for p in net.parameters()))


@pytest.mark.timeout(200)
def test_mode_no_single_worker_matches_plain_loop(tmp_path):
    codes, outs = _run_job(tmp_path, 1, epochs=2)
    assert codes == [0, 0], open(tmp_path / "w0.log").read()[-2000:]
    ref = _single_process(1, 2, 400, 50)
    assert abs(outs[0]["weights_sum"] - ref) < 1e-4
    assert len(outs[0]["epoch_loss"]) == 2


@pytest.mark.timeout(300)
@pytest.mark.parametrize("stepwise", [False, True])
def test_dp_two_workers_match_single_process(tmp_path, stepwise):
    extra = ["--stepwise"] if stepwise else []
    codes, outs = _run_job(tmp_path, 2, extra_sched=extra)
    assert codes == [0, 0, 0], open(tmp_path / "w0.log").read()[-2000:]
    assert abs(outs[0]["weights_sum"] - outs[1]["weights_sum"]) < 1e-9
    ref = _single_process(2, 1, 400, 50)
    assert abs(outs[0]["weights_sum"] - ref) < 1e-3


@pytest.mark.timeout(300)
def test_dp_with_2bit_gradient_compression_keeps_ranks_in_sync(tmp_path):
    codes, outs = _run_job(tmp_path, 2, extra_worker=["--grad-comp-threshold", "0.001"])
    assert codes == [0, 0, 0], open(tmp_path / "w0.log").read()[-2000:]
    assert abs(outs[0]["weights_sum"] - outs[1]["weights_sum"]) < 1e-9


@pytest.mark.timeout(120)
def test_scheduler_aborts_when_a_worker_never_registers(tmp_path):
    sys.path.insert(0, ROOT)
    from necklace_b200.trainer.service import SVCScheduler
    svc = SVCScheduler({"url": f"ipc://{tmp_path}/svr.ipc", "workers": 2, "epochs": 1,
                        "register_timeout": 1.0})
    t0 = time.time()
    svc.loop()
    assert time.time() - t0 < 20
    assert svc.exit_status.startswith("aborted") and "registered" in svc.exit_status


class _StallTrainer:
    """Fake operator: acknowledges communicator bring-up, then one rank never answers."""

    def __init__(self, cfg):
        self.cfg = cfg
        self.ti = cfg["ti"]

    def cre_nccl(self, msg=None):
        return "ok"

    def cre_nccl_nuid(self, msg=None):
        return {"master_addr": "127.0.0.1", "master_port": 1}

    def init_nccl_comm(self, msg=None):
        return "ok"

    def del_nccl_comm(self, msg=None):
        pass

    def check_msg(self, msg):
        if self.cfg.get("mode") == "raise" and msg["cmd"] == "run_epoch" and self.ti == 1:
            raise RuntimeError("injected failure in the training step")
        if self.cfg.get("mode") == "stall" and msg["cmd"] == "run_epoch" and self.ti == 1:
            time.sleep(30)
        if self.cfg.get("mode") == "slow" and msg["cmd"] == "run_epoch":
            time.sleep(3)
        return {"ret": {"weights_sync": "weights_synced", "run_epoch": "epoch_end",
                        "next_epoch": "next_epoch"}[msg["cmd"]]}

    def clear(self):
        pass


def _worker_thread(tmp_path, rank, mode):
    from necklace_b200.trainer.service import SVCWorker
    svc = SVCWorker({"url": f"ipc://{tmp_path}/w{rank}.ipc",
                     "scheduler_url": f"ipc://{tmp_path}/svr.ipc", "rank": rank,
                     "trainer_cls": _StallTrainer, "trainer_cfg": {"mode": mode},
                     "heartbeat": 0.2})
    svc.loop()
    return svc


@pytest.mark.timeout(120)
@pytest.mark.parametrize("mode,needle", [("raise", "injected failure"), ("stall", "timed out")])
def test_worker_failure_mid_step_aborts_everyone(tmp_path, mode, needle):
    """A rank raises inside a step (reported at once) or goes silent (phase deadline):
    the scheduler broadcasts abort and every survivor leaves its loop."""
    import threading
    sys.path.insert(0, ROOT)
    from necklace_b200.trainer.service import SVCScheduler
    results = {}
    ths = [threading.Thread(target=lambda r=r: results.__setitem__(r, _worker_thread(tmp_path, r, mode)),
                            daemon=True) for r in range(2)]
    for t in ths:
        t.start()
    svc = SVCScheduler({"url": f"ipc://{tmp_path}/svr.ipc", "workers": 2, "epochs": 1,
                        "phase_timeout": 2.0, "register_timeout": 30})
    svc.loop()
    assert svc.exit_status.startswith("aborted") and needle in svc.exit_status, svc.exit_status
    ths[0].join(timeout=10)
    assert not ths[0].is_alive()
    assert results[0].exit_status == "aborted"


def _worker_proc(tmp, rank, mode):
    sys.path.insert(0, ROOT)
    _worker_thread(tmp, rank, mode)


@pytest.mark.timeout(120)
def test_killed_worker_is_noticed_by_missing_heartbeats(tmp_path):
    """Rank 1 is killed (SIGKILL) while it sits in ``run_epoch``.  The phase deadline is far
    away (300 s); the scheduler must abort because the heartbeats stopped."""
    import multiprocessing as mp
    import threading
    sys.path.insert(0, ROOT)
    from necklace_b200.trainer.service import SVCScheduler
    ctx = mp.get_context("spawn")
    victim = ctx.Process(target=_worker_proc, args=(str(tmp_path), 1, "stall"), daemon=True)
    victim.start()
    results = {}
    th = threading.Thread(target=lambda: results.__setitem__(0, _worker_thread(tmp_path, 0, "stall")),
                          daemon=True)
    th.start()
    svc = SVCScheduler({"url": f"ipc://{tmp_path}/svr.ipc", "workers": 2, "epochs": 1,
                        "phase_timeout": 300.0, "heartbeat_timeout": 1.5,
                        "register_timeout": 60})

    def killer():
        while not any(fn == "fn_weights_sync_start" for fn, _ in svc.history):
            time.sleep(0.05)
        time.sleep(1.0)            # run_epoch has been sent; rank 1 is asleep inside it
        victim.kill()

    threading.Thread(target=killer, daemon=True).start()
    t0 = time.time()
    svc.loop()
    assert svc.exit_status.startswith("aborted") and "heartbeat" in svc.exit_status, svc.exit_status
    assert time.time() - t0 < 60
    th.join(timeout=10)
    assert results[0].exit_status == "aborted"


@pytest.mark.timeout(120)
def test_slow_but_healthy_epoch_is_not_aborted(tmp_path):
    """An epoch longer than the heartbeat timeout: the heartbeat thread keeps talking while the
    service thread is busy, so nobody is aborted."""
    import threading
    sys.path.insert(0, ROOT)
    from necklace_b200.trainer.service import SVCScheduler
    ths = [threading.Thread(target=_worker_thread, args=(tmp_path, r, "slow"), daemon=True)
           for r in range(2)]
    for t in ths:
        t.start()
    svc = SVCScheduler({"url": f"ipc://{tmp_path}/svr.ipc", "workers": 2, "epochs": 1,
                        "phase_timeout": 60.0, "heartbeat_timeout": 1.0, "register_timeout": 30})
    svc.loop()
    assert svc.exit_status == "finished", svc.exit_status


@pytest.mark.timeout(120)
def test_protocol_phases_against_fake_trainer(tmp_path):
    """Stepwise DP protocol: the scheduler issues the reference's phase sequence."""
    import threading
    sys.path.insert(0, ROOT)
    from necklace_b200.trainer.service import SVCScheduler, SVCWorker

    class Fake(_StallTrainer):
        def __init__(self, cfg):
            super().__init__(cfg)
            self.steps = 0

        def check_msg(self, msg):
            c = msg["cmd"]
            if c == "one_step":
                self.steps += 1
                return {"ret": "one_step" if self.steps <= 2 else "epoch_end"}
            return {"ret": {"weights_sync": "weights_synced", "nccl_all_reduce": "nccl_all_reduced",
                            "next_epoch": "next_epoch"}[c]}

    def worker(rank):
        SVCWorker({"url": f"ipc://{tmp_path}/w{rank}.ipc", "scheduler_url": f"ipc://{tmp_path}/svr.ipc",
                   "rank": rank, "trainer_cls": Fake, "trainer_cfg": {}, "heartbeat": 0}).loop()

    ths = [threading.Thread(target=worker, args=(r,), daemon=True) for r in range(2)]
    for t in ths:
        t.start()
    svc = SVCScheduler({"url": f"ipc://{tmp_path}/svr.ipc", "workers": 2, "epochs": 1,
                        "stepwise": True, "phase_timeout": 20})
    svc.loop()
    assert svc.exit_status == "finished"
    seq = [fn for fn, _ in svc.history]
    assert seq == ["fn_init_nccl_comm", "fn_weights_sync_start", "fn_one_step_start",
                   "fn_nccl_all_reduce_start", "fn_one_step_start", "fn_nccl_all_reduce_start",
                   "fn_one_step_start", "fn_next_epoch_start"]
    assert svc.history[-2][1] == {0: "epoch_end", 1: "epoch_end"}


@pytest.mark.timeout(300)
def test_gpt2_zero_through_scheduler_and_workers_cpu(tmp_path):
    """The headline's process model on CPU: scheduler + 2 workers over ipc, ZeRO trainer with
    the native engine (gloo stand-in group), timed by the trainer hook."""
    script = os.path.join(ROOT, "examples", "gpt2", "train_gpt2_necklace.py")
    svr = f"ipc://{tmp_path}/svr.ipc"
    procs = [subprocess.Popen([sys.executable, script, "-r", "scheduler", "-w", "2", "-u", svr,
                               "-e", "1"], stdout=open(tmp_path / "s.log", "w"),
                              stderr=subprocess.STDOUT, cwd=ROOT)]
    for r in range(2):
        procs.append(subprocess.Popen(
            [sys.executable, script, "-r", "worker", "-w", "2", "-k", str(r), "-u",
             f"ipc://{tmp_path}/w{r}.ipc", "-s", svr, "-t", "dp+zr", "-dpsz", "1", "-zrsz", "2",
             "--no-cuda", "--time-steps", "3", "--time-warmup", "2", "--micro-batch", "2",
             "--out", str(tmp_path / f"o{r}.json")],
            stdout=open(tmp_path / f"w{r}.log", "w"), stderr=subprocess.STDOUT, cwd=ROOT))
    codes = []
    for p in procs:
        try:
            codes.append(p.wait(timeout=240))
        except subprocess.TimeoutExpired:
            p.kill()
            codes.append(-9)
    assert codes == [0, 0, 0], open(tmp_path / "w0.log").read()[-2000:]
    outs = [json.load(open(tmp_path / f"o{r}.json")) for r in range(2)]
    assert all(o["steps"] == 3 and o["ms"] > 0 and o["loss"] < 7.5 for o in outs)


@pytest.mark.timeout(420)
def test_job_restarts_from_its_checkpoint_after_a_worker_failure(tmp_path):
    """Elastic recovery on the host: worker 1 raises at the start of the second epoch, the
    services abort the job, the supervisor starts it again with ``--resume``, scheduler and
    workers continue after the first epoch, and the final weights equal those of a run that
    was never interrupted."""
    from necklace_b200.trainer import resume
    from necklace_b200.utils.supervise import run_job
    script = os.path.join(ROOT, "examples", "dp", "train_mnist_dp.py")

    def cmds(d, extra):
        svr = f"ipc://{d}/s.ipc"
        base = ["--checkpoint-dir", str(d / "ckpt")]
        out = [[sys.executable, script, "-r", "scheduler", "-w", "2", "-u", svr, "-e", "3", *base]]
        for r in range(2):
            out.append([sys.executable, script, "-r", "worker", "-w", "2", "-k", str(r), "-u",
                        f"ipc://{d}/w{r}.ipc", "-s", svr, "-t", "dp", "-e", "3", "--no-cuda",
                        "--dataset-len", "160", "-b", "20", "--momentum", "0.9", "--out",
                        str(d / f"o{r}.json"), *base, *extra])
        return out

    def kw(d):
        def per_attempt(attempt):
            return [{"stdout": open(d / f"p{i}_a{attempt}.log", "w"), "stderr": subprocess.STDOUT,
                     "cwd": ROOT} for i in range(3)]
        return per_attempt

    plain, broken = tmp_path / "plain", tmp_path / "broken"
    for d in (plain, broken):
        (d / "ckpt").mkdir(parents=True)
    codes, restarts = run_job(cmds(plain, []), max_restarts=0, timeout=180, popen_kwargs=kw(plain))
    assert codes == [0, 0, 0] and restarts == 0
    codes, restarts = run_job(cmds(broken, ["--fail-at-epoch", "1"]), max_restarts=2, timeout=180,
                              popen_kwargs=kw(broken))
    logs = "".join(open(f).read()[-1500:] for f in sorted(broken.glob("p*_a*.log")))
    assert codes == [0, 0, 0] and restarts == 1, (codes, restarts, logs)
    assert "injected failure" in open(broken / "p2_a0.log").read()
    assert "resumed after 1 epoch(s)" in open(broken / "p1_a1.log").read()
    assert resume.resume_epoch(str(broken / "ckpt"), 2) == 3
    a = json.load(open(plain / "o0.json"))["weights_sum"]
    b = [json.load(open(broken / f"o{r}.json"))["weights_sum"] for r in range(2)]
    assert abs(b[0] - b[1]) < 1e-9 and abs(a - b[0]) < 1e-7, (a, b)


def test_flavour_modules_pick_their_protocol_and_default_mode(tmp_path):
    """A script that builds ``tndszr.MPSVCScheduler`` with the reference's default
    ``nccl_allreduce_typ='grad'`` gets the ZeRO program (not the data-parallel weight sync),
    and an operator without ``tmode`` forms one group of its own flavour."""
    from necklace_b200.trainer import ppoppt, tndsnc, tndspp, tndszd, tndszr, tnoppt, zroppt
    assert tndszr.MPSVCScheduler.FLAVOUR == "zr" and tndszd.MPSVCScheduler.FLAVOUR == "zr"
    assert tndspp.MPSVCScheduler.FLAVOUR == "pp" and tndsnc.SVCScheduler.FLAVOUR is None
    assert (tnoppt.TrainerOPPytorch.DEFAULT_TMODE, ppoppt.TrainerMPOPPytorch.DEFAULT_TMODE,
            zroppt.TrainerMPOPPytorch.DEFAULT_TMODE) == ("dp", "pp", "zr")
    ran = []
    for cls, want in ((tndszr.MPSVCScheduler, "zr:oozr"), (tndsnc.SVCScheduler, "dp:grad")):
        svc = cls({"url": f"ipc://{tmp_path}/{want[:2]}.ipc", "workers": 1, "epochs": 1,
                   "nccl_allreduce_typ": "grad"})
        svc.prog_init = lambda: iter(())
        svc.prog_zr = lambda s=svc: iter([ran.append("zr:" + s.typ)])
        svc.prog_dp = lambda s=svc: iter([ran.append("dp:" + s.typ)])
        list(svc.make_program())
        svc.svr.stop() if hasattr(svc.svr, "stop") else None
    assert ran == ["zr:oozr", "dp:grad"]
