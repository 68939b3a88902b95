"""The reference's own example scripts, unedited, against this package on the CPU.

Needs the reference's ``examples`` directory: set ``NKB_REFERENCE_EXAMPLES`` to it (skipped
otherwise).  Every case starts one scheduler and N workers with the arguments the script's own
comments give, through ``tests/refexamples/run_example.py`` (import alias, synthetic MNIST,
CPU device), and expects every process to end with exit code 0 after the last epoch."""
import os
import subprocess
import sys

import pytest

EX = os.environ.get("NKB_REFERENCE_EXAMPLES", "")
RUN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "refexamples", "run_example.py")

CASES = [
    ("dp/mnist/pytorch/train_ngn_mnist_1.py", 2, ["--gpus", "0", "-x", "nccl"], {}),
    ("dp/mnist/pytorch/train_ngn_mnist_2_dtpt.py", 2, ["--gpus", "0"], {}),
    ("dp/mnist/pytorch/train_nklc_nccl_mnist_1_mpirun.py", 2, ["--gpus", "0", "-n", "2", "-x", "nccl"],
     {"mpirun": True}),
    ("mp/mnist/pytorch/train_mnist_mpnn_21_one_grp.py", 2, ["-g", "0", "-t", "mp"], {}),
    ("mp/mnist/pytorch/train_mnist_mpnn_22_mpdp_grps.py", 4,
     ["-g", "0", "-t", "dp+mp", "-dpsz", "2", "-mpsz", "2"], {}),
    ("pp/mnist/pytorch/train_mnist_mp_5_nklc.py", 2, ["--gpus", "0"], {}),
    ("pp/mnist/pytorch/train_mnist_pp_31_one_grp.py", 2, ["--gpus", "0"], {}),
    ("pp/mnist/pytorch/train_mnist_pp_32_dppp_grps.py", 4,
     ["-g", "0", "-t", "dp+pp", "-dpsz", "2", "-ppsz", "2"], {}),
    ("zero/mnist/pytorch/train_mnist_zr_1.py", 3, ["--gpus", "0"], {}),
    ("zero/mnist/pytorch/train_mnist_zf_1.py", 3, ["--gpus", "0"], {}),
    ("zero/mnist/pytorch/train_mnist_zr_5_dpzr_2.py", 4,
     ["-g", "0", "-t", "dp+zr", "-dpsz", "2", "-zrsz", "2"], {}),
    ("pp/mnist/pytorch/train_mnist_pp_33_dppp_grps_n3.py", 6,
     ["-g", "0", "-t", "dp+pp", "-dpsz", "2", "-ppsz", "3"], {}),
    ("pp/mnist/pytorch/train_mnist_mp_5_nklc_w3.py", 3, ["--gpus", "0"], {}),
    ("dp/mnist/pytorch/train_nklc_nccl_mnist_3_mlpmx.py", 2, ["--gpus", "0"], {}),
    ("zero/mnist/pytorch/train_mnist_zr_8_dpzrmp_3.py", 8,
     ["-g", "0", "-t", "dp+zr+mp", "-dpsz", "2", "-zrsz", "2", "-mpsz", "2"], {}),
    # the same scripts under the reference's per-phase protocol (NKB_STEPWISE=1: one RPC round
    # per step phase instead of one command per epoch)
    ("dp/mnist/pytorch/train_ngn_mnist_1.py", 2, ["--gpus", "0", "-x", "nccl"], {"stepwise": True}),
    ("pp/mnist/pytorch/train_mnist_pp_32_dppp_grps.py", 4,
     ["-g", "0", "-t", "dp+pp", "-dpsz", "2", "-ppsz", "2"], {"stepwise": True}),
    ("zero/mnist/pytorch/train_mnist_zr_1.py", 3, ["--gpus", "0"], {"stepwise": True}),
    ("zero/mnist/pytorch/train_mnist_zr_5_dpzr_2.py", 4,
     ["-g", "0", "-t", "dp+zr", "-dpsz", "2", "-zrsz", "2"], {"stepwise": True}),
]


@pytest.mark.skipif(not os.path.isdir(EX), reason="NKB_REFERENCE_EXAMPLES is not set")
@pytest.mark.timeout(600)
@pytest.mark.parametrize("rel,world,extra,opts", CASES,
                         ids=[c[0].split("/")[-1] + ("-stepwise" if c[3].get("stepwise") else "")
                              for c in CASES])
def test_reference_example_runs_unedited(tmp_path, rel, world, extra, opts):
    script = os.path.join(EX, rel)
    svr = f"ipc://{tmp_path}/s.ipc"
    group = [a for a in extra if a in ("-t", "-dpsz", "-mpsz", "-ppsz", "-zrsz") or
             (extra.index(a) > 0 and extra[extra.index(a) - 1] in ("-t", "-dpsz", "-mpsz", "-ppsz",
                                                                   "-zrsz"))]
    sched = [sys.executable, RUN, script, "-r", "scheduler", "-w", str(world), "-k", "0",
             "--epochs", "1", "-u", svr, *group]
    if opts.get("mpirun"):
        sched += ["-n", "2"]
    base_env = dict(os.environ, NKB_STEPWISE="1" if opts.get("stepwise") else "0")
    procs = [subprocess.Popen(sched, stdout=open(tmp_path / "s.log", "w"), stderr=subprocess.STDOUT,
                              env=base_env)]
    for r in range(world):
        env = dict(base_env)
        if opts.get("mpirun"):      # rank and size the way mpirun hands them over
            env.update(OMPI_COMM_WORLD_RANK=str(r), OMPI_COMM_WORLD_SIZE=str(world))
            who, url = ["-k", "0"], f"ipc://{tmp_path}/w@{{LOCAL_RANK}}.ipc"
        else:
            who, url = ["-k", str(r)], f"ipc://{tmp_path}/w{r}.ipc"
        procs.append(subprocess.Popen(
            [sys.executable, RUN, script, "-r", "worker", "-w", str(world), *who, "-u", url, "-s",
             svr, "-b", "32", *extra],
            stdout=open(tmp_path / f"w{r}.log", "w"), stderr=subprocess.STDOUT, env=env))
    codes = []
    for p in procs:
        try:
            codes.append(p.wait(timeout=500))
        except subprocess.TimeoutExpired:
            p.kill()
            codes.append(-9)
    logs = {n: open(tmp_path / n).read() for n in ["s.log"] + [f"w{r}.log" for r in range(world)]}
    tail = "".join(v[-700:] for v in logs.values())
    assert codes == [0] * (world + 1), (codes, tail)
    # the scripts return 0 whatever happened: an aborted job shows in the logs
    for name, text in logs.items():
        assert "Traceback" not in text and "failed in state" not in text and \
            "scheduler: abort" not in text, (name, text[-1500:])
    # training happened: a metric line or the scripts' own loss print
    assert any("Epoch[" in logs[f"w{r}.log"] or "loss" in logs[f"w{r}.log"]
               for r in range(world)), tail
