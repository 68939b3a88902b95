"""Example scripts run as a user would start them (CPU, gloo, ipc urls) and match their
stock single-process counterparts."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _wait(procs, timeout):
    codes = []
    for p in procs:
        try:
            codes.append(p.wait(timeout=timeout))
        except subprocess.TimeoutExpired:
            p.kill()
            codes.append(-9)
    return codes


@pytest.mark.timeout(300)
@pytest.mark.parametrize("extra", [[], ["--flat"]])
def test_mixer_zero_example_matches_stock_loop(tmp_path, extra):
    script = os.path.join(ROOT, "examples", "zero", "train_mnist_mixer_zr.py")
    svr = f"ipc://{tmp_path}/s.ipc"
    procs = [subprocess.Popen([sys.executable, script, "-r", "scheduler", "-w", "2", "-u", svr,
                               "-e", "1"], stdout=open(tmp_path / "s.log", "w"),
                              stderr=subprocess.STDOUT, cwd=ROOT)]
    for r in range(2):
        procs.append(subprocess.Popen(
            [sys.executable, script, "-r", "worker", "-w", "2", "-k", str(r), "-u",
             f"ipc://{tmp_path}/w{r}.ipc", "-s", svr, "--no-cuda", "--out",
             str(tmp_path / f"o{r}.json"), *extra],
            stdout=open(tmp_path / f"w{r}.log", "w"), stderr=subprocess.STDOUT, cwd=ROOT))
    ref = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "zero", "main_mixer.py"),
                          "--parts", "2", "--replicas", "2", "--out", str(tmp_path / "ref.json")],
                         cwd=ROOT, capture_output=True, timeout=200)
    assert ref.returncode == 0, ref.stderr[-1000:]
    assert _wait(procs, 200) == [0, 0, 0], open(tmp_path / "w0.log").read()[-2000:]
    got = json.load(open(tmp_path / "o0.json"))
    want = json.load(open(tmp_path / "ref.json"))
    assert abs(got["weights_sum"] - want["weights_sum"]) < 1e-3
    assert got["acc"] and got["status"] == "stopped"


@pytest.mark.timeout(300)
def test_launcher_example_reads_rank_from_environment(tmp_path):
    """Workers started the way ``mpirun`` starts them: rank / size in the environment, url
    template expanded by ``args_remake``."""
    dp = os.path.join(ROOT, "examples", "dp")
    svr = f"ipc://{tmp_path}/s.ipc"
    procs = [subprocess.Popen([sys.executable, os.path.join(dp, "train_mnist_dp.py"), "-r",
                               "scheduler", "-w", "2", "-u", svr, "-e", "1"],
                              stdout=open(tmp_path / "s.log", "w"), stderr=subprocess.STDOUT,
                              cwd=ROOT)]
    for r in range(2):
        env = dict(os.environ, OMPI_COMM_WORLD_RANK=str(r), OMPI_COMM_WORLD_SIZE="2")
        procs.append(subprocess.Popen(
            [sys.executable, os.path.join(dp, "train_mnist_dp_launcher.py"), "--nslot", "2", "-u",
             f"ipc://{tmp_path}/w@{{LOCAL_RANK}}.ipc", "-s", svr, "--no-cuda", "--dataset-len",
             "400", "-b", "50", "--out", str(tmp_path / f"o{r}.json")],
            stdout=open(tmp_path / f"w{r}.log", "w"), stderr=subprocess.STDOUT, cwd=ROOT, env=env))
    assert _wait(procs, 200) == [0, 0, 0], open(tmp_path / "w1.log").read()[-2000:]
    outs = [json.load(open(tmp_path / f"o{r}.json")) for r in range(2)]
    assert abs(outs[0]["weights_sum"] - outs[1]["weights_sum"]) < 1e-9
