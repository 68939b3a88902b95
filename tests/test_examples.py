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


def _run_family(tmp_path, script, world, tmode, sizes, extra=()):
    svr = f"ipc://{tmp_path}/s.ipc"
    common = ["-w", str(world), "-t", tmode, "-e", "1", *sizes]
    procs = [subprocess.Popen([sys.executable, script, "-r", "scheduler", "-u", svr, *common],
                              stdout=open(tmp_path / "s.log", "w"), stderr=subprocess.STDOUT,
                              cwd=ROOT)]
    for r in range(world):
        procs.append(subprocess.Popen(
            [sys.executable, script, "-r", "worker", "-k", str(r), "-u",
             f"ipc://{tmp_path}/w{r}.ipc", "-s", svr, "--no-cuda", "--dataset-len", "128", "-b",
             "16", "--out", str(tmp_path / f"o{r}.json"), *common, *extra],
            stdout=open(tmp_path / f"w{r}.log", "w"), stderr=subprocess.STDOUT, cwd=ROOT))
    codes = _wait(procs, 240)
    logs = "".join(open(tmp_path / f"w{r}.log").read()[-600:] for r in range(world))
    assert codes == [0] * (world + 1), (codes, logs)
    return [json.load(open(tmp_path / f"o{r}.json")) for r in range(world)]


@pytest.mark.timeout(300)
def test_pipeline_lenet_example_dp_pp(tmp_path):
    """dp=2 x pp=2, two micro-batches: both replicas of a stage end with the same weights, the
    last stage reports a finite loss."""
    script = os.path.join(ROOT, "examples", "pp", "train_mnist_pp.py")
    outs = _run_family(tmp_path, script, 4, "dp+pp", ["-dpsz", "2", "-ppsz", "2"],
                       ["--micro-batches", "2"])
    assert all(o["status"] == "stopped" for o in outs)
    by_weights = {}
    for o in outs:
        by_weights.setdefault(tuple(sorted(o["weights"])), []).append(o["weights"])
    assert len(by_weights) == 2                      # two stages, two replicas each
    for a, b in by_weights.values():
        assert all(abs(a[k] - b[k]) < 1e-6 for k in a)
    losses = [o["loss"] for o in outs if o["loss"] is not None]
    assert losses and all(0 < l < 10 for l in losses)


@pytest.mark.timeout(300)
def test_pipeline_lenet_example_three_stages(tmp_path):
    script = os.path.join(ROOT, "examples", "pp", "train_mnist_pp.py")
    outs = _run_family(tmp_path, script, 3, "pp", ["-ppsz", "3"])
    assert all(o["status"] == "stopped" for o in outs)
    assert len({tuple(sorted(o["weights"].items())) for o in outs}) == 3   # three different units
    assert sum(o["loss"] is not None for o in outs) >= 1


@pytest.mark.timeout(300)
def test_tensor_parallel_lenet_example_dp_mp(tmp_path):
    """dp=2 x mp=2: replicated convolutions agree on all four ranks, classifier shards agree
    between the two replicas of the same model-parallel rank."""
    script = os.path.join(ROOT, "examples", "mp", "train_mnist_mpnn.py")
    outs = _run_family(tmp_path, script, 4, "dp+mp", ["-dpsz", "2", "-mpsz", "2"])
    assert all(o["status"] == "stopped" and o["loss"] is not None for o in outs)
    conv = [k for k in outs[0]["weights"] if "fc" not in k]
    assert len(conv) == 4                            # two convolutions: weight and bias
    for o in outs[1:]:
        assert all(abs(o["weights"][k] - outs[0]["weights"][k]) < 1e-5 for k in conv)


@pytest.mark.timeout(300)
@pytest.mark.parametrize("loader", ["shm", "obj"])
def test_dp_example_fed_from_shared_memory_loaders(tmp_path, loader):
    """Two data-parallel workers fed by loader processes end with the same weights as the same
    run fed by the in-process loader (same sampler, same order)."""
    script = os.path.join(ROOT, "examples", "dp", "train_mnist_dp.py")
    sums = {}
    for kind in ("ngn", loader):
        d = tmp_path / kind
        d.mkdir()
        svr = f"ipc://{d}/s.ipc"
        procs = [subprocess.Popen([sys.executable, script, "-r", "scheduler", "-w", "2", "-u", svr,
                                   "-e", "1"], stdout=open(d / "s.log", "w"),
                                  stderr=subprocess.STDOUT, cwd=ROOT)]
        for r in range(2):
            procs.append(subprocess.Popen(
                [sys.executable, script, "-r", "worker", "-w", "2", "-k", str(r), "-u",
                 f"ipc://{d}/w{r}.ipc", "-s", svr, "-t", "dp", "--no-cuda", "--dataset-len", "240",
                 "-b", "20", "--loader", kind, "--out", str(d / f"o{r}.json")],
                stdout=open(d / f"w{r}.log", "w"), stderr=subprocess.STDOUT, cwd=ROOT))
        assert _wait(procs, 200) == [0, 0, 0], open(d / "w0.log").read()[-2000:]
        sums[kind] = [json.load(open(d / f"o{r}.json"))["weights_sum"] for r in range(2)]
        assert abs(sums[kind][0] - sums[kind][1]) < 1e-9
    assert abs(sums["ngn"][0] - sums[loader][0]) < 1e-6


@pytest.mark.timeout(300)
def test_dp_example_with_the_mixer_model(tmp_path):
    script = os.path.join(ROOT, "examples", "dp", "train_mnist_dp.py")
    svr = f"ipc://{tmp_path}/s.ipc"
    procs = [subprocess.Popen([sys.executable, script, "-r", "scheduler", "-w", "2", "-u", svr,
                               "-e", "1"], stdout=open(tmp_path / "s.log", "w"),
                              stderr=subprocess.STDOUT, cwd=ROOT)]
    for r in range(2):
        procs.append(subprocess.Popen(
            [sys.executable, script, "-r", "worker", "-w", "2", "-k", str(r), "-u",
             f"ipc://{tmp_path}/w{r}.ipc", "-s", svr, "-t", "dp", "--no-cuda", "--dataset-len",
             "200", "-b", "20", "--model", "mixer", "--out", str(tmp_path / f"o{r}.json")],
            stdout=open(tmp_path / f"w{r}.log", "w"), stderr=subprocess.STDOUT, cwd=ROOT))
    assert _wait(procs, 200) == [0, 0, 0], open(tmp_path / "w0.log").read()[-2000:]
    outs = [json.load(open(tmp_path / f"o{r}.json")) for r in range(2)]
    assert abs(outs[0]["weights_sum"] - outs[1]["weights_sum"]) < 1e-9
    assert 0 < outs[0]["epoch_loss"][-1] < 10
