"""Every trainer mode, as scheduler + worker processes on CPU (gloo), against a
single-process run of the same model on the same data with the same seed."""
import json
import os
import subprocess
import sys
import time

import pytest
import torch
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXAMPLE = os.path.join(ROOT, "examples", "hybrid", "train_mlp_hybrid.py")
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(EXAMPLE))


def _run(tmp_path, world, tmode, sizes=(), extra=(), timeout=240):
    svr = f"ipc://{tmp_path}/s.ipc"
    common = ["-w", str(world), "-t", tmode, "-e", "1", *sizes, *extra]
    procs = [subprocess.Popen([sys.executable, EXAMPLE, "-r", "scheduler", "-u", svr, *common],
                              stdout=open(tmp_path / "s.log", "w"), stderr=subprocess.STDOUT)]
    for r in range(world):
        procs.append(subprocess.Popen(
            [sys.executable, EXAMPLE, "-r", "worker", "-k", str(r), "-u",
             f"ipc://{tmp_path}/w{r}.ipc", "-s", svr, "--no-cuda", "--out",
             str(tmp_path / f"o{r}.json"), *common],
            stdout=open(tmp_path / f"w{r}.log", "w"), stderr=subprocess.STDOUT))
    t0 = time.time()
    codes = []
    for p in procs:
        try:
            codes.append(p.wait(timeout=max(1, timeout - (time.time() - t0))))
        except subprocess.TimeoutExpired:
            p.kill()
            codes.append(-9)
    logs = "".join(open(tmp_path / f"w{r}.log").read()[-800:] for r in range(world))
    assert all(c == 0 for c in codes), (codes, logs)
    return [json.load(open(tmp_path / f"o{r}.json")) for r in range(world)]


def _reference_last_losses(n_parts, use_mp, n_replica, dataset_len=256, batch=32, lr=0.05, seed=1):
    """Single process: global batch = all replicas' batches, averaged gradients.
    Returns the per-replica loss of the last step."""
    from necklace_b200.comm import groups as G
    from necklace_b200.data.dtset import SyntheticDataset
    import train_mlp_hybrid as ex
    G.reset_nccl_groups_map()
    parts = ex.build_parts(n_parts, use_mp, seed)
    net = nn.Sequential(*parts)
    opt = torch.optim.SGD(net.parameters(), lr=lr)
    ds = SyntheticDataset(dataset_len, (784,), classes=10, seed=seed)
    per = dataset_len // n_replica
    ce = nn.CrossEntropyLoss()
    last = None
    for i in range(per // batch):
        opt.zero_grad()
        losses = []
        for r in range(n_replica):
            idx = range(r * per + i * batch, r * per + (i + 1) * batch)
            x = torch.stack([ds[j][0] for j in idx])
            y = torch.tensor([ds[j][1] for j in idx])
            losses.append(ce(net(x), y))
        (sum(losses) / n_replica).backward()
        opt.step()
        last = [float(l) for l in losses]
    return last


CASES = [
    # tmode, world, size flags, parts, uses mp, replicas, extra flags
    ("dp", 2, (), 1, False, 2, ()),
    ("mp", 2, (), 1, True, 1, ()),
    ("dp+mp", 4, ("-dpsz", "2", "-mpsz", "2"), 1, True, 2, ()),
    ("pp", 2, (), 2, False, 1, ("--micro-batches", "2")),
    ("pp", 3, (), 3, False, 1, ("--stepwise",)),
    ("dp+pp", 4, ("-dpsz", "2", "-ppsz", "2"), 2, False, 2, ()),
    ("zr", 2, (), 3, False, 2, ()),
    ("zr", 2, (), 3, False, 2, ("--stepwise", "--zr-flat")),
    ("dp+zr", 4, ("-dpsz", "2", "-zrsz", "2"), 3, False, 4, ("--zr-offload",)),
    ("zr+mp", 4, ("-zrsz", "2", "-mpsz", "2"), 3, True, 2, ()),
]


@pytest.mark.timeout(400)
@pytest.mark.parametrize("tmode,world,sizes,parts,use_mp,replicas,extra", CASES)
def test_mode_matches_single_process(tmp_path, tmode, world, sizes, parts, use_mp, replicas, extra):
    outs = _run(tmp_path, world, tmode, sizes, extra)
    ref = _reference_last_losses(parts, use_mp, replicas)
    got = sorted(o["loss"] for o in outs if o["loss"] is not None)
    assert got, outs
    # every reported loss is one of the per-replica losses of the reference's last step
    for g in got:
        assert min(abs(g - r) for r in ref) < 2e-4, (got, ref)
    # and every replica is represented
    for r in ref:
        assert min(abs(g - r) for g in got) < 2e-4, (got, ref)


@pytest.mark.timeout(600)
def test_three_way_hybrids_8_ranks(tmp_path):
    """dp+pp+mp 2x2x2 (the reference's headline example layout) and dp+zr+mp 2x2x2."""
    outs = _run(tmp_path, 8, "dp+pp+mp", ("-dpsz", "2", "-ppsz", "2", "-mpsz", "2"), timeout=400)
    ref = _reference_last_losses(2, True, 2)
    got = sorted(o["loss"] for o in outs if o["loss"] is not None)
    assert len(got) == 4  # the two mp ranks of the last stage of both pipelines
    for g in got:
        assert min(abs(g - r) for r in ref) < 2e-4, (got, ref)
    (tmp_path / "b").mkdir()
    outs = _run(tmp_path / "b", 8, "dp+zr+mp", ("-dpsz", "2", "-zrsz", "2", "-mpsz", "2"),
                timeout=400)
    ref = _reference_last_losses(3, True, 4)
    got = sorted(o["loss"] for o in outs if o["loss"] is not None)
    for g in got:
        assert min(abs(g - r) for r in ref) < 2e-4, (got, ref)
