"""The data-parallel LeNet example for workers started by a launcher (``mpirun``, ``srun``,
``torchrun``): rank and world size come from the launcher's environment, the worker's RPC url
is a template, and ``args_remake`` fills in the node's address and the local rank, as in
the reference's launcher example
(examples/dp/mnist/pytorch/train_nklc_nccl_mnist_1_mpirun.py:240-269, :344-354):

    python train_mnist_dp.py -r scheduler -w 4 -u tcp://10.0.0.1:11000 -e 1
    mpirun -np 4 -H node1:2,node2:2 python train_mnist_dp_launcher.py --nslot 2 \
        -u "tcp://@{MY_IP}:1200@{LOCAL_RANK}" -s tcp://10.0.0.1:11000 -rp 10.0.

Environment read (first that is set): ``OMPI_COMM_WORLD_RANK/SIZE``, ``PMI_RANK/SIZE``,
``SLURM_PROCID/NTASKS``, ``RANK/WORLD_SIZE``.  Everything else is ``train_mnist_dp.py``."""
from __future__ import annotations

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, HERE)

from necklace_b200.utils import argutils  # noqa: E402

_ENV = (("OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE"), ("PMI_RANK", "PMI_SIZE"),
        ("SLURM_PROCID", "SLURM_NTASKS"), ("RANK", "WORLD_SIZE"))


def launcher_rank_size():
    for rk, sz in _ENV:
        if rk in os.environ and sz in os.environ:
            return int(os.environ[rk]), int(os.environ[sz])
    raise SystemExit("no launcher environment found (mpirun / srun / torchrun)")


def main():
    import argparse
    ap = argparse.ArgumentParser(add_help=False)
    ap.add_argument("--nslot", "-n", type=int, default=1, help="workers (GPUs) per node")
    ap.add_argument("--url", "-u", default="tcp://@{MY_IP}:1200@{LOCAL_RANK}")
    ap.add_argument("--rpc_ifname", "-ri", default="")
    ap.add_argument("--rpc_ip_prefix", "-rp", default="")
    ap.add_argument("--comm_ifname", "-ci", default="")
    known, rest = ap.parse_known_args()
    known.rank, world = launcher_rank_size()
    argutils.args_remake(known)                 # fills url, gpu_dev_i, NCCL_SOCKET_IFNAME
    argv = ["-r", "worker", "-w", str(world), "-k", str(known.rank), "-g", str(known.gpu_dev_i),
            "-u", known.url, "-t", "dp" if world > 1 else "no", *rest]
    import train_mnist_dp
    sys.argv = [sys.argv[0], *argv]
    return train_mnist_dp.main()


if __name__ == "__main__":
    sys.exit(main())
