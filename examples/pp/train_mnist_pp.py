"""Pipeline-parallel LeNet on MNIST-shaped data: the network is cut into 2 or 3 ``net_map``
units, one per pipeline stage, and a step runs ``--micro-batches`` micro-batches through the
stages (1 = the sequential model-parallel hand-over of the reference's
examples/pp/mnist/pytorch/train_mnist_mp_5_nklc.py; more = the 1F1B schedule).  Modes and
their reference counterparts:

    pp        -w 2 -t pp -ppsz 2                       train_mnist_pp_31_one_grp.py
    pp, 3     -w 3 -t pp -ppsz 3                       train_mnist_mp_5_nklc_w3.py
    dp+pp     -w 4 -t dp+pp -dpsz 2 -ppsz 2            train_mnist_pp_32_dppp_grps.py
    dp+pp, 3  -w 6 -t dp+pp -dpsz 2 -ppsz 3            train_mnist_pp_33_dppp_grps_n3.py
    dp+pp+mp  -w 8 -t dp+pp+mp -dpsz 2 -ppsz 2 -mpsz 2 train_mnist_pp_81_dpppmp_3.py

Start one scheduler and ``-w`` workers from this script:

    python train_mnist_pp.py -r scheduler -w 4 -t dp+pp -dpsz 2 -ppsz 2 -u ipc:///tmp/s.ipc
    python train_mnist_pp.py -r worker -w 4 -k <r> -t dp+pp -dpsz 2 -ppsz 2 \\
        -u ipc:///tmp/w<r>.ipc -s ipc:///tmp/s.ipc --micro-batches 4 [--no-cuda]
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, os.path.join(HERE, "..", "hybrid"))
sys.path.insert(0, HERE)

from lenet_parts import lenet_parts  # noqa: E402
from train_mlp_hybrid import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main(build=lenet_parts, in_shape=(1, 28, 28)))
