"""Tensor-parallel LeNet: the classifier's two linear layers are a
``mpnn.ColumnParallelLinear`` / ``mpnn.RowParallelLinear`` pair split over the model-parallel
group, the convolutions are replicated; the group's ranks share every batch (rank 0 of the
group loads it and broadcasts it).  Modes and their reference counterparts:

    mp     -w 2 -t mp -mpsz 2                 examples/mp/mnist/pytorch/train_mnist_mpnn_21_one_grp.py
    dp+mp  -w 4 -t dp+mp -dpsz 2 -mpsz 2      examples/mp/mnist/pytorch/train_mnist_mpnn_22_mpdp_grps.py

    python train_mnist_mpnn.py -r scheduler -w 4 -t dp+mp -dpsz 2 -mpsz 2 -u ipc:///tmp/s.ipc
    python train_mnist_mpnn.py -r worker -w 4 -k <r> -t dp+mp -dpsz 2 -mpsz 2 \\
        -u ipc:///tmp/w<r>.ipc -s ipc:///tmp/s.ipc [--no-cuda]
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, os.path.join(HERE, "..", "hybrid"))
sys.path.insert(0, os.path.join(HERE, "..", "pp"))

from lenet_parts import lenet_parts  # noqa: E402
from train_mlp_hybrid import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main(build=lenet_parts, in_shape=(1, 28, 28)))
