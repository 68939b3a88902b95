"""Rank and size of a process started by an MPI-style launcher (``necklace.pympi`` is imported
by the reference's examples/dp/mnist/pytorch/train_nklc_nccl_mnist_1_mpirun.py:241-246 but is
absent from the reference's own tree)."""
