"""Activation checkpointing under the reference's module name (necklace/frmwrk/pytorch/
ptacts.py is an empty placeholder there): the two implementations this framework has."""
from .mdwrp import MdWrpWithSelfBkwd  # noqa: F401  (re-computation inside a net_map unit)
from .mpnn.checkpointing import checkpoint, get_cuda_rng_tracker  # noqa: F401
