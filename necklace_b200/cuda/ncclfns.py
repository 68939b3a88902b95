"""Collectives under the reference's module name (necklace/cuda/ncclfns.py)."""
from ..comm.fns import *  # noqa: F401,F403
from ..comm.fns import all_gather, all_reduce, broadcast, reduce  # noqa: F401
