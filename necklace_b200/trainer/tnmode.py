"""Trainer modes (reference: necklace/trainer/tnmode.py:3-20; that list misses a comma
between 'no' and 'dp', fixed here)."""
from ..comm.groups import SUPPORTED_MODES, UNSUPPORTED_MODES  # noqa: F401

TRN_MODES = list(SUPPORTED_MODES)
TRN_MODES_NOT_SUPPORTED = list(UNSUPPORTED_MODES)
