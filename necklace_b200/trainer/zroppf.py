"""ZeRO operator, flat-buffer flavour (reference: necklace/trainer/zroppf.py): inactive
sub-modules live in pinned host buffers and move through one flat device weight buffer
and one flat gradient buffer, so each broadcast / reduce is one collective."""
from .zroppt import TrainerMPOPPytorch as _Base


class TrainerMPOPPytorch(_Base):
    FLAT = True
