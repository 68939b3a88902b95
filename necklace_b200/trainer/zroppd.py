"""ZeRO operator for ``dp+zr`` / ``zr+mp`` / ``dp+zr+mp`` (reference:
necklace/trainer/zroppd.py); ``typ`` = ``dpzr`` / ``dpzrmp`` averages the owners' weights
over the dp group after each step, ``zrmp`` does not."""
from .zroppt import TrainerMPOPPytorch  # noqa: F401
