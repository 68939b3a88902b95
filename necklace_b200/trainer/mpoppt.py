"""Sequential-stage pipeline operator under the reference's module name
(necklace/trainer/mpoppt.py); the implementation is shared with ``ppoppt``."""
from .ppoppt import TrainerMPOPPytorch  # noqa: F401
