"""MXNet Gluon operator under the reference's module name (necklace/trainer/tnopmx.py:26-362;
broken there: it imports modules that its tree does not have).  MXNet is not part of this
build, so the class exists for import parity and refuses to be constructed; the state it was
meant to keep for gradient compression (residual, per-rank code buffers) lives in
``frmwrk.pytorch.ptprms`` and in the fused kernel ``PeerGroup.dp_quant_allreduce``."""
from .tnopbs import TrainerOPBase


class TrainerOPGluon(TrainerOPBase):
    def __init__(self, cfg=None):
        try:
            import mxnet  # noqa: F401
        except ImportError as e:
            raise RuntimeError("TrainerOPGluon needs MXNet, which this build does not include; "
                               "use trainer.tnoppt.TrainerOPPytorch") from e
        super().__init__(cfg or {})
