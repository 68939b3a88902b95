"""Placeholder package, as in the reference (necklace/frmwrk/mxnet/ holds only ``__init__.py``).
MXNet is not part of this build; the Gluon operator ``trainer.tnopmx`` says so when used."""
