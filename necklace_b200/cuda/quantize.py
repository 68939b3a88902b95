"""2-bit codec under the reference's module name (necklace/cuda/quantize.py)."""
from ..ops.quant import *  # noqa: F401,F403
from ..ops.quant import cu_fn_matrix_dequantize_e, cu_fn_matrix_quantize_e  # noqa: F401
