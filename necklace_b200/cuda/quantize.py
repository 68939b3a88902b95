"""2-bit codec under the reference's module name (necklace/cuda/quantize.py)."""
from ..ops.quant import *  # noqa: F401,F403
from ..ops.quant import cu_fn_matrix_dequantize_e, cu_fn_matrix_quantize_e  # noqa: F401
from ..ops.quant import CMP_RATIO  # noqa: F401

# The reference's kernel objects are numba kernels that its wrappers launch over a grid
# (necklace/cuda/quantize.py:16-87); here the kernels are native and the wrappers call them,
# so the kernel names resolve to the wrappers (same arguments, no launch configuration).
cu_knl_matrix_quantize_e = cu_fn_matrix_quantize_e
cu_knl_matrix_dequantize_e = cu_fn_matrix_dequantize_e
